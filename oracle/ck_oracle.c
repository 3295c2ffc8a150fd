/*
 * TEST INFRASTRUCTURE - not part of the product.  A plain C (OpenMP) restatement of the
 * reference's eager quantizers and dequantizers, bit-identical to oracle/ck_oracle.py and
 * pinned by the same golden vectors (tests/test_oracle_golden.py).  It exists so that the
 * parity tests can check full-size tensors in milliseconds and so that the CPU baseline of
 * bench.py uses every host core.  Only tests/, __graft_entry__.smoke() and bench.py's CPU
 * legs may load it.
 *
 * Arithmetic follows the reference file by file:
 *   quantize_nvfp4    comfy_kitchen/backends/eager/quantization.py:115-160
 *   dequantize_nvfp4  comfy_kitchen/backends/eager/quantization.py:171-219
 *   quantize_mxfp8    comfy_kitchen/backends/eager/quantization.py:257-324
 *   dequantize_mxfp8  comfy_kitchen/backends/eager/quantization.py:327-364
 *   E2M1 cast         comfy_kitchen/float_utils.py:41-150 (decision thresholds), packing :253-260
 *   scale tiling      comfy_kitchen/float_utils.py:292-352
 * Build: oracle/build.py (gcc -O2 -fopenmp, no fast-math, no FMA contraction: every float
 * operation below is one IEEE binary32 operation, as in the reference's torch ops).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bits_to_f32(uint32_t b) {
  float f;
  memcpy(&f, &b, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  return b;
}

/* float32 -> float8_e4m3fn byte, round to nearest even, saturating at 448 (float_utils.py:37-38) */
static inline uint8_t f32_to_e4m3(float x) {
  const uint32_t bits = f32_to_bits(x);
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
  const uint32_t mag = bits & 0x7FFFFFFFu;
  const float a = bits_to_f32(mag);
  int64_t code;
  if (a != a) return (uint8_t)(0x7F | sign);
  if (a >= 0x1p-6f) {
    const uint32_t r = mag + 0x7FFFFu + ((mag >> 20) & 1u);
    code = (int64_t)(r >> 20) - ((127 - 7) << 3);
  } else {
    code = (int64_t)rintf(a * 512.0f); /* uniform grid of step 2^-9 below 2^-6 */
  }
  if (code > 0x7E) code = 0x7E;
  return (uint8_t)((uint8_t)code | sign);
}

static inline float e4m3_to_f32(uint8_t b) {
  const uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
  float v;
  if (e == 0) {
    v = (float)m * 0x1p-9f;
  } else {
    v = bits_to_f32(((e - 7 + 127) << 23) | (m << 20));
  }
  return (b & 0x80u) ? -v : v;
}

/* E2M1 code of y (already clamped to [-6, 6]); ties to even; the sign bit is kept for zeros */
static inline uint8_t f32_to_e2m1(float y) {
  const uint8_t sign = (f32_to_bits(y) >> 31) ? 8u : 0u;
  const float a = fabsf(y);
  uint8_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return (uint8_t)(c | sign);
}

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

static inline int64_t tiled_offset(int64_t r, int64_t c, int64_t col_tiles) {
  const int64_t tile = (r >> 7) * col_tiles + (c >> 2);
  return tile * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c & 3);
}

static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

/*
 * x: [rows, cols] float32 values (bf16/f16 inputs widened exactly by the caller), read with a
 * zero border up to [rows_pad, cols_pad] (the pad_16x case); cols_pad % 16 == 0.
 * codes: [rows_pad, cols_pad/2]; scales: tiled [roundup(rows_pad,128), roundup(cols_pad/16,4)], zeroed here.
 */
void ck_oracle_quantize_nvfp4(const float* x, int64_t rows, int64_t cols, int64_t rows_pad, int64_t cols_pad,
                              float global_scale, int hi_first, uint8_t* codes, uint8_t* scales) {
  const int64_t n_sc = cols_pad / 16;
  const int64_t col_tiles = round_up(n_sc, 4) / 4;
  memset(scales, 0, (size_t)(round_up(rows_pad, 128) * col_tiles * 4));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows_pad; ++r) {
    for (int64_t b = 0; b < n_sc; ++b) {
      float v[16];
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        const int64_t c = b * 16 + i;
        v[i] = (r < rows && c < cols) ? x[r * cols + c] : 0.0f;
        const float a = fabsf(v[i]);
        if (a > amax) amax = a;
      }
      float s = (amax / 6.0f) / global_scale; /* :139-140 */
      if (s > 448.0f) s = 448.0f;             /* :141 */
      const uint8_t s8 = f32_to_e4m3(s);      /* :142 */
      const float total = global_scale * e4m3_to_f32(s8); /* :143 */
      const int dead = (total == 0.0f);
      const float safe = dead ? 1.0f : total;
      uint8_t code[16];
      for (int i = 0; i < 16; ++i) {
        float y = dead ? 0.0f : v[i] / safe; /* :149-150 */
        if (y > 6.0f) y = 6.0f;
        if (y < -6.0f) y = -6.0f;
        code[i] = f32_to_e2m1(y);
      }
      uint8_t* dst = codes + r * (cols_pad / 2) + b * 8;
      for (int i = 0; i < 8; ++i) {
        dst[i] = hi_first ? (uint8_t)((code[2 * i] << 4) | code[2 * i + 1]) : (uint8_t)((code[2 * i + 1] << 4) | code[2 * i]);
      }
      scales[tiled_offset(r, b, col_tiles)] = s8;
    }
  }
}

/* out: [rows, cols] float32 (the reference's float32 output; other dtypes are one rounding of it) */
void ck_oracle_dequantize_nvfp4(const uint8_t* codes, const uint8_t* scales, float global_scale, int64_t rows,
                                int64_t cols, int hi_first, float* out) {
  const int64_t col_tiles = round_up(cols / 16, 4) / 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b = 0; b < cols / 16; ++b) {
      const float total = global_scale * e4m3_to_f32(scales[tiled_offset(r, b, col_tiles)]);
      const uint8_t* src = codes + r * (cols / 2) + b * 8;
      for (int i = 0; i < 8; ++i) {
        const uint8_t hi = src[i] >> 4, lo = src[i] & 15u;
        const uint8_t c0 = hi_first ? hi : lo, c1 = hi_first ? lo : hi;
        const float v0 = (c0 & 8u) ? -kE2M1[c0 & 7u] : kE2M1[c0 & 7u];
        const float v1 = (c1 & 8u) ? -kE2M1[c1 & 7u] : kE2M1[c1 & 7u];
        out[r * cols + b * 16 + 2 * i] = v0 * total;
        out[r * cols + b * 16 + 2 * i + 1] = v1 * total;
      }
    }
  }
}

/* clamp(ceil(log2(r)) + 127, 0, 254) by exponent bits (exact for quotients of 16-bit inputs) */
static inline uint32_t ceil_log2_biased(float r) {
  const uint32_t bits = f32_to_bits(r);
  const uint32_t e = (bits >> 23) & 0xFFu;
  const uint32_t frac = (bits & 0x7FFFFFu) != 0;
  uint32_t biased = (e == 0) ? frac : e + frac;
  return biased > 254u ? 254u : biased;
}

/* data: [rows_pad, cols_pad] e4m3 bytes; scales: tiled E8M0 bytes, zeroed here; cols_pad % 32 == 0 */
void ck_oracle_quantize_mxfp8(const float* x, int64_t rows, int64_t cols, int64_t rows_pad, int64_t cols_pad,
                              uint8_t* data, uint8_t* scales) {
  const int64_t n_sc = cols_pad / 32;
  const int64_t col_tiles = round_up(n_sc, 4) / 4;
  memset(scales, 0, (size_t)(round_up(rows_pad, 128) * col_tiles * 4));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows_pad; ++r) {
    for (int64_t b = 0; b < n_sc; ++b) {
      float v[32];
      float amax = 0.0f;
      for (int i = 0; i < 32; ++i) {
        const int64_t c = b * 32 + i;
        v[i] = (r < rows && c < cols) ? x[r * cols + c] : 0.0f;
        const float a = fabsf(v[i]);
        if (a > amax) amax = a;
      }
      float need = amax / 448.0f; /* :294 */
      if (need < 0x1p-127f) need = 0x1p-127f;
      const uint32_t e = ceil_log2_biased(need); /* :298-302 */
      const int dead = (amax == 0.0f);
      float scale = (e == 0) ? 0.0f : bits_to_f32(e << 23); /* float_utils.py:376-382 */
      if (dead) scale = 1.0f;
      for (int i = 0; i < 32; ++i) {
        float y = dead ? 0.0f : v[i] / scale;
        if (y > 448.0f) y = 448.0f;
        if (y < -448.0f) y = -448.0f;
        data[r * cols_pad + b * 32 + i] = f32_to_e4m3(y);
      }
      scales[tiled_offset(r, b, col_tiles)] = dead ? 0 : (uint8_t)e;
    }
  }
}

void ck_oracle_dequantize_mxfp8(const uint8_t* data, const uint8_t* scales, int64_t rows, int64_t cols, float* out) {
  const int64_t col_tiles = round_up(cols / 32, 4) / 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b = 0; b < cols / 32; ++b) {
      const uint32_t e = scales[tiled_offset(r, b, col_tiles)];
      const float scale = (e == 0) ? 0.0f : bits_to_f32(e << 23);
      for (int i = 0; i < 32; ++i) out[r * cols + b * 32 + i] = e4m3_to_f32(data[r * cols + b * 32 + i]) * scale;
    }
  }
}

/* float32 -> bfloat16 bits, round to nearest even (the GEMM contract's final cast) */
void ck_oracle_f32_to_bf16(const float* x, int64_t n, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t b = f32_to_bits(x[i]);
    out[i] = (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
  }
}

/* Number of OpenMP threads the row loops use from now on (a launcher may have exported
 * OMP_NUM_THREADS=1; callers that time this code set the count they report). */
void ck_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int ck_oracle_threads(void) {
  int n = 1;
#ifdef _OPENMP
#pragma omp parallel
  {
#pragma omp master
    n = omp_get_num_threads();
  }
#endif
  return n;
}
