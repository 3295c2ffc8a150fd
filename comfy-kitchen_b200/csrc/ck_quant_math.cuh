// Arithmetic of one NVFP4 / MXFP8 scale block, shared by the stand-alone quantizers and the
// re-quantizing GEMM epilogue.  Results are bit-identical to the reference's eager path
// (comfy_kitchen/backends/eager/quantization.py:115-160); translation units that include
// this header must not be compiled with fast-math.
#pragma once

#include "ck_common.cuh"

#include <type_traits>

namespace ck {
namespace quant {

// ---------------------------------------------------------------------------
// small-float converts (hardware cvt; rounding = nearest-even, saturating)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f32_to_e4m3_byte(float v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
  return r & 0xFFu;
}

__device__ __forceinline__ float e4m3_byte_to_f32(uint32_t b) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(b)));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFFu)));
}

// byte = e2m1(hi) << 4 | e2m1(lo)
__device__ __forceinline__ uint32_t f32x2_to_e2m1_byte(float hi, float lo) {
  uint16_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; mov.b16 %0, {t, 0}; }" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// 16-bit = e4m3(hi) << 8 | e4m3(lo)
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float hi, float lo) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// ---------------------------------------------------------------------------
// a / b, correctly rounded, from y = RN(1/b) with five FMA-class operations.
//
// q0 = RN(a*y) is within 2 ulp of a/b; one residual correction makes q1 a faithful
// quotient (error of q0 + r0*y against a/b is below 2^-46 relative), and by Markstein's
// theorem a second correction from a faithful quotient with a correctly rounded
// reciprocal yields RN(a/b), provided every residual is exact.  The caller guarantees
// the exponent window in which that holds (see nvfp4_block) and falls back to
// __fdiv_rn outside it.  The sign of `a` is re-applied at the end because an all-zero
// FMA chain loses a negative zero.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float div_markstein(float a, float b, float y) {
  float q = __fmul_rn(a, y);
  float r = __fmaf_rn(-b, q, a);
  q = __fmaf_rn(r, y, q);
  r = __fmaf_rn(-b, q, a);
  q = __fmaf_rn(r, y, q);
  return copysignf(q, a);
}

__device__ __forceinline__ float amax16(const float (&v)[16]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

// Merge the scale bytes of the 4 lanes that share one 4-byte group of the scale tile and
// store them with one 32-bit store from the first of the four lanes.
// ---------------------------------------------------------------------------
// NVFP4
// ---------------------------------------------------------------------------
// One 16-element block -> 8 code bytes (returned as two words) and one E4M3 scale byte.
// Steps follow comfy_kitchen/backends/eager/quantization.py:137-158 one to one.
template <bool kFastDiv>
__device__ __forceinline__ void nvfp4_block(const float (&v)[16], float g, bool hi_first, uint32_t& lo_word,
                                            uint32_t& hi_word, uint32_t& scale_byte) {
  const float amax = amax16(v);
  float s = __fdiv_rn(__fdiv_rn(amax, 6.0f), g);  // :139-140, two true divisions
  s = fminf(s, 448.0f);                           // :141
  scale_byte = f32_to_e4m3_byte(s);               // :142
  const float total = __fmul_rn(g, e4m3_byte_to_f32(scale_byte));  // :143
  const bool dead = (total == 0.0f);              // :146
  const float safe = dead ? 1.0f : total;         // :147

  float q[16];
  // The reciprocal-FMA quotient is exact while no residual can underflow and no
  // quotient can overflow: divisor within 2^+-60 and amax no more than 2^20 divisors.
  // Elements so small that their residual would underflow (|x| < 2^-90) have a
  // quotient below 2^-30 and encode as (signed) zero under either formula.
  const bool window = kFastDiv && (safe >= 0x1p-60f) && (safe <= 0x1p60f);
  // :154-158 clamp to +-6, round to E2M1 (satfinite does the clamp), pack two per byte.
  auto pack = [&](const float (&e)[16]) {
    uint32_t b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      b[i] = hi_first ? f32x2_to_e2m1_byte(e[2 * i], e[2 * i + 1]) : f32x2_to_e2m1_byte(e[2 * i + 1], e[2 * i]);
    }
    lo_word = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
    hi_word = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
  };
  bool done = false;
  if (window) {
    // Codes from the two products that bracket the exact quotient (see nvfp4_block_packed);
    // accepted when they agree, which is the rule for all but a few blocks in ten thousand.
    const float y = __frcp_rn(safe);
    const float y_hi = __fmul_rn(y, 0x1.000008p0f), y_lo = __fmul_rn(y, 0x1.fffffp-1f);
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = v[i] * y_hi;
    pack(q);
    const uint32_t lo_a = lo_word, hi_a = hi_word;
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = v[i] * y_lo;
    pack(q);
    done = ((lo_a ^ lo_word) | (hi_a ^ hi_word)) == 0u;
    if (!done && amax <= safe * 0x1p20f) {
#pragma unroll
      for (int i = 0; i < 16; ++i) q[i] = div_markstein(v[i], safe, y);
      pack(q);
      done = true;
    }
  }
  if (!done) {
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(v[i], safe);  // :149
    pack(q);
  }
  if (dead) {  // :150 (positive zeros, signs dropped)
    lo_word = 0;
    hi_word = 0;
  }
}

// ---------------------------------------------------------------------------
// NVFP4 block for the streaming quantizer: 16 elements of a 16-bit type as eight packed
// words.  Same arithmetic as nvfp4_block, arranged for a low instruction count: packed
// abs-max, the two per-block divisions (by 6, by the tensor scale) as reciprocal-FMA
// quotients with reciprocals prepared once per thread, the zero-scale case resolved on the
// packed words, four E2M1 converts packed per 32-bit word, and the nibble order a
// template parameter.
// ---------------------------------------------------------------------------

// word = bytes {e2m1x2(f0,f1), e2m1x2(f2,f3), e2m1x2(f4,f5), e2m1x2(f6,f7)}, lowest byte first;
// within a byte the first argument goes to the high nibble.
__device__ __forceinline__ uint32_t f32x8_to_e2m1_word(float f0, float f1, float f2, float f3, float f4, float f5,
                                                       float f6, float f7) {
  uint32_t r;
  asm("{ .reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %1, %2;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %3, %4;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %5, %6;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %7, %8;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3}; }"
      : "=r"(r)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
  return r;
}

// a / b for a >= 0 (no sign to restore) with y = RN(1/b); see div_markstein.
__device__ __forceinline__ float div_markstein_nonneg(float a, float b, float y) {
  float q = __fmul_rn(a, y);
  float r = __fmaf_rn(-b, q, a);
  q = __fmaf_rn(r, y, q);
  r = __fmaf_rn(-b, q, a);
  return __fmaf_rn(r, y, q);
}

// max |.| over the 16 values packed in eight words, as a float
template <typename T>
__device__ __forceinline__ float amax16_packed(const uint32_t (&w)[8]) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[0]));
#pragma unroll
    for (int i = 1; i < 8; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i])));
    const uint32_t b = *reinterpret_cast<uint32_t*>(&m);
    return fmaxf(__uint_as_float(b << 16), __uint_as_float(b & 0xFFFF0000u));
  } else {
    __half2 m = __habs2(*reinterpret_cast<const __half2*>(&w[0]));
#pragma unroll
    for (int i = 1; i < 8; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __half2*>(&w[i])));
    const float2 f = __half22float2(m);
    return fmaxf(f.x, f.y);
  }
}

// Per-thread constants of the tensor scale g: its reciprocal and whether g lies in the
// range where the reciprocal-FMA quotients below are exact.
struct TensorScale {
  float g, rcp;
  bool in_window;
};
__device__ __forceinline__ TensorScale make_tensor_scale(float g) {
  TensorScale t;
  t.g = g;
  t.in_window = (g >= 0x1p-40f) && (g <= 0x1p40f);
  t.rcp = __frcp_rn(t.in_window ? g : 1.0f);
  return t;
}

template <typename T>
__device__ __forceinline__ void widen16(const uint32_t (&w)[8], float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
}

// The IEEE-division path of a packed block, out of line: it is taken only outside the
// exactness window (tiny or huge scales), and keeping it out of the caller's body keeps the
// caller's register allocation that of the common path.  Arguments and result travel in
// registers (words by value, a small struct back).
struct BlockCodes {
  uint32_t lo, hi, scale_byte;
};
template <typename T, bool kHiFirst>
__device__ __noinline__ BlockCodes nvfp4_block_packed_ieee(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t w4,
                                                           uint32_t w5, uint32_t w6, uint32_t w7, float g) {
  const uint32_t w[8] = {w0, w1, w2, w3, w4, w5, w6, w7};
  float v[16];
  widen16<T>(w, v);
  BlockCodes r;
  nvfp4_block<false>(v, g, kHiFirst, r.lo, r.hi, r.scale_byte);
  return r;
}

// Codes of 16 exact quotients x / safe by the reciprocal-FMA chain (see div_markstein), out of
// line: the streaming path below needs it only for blocks in which some quotient lies within
// 2^-21 (relative) of an E2M1 rounding boundary.
template <typename T, bool kHiFirst>
__device__ __noinline__ uint2 nvfp4_codes_exact(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t w4,
                                                uint32_t w5, uint32_t w6, uint32_t w7, float safe, float y) {
  const uint32_t w[8] = {w0, w1, w2, w3, w4, w5, w6, w7};
  float v[16], q[16];
  widen16<T>(w, v);
#pragma unroll
  for (int i = 0; i < 16; ++i) q[i] = div_markstein(v[i], safe, y);
  uint2 r;
  if constexpr (kHiFirst) {
    r.x = f32x8_to_e2m1_word(q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7]);
    r.y = f32x8_to_e2m1_word(q[8], q[9], q[10], q[11], q[12], q[13], q[14], q[15]);
  } else {
    r.x = f32x8_to_e2m1_word(q[1], q[0], q[3], q[2], q[5], q[4], q[7], q[6]);
    r.y = f32x8_to_e2m1_word(q[9], q[8], q[11], q[10], q[13], q[12], q[15], q[14]);
  }
  return r;
}

// 8 products v[i] * y -> one word of codes (nibble order as requested)
template <bool kHiFirst>
__device__ __forceinline__ uint32_t scaled_e2m1_word(const float* v, float y) {
  if constexpr (kHiFirst) {
    return f32x8_to_e2m1_word(v[0] * y, v[1] * y, v[2] * y, v[3] * y, v[4] * y, v[5] * y, v[6] * y, v[7] * y);
  } else {
    return f32x8_to_e2m1_word(v[1] * y, v[0] * y, v[3] * y, v[2] * y, v[5] * y, v[4] * y, v[7] * y, v[6] * y);
  }
}

// The element quotients are not computed at all in the common case.  The code of x / total is
// a monotone step function of the quotient, and RN(x / total) lies strictly between
// x * y_lo and x * y_hi with y_lo = y (1 - 2^-21), y_hi = y (1 + 2^-21), y = RN(1 / total)
// (the three roundings involved are below 2^-23 each, the quotient's own below 2^-24).  So
// when both bracketing products convert to the same codes for a whole block - two multiplies
// and one convert per element - those are the codes of the exact quotients; only a block in
// which some product straddles a rounding boundary is redone with exact quotients.  A zero
// keeps its sign through the multiplication, as the reference's cast keeps it.
template <typename T, bool kHiFirst>
__device__ __forceinline__ void nvfp4_block_packed(const uint32_t (&w)[8], const TensorScale& ts, uint32_t& lo_word,
                                                   uint32_t& hi_word, uint32_t& scale_byte) {
  static_assert(sizeof(T) == 2, "packed 16-bit inputs");
  const float amax = amax16_packed<T>(w);
  // Exactness window of the reciprocal-FMA quotients amax/6/g (all residuals representable):
  // tensor scale within 2^+-40, amax zero or within 2^+-60; then total = g * scale is a normal
  // number within 2^+-50 and its reciprocal is too.  Anything else takes the IEEE-division path.
  const bool fast_s = ts.in_window && (amax <= 0x1p60f) && (amax >= 0x1p-60f || amax == 0.0f);
  if (fast_s) {
    float s = div_markstein_nonneg(div_markstein_nonneg(amax, 6.0f, 0x1.555556p-3f /* RN(1/6) */), ts.g, ts.rcp);
    s = fminf(s, 448.0f);
    scale_byte = f32_to_e4m3_byte(s);
    const float total = __fmul_rn(ts.g, e4m3_byte_to_f32(scale_byte));
    const bool dead = (total == 0.0f);
    const float safe = dead ? 1.0f : total;
    const float y = __frcp_rn(safe);
    const float y_hi = __fmul_rn(y, 0x1.000008p0f), y_lo = __fmul_rn(y, 0x1.fffffp-1f);
    float v[16];
    widen16<T>(w, v);
    lo_word = scaled_e2m1_word<kHiFirst>(v, y_hi);
    hi_word = scaled_e2m1_word<kHiFirst>(v + 8, y_hi);
    const uint32_t lo_b = scaled_e2m1_word<kHiFirst>(v, y_lo);
    const uint32_t hi_b = scaled_e2m1_word<kHiFirst>(v + 8, y_lo);
    if (((lo_word ^ lo_b) | (hi_word ^ hi_b)) != 0u) {
      if (amax <= total * 0x1p20f) {  // residuals of the exact chain representable
        const uint2 r = nvfp4_codes_exact<T, kHiFirst>(w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7], safe, y);
        lo_word = r.x;
        hi_word = r.y;
      } else {
        const BlockCodes r = nvfp4_block_packed_ieee<T, kHiFirst>(w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7], ts.g);
        lo_word = r.lo;
        hi_word = r.hi;
      }
    }
    if (dead) {  // zero scale: every code is +0
      lo_word = 0;
      hi_word = 0;
    }
    return;
  }
  const BlockCodes r = nvfp4_block_packed_ieee<T, kHiFirst>(w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7], ts.g);
  lo_word = r.lo;
  hi_word = r.hi;
  scale_byte = r.scale_byte;
}

}  // namespace quant
}  // namespace ck
