// Arithmetic of one NVFP4 / MXFP8 scale block, shared by the stand-alone quantizers and the
// re-quantizing GEMM epilogue.  Results are bit-identical to the reference's eager path
// (comfy_kitchen/backends/eager/quantization.py:115-160); translation units that include
// this header must not be compiled with fast-math.
#pragma once

#include "ck_common.cuh"

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
  const bool window = kFastDiv && (safe >= 0x1p-60f) && (safe <= 0x1p60f) && (amax <= safe * 0x1p20f);
  if (window) {
    const float y = __frcp_rn(safe);
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = div_markstein(v[i], safe, y);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(v[i], safe);  // :149
  }
  if (dead) {
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = 0.0f;  // :150 (positive zero, sign dropped)
  }
  // :154-158 clamp to +-6, round to E2M1 (satfinite does the clamp), pack two per byte.
  uint32_t b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    b[i] = hi_first ? f32x2_to_e2m1_byte(q[2 * i], q[2 * i + 1]) : f32x2_to_e2m1_byte(q[2 * i + 1], q[2 * i]);
  }
  lo_word = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
  hi_word = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
}

}  // namespace quant
}  // namespace ck
