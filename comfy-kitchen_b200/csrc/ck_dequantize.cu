// Dequantizers for sm_100a: NVFP4 (packed E2M1 + tiled E4M3 scales + fp32 tensor scale) and
// MXFP8 (E4M3 + tiled E8M0 scales) back to f32 / f16 / bf16.  Streaming kernels bounded by
// the output write: one thread per scale block, 256-bit stores.
//
// Arithmetic contract (bit-identical to the reference's eager path):
//   NVFP4, comfy_kitchen/backends/eager/quantization.py:171-219: everything happens in the
//     OUTPUT dtype: total = out_t(tensor_scale) * out_t(block_scale), value = lut * total.
//   MXFP8, :327-364: float32(e4m3) * 2^(e-127) in float32 (scale byte 0 decodes to 0), then
//     one cast to the output dtype.
#include "ck_common.cuh"

#include <type_traits>

namespace ck {
namespace {

constexpr int kThreads = 256;

template <typename OutT>
__device__ __forceinline__ float round_to(float v) {
  if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
    return __bfloat162float(__float2bfloat16_rn(v));
  } else if constexpr (std::is_same<OutT, __half>::value) {
    return __half2float(__float2half_rn(v));
  } else {
    return v;
  }
}

template <typename OutT>
__device__ __forceinline__ void store16(OutT* dst, const float (&v)[16]) {
  if constexpr (sizeof(OutT) == 2) {
    Vec256 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
        __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        o.w[i] = *reinterpret_cast<uint32_t*>(&p);
      } else {
        __half2 p = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        o.w[i] = *reinterpret_cast<uint32_t*>(&p);
      }
    }
    st_global_256(dst, o);
  } else {
    Vec256 a, b;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a.w[i] = __float_as_uint(v[i]);
      b.w[i] = __float_as_uint(v[8 + i]);
    }
    st_global_256(dst, a);
    st_global_256(dst + 8, b);
  }
}

__device__ __forceinline__ float e4m3_byte_to_f32(uint32_t b) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(b)));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFFu)));
}

// Four packed bytes (eight E2M1 codes) -> four f16x2 pairs with the hardware convert; in each
// pair the low half comes from the low nibble of its byte.  Every E2M1 value is exact in f16.
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t word, uint32_t (&h)[4]) {
  asm("{ .reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3; }"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(word));
}

// one thread = one 16-element block of one row
template <typename OutT, bool kHiFirst>
__global__ void __launch_bounds__(kThreads)
dequantize_nvfp4_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ global_scale,
                        const uint8_t* __restrict__ scales, OutT* __restrict__ out, int64_t rows, int64_t cols) {
  const int64_t n_sc = cols >> 4;
  const int64_t sc = static_cast<int64_t>(blockIdx.y) * 64 + threadIdx.x;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + threadIdx.y;
  if (row >= rows || sc >= n_sc) return;
  const uint2 packed = *reinterpret_cast<const uint2*>(codes + row * (cols >> 1) + sc * 8);
  const uint32_t sbyte = scales[swizzled_scale_offset(row, sc, ceil_div(n_sc, 4))];
  // :211 total scale in the output dtype
  const float ts = round_to<OutT>(__ldg(global_scale));
  const float bs = e4m3_byte_to_f32(sbyte);  // exact in every output dtype
  const float total = round_to<OutT>(ts * bs);
  float v[16];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    uint32_t h[4];
    e2m1x8_to_f16x2(w == 0 ? packed.x : packed.y, h);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));  // (low nibble, high nibble)
      // :214, rounded by the store; the product of two OutT numbers is exact in float32
      v[8 * w + 2 * i] = (kHiFirst ? f.y : f.x) * total;
      v[8 * w + 2 * i + 1] = (kHiFirst ? f.x : f.y) * total;
    }
  }
  store16<OutT>(out + row * cols + sc * 16, v);
}

// one thread = one 32-element block of one row
template <typename OutT>
__global__ void __launch_bounds__(kThreads)
dequantize_mxfp8_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
                        OutT* __restrict__ out, int64_t rows, int64_t cols) {
  const int64_t n_sc = cols >> 5;
  const int64_t sc = static_cast<int64_t>(blockIdx.y) * 64 + threadIdx.x;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + threadIdx.y;
  if (row >= rows || sc >= n_sc) return;
  const Vec256 raw = ld_global_stream_256(data + row * cols + sc * 32);
  const uint32_t e = scales[swizzled_scale_offset(row, sc, ceil_div(n_sc, 4))];
  const float scale = __uint_as_float(e << 23);  // byte 0 -> 0.0 (float_utils.py:376-382)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = raw.w[h * 4 + i];
      v[4 * i + 0] = e4m3_byte_to_f32(w & 0xFFu) * scale;
      v[4 * i + 1] = e4m3_byte_to_f32((w >> 8) & 0xFFu) * scale;
      v[4 * i + 2] = e4m3_byte_to_f32((w >> 16) & 0xFFu) * scale;
      v[4 * i + 3] = e4m3_byte_to_f32(w >> 24) * scale;
    }
    store16<OutT>(out + row * cols + sc * 32 + h * 16, v);
  }
}

int check_common(const char* op, const void* in, const void* scales, const void* out, int out_dtype, int64_t rows,
                 int64_t cols, int64_t block) {
  CK_REQUIRE(in && scales && out, "%s: null pointer", op);
  CK_REQUIRE(rows > 0 && cols > 0 && cols % block == 0, "%s: bad shape [%lld, %lld]", op, (long long)rows,
             (long long)cols);
  CK_REQUIRE(out_dtype == CK_DTYPE_F32 || out_dtype == CK_DTYPE_F16 || out_dtype == CK_DTYPE_BF16,
             "%s: unsupported output dtype code %d", op, out_dtype);
  CK_REQUIRE(reinterpret_cast<uintptr_t>(out) % 32 == 0, "%s: output must be 32-byte aligned", op);
  CK_REQUIRE(ceil_div(rows, 4) <= 0x7FFFFFFF && ceil_div(cols / block, 64) <= 65535, "%s: tensor too large", op);
  return CK_OK;
}

}  // namespace
}  // namespace ck

extern "C" int ck_dequantize_nvfp4(const void* codes, const float* global_scale, const void* block_scales, void* out,
                                   int out_dtype, int64_t rows, int64_t cols, int hi_first, void* stream) {
  using namespace ck;
  if (int rc = check_common("dequantize_nvfp4", codes, block_scales, out, out_dtype, rows, cols, 16)) return rc;
  CK_REQUIRE(global_scale != nullptr, "dequantize_nvfp4: null global_scale");
  CK_REQUIRE(reinterpret_cast<uintptr_t>(codes) % 8 == 0, "dequantize_nvfp4: codes must be 8-byte aligned");
  const dim3 grid(static_cast<unsigned>(ceil_div(rows, 4)), static_cast<unsigned>(ceil_div(cols / 16, 64))), block(64, 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint8_t* c = static_cast<const uint8_t*>(codes);
  const uint8_t* sc = static_cast<const uint8_t*>(block_scales);
  if (out_dtype == CK_DTYPE_BF16) {
    if (hi_first) dequantize_nvfp4_kernel<__nv_bfloat16, true><<<grid, block, 0, s>>>(c, global_scale, sc, static_cast<__nv_bfloat16*>(out), rows, cols);
    else dequantize_nvfp4_kernel<__nv_bfloat16, false><<<grid, block, 0, s>>>(c, global_scale, sc, static_cast<__nv_bfloat16*>(out), rows, cols);
  } else if (out_dtype == CK_DTYPE_F16) {
    if (hi_first) dequantize_nvfp4_kernel<__half, true><<<grid, block, 0, s>>>(c, global_scale, sc, static_cast<__half*>(out), rows, cols);
    else dequantize_nvfp4_kernel<__half, false><<<grid, block, 0, s>>>(c, global_scale, sc, static_cast<__half*>(out), rows, cols);
  } else {
    if (hi_first) dequantize_nvfp4_kernel<float, true><<<grid, block, 0, s>>>(c, global_scale, sc, static_cast<float*>(out), rows, cols);
    else dequantize_nvfp4_kernel<float, false><<<grid, block, 0, s>>>(c, global_scale, sc, static_cast<float*>(out), rows, cols);
  }
  CK_CUDA(cudaGetLastError());
  return CK_OK;
}

extern "C" int ck_dequantize_mxfp8(const void* data, const void* block_scales, void* out, int out_dtype, int64_t rows,
                                   int64_t cols, void* stream) {
  using namespace ck;
  if (int rc = check_common("dequantize_mxfp8", data, block_scales, out, out_dtype, rows, cols, 32)) return rc;
  CK_REQUIRE(reinterpret_cast<uintptr_t>(data) % 32 == 0, "dequantize_mxfp8: data must be 32-byte aligned");
  const dim3 grid(static_cast<unsigned>(ceil_div(rows, 4)), static_cast<unsigned>(ceil_div(cols / 32, 64))), block(64, 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint8_t* d = static_cast<const uint8_t*>(data);
  const uint8_t* sc = static_cast<const uint8_t*>(block_scales);
  if (out_dtype == CK_DTYPE_BF16) {
    dequantize_mxfp8_kernel<<<grid, block, 0, s>>>(d, sc, static_cast<__nv_bfloat16*>(out), rows, cols);
  } else if (out_dtype == CK_DTYPE_F16) {
    dequantize_mxfp8_kernel<<<grid, block, 0, s>>>(d, sc, static_cast<__half*>(out), rows, cols);
  } else {
    dequantize_mxfp8_kernel<<<grid, block, 0, s>>>(d, sc, static_cast<float*>(out), rows, cols);
  }
  CK_CUDA(cudaGetLastError());
  return CK_OK;
}
