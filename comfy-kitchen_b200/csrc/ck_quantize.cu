// Block quantizers for sm_100a: bf16/f16/f32 -> NVFP4 (E2M1 codes + E4M3 scales per
// 16 elements) and -> MXFP8 (E4M3 data + E8M0 scales per 32 elements), both with the
// scale bytes written straight into the 128x4-tiled layout the tensor cores consume.
//
// Both kernels are streaming kernels whose floor is HBM bandwidth.  One thread owns one scale
// block of one row (2-D block and grid indices, no integer division), so a warp reads 32
// consecutive blocks (1 KiB / 2 KiB of bf16) with 256-bit loads,
// writes 256 B / 1 KiB of codes with 64-bit / 256-bit stores, and the four lanes that
// share a 4-byte group of the scale tile merge their bytes by shuffle into one 32-bit
// store.  The thread grid spans the *padded* scale tensor so that its padding bytes are
// written as zero by the same launch (no separate memset).
//
// Arithmetic contract: results are bit-identical to the reference's eager path
// (comfy_kitchen/backends/eager/quantization.py:115-160 and :257-324), which uses true
// IEEE fp32 divisions.  This translation unit is therefore compiled without fast-math,
// and every division below is either __fdiv_rn or a reciprocal-FMA sequence that is
// proven to round identically (see div_markstein).
#include "ck_quant_math.cuh"

#include <atomic>
#include <cstdlib>
#include <type_traits>

namespace ck {
namespace {

using namespace quant;

constexpr int kColsPerBlock = 64;  // scale columns per thread block (two warps wide)
constexpr int kRowsPerBlock = 4;
constexpr int kThreads = kColsPerBlock * kRowsPerBlock;

// ---------------------------------------------------------------------------
// loading N consecutive elements of one row as exact float values
// ---------------------------------------------------------------------------
template <typename T>
struct SrcTraits;
template <>
struct SrcTraits<__nv_bfloat16> {
  __device__ static float to_f32(const __nv_bfloat16& v) { return __bfloat162float(v); }
};
template <>
struct SrcTraits<__half> {
  __device__ static float to_f32(const __half& v) { return __half2float(v); }
};
template <>
struct SrcTraits<float> {
  __device__ static float to_f32(const float& v) { return v; }
};

// 16 consecutive elements starting at `p` (32-byte aligned for 2-byte types).
template <typename T>
__device__ __forceinline__ void load16_vec(const T* p, float (&v)[16]) {
  if constexpr (sizeof(T) == 2) {
    const Vec256 raw = ld_global_stream_256(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        v[2 * i] = __uint_as_float(raw.w[i] << 16);
        v[2 * i + 1] = __uint_as_float(raw.w[i] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw.w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
    }
  } else {
    const Vec256 lo = ld_global_stream_256(p);
    const Vec256 hi = ld_global_stream_256(p + 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = __uint_as_float(lo.w[i]);
      v[8 + i] = __uint_as_float(hi.w[i]);
    }
  }
}

// Same, element by element with bounds checks (ragged or misaligned inputs).
template <typename T>
__device__ __forceinline__ void load16_guarded(const T* base, int64_t row, int64_t col0, int64_t rows, int64_t cols,
                                               float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t c = col0 + i;
    v[i] = (row < rows && c < cols) ? SrcTraits<T>::to_f32(base[row * cols + c]) : 0.0f;
  }
}

// Executed by every lane of the warp; lanes past the padded width (`inside` false) do not store.
__device__ __forceinline__ void store_scale_quad(uint8_t* scales, int64_t row, int64_t sc, int64_t col_tiles,
                                                 uint32_t byte, bool inside) {
  uint32_t w = byte | (__shfl_xor_sync(0xFFFFFFFFu, byte, 1) << 8);
  w |= __shfl_xor_sync(0xFFFFFFFFu, w, 2) << 16;
  if (inside && (sc & 3) == 0) {
    *reinterpret_cast<uint32_t*>(scales + swizzled_scale_offset(row, sc, col_tiles)) = w;
  }
}

// A thread owns one (row, scale column) of the padded scale tensor [rows_pad, sc_pad]:
// block = (kColsPerBlock scale columns, kRowsPerBlock rows), grid = (row groups, column
// chunks).  sc_pad is a multiple of 4 and a warp is 32 consecutive scale columns of one
// row, so aligned lane quads share a row and a 4-byte scale group.
template <typename T, bool kVec, bool kFastDiv>
__global__ void __launch_bounds__(kThreads)
quantize_nvfp4_kernel(const T* x, const float* global_scale, uint8_t* __restrict__ codes,
                      uint8_t* __restrict__ scales, int64_t orig_rows, int64_t orig_cols, int64_t num_rows,
                      int64_t num_cols, int64_t sc_pad, int hi_first) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t sc = blockIdx.y * kColsPerBlock + threadIdx.x;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + threadIdx.y;
  const int64_t n_sc = num_cols >> 4;
  uint32_t scale_byte = 0;
  if (row < num_rows && sc < n_sc) {
    float v[16];
    if constexpr (kVec) {
      load16_vec(x + row * orig_cols + sc * 16, v);
    } else {
      load16_guarded(x, row, sc * 16, orig_rows, orig_cols, v);
    }
    const float g = ld_f32_dependent(global_scale);
    uint32_t lo, hi;
    nvfp4_block<kFastDiv>(v, g, hi_first != 0, lo, hi, scale_byte);
    *reinterpret_cast<uint2*>(codes + row * (num_cols >> 1) + sc * 8) = make_uint2(lo, hi);
  }
  store_scale_quad(scales, row, sc, sc_pad >> 2, scale_byte, sc < sc_pad);
}

// Streaming variant for 16-bit inputs whose rows are whole pairs of scale blocks (32
// elements) and need no padding of the data: a thread owns two adjacent blocks of one row
// (two 256-bit loads, one 128-bit code store), the two lanes that share a 4-byte scale group
// merge with one shuffle, per-thread constants (tensor scale, its reciprocal) are set up
// once, and a block of 32 x 8 threads walks row groups with a grid stride so that every SM
// holds the same amount of work.
constexpr int kPairRows = 16;  // rows per thread block; 32 lanes x 2 blocks x 16 = 1024 columns per warp

template <typename T, bool kHiFirst>
__global__ void __launch_bounds__(32 * kPairRows, 2)
quantize_nvfp4_pair_kernel(const T* x, const float* global_scale,
                           uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int rows, int cols,
                           int rows_pad, int sc_pad, int row_groups) {
  pdl_launch_dependents();
  const int pc = blockIdx.y * 32 + threadIdx.x;  // scale columns 2*pc and 2*pc + 1
  const bool has_data = pc < (cols >> 5);
  const bool has_scale = (threadIdx.x & 1) == 0 && 2 * pc < sc_pad;
  // Ahead of the dependency wait: ask L2 for this block's first two row groups.  A prefetch only
  // warms the cache (L2 is the point of coherence: what the previous kernel still writes is seen
  // by the loads after the wait), and it takes the DRAM latency of the first loads off the
  // critical path of a kernel that only runs for a few microseconds.
  if (has_data && (threadIdx.x & 1) == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = (blockIdx.x + i * gridDim.x) * kPairRows + threadIdx.y;
      if (row < rows) prefetch_l2(x + static_cast<int64_t>(row) * cols + pc * 32);  // one 128-byte line per lane pair
    }
  }
  pdl_wait();  // the tensor scale and x may come from the kernel before this one
  const TensorScale ts = make_tensor_scale(ld_f32_dependent(global_scale));
  const int col_tiles = sc_pad >> 2;
  const int code_pitch = cols >> 1;
  // The loads of the next row group are issued before the arithmetic of the current one, so
  // memory stays busy while the warps compute.
  Vec256 a = {}, b = {};
  {
    const int row = blockIdx.x * kPairRows + threadIdx.y;
    if (has_data && row < rows) {
      const T* src = x + static_cast<int64_t>(row) * cols + pc * 32;
      a = ld_global_stream_256(src);
      b = ld_global_stream_256(src + 16);
    }
  }
  for (int rg = blockIdx.x; rg < row_groups; rg += gridDim.x) {
    const int row = rg * kPairRows + threadIdx.y;
    const int next_row = row + gridDim.x * kPairRows;
    Vec256 an = {}, bn = {};
    if (has_data && next_row < rows) {
      const T* src = x + static_cast<int64_t>(next_row) * cols + pc * 32;
      an = ld_global_stream_256(src);
      bn = ld_global_stream_256(src + 16);
    }
    uint32_t sb = 0;
    if (has_data && row < rows) {
      uint32_t w0, w1, w2, w3, s0, s1;
      nvfp4_block_packed<T, kHiFirst>(a.w, ts, w0, w1, s0);
      nvfp4_block_packed<T, kHiFirst>(b.w, ts, w2, w3, s1);
      *reinterpret_cast<uint4*>(codes + static_cast<int64_t>(row) * code_pitch + pc * 16) = make_uint4(w0, w1, w2, w3);
      sb = s0 | (s1 << 8);
    }
    const uint32_t word = sb | (__shfl_xor_sync(0xFFFFFFFFu, sb, 1) << 16);
    if (has_scale && row < rows_pad) {
      *reinterpret_cast<uint32_t*>(scales + swizzled_scale_offset(row, 2 * pc, col_tiles)) = word;
    }
    a = an;
    b = bn;
  }
}

// ---------------------------------------------------------------------------
// MXFP8
// ---------------------------------------------------------------------------
// clamp(ceil(log2(r)) + 127, 0, 254) for r >= 2^-127, from the bits of r
// (comfy_kitchen/backends/eager/quantization.py:295-300).  r = amax/448 with amax an
// f16/bf16 number is either an exact power of two or far enough from one that the
// reference's float32 log2 cannot round across an integer, so this integer form is
// bit-identical for those input types.
__device__ __forceinline__ uint32_t e8m0_ceil_exponent(float r) {
  const uint32_t bits = __float_as_uint(r);
  const uint32_t e = bits >> 23;  // r > 0
  const uint32_t frac = bits & 0x7FFFFFu;
  uint32_t biased;
  if (e == 0) {
    biased = frac > 0x400000u ? 1u : 0u;  // [2^-127, 2^-126): exactly 2^-127 -> 0
  } else {
    biased = e + (frac != 0u);
  }
  return min(biased, 254u);
}

template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads)
quantize_mxfp8_kernel(const T* x, uint8_t* __restrict__ data, uint8_t* __restrict__ scales,
                      int64_t orig_rows, int64_t orig_cols, int64_t num_rows, int64_t num_cols, int64_t sc_pad) {
  pdl_launch_dependents();
  const int64_t sc = blockIdx.y * kColsPerBlock + threadIdx.x;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + threadIdx.y;
  const int64_t n_sc = num_cols >> 5;
  if constexpr (kVec) {
    // ahead of the dependency wait: ask L2 for the thread pair's 128-byte line (warms the cache only)
    if (row < num_rows && sc < n_sc && (threadIdx.x & 1) == 0) prefetch_l2(x + row * orig_cols + sc * 32);
  }
  pdl_wait();
  uint32_t scale_byte = 0;
  if (row < num_rows && sc < n_sc) {
    float lo[16], hi[16];
    if constexpr (kVec) {
      load16_vec(x + row * orig_cols + sc * 32, lo);
      load16_vec(x + row * orig_cols + sc * 32 + 16, hi);
    } else {
      load16_guarded(x, row, sc * 32, orig_rows, orig_cols, lo);
      load16_guarded(x, row, sc * 32 + 16, orig_rows, orig_cols, hi);
    }
    const float amax = fmaxf(amax16(lo), amax16(hi));          // :292
    const float need = fmaxf(__fdiv_rn(amax, 448.0f), 0x1p-127f);  // :294-295
    const uint32_t e = e8m0_ceil_exponent(need);               // :298-302
    const bool dead = (amax == 0.0f);                          // :306
    // :303-310: divide by 2^(e-127).  For e in [1, 253] that is an exact multiplication by
    // 2^(127-e); e == 254 needs the subnormal 2^-127; e == 0 decodes to a zero scale and
    // the reference divides by zero (inputs below 448 * 2^-127, outside the pinned domain).
    float inv;
    if (e == 0) {
      inv = __int_as_float(0x7F800000);
    } else if (e == 254) {
      inv = 0x1p-127f;
    } else {
      inv = __uint_as_float((254u - e) << 23);
    }
    if (dead) inv = 0.0f;  // :307,311 -> all zeros (positive)
    Vec256 out;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // :314-315 clamp to +-448 and round to E4M3: satfinite performs the clamp
      const uint32_t p0 = f32x2_to_e4m3x2(dead ? 0.0f : lo[4 * i + 1] * inv, dead ? 0.0f : lo[4 * i] * inv);
      const uint32_t p1 = f32x2_to_e4m3x2(dead ? 0.0f : lo[4 * i + 3] * inv, dead ? 0.0f : lo[4 * i + 2] * inv);
      out.w[i] = p0 | (p1 << 16);
      const uint32_t p2 = f32x2_to_e4m3x2(dead ? 0.0f : hi[4 * i + 1] * inv, dead ? 0.0f : hi[4 * i] * inv);
      const uint32_t p3 = f32x2_to_e4m3x2(dead ? 0.0f : hi[4 * i + 3] * inv, dead ? 0.0f : hi[4 * i + 2] * inv);
      out.w[4 + i] = p2 | (p3 << 16);
    }
    st_global_256(data + row * num_cols + sc * 32, out);
    scale_byte = dead ? 0u : e;  // :318
  }
  store_scale_quad(scales, row, sc, sc_pad >> 2, scale_byte, sc < sc_pad);
}

std::atomic<int> g_exact_division{-1};  // -1: not set, follow CK_EXACT_DIV

bool use_exact_division() {
  const int v = g_exact_division.load(std::memory_order_relaxed);
  if (v >= 0) return v != 0;
  // CK_EXACT_DIV=1 forces __fdiv_rn for every element (validation of the fast quotient).
  static const bool env = [] {
    const char* e = getenv("CK_EXACT_DIV");
    return e != nullptr && e[0] == '1';
  }();
  return env;
}

template <typename T>
int launch_nvfp4(const void* input, const float* gs, void* codes, void* scales, int64_t orig_rows, int64_t orig_cols,
                 int64_t num_rows, int64_t num_cols, int hi_first, cudaStream_t stream) {
  const int64_t sc_pad = round_up(num_cols / 16, 4);
  const int64_t grid_rows = round_up(num_rows, 128) / kRowsPerBlock;
  const int64_t grid_cols = ceil_div(sc_pad, kColsPerBlock);
  CK_REQUIRE(grid_rows <= 0x7FFFFFFF && grid_cols <= 65535, "quantize_nvfp4: tensor too large for one launch");
  const dim3 grid(static_cast<unsigned>(grid_rows), static_cast<unsigned>(grid_cols)), block(kColsPerBlock, kRowsPerBlock);
  // vector path: every 16-element run is inside the input and 32-byte aligned
  const bool vec = (orig_rows == num_rows) && (orig_cols == num_cols) &&
                   (reinterpret_cast<uintptr_t>(input) % 32 == 0);
  const T* x = static_cast<const T*>(input);
  uint8_t* c = static_cast<uint8_t*>(codes);
  uint8_t* s = static_cast<uint8_t*>(scales);
  const bool exact = use_exact_division();
  if constexpr (sizeof(T) == 2) {
    if (vec && !exact && num_cols % 32 == 0 && reinterpret_cast<uintptr_t>(codes) % 16 == 0 &&
        num_rows < (1 << 30) && num_cols < (1 << 30)) {
      const int rows_pad = static_cast<int>(round_up(num_rows, 128));
      const int row_groups = rows_pad / kPairRows;
      const int col_chunks = static_cast<int>(ceil_div(sc_pad, 64));
      auto kernel = hi_first ? quantize_nvfp4_pair_kernel<T, true> : quantize_nvfp4_pair_kernel<T, false>;
      // All blocks resident at once and all of the same length: the grid is the number of
      // row groups divided into the fewest equal passes that fit the device.
      static std::atomic<int> blocks_per_sm[2] = {{0}, {0}};
      int per_sm = blocks_per_sm[hi_first ? 1 : 0].load(std::memory_order_relaxed);
      if (per_sm == 0) {
        CK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 32 * kPairRows, 0));
        per_sm = max(per_sm, 1);
        blocks_per_sm[hi_first ? 1 : 0].store(per_sm, std::memory_order_relaxed);
      }
      const int per_wave = max(1, sm_count() * per_sm / col_chunks);
      const int waves = static_cast<int>(ceil_div(row_groups, per_wave));
      const int grid_x = static_cast<int>(ceil_div(row_groups, waves));
      const dim3 pgrid(static_cast<unsigned>(grid_x), static_cast<unsigned>(col_chunks)), pblock(32, kPairRows);
      CK_CUDA(launch_pdl(kernel, pgrid, pblock, 0, stream, x, gs, c, s, static_cast<int>(num_rows),
                         static_cast<int>(num_cols), rows_pad, static_cast<int>(sc_pad), row_groups));
      return CK_OK;
    }
  }
#define CK_LAUNCH(VEC, FAST)                                                                                  \
  CK_CUDA(launch_pdl(quantize_nvfp4_kernel<T, VEC, FAST>, grid, block, 0, stream, x, gs, c, s, orig_rows, orig_cols, \
                     num_rows, num_cols, sc_pad, hi_first))
  if (vec) {
    if (exact) CK_LAUNCH(true, false); else CK_LAUNCH(true, true);
  } else {
    if (exact) CK_LAUNCH(false, false); else CK_LAUNCH(false, true);
  }
#undef CK_LAUNCH
  CK_CUDA(cudaGetLastError());
  return CK_OK;
}

template <typename T>
int launch_mxfp8(const void* input, void* data, void* scales, int64_t orig_rows, int64_t orig_cols, int64_t num_rows,
                 int64_t num_cols, cudaStream_t stream) {
  const int64_t sc_pad = round_up(num_cols / 32, 4);
  const int64_t grid_rows = round_up(num_rows, 128) / kRowsPerBlock;
  const int64_t grid_cols = ceil_div(sc_pad, kColsPerBlock);
  CK_REQUIRE(grid_rows <= 0x7FFFFFFF && grid_cols <= 65535, "quantize_mxfp8: tensor too large for one launch");
  const dim3 grid(static_cast<unsigned>(grid_rows), static_cast<unsigned>(grid_cols)), block(kColsPerBlock, kRowsPerBlock);
  const bool vec = (orig_rows == num_rows) && (orig_cols == num_cols) &&
                   (reinterpret_cast<uintptr_t>(input) % 32 == 0) && (reinterpret_cast<uintptr_t>(data) % 32 == 0);
  const T* x = static_cast<const T*>(input);
  uint8_t* d = static_cast<uint8_t*>(data);
  uint8_t* s = static_cast<uint8_t*>(scales);
  if (vec) {
    CK_CUDA(launch_pdl(quantize_mxfp8_kernel<T, true>, grid, block, 0, stream, x, d, s, orig_rows, orig_cols, num_rows,
                       num_cols, sc_pad));
  } else {
    CK_REQUIRE(reinterpret_cast<uintptr_t>(data) % 32 == 0, "quantize_mxfp8: output must be 32-byte aligned");
    CK_CUDA(launch_pdl(quantize_mxfp8_kernel<T, false>, grid, block, 0, stream, x, d, s, orig_rows, orig_cols, num_rows,
                       num_cols, sc_pad));
  }
  CK_CUDA(cudaGetLastError());
  return CK_OK;
}

int check_quant_shapes(const char* op, int64_t block, const void* input, const void* out, const void* scales,
                       int64_t orig_rows, int64_t orig_cols, int64_t num_rows, int64_t num_cols) {
  CK_REQUIRE(input && out && scales, "%s: null pointer", op);
  CK_REQUIRE(orig_rows > 0 && orig_cols > 0, "%s: empty input [%lld, %lld]", op, (long long)orig_rows,
             (long long)orig_cols);
  CK_REQUIRE(num_cols % block == 0, "%s: num_cols=%lld is not a multiple of %lld", op, (long long)num_cols,
             (long long)block);
  const bool same = (num_rows == orig_rows && num_cols == orig_cols);
  const bool padded = (num_rows == round_up(orig_rows, block) && num_cols == round_up(orig_cols, block));
  CK_REQUIRE(same || padded, "%s: output [%lld, %lld] is neither the input shape [%lld, %lld] nor its %lld-padding",
             op, (long long)num_rows, (long long)num_cols, (long long)orig_rows, (long long)orig_cols,
             (long long)block);
  CK_REQUIRE(reinterpret_cast<uintptr_t>(scales) % 4 == 0, "%s: block_scales must be 4-byte aligned", op);
  return CK_OK;
}

}  // namespace
}  // namespace ck

extern "C" int ck_debug_set_exact_division(int on) {
  const bool before = ck::use_exact_division();
  ck::g_exact_division.store(on != 0 ? 1 : 0, std::memory_order_relaxed);
  return before ? 1 : 0;
}

extern "C" int ck_quantize_nvfp4(const void* input, int input_dtype, const float* global_scale, void* codes,
                                 void* block_scales, int64_t orig_rows, int64_t orig_cols, int64_t num_rows,
                                 int64_t num_cols, int hi_first, void* stream) {
  using namespace ck;
  if (int rc = check_quant_shapes("quantize_nvfp4", 16, input, codes, block_scales, orig_rows, orig_cols, num_rows,
                                  num_cols))
    return rc;
  CK_REQUIRE(global_scale != nullptr, "quantize_nvfp4: null global_scale");
  CK_REQUIRE(reinterpret_cast<uintptr_t>(codes) % 8 == 0, "quantize_nvfp4: codes must be 8-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (input_dtype) {
    case CK_DTYPE_BF16:
      return launch_nvfp4<__nv_bfloat16>(input, global_scale, codes, block_scales, orig_rows, orig_cols, num_rows,
                                         num_cols, hi_first, s);
    case CK_DTYPE_F16:
      return launch_nvfp4<__half>(input, global_scale, codes, block_scales, orig_rows, orig_cols, num_rows, num_cols,
                                  hi_first, s);
    case CK_DTYPE_F32:
      return launch_nvfp4<float>(input, global_scale, codes, block_scales, orig_rows, orig_cols, num_rows, num_cols,
                                 hi_first, s);
    default:
      return fail(CK_ERR_INVALID_ARGUMENT, "quantize_nvfp4: unsupported input dtype code %d", input_dtype);
  }
}

extern "C" int ck_quantize_mxfp8(const void* input, int input_dtype, void* data, void* block_scales,
                                 int64_t orig_rows, int64_t orig_cols, int64_t num_rows, int64_t num_cols,
                                 void* stream) {
  using namespace ck;
  if (int rc = check_quant_shapes("quantize_mxfp8", 32, input, data, block_scales, orig_rows, orig_cols, num_rows,
                                  num_cols))
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (input_dtype) {
    case CK_DTYPE_BF16:
      return launch_mxfp8<__nv_bfloat16>(input, data, block_scales, orig_rows, orig_cols, num_rows, num_cols, s);
    case CK_DTYPE_F16:
      return launch_mxfp8<__half>(input, data, block_scales, orig_rows, orig_cols, num_rows, num_cols, s);
    case CK_DTYPE_F32:
      return launch_mxfp8<float>(input, data, block_scales, orig_rows, orig_cols, num_rows, num_cols, s);
    default:
      return fail(CK_ERR_INVALID_ARGUMENT, "quantize_mxfp8: unsupported input dtype code %d", input_dtype);
  }
}
