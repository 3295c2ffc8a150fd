// Dynamic per-tensor NVFP4 scale: scale = amax(|x|) / (448 * 6), evaluated the way the
// reference's layout does it (comfy_kitchen/tensor/nvfp4.py:64-69): the maximum and the
// division by 2688 in x's dtype, then a cast to float32.  One pass over x, HBM-bound
// (2 bytes per bf16 element, no output traffic to speak of).
//
// Each thread block reduces a fixed chunk of kChunk elements to one partial maximum in
// scratch memory; the block that finishes last (ticket counter, also in scratch) reduces
// the partials, writes the scale and resets the counter, so the scratch area needs to be
// zeroed only once, before its first use.  Scratch layout: word 0 = ticket counter,
// words 64.. = one float per block (the gap keeps the counter on its own 256-byte line).
#include "ck_common.cuh"

#include <mutex>
#include <type_traits>

namespace ck {
namespace {

constexpr int kThreads = 256;
constexpr int kElemsPerThread = 64;
constexpr int kChunk = kThreads * kElemsPerThread;  // elements per block
constexpr int kPartialOffset = 64;                  // words

template <typename T>
__device__ __forceinline__ float round_to_input_dtype(float v) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    return __bfloat162float(__float2bfloat16_rn(v));
  } else if constexpr (std::is_same<T, __half>::value) {
    return __half2float(__float2half_rn(v));
  } else {
    return v;
  }
}

template <typename T>
__device__ __forceinline__ float abs_max_of_vec(const Vec256& raw) {
  float m = 0.0f;
  if constexpr (sizeof(T) == 2) {
    // |x| of a 16-bit float is its bit pattern without the sign, and for non-negative
    // floats of one format the integer order of the bit patterns is the numeric order:
    // reduce the eight packed pairs as unsigned 16-bit integers, convert once.
    uint32_t p = raw.w[0] & 0x7FFF7FFFu;
#pragma unroll
    for (int i = 1; i < 8; ++i) p = __vmaxu2(p, raw.w[i] & 0x7FFF7FFFu);
    const uint32_t top = max(p & 0xFFFFu, p >> 16);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      m = __uint_as_float(top << 16);
    } else {
      m = __half2float(__ushort_as_half(static_cast<unsigned short>(top)));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(__uint_as_float(raw.w[i])));
  }
  return m;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
nvfp4_tensor_scale_kernel(const T* x, int64_t n, float* scale_out, unsigned int* scratch) {
  constexpr int kPerVec = 32 / sizeof(T);  // elements per 256-bit load
  constexpr int kVecs = kElemsPerThread / kPerVec;
  pdl_launch_dependents();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kChunk;
  float m = 0.0f;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 31u) == 0;
  pdl_wait();  // x may be the output of the kernel before this one
  if (aligned && base + kChunk <= n) {
    // whole chunk in range: all loads are issued before the first one is consumed
    Vec256 raw[kVecs];
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      raw[v] = ld_global_stream_256(x + base + (static_cast<int64_t>(v) * kThreads + threadIdx.x) * kPerVec);
    }
#pragma unroll
    for (int v = 0; v < kVecs; ++v) m = fmaxf(m, abs_max_of_vec<T>(raw[v]));
  } else {
    for (int v = 0; v < kVecs; ++v) {
      const int64_t i = base + (static_cast<int64_t>(v) * kThreads + threadIdx.x) * kPerVec;
      if (aligned && i + kPerVec <= n) {
        m = fmaxf(m, abs_max_of_vec<T>(ld_global_stream_256(x + i)));
      } else {
        for (int j = 0; j < kPerVec; ++j) {
          if (i + j < n) {
            float f;
            if constexpr (std::is_same<T, __nv_bfloat16>::value) f = __bfloat162float(x[i + j]);
            else if constexpr (std::is_same<T, __half>::value) f = __half2float(x[i + j]);
            else f = x[i + j];
            m = fmaxf(m, fabsf(f));
          }
        }
      }
    }
  }
  // block reduction
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  __shared__ float warp_max[kThreads / 32];
  __shared__ bool is_last;
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = warp_max[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) b = fmaxf(b, warp_max[w]);
    reinterpret_cast<float*>(scratch + kPartialOffset)[blockIdx.x] = b;
    __threadfence();
    const unsigned int ticket = atomicAdd(scratch, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  // last block: all partials are visible (each writer fenced before taking its ticket)
  __threadfence();
  float t = 0.0f;
  const volatile float* partials = reinterpret_cast<const volatile float*>(scratch + kPartialOffset);
  for (unsigned int i = threadIdx.x; i < gridDim.x; i += kThreads) t = fmaxf(t, partials[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xFFFFFFFFu, t, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = t;
  __syncthreads();
  if (threadIdx.x == 0) {
    float amax = warp_max[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, warp_max[w]);
    // amax / (448 * 6) in the input dtype (a true division, then rounded), then float32
    *scale_out = round_to_input_dtype<T>(__fdiv_rn(amax, 2688.0f));
    scratch[0] = 0;  // ready for the next call
  }
}

int64_t blocks_for(int64_t n) { return ceil_div(n, kChunk); }

template <typename T>
void launch(const void* x, int64_t n, float* scale_out, unsigned int* scratch, cudaStream_t s) {
  launch_pdl(nvfp4_tensor_scale_kernel<T>, dim3(static_cast<unsigned>(blocks_for(n))), dim3(kThreads), 0, s,
             static_cast<const T*>(x), n, scale_out, scratch);
}

int run(const char* op, const void* x, int dtype, int64_t n, float* scale_out, unsigned int* scratch,
        int64_t scratch_bytes, cudaStream_t s) {
  CK_REQUIRE(x && scale_out && scratch, "%s: null pointer", op);
  CK_REQUIRE(n > 0, "%s: empty input", op);
  const int64_t need = (kPartialOffset + blocks_for(n)) * 4;
  CK_REQUIRE(blocks_for(n) <= 0x7FFFFFFF, "%s: tensor too large", op);
  CK_REQUIRE(scratch_bytes >= need, "%s: %lld elements need %lld bytes of scratch, %lld given", op, (long long)n,
             (long long)need, (long long)scratch_bytes);
  CK_REQUIRE(reinterpret_cast<uintptr_t>(scratch) % 4 == 0, "%s: scratch must be 4-byte aligned", op);
  switch (dtype) {
    case CK_DTYPE_BF16: launch<__nv_bfloat16>(x, n, scale_out, scratch, s); break;
    case CK_DTYPE_F16: launch<__half>(x, n, scale_out, scratch, s); break;
    case CK_DTYPE_F32: launch<float>(x, n, scale_out, scratch, s); break;
    default: return fail(CK_ERR_INVALID_ARGUMENT, "%s: unsupported input dtype code %d", op, dtype);
  }
  CK_CUDA(cudaGetLastError());
  return CK_OK;
}

// ---------------------------------------------------------------------------
// Variant with built-in scratch, for callers that must not allocate.
// ---------------------------------------------------------------------------
// The partial maxima and the ticket counter live in this fixed device array instead of a
// caller-supplied buffer.  It exists once per GPU that loads the library and stays
// resident until the process exits.  In host code the name below is only a handle, not a
// device address; the address is looked up once per device (static_scratch_for_device).
constexpr int64_t kStaticMaxBlocks = 8192;                           // 32 KiB of partials
constexpr int64_t kStaticMaxElements = kStaticMaxBlocks * kChunk;    // 134 217 728 elements
static __device__ __align__(256) unsigned int g_static_scratch[kPartialOffset + kStaticMaxBlocks];

// Device address of g_static_scratch on the current device.  The first call on a device
// performs the lookup (which may make the runtime load this module), later calls reuse it.
int static_scratch_for_device(unsigned int** out) {
  static std::mutex mu;
  static unsigned int* per_device[64] = {nullptr};
  int dev = 0;
  CK_CUDA(cudaGetDevice(&dev));
  CK_REQUIRE(dev >= 0 && dev < 64, "nvfp4_tensor_scale_noalloc: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    unsigned int* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      return fail(CK_ERR_CUDA, "cudaGetSymbolAddress(g_static_scratch) failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    }
    per_device[dev] = ptr;
  }
  *out = per_device[dev];
  return CK_OK;
}

}  // namespace
}  // namespace ck

extern "C" int ck_nvfp4_tensor_scale_noalloc(const void* input, int input_dtype, int64_t num_elements,
                                             float* scale_out, void* stream) {
  using namespace ck;
  CK_REQUIRE(num_elements <= kStaticMaxElements,
             "nvfp4_tensor_scale_noalloc: %lld elements exceed the built-in scratch (at most %lld elements); use "
             "ck_nvfp4_tensor_scale with your own scratch buffer",
             (long long)num_elements, (long long)kStaticMaxElements);
  unsigned int* scratch = nullptr;
  if (int rc = static_scratch_for_device(&scratch)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  Only the ticket counter has to start
  // at zero (every partial that is read is written first); clear it in stream order.
  CK_CUDA(cudaMemsetAsync(scratch, 0, sizeof(unsigned int), s));
  return run("nvfp4_tensor_scale_noalloc", input, input_dtype, num_elements, scale_out, scratch,
             static_cast<int64_t>(sizeof(unsigned int)) * (kPartialOffset + kStaticMaxBlocks), s);
}

extern "C" int64_t ck_nvfp4_tensor_scale_scratch_bytes(int64_t num_elements) {
  if (num_elements <= 0) return 0;
  return (ck::kPartialOffset + ck::blocks_for(num_elements)) * 4;
}

extern "C" int ck_nvfp4_tensor_scale(const void* input, int input_dtype, int64_t num_elements, float* scale_out,
                                     void* scratch, int64_t scratch_bytes, void* stream) {
  return ck::run("nvfp4_tensor_scale", input, input_dtype, num_elements, scale_out,
                 static_cast<unsigned int*>(scratch), scratch_bytes, static_cast<cudaStream_t>(stream));
}
