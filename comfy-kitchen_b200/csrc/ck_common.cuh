// Shared host/device helpers of the sm_100a quantized-linear library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>

#include "../../include/ck_b200.h"

namespace ck {

// ---- error reporting --------------------------------------------------------
// The message buffer is thread-local: the C entry points are re-entrant and a
// failure on one thread never overwrites the message another thread reads.
char* last_error_buffer();
int fail(int code, const char* fmt, ...);

#define CK_REQUIRE(cond, ...)                                            \
  do {                                                                   \
    if (!(cond)) return ::ck::fail(CK_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define CK_CUDA(call)                                                              \
  do {                                                                             \
    cudaError_t e__ = (call);                                                      \
    if (e__ != cudaSuccess)                                                        \
      return ::ck::fail(CK_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

__host__ __device__ constexpr int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
__host__ __device__ constexpr int64_t ceil_div(int64_t x, int64_t m) { return (x + m - 1) / m; }

// Number of SMs of the current device (cached per device).
int sm_count();

// Device address of the GEMM kernels' status word on the current device (ck_gemm.cu).
int gemm_status_word(int** out);

// Caller-owned GEMM workspace: the first kWorkspaceTicketBytes hold the arrival counters of the
// small-M path (zero before the first use, left zero by every call); partial tiles of either
// split-K path follow.
constexpr int64_t kWorkspaceTicketBytes = 65536;

// GEMMs with few activation rows (ck_gemm_smallm.cu).
bool small_m_applies(int64_t M, int64_t N, int64_t K);
int64_t small_m_workspace_bytes(bool is_mxfp8, int64_t M, int64_t N, int64_t K);
int scaled_mm_small_m(bool is_mxfp8, const void* a, const void* b, const void* sfa, const void* sfb, const float* tsa,
                      const float* tsb, const float* alpha, const void* bias, int bias_dtype, void* out, int out_dtype,
                      int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes, cudaStream_t stream);

// ---- programmatic dependent launch ------------------------------------------------------
// The streaming kernels and the GEMMs of this library are launched with programmatic stream
// serialization: each kernel lets its successor start being scheduled at once
// (pdl_launch_dependents at its top) and itself waits for its predecessor in the stream to
// have completed and flushed (pdl_wait) before it touches global memory.  The successor's
// launch latency and set-up then overlap the predecessor's tail instead of following it.
// A kernel launched this way behind a kernel that never triggers simply starts when that one
// ends; CK_PDL=0 turns the attribute off.
bool pdl_enabled();

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---- swizzled scale layout --------------------------------------------------
// Byte offset of the scale of (row r, scale column c) in the 128x4-tiled
// buffer: each tile of 128 rows x 4 columns is 512 contiguous bytes laid out
// as 32 rows of 16 bytes; `col_tiles` = ceil(columns / 4).
__host__ __device__ __forceinline__ int64_t swizzled_scale_offset(int64_t r, int64_t c, int64_t col_tiles) {
  const int64_t tile = (r >> 7) * col_tiles + (c >> 2);
  return tile * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c & 3);
}

// ---- 256-bit global memory access (sm_100) ------------------------------------
struct __align__(32) Vec256 {
  uint32_t w[8];
};

__device__ __forceinline__ Vec256 ld_global_stream_256(const void* p) {
  Vec256 r;
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]),
                 "=r"(r.w[6]), "=r"(r.w[7])
               : "l"(p));
  return r;
}

// Scalar read of a value the previous kernel in the stream may have produced (a tensor scale,
// alpha).  Kernels launched with programmatic stream serialization start before their predecessor
// has finished; a read-only-cache load (__ldg, or what the compiler makes of a const __restrict__
// pointer) is "invariant" to the compiler, which may then hoist it above griddepcontrol.wait and
// read the value of the launch before.  This is an ordinary coherent load that stays where it is.
__device__ __forceinline__ float ld_f32_dependent(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Ask L2 for the 128-byte line that holds *p (no data is returned, nothing is tracked).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ void st_global_256(void* p, const Vec256& r) {
  asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.w[0]), "r"(r.w[1]),
               "r"(r.w[2]), "r"(r.w[3]), "r"(r.w[4]), "r"(r.w[5]), "r"(r.w[6]), "r"(r.w[7])
               : "memory");
}

// The same store without a line allocated in L1: for results that this SM will not read again.  In
// the GEMM epilogue (32 rows = 32 lines per store instruction) it is 3-5 % of the kernel's time.
__device__ __forceinline__ void st_global_256_no_allocate(void* p, const Vec256& r) {
  asm volatile("st.global.L1::no_allocate.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.w[0]), "r"(r.w[1]),
               "r"(r.w[2]), "r"(r.w[3]), "r"(r.w[4]), "r"(r.w[5]), "r"(r.w[6]), "r"(r.w[7])
               : "memory");
}

}  // namespace ck
