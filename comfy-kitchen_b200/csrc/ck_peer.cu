// Cross-GPU barrier for the column-sharded GEMM with a fused all-gather: every rank's GEMM
// stores its output tiles into all ranks' result buffers (peer memory over NVLink); this
// kernel, launched behind the GEMM on every rank, tells the other ranks "my stores are done"
// and waits until all of them have said the same.
//
// Each rank owns an array of `world` 32-bit flags that is mapped into every process.  Rank r
// writes `epoch` into slot r of every rank's array (system-scope release, after a system-scope
// fence that orders the GEMM's peer stores before it) and polls the slots of its own array
// (system-scope acquire).  The wait is bounded: after about a second without progress the
// kernel records an error status (ck_peer_status) and returns, so a rank that never arrives
// cannot hang the others.  One launch per GPU - the ranks that wait on one another run on
// different devices.
#include "ck_common.cuh"

namespace ck {
namespace {

constexpr int kMaxRanks = 8;
constexpr uint32_t kPollLimit = 1u << 20;     // x (500 ns sleep + one remote read) ~ 1 s
constexpr uint32_t kMaxPollLimit = 1u << 26;  // callers may raise the bound, but it stays finite (~1 min)

struct PeerFlags {
  uint32_t* ptr[kMaxRanks];
};

__device__ int g_peer_status = 0;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void peer_barrier_kernel(const PeerFlags flags, int rank, int world, uint32_t epoch, uint32_t poll_limit,
                                    int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys(flags.ptr[t] + rank, epoch);
  const uint32_t* mine = flags.ptr[rank] + t;
  for (uint32_t i = 0; i < poll_limit; ++i) {
    // epochs only grow; a signed difference keeps the test valid across wrap-around
    if (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) >= 0) return;
    __nanosleep(500);
  }
  atomicExch(status, 1 + t);  // rank t never arrived
}

}  // namespace
}  // namespace ck

extern "C" int ck_peer_barrier_bounded(void* const* flag_ptrs, int rank, int world, uint32_t epoch, uint32_t max_polls,
                                       void* stream) {
  using namespace ck;
  CK_REQUIRE(max_polls >= 1 && max_polls <= kMaxPollLimit, "peer_barrier: poll limit %u outside [1, %u]", max_polls,
             kMaxPollLimit);
  CK_REQUIRE(flag_ptrs != nullptr, "peer_barrier: null flag pointers");
  CK_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "peer_barrier: rank %d of %d", rank, world);
  PeerFlags f = {};
  for (int r = 0; r < world; ++r) {
    CK_REQUIRE(flag_ptrs[r] != nullptr && reinterpret_cast<uintptr_t>(flag_ptrs[r]) % 4 == 0,
               "peer_barrier: flag array of rank %d is null or misaligned", r);
    f.ptr[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  }
  int* status = nullptr;
  CK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_peer_status));
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, rank, world, epoch, max_polls, status);
  CK_CUDA(cudaGetLastError());
  return CK_OK;
}

extern "C" int ck_peer_barrier(void* const* flag_ptrs, int rank, int world, uint32_t epoch, void* stream) {
  return ck_peer_barrier_bounded(flag_ptrs, rank, world, epoch, ck::kPollLimit, stream);
}

extern "C" int ck_peer_status(int* status_out) {
  using namespace ck;
  int v = 0;
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyFromSymbol(&v, g_peer_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    CK_CUDA(cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int)));
  }
  if (status_out != nullptr) *status_out = v;
  return CK_OK;
}
