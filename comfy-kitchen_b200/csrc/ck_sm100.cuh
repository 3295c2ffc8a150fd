// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use: mbarriers with
// bounded waits, TMA (tiled and linear bulk copies into shared memory), tensor memory
// allocation, tcgen05 block-scaled MMA, tcgen05.cp / tcgen05.ld, and the shared-memory /
// instruction descriptor encodings.
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the driver is resolved at run time)

#include "ck_common.cuh"

namespace ck {
namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait in the GEMM kernels goes through this function.  It gives up after
// `kSpinLimit` polls (each poll itself blocks for a hardware-defined interval), records
// the failure in the CTA-wide `abort_flag` (shared memory) and returns false.  Once the
// flag is set every later wait of the CTA returns immediately, so a protocol error
// degrades into wrong output plus an error status, never into a hang.
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;  // common case: no shared-memory read of the flag
  if (*abort_flag) return false;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// ---------------------------------------------------------------------------
// thread-block clusters (CTA pairs)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// Cluster-wide barrier in its two halves: every thread of every CTA of the cluster arrives
// once and waits once per phase (whole warps, converged).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
  cluster_arrive();
  cluster_wait();
}

// CTA-local named barrier `id` (1..15) over `threads` threads: arrive without waiting / wait.
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Arrive on an mbarrier of another CTA of the cluster (address from map_to_cta).  The
// barriers of the GEMM kernels order tensor-memory and asynchronous-proxy traffic only (the
// tcgen05 fences and commits carry that ordering), never data written with ordinary stores,
// so CTA-scope barrier semantics are enough for waits and arrivals that cross the pair; the
// cluster-scope forms cost several hundred cycles per call.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// One lane of a converged warp (the same lane every time for a full warp).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xFFFFFFFF;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tiled load: box at (x = innermost coordinate in elements, y = row) -> shared memory.
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Asks L2 for the box a later tiled load will fetch (no destination, nothing to wait for).  The
// same alignment rule as for the load: x * element size a multiple of 16 bytes.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y)
               : "memory");
}

// CTA-pair forms: the data lands in the executing CTA's shared memory, the byte count is
// reported to the barrier at the same offset in the pair's leader (even-ranked) CTA.  In the
// cluster-wide shared address space bit 24 of an address selects the CTA of the pair.
constexpr uint32_t kPairLeaderMask = 0xFEFFFFFFu;

__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & kPairLeaderMask), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                                 int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & kPairLeaderMask), "r"(x), "r"(y),
      "r"(z)
      : "memory");
}

// Linear bulk copy global -> shared memory; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// 2-D tiled store shared memory -> global (bulk async group of the executing thread).  The
// box is clipped at the tensor's bounds; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d_addr(const CUtensorMap* map, uint32_t smem_addr, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_addr), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once the bulk stores committed by this thread have finished READING shared memory.
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Returns once they have completed entirely (writes performed).
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// ... until at most kPending of them are still reading.
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

__device__ __forceinline__ void st_shared_128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ---------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------
// Executed by one whole warp (with CTAS == 2: by the same warp of both CTAs of the pair, with
// the same shared-memory offset).  Writes the base address of `ncols` columns to *smem_dst.
template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  if constexpr (CTAS == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}

template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTAS == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  }
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrive on the mbarrier at shared::cluster address `bar_addr` (own CTA or the pair's other
// CTA) once every tcgen05 operation issued so far by this thread has completed.
template <int CTAS>
__device__ __forceinline__ void tc_commit(uint32_t bar_addr) {
  if constexpr (CTAS == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr)
                 : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr)
                 : "memory");
  }
}

// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated into the
// four 32-lane quarters (the layout block-scaled MMAs read their scale factors from).
// With CTAS == 2 each CTA of the pair copies from its own shared memory to its own tensor memory.
template <int CTAS>
__device__ __forceinline__ void tc_copy_scales_32x128b(uint32_t taddr, uint64_t sdesc) {
  if constexpr (CTAS == 1) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
  } else {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
  }
}

// One warp reads 32 lanes x 32 consecutive 32-bit columns: thread i gets row (lane base + i).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------
// 64-bit shared-memory matrix descriptor: start address [0,14) and the two byte offsets
// [16,30), [32,46) in units of 16 bytes, descriptor version 1 in [46,48), swizzle mode in
// [61,64) (0 = none, 2 = 128-byte).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes,
                                                   uint32_t swizzle_mode) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(swizzle_mode & 7u) << 61;
  return d;
}

__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// K-major operand tile whose rows are 128 bytes, written by TMA with the 128-byte swizzle:
// 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_operand_desc_sw128(uint32_t smem_addr) {
  return make_smem_desc(smem_addr, 16, 1024, 2);
}

// One 512-byte scale tile (32 rows x 16 bytes, unswizzled): 8-row groups are 128 bytes apart.
__device__ __forceinline__ uint64_t make_scale_desc(uint32_t smem_addr) { return make_smem_desc(smem_addr, 0, 128, 0); }

// 32-bit instruction descriptor of the block-scaled MMA kinds: operand formats [7,10) and
// [10,13), both operands K-major (bits 15, 16 clear), N/8 in [17,23), scale format in bit
// 23 (0 = E4M3, 1 = E8M0), M/16 in [24,29); the scale-factor ids (byte of the 32-bit scale
// column the MMA uses) go to [4,6) for B and [29,31) for A.
__host__ __device__ constexpr uint32_t make_block_scaled_idesc(uint32_t ab_format, uint32_t scale_is_e8m0, uint32_t m,
                                                               uint32_t n) {
  return (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | (scale_is_e8m0 << 23) | ((m >> 4) << 24);
}

__device__ __forceinline__ uint32_t idesc_with_scale_ids(uint32_t idesc, uint32_t sf_id) {
  return idesc | (sf_id << 4) | (sf_id << 29);
}

// D[tmem] (+)= A[smem] * B[smem]^T with per-block scales read from tensor memory.
// NVFP4: E2M1 operands, E4M3 scales, one scale per 16 elements, K = 64 per instruction.
// With CTAS == 2 one instruction drives the tensor cores of both CTAs of the pair: M = 256
// (128 rows of A from each CTA), each CTA supplies half of B's rows and accumulates its own
// 128 x N block in its own tensor memory.
template <int CTAS>
__device__ __forceinline__ void mma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if constexpr (CTAS == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

// MXFP8: E4M3 operands, E8M0 scales, one scale per 32 elements, K = 32 per instruction.
template <int CTAS>
__device__ __forceinline__ void mma_mxfp8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if constexpr (CTAS == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

}  // namespace sm100
}  // namespace ck
