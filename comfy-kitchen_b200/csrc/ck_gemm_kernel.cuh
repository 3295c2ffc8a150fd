// Kernel template and launcher of the block-scaled GEMMs for sm_100a: out[M,N] = cast((A[M,K] . B[N,K]^T) * alpha + bias).
//
//   NVFP4: A, B packed E2M1 (two per byte), E4M3 scale per 16 elements  (kind::mxf4nvf4)
//   MXFP8: A, B E4M3 bytes,                  E8M0 scale per 32 elements  (kind::mxf8f6f4)
//
// One persistent CTA per SM (or, for large problems, one CTA pair per two SMs computing
// 256 x 256 tiles with cta_group::2 instructions), warps with fixed roles:
//   warp 0    TMA producer: per pipeline stage one 128-row x 128-byte box of A, one box of B
//             (128-byte swizzle) and the matching 512-byte scale tiles (linear bulk copies, or
//             3-D tensor maps in a pair) into a STAGES-deep shared-memory ring.
//   warp 1    MMA issuer: per landed stage, copies the stage's scale tiles shared -> tensor
//             memory (tcgen05.cp, up to 12) and issues four tcgen05.mma (32 bytes of K each) into
//             a fp32 accumulator in tensor memory; releases the stage / publishes the accumulator
//             with tcgen05.commit.  The tensor-memory scale columns are buffered per stage like
//             the ring.  (Scale copies on a warp of their own were measured: the extra barrier
//             hop between landing and issue costs 3-15 % at every shape.)
//   warps 2.. epilogue (8 warps; 16 for the fused epilogue, 4 for 64-wide tiles): tcgen05.ld
//             the accumulator into registers, hand it back at once, then alpha * acc + bias,
//             convert, stage the rows in swizzled shared memory and write them with TMA stores
//             while the next tile computes.  The fused variant applies GELU and
//             re-quantizes to NVFP4 instead; split-K items store raw fp32 partial tiles to a
//             workspace; the all-gather variant stores every tile into all ranks' results.
// With NUM_ACC == 2 the epilogue of tile i overlaps the main loop of tile i+1 entirely.
//
// All synchronisation is by mbarriers with bounded waits (ck_sm100.cuh): a protocol error
// raises the device status word instead of hanging.  Kernels are launched with programmatic
// stream serialization; each role waits for the previous kernel (griddepcontrol.wait) only
// before its own first global access.
#pragma once
#include "ck_sm100.cuh"
#include "ck_quant_math.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <vector>

namespace ck {
namespace {

using namespace sm100;

enum class Kind { kNvfp4, kMxfp8 };

constexpr int kTileM = 128;
constexpr int kStageKBytes = 128;   // bytes of K per operand row per stage (one swizzle atom)
constexpr int kMmaKBytes = 32;      // bytes of K per tcgen05.mma
constexpr int kMmaPerStage = kStageKBytes / kMmaKBytes;
// Epilogue warps per CTA: two per 32-lane quarter of tensor memory for the plain epilogue,
// four for the fused one (its activation + quantization arithmetic is ~30 instructions per
// element and must keep up with the tensor pipe), one for a 64-wide tile.
// Timeline builds (-DCK_GEMM_TRACE) keep per-tile stamps in shared memory behind the barriers.
#ifdef CK_GEMM_TRACE
constexpr int kTraceTiles = 40;
constexpr int kTraceSlots = 16;
constexpr int kTraceSmemTiles = 12;
constexpr int kTraceSmemBytes = kTraceSmemTiles * kTraceSlots * 4;
#else
constexpr int kTraceSmemBytes = 0;
#endif

constexpr int epilogue_warps(bool fused, int tile_n) { return (fused && tile_n >= 256) ? 16 : (tile_n <= 64) ? 4 : 8; }
constexpr int num_threads(bool fused, int tile_n) {
  return 64 + 32 * epilogue_warps(fused, tile_n);  // + TMA and MMA warps
}
constexpr int pow2_at_least(int x) { return x <= 32 ? 32 : x <= 64 ? 64 : x <= 128 ? 128 : x <= 256 ? 256 : 512; }

// CTAS == 2: a pair of CTAs (a 2-CTA cluster on neighbouring SMs) computes one 256 x TILE_N
// tile with cta_group::2 instructions.  Each CTA loads its own 128 rows of A and only its
// own half of B's rows, which halves the shared-memory traffic for B - the limiter of the
// single-CTA FP4 kernel.
// OUT_STAGE: the plain epilogue stages the converted tile in shared memory (4 KiB per
// epilogue warp) and writes it with TMA stores.  Storing rows straight from registers puts 32
// partial-line writes per instruction into the SM's memory pipeline, which delays the MMA
// warp's own instructions in that pipeline and starves the tensor cores.
// (OUT_STAGE = number of 4 KiB boxes per epilogue warp, used as a ring; 0 = store from registers.)
template <Kind KIND, int TILE_N, int NUM_ACC, int STAGES, int CTAS, int OUT_STAGE = 0>
struct Config {
  static constexpr int kTileRows = kTileM * CTAS;      // rows of the output tile
  static constexpr int kBRows = TILE_N / CTAS;         // rows of B each CTA loads
  static constexpr int kABytes = kTileM * kStageKBytes;
  static constexpr int kBBytes = kBRows * kStageKBytes;
  // 512-byte scale tiles (128 rows x 4 scale columns) one 128-row block needs per stage:
  // NVFP4 has 16 scale columns per 256 elements, MXFP8 4 per 128 elements.
  static constexpr int kSfTilesPerStage = (KIND == Kind::kNvfp4) ? 4 : 1;
  // 128-row blocks of B's scale tensor a tile can touch (a 192-wide tile straddles two);
  // every CTA needs the scales of all TILE_N columns in its tensor memory.
  static constexpr int kSfbRowBlocks = (TILE_N + 127) / 128;
  static constexpr int kSfaBytes = kSfTilesPerStage * 512;
  static constexpr int kSfbBytes = kSfbRowBlocks * kSfTilesPerStage * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kOutStageBytes = OUT_STAGE * epilogue_warps(false, TILE_N) * 4096;
  static constexpr int kRingBytes = (STAGES * kStageBytes + 1023) / 1024 * 1024;
  static constexpr int kSmemBytes = kRingBytes + kOutStageBytes + 3 * TILE_N * 4 /*bias*/ +
                                    1024 /*alignment slack*/ + 256 /*barriers*/ + kTraceSmemBytes;
  // tensor memory columns
  static constexpr int kAccCols = TILE_N;
  static constexpr int kSfaCol = NUM_ACC * kAccCols;
  static constexpr int kSfaColsPerStage = kSfTilesPerStage * 4;
  static constexpr int kSfbCol = kSfaCol + kSfaColsPerStage;  // within one scale buffer
  static constexpr int kSfbColsPerTile = kSfbRowBlocks * 4;
  static constexpr int kSfbColsPerStage = kSfTilesPerStage * kSfbColsPerTile;
  // One set of scale columns per ring stage: the copy of stage s lands in set s, which the
  // stage's "empty" barrier (MMAs retired) frees together with the shared-memory slot.
  static constexpr int kSfColsPerBuf = kSfaColsPerStage + kSfbColsPerStage;
  static_assert(kSfaCol + STAGES * kSfColsPerBuf <= 512, "tensor memory budget exceeded");
  // allocated columns: a power of two; configurations that need at most 256 can share an SM
  static constexpr int kTmemCols = pow2_at_least(kSfaCol + STAGES * kSfColsPerBuf);
  static_assert(CTAS == 1 || CTAS == 2, "one CTA or a CTA pair");
  static_assert(CTAS == 1 || TILE_N % 32 == 0, "a CTA pair needs N % 32 == 0");
  static_assert(TILE_N % 16 == 0 && TILE_N >= 16 && TILE_N <= 256, "invalid MMA N");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget exceeded");
  static constexpr uint32_t kIdesc = make_block_scaled_idesc(KIND == Kind::kNvfp4 ? 1u : 0u,
                                                             KIND == Kind::kNvfp4 ? 0u : 1u, kTileRows, TILE_N);
};

struct GemmParams {
  const uint8_t* sfa;      // A scales, tiled layout, [ceil(M/128)][sf_col_tiles] tiles of 512 bytes
  const uint8_t* sfb;      // B scales, same layout over N
  const float* tsa;        // per-tensor scales (device), or null
  const float* tsb;
  const float* alpha;      // overrides tsa*tsb when non-null
  const void* bias;        // [N] or null
  void* out;               // [M, N] row-major
  int bias_dtype;
  int out_dtype;
  int M, N;
  int k_bytes;             // bytes of K per operand row
  int sf_col_tiles;        // 512-byte scale tiles per 128-row block = ceil(K / (4 * block))
  int n_row_blocks_a;      // ceil(M / 128)
  int n_row_blocks_b;      // ceil(N / 128)
  int tiles_m, tiles_n;
  int raster;              // order in which workers walk the tiles: 0 = down the rows first, 1 = along the columns first
  int out_tma;             // the output qualifies for TMA stores (16-byte aligned base and pitch)
  int n_out;               // destinations of every output tile (1, or one per GPU of an all-gather)
  int splits;              // split-K: work items per tile (1 = off); item s of a tile covers pipeline stages
  int k_stages_per_split;  //   [s * k_stages_per_split, ...) and stores its raw fp32 partial to destination s
  float* partials;         // swapped-operand split-K: raw fp32 partial tiles, [item][epilogue warp][its slice]
  unsigned int* tickets;   //   and one arrival counter per tile and epilogue warp (zero between launches)
  int* status;             // device status word: set non-zero when a wait gave up
  int trace_launch;        // sequence number of the launch (timeline builds only)
  // fused epilogue (FUSED kernels only)
  int activation;          // CK_ACT_*
  uint8_t* rq_codes;       // [M, N/2] NVFP4 codes of the (activated) output, or null
  uint8_t* rq_scales;      // its tiled E4M3 block scales, [roundup(M,128), N/16]
  const float* rq_scale;   // its per-tensor scale (device)
};


// Tile index -> (row block, column block) in the walking order the launch chose.
__device__ __forceinline__ int tile_row_block(const GemmParams& p, int tile) {
  return p.raster == 0 ? tile % p.tiles_m : tile / p.tiles_n;
}
__device__ __forceinline__ int tile_col_block(const GemmParams& p, int tile) {
  return p.raster == 0 ? tile / p.tiles_m : tile % p.tiles_n;
}

// Destinations of the output tile: one tensor map for a plain GEMM; for the column-sharded
// GEMM with a fused all-gather, one per GPU - each a window [M, N_local] at this rank's column
// offset inside that GPU's full [M, N_total] result (peer memory mapped into this process).
constexpr int kMaxOutputs = 8;
struct OutputMaps {
  CUtensorMap m[kMaxOutputs];
};

// Optional per-tile timeline (SM cycle counter) for tuning; compiled in with -DCK_GEMM_TRACE only.
// Per-tile stamps are kept in shared memory (32-bit counts, 12 tiles x 16 slots) and written out
// when the CTA is done: a stamp costs one shared-memory store, so the instrumented kernel behaves
// like the production one (global stores in the loops would queue behind the epilogue's).
// -DCK_GEMM_TRACE_STAGES adds per-stage stamps of the MMA warp, stored to global memory as they
// are taken (these do perturb the kernel).
#ifdef CK_GEMM_TRACE
__device__ long long g_trace[160 * kTraceTiles * kTraceSlots];
__device__ long long g_trace2[160 * 4 * 64];
// per launch (ring of 8) and CTA: global timer (ns) and SM clock at entry, after the dependency wait, at exit
__device__ long long g_trace3[8 * 160 * 8];
__device__ __forceinline__ long long global_timer_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define CK_TRACE3(slot)                                                                              \
  do {                                                                                               \
    if (threadIdx.x == 0 && blockIdx.x < 160) {                                                      \
      long long* t3 = g_trace3 + ((p.trace_launch & 7) * 160 + blockIdx.x) * 8 + 2 * (slot);         \
      t3[0] = global_timer_ns();                                                                     \
      t3[1] = clock64();                                                                             \
    }                                                                                                \
  } while (0)
#ifdef CK_GEMM_TRACE_STAGES
#define CK_TRACE2(kind, idx)                                                                         \
  do {                                                                                               \
    if (lane == 0 && (idx) < 64 && blockIdx.x < 160) g_trace2[(blockIdx.x * 4 + (kind)) * 64 + (idx)] = clock64(); \
  } while (0)
#else
#define CK_TRACE2(kind, idx) \
  do {                       \
  } while (0)
#endif
#define CK_TRACE(slot)                                                                               \
  do {                                                                                               \
    if (lane == 0 && tile_it < kTraceSmemTiles) trace_s[tile_it * kTraceSlots + (slot)] = static_cast<uint32_t>(clock64()); \
  } while (0)
#define CK_TRACE_ELECTED(slot)                                                                       \
  do {                                                                                               \
    if (tile_it < kTraceSmemTiles) trace_s[tile_it * kTraceSlots + (slot)] = static_cast<uint32_t>(clock64()); \
  } while (0)
#else
#define CK_TRACE3(slot) \
  do {                  \
  } while (0)
#define CK_TRACE(slot) \
  do {                 \
  } while (0)
#define CK_TRACE2(kind, idx) \
  do {                       \
  } while (0)
#define CK_TRACE_ELECTED(slot) \
  do {                         \
  } while (0)
#endif

// alpha * acc + bias for 32 consecutive output columns of one row.  `bias_s` points at the 32
// fp32 bias values of these columns in shared memory (all lanes read the same addresses).
__device__ __forceinline__ void scale_and_bias(const uint32_t (&raw)[32], float alpha, const float* bias_s,
                                               float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 b = reinterpret_cast<const float4*>(bias_s)[i];
    v[4 * i + 0] = fmaf(__uint_as_float(raw[4 * i + 0]), alpha, b.x);
    v[4 * i + 1] = fmaf(__uint_as_float(raw[4 * i + 1]), alpha, b.y);
    v[4 * i + 2] = fmaf(__uint_as_float(raw[4 * i + 2]), alpha, b.z);
    v[4 * i + 3] = fmaf(__uint_as_float(raw[4 * i + 3]), alpha, b.w);
  }
}

// Convert and store 32 consecutive output columns of one row.  `vec_ok`: the row pitch and
// column offset allow 32-byte aligned vector stores.
template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* dst, const float (&v)[32], int valid, bool vec_ok) {
  if (valid == 32 && vec_ok) {
    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        Vec256 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
            __nv_bfloat162 q = __floats2bfloat162_rn(v[h * 16 + 2 * j], v[h * 16 + 2 * j + 1]);
            o.w[j] = *reinterpret_cast<uint32_t*>(&q);
          } else {
            __half2 q = __floats2half2_rn(v[h * 16 + 2 * j], v[h * 16 + 2 * j + 1]);
            o.w[j] = *reinterpret_cast<uint32_t*>(&q);
          }
        }
        st_global_256_no_allocate(reinterpret_cast<uint8_t*>(dst) + h * 32, o);
      }
    } else {
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        Vec256 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.w[j] = __float_as_uint(v[h * 8 + j]);
        st_global_256_no_allocate(reinterpret_cast<uint8_t*>(dst) + h * 32, o);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if (i < valid) {
      if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
        dst[i] = __float2bfloat16_rn(v[i]);
      } else if constexpr (std::is_same<OutT, __half>::value) {
        dst[i] = __float2half_rn(v[i]);
      } else {
        dst[i] = v[i];
      }
    }
  }
}

// Two floats rounded to a 16-bit OutT and packed (first value in the low half), and back.
template <typename OutT>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
    __nv_bfloat162 q = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&q);
  } else {
    __half2 q = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&q);
  }
}
template <typename OutT>
__device__ __forceinline__ void unpack_pair(uint32_t w, float& lo, float& hi) {
  if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
}

template <typename OutT>
__device__ __forceinline__ float round_to_out(float x) {
  if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
    return __bfloat162float(__float2bfloat16_rn(x));
  } else if constexpr (std::is_same<OutT, __half>::value) {
    return __half2float(__float2half_rn(x));
  } else {
    return x;
  }
}

// tanh-approximated GELU in fp32: 0.5 x (1 + tanh(u)), u = sqrt(2/pi) (x + 0.044715 x^3),
// evaluated as x * sigmoid(2u) = x / (1 + 2^(-2u log2 e)) with the hardware exp2 and
// reciprocal (relative error ~1e-6, far below the rounding of a 16-bit output type).
__device__ __forceinline__ float gelu_tanh(float x) {
  // x * sigmoid(2u) = x / (1 + 2^(x * (k1 + k2 x^2))), k1 = -2 log2(e) sqrt(2/pi), k2 = 0.044715 k1.
  // The flush-to-zero forms only differ where 1 + 2^(..) exceeds 2^126, i.e. where the exact
  // result is a zero anyway (x below about -10).
  const float w = fmaf(-0.10294324f, x * x, -2.3022082f);
  float t, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(x * w));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + t));
  return x * r;
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int n) {
  if (dtype == CK_DTYPE_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
  if (dtype == CK_DTYPE_F16) return __half2float(static_cast<const __half*>(bias)[n]);
  return static_cast<const float*>(bias)[n];
}

// FUSED: the epilogue applies an activation to the output rounded to OutT (what an unfused
// caller would see), optionally stores it, and optionally re-quantizes it to NVFP4 (codes +
// tiled block scales against a static per-tensor scale) as the A operand of the next GEMM.
// SWAP: the operands have changed places - "A" (128-row tiles, tensor-memory lanes) is the weight
// [N, K] and "B" (the MMA's N dimension, TILE_N >= M) is the small activation [M, K] - so that a GEMM
// with few activation rows fills the 128-row MMA dimension with weight rows and streams the weight
// once.  p.M / p.N are then the weight's and the activation's row counts, the output is written
// transposed (out[b_row][a_row]), the bias runs along the A rows, and a tile's K range may be split
// over several CTAs that add their raw fp32 partial tiles through a workspace: every CTA stores its
// partial and takes a ticket, the one that takes the last ticket adds all partials in split order
// (deterministic) and writes the result - nobody waits for anybody.
template <Kind KIND, int TILE_N, int NUM_ACC, int STAGES, int CTAS, typename OutT, bool FUSED, int OUT_STAGE, bool SWAP = false>
__global__ void __launch_bounds__(num_threads(FUSED, TILE_N), (SWAP && TILE_N <= 128) ? 2 : 1)
block_scaled_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                         const __grid_constant__ OutputMaps maps_out, const GemmParams p) {
  using Cfg = Config<KIND, TILE_N, NUM_ACC, STAGES, CTAS, OUT_STAGE>;
  static_assert(!(FUSED && OUT_STAGE != 0), "the fused epilogue stores from registers");
  static_assert(!SWAP || (!FUSED && OUT_STAGE == 0 && CTAS == 1), "swapped operands: plain epilogue, one CTA");
  constexpr int kNumEpilogueWarps = epilogue_warps(FUSED, TILE_N);
  constexpr int kThreads = num_threads(FUSED, TILE_N);
  static_assert(TILE_N <= 32 * kNumEpilogueWarps, "one bias value per epilogue thread");
  // Everything the kernel does until a role's griddepcontrol.wait is independent of the kernel
  // before it in the stream, so the next kernel may be scheduled as early as resources allow.
  pdl_launch_dependents();
  // In a CTA pair, rank 0 (the leader) issues the MMAs and scale copies for both CTAs.
  const uint32_t cta_rank = (CTAS == 2) ? cluster_cta_rank() : 0u;
  const int worker = blockIdx.x / CTAS;        // index of this CTA (pair) among the tile workers
  const int num_workers = gridDim.x / CTAS;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + STAGES * Cfg::kABytes;
  uint8_t* smem_sfa = smem_b + STAGES * Cfg::kBBytes;
  uint8_t* smem_sfb = smem_sfa + STAGES * Cfg::kSfaBytes;
  uint8_t* smem_out = smem + Cfg::kRingBytes;  // 1024-byte aligned (swizzled store boxes)
  float* smem_bias = reinterpret_cast<float*>(smem_out + Cfg::kOutStageBytes);  // [3][TILE_N]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_bias + 3 * TILE_N);
  uint64_t* full_bar = bars;                       // [STAGES] producer -> MMA (operands and scales landed)
  uint64_t* empty_bar = bars + STAGES;             // [STAGES] MMA -> producer (stage and its scale columns free)
  uint64_t* acc_full_bar = bars + 2 * STAGES;      // [NUM_ACC] MMA -> epilogue
  uint64_t* acc_empty_bar = acc_full_bar + NUM_ACC;  // [NUM_ACC] epilogue -> MMA
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + NUM_ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
#ifdef CK_GEMM_TRACE
  uint32_t* trace_s = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(bars) + 256);
#endif
  static_assert((2 * STAGES + 2 * NUM_ACC) * 8 + 8 <= 256, "barrier area");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  CK_TRACE3(0);

  // Weight streaming (SWAP): first thing, ahead of the set-up and of the dependency wait, ask L2 for
  // the operand boxes of this CTA's first stages.  A prefetch only warms the cache (L2 is the point
  // of coherence: what the previous kernel still writes is seen by the loads after the wait); the
  // DRAM latency of the first loads then overlaps barrier set-up, tensor-memory allocation and the
  // wait itself (1-3 % of these 6-10 us kernels).  The tile configurations are slower with it
  // (config 2: 18.7 vs 18.5 us; the requests share the TMA unit with the first loads).
  if (SWAP && warp == 0 && elect_one()) {
    const int pf_splits = p.splits;
    const int pf_k_stages = (p.k_bytes + kStageKBytes - 1) / kStageKBytes;
    if (worker < p.tiles_m * p.tiles_n * pf_splits) {
      const int tile0 = worker / pf_splits;
      const int ks0 = (worker - tile0 * pf_splits) * p.k_stages_per_split;
      const int ks1 = min(min(pf_k_stages, ks0 + p.k_stages_per_split), ks0 + STAGES);
      const int pm0 = tile_row_block(p, tile0) * Cfg::kTileRows + static_cast<int>(cta_rank) * kTileM;
      const int pn0 = tile_col_block(p, tile0) * TILE_N + static_cast<int>(cta_rank) * Cfg::kBRows;
      for (int ks = ks0; ks < ks1; ++ks) {
        tma_prefetch_2d(&map_a, ks * kStageKBytes, pm0);
        tma_prefetch_2d(&map_b, ks * kStageKBytes, pn0);
      }
    }
  }

  // ------------------------------------------------------------------ set-up
  // The producer warp creates the barriers and goes straight to its loads; the other warps
  // meet it at a named barrier it only arrives on (tensor memory is allocated meanwhile).
  // In a pair, every thread arrives on the cluster barrier at once and waits where it first
  // needs the other CTA's barriers to exist.
  uint32_t tmem_base = 0;
  if (warp == 0) {
#ifdef CK_GEMM_TRACE
    for (int i = lane; i < kTraceSmemTiles * kTraceSlots; i += 32) trace_s[i] = 0u;
    __syncwarp();
#endif
    if (lane == 0) {
      *abort_flag = 0;
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], 1);
      }
      for (int a = 0; a < NUM_ACC; ++a) {
        mbar_init(&acc_full_bar[a], 1);
        mbar_init(&acc_empty_bar[a], kNumEpilogueWarps * CTAS);  // one arrival per epilogue warp (of both CTAs)
      }
      fence_barrier_init();
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      if constexpr (CTAS == 2) {
        prefetch_tensormap(&map_sfa);
        prefetch_tensormap(&map_sfb);
      }
      if constexpr (OUT_STAGE != 0) {
        for (int d = 0; d < p.n_out; ++d) prefetch_tensormap(&maps_out.m[d]);
      }
      __threadfence_block();
    }
    __syncwarp();
    if constexpr (CTAS == 2) {
      cluster_arrive();
      cluster_wait();  // the other CTA's barriers exist before this one's loads report to them
    }
    named_barrier_arrive(2, kThreads);
  } else {
    if constexpr (CTAS == 2) cluster_arrive();
    if (warp == 1) tmem_alloc<CTAS>(tmem_base_slot, Cfg::kTmemCols);
    tc_fence_before_sync();
    named_barrier_sync(2, kThreads);
    if constexpr (CTAS == 2) cluster_wait();
    tc_fence_after_sync();
    tmem_base = *tmem_base_slot;
  }
  CK_TRACE3(1);

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int splits = p.splits;
  const int num_items = num_tiles * splits;
  const int k_stages = (p.k_bytes + kStageKBytes - 1) / kStageKBytes;
  const int total_mma = (p.k_bytes + kMmaKBytes - 1) / kMmaKBytes;

  // The role loops below are executed by whole warps with warp-uniform control flow; the
  // asynchronous instructions themselves are issued by one elected lane.
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    pdl_wait();  // operands and scales may come from the kernel before this one
    CK_TRACE3(2);
    int ring_s = 0;
    uint32_t ring_ph = 0;
    [[maybe_unused]] uint32_t tile_it = 0;
    for (int item = worker; item < num_items; item += num_workers, ++tile_it) {
      const int tile = item / splits;
      const int ks_begin = (item - tile * splits) * p.k_stages_per_split;
      const int ks_end = min(k_stages, ks_begin + p.k_stages_per_split);
      // consecutive workers take neighbouring tiles in the walking order the launch chose (p.raster)
      const int tile_m = tile_row_block(p, tile);
      const int tile_n = tile_col_block(p, tile);
      const int m0 = tile_m * Cfg::kTileRows + static_cast<int>(cta_rank) * kTileM;  // this CTA's rows of A
      const int n0 = tile_n * TILE_N;
      const int rb_b0 = n0 / 128;
      int rb_b_count = 0;
#pragma unroll
      for (int r = 0; r < Cfg::kSfbRowBlocks; ++r) rb_b_count += (rb_b0 + r < p.n_row_blocks_b) ? 1 : 0;
      // the second CTA of a pair may own rows past M: it then has no scale row block to load
      const bool have_sfa = (m0 / kTileM) < p.n_row_blocks_a;
      const uint8_t* sfa_src = p.sfa + static_cast<int64_t>(m0 / kTileM) * p.sf_col_tiles * 512;
      const uint8_t* sfb_src = p.sfb + static_cast<int64_t>(rb_b0) * p.sf_col_tiles * 512;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        // ring position and phase as running counters (STAGES is not a power of two)
        const int s = ring_s;
        const uint32_t ph = ring_ph;
        if (++ring_s == STAGES) {
          ring_s = 0;
          ring_ph ^= 1u;
        }
        mbar_wait(&empty_bar[s], ph ^ 1, abort_flag);  // in a pair: signalled from the leader CTA
        if (ks == ks_begin) CK_TRACE(4);
        if (ks == ks_end - 1) CK_TRACE(5);
        if constexpr (CTAS == 2) {
          // Every load of both CTAs reports its bytes to the leader's barrier; scale tiles
          // come through 3-D tensor maps {512 B, column tile, row block} so that tiles past
          // the end read as zeros and every stage has the same byte count.
          if (elect_one()) {
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * Cfg::kStageBytes);
            const int sf_tile0 = ks * Cfg::kSfTilesPerStage;
            tma_load_2d_pair(smem_a + s * Cfg::kABytes, &map_a, &full_bar[s], ks * kStageKBytes, m0);
            tma_load_2d_pair(smem_b + s * Cfg::kBBytes, &map_b, &full_bar[s], ks * kStageKBytes,
                             n0 + static_cast<int>(cta_rank) * Cfg::kBRows);
            tma_load_3d_pair(smem_sfa + s * Cfg::kSfaBytes, &map_sfa, &full_bar[s], 0, sf_tile0, m0 / kTileM);
#pragma unroll
            for (int r = 0; r < Cfg::kSfbRowBlocks; ++r) {
              tma_load_3d_pair(smem_sfb + s * Cfg::kSfbBytes + r * Cfg::kSfTilesPerStage * 512, &map_sfb, &full_bar[s],
                               0, sf_tile0, rb_b0 + r);
            }
          }
          __syncwarp();
          continue;
        }
        if (elect_one()) {
          const int sf_tile0 = ks * Cfg::kSfTilesPerStage;
          const uint32_t sf_bytes = static_cast<uint32_t>(min(Cfg::kSfTilesPerStage, p.sf_col_tiles - sf_tile0)) * 512u;
          mbar_arrive_expect_tx(&full_bar[s],
                                Cfg::kABytes + Cfg::kBBytes + sf_bytes * ((have_sfa ? 1 : 0) + rb_b_count));
          tma_load_2d(smem_a + s * Cfg::kABytes, &map_a, &full_bar[s], ks * kStageKBytes, m0);
          tma_load_2d(smem_b + s * Cfg::kBBytes, &map_b, &full_bar[s], ks * kStageKBytes,
                      n0 + static_cast<int>(cta_rank) * Cfg::kBRows);
          if (have_sfa) bulk_load_1d(smem_sfa + s * Cfg::kSfaBytes, sfa_src + sf_tile0 * 512, sf_bytes, &full_bar[s]);
#pragma unroll
          for (int r = 0; r < Cfg::kSfbRowBlocks; ++r) {
            if (r < rb_b_count) {
              bulk_load_1d(smem_sfb + s * Cfg::kSfbBytes + r * Cfg::kSfTilesPerStage * 512,
                           sfb_src + (static_cast<int64_t>(r) * p.sf_col_tiles + sf_tile0) * 512, sf_bytes,
                           &full_bar[s]);
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1 && cta_rank != 0) {
    // second CTA of a pair: the leader issues the MMAs and the scale copies for both
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Nothing can land before the producer's own dependency wait is over; waiting here too keeps
    // the bounded barrier waits below from running (and giving up) while a long predecessor - a
    // cross-GPU barrier that waits for a late rank, say - is still executing.
    pdl_wait();
    // Descriptors differ between stages only in their start-address field, so the loop
    // carries 32-bit low words; the high words are constants.
    const uint32_t a_lo0 = static_cast<uint32_t>(make_operand_desc_sw128(smem_u32(smem_a)));
    const uint32_t b_lo0 = static_cast<uint32_t>(make_operand_desc_sw128(smem_u32(smem_b)));
    const uint32_t op_hi = static_cast<uint32_t>(make_operand_desc_sw128(0) >> 32);
    const uint32_t sfa_lo0 = static_cast<uint32_t>(make_scale_desc(smem_u32(smem_sfa)));
    const uint32_t sfb_lo0 = static_cast<uint32_t>(make_scale_desc(smem_u32(smem_sfb)));
    const uint32_t sf_hi = static_cast<uint32_t>(make_scale_desc(0) >> 32);
    const uint32_t t_sfa0 = tmem_base + Cfg::kSfaCol;
    const uint32_t t_sfb0 = tmem_base + Cfg::kSfbCol;
    const uint32_t empty_addr = smem_u32(empty_bar);
    const uint32_t acc_full_addr = smem_u32(acc_full_bar);
    const uint32_t empty_addr_peer = (CTAS == 2) ? map_to_cta(empty_addr, 1) : 0u;
    const uint32_t acc_full_addr_peer = (CTAS == 2) ? map_to_cta(acc_full_addr, 1) : 0u;
    [[maybe_unused]] uint32_t it = 0;
    int ring_s = 0;
    uint32_t ring_ph = 0;
    uint32_t tile_it = 0;
    for (int item = worker; item < num_items; item += num_workers, ++tile_it) {
      const int tile = item / splits;
      const int ks_begin = (item - tile * splits) * p.k_stages_per_split;
      const int ks_end = min(k_stages, ks_begin + p.k_stages_per_split);
      const int n0 = tile_col_block(p, tile) * TILE_N;
      const int acc = tile_it % NUM_ACC;
      const uint32_t acc_ph = (tile_it / NUM_ACC) & 1;
      const uint32_t d_tmem = tmem_base + acc * Cfg::kAccCols;
      // B scale words of this tile start (n0 % 128) / 32 columns into the first row block
      const uint32_t sfb_shift = (n0 % 128) / 32;
      for (int ks = ks_begin; ks < ks_end; ++ks, ++it) {
        const int s = ring_s;
        const uint32_t ph = ring_ph;
        if (++ring_s == STAGES) {
          ring_s = 0;
          ring_ph ^= 1u;
        }
        CK_TRACE2(1, it);
        mbar_wait(&full_bar[s], ph, abort_flag);
        if (ks == ks_begin) CK_TRACE(2);
        if (ks == ks_end - 1) CK_TRACE(3);
        CK_TRACE2(2, it);
        tc_fence_after_sync();
        if (elect_one()) {
          const uint32_t a_lo = a_lo0 + s * (Cfg::kABytes >> 4);
          const uint32_t b_lo = b_lo0 + s * (Cfg::kBBytes >> 4);
          const int n_mma = min(kMmaPerStage, total_mma - ks * kMmaPerStage);
          const uint32_t t_sfa = t_sfa0 + s * Cfg::kSfColsPerBuf;
          const uint32_t t_sfb_tile = t_sfb0 + s * Cfg::kSfColsPerBuf + sfb_shift;
          // scale tiles of this stage: shared -> tensor memory (512 bytes = 32 descriptor units);
          // the tensor pipe runs them in order ahead of the MMAs that read them
          const uint32_t sfa_lo = sfa_lo0 + s * (Cfg::kSfaBytes >> 4);
          const uint32_t sfb_lo = sfb_lo0 + s * (Cfg::kSfbBytes >> 4);
          const uint32_t t_sfb = t_sfb0 + s * Cfg::kSfColsPerBuf;
#pragma unroll
          for (int t = 0; t < Cfg::kSfTilesPerStage; ++t) {
            tc_copy_scales_32x128b<CTAS>(t_sfa + t * 4, desc64(sfa_lo + t * 32, sf_hi));
#pragma unroll
            for (int r = 0; r < Cfg::kSfbRowBlocks; ++r) {
              tc_copy_scales_32x128b<CTAS>(t_sfb + t * Cfg::kSfbColsPerTile + r * 4,
                                           desc64(sfb_lo + (r * Cfg::kSfTilesPerStage + t) * 32, sf_hi));
            }
          }
          if (ks == ks_begin) {
            // Only now does the tile need its accumulator: the wait for the epilogue to have
            // drained it comes after the first stage has landed.
            CK_TRACE_ELECTED(0);
            mbar_wait(&acc_empty_bar[acc], acc_ph ^ 1, abort_flag);
            CK_TRACE_ELECTED(1);
            tc_fence_after_sync();
          }
#pragma unroll
          for (int kb = 0; kb < kMmaPerStage; ++kb) {
            if (kb < n_mma) {
              const uint32_t accumulate = (ks != ks_begin || kb != 0) ? 1u : 0u;
              // advancing K inside the swizzle atom = advancing the start address (32 B = 2 units)
              const uint64_t a_desc = desc64(a_lo + kb * 2, op_hi);
              const uint64_t b_desc = desc64(b_lo + kb * 2, op_hi);
              if constexpr (KIND == Kind::kNvfp4) {
                mma_nvfp4<CTAS>(d_tmem, a_desc, b_desc, Cfg::kIdesc, t_sfa + kb * 4,
                                t_sfb_tile + kb * Cfg::kSfbColsPerTile, accumulate);
              } else {
                // one scale tile serves the four MMAs of the stage: byte kb of each scale word
                mma_mxfp8<CTAS>(d_tmem, a_desc, b_desc, idesc_with_scale_ids(Cfg::kIdesc, kb), t_sfa, t_sfb_tile,
                                accumulate);
              }
            }
          }
          // stage (and its scale columns) reusable once these MMAs retire; in a pair both CTAs are told
          tc_commit<CTAS>(empty_addr + s * 8);
          if constexpr (CTAS == 2) tc_commit<CTAS>(empty_addr_peer + s * 8);
          if (ks == ks_end - 1) {
            tc_commit<CTAS>(acc_full_addr + acc * 8);
            if constexpr (CTAS == 2) tc_commit<CTAS>(acc_full_addr_peer + acc * 8);
          }
        }
        __syncwarp();
        CK_TRACE2(3, it);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2 ..)
    // Two warps share each 32-lane quarter of tensor memory and split the tile's columns.
    // A warp pulls its whole share of the accumulator into registers with back-to-back
    // tcgen05.ld, hands the accumulator back to the MMA warp at once, and only then does
    // the arithmetic and the stores - so the next tile's main loop overlaps them.
    pdl_wait();  // alpha, bias and the output buffer may belong to the kernel before this one
    const int quarter = warp & 3;  // tensor-memory lanes this warp may read: 32*quarter .. +31
    const int half = (warp - 2) >> 2;  // which share of the tile's columns
    constexpr int kColsPerWarp = TILE_N / (kNumEpilogueWarps / 4);
    constexpr int kChunks = kColsPerWarp / 32;
    static_assert(kColsPerWarp % 32 == 0, "tile width must split into 32-column chunks per warp");
    const int et = threadIdx.x - 64;  // 0 .. 32*kNumEpilogueWarps-1 among the epilogue threads
    float alpha = 1.0f;
    if (p.alpha != nullptr) {
      alpha = ld_f32_dependent(p.alpha);
    } else if (p.tsa != nullptr && p.tsb != nullptr) {
      alpha = ld_f32_dependent(p.tsa) * ld_f32_dependent(p.tsb);
    }
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_ok = (static_cast<int64_t>(p.N) * sizeof(OutT)) % 32 == 0 &&
                        (reinterpret_cast<uintptr_t>(p.out) & 31u) == 0 && (TILE_N * sizeof(OutT)) % 32 == 0;
    const uint32_t acc_empty_leader = (CTAS == 2) ? map_to_cta(smem_u32(acc_empty_bar), 0) : 0u;
    [[maybe_unused]] uint32_t out_box = 0;  // boxes this warp has staged so far (ring index)
    uint32_t tile_it = 0;
    for (int item = worker; item < num_items; item += num_workers, ++tile_it) {
      const int tile = item / splits;
      const int split = item - tile * splits;
      const int tile_m = tile_row_block(p, tile);
      const int tile_n = tile_col_block(p, tile);
      const int row = tile_m * Cfg::kTileRows + static_cast<int>(cta_rank) * kTileM + quarter * 32 + lane;
      const int n0 = tile_n * TILE_N;
      const int acc = tile_it % NUM_ACC;
      const uint32_t acc_ph = (tile_it / NUM_ACC) & 1;
      if constexpr (SWAP) {
        // ---- swapped operands: lane = weight row (output column), accumulator columns = activation rows
        const int r_in_tile = quarter * 32 + lane;
        const int a_row = tile_m * kTileM + r_in_tile;  // weight row = output column
        const int c0 = half * kColsPerWarp;
        // fetched ahead of the accumulator wait, which hides the latency
        const float bias_v = (p.bias != nullptr && a_row < p.M) ? load_bias(p.bias, p.bias_dtype, a_row) : 0.0f;
        if (warp == 2) CK_TRACE(6);
        mbar_wait(&acc_full_bar[acc], acc_ph, abort_flag);
        if (warp == 2) CK_TRACE(7);
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + acc * Cfg::kAccCols + (static_cast<uint32_t>(quarter * 32) << 16) + c0;
        uint32_t buf[kChunks][32];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tmem_load_32x32(t_row + c * 32, buf[c]);
        tmem_load_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
        if (warp == 2) CK_TRACE(8);
        if (splits > 1) {
          // Each epilogue warp settles its own 32 rows x kColsPerWarp slice of the tile with the same
          // warps of the CTAs that hold the tile's other K ranges: store the raw partial slice (16-byte
          // units laid out so that the 32 lanes of a store are contiguous), take a ticket of the slice's
          // counter with release / acquire semantics, and if it was the last one add all partials in
          // split order.  No CTA-wide barrier, no waiting.
          constexpr int kUnits = kColsPerWarp / 4;                      // 16-byte units per row of the slice
          constexpr int kSliceFloats = 32 * kColsPerWarp;
          const int slice = warp - 2;
          const auto slice_of = [&](int it) {
            return p.partials + (static_cast<int64_t>(it) * kNumEpilogueWarps + slice) * kSliceFloats;
          };
          float4* mine = reinterpret_cast<float4*>(slice_of(item));
#pragma unroll
          for (int u = 0; u < kUnits; ++u) {
            const int c = u / 8, j = u % 8;
            mine[u * 32 + lane] = make_float4(__uint_as_float(buf[c][4 * j]), __uint_as_float(buf[c][4 * j + 1]),
                                              __uint_as_float(buf[c][4 * j + 2]), __uint_as_float(buf[c][4 * j + 3]));
          }
          __syncwarp();  // the lanes' stores are ordered before lane 0's release below
          unsigned int ticket = 0;
          unsigned int* counter = p.tickets + tile * kNumEpilogueWarps + slice;
          if (lane == 0) {
            asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(counter) : "memory");
            if (ticket == static_cast<unsigned int>(splits - 1)) *counter = 0;  // all arrived: ready for the next launch
          }
          ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
          if (warp == 2) CK_TRACE(12);
          if (ticket != static_cast<unsigned int>(splits - 1)) continue;
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) buf[c][i] = 0u;
          }
          for (int sidx = 0; sidx < splits; ++sidx) {
            const float4* theirs = reinterpret_cast<const float4*>(slice_of(tile * splits + sidx));
            float4 t[kUnits];
#pragma unroll
            for (int u = 0; u < kUnits; ++u) t[u] = __ldcg(theirs + u * 32 + lane);
#pragma unroll
            for (int u = 0; u < kUnits; ++u) {
              const int c = u / 8, j = u % 8;
              buf[c][4 * j + 0] = __float_as_uint(__uint_as_float(buf[c][4 * j + 0]) + t[u].x);
              buf[c][4 * j + 1] = __float_as_uint(__uint_as_float(buf[c][4 * j + 1]) + t[u].y);
              buf[c][4 * j + 2] = __float_as_uint(__uint_as_float(buf[c][4 * j + 2]) + t[u].z);
              buf[c][4 * j + 3] = __float_as_uint(__uint_as_float(buf[c][4 * j + 3]) + t[u].w);
            }
          }
        }
        if (warp == 2) CK_TRACE(13);
        if (a_row < p.M) {
          OutT* dst = out + a_row;
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int b_row = n0 + c0 + c * 32 + i;  // activation row = output row
              if (c == 0 && i == 1 && warp == 2) CK_TRACE(14);
              if (c == 0 && i == 8 && warp == 2) CK_TRACE(15);
              if (b_row < p.N) {
                const float y = fmaf(__uint_as_float(buf[c][i]), alpha, bias_v);
                if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
                  dst[static_cast<int64_t>(b_row) * p.M] = __float2bfloat16_rn(y);
                } else if constexpr (std::is_same<OutT, __half>::value) {
                  dst[static_cast<int64_t>(b_row) * p.M] = __float2half_rn(y);
                } else {
                  dst[static_cast<int64_t>(b_row) * p.M] = y;
                }
              }
            }
          }
        }
        if (warp == 2) CK_TRACE(9);
        continue;
      }
      // Bias of a tile's columns as fp32 in shared memory, three buffers in rotation: the
      // buffer of tile t is filled while tile t - 1 is in its epilogue (right after the drain,
      // where the warps are aligned anyway), so no barrier stands between the end of one
      // epilogue and the wait for the next accumulator.  A warp can run at most one tile ahead
      // of the slowest one (the barrier below), hence the third buffer.  Each epilogue thread
      // fetches one value of the next tile before it waits for the accumulator, so the load's
      // latency hides behind that wait.
      float* bias_s = smem_bias + (tile_it % 3) * TILE_N;
      const bool with_bias = p.bias != nullptr && splits == 1;
      if (tile_it == 0) {
        if (et < TILE_N) bias_s[et] = (with_bias && n0 + et < p.N) ? load_bias(p.bias, p.bias_dtype, n0 + et) : 0.0f;
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kNumEpilogueWarps) : "memory");  // epilogue warps only
      }
      const int next_item = item + num_workers;
      const bool has_next = next_item < num_items;
      float bias_prefetched = 0.0f;
      if (has_next && et < TILE_N) {
        const int n = tile_col_block(p, next_item / splits) * TILE_N + et;
        if (with_bias && n < p.N) bias_prefetched = load_bias(p.bias, p.bias_dtype, n);
      }
      if (warp == 2) CK_TRACE(6);
      mbar_wait(&acc_full_bar[acc], acc_ph, abort_flag);  // in a pair: committed from the leader CTA
      if (warp == 2) CK_TRACE(7);
      tc_fence_after_sync();
      const int c0 = half * kColsPerWarp;
      const uint32_t t_row = tmem_base + acc * Cfg::kAccCols + (static_cast<uint32_t>(quarter * 32) << 16) + c0;
      // The fused 16-bit epilogue never holds the raw accumulator: it drains 32 columns at a
      // time and keeps alpha * acc + bias rounded to OutT as packed pairs (a quarter of the
      // registers); the others pull their whole share with back-to-back loads.
      constexpr bool kPackedDrain = FUSED && sizeof(OutT) == 2;
      uint32_t buf[kPackedDrain ? 1 : kChunks][32];
      [[maybe_unused]] uint32_t pk[kPackedDrain ? kChunks : 1][16];
      if constexpr (kPackedDrain) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          tmem_load_32x32(t_row + c * 32, buf[0]);
          tmem_load_wait();
          const float2* b2 = reinterpret_cast<const float2*>(bias_s + c0 + c * 32);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 b = b2[i];
            pk[c][i] = pack_pair<OutT>(fmaf(__uint_as_float(buf[0][2 * i]), alpha, b.x),
                                       fmaf(__uint_as_float(buf[0][2 * i + 1]), alpha, b.y));
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tmem_load_32x32(t_row + c * 32, buf[c]);
        tmem_load_wait();
      }
      if (warp == 2) CK_TRACE(8);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 2) {
          mbar_arrive_cluster(acc_empty_leader + acc * 8);  // the leader's barrier counts both CTAs' warps
        } else {
          mbar_arrive(&acc_empty_bar[acc]);
        }
      }
      if (has_next) {
        if (et < TILE_N) smem_bias[((tile_it + 1) % 3) * TILE_N + et] = bias_prefetched;
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kNumEpilogueWarps) : "memory");  // epilogue warps only
      }
      OutT* out_row = out + static_cast<int64_t>(row) * p.N + n0 + c0;
      if constexpr (!FUSED) {
        bool staged = false;
        if constexpr (OUT_STAGE != 0) staged = p.out_tma != 0;
        if (staged) {
          if constexpr (OUT_STAGE != 0) {
            // The warp's 32 rows x 128 bytes of converted output go to its staging box in the
            // 128-byte-swizzled layout (16-byte unit j of row r at r*128 + ((j ^ r%8) * 16):
            // conflict-free for the 8 lanes of a store phase), then one TMA store writes whole
            // lines; rows past M and columns past N are clipped by the tensor map.
            constexpr int kBoxCols = 128 / static_cast<int>(sizeof(OutT));
            constexpr int kChunksPerBox = kBoxCols / 32;          // 2 for 16-bit outputs, 1 for fp32
            constexpr int kUnitsPerChunk = 32 * static_cast<int>(sizeof(OutT)) / 16;
            static_assert((kChunks / kChunksPerBox - 1) * kNumEpilogueWarps * 4096 <= Cfg::kRingBytes,
                          "the last tile's extra store boxes fit in the idle operand ring");
            const uint32_t stage_warp = smem_u32(smem_out) + (warp - 2) * (OUT_STAGE * 4096);
            const int row0 = tile_m * Cfg::kTileRows + static_cast<int>(cta_rank) * kTileM + quarter * 32;
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
              // A CTA's last tile finds the operand ring idle (every load has landed and every
              // MMA has retired before its accumulator was published): its second and later
              // boxes are staged there, so the warp never waits for a store to release a box.
              const bool in_ring = !has_next && c >= kChunksPerBox;
              const uint32_t stage_box =
                  in_ring ? smem_u32(smem) + ((c / kChunksPerBox - 1) * kNumEpilogueWarps + (warp - 2)) * 4096
                          : stage_warp + (out_box % OUT_STAGE) * 4096;
              const uint32_t stage_row = stage_box + lane * 128;
              if (c == 0 && warp == 2) CK_TRACE(10);
              if (c % kChunksPerBox == 0 && !in_ring) {
                if (lane == 0) bulk_wait_group_read<OUT_STAGE - 1>();  // the store that last used this box has read it
                __syncwarp();
              }
              if (c == 0 && warp == 2) CK_TRACE(11);
              if (c == 2 && warp == 2) CK_TRACE(14);
              float v[32];
              scale_and_bias(buf[c], alpha, bias_s + c0 + c * 32, v);
#pragma unroll
              for (int u = 0; u < kUnitsPerChunk; ++u) {
                uint32_t w[4];
                if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
                      __nv_bfloat162 q = __floats2bfloat162_rn(v[u * 8 + 2 * j], v[u * 8 + 2 * j + 1]);
                      w[j] = *reinterpret_cast<uint32_t*>(&q);
                    } else {
                      __half2 q = __floats2half2_rn(v[u * 8 + 2 * j], v[u * 8 + 2 * j + 1]);
                      w[j] = *reinterpret_cast<uint32_t*>(&q);
                    }
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 4; ++j) w[j] = __float_as_uint(v[u * 4 + j]);
                }
                const int unit = (c % kChunksPerBox) * kUnitsPerChunk + u;
                st_shared_128(stage_row + (((unit ^ lane) & 7) << 4), w[0], w[1], w[2], w[3]);
              }
              if (c == 0 && warp == 2) CK_TRACE(12);
              if (c == 1 && warp == 2) CK_TRACE(13);
              if (c % kChunksPerBox == kChunksPerBox - 1) {
                fence_proxy_async();  // the staged bytes become visible to the TMA engine
                __syncwarp();
                const int col = n0 + c0 + (c / kChunksPerBox) * kBoxCols;
                if (lane == 0 && row0 < p.M && col < p.N) {
                  if (splits > 1) {
                    tma_store_2d_addr(&maps_out.m[split], stage_box, col, row0);  // this item's partial
                  } else {
                    // the same staged box goes to every destination (peer stores cross NVLink)
                    for (int d = 0; d < p.n_out; ++d) tma_store_2d_addr(&maps_out.m[d], stage_box, col, row0);
                  }
                }
                // (an empty group when nothing was stored keeps the ring's group count in step)
                if (lane == 0) bulk_commit_group();
                if (c == 1 && warp == 2) CK_TRACE(15);
                if (!in_ring) ++out_box;
              }
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
            const int valid = min(32, p.N - (n0 + c0 + c * 32));
            if (row < p.M && valid > 0) {
              float v[32];
              scale_and_bias(buf[c], alpha, bias_s + c0 + c * 32, v);
              store_row_chunk<OutT>(out_row + c * 32, v, valid, vec_ok);
            }
          }
        }
      } else {
        // Re-quantization needs whole 64-column groups (4 scale columns = one 32-bit word of
        // the tiled scale layout); the host guarantees N % 64 == 0 when it is requested.
        static_assert(kChunks % 2 == 0, "fused epilogue works on pairs of 32-column chunks");  // 64-column groups
        const float rq_g = (p.rq_codes != nullptr) ? ld_f32_dependent(p.rq_scale) : 1.0f;
        const int rq_col_tiles = (p.N / 16 + 3) / 4;
        const int rows_pad = (p.M + 127) / 128 * 128;
        uint32_t scale_word = 0;
        if constexpr (kPackedDrain) {
          // The values an unfused caller would see are the accumulators rounded to OutT: the
          // activation works on the packed pairs, and the re-quantization runs on the packed
          // words exactly as the stand-alone quantizer does.
          const quant::TensorScale rq_ts = quant::make_tensor_scale(rq_g);
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
            const int col = n0 + c0 + c * 32;
            const int valid = min(32, p.N - col);
            if (valid <= 0) continue;
            if (row < p.M) {
              if (p.activation == CK_ACT_GELU_TANH) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  float a, b;
                  unpack_pair<OutT>(pk[c][i], a, b);
                  pk[c][i] = pack_pair<OutT>(gelu_tanh(a), gelu_tanh(b));
                }
              }
              if (p.out != nullptr) {
                if (vec_ok && valid == 32) {
                  Vec256 o0, o1;
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    o0.w[i] = pk[c][i];
                    o1.w[i] = pk[c][8 + i];
                  }
                  st_global_256_no_allocate(out_row + c * 32, o0);
                  st_global_256_no_allocate(out_row + c * 32 + 16, o1);
                } else {
#pragma unroll
                  for (int i = 0; i < 16; ++i) {  // N % 8 == 0: pairs never straddle the edge
                    if (2 * i < valid) *reinterpret_cast<uint32_t*>(out_row + c * 32 + 2 * i) = pk[c][i];
                  }
                }
              }
            }
            if (p.rq_codes != nullptr) {  // N % 64 == 0 here: every chunk is whole
              if (row < p.M) {
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  lo[i] = pk[c][i];
                  hi[i] = pk[c][8 + i];
                }
                uint32_t w0, w1, w2, w3, s0, s1;
                quant::nvfp4_block_packed<OutT, true>(lo, rq_ts, w0, w1, s0);
                quant::nvfp4_block_packed<OutT, true>(hi, rq_ts, w2, w3, s1);
                *reinterpret_cast<uint4*>(p.rq_codes + static_cast<int64_t>(row) * (p.N >> 1) + (col >> 1)) =
                    make_uint4(w0, w1, w2, w3);
                scale_word |= (s0 | (s1 << 8)) << (16 * (c & 1));
              }
              if ((c & 1) && row < rows_pad) {
                // rows between M and the next multiple of 128 are padding of the scale tensor: zero
                // this chunk and the previous one cover scale columns (col/16 - 2) .. (col/16 + 1)
                const int64_t off = swizzled_scale_offset(row, (col >> 4) - 2, rq_col_tiles);
                *reinterpret_cast<uint32_t*>(p.rq_scales + off) = scale_word;
                scale_word = 0;
              }
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
            const int col = n0 + c0 + c * 32;
            const int valid = min(32, p.N - col);
            if (valid <= 0) continue;
            float v[32];
            if (row < p.M) {
              scale_and_bias(buf[c], alpha, bias_s + c0 + c * 32, v);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                float y = round_to_out<OutT>(v[i]);
                if (p.activation == CK_ACT_GELU_TANH) y = round_to_out<OutT>(gelu_tanh(y));
                v[i] = y;
              }
              if (p.out != nullptr) store_row_chunk<OutT>(out_row + c * 32, v, valid, vec_ok);
            }
            if (p.rq_codes != nullptr) {
              if (row < p.M) {
                float lo16[16], hi16[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  lo16[i] = v[i];
                  hi16[i] = v[16 + i];
                }
                uint32_t w0, w1, w2, w3, s0, s1;
                quant::nvfp4_block<true>(lo16, rq_g, true, w0, w1, s0);
                quant::nvfp4_block<true>(hi16, rq_g, true, w2, w3, s1);
                *reinterpret_cast<uint4*>(p.rq_codes + static_cast<int64_t>(row) * (p.N >> 1) + (col >> 1)) =
                    make_uint4(w0, w1, w2, w3);
                scale_word |= (s0 | (s1 << 8)) << (16 * (c & 1));
              }
              if ((c & 1) && row < rows_pad) {
                const int64_t off = swizzled_scale_offset(row, (col >> 4) - 2, rq_col_tiles);
                *reinterpret_cast<uint32_t*>(p.rq_scales + off) = scale_word;
                scale_word = 0;
              }
            }
          }
        }
      }
      if (warp == 2) CK_TRACE(9);
    }
    if constexpr (OUT_STAGE != 0) {
      // shared memory stays valid until the last store has read it; stores to other GPUs are
      // waited for to the end, so that they precede whatever follows this kernel on the stream
      if (lane == 0) {
        if (p.n_out > 1) {
          bulk_wait_group0();
        } else {
          bulk_wait_group_read0();
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  CK_TRACE3(3);
#ifdef CK_GEMM_TRACE
  if (blockIdx.x < 160) {
    for (int i = threadIdx.x; i < kTraceSmemTiles * kTraceSlots; i += blockDim.x) {
      g_trace[(blockIdx.x * kTraceTiles + i / kTraceSlots) * kTraceSlots + i % kTraceSlots] = trace_s[i];
    }
  }
#endif
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(p.status, 1);
    // give copies that may still be in flight time to land before the CTA's memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if constexpr (CTAS == 2) cluster_sync_all();  // no CTA leaves while its partner may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<CTAS>(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

// Tensor maps are a pure function of (address, extents, box): a small per-thread table keeps the
// ones of recent calls, so that a layer called again with the same buffers pays no encode.
struct MapKey {
  int tag;
  const void* base;
  int64_t d0, d1, d2, d3;
  bool operator==(const MapKey& o) const {
    return tag == o.tag && base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && d3 == o.d3;
  }
};

template <typename Encode>
int cached_map(CUtensorMap* map, const MapKey& key, Encode&& encode) {
  struct Entry {
    MapKey key;
    CUtensorMap map;
    bool valid;
  };
  constexpr int kEntries = 128;
  thread_local std::vector<Entry> table(kEntries);  // on the heap: keeps the library's TLS block small
  uint64_t h = reinterpret_cast<uintptr_t>(key.base) >> 8;
  h = (h ^ (h >> 17) ^ static_cast<uint64_t>(key.tag) * 0x9E3779B97F4A7C15ull ^ static_cast<uint64_t>(key.d1) * 0xC2B2AE3D27D4EB4Full);
  Entry& e = table[(h ^ (h >> 29)) % kEntries];
  if (e.valid && e.key == key) {
    *map = e.map;
    return CK_OK;
  }
  if (int rc = encode(map)) return rc;
  e.key = key;
  e.map = *map;
  e.valid = true;
  return CK_OK;
}

// Row-major [rows, row_bytes] byte matrix, boxes of 128 bytes x box_rows rows, 128-byte swizzle.
int encode_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(CK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kStageKBytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                        elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return CK_OK;
}

// Scale tensor in the tiled layout as a 3-D array {128 x uint32 (one 512-byte tile), column
// tile, row block}; a box is `tiles` consecutive column tiles of one row block.
int encode_scale_map(CUtensorMap* map, const void* base, int64_t row_blocks, int64_t col_tiles, int tiles) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(CK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(col_tiles), static_cast<cuuint64_t>(row_blocks)};
  const cuuint64_t strides[2] = {512, static_cast<cuuint64_t>(col_tiles) * 512};
  const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(tiles), 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box,
                        elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CK_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with code %d", static_cast<int>(r));
  return CK_OK;
}

// Row-major [rows, cols] output of `elem_bytes`-wide elements: boxes of 32 rows x 128 bytes,
// 128-byte swizzle (the layout the epilogue stages its rows in).
int encode_output_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int elem_bytes, int64_t pitch_elems) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(CK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const CUtensorMapDataType type = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), 32};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = fn(map, type, 2, base, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CK_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with code %d", static_cast<int>(r));
  return CK_OK;
}

int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  return cached_map(map, MapKey{0, base, rows, row_bytes, box_rows, 0},
                    [&](CUtensorMap* m) { return encode_operand_map(m, base, rows, row_bytes, box_rows); });
}

int make_scale_map(CUtensorMap* map, const void* base, int64_t row_blocks, int64_t col_tiles, int tiles) {
  return cached_map(map, MapKey{1, base, row_blocks, col_tiles, tiles, 0},
                    [&](CUtensorMap* m) { return encode_scale_map(m, base, row_blocks, col_tiles, tiles); });
}

int make_output_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int elem_bytes, int64_t pitch_elems) {
  return cached_map(map, MapKey{2, base, rows, cols, elem_bytes, pitch_elems},
                    [&](CUtensorMap* m) { return encode_output_map(m, base, rows, cols, elem_bytes, pitch_elems); });
}

// Where the output goes (host side): `n` buffers (1 = plain GEMM), each holding this GEMM's
// [M, N] block at column `col_offset` of a row-major matrix with `pitch` columns.
struct OutputSpec {
  void* const* ptrs = nullptr;
  int n = 1;
  int64_t pitch = 0;
  int64_t col_offset = 0;
  bool plain(int64_t N) const { return n == 1 && pitch == N && col_offset == 0; }
};

// The two operand matrices (device pointers): A [M, k_bytes], B [N, k_bytes] row-major bytes.
struct Operands {
  const void* a;
  const void* b;
};

template <Kind KIND, int TILE_N, int NUM_ACC, int STAGES, int CTAS, typename OutT, bool FUSED, int OUT_STAGE = 0, bool SWAP = false>
int launch_config(const Operands& ops, GemmParams p, const OutputSpec& os, cudaStream_t stream) {
  using Cfg = Config<KIND, TILE_N, NUM_ACC, STAGES, CTAS, OUT_STAGE>;
  auto kernel = block_scaled_gemm_kernel<KIND, TILE_N, NUM_ACC, STAGES, CTAS, OutT, FUSED, OUT_STAGE, SWAP>;
  // only the tensor maps this configuration uses are encoded (host time is visible for small problems)
  CUtensorMap map_a, map_b;
  if (int rc = make_operand_map(&map_a, ops.a, p.M, p.k_bytes, kTileM)) return rc;
  if (int rc = make_operand_map(&map_b, ops.b, p.N, p.k_bytes, Cfg::kBRows)) return rc;
  // the dynamic shared-memory opt-in is per device: do it once for each device that launches
  static std::atomic<bool> configured[64];
  int dev = 0;
  CK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    CK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  p.tiles_m = static_cast<int>(ceil_div(p.M, Cfg::kTileRows));
  p.tiles_n = static_cast<int>(ceil_div(p.N, TILE_N));
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(num_threads(FUSED, TILE_N));
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  // Persistent workers must all be resident at once.  For CTA pairs the number of
  // co-resident clusters can be below sm_count / 2 (pairs must sit in one GPC): ask.
  static std::atomic<int> max_workers[64];
  int resident = (dev >= 0 && dev < 64) ? max_workers[dev].load(std::memory_order_acquire) : 0;
  if (resident == 0) {
    resident = sm_count() / CTAS * ((SWAP && TILE_N <= 128) ? 2 : 1);  // the small swapped configurations share an SM
    if (CTAS > 1) {
      cfg.gridDim = dim3(sm_count() / CTAS * CTAS);
      int clusters = 0;
      CK_CUDA(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
      if (clusters > 0) resident = min(resident, clusters);
    }
    if (dev >= 0 && dev < 64) max_workers[dev].store(resident, std::memory_order_release);
  }
  int workers = min(p.tiles_m * p.tiles_n * p.splits, resident);
#ifdef CK_GEMM_TRACE
  if (const char* e = getenv("CK_GEMM_MAX_WORKERS")) workers = min(workers, atoi(e));
  static std::atomic<int> launch_seq{0};
  p.trace_launch = launch_seq.fetch_add(1);
#endif
  cfg.gridDim = dim3(workers * CTAS);
  CUtensorMap map_sfa = {}, map_sfb = {};
  if (CTAS == 2) {
    if (int rc = make_scale_map(&map_sfa, p.sfa, p.n_row_blocks_a, p.sf_col_tiles, Cfg::kSfTilesPerStage)) return rc;
    if (int rc = make_scale_map(&map_sfb, p.sfb, p.n_row_blocks_b, p.sf_col_tiles, Cfg::kSfTilesPerStage)) return rc;
  }
  // Walking order of the tiles: the one whose concurrently running tiles touch fewer operand bytes
  // (A row blocks + B column blocks of one wave), so that a long operand is not pulled through L2
  // once per tile column (M = 16384, K = 12288: 100 MB of A per wave down the rows, 28 MB along the
  // columns).
  if (!SWAP) {
    const int64_t a_block = static_cast<int64_t>(Cfg::kTileRows) * p.k_bytes, b_block = static_cast<int64_t>(TILE_N) * p.k_bytes;
    const int64_t w = workers, tm = p.tiles_m, tn = p.tiles_n;
    const int64_t down = (w < tm ? w : tm) * a_block + ceil_div(w, tm) * b_block;
    const int64_t along = ceil_div(w, tn) * a_block + (w < tn ? w : tn) * b_block;
    p.raster = along < down ? 1 : 0;
  }
  OutputMaps maps_out = {};
  p.out_tma = 0;
  p.n_out = 1;
  if constexpr (OUT_STAGE != 0) {
    // TMA stores need 16-byte aligned bases and row pitch.  A single dense [M, N] result whose rows
    // start on 32-byte boundaries is written straight from registers instead (256-bit stores, whole
    // sectors): measured 1-3 % faster than staging it for TMA stores, whose shared-memory traffic
    // slows the next tile's main loop.  Partial tiles of a split and multi-destination stores
    // (all-gather) go through the staged path.
    bool ok = p.out != nullptr && (os.pitch * static_cast<int64_t>(sizeof(OutT))) % 16 == 0 &&
              (os.col_offset * static_cast<int64_t>(sizeof(OutT))) % 16 == 0;
    for (int d = 0; ok && d < os.n; ++d) ok = os.ptrs[d] != nullptr && reinterpret_cast<uintptr_t>(os.ptrs[d]) % 16 == 0;
    const bool direct = os.n == 1 && p.splits == 1 && os.plain(p.N) && p.out != nullptr &&
                        (static_cast<int64_t>(p.N) * sizeof(OutT)) % 32 == 0 && reinterpret_cast<uintptr_t>(p.out) % 32 == 0;
    ok = ok && !direct;
    if (ok) {
      for (int d = 0; d < os.n; ++d) {
        void* base = static_cast<uint8_t*>(os.ptrs[d]) + os.col_offset * static_cast<int64_t>(sizeof(OutT));
        if (int rc = make_output_map(&maps_out.m[d], base, p.M, p.N, sizeof(OutT), os.pitch)) return rc;
      }
      p.out_tma = 1;
      p.n_out = os.n;
    }
  }
  if (p.out_tma == 0 && !os.plain(p.N)) {
    return fail(CK_ERR_INVALID_ARGUMENT, "strided or multiple outputs need 16-byte aligned buffers, pitch and column offset");
  }
  CK_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_sfa, map_sfb, maps_out, p));
  return CK_OK;
}

}  // namespace
}  // namespace ck
