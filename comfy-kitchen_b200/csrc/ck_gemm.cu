// Block-scaled GEMMs for sm_100a: out[M,N] = cast((A[M,K] . B[N,K]^T) * alpha + bias).
//
//   NVFP4: A, B packed E2M1 (two per byte), E4M3 scale per 16 elements  (kind::mxf4nvf4)
//   MXFP8: A, B E4M3 bytes,                  E8M0 scale per 32 elements  (kind::mxf8f6f4)
//
// One persistent CTA per SM, six warps with fixed roles:
//   warp 0    TMA producer: per pipeline stage one 128-row x 128-byte box of A, one
//             TILE_N-row box of B (128-byte swizzle) and the matching 512-byte scale tiles
//             (linear bulk copies - in the tiled scale layout the tiles a stage needs are
//             contiguous in global memory) into a STAGES-deep shared-memory ring.
//   warp 1    MMA issuer: copies the stage's scale tiles shared -> tensor memory
//             (tcgen05.cp), issues four tcgen05.mma per stage (32 bytes of K each) into a
//             fp32 accumulator in tensor memory, and releases the stage / publishes the
//             accumulator with tcgen05.commit.
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp its own 32-lane quarter),
//             scale by alpha, add bias, convert, store; then hand the accumulator back.
// With NUM_ACC == 2 the epilogue of tile i overlaps the main loop of tile i+1.
//
// All synchronisation is by mbarriers with bounded waits (ck_sm100.cuh): a protocol error
// raises the device status word instead of hanging.
#include "ck_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <mutex>
#include <type_traits>

namespace ck {
namespace {

using namespace sm100;

enum class Kind { kNvfp4, kMxfp8 };

constexpr int kTileM = 128;
constexpr int kStageKBytes = 128;   // bytes of K per operand row per stage (one swizzle atom)
constexpr int kMmaKBytes = 32;      // bytes of K per tcgen05.mma
constexpr int kMmaPerStage = kStageKBytes / kMmaKBytes;
constexpr int kNumThreads = 192;    // 6 warps
constexpr int kTmemCols = 512;

template <Kind KIND, int TILE_N, int NUM_ACC, int STAGES>
struct Config {
  static constexpr int kABytes = kTileM * kStageKBytes;
  static constexpr int kBBytes = TILE_N * kStageKBytes;
  // 512-byte scale tiles (128 rows x 4 scale columns) one 128-row block needs per stage:
  // NVFP4 has 16 scale columns per 256 elements, MXFP8 4 per 128 elements.
  static constexpr int kSfTilesPerStage = (KIND == Kind::kNvfp4) ? 4 : 1;
  // 128-row blocks of B's scale tensor a tile can touch (a 192-wide tile straddles two)
  static constexpr int kSfbRowBlocks = (TILE_N + 127) / 128;
  static constexpr int kSfaBytes = kSfTilesPerStage * 512;
  static constexpr int kSfbBytes = kSfbRowBlocks * kSfTilesPerStage * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kSmemBytes = STAGES * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // tensor memory columns
  static constexpr int kAccCols = TILE_N;
  static constexpr int kSfaCol = NUM_ACC * kAccCols;
  static constexpr int kSfaColsPerStage = kSfTilesPerStage * 4;
  static constexpr int kSfbCol = kSfaCol + kSfaColsPerStage;
  static constexpr int kSfbColsPerTile = kSfbRowBlocks * 4;
  static constexpr int kSfbColsPerStage = kSfTilesPerStage * kSfbColsPerTile;
  static_assert(kSfbCol + kSfbColsPerStage <= kTmemCols, "tensor memory budget exceeded");
  static_assert(TILE_N % 16 == 0 && TILE_N >= 16 && TILE_N <= 256, "invalid MMA N");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget exceeded");
  static constexpr uint32_t kIdesc = make_block_scaled_idesc(KIND == Kind::kNvfp4 ? 1u : 0u,
                                                             KIND == Kind::kNvfp4 ? 0u : 1u, kTileM, TILE_N);
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
  int n_row_blocks_b;      // ceil(N / 128)
  int tiles_m, tiles_n;
  int* status;             // device status word: set non-zero when a wait gave up
};

__device__ int g_gemm_status = 0;

template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* dst, const float (&v)[32], int valid) {
  // dst points at 32 consecutive output columns of one row; `valid` of them exist.
  if constexpr (sizeof(OutT) == 2) {
    if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
            __nv_bfloat162 p = __floats2bfloat162_rn(v[i * 8 + 2 * j], v[i * 8 + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&p);
          } else {
            __half2 p = __floats2half2_rn(v[i * 8 + 2 * j], v[i * 8 + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&p);
          }
        }
        reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i < valid) {
        if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
          dst[i] = __float2bfloat16_rn(v[i]);
        } else {
          dst[i] = __float2half_rn(v[i]);
        }
      }
    }
  } else {
    if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      return;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = v[i];
  }
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int n) {
  if (dtype == CK_DTYPE_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
  if (dtype == CK_DTYPE_F16) return __half2float(static_cast<const __half*>(bias)[n]);
  return static_cast<const float*>(bias)[n];
}

template <Kind KIND, int TILE_N, int NUM_ACC, int STAGES, typename OutT>
__global__ void __launch_bounds__(kNumThreads, 1)
block_scaled_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p) {
  using Cfg = Config<KIND, TILE_N, NUM_ACC, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + STAGES * Cfg::kABytes;
  uint8_t* smem_sfa = smem_b + STAGES * Cfg::kBBytes;
  uint8_t* smem_sfb = smem_sfa + STAGES * Cfg::kSfaBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_sfb + STAGES * Cfg::kSfbBytes);
  uint64_t* full_bar = bars;                       // [STAGES] producer -> MMA
  uint64_t* empty_bar = bars + STAGES;             // [STAGES] MMA -> producer
  uint64_t* acc_full_bar = bars + 2 * STAGES;      // [NUM_ACC] MMA -> epilogue
  uint64_t* acc_empty_bar = acc_full_bar + NUM_ACC;  // [NUM_ACC] epilogue -> MMA
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + NUM_ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], 4);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) tmem_alloc(tmem_base_slot, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_stages = (p.k_bytes + kStageKBytes - 1) / kStageKBytes;
  const int total_mma = (p.k_bytes + kMmaKBytes - 1) / kMmaKBytes;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        // consecutive CTAs work on tiles that share the B columns (tile_m fastest)
        const int tile_m = tile % p.tiles_m;
        const int tile_n = tile / p.tiles_m;
        const int m0 = tile_m * kTileM;
        const int n0 = tile_n * TILE_N;
        const int rb_b0 = n0 / 128;
        for (int ks = 0; ks < k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          mbar_wait(&empty_bar[s], ph ^ 1, abort_flag);
          const int sf_tile0 = ks * Cfg::kSfTilesPerStage;
          const int sf_tiles = min(Cfg::kSfTilesPerStage, p.sf_col_tiles - sf_tile0);
          int rb_b_count = 0;
          for (int r = 0; r < Cfg::kSfbRowBlocks; ++r) rb_b_count += (rb_b0 + r < p.n_row_blocks_b) ? 1 : 0;
          const uint32_t tx = Cfg::kABytes + Cfg::kBBytes + static_cast<uint32_t>(sf_tiles) * 512u * (1 + rb_b_count);
          mbar_arrive_expect_tx(&full_bar[s], tx);
          tma_load_2d(smem_a + s * Cfg::kABytes, &map_a, &full_bar[s], ks * kStageKBytes, m0);
          tma_load_2d(smem_b + s * Cfg::kBBytes, &map_b, &full_bar[s], ks * kStageKBytes, n0);
          bulk_load_1d(smem_sfa + s * Cfg::kSfaBytes,
                       p.sfa + (static_cast<int64_t>(tile_m) * p.sf_col_tiles + sf_tile0) * 512, sf_tiles * 512,
                       &full_bar[s]);
          for (int r = 0; r < Cfg::kSfbRowBlocks; ++r) {
            if (rb_b0 + r < p.n_row_blocks_b) {
              bulk_load_1d(smem_sfb + s * Cfg::kSfbBytes + r * Cfg::kSfTilesPerStage * 512,
                           p.sfb + (static_cast<int64_t>(rb_b0 + r) * p.sf_col_tiles + sf_tile0) * 512, sf_tiles * 512,
                           &full_bar[s]);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t tile_it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_it) {
        const int tile_n = tile / p.tiles_m;
        const int n0 = tile_n * TILE_N;
        const int acc = tile_it % NUM_ACC;
        const uint32_t acc_ph = (tile_it / NUM_ACC) & 1;
        mbar_wait(&acc_empty_bar[acc], acc_ph ^ 1, abort_flag);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * Cfg::kAccCols;
        // B scale words of this tile start (n0 % 128) / 32 columns into the first row block
        const uint32_t sfb_shift = (n0 % 128) / 32;
        for (int ks = 0; ks < k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          mbar_wait(&full_bar[s], ph, abort_flag);
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * Cfg::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + s * Cfg::kBBytes);
          const uint32_t sfa_addr = smem_u32(smem_sfa + s * Cfg::kSfaBytes);
          const uint32_t sfb_addr = smem_u32(smem_sfb + s * Cfg::kSfbBytes);
          // scale tiles of this stage: shared -> tensor memory
#pragma unroll
          for (int t = 0; t < Cfg::kSfTilesPerStage; ++t) {
            tc_copy_scales_32x128b(tmem_base + Cfg::kSfaCol + t * 4, make_scale_desc(sfa_addr + t * 512));
#pragma unroll
            for (int r = 0; r < Cfg::kSfbRowBlocks; ++r) {
              tc_copy_scales_32x128b(tmem_base + Cfg::kSfbCol + t * Cfg::kSfbColsPerTile + r * 4,
                                     make_scale_desc(sfb_addr + (r * Cfg::kSfTilesPerStage + t) * 512));
            }
          }
          const uint64_t a_desc = make_operand_desc_sw128(a_addr);
          const uint64_t b_desc = make_operand_desc_sw128(b_addr);
#pragma unroll
          for (int kb = 0; kb < kMmaPerStage; ++kb) {
            if (ks * kMmaPerStage + kb < total_mma) {
              const uint32_t accumulate = (ks > 0 || kb > 0) ? 1u : 0u;
              // advancing K inside the swizzle atom = advancing the start address
              const uint64_t koff = static_cast<uint64_t>((kb * kMmaKBytes) >> 4);
              if constexpr (KIND == Kind::kNvfp4) {
                mma_nvfp4(d_tmem, a_desc + koff, b_desc + koff, Cfg::kIdesc, tmem_base + Cfg::kSfaCol + kb * 4,
                          tmem_base + Cfg::kSfbCol + kb * Cfg::kSfbColsPerTile + sfb_shift, accumulate);
              } else {
                // one scale tile serves the four MMAs of the stage; byte kb of each scale word
                mma_mxfp8(d_tmem, a_desc + koff, b_desc + koff, idesc_with_scale_ids(Cfg::kIdesc, kb),
                          tmem_base + Cfg::kSfaCol, tmem_base + Cfg::kSfbCol + sfb_shift, accumulate);
              }
            }
          }
          tc_commit(&empty_bar[s]);  // stage reusable once these MMAs (and copies) retire
        }
        tc_commit(&acc_full_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // tensor-memory lanes this warp may read: 32*quarter .. +31
    float alpha = 1.0f;
    if (p.alpha != nullptr) {
      alpha = __ldg(p.alpha);
    } else if (p.tsa != nullptr && p.tsb != nullptr) {
      alpha = __ldg(p.tsa) * __ldg(p.tsb);
    }
    OutT* out = static_cast<OutT*>(p.out);
    uint32_t tile_it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_it) {
      const int tile_m = tile % p.tiles_m;
      const int tile_n = tile / p.tiles_m;
      const int row = tile_m * kTileM + quarter * 32 + lane;
      const int n0 = tile_n * TILE_N;
      const int acc = tile_it % NUM_ACC;
      const uint32_t acc_ph = (tile_it / NUM_ACC) & 1;
      mbar_wait(&acc_full_bar[acc], acc_ph, abort_flag);
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * Cfg::kAccCols + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < TILE_N; c += 32) {
        uint32_t raw[32];
        tmem_load_32x32(t_row + c, raw);
        tmem_load_wait();
        if (c + 32 >= TILE_N) {
          // last read of this accumulator: hand it back before the stores
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
        }
        const int col = n0 + c;
        const int valid = min(32, p.N - col);
        if (row < p.M && valid > 0) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]) * alpha;
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) v[i] += load_bias(p.bias, p.bias_dtype, col + i);
          }
          store_row_chunk<OutT>(out + static_cast<int64_t>(row) * p.N + col, v, valid);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(p.status, 1);
    // give copies that may still be in flight time to land before the CTA's memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
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

// Row-major [rows, row_bytes] byte matrix, boxes of 128 bytes x box_rows rows, 128-byte swizzle.
int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
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

template <Kind KIND, int TILE_N, int NUM_ACC, int STAGES, typename OutT>
int launch_config(const CUtensorMap& map_a, const CUtensorMap& map_b, GemmParams p, cudaStream_t stream) {
  using Cfg = Config<KIND, TILE_N, NUM_ACC, STAGES>;
  auto kernel = block_scaled_gemm_kernel<KIND, TILE_N, NUM_ACC, STAGES, OutT>;
  // the dynamic shared-memory opt-in is per device: do it once for each device that launches
  static std::atomic<bool> configured[64];
  int dev = 0;
  CK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    CK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  p.tiles_m = static_cast<int>(ceil_div(p.M, kTileM));
  p.tiles_n = static_cast<int>(ceil_div(p.N, TILE_N));
  const int grid = min(p.tiles_m * p.tiles_n, sm_count());
  kernel<<<grid, kNumThreads, Cfg::kSmemBytes, stream>>>(map_a, map_b, p);
  CK_CUDA(cudaGetLastError());
  return CK_OK;
}

template <Kind KIND, typename OutT>
int launch_for_shape(const CUtensorMap& map_a, const CUtensorMap& map_b128, const CUtensorMap& map_b256,
                     const GemmParams& p, cudaStream_t stream) {
  // Wide tiles when the problem fills the machine with them, else narrower tiles for more CTAs.
  const int64_t tiles256 = ceil_div(p.M, kTileM) * ceil_div(p.N, 256);
  if (tiles256 >= sm_count()) return launch_config<KIND, 256, 1, 4, OutT>(map_a, map_b256, p, stream);
  return launch_config<KIND, 128, 2, 6, OutT>(map_a, map_b128, p, stream);
}

template <Kind KIND>
int scaled_mm(const char* op, const void* a, const void* b, const void* sfa, const void* sfb, const float* tsa,
              const float* tsb, const float* alpha, const void* bias, int bias_dtype, void* out, int out_dtype,
              int64_t M, int64_t N, int64_t K, void* stream) {
  CK_REQUIRE(a && b && sfa && sfb && out, "%s: null pointer", op);
  CK_REQUIRE(M > 0 && N > 0 && K > 0, "%s: empty problem M=%lld N=%lld K=%lld", op, (long long)M, (long long)N,
             (long long)K);
  CK_REQUIRE(M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30), "%s: dimension too large", op);
  CK_REQUIRE(K % 32 == 0, "%s: K=%lld must be a multiple of 32", op, (long long)K);
  CK_REQUIRE(N % 8 == 0, "%s: N=%lld must be a multiple of 8", op, (long long)N);
  CK_REQUIRE(out_dtype == CK_DTYPE_F32 || out_dtype == CK_DTYPE_F16 || out_dtype == CK_DTYPE_BF16,
             "%s: unsupported output dtype code %d", op, out_dtype);
  CK_REQUIRE(bias == nullptr || bias_dtype == CK_DTYPE_F32 || bias_dtype == CK_DTYPE_F16 || bias_dtype == CK_DTYPE_BF16,
             "%s: unsupported bias dtype code %d", op, bias_dtype);
  CK_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0,
             "%s: operands must be 16-byte aligned", op);
  CK_REQUIRE(reinterpret_cast<uintptr_t>(sfa) % 16 == 0 && reinterpret_cast<uintptr_t>(sfb) % 16 == 0,
             "%s: block scales must be 16-byte aligned", op);
  if (KIND == Kind::kNvfp4) CK_REQUIRE(alpha != nullptr || (tsa != nullptr && tsb != nullptr), "%s: null tensor scale", op);

  const int block = (KIND == Kind::kNvfp4) ? 16 : 32;
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.tsa = tsa;
  p.tsb = tsb;
  p.alpha = alpha;
  p.bias = bias;
  p.out = out;
  p.bias_dtype = bias_dtype;
  p.out_dtype = out_dtype;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.k_bytes = static_cast<int>(KIND == Kind::kNvfp4 ? K / 2 : K);
  p.sf_col_tiles = static_cast<int>(ceil_div(K / block, 4));
  p.n_row_blocks_b = static_cast<int>(ceil_div(N, 128));
  CK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.status), g_gemm_status));

  CUtensorMap map_a, map_b128, map_b256;
  if (int rc = make_operand_map(&map_a, a, M, p.k_bytes, kTileM)) return rc;
  if (int rc = make_operand_map(&map_b128, b, N, p.k_bytes, 128)) return rc;
  if (int rc = make_operand_map(&map_b256, b, N, p.k_bytes, 256)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case CK_DTYPE_BF16:
      return launch_for_shape<KIND, __nv_bfloat16>(map_a, map_b128, map_b256, p, s);
    case CK_DTYPE_F16:
      return launch_for_shape<KIND, __half>(map_a, map_b128, map_b256, p, s);
    default:
      return launch_for_shape<KIND, float>(map_a, map_b128, map_b256, p, s);
  }
}

}  // namespace
}  // namespace ck

extern "C" int ck_scaled_mm_nvfp4(const void* a, const void* b, const void* sfa, const void* sfb,
                                  const float* tensor_scale_a, const float* tensor_scale_b, const float* alpha,
                                  const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N,
                                  int64_t K, void* stream) {
  return ck::scaled_mm<ck::Kind::kNvfp4>("scaled_mm_nvfp4", a, b, sfa, sfb, tensor_scale_a, tensor_scale_b, alpha, bias,
                                         bias_dtype, out, out_dtype, M, N, K, stream);
}

extern "C" int ck_scaled_mm_mxfp8(const void* a, const void* b, const void* sfa, const void* sfb, const void* bias,
                                  int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                                  void* stream) {
  return ck::scaled_mm<ck::Kind::kMxfp8>("scaled_mm_mxfp8", a, b, sfa, sfb, nullptr, nullptr, nullptr, bias, bias_dtype,
                                         out, out_dtype, M, N, K, stream);
}

// Device status word of the GEMM kernels: 0 = every wait completed; non-zero = some wait
// gave up (results of that launch are invalid).  Synchronises the device; resets the word.
extern "C" int ck_gemm_status(int* status_out) {
  int v = 0;
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyFromSymbol(&v, ck::g_gemm_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    CK_CUDA(cudaMemcpyToSymbol(ck::g_gemm_status, &zero, sizeof(int)));
  }
  if (status_out != nullptr) *status_out = v;
  return CK_OK;
}
