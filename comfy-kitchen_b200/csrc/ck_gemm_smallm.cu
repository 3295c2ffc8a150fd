// Block-scaled GEMMs with very few activation rows (M <= 32): weight streaming.
//
// out[M, N] = x[M, K] . W[N, K]^T with M small reads the whole weight once and does almost no
// arithmetic: it is bound by HBM (0.5625 bytes per NVFP4 weight element) and by fixed latencies.
// The 128-row tile configurations spend their MMA rows, their operand loads and their epilogue on
// padding.  Here the operands change places (ck_gemm_kernel.cuh, SWAP): weight rows fill the 128
// tensor-memory lanes, the activation rows are the MMA's N (32), the accumulator is 32 columns
// wide and the epilogue writes 32 values per thread.  When the weight has few 128-row tiles and a
// long K, every tile's K range is cut into work items so that all SMs stream (two CTAs fit on an
// SM); the items of a tile are added through a workspace by whichever warp finishes last, in
// split order.  Measured against the tile path: wins up to 32 rows, loses from 64 rows on.
#include "ck_gemm_kernel.cuh"

namespace ck {
namespace {

constexpr int kMaxSmallM = 32;
constexpr int kSmallTileN = 32;  // the MMA's N: activation rows, padded

struct SmallPlan {
  int splits;              // work items per 128-row weight tile
  int k_stages_per_split;
  int64_t partial_bytes;   // splits > 1: tiles x splits x 128 x tile_n floats
};

SmallPlan plan_small(int64_t N, int k_bytes) {
  SmallPlan pl{};
  const int k_stages = static_cast<int>(ceil_div(k_bytes, kStageKBytes));
  const int64_t tiles = ceil_div(N, kTileM);
  // Splitting K costs a round trip through L2 per item (measured: it pays only when a third of the
  // SMs or fewer would stream otherwise and every item keeps at least four pipeline stages).
  int64_t splits = 1;
  if (tiles * 3 <= sm_count() && k_stages >= 16) {
    splits = 2 * static_cast<int64_t>(sm_count()) / tiles;
    if (splits > 8) splits = 8;
    if (splits > k_stages / 4) splits = k_stages / 4;
    if (splits < 1) splits = 1;
  }
  pl.k_stages_per_split = static_cast<int>(ceil_div(k_stages, splits));
  pl.splits = static_cast<int>(ceil_div(k_stages, pl.k_stages_per_split));
  if (tiles * 8 * 4 > kWorkspaceTicketBytes) {  // more tiles than counters (one per tile and epilogue warp): no need to split
    pl.splits = 1;
    pl.k_stages_per_split = k_stages;
  }
  pl.partial_bytes = pl.splits > 1 ? tiles * pl.splits * kTileM * kSmallTileN * 4 : 0;
  return pl;
}

template <Kind KIND, typename OutT>
int launch_small(const Operands& ops, const GemmParams& p, cudaStream_t stream) {
  OutputSpec os;
  void* const single[1] = {p.out};
  os.ptrs = single;
  os.n = 1;
  os.pitch = p.N;
  os.col_offset = 0;
  return launch_config<KIND, kSmallTileN, 2, 4, 1, OutT, false, 0, true>(ops, p, os, stream);
}

}  // namespace

bool small_m_applies(int64_t M, int64_t N, int64_t K) { return M >= 1 && M <= kMaxSmallM && N >= 1 && K >= 32; }

int64_t small_m_workspace_bytes(bool is_mxfp8, int64_t M, int64_t N, int64_t K) {
  if (!small_m_applies(M, N, K)) return 0;
  const SmallPlan pl = plan_small(N, static_cast<int>(is_mxfp8 ? K : K / 2));
  return pl.splits > 1 ? kWorkspaceTicketBytes + pl.partial_bytes : 0;
}

// a: activation [M, K], b: weight [N, K] (the public argument order); shapes and pointers were validated by the caller.
int scaled_mm_small_m(bool is_mxfp8, const void* a, const void* b, const void* sfa, const void* sfb, const float* tsa,
                      const float* tsb, const float* alpha, const void* bias, int bias_dtype, void* out, int out_dtype,
                      int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes, cudaStream_t stream) {
  const int block = is_mxfp8 ? 32 : 16;
  GemmParams p{};
  // operands change places: the kernel's "A" is the weight
  p.sfa = static_cast<const uint8_t*>(sfb);
  p.sfb = static_cast<const uint8_t*>(sfa);
  p.tsa = tsa;
  p.tsb = tsb;
  p.alpha = alpha;
  p.bias = bias;
  p.out = out;
  p.bias_dtype = bias_dtype;
  p.out_dtype = out_dtype;
  p.M = static_cast<int>(N);
  p.N = static_cast<int>(M);
  p.k_bytes = static_cast<int>(is_mxfp8 ? K : K / 2);
  p.sf_col_tiles = static_cast<int>(ceil_div(K / block, 4));
  p.n_row_blocks_a = static_cast<int>(ceil_div(N, 128));
  p.n_row_blocks_b = static_cast<int>(ceil_div(M, 128));
  if (int rc = gemm_status_word(&p.status)) return rc;
  SmallPlan pl = plan_small(N, p.k_bytes);
  const int64_t need = kWorkspaceTicketBytes + pl.partial_bytes;
  if (pl.splits > 1 && (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 16 != 0)) {
    pl.splits = 1;  // no (usable) workspace: one item per tile
    pl.k_stages_per_split = static_cast<int>(ceil_div(p.k_bytes, kStageKBytes));
  }
  p.splits = pl.splits;
  p.k_stages_per_split = pl.k_stages_per_split;
  if (pl.splits > 1) {
    p.tickets = static_cast<unsigned int*>(workspace);
    p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kWorkspaceTicketBytes);
  }
  const Operands ops = {b, a};
  if (is_mxfp8) {
    switch (out_dtype) {
      case CK_DTYPE_BF16: return launch_small<Kind::kMxfp8, __nv_bfloat16>(ops, p, stream);
      case CK_DTYPE_F16: return launch_small<Kind::kMxfp8, __half>(ops, p, stream);
      default: return launch_small<Kind::kMxfp8, float>(ops, p, stream);
    }
  }
  switch (out_dtype) {
    case CK_DTYPE_BF16: return launch_small<Kind::kNvfp4, __nv_bfloat16>(ops, p, stream);
    case CK_DTYPE_F16: return launch_small<Kind::kNvfp4, __half>(ops, p, stream);
    default: return launch_small<Kind::kNvfp4, float>(ops, p, stream);
  }
}

}  // namespace ck

#ifdef CK_GEMM_TRACE
// Timeline buffers of this translation unit's kernels (see gemm_timeline.py --small-m).
extern "C" __attribute__((visibility("default"))) int ck_debug_trace_smallm(long long* host_out) {
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyFromSymbol(host_out, ck::g_trace, sizeof(long long) * 160 * ck::kTraceTiles * ck::kTraceSlots));
  return CK_OK;
}
extern "C" __attribute__((visibility("default"))) int ck_debug_trace3_smallm(long long* host_out) {
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyFromSymbol(host_out, ck::g_trace3, sizeof(long long) * 8 * 160 * 8));
  return CK_OK;
}
#endif
