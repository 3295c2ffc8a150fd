// Block-scaled GEMM entry points (scaled_mm_nvfp4 / scaled_mm_mxfp8, fused linear, split-K with a
// workspace, all-gather variants): shape-based choice of the kernel configuration of
// ck_gemm_kernel.cuh, argument validation, and the device status word.
#include "ck_gemm_kernel.cuh"

namespace ck {

__device__ int g_gemm_status = 0;

// Device address of the status word on the current device (looked up once per device).
int gemm_status_word(int** out) {
  static std::atomic<int*> cached[64];
  int dev = 0;
  CK_CUDA(cudaGetDevice(&dev));
  int* ptr = (dev >= 0 && dev < 64) ? cached[dev].load(std::memory_order_acquire) : nullptr;
  if (ptr == nullptr) {
    CK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_gemm_status));
    if (dev >= 0 && dev < 64) cached[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return CK_OK;
}

namespace {

int forced_config() {
  // CK_GEMM_CONFIG pins the kernel configuration (used by the tests to cover each one); unset =
  // choose by shape.
  //   1 = one CTA, 128 x 128 tiles (two accumulators)   3 = one CTA, 128 x 256 tiles
  //   4 = CTA pair, 256 x 256 tiles                      7 = one CTA, 128 x 64 tiles (small problems)
  const char* e = getenv("CK_GEMM_CONFIG");
  return e ? atoi(e) : 0;
}

template <Kind KIND, typename OutT, bool FUSED>
int launch_for_shape(const Operands& ops, const GemmParams& p, const OutputSpec& os, cudaStream_t stream) {
  int config = forced_config();
  if (config == 0) {
    const int64_t pair_tiles = ceil_div(p.M, 256) * ceil_div(p.N, 256);
    if (pair_tiles * 4 >= sm_count()) {
      config = 4;  // measured: from about a quarter of the SM count in pair tiles the pair wins
    } else if (ceil_div(p.M, kTileM) * ceil_div(p.N, 128) * 4 <= sm_count()) {
      config = 7;  // so few 128 x 128 tiles that halving them still leaves SMs idle: more, smaller CTAs
    } else {
      config = 1;
    }
  }
  // strided / multiple destinations exist only in the configurations with a staged epilogue
  if (!os.plain(p.N) && config != 4 && config != 7) config = 1;
  switch (config) {
    case 7:
      if constexpr (!FUSED) return launch_config<KIND, 64, 2, 6, 1, OutT, false, 1>(ops, p, os, stream);
      return launch_config<KIND, 128, 2, 6, 1, OutT, FUSED>(ops, p, os, stream);
    case 4:
      return launch_config<KIND, 256, 1, 5, 2, OutT, FUSED, FUSED ? 0 : 1>(ops, p, os, stream);
    case 3:
      return launch_config<KIND, 256, 1, 4, 1, OutT, FUSED>(ops, p, os, stream);
    default:
      if constexpr (!FUSED) return launch_config<KIND, 128, 2, 5, 1, OutT, false, 1>(ops, p, os, stream);
      return launch_config<KIND, 128, 2, 6, 1, OutT, FUSED>(ops, p, os, stream);
  }
}

// ---------------------------------------------------------------------------
// split-K
// ---------------------------------------------------------------------------
struct SplitPlan {
  int splits;
  int k_stages_per_split;
};

// More than one split only when the 128 x 128 tiles leave at least half of the SMs idle and K is
// long enough (>= 16 pipeline stages) for the extra pass over the partial tiles to pay.
SplitPlan plan_splits(int64_t M, int64_t N, int k_bytes) {
  const int k_stages = static_cast<int>(ceil_div(k_bytes, kStageKBytes));
  const int64_t tiles = ceil_div(M, kTileM) * ceil_div(N, 128);
  SplitPlan plan = {1, k_stages};
  if (tiles * 2 > sm_count() || k_stages < 16) return plan;
  const int64_t by_sms = sm_count() / tiles;
  int splits = min(kMaxOutputs, k_stages / 6);
  if (by_sms < splits) splits = static_cast<int>(by_sms);
  if (splits < 2) return plan;
  plan.k_stages_per_split = static_cast<int>(ceil_div(k_stages, splits));
  plan.splits = static_cast<int>(ceil_div(k_stages, plan.k_stages_per_split));
  return plan;
}

// out = cast(alpha * (partial_0 + partial_1 + ...) + bias), four consecutive columns per thread;
// the partials are added in index order, so the result does not depend on scheduling.
template <typename OutT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* partials, int splits, int64_t mn, int n_cols, const float* alpha_ptr, const float* tsa,
                     const float* tsb, const void* bias, int bias_dtype, OutT* out) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= mn) return;
  float alpha = 1.0f;
  if (alpha_ptr != nullptr) {
    alpha = ld_f32_dependent(alpha_ptr);
  } else if (tsa != nullptr && tsb != nullptr) {
    alpha = ld_f32_dependent(tsa) * ld_f32_dependent(tsb);
  }
  float4 acc = *reinterpret_cast<const float4*>(partials + i);
  for (int sidx = 1; sidx < splits; ++sidx) {
    const float4 v = *reinterpret_cast<const float4*>(partials + sidx * mn + i);
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
  }
  const int n = static_cast<int>(i % n_cols);
  float b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = load_bias(bias, bias_dtype, n + j);
  }
  const float r[4] = {fmaf(acc.x, alpha, b[0]), fmaf(acc.y, alpha, b[1]), fmaf(acc.z, alpha, b[2]), fmaf(acc.w, alpha, b[3])};
  if constexpr (std::is_same<OutT, float>::value) {
    *reinterpret_cast<float4*>(out + i) = make_float4(r[0], r[1], r[2], r[3]);
  } else {
    uint2 o;
    o.x = pack_pair<OutT>(r[0], r[1]);
    o.y = pack_pair<OutT>(r[2], r[3]);
    *reinterpret_cast<uint2*>(out + i) = o;
  }
}

int launch_splitk_reduce(const float* partials, int splits, int64_t M, int64_t N, const GemmParams& p, cudaStream_t stream) {
  const int64_t mn = M * N;
  const dim3 grid(static_cast<unsigned>(ceil_div(mn / 4, 256))), block(256);
  const int n_cols = static_cast<int>(N);
  switch (p.out_dtype) {
    case CK_DTYPE_BF16:
      CK_CUDA(launch_pdl(splitk_reduce_kernel<__nv_bfloat16>, grid, block, 0, stream, partials, splits, mn, n_cols, p.alpha, p.tsa,
                         p.tsb, p.bias, p.bias_dtype, static_cast<__nv_bfloat16*>(p.out)));
      break;
    case CK_DTYPE_F16:
      CK_CUDA(launch_pdl(splitk_reduce_kernel<__half>, grid, block, 0, stream, partials, splits, mn, n_cols, p.alpha, p.tsa, p.tsb,
                         p.bias, p.bias_dtype, static_cast<__half*>(p.out)));
      break;
    default:
      CK_CUDA(launch_pdl(splitk_reduce_kernel<float>, grid, block, 0, stream, partials, splits, mn, n_cols, p.alpha, p.tsa, p.tsb,
                         p.bias, p.bias_dtype, static_cast<float*>(p.out)));
  }
  return CK_OK;
}

struct FusedArgs {
  bool enabled = false;
  int activation = CK_ACT_NONE;
  void* rq_codes = nullptr;
  void* rq_scales = nullptr;
  const float* rq_scale = nullptr;
};

template <Kind KIND>
int scaled_mm(const char* op, const void* a, const void* b, const void* sfa, const void* sfb, const float* tsa,
              const float* tsb, const float* alpha, const void* bias, int bias_dtype, void* out, int out_dtype,
              int64_t M, int64_t N, int64_t K, void* stream, const FusedArgs& fused = FusedArgs(),
              const OutputSpec* out_spec = nullptr, void* workspace = nullptr, int64_t workspace_bytes = 0) {
  CK_REQUIRE(a && b && sfa && sfb, "%s: null pointer", op);
  CK_REQUIRE(out != nullptr || (fused.enabled && fused.rq_codes != nullptr), "%s: no output requested", op);
  if (fused.enabled) {
    CK_REQUIRE(fused.activation == CK_ACT_NONE || fused.activation == CK_ACT_GELU_TANH, "%s: unknown activation %d", op,
               fused.activation);
    if (fused.rq_codes != nullptr) {
      CK_REQUIRE(fused.rq_scales != nullptr && fused.rq_scale != nullptr, "%s: re-quantization needs scales", op);
      CK_REQUIRE(N % 64 == 0, "%s: re-quantized output needs N %% 64 == 0, got %lld", op, (long long)N);
      CK_REQUIRE(reinterpret_cast<uintptr_t>(fused.rq_codes) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(fused.rq_scales) % 4 == 0,
                 "%s: re-quantized outputs must be 16-byte (codes) and 4-byte (scales) aligned", op);
    }
  }
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
  p.activation = fused.activation;
  p.rq_codes = static_cast<uint8_t*>(fused.rq_codes);
  p.rq_scales = static_cast<uint8_t*>(fused.rq_scales);
  p.rq_scale = fused.rq_scale;
  p.n_row_blocks_a = static_cast<int>(ceil_div(M, 128));
  p.n_row_blocks_b = static_cast<int>(ceil_div(N, 128));
  p.splits = 1;
  p.k_stages_per_split = static_cast<int>(ceil_div(p.k_bytes, kStageKBytes));
  if (int rc = gemm_status_word(&p.status)) return rc;
  const Operands ops = {a, b};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  OutputSpec os;
  void* const single[1] = {out};
  if (out_spec != nullptr) {
    os = *out_spec;
    CK_REQUIRE(!fused.enabled, "%s: the fused epilogue has one plain output", op);
    CK_REQUIRE(os.n >= 1 && os.n <= kMaxOutputs && os.ptrs != nullptr, "%s: 1..%d output buffers", op, kMaxOutputs);
    CK_REQUIRE(os.col_offset >= 0 && os.col_offset + N <= os.pitch, "%s: columns [%lld, %lld) outside a pitch of %lld", op,
               (long long)os.col_offset, (long long)(os.col_offset + N), (long long)os.pitch);
  } else {
    os.ptrs = single;
    os.n = 1;
    os.pitch = N;
    os.col_offset = 0;
  }
  // Few activation rows: the weight-streaming path (operands swapped, K split over all SMs).
  // CK_GEMM_CONFIG=9 forces it, any other forced configuration keeps it off.
  if (!fused.enabled && out_spec == nullptr && small_m_applies(M, N, K) && (forced_config() == 0 || forced_config() == 9)) {
    return scaled_mm_small_m(KIND == Kind::kMxfp8, a, b, sfa, sfb, tsa, tsb, alpha, bias, bias_dtype, out, out_dtype, M, N, K,
                             workspace, workspace_bytes, s);
  }
  // Split-K for problems with few tiles and a long K (small M): the tiles' K ranges are spread
  // over otherwise idle SMs as separate work items that store raw fp32 partial tiles to the
  // caller's workspace; a second kernel adds them in a fixed order and applies alpha and bias.
  if (workspace != nullptr && !fused.enabled && out_spec == nullptr && forced_config() == 0) {
    const SplitPlan plan = plan_splits(M, N, p.k_bytes);
    const int64_t need = kWorkspaceTicketBytes + static_cast<int64_t>(plan.splits) * M * N * 4;
    if (plan.splits > 1 && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 16 == 0 && (N * 4) % 16 == 0) {
      workspace = static_cast<uint8_t*>(workspace) + kWorkspaceTicketBytes;  // the counters of the small-M path stay untouched
      GemmParams ps = p;
      ps.tsa = ps.tsb = ps.alpha = nullptr;
      ps.bias = nullptr;
      ps.out = workspace;
      ps.out_dtype = CK_DTYPE_F32;
      ps.splits = plan.splits;
      ps.k_stages_per_split = plan.k_stages_per_split;
      void* parts[kMaxOutputs] = {};
      for (int i = 0; i < plan.splits; ++i) parts[i] = static_cast<uint8_t*>(workspace) + static_cast<int64_t>(i) * M * N * 4;
      OutputSpec ws_spec;
      ws_spec.ptrs = parts;
      ws_spec.n = plan.splits;
      ws_spec.pitch = N;
      ws_spec.col_offset = 0;
      if (int rc = launch_config<KIND, 128, 2, 5, 1, float, false, 1>(ops, ps, ws_spec, s)) return rc;
      return launch_splitk_reduce(static_cast<const float*>(workspace), plan.splits, M, N, p, s);
    }
  }
  if constexpr (KIND == Kind::kNvfp4) {
    if (fused.enabled) {
      switch (out_dtype) {
        case CK_DTYPE_BF16:
          return launch_for_shape<KIND, __nv_bfloat16, true>(ops, p, os, s);
        case CK_DTYPE_F16:
          return launch_for_shape<KIND, __half, true>(ops, p, os, s);
        default:
          return launch_for_shape<KIND, float, true>(ops, p, os, s);
      }
    }
  }
  switch (out_dtype) {
    case CK_DTYPE_BF16:
      return launch_for_shape<KIND, __nv_bfloat16, false>(ops, p, os, s);
    case CK_DTYPE_F16:
      return launch_for_shape<KIND, __half, false>(ops, p, os, s);
    default:
      return launch_for_shape<KIND, float, false>(ops, p, os, s);
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

extern "C" int ck_linear_nvfp4_fused(const void* a, const void* b, const void* sfa, const void* sfb,
                                     const float* tensor_scale_a, const float* tensor_scale_b, const float* alpha,
                                     const void* bias, int bias_dtype, int activation, void* out, int out_dtype,
                                     void* requant_codes, void* requant_block_scales, const float* requant_scale,
                                     int64_t M, int64_t N, int64_t K, void* stream) {
  ck::FusedArgs f;
  f.enabled = true;
  f.activation = activation;
  f.rq_codes = requant_codes;
  f.rq_scales = requant_block_scales;
  f.rq_scale = requant_scale;
  return ck::scaled_mm<ck::Kind::kNvfp4>("linear_nvfp4_fused", a, b, sfa, sfb, tensor_scale_a, tensor_scale_b, alpha, bias,
                                         bias_dtype, out, out_dtype, M, N, K, stream, f);
}

extern "C" int64_t ck_scaled_mm_workspace_bytes(int is_mxfp8, int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || M >= (1ll << 30) || N >= (1ll << 30) || K >= (1ll << 30)) return 0;
  if (ck::small_m_applies(M, N, K)) return ck::small_m_workspace_bytes(is_mxfp8 != 0, M, N, K);
  const ck::SplitPlan plan = ck::plan_splits(M, N, static_cast<int>(is_mxfp8 ? K : K / 2));
  return plan.splits > 1 ? ck::kWorkspaceTicketBytes + static_cast<int64_t>(plan.splits) * M * N * 4 : 0;
}

extern "C" int ck_scaled_mm_nvfp4_ws(const void* a, const void* b, const void* sfa, const void* sfb,
                                     const float* tensor_scale_a, const float* tensor_scale_b, const float* alpha,
                                     const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N,
                                     int64_t K, void* workspace, int64_t workspace_bytes, void* stream) {
  return ck::scaled_mm<ck::Kind::kNvfp4>("scaled_mm_nvfp4", a, b, sfa, sfb, tensor_scale_a, tensor_scale_b, alpha, bias,
                                         bias_dtype, out, out_dtype, M, N, K, stream, ck::FusedArgs(), nullptr, workspace,
                                         workspace_bytes);
}

extern "C" int ck_scaled_mm_mxfp8_ws(const void* a, const void* b, const void* sfa, const void* sfb, const void* bias,
                                     int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                                     void* workspace, int64_t workspace_bytes, void* stream) {
  return ck::scaled_mm<ck::Kind::kMxfp8>("scaled_mm_mxfp8", a, b, sfa, sfb, nullptr, nullptr, nullptr, bias, bias_dtype,
                                         out, out_dtype, M, N, K, stream, ck::FusedArgs(), nullptr, workspace,
                                         workspace_bytes);
}

extern "C" int ck_scaled_mm_nvfp4_allgather(const void* a, const void* b, const void* sfa, const void* sfb,
                                            const float* tensor_scale_a, const float* tensor_scale_b, const float* alpha,
                                            const void* bias, int bias_dtype, void* const* out_ptrs, int world,
                                            int out_dtype, int64_t M, int64_t N_local, int64_t K, int64_t n_total,
                                            int64_t col_offset, void* stream) {
  ck::OutputSpec os;
  os.ptrs = out_ptrs;
  os.n = world;
  os.pitch = n_total;
  os.col_offset = col_offset;
  CK_REQUIRE(out_ptrs != nullptr && world >= 1 && world <= ck::kMaxOutputs, "scaled_mm_nvfp4_allgather: 1..%d destinations",
             ck::kMaxOutputs);
  return ck::scaled_mm<ck::Kind::kNvfp4>("scaled_mm_nvfp4_allgather", a, b, sfa, sfb, tensor_scale_a, tensor_scale_b, alpha,
                                         bias, bias_dtype, out_ptrs[0], out_dtype, M, N_local, K, stream, ck::FusedArgs(), &os);
}

extern "C" int ck_scaled_mm_mxfp8_allgather(const void* a, const void* b, const void* sfa, const void* sfb,
                                            const void* bias, int bias_dtype, void* const* out_ptrs, int world,
                                            int out_dtype, int64_t M, int64_t N_local, int64_t K, int64_t n_total,
                                            int64_t col_offset, void* stream) {
  ck::OutputSpec os;
  os.ptrs = out_ptrs;
  os.n = world;
  os.pitch = n_total;
  os.col_offset = col_offset;
  CK_REQUIRE(out_ptrs != nullptr && world >= 1 && world <= ck::kMaxOutputs, "scaled_mm_mxfp8_allgather: 1..%d destinations",
             ck::kMaxOutputs);
  return ck::scaled_mm<ck::Kind::kMxfp8>("scaled_mm_mxfp8_allgather", a, b, sfa, sfb, nullptr, nullptr, nullptr, bias,
                                         bias_dtype, out_ptrs[0], out_dtype, M, N_local, K, stream, ck::FusedArgs(), &os);
}

#ifdef CK_GEMM_TRACE
// Copies the per-tile timeline to the host: [160 CTAs][40 tiles][16 slots] of SM cycle counts.
extern "C" __attribute__((visibility("default"))) int ck_debug_trace(long long* host_out) {
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyFromSymbol(host_out, ck::g_trace, sizeof(long long) * 160 * ck::kTraceTiles * ck::kTraceSlots));
  return CK_OK;
}
extern "C" __attribute__((visibility("default"))) int ck_debug_trace3(long long* host_out) {
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyFromSymbol(host_out, ck::g_trace3, sizeof(long long) * 8 * 160 * 8));
  return CK_OK;
}
extern "C" __attribute__((visibility("default"))) int ck_debug_trace2(long long* host_out) {
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyFromSymbol(host_out, ck::g_trace2, sizeof(long long) * 160 * 4 * 64));
  return CK_OK;
}
#endif

// Validation aid: sets the status word from the host, so that the error path of callers can be
// tested without making a kernel fail.
extern "C" int ck_debug_set_gemm_status(int value) {
  CK_CUDA(cudaDeviceSynchronize());
  CK_CUDA(cudaMemcpyToSymbol(ck::g_gemm_status, &value, sizeof(int)));
  return CK_OK;
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
