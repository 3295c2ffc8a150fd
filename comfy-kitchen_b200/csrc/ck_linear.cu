// One-call NVFP4 linear on a dense activation: (dynamic tensor scale ->) quantize -> GEMM.
//
// The layout path of the reference runs this as separate operator calls
// (comfy_kitchen/tensor/nvfp4.py:51-82 quantize, then :214-264 linear), each with its own
// Python dispatch.  Here the three kernels are enqueued by one C call, chained with
// programmatic dependent launch; the quantized activation lives in a caller-owned workspace
// and is still in L2 when the GEMM's loads start.
#include "ck_common.cuh"

namespace ck {
namespace {

struct FromFloatLayout {
  int64_t scratch_off, scale_off, codes_off, scales_off, total;
};

// Workspace layout: tensor-scale scratch | dynamic tensor scale | codes [M, K/2] | tiled block scales.
// The scratch comes first and has a fixed size: it must read as zero at the start of every call, and
// only a region that no other part of any shape's layout ever overlaps stays that way.
constexpr int64_t kScaleScratchBytes = 256 * 1024;  // covers 2^30 elements

FromFloatLayout from_float_layout(int64_t M, int64_t K) {
  FromFloatLayout l{};
  l.scratch_off = 0;
  l.scale_off = kScaleScratchBytes;
  l.codes_off = l.scale_off + 256;
  l.scales_off = l.codes_off + round_up(M * (K / 2), 256);
  l.total = l.scales_off + round_up(round_up(M, 128) * round_up(K / 16, 4), 256);
  return l;
}

}  // namespace
}  // namespace ck

extern "C" int64_t ck_linear_nvfp4_from_float_workspace_bytes(int64_t M, int64_t K, int dynamic_scale) {
  if (M <= 0 || K <= 0 || K % 32 != 0 || M >= (1ll << 30) || K >= (1ll << 30)) return 0;
  if (dynamic_scale != 0 && ck_nvfp4_tensor_scale_scratch_bytes(M * K) > ck::kScaleScratchBytes) return 0;
  return ck::from_float_layout(M, K).total;
}

extern "C" int ck_linear_nvfp4_from_float(const void* x, int x_dtype, const float* x_scale, const void* w_codes,
                                          const void* w_block_scales, const float* w_scale, const void* bias,
                                          int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                                          void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace ck;
  CK_REQUIRE(x && w_codes && w_block_scales && w_scale && out && workspace, "linear_nvfp4_from_float: null pointer");
  CK_REQUIRE(M > 0 && N > 0 && K > 0 && M < (1ll << 30) && K < (1ll << 30), "linear_nvfp4_from_float: bad shape");
  CK_REQUIRE(K % 32 == 0, "linear_nvfp4_from_float: K=%lld must be a multiple of 32", (long long)K);
  CK_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "linear_nvfp4_from_float: workspace must be 256-byte aligned");
  const bool dynamic = x_scale == nullptr;
  CK_REQUIRE(!dynamic || ck_nvfp4_tensor_scale_scratch_bytes(M * K) <= kScaleScratchBytes,
             "linear_nvfp4_from_float: %lld x %lld elements are too many for the dynamic scale of this entry point",
             (long long)M, (long long)K);
  const FromFloatLayout l = from_float_layout(M, K);
  CK_REQUIRE(workspace_bytes >= l.total, "linear_nvfp4_from_float: workspace of %lld bytes, %lld needed",
             (long long)workspace_bytes, (long long)l.total);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* codes = ws + l.codes_off;
  uint8_t* scales = ws + l.scales_off;
  const float* scale = x_scale;
  if (dynamic) {
    float* dyn = reinterpret_cast<float*>(ws + l.scale_off);
    if (int rc = ck_nvfp4_tensor_scale(x, x_dtype, M * K, dyn, ws + l.scratch_off, kScaleScratchBytes, stream)) return rc;
    scale = dyn;
  }
  if (int rc = ck_quantize_nvfp4(x, x_dtype, scale, codes, scales, M, K, M, K, /*hi_first=*/1, stream)) return rc;
  return ck_scaled_mm_nvfp4(codes, w_codes, scales, w_block_scales, scale, w_scale, nullptr, bias, bias_dtype, out,
                            out_dtype, M, N, K, stream);
}

// ---------------------------------------------------------------------------------------------
// MXFP8: quantize -> GEMM.  Workspace layout: data [M, K] | tiled E8M0 block scales.
// ---------------------------------------------------------------------------------------------
extern "C" int64_t ck_linear_mxfp8_from_float_workspace_bytes(int64_t M, int64_t K) {
  if (M <= 0 || K <= 0 || K % 32 != 0 || M >= (1ll << 30) || K >= (1ll << 30)) return 0;
  return ck::round_up(M * K, 256) + ck::round_up(ck::round_up(M, 128) * ck::round_up(K / 32, 4), 256);
}

extern "C" int ck_linear_mxfp8_from_float(const void* x, int x_dtype, const void* w_data, const void* w_block_scales,
                                          const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N,
                                          int64_t K, void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace ck;
  CK_REQUIRE(x && w_data && w_block_scales && out && workspace, "linear_mxfp8_from_float: null pointer");
  CK_REQUIRE(M > 0 && N > 0 && K > 0 && M < (1ll << 30) && K < (1ll << 30), "linear_mxfp8_from_float: bad shape");
  CK_REQUIRE(K % 32 == 0, "linear_mxfp8_from_float: K=%lld must be a multiple of 32", (long long)K);
  CK_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "linear_mxfp8_from_float: workspace must be 256-byte aligned");
  const int64_t need = ck_linear_mxfp8_from_float_workspace_bytes(M, K);
  CK_REQUIRE(workspace_bytes >= need, "linear_mxfp8_from_float: workspace of %lld bytes, %lld needed",
             (long long)workspace_bytes, (long long)need);
  uint8_t* data = static_cast<uint8_t*>(workspace);
  uint8_t* scales = data + round_up(M * K, 256);
  if (int rc = ck_quantize_mxfp8(x, x_dtype, data, scales, M, K, M, K, stream)) return rc;
  return ck_scaled_mm_mxfp8(data, w_data, scales, w_block_scales, bias, bias_dtype, out, out_dtype, M, N, K, stream);
}
