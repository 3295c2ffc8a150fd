/*
 * C ABI of the B200 (sm_100a) quantized-linear backend.
 *
 * Every entry point is launch-only: it validates its arguments on the host,
 * enqueues kernels on the caller's stream and returns.  It never allocates or
 * frees device memory, never synchronises and never reads device data on the
 * host, so all of them may be called during CUDA-graph capture.  All pointers
 * are device pointers unless stated; all buffers are owned by the caller.
 *
 * Return value: CK_OK (0) or a CK_ERR_* code; ck_last_error() returns a
 * thread-local description of the last failure on the calling thread.
 *
 * Each declaration names the interface of the reference project
 * (kijai/comfy-kitchen, paths relative to its root) that it replaces.
 */
#ifndef CK_B200_H_
#define CK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CK_ABI_VERSION 1

#if defined(__GNUC__)
#define CK_API __attribute__((visibility("default")))
#else
#define CK_API
#endif

/* status codes */
#define CK_OK 0
#define CK_ERR_INVALID_ARGUMENT 1 /* bad pointer, shape, alignment or dtype code */
#define CK_ERR_UNSUPPORTED 2      /* valid request this build has no kernel for */
#define CK_ERR_CUDA 3             /* a CUDA runtime / driver call failed */

/* dtype codes, identical to the reference's
 * (comfy_kitchen/backends/cuda/dtype_dispatch.cuh:36-42,
 *  comfy_kitchen/backends/eager/quantization.py:31-39) */
#define CK_DTYPE_F32 0
#define CK_DTYPE_F16 1
#define CK_DTYPE_BF16 2

/* epilogue activations of the fused linear entry points */
#define CK_ACT_NONE 0
#define CK_ACT_GELU_TANH 1

/* ABI version of the loaded library (compare with CK_ABI_VERSION). */
CK_API int ck_abi_version(void);

/* Thread-local message of the last error returned on this thread ("" if none). */
CK_API const char* ck_last_error(void);

/* 1 if `device` is a compute-capability 10.x GPU these kernels can run on,
 * 0 if not, negative CK_ERR_* on a CUDA error.  Replaces the import-time
 * availability probe of comfy_kitchen/backends/cuda/__init__.py:672-691. */
CK_API int ck_device_supported(int device);

/* Validation aid with no counterpart in the reference: on != 0 makes
 * ck_quantize_nvfp4 use an IEEE division instruction sequence for every element
 * instead of the reciprocal-FMA quotient (the two are bit-identical; tests prove
 * it by comparing them).  Process-wide; returns the previous setting. */
CK_API int ck_debug_set_exact_division(int on);

/*
 * NVFP4 quantization: [orig_rows, orig_cols] f32/f16/bf16 row-major contiguous
 * input -> packed E2M1 codes uint8 [num_rows, num_cols/2] and E4M3 block
 * scales (one per 16 elements of a row) in the 128x4-tiled "swizzled" layout,
 * uint8 [roundup(num_rows,128), roundup(num_cols/16,4)], padding entries
 * written as 0.  num_rows/num_cols are the output's logical dimensions: equal
 * to orig_* or, with padding, orig_* rounded up to a multiple of 16 (the pad
 * reads as zeros).  num_cols must be a multiple of 16.  global_scale points to
 * one fp32 value in device memory.  hi_first != 0 puts the even-indexed
 * element of each pair in the high nibble.
 * Arithmetic is bit-identical to comfy_kitchen/backends/eager/quantization.py:115-160.
 * Replaces launch_quantize_nvfp4_kernel,
 * comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu:323-335.
 */
CK_API int ck_quantize_nvfp4(const void* input, int input_dtype, const float* global_scale,
                      void* codes, void* block_scales,
                      int64_t orig_rows, int64_t orig_cols,
                      int64_t num_rows, int64_t num_cols,
                      int hi_first, void* stream);

/*
 * MXFP8 quantization: same input contract -> E4M3 data uint8 [num_rows,
 * num_cols] and E8M0 block scales (one per 32 elements of a row) in the
 * swizzled layout, uint8 [roundup(num_rows,128), roundup(num_cols/32,4)].
 * num_cols must be a multiple of 32; num_rows/num_cols equal orig_* or orig_*
 * rounded up to a multiple of 32.
 * Arithmetic is bit-identical to comfy_kitchen/backends/eager/quantization.py:257-324
 * for f16/bf16 inputs.
 * Replaces launch_quantize_mxfp8_kernel,
 * comfy_kitchen/backends/cuda/ops/quantize_mxfp8.cu:148-157.
 */
CK_API int ck_quantize_mxfp8(const void* input, int input_dtype,
                      void* data, void* block_scales,
                      int64_t orig_rows, int64_t orig_cols,
                      int64_t num_rows, int64_t num_cols,
                      void* stream);

/*
 * Dynamic NVFP4 per-tensor scale: *scale_out = float32(dtype(amax(|input|)) / 2688) with the
 * division carried out in the input dtype, i.e. the expression
 * `torch.amax(x.abs()) / (448 * 6)` followed by `.to(float32)` of
 * comfy_kitchen/tensor/nvfp4.py:64-69, in one kernel instead of three.
 * `scratch` is device memory of at least ck_nvfp4_tensor_scale_scratch_bytes(num_elements)
 * bytes that must be zero before the FIRST call; every call leaves it zeroed again, so one
 * buffer can serve all calls that do not overlap on the GPU (calls that run concurrently
 * need separate buffers).
 */
CK_API int64_t ck_nvfp4_tensor_scale_scratch_bytes(int64_t num_elements);
CK_API int ck_nvfp4_tensor_scale(const void* input, int input_dtype, int64_t num_elements, float* scale_out,
                          void* scratch, int64_t scratch_bytes, void* stream);

/*
 * Same result as ck_nvfp4_tensor_scale, for callers that cannot hand in a scratch buffer
 * because they must not allocate device memory at that point: plugins that live inside a
 * host application with a fixed memory budget, or serving loops where a cudaMalloc would
 * stall every stream of the device.  This entry point has no counterpart in the reference.  It allocates
 * nothing: its scratch is a fixed array inside the library (about 32 KiB per GPU, resident
 * from the moment the library is loaded on that GPU until the process exits).
 *   - Limit: num_elements <= 134 217 728 (8192 blocks of 16384 elements); larger inputs
 *     are refused with CK_ERR_INVALID_ARGUMENT - use ck_nvfp4_tensor_scale instead.
 *   - The first call on each device looks up the array's device address (one-off set-up
 *     that may make the CUDA runtime load the library's kernels); make that first call
 *     before any stream capture starts.
 *   - All calls on one device share the array: two calls whose kernels can overlap on the
 *     GPU (different streams without an ordering between them) race and return garbage.
 */
CK_API int ck_nvfp4_tensor_scale_noalloc(const void* input, int input_dtype, int64_t num_elements,
                                  float* scale_out, void* stream);

/*
 * NVFP4 dequantization: packed codes uint8 [rows, cols/2] + swizzled E4M3 block
 * scales + one fp32 tensor scale -> [rows, cols] of out_dtype (f32/f16/bf16).
 * The arithmetic is done in the output dtype exactly as
 * comfy_kitchen/backends/eager/quantization.py:171-219 does.  cols % 16 == 0.
 * Replaces launch_dequantize_nvfp4_kernel,
 * comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu:386-435.
 */
CK_API int ck_dequantize_nvfp4(const void* codes, const float* global_scale, const void* block_scales,
                        void* out, int out_dtype, int64_t rows, int64_t cols, int hi_first, void* stream);

/*
 * MXFP8 dequantization: E4M3 bytes [rows, cols] + swizzled E8M0 block scales ->
 * [rows, cols] of out_dtype, float32 arithmetic then one cast
 * (comfy_kitchen/backends/eager/quantization.py:327-364; the reference has no
 * native kernel for this operator).  cols % 32 == 0.
 */
CK_API int ck_dequantize_mxfp8(const void* data, const void* block_scales, void* out, int out_dtype,
                        int64_t rows, int64_t cols, void* stream);

/*
 * NVFP4 GEMM with linear semantics:
 *   out[M,N] = cast( (deq(a)[M,K] . deq(b)[N,K]^T) * alpha + bias[N] )
 * a: uint8 [M, K/2], b: uint8 [N, K/2] packed E2M1 (both operands with the same
 * nibble order), sfa/sfb: E4M3 block scales in the swizzled layout with
 * roundup(M|N,128) x roundup(K/16,4) bytes.  alpha = *alpha when alpha is
 * non-null, else *tensor_scale_a * *tensor_scale_b (fp32, device memory).
 * bias: null or [N] of bias_dtype (f16/bf16/f32).  out: [M,N] row-major of
 * out_dtype (f32/f16/bf16).  K must be a multiple of 32, N a multiple of 8.
 * fp32 accumulation in tensor memory (tcgen05 block-scaled MMA).
 * Replaces launch_cublas_gemm_blockwise_fp4_kernel,
 * comfy_kitchen/backends/cuda/ops/cublas_gemm_nvfp4.cu:297-311.
 */
CK_API int ck_scaled_mm_nvfp4(const void* a, const void* b, const void* sfa, const void* sfb,
                       const float* tensor_scale_a, const float* tensor_scale_b,
                       const float* alpha,
                       const void* bias, int bias_dtype,
                       void* out, int out_dtype,
                       int64_t M, int64_t N, int64_t K, void* stream);

/*
 * NVFP4 linear with a fused epilogue for the next layer:
 *   y = round_out(deq(a).deq(b)^T * alpha + bias)          (rounded to out_dtype, as an
 *   h = round_out(act(y))                                    unfused caller would see it)
 * `out` (nullable) receives h as [M,N] of out_dtype; `requant_codes` (nullable) receives
 * quantize_nvfp4(h, *requant_scale): packed codes uint8 [M, N/2] (even element in the high
 * nibble) and E4M3 block scales in the swizzled layout, uint8 [roundup(M,128), N/16],
 * bit-identical to ck_quantize_nvfp4 applied to h.  Re-quantization needs N % 64 == 0 and a
 * static per-tensor scale in device memory (the output's amax is unknown until the GEMM
 * ends; the reference's own model example uses static scales too,
 * tests/test_integration.py:44-53, samples/nvfp4_linear.py:55-62,79).
 * activation: CK_ACT_NONE or CK_ACT_GELU_TANH.  Other arguments as ck_scaled_mm_nvfp4.
 * Fuses the sequence scaled_mm_nvfp4 -> gelu -> quantize_nvfp4 of the reference
 * (comfy_kitchen/tensor/nvfp4.py:214-264 followed by tensor/nvfp4.py:51-82).
 */
CK_API int ck_linear_nvfp4_fused(const void* a, const void* b, const void* sfa, const void* sfb,
                          const float* tensor_scale_a, const float* tensor_scale_b, const float* alpha,
                          const void* bias, int bias_dtype, int activation,
                          void* out, int out_dtype,
                          void* requant_codes, void* requant_block_scales, const float* requant_scale,
                          int64_t M, int64_t N, int64_t K, void* stream);

/*
 * NVFP4 linear on a dense activation in one call: x [M,K] (f32/f16/bf16, row-major, contiguous) is
 * quantized to NVFP4 (codes + tiled block scales, as ck_quantize_nvfp4 with hi_first = 1 writes
 * them) and multiplied with a pre-quantized weight:
 *   out[M,N] = cast( deq(quantize(x)) . deq(w)^T * (x_scale * w_scale) + bias )
 * x_scale: the activation's per-tensor scale in device memory, or NULL for the dynamic scale
 * amax(|x|)/2688 of ck_nvfp4_tensor_scale (one more kernel).  The kernels are enqueued back to
 * back on `stream` and chained with programmatic dependent launch; results are bit-identical to
 * calling ck_nvfp4_tensor_scale, ck_quantize_nvfp4 and ck_scaled_mm_nvfp4 one after the other.
 * The quantized activation is written to `workspace` (device memory, 256-byte aligned, at least
 * ck_linear_nvfp4_from_float_workspace_bytes(M, K, x_scale == NULL) bytes; 0 = this shape is not
 * supported).  The first 256 KiB of the workspace are the scale kernel's scratch: they must have
 * been zero-filled once before the first call with a dynamic scale and are left zeroed by every
 * call, whatever the shapes of the calls that share the workspace; calls that can overlap on the
 * GPU need separate workspaces.  K % 32 == 0, N % 8 == 0; with a dynamic scale M x K <= 2^30.
 * Replaces the sequence QuantizedTensor.from_float -> F.linear of the reference
 * (comfy_kitchen/tensor/nvfp4.py:51-82 followed by tensor/nvfp4.py:214-264; the caller side is
 * samples/nvfp4_linear.py:77-80).
 */
CK_API int64_t ck_linear_nvfp4_from_float_workspace_bytes(int64_t M, int64_t K, int dynamic_scale);
CK_API int ck_linear_nvfp4_from_float(const void* x, int x_dtype, const float* x_scale,
                               const void* w_codes, const void* w_block_scales, const float* w_scale,
                               const void* bias, int bias_dtype, void* out, int out_dtype,
                               int64_t M, int64_t N, int64_t K,
                               void* workspace, int64_t workspace_bytes, void* stream);

/*
 * The MXFP8 counterpart: x [M,K] is quantized to MXFP8 (E4M3 data + tiled E8M0 block scales, as
 * ck_quantize_mxfp8 writes them) into `workspace` and multiplied with a pre-quantized weight,
 *   out[M,N] = cast( deq(quantize(x)) . deq(w)^T + bias ),
 * by two kernels enqueued back to back; bit-identical to ck_quantize_mxfp8 followed by
 * ck_scaled_mm_mxfp8.  K % 32 == 0, N % 8 == 0; workspace 256-byte aligned, at least
 * ck_linear_mxfp8_from_float_workspace_bytes(M, K) bytes (0 = shape not supported), no
 * zero-fill needed.  Replaces QuantizedTensor.from_float -> F.linear of the reference's MXFP8
 * layout (comfy_kitchen/tensor/mxfp8.py:45-66 followed by tensor/mxfp8.py:211-236; caller side
 * samples/mxfp8_model_patcher.py:57-75).
 */
CK_API int64_t ck_linear_mxfp8_from_float_workspace_bytes(int64_t M, int64_t K);
CK_API int ck_linear_mxfp8_from_float(const void* x, int x_dtype, const void* w_data,
                               const void* w_block_scales, const void* bias, int bias_dtype,
                               void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                               void* workspace, int64_t workspace_bytes, void* stream);

/*
 * MXFP8 GEMM with linear semantics: out[M,N] = cast(deq(a) . deq(b)^T + bias).
 * a: E4M3 bytes [M,K], b: E4M3 bytes [N,K], sfa/sfb: E8M0 block scales in the
 * swizzled layout with roundup(M|N,128) x roundup(K/32,4) bytes.  K must be a
 * multiple of 32, N a multiple of 8.
 * Replaces the torch.nn.functional.scaled_mm call of
 * comfy_kitchen/scaled_mm_v2.py:40-53 reached from
 * comfy_kitchen/backends/eager/quantization.py:367-402 (the reference has no
 * native kernel for this operator).
 */
CK_API int ck_scaled_mm_mxfp8(const void* a, const void* b, const void* sfa, const void* sfb,
                       const void* bias, int bias_dtype,
                       void* out, int out_dtype,
                       int64_t M, int64_t N, int64_t K, void* stream);

/*
 * Variants of the two GEMMs that may use a caller-owned workspace (the reference hands its
 * cuBLASLt call a workspace the same way, comfy_kitchen/backends/cuda/__init__.py:117-124,
 * ops/cublas_gemm_nvfp4.cu:297-311).  ck_scaled_mm_workspace_bytes says how many bytes the
 * library would use for this shape: non-zero only for problems with few output tiles and a long
 * K (small M), which are then computed split-K - partial fp32 tiles in the workspace, added in a
 * fixed order (deterministic) either by a second kernel or, for at most 32 activation rows, by
 * the warp that finishes a tile last.  With a null or too small workspace the calls behave
 * exactly like ck_scaled_mm_nvfp4 / ck_scaled_mm_mxfp8.  The workspace must be 16-byte aligned,
 * must have been zero-filled once before its first use (its first 64 KiB hold arrival counters
 * that every call leaves at zero) and must not be shared by calls that can overlap.
 */
CK_API int64_t ck_scaled_mm_workspace_bytes(int is_mxfp8, int64_t M, int64_t N, int64_t K);
CK_API int ck_scaled_mm_nvfp4_ws(const void* a, const void* b, const void* block_scale_a,
                          const void* block_scale_b, const float* tensor_scale_a,
                          const float* tensor_scale_b, const float* alpha, const void* bias,
                          int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                          void* workspace, int64_t workspace_bytes, void* stream);
CK_API int ck_scaled_mm_mxfp8_ws(const void* a, const void* b, const void* block_scale_a,
                          const void* block_scale_b, const void* bias, int bias_dtype, void* out,
                          int out_dtype, int64_t M, int64_t N, int64_t K, void* workspace,
                          int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ multi-GPU (one node) */
/*
 * Column-sharded GEMM with the all-gather of the output fused into the epilogue.  No
 * counterpart in the reference, which has no multi-device code; the operand arguments are
 * those of ck_scaled_mm_nvfp4 / ck_scaled_mm_mxfp8 for this rank's shard of the weight
 * (b: [N_local, K], its own tiled scales, its slice of the bias).
 *
 * Every output tile is written to `world` destinations: out_ptrs[d] (HOST array of device
 * pointers) is the full row-major [M, n_total] result buffer of rank d, mapped into this
 * process (peer memory); the tile lands at columns [col_offset, col_offset + N_local).  The
 * stores are plain (non-multicast) bulk tensor stores, so the transfer over NVLink overlaps
 * the tensor-core work tile by tile.  Buffers, n_total and col_offset must keep 16-byte
 * alignment (col_offset and n_total multiples of 8 for 16-bit outputs).
 *
 * The call only launches.  The results are complete on every rank once each rank has run
 * ck_peer_barrier behind its GEMM on the same stream.
 */
CK_API int ck_scaled_mm_nvfp4_allgather(const void* a, const void* b, const void* block_scale_a,
                                 const void* block_scale_b, const float* tensor_scale_a,
                                 const float* tensor_scale_b, const float* alpha, const void* bias,
                                 int bias_dtype, void* const* out_ptrs, int world, int out_dtype,
                                 int64_t M, int64_t N_local, int64_t K, int64_t n_total,
                                 int64_t col_offset, void* stream);
CK_API int ck_scaled_mm_mxfp8_allgather(const void* a, const void* b, const void* block_scale_a,
                                 const void* block_scale_b, const void* bias, int bias_dtype,
                                 void* const* out_ptrs, int world, int out_dtype, int64_t M,
                                 int64_t N_local, int64_t K, int64_t n_total, int64_t col_offset,
                                 void* stream);

/*
 * Barrier between the GPUs of one node over peer-mapped flags.  flag_ptrs[r] (HOST array of
 * device pointers) is rank r's array of `world` 32-bit flags, zero before the first use and
 * mapped into every process.  `epoch` must grow by one per barrier (all ranks pass the same
 * value).  The kernel orders this rank's earlier stores on the stream (peer stores included)
 * before its signal, and returns when every rank has signalled this epoch - or after about a
 * second, in which case it records the missing rank (ck_peer_status) instead of hanging.
 * Each rank launches it on its own GPU.  No counterpart in the reference.
 */
CK_API int ck_peer_barrier(void* const* flag_ptrs, int rank, int world, uint32_t epoch, void* stream);

/* The same barrier with the caller's bound on the wait: max_polls polls of about 0.5 us each
 * (ck_peer_barrier uses 2^20, about a second; at most 2^26).  For the first barrier after
 * start-up, where ranks can be seconds apart (module loading, first-call set-up), a larger
 * bound keeps a slow rank from being reported as missing.  The results of a GEMM with a fused
 * all-gather are valid only if ck_peer_status reports 0 afterwards. */
CK_API int ck_peer_barrier_bounded(void* const* flag_ptrs, int rank, int world, uint32_t epoch,
                            uint32_t max_polls, void* stream);

/* Synchronises the current device and reports (then clears) the barrier status word:
 * 0 = every barrier completed, 1 + r = rank r did not arrive in time.  Host pointer. */
CK_API int ck_peer_status(int* status_out);

/*
 * Device status word of the GEMM kernels.  Every wait inside them is bounded; a
 * wait that gives up sets the word instead of hanging.  The launching call has
 * returned CK_OK long before: a return code of 0 says the launch was accepted, not
 * that every wait completed, so callers that need that guarantee read this word
 * (the Python package does after each call chain when CK_STRICT=1).  This call synchronises
 * the current device, writes the word to *status_out (0 = all launches since the
 * last call completed their waits) and clears it.  Host pointer.  Not for use
 * during graph capture.  No counterpart in the reference (its GEMM is a cuBLASLt
 * call, comfy_kitchen/backends/cuda/ops/cublas_gemm_nvfp4.cu:256-272).
 */
CK_API int ck_gemm_status(int* status_out);

/* Validation aid with no counterpart in the reference: writes `value` into the GEMM status
 * word of the current device from the host (synchronises first), so that a caller's handling
 * of a non-zero status can be tested without making any kernel fail. */
CK_API int ck_debug_set_gemm_status(int value);

#ifdef __cplusplus
}
#endif
#endif /* CK_B200_H_ */
