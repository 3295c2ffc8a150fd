"""torch.library custom operators of the quantized-linear path.

Operator names, schemas (dtype passed as an integer code; ``float epsilon, bool
pad_16x, bool hi_first``) and fake (meta) shape functions match the reference's
comfy_kitchen/backends/eager/quantization.py:471-730, so graphs traced against the
reference resolve against this build.  Each operator looks its implementation up in
the registry with keyword arguments, exactly as the reference does (:492-496).
"""
from __future__ import annotations

import torch

from .float_utils import roundup

# dtype codes shared with the C ABI (comfy_kitchen/backends/eager/quantization.py:31-39)
DTYPE_CODE_TO_DTYPE = {
    0: torch.float32,
    1: torch.float16,
    2: torch.bfloat16,
    5: torch.float8_e4m3fn,
    6: torch.float8_e5m2,
}
DTYPE_TO_CODE = {v: k for k, v in DTYPE_CODE_TO_DTYPE.items()}


def _impl(name: str, kwargs: dict):
    from .registry import registry

    return registry.get_implementation(name, kwargs=kwargs)(**kwargs)


@torch.library.custom_op("comfy_kitchen::quantize_nvfp4", mutates_args=())
def _op_quantize_nvfp4(x: torch.Tensor, per_tensor_scale: torch.Tensor, epsilon: float, pad_16x: bool,
                       hi_first: bool) -> tuple[torch.Tensor, torch.Tensor]:
    return _impl("quantize_nvfp4", {"x": x, "per_tensor_scale": per_tensor_scale, "epsilon": epsilon,
                                    "pad_16x": pad_16x, "hi_first": hi_first})


@_op_quantize_nvfp4.register_fake
def _(x, per_tensor_scale, epsilon, pad_16x, hi_first):
    rows, cols = x.shape
    if pad_16x:
        rows, cols = roundup(rows, 16), roundup(cols, 16)
    return (x.new_empty((rows, cols // 2), dtype=torch.uint8),
            x.new_empty((roundup(rows, 128), roundup(cols // 16, 4)), dtype=torch.float8_e4m3fn))


@torch.library.custom_op("comfy_kitchen::dequantize_nvfp4", mutates_args=())
def _op_dequantize_nvfp4(qx: torch.Tensor, per_tensor_scale: torch.Tensor, block_scales: torch.Tensor,
                         output_dtype_code: int, hi_first: bool) -> torch.Tensor:
    return _impl("dequantize_nvfp4", {"qx": qx, "per_tensor_scale": per_tensor_scale, "block_scales": block_scales,
                                      "output_type": DTYPE_CODE_TO_DTYPE[output_dtype_code], "hi_first": hi_first})


@_op_dequantize_nvfp4.register_fake
def _(qx, per_tensor_scale, block_scales, output_dtype_code, hi_first):
    rows, packed = qx.shape
    return qx.new_empty((rows, packed * 2), dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@torch.library.custom_op("comfy_kitchen::scaled_mm_nvfp4", mutates_args=())
def _op_scaled_mm_nvfp4(a: torch.Tensor, b: torch.Tensor, tensor_scale_a: torch.Tensor, tensor_scale_b: torch.Tensor,
                        block_scale_a: torch.Tensor, block_scale_b: torch.Tensor, bias: torch.Tensor | None,
                        output_dtype_code: int, alpha: torch.Tensor | None) -> torch.Tensor:
    return _impl("scaled_mm_nvfp4", {
        "a": a, "b": b, "tensor_scale_a": tensor_scale_a, "tensor_scale_b": tensor_scale_b,
        "block_scale_a": block_scale_a, "block_scale_b": block_scale_b, "bias": bias,
        "out_dtype": DTYPE_CODE_TO_DTYPE[output_dtype_code], "alpha": alpha})


@_op_scaled_mm_nvfp4.register_fake
def _(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b, bias, output_dtype_code, alpha):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@torch.library.custom_op("comfy_kitchen::quantize_mxfp8", mutates_args=())
def _op_quantize_mxfp8(x: torch.Tensor, pad_32x: bool) -> tuple[torch.Tensor, torch.Tensor]:
    return _impl("quantize_mxfp8", {"x": x, "pad_32x": pad_32x})


@_op_quantize_mxfp8.register_fake
def _(x, pad_32x):
    rows, cols = x.shape
    if pad_32x:
        rows, cols = roundup(rows, 32), roundup(cols, 32)
    return (x.new_empty((rows, cols), dtype=torch.float8_e4m3fn),
            x.new_empty((roundup(rows, 128), roundup(cols // 32, 4)), dtype=torch.float8_e8m0fnu))


@torch.library.custom_op("comfy_kitchen::dequantize_mxfp8", mutates_args=())
def _op_dequantize_mxfp8(qx: torch.Tensor, block_scales: torch.Tensor, output_dtype_code: int) -> torch.Tensor:
    return _impl("dequantize_mxfp8", {"qx": qx, "block_scales": block_scales,
                                      "output_type": DTYPE_CODE_TO_DTYPE[output_dtype_code]})


@_op_dequantize_mxfp8.register_fake
def _(qx, block_scales, output_dtype_code):
    return torch.empty_like(qx, dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@torch.library.custom_op("comfy_kitchen::scaled_mm_mxfp8", mutates_args=())
def _op_scaled_mm_mxfp8(a: torch.Tensor, b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                        bias: torch.Tensor | None, output_dtype_code: int) -> torch.Tensor:
    return _impl("scaled_mm_mxfp8", {"a": a, "b": b, "block_scale_a": block_scale_a, "block_scale_b": block_scale_b,
                                     "bias": bias, "out_dtype": DTYPE_CODE_TO_DTYPE[output_dtype_code]})


@_op_scaled_mm_mxfp8.register_fake
def _(a, b, block_scale_a, block_scale_b, bias, output_dtype_code):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])
