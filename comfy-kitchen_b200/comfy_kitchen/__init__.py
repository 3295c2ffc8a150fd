"""comfy_kitchen operator API backed by a single sm_100a (B200) C-ABI library.

Function names, signatures, defaults and return shapes/dtypes follow the reference's
comfy_kitchen/__init__.py:118-272 and :311-366 for the quantized-linear path:
``quantize_nvfp4``, ``scaled_mm_nvfp4``, ``quantize_mxfp8``, ``scaled_mm_mxfp8`` and the
backend-configuration calls.  Every operator goes through its
``torch.ops.comfy_kitchen.*`` custom op and from there to the one registered backend;
there is no CPU implementation behind these calls.
"""
from __future__ import annotations

import torch

from . import ops as _ops  # noqa: F401  (defines torch.ops.comfy_kitchen.*)
from .backends import cuda as _cuda_backend  # noqa: F401
from .backends import eager as _eager_backend  # noqa: F401
from .backends import triton as _triton_backend  # noqa: F401
from .exceptions import BackendError, BackendNotFoundError, BackendNotImplementedError, NoCapableBackendError
from .float_utils import from_blocked, swap_nibbles, to_blocked
from .ops import DTYPE_TO_CODE
from .registry import registry

__version__ = "0.1.0"

__all__ = [
    "quantize_nvfp4",
    "dequantize_nvfp4",
    "quantize_mxfp8",
    "dequantize_mxfp8",
    "scaled_mm_nvfp4",
    "scaled_mm_mxfp8",
    "swap_nibbles",
    "to_blocked",
    "from_blocked",
    "list_backends",
    "set_backend_priority",
    "enable_backend",
    "disable_backend",
    "use_backend",
    "BackendError",
    "BackendNotFoundError",
    "BackendNotImplementedError",
    "NoCapableBackendError",
]


def quantize_nvfp4(x: torch.Tensor, per_tensor_scale: torch.Tensor, epsilon: float = 0.0, pad_16x: bool = False,
                   hi_first: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize a 2-D tensor to NVFP4.

    Returns ``(codes, block_scales)``: packed E2M1 codes ``uint8 [M', K'/2]`` and E4M3
    scales of 16-element blocks ``float8_e4m3fn [roundup(M',128), roundup(K'/16,4)]`` in
    the swizzled tensor-core layout.  With ``pad_16x`` both dimensions are zero-padded
    to multiples of 16.  ``hi_first`` puts the even-indexed element of each pair in the
    high nibble.  ``epsilon`` is unused (kept for signature compatibility).
    """
    return torch.ops.comfy_kitchen.quantize_nvfp4(x, per_tensor_scale, epsilon, pad_16x, hi_first)


def dequantize_nvfp4(qx: torch.Tensor, per_tensor_scale: torch.Tensor, block_scales: torch.Tensor,
                     output_type: torch.dtype = torch.bfloat16, hi_first: bool = True) -> torch.Tensor:
    """Inverse of :func:`quantize_nvfp4` into ``output_type`` (float32, float16 or bfloat16)."""
    return torch.ops.comfy_kitchen.dequantize_nvfp4(qx, per_tensor_scale, block_scales, DTYPE_TO_CODE[output_type],
                                                    hi_first)


def scaled_mm_nvfp4(a: torch.Tensor, b: torch.Tensor, tensor_scale_a: torch.Tensor, tensor_scale_b: torch.Tensor,
                    block_scale_a: torch.Tensor, block_scale_b: torch.Tensor, bias: torch.Tensor | None = None,
                    out_dtype: torch.dtype | None = None, alpha: torch.Tensor | None = None) -> torch.Tensor:
    """``(a @ b.T) * (tensor_scale_a * tensor_scale_b) + bias`` on NVFP4 operands; ``[M, N]`` in ``out_dtype`` (bf16 by default)."""
    if out_dtype is None:
        out_dtype = torch.bfloat16
    return torch.ops.comfy_kitchen.scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b,
                                                   bias, DTYPE_TO_CODE[out_dtype], alpha)


def quantize_mxfp8(x: torch.Tensor, pad_32x: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize a 2-D tensor to MXFP8: ``(float8_e4m3fn [M', K'], float8_e8m0fnu swizzled scales of 32-element blocks)``."""
    return torch.ops.comfy_kitchen.quantize_mxfp8(x, pad_32x)


def dequantize_mxfp8(qx: torch.Tensor, block_scales: torch.Tensor,
                     output_type: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Inverse of :func:`quantize_mxfp8` into ``output_type``."""
    return torch.ops.comfy_kitchen.dequantize_mxfp8(qx, block_scales, DTYPE_TO_CODE[output_type])


def scaled_mm_mxfp8(a: torch.Tensor, b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                    bias: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``a @ b.T + bias`` on MXFP8 operands; ``[M, N]`` in ``out_dtype`` (bf16 by default)."""
    if out_dtype is None:
        out_dtype = torch.bfloat16
    return torch.ops.comfy_kitchen.scaled_mm_mxfp8(a, b, block_scale_a, block_scale_b, bias, DTYPE_TO_CODE[out_dtype])


# ---- backend configuration (comfy_kitchen/__init__.py:311-366 of the reference) ----------------
def set_backend_priority(priority: list[str]) -> None:
    registry.set_priority(priority)


def disable_backend(name: str) -> None:
    registry.disable(name)


def enable_backend(name: str) -> None:
    registry.enable(name)


def list_backends() -> dict:
    """``{name: {"available", "disabled", "unavailable_reason", "capabilities"}}`` for ``cuda``, ``eager`` and ``triton``."""
    return registry.list_backends()


def use_backend(name: str):
    """Context manager forcing one backend for the calling thread."""
    return registry.use_backend(name)
