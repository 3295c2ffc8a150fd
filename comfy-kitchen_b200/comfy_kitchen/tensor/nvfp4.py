"""NVFP4 layout: packed E2M1 codes, E4M3 scales per 16 elements (tiled), one fp32 tensor scale."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch

import comfy_kitchen as ck
from comfy_kitchen.float_utils import F4_E2M1_MAX, F8_E4M3_MAX, roundup

from .base import BaseLayoutParams, QuantizedLayout
from .blockwise import direct_backend, install_handlers


class TensorCoreNVFP4Layout(QuantizedLayout):
    """2-D tensors only; both dimensions are zero-padded to multiples of 16.

    Same contract as the reference's comfy_kitchen/tensor/nvfp4.py:21-118: the dynamic tensor
    scale is ``amax(|x|) / (448 * 6)`` evaluated in x's dtype and then cast to float32;
    ``state_dict_tensors`` uses the key suffixes "", "_scale" (block scales) and "_scale_2"
    (tensor scale); ``linear``, ``mm`` with a transposed right operand and ``t`` are handled,
    ``addmm`` and everything else dequantize.
    """

    MIN_SM_VERSION = (10, 0)

    @dataclass(frozen=True)
    class Params(BaseLayoutParams):
        block_scale: torch.Tensor
        transposed: bool = False

        def _tensor_fields(self) -> list[str]:
            return ["scale", "block_scale"]

        def _validate_tensor_fields(self) -> None:
            if isinstance(self.scale, torch.Tensor) and self.scale.dtype != torch.float32:
                object.__setattr__(self, "scale", self.scale.to(dtype=torch.float32, non_blocking=True))

    @classmethod
    def params_like(cls, params, **changes):
        return dataclasses.replace(params, **changes)

    @classmethod
    def quantize(cls, tensor: torch.Tensor, scale=None, **kwargs):
        if tensor.dim() != 2:
            raise ValueError(f"NVFP4 requires 2D tensor, got {tensor.dim()}D")
        orig_shape = tuple(tensor.shape)
        if scale is None or (isinstance(scale, str) and scale == "recalculate"):
            fused = direct_backend(tensor) if tensor.is_contiguous() else None
            if fused is not None and tensor.dtype in (torch.bfloat16, torch.float16, torch.float32):
                scale = fused.nvfp4_tensor_scale(tensor)  # one kernel for abs, amax and the division
            else:
                scale = torch.amax(tensor.abs()) / (F8_E4M3_MAX * F4_E2M1_MAX)
        if not isinstance(scale, torch.Tensor):
            scale = torch.tensor(scale)
        scale = scale.to(device=tensor.device, dtype=torch.float32)
        pad = cls.get_padded_shape(orig_shape) != orig_shape
        backend = direct_backend(tensor) if tensor.is_contiguous() else None
        if backend is not None:
            qdata, block_scale = backend.quantize_nvfp4(tensor, scale, pad_16x=pad)
        else:
            qdata, block_scale = ck.quantize_nvfp4(tensor, scale, pad_16x=pad)
        return qdata, cls.Params(scale=scale, orig_dtype=tensor.dtype, orig_shape=orig_shape, block_scale=block_scale)

    @classmethod
    def dequantize(cls, qdata: torch.Tensor, params) -> torch.Tensor:
        return ck.dequantize_nvfp4(qdata, params.scale, params.block_scale, params.orig_dtype)

    @classmethod
    def get_plain_tensors(cls, qtensor):
        return qtensor._qdata, qtensor._params.scale, qtensor._params.block_scale

    @classmethod
    def state_dict_tensors(cls, qdata: torch.Tensor, params) -> dict[str, torch.Tensor]:
        return {"": qdata, "_scale": params.block_scale, "_scale_2": params.scale}

    @classmethod
    def get_padded_shape(cls, orig_shape):
        if len(orig_shape) != 2:
            raise ValueError(f"NVFP4 requires 2D shape, got {len(orig_shape)}D")
        return (roundup(orig_shape[0], 16), roundup(orig_shape[1], 16))

    @classmethod
    def get_storage_shape(cls, orig_shape):
        rows, cols = cls.get_padded_shape(orig_shape)
        return (rows, cols // 2)

    @classmethod
    def get_logical_shape_from_storage(cls, storage_shape):
        return (storage_shape[0], storage_shape[1] * 2)

    @classmethod
    def scaled_mm(cls, a, b, bias, out_dtype):
        qa, sa, bsa = cls.get_plain_tensors(a)
        qb, sb, bsb = cls.get_plain_tensors(b)
        backend = direct_backend(qa, qb, bias)
        if backend is not None:
            return backend.scaled_mm_nvfp4(qa, qb, sa, sb, bsa, bsb, bias=bias, out_dtype=out_dtype)
        return ck.scaled_mm_nvfp4(qa, qb, tensor_scale_a=sa, tensor_scale_b=sb, block_scale_a=bsa, block_scale_b=bsb,
                                  bias=bias, out_dtype=out_dtype)


# addmm: the reference has no NVFP4 handler (its aten.addmm falls to the dequantize path); outside
# inference mode F.linear with a bias reaches a tensor subclass as t + addmm, so without one a
# biased linear in grad mode would leave the tensor-core path.  The handler takes the fast path
# under the same condition as mm (b carries a deferred transpose) and falls back otherwise.
install_handlers(TensorCoreNVFP4Layout, name="NVFP4", with_addmm=True)
