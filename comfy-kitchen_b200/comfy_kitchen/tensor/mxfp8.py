"""MXFP8 layout: E4M3 data, E8M0 (power-of-two) scales per 32 elements (tiled)."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch

import comfy_kitchen as ck
from comfy_kitchen.float_utils import roundup

from .base import BaseLayoutParams, QuantizedLayout
from .blockwise import direct_backend, install_handlers


class TensorCoreMXFP8Layout(QuantizedLayout):
    """2-D tensors only; both dimensions are zero-padded to multiples of 32.

    Same contract as the reference's comfy_kitchen/tensor/mxfp8.py:21-102: ``Params.scale``
    holds the block scales, ``state_dict_tensors`` uses the suffixes "" and "_scale", and
    ``linear``, ``mm`` / ``addmm`` with a transposed right operand and ``t`` are handled.
    """

    MIN_SM_VERSION = (10, 0)

    @dataclass(frozen=True)
    class Params(BaseLayoutParams):
        transposed: bool = False

    @classmethod
    def params_like(cls, params, **changes):
        return dataclasses.replace(params, **changes)

    @classmethod
    def quantize(cls, tensor: torch.Tensor, **kwargs):
        if tensor.dim() != 2:
            raise ValueError(f"MXFP8 requires 2D tensor, got {tensor.dim()}D")
        orig_shape = tuple(tensor.shape)
        pad = cls.get_padded_shape(orig_shape) != orig_shape
        backend = direct_backend(tensor) if tensor.is_contiguous() else None
        if backend is not None:
            qdata, block_scale = backend.quantize_mxfp8(tensor, pad_32x=pad)
        else:
            qdata, block_scale = ck.quantize_mxfp8(tensor, pad_32x=pad)
        return qdata, cls.Params(scale=block_scale, orig_dtype=tensor.dtype, orig_shape=orig_shape)

    @classmethod
    def dequantize(cls, qdata: torch.Tensor, params) -> torch.Tensor:
        return ck.dequantize_mxfp8(qdata, params.scale, params.orig_dtype)

    @classmethod
    def get_plain_tensors(cls, qtensor):
        return qtensor._qdata, qtensor._params.scale

    @classmethod
    def state_dict_tensors(cls, qdata: torch.Tensor, params) -> dict[str, torch.Tensor]:
        return {"": qdata, "_scale": params.scale}

    @classmethod
    def get_padded_shape(cls, orig_shape):
        if len(orig_shape) != 2:
            raise ValueError(f"MXFP8 requires 2D shape, got {len(orig_shape)}D")
        return (roundup(orig_shape[0], 32), roundup(orig_shape[1], 32))

    @classmethod
    def get_storage_shape(cls, orig_shape):
        return cls.get_padded_shape(orig_shape)

    @classmethod
    def get_logical_shape_from_storage(cls, storage_shape):
        return tuple(storage_shape)

    @classmethod
    def scaled_mm(cls, a, b, bias, out_dtype):
        qa, sa = cls.get_plain_tensors(a)
        qb, sb = cls.get_plain_tensors(b)
        backend = direct_backend(qa, qb, bias)
        if backend is not None:
            return backend.scaled_mm_mxfp8(qa, qb, sa, sb, bias=bias, out_dtype=out_dtype)
        return ck.scaled_mm_mxfp8(qa, qb, block_scale_a=sa, block_scale_b=sb, bias=bias, out_dtype=out_dtype)


install_handlers(TensorCoreMXFP8Layout, name="MXFP8", with_addmm=True)
