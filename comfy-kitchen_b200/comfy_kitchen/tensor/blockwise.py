"""What the two block-scaled tensor-core layouts (NVFP4, MXFP8) have in common.

Both pad a 2-D tensor to a multiple of their block granule, keep a ``transposed`` flag
instead of moving bytes on ``.t()``, and route ``linear`` / ``mm`` (and for MXFP8 ``addmm``)
to one ``scaled_mm`` kernel that computes ``a @ b_physical.T``; every other configuration
dequantizes and runs the dense op.  The handler logic of the reference
(comfy_kitchen/tensor/nvfp4.py:124-264, comfy_kitchen/tensor/mxfp8.py:105-236) is written
once here and parameterised by the layout.
"""
from __future__ import annotations

import logging
import os

import torch

from .base import QuantizedTensor, dequantize_args, register_layout_op

logger = logging.getLogger(__name__)


def strict_mode() -> bool:
    """CK_STRICT=1: a failing fast path raises instead of silently falling back to dequantization."""
    return os.environ.get("CK_STRICT", "0") == "1"


def strict_status_check(what: str) -> None:
    """Under CK_STRICT=1: read the device status words after a call chain and raise if a bounded
    wait inside a kernel gave up (a launch returns 0 long before that can be known).  Synchronises
    the device, so it is skipped while a CUDA graph is being captured."""
    if not strict_mode() or not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
        return
    from comfy_kitchen.backends import cuda as backend

    if backend.is_loaded():
        backend.check_device_status(what)


def direct_backend(*tensors):
    """The CUDA backend module when the kernels can be called without the operator dispatcher: all
    tensors on a CUDA device and nothing is being traced.  ``ck.<op>`` goes through a custom op and
    the backend registry (what ``torch.compile`` needs, and what CPU tensors need to raise the
    documented error); eager CUDA calls from the layouts skip those ~50 us of host work per call."""
    if torch.compiler.is_compiling():
        return None
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            continue
        # fake / functional / proxy tensors (what the compiler's tracing passes hand to
        # __torch_dispatch__) have no data pointer: only plain tensors may skip the dispatcher
        if (type(t) is not torch.Tensor and type(t) is not torch.nn.Parameter) or not t.is_cuda:
            return None
    from comfy_kitchen.backends import cuda as backend

    return backend if backend.is_loaded() else None


def crop(result: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Cut a padded matmul result back to the logical output shape."""
    if result.shape[0] != rows or result.shape[1] != cols:
        return result[:rows, :cols]
    return result


def _is_transposed(t) -> bool:
    return getattr(t._params, "transposed", False)


def _both_quantized_2d(a, b) -> bool:
    return isinstance(a, QuantizedTensor) and isinstance(b, QuantizedTensor) and a._qdata.dim() == 2


def quantized_linear(x: QuantizedTensor, w: QuantizedTensor, bias: torch.Tensor | None = None,
                     out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``linear(x, w, bias)`` on two quantized 2-D tensors of the same block-scaled layout, straight
    through the layout's kernel - the body of the ``aten.linear`` handler without the dispatcher, for
    callers (module ``forward``) that must reach the fast path in every grad mode: outside
    ``torch.inference_mode()`` ``F.linear`` is decomposed into ``t`` + ``addmm`` before the tensor
    subclass sees it."""
    layout = x.layout_cls
    if w.layout_cls is not layout or not _both_quantized_2d(x, w) or _is_transposed(x) or _is_transposed(w):
        return torch.nn.functional.linear(*dequantize_args((x, w, bias)))
    out_dtype = out_dtype or x._params.orig_dtype
    try:
        y = layout.scaled_mm(x, w, bias, out_dtype)
        strict_status_check(f"{layout.__name__} linear")
    except (RuntimeError, TypeError) as e:
        if strict_mode():
            raise
        logger.warning(f"{layout.__name__} linear failed: {e}, falling back to dequantization")
        return torch.nn.functional.linear(*dequantize_args((x, w, bias)))
    return crop(y, x._params.orig_shape[0], w._params.orig_shape[0])


def install_handlers(layout, *, name: str, with_addmm: bool) -> None:
    """Register the aten.t / mm / linear (/ addmm) handlers of a block-scaled layout.

    ``layout.scaled_mm(a, b, bias, out_dtype)`` runs the fused kernel on two QuantizedTensors.
    """

    def fast(dense_op, dense_args, a, b, bias, out_dtype, rows, cols, what):
        try:
            y = crop(layout.scaled_mm(a, b, bias, out_dtype), rows, cols)
            strict_status_check(f"{name} {what}")
            return y
        except (RuntimeError, TypeError) as e:
            if strict_mode():
                raise
            logger.warning(f"{name} {what} failed: {e}, falling back to dequantization")
            return dense_op(*dequantize_args(dense_args))

    @register_layout_op(torch.ops.aten.t.default, layout)
    def _transpose(qt, args, kwargs):
        # no bytes move: the logical shape is swapped and the flag flipped
        src = args[0]
        if not isinstance(src, QuantizedTensor):
            return torch.ops.aten.t.default(*args, **kwargs)
        rows, cols = src._params.orig_shape
        params = layout.params_like(src._params, orig_shape=(cols, rows), transposed=not _is_transposed(src))
        return QuantizedTensor(src._qdata, layout.__name__, params)

    @register_layout_op(torch.ops.aten.mm.default, layout)
    def _mm(qt, args, kwargs):
        # a @ b is the kernel's a @ b_physical.T exactly when b carries a deferred transpose
        # (the torch.compile decomposition linear(x, w) -> mm(x, w.t()))
        a, b = args[0], args[1]
        if not _both_quantized_2d(a, b) or _is_transposed(a) or not _is_transposed(b):
            return torch.mm(*dequantize_args(args))
        out_dtype = kwargs.get("out_dtype", a._params.orig_dtype)
        return fast(torch.mm, args, a, b, None, out_dtype, a._params.orig_shape[0], b._params.orig_shape[1], "mm")

    @register_layout_op(torch.ops.aten.linear.default, layout)
    def _linear(qt, args, kwargs):
        x, w = args[0], args[1]
        bias = args[2] if len(args) > 2 else None
        dense_args = (x, w, bias)
        if not _both_quantized_2d(x, w) or _is_transposed(x) or _is_transposed(w):
            return torch.nn.functional.linear(*dequantize_args(dense_args))
        out_dtype = kwargs.get("out_dtype", x._params.orig_dtype)
        return fast(torch.nn.functional.linear, dense_args, x, w, bias, out_dtype, x._params.orig_shape[0],
                    w._params.orig_shape[0], "scaled_mm")

    if with_addmm:
        @register_layout_op(torch.ops.aten.addmm.default, layout)
        def _addmm(qt, args, kwargs):
            bias, a, b = args[0], args[1], args[2]
            if not _both_quantized_2d(a, b) or _is_transposed(a) or not _is_transposed(b):
                return torch.addmm(*dequantize_args((bias, a, b)))
            return fast(torch.addmm, (bias, a, b), a, b, bias, a._params.orig_dtype, a._params.orig_shape[0],
                        b._params.orig_shape[1], "addmm")
