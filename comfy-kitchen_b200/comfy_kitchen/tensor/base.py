"""QuantizedTensor: a tensor subclass that carries quantized storage plus typed layout parameters.

Behaviour follows the reference's comfy_kitchen/tensor/base.py:40-511: the wrapper
reports the logical (unpadded) shape and the original dtype, ``__torch_dispatch__``
looks an aten op up first in a layout-agnostic table, then in a per-layout table
(walking the layout's MRO), and otherwise dequantizes its arguments and runs the dense
op.  Layouts are registered and referred to by string name so that the subclass can be
flattened for ``torch.compile``.
"""
from __future__ import annotations

import contextlib
import dataclasses
import logging
from dataclasses import dataclass
from functools import lru_cache
from typing import Any

import torch

logger = logging.getLogger(__name__)

LAYOUTS: dict[str, type] = {}


def register_layout_class(name: str, cls) -> None:
    LAYOUTS[name] = cls


def get_layout_class(name: str):
    return LAYOUTS[name]


@lru_cache(maxsize=1)
def get_cuda_capability() -> tuple[int, int] | None:
    """(major, minor) of the current CUDA device, or None without CUDA."""
    return torch.cuda.get_device_capability() if torch.cuda.is_available() else None


# --------------------------------------------------------------------------------------------
# layout parameters
# --------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class BaseLayoutParams:
    """Fields every layout has; subclasses add theirs and list tensor-valued ones in ``_tensor_fields``."""

    scale: torch.Tensor
    orig_dtype: torch.dtype
    orig_shape: tuple[int, ...]

    def __post_init__(self):
        self._validate_tensor_fields()

    def _validate_tensor_fields(self) -> None:
        """Hook for subclasses (for example to normalise the dtype of ``scale``)."""

    def _tensor_fields(self) -> list[str]:
        return ["scale"]

    def _rebuilt(self, fn) -> "BaseLayoutParams":
        values = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        for name in self._tensor_fields():
            values[name] = fn(values[name])
        return type(self)(**values)

    def to_device(self, device) -> "BaseLayoutParams":
        return self._rebuilt(lambda t: t.to(device=device))

    def clone(self) -> "BaseLayoutParams":
        return self._rebuilt(lambda t: t.clone())

    def copy_from(self, src: "BaseLayoutParams", non_blocking: bool = False) -> None:
        """In-place: tensor fields are copied into the existing storage, the rest is taken over."""
        tensor_names = set(self._tensor_fields())
        for f in dataclasses.fields(self):
            value = getattr(src, f.name)
            if f.name in tensor_names:
                getattr(self, f.name).copy_(value, non_blocking=non_blocking)
            else:
                object.__setattr__(self, f.name, value)


class QuantizedLayout:
    """Interface of a quantization layout.  ``Params`` is the layout's parameter dataclass."""

    Params: type[Any]
    MIN_SM_VERSION: tuple[int, int] | None = None  # minimum compute capability of the fast matmul

    @classmethod
    def quantize(cls, tensor: torch.Tensor, **kwargs) -> tuple[torch.Tensor, Any]:
        raise NotImplementedError

    @classmethod
    def dequantize(cls, qdata: torch.Tensor, params: Any) -> torch.Tensor:
        raise NotImplementedError

    @classmethod
    def get_plain_tensors(cls, qtensor: "QuantizedTensor") -> tuple[torch.Tensor, ...]:
        raise NotImplementedError

    @classmethod
    def state_dict_tensors(cls, qdata: torch.Tensor, params: Any) -> dict[str, torch.Tensor]:
        raise NotImplementedError

    @classmethod
    def supports_fast_matmul(cls) -> bool:
        if cls.MIN_SM_VERSION is None:
            return True
        cap = get_cuda_capability()
        return cap is not None and cap >= cls.MIN_SM_VERSION

    @classmethod
    def get_requirements(cls) -> dict[str, Any]:
        return {"layout": cls.__name__, "min_sm_version": cls.MIN_SM_VERSION,
                "current_sm_version": get_cuda_capability(), "fast_matmul_supported": cls.supports_fast_matmul()}


# --------------------------------------------------------------------------------------------
# the tensor subclass
# --------------------------------------------------------------------------------------------
class QuantizedTensor(torch.Tensor):
    """Wrapper subclass over (``_qdata``, layout name, ``_params``).

    ``shape`` / ``dtype`` are those of the tensor that was quantized; ``storage_shape`` /
    ``storage_dtype`` describe the quantized bytes (possibly padded).
    """

    @staticmethod
    def __new__(cls, qdata: torch.Tensor, layout_cls: str, params: Any):
        return torch.Tensor._make_wrapper_subclass(cls, params.orig_shape, device=qdata.device,
                                                   dtype=params.orig_dtype, requires_grad=False)

    def __init__(self, qdata: torch.Tensor, layout_cls: str, params: Any):
        assert isinstance(layout_cls, str), "layouts are referred to by their registered name"
        self._qdata = qdata
        self._layout_cls = layout_cls
        self._params = params

    def __repr__(self) -> str:  # noqa: D105
        return (f"QuantizedTensor(shape={tuple(self.shape)}, storage_shape={self.storage_shape}, "
                f"layout={self._layout_cls}, dtype={self._params.orig_dtype})")

    # ---- views of the storage --------------------------------------------------------------
    @property
    def storage_shape(self) -> tuple[int, ...]:
        return tuple(self._qdata.shape)

    @property
    def storage_dtype(self) -> torch.dtype:
        return self._qdata.dtype

    @property
    def nbytes(self) -> int:
        """Bytes of the quantized data (not of the logical dtype)."""
        return self._qdata.nbytes

    @property
    def padded_shape(self) -> tuple[int, ...]:
        layout = self.layout_cls
        to_logical = getattr(layout, "get_logical_shape_from_storage", None)
        return to_logical(self.storage_shape) if to_logical else self.storage_shape

    @property
    def is_padded(self) -> bool:
        return self._params.orig_shape != self.padded_shape

    @property
    def layout_cls(self) -> type[QuantizedLayout]:
        return get_layout_class(self._layout_cls)

    @property
    def params(self) -> Any:
        return self._params

    def data_ptr(self):
        return self._qdata.data_ptr()

    def is_pinned(self):
        return self._qdata.is_pinned()

    def storage(self):
        return self._qdata.storage()

    # ---- construction -----------------------------------------------------------------------
    @classmethod
    def from_float(cls, tensor: torch.Tensor, layout_cls: str, **kwargs) -> "QuantizedTensor":
        qdata, params = get_layout_class(layout_cls).quantize(tensor, **kwargs)
        return cls(qdata, layout_cls, params)

    def _copy_with(self, qdata: torch.Tensor | None = None, params: Any | None = None,
                   clone_params: bool = True) -> "QuantizedTensor":
        if params is None:
            params = self._params.clone() if clone_params else self._params
        return QuantizedTensor(self._qdata if qdata is None else qdata, self._layout_cls, params)

    # ---- value -----------------------------------------------------------------------------
    def dequantize(self) -> torch.Tensor:
        """Dense tensor of the logical shape (padding cut off, a deferred transpose applied)."""
        qdata = self._qdata if self._qdata.is_contiguous() else self._qdata.contiguous()
        full = self.layout_cls.dequantize(qdata, self._params)
        logical = tuple(self._params.orig_shape)
        if getattr(self._params, "transposed", False):
            physical = (logical[1], logical[0])
            if tuple(full.shape[:2]) != physical:
                full = full[: physical[0], : physical[1]]
            return full.t()
        if tuple(full.shape) != logical:
            full = full[tuple(slice(0, n) for n in logical)]
        return full

    def state_dict(self, prefix: str = "") -> dict[str, torch.Tensor]:
        return {f"{prefix}{suffix}": t for suffix, t in self.layout_cls.state_dict_tensors(self._qdata, self._params).items()}

    # ---- torch.compile flattening ----------------------------------------------------------------
    def __tensor_flatten__(self):
        names = ["_qdata"]
        tensor_fields, plain_fields = {}, {}
        for f in dataclasses.fields(self._params):
            value = getattr(self._params, f.name)
            if isinstance(value, torch.Tensor):
                attr = f"_param_{f.name}"
                object.__setattr__(self, attr, value)
                names.append(attr)
                tensor_fields[f.name] = attr
            else:
                plain_fields[f.name] = value
        return names, {"layout_cls": self._layout_cls, "params_class": type(self._params),
                       "tensor_fields": tensor_fields, "non_tensor_fields": plain_fields}

    @staticmethod
    def __tensor_unflatten__(inner_tensors, ctx, outer_size, outer_stride):
        fields = dict(ctx["non_tensor_fields"])
        fields.update({name: inner_tensors[attr] for name, attr in ctx["tensor_fields"].items()})
        return QuantizedTensor(inner_tensors["_qdata"], ctx["layout_cls"], ctx["params_class"](**fields))

    # ---- dispatch ------------------------------------------------------------------------------
    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        first = args[0] if args else None
        generic = _DISPATCH_TABLE.get(func)
        if generic is not None:
            return generic(first, args, kwargs)
        layout = _get_layout_from_args(args)
        per_layout = _LAYOUT_DISPATCH_TABLE.get(func)
        if layout is not None and per_layout:
            for klass in layout.__mro__:
                handler = per_layout.get(klass)
                if handler is not None:
                    return handler(first, args, kwargs)
        logger.debug("Unhandled op %s for %s, dequantizing", func, layout.__name__ if layout else "unknown")
        return cls._dequant_and_fallback(func, args, kwargs)

    @classmethod
    def _dequant_and_fallback(cls, func, args, kwargs):
        return func(*dequantize_args(args), **dequantize_args(kwargs))


def dequantize_args(args):
    """Replace every QuantizedTensor inside (nested) args / kwargs by its dequantized value."""
    if isinstance(args, QuantizedTensor):
        return args.dequantize()
    if isinstance(args, dict):
        return {k: dequantize_args(v) for k, v in args.items()}
    if isinstance(args, (list, tuple)):
        return type(args)(dequantize_args(a) for a in args)
    return args


# --------------------------------------------------------------------------------------------
# layout-agnostic handlers
# --------------------------------------------------------------------------------------------
def _parse_to_args(args, kwargs):
    device, dtype = kwargs.get("device"), kwargs.get("dtype")
    for a in args[1:]:
        if isinstance(a, torch.device):
            device = a
        elif isinstance(a, torch.dtype):
            dtype = a
        elif isinstance(a, str):
            with contextlib.suppress(Exception):
                device = torch.device(a)
    if isinstance(device, str):
        device = torch.device(device)
    return device, dtype


def _handle_detach(qt, args, kwargs):
    return qt._copy_with(qdata=qt._qdata.detach())


def _handle_clone(qt, args, kwargs):
    return qt._copy_with(qdata=qt._qdata.clone())


def _handle_to(qt, args, kwargs, force_copy: bool = False):
    device, dtype = _parse_to_args(args, kwargs)
    move = device is not None and device != qt._qdata.device
    retype = dtype is not None and dtype != qt._params.orig_dtype
    if not (move or retype or force_copy):
        return qt
    if move:
        qdata, params = qt._qdata.to(device=device), qt._params.to_device(device)
    else:
        qdata, params = (qt._qdata.clone() if force_copy else qt._qdata), qt._params.clone()
    if retype:
        params = dataclasses.replace(params, orig_dtype=dtype)
    return qt._copy_with(qdata=qdata, params=params, clone_params=False)


def _handle_to_copy(qt, args, kwargs):
    return _handle_to(qt, args, kwargs, force_copy=True)


def _handle_contiguous(qt, args, kwargs):
    return qt if qt._qdata.is_contiguous() else qt._copy_with(qdata=qt._qdata.contiguous())


def _handle_is_contiguous(qt, args, kwargs):
    return qt._qdata.is_contiguous()


def _handle_copy_(qt, args, kwargs):
    dst, src = args[0], args[1]
    if not isinstance(src, QuantizedTensor):
        raise TypeError(f"Cannot copy {type(src).__name__} to QuantizedTensor")
    if dst._layout_cls != src._layout_cls:
        raise TypeError(f"Layout mismatch: {dst._layout_cls} vs {src._layout_cls}")
    keep_dtype = dst._params.orig_dtype
    non_blocking = kwargs.get("non_blocking", len(args) >= 3)
    dst._qdata.copy_(src._qdata, non_blocking=non_blocking)
    dst._params.copy_from(src._params, non_blocking=non_blocking)
    dst._params = dataclasses.replace(dst._params, orig_dtype=keep_dtype)
    return dst


def _handle_empty_like(qt, args, kwargs):
    dtype = kwargs.pop("dtype", None)
    device = kwargs.get("device")
    params = qt._params.clone()
    if device is not None:
        params = params.to_device(device)
    if dtype is not None:
        params = dataclasses.replace(params, orig_dtype=dtype)
    return qt._copy_with(qdata=torch.empty_like(qt._qdata, device=device), params=params, clone_params=False)


_DISPATCH_TABLE = {
    torch.ops.aten.detach.default: _handle_detach,
    torch.ops.aten.clone.default: _handle_clone,
    torch.ops.aten._to_copy.default: _handle_to_copy,
    torch.ops.aten.to.dtype_layout: _handle_to,
    torch.ops.aten.to.dtype: _handle_to,
    torch.ops.aten.contiguous.default: _handle_contiguous,
    torch.ops.aten.is_contiguous.default: _handle_is_contiguous,
    torch.ops.aten.copy_.default: _handle_copy_,
    torch.ops.aten.empty_like.default: _handle_empty_like,
    torch.ops.aten._has_compatible_shallow_copy_type.default: lambda qt, args, kwargs: True,
}

# {aten op: {layout class: handler}}
_LAYOUT_DISPATCH_TABLE: dict[Any, dict[type, Any]] = {}


def register_layout_op(torch_op: Any, layout_cls: type):
    """Decorator: ``handler(qt, args, kwargs)`` implements ``torch_op`` for tensors of ``layout_cls``."""
    def decorator(handler):
        _LAYOUT_DISPATCH_TABLE.setdefault(torch_op, {})[layout_cls] = handler
        return handler
    return decorator


def _get_layout_from_args(args):
    for a in args:
        if isinstance(a, QuantizedTensor):
            return get_layout_class(a._layout_cls)
        if isinstance(a, (list, tuple)):
            for item in a:
                if isinstance(item, QuantizedTensor):
                    return get_layout_class(item._layout_cls)
    return None
