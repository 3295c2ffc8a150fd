"""Quantized ``nn.Linear`` replacements, a model patcher and an offline weight quantizer.

Same behaviour as the reference's samples (samples/nvfp4_linear.py:10-82 for the NVFP4 layer
and its checkpoint keys, samples/mxfp8_model_patcher.py:20-144 for the MXFP8 layer, 3-D input
flattening and the patcher's skip rules), packaged so that a model can be switched to the
quantized-linear path without writing that glue again:

* ``NVFP4Linear`` keeps its weight only as a ``QuantizedTensor`` (packed codes + tiled block
  scales + fp32 tensor scale).  Checkpoint keys: ``weight`` (uint8 codes), ``weight_scale``
  (block scales, stored as uint8 or float8_e4m3fn), ``weight_scale_2`` (tensor scale) and the
  optional ``input_scale`` (static activation scale; without it the activation scale is computed
  per call by the one-kernel amax).
* ``MXFP8Linear`` is the MXFP8 counterpart (``weight`` float8_e4m3fn / uint8, ``weight_scale``
  E8M0 bytes).
* ``NVFP4MLP`` runs ``fc2(gelu_tanh(fc1(x)))`` on two NVFP4 layers with the activation and the
  quantization of the hidden tensor fused into the first GEMM's epilogue, when the second layer
  has a static ``input_scale``.
* ``patch_model`` swaps every suitable ``nn.Linear`` of a model in place.
* ``quantize_state_dict`` turns the dense weights of a checkpoint into those keys (the offline
  quantizer; runs the library's kernels, so it needs the GPU).

Inputs with more than two dimensions are flattened to ``[tokens, features]`` for the GEMM.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .tensor import QuantizedTensor, TensorCoreMXFP8Layout, TensorCoreNVFP4Layout
from .tensor.blockwise import direct_backend, quantized_linear, strict_mode, strict_status_check

NVFP4 = "TensorCoreNVFP4Layout"
MXFP8 = "TensorCoreMXFP8Layout"


def _as_e4m3(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.float8_e4m3fn else t.view(torch.float8_e4m3fn)


def _as_e8m0(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.float8_e8m0fnu else t.view(torch.float8_e8m0fnu)


class _QuantizedLinearBase(nn.Module):
    layout_name: str = ""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.device = torch.device("cpu" if device is None else device)
        self.compute_dtype = torch.bfloat16 if dtype is None else dtype
        self.weight = None  # set by load_state_dict / from_linear
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, dtype=self.compute_dtype, device=self.device),
                                     requires_grad=False)
        else:
            self.register_parameter("bias", None)

    def _target_device(self, incoming: torch.Tensor | None = None) -> torch.device:
        """Where loaded tensors belong: next to the tensors this module holds now (it may have been
        moved since construction), else the construction device; a module that holds nothing yet and
        was built without a device follows the incoming tensor."""
        for held in (self.bias, self.weight):
            if isinstance(held, torch.Tensor):
                return held.device
        if self.device.type == "cpu" and incoming is not None and incoming.device.type != "cpu":
            return incoming.device
        return self.device

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        for held in (self.bias, self.weight):
            if isinstance(held, torch.Tensor):
                self.device = held.device
                break
        return out

    def _load_plain_entries(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs,
                            handled: set) -> None:
        """The bias (and whatever else nn.Module loads itself); ``handled`` keys are this class's own."""
        before = len(missing_keys)
        nn.Module._load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                        error_msgs)
        missing_keys[before:] = [k for k in missing_keys[before:] if k not in handled]

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, " \
               f"layout={self.layout_name}"

    def _quantize_input(self, x: torch.Tensor) -> QuantizedTensor:
        raise NotImplementedError

    def quantize_input(self, x: torch.Tensor) -> QuantizedTensor:
        """Quantize a 2-D activation the way ``forward`` would, for callers that feed the same
        activation to several layers (pass the result to each layer's ``forward``)."""
        return self._quantize_input(x if x.is_contiguous() else x.contiguous())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if isinstance(x, QuantizedTensor):
            return quantized_linear(x, self.weight, self.bias)
        shape = x.shape
        if x.dim() != 2:
            x = x.reshape(-1, shape[-1])
        if not x.is_contiguous():
            x = x.contiguous()
        y = quantized_linear(self._quantize_input(x), self.weight, self.bias)
        if len(shape) != 2:
            y = y.reshape(*shape[:-1], self.out_features)
        return y

    def state_dict(self, *args, **kwargs):
        sd = super().state_dict(*args, **kwargs)
        prefix = kwargs.get("prefix", args[1] if len(args) > 1 else "")
        key = prefix + "weight"
        if key in sd:
            del sd[key]  # the QuantizedTensor itself is not a checkpoint entry
        if self.weight is not None:
            sd.update(self.weight.state_dict(key))
        return sd


class NVFP4Linear(_QuantizedLinearBase):
    """Linear layer whose weight lives in NVFP4; activations are quantized on the fly."""

    layout_name = NVFP4

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None) -> None:
        super().__init__(in_features, out_features, bias, device, dtype)
        self.input_scale = None

    def _set_weight(self, codes: torch.Tensor, block_scale: torch.Tensor, tensor_scale: torch.Tensor) -> None:
        params = TensorCoreNVFP4Layout.Params(scale=tensor_scale.reshape(()).to(torch.float32),
                                              orig_dtype=self.compute_dtype,
                                              orig_shape=(self.out_features, self.in_features),
                                              block_scale=_as_e4m3(block_scale))
        self.weight = nn.Parameter(QuantizedTensor(codes, NVFP4, params), requires_grad=False)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        names = ["weight", "weight_scale", "weight_scale_2"]
        handled = {prefix + "weight", prefix + "input_scale"}
        absent = [n for n in names if prefix + n not in state_dict]
        if absent:
            # the quantized weight cannot be built; the bias is still loaded
            missing_keys.extend(prefix + n for n in absent)
            self._load_plain_entries(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs,
                                     handled | {prefix + n for n in names})
            return
        device = self._target_device(state_dict[prefix + "weight"])
        codes = state_dict.pop(prefix + "weight").to(device=device)
        block_scale = state_dict.pop(prefix + "weight_scale").to(device=device)
        tensor_scale = state_dict.pop(prefix + "weight_scale_2").to(device=device)
        sc_cols = (self.in_features // 16 + 3) // 4 * 4
        sc_rows = (self.out_features + 127) // 128 * 128
        if block_scale.numel() != sc_rows * sc_cols:
            error_msgs.append(f"{prefix}weight_scale has {block_scale.numel()} entries, the tiled layout of a "
                              f"[{self.out_features}, {self.in_features}] weight has {sc_rows * sc_cols}")
            return
        self._set_weight(codes.view(torch.uint8).contiguous(), block_scale.reshape(sc_rows, sc_cols).contiguous(), tensor_scale)
        input_scale = state_dict.pop(prefix + "input_scale", None)
        if input_scale is None:
            self.input_scale = None  # dynamic activation scale
        else:
            self.input_scale = nn.Parameter(input_scale.to(device=device, dtype=torch.float32).reshape(()),
                                            requires_grad=False)
        self._load_plain_entries(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs, handled)

    @classmethod
    def from_linear(cls, linear: nn.Linear, input_scale: torch.Tensor | float | None = None) -> "NVFP4Linear":
        """Quantize the weight of a dense layer (on its device, which must be the GPU)."""
        w = linear.weight.detach()
        new = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, device=w.device, dtype=w.dtype)
        q = QuantizedTensor.from_float(w.contiguous(), NVFP4)
        new.weight = nn.Parameter(q, requires_grad=False)
        if linear.bias is not None:
            new.bias = nn.Parameter(linear.bias.detach().to(w.dtype), requires_grad=False)
        if input_scale is not None:
            new.input_scale = nn.Parameter(torch.as_tensor(input_scale, dtype=torch.float32, device=w.device).reshape(()),
                                           requires_grad=False)
        return new

    def _quantize_input(self, x: torch.Tensor) -> QuantizedTensor:
        return QuantizedTensor.from_float(x, NVFP4, scale=self.input_scale)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Dense CUDA activations take the one-call path (tensor scale, quantize and GEMM enqueued by a
        single library call: a third of the host time per layer of the layout path, same bits); quantized
        inputs, traced calls and anything the call refuses take the layout path."""
        w = self.weight
        if not isinstance(x, QuantizedTensor) and w is not None and x.dim() >= 2 and x.shape[-1] % 32 == 0 and \
                x.dtype in (torch.bfloat16, torch.float16, torch.float32) and not getattr(w._params, "transposed", False):
            backend = direct_backend(x, w._qdata, self.bias, self.input_scale)
            if backend is not None:
                shape = x.shape
                x2 = x.reshape(-1, shape[-1])
                if not x2.is_contiguous():
                    x2 = x2.contiguous()
                try:
                    y = backend.linear_nvfp4_from_float(x2, w._qdata, w._params.scale, w._params.block_scale, bias=self.bias,
                                                        x_scale=self.input_scale, out_dtype=x.dtype)
                    strict_status_check("NVFP4Linear")
                    if y.shape[1] != self.out_features:  # weight rows padded to the block size
                        y = y[:, :self.out_features]
                    return y if len(shape) == 2 else y.reshape(*shape[:-1], self.out_features)
                except (RuntimeError, TypeError, AssertionError):
                    if strict_mode():
                        raise
        return super().forward(x)


class MXFP8Linear(_QuantizedLinearBase):
    """Linear layer whose weight lives in MXFP8 (E4M3 data, E8M0 scale per 32 elements)."""

    layout_name = MXFP8

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        names = ["weight", "weight_scale"]
        absent = [n for n in names if prefix + n not in state_dict]
        if absent:
            missing_keys.extend(prefix + n for n in absent)
            self._load_plain_entries(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs,
                                     {prefix + n for n in names})
            return
        device = self._target_device(state_dict[prefix + "weight"])
        data = state_dict.pop(prefix + "weight").to(device=device)
        block_scale = state_dict.pop(prefix + "weight_scale").to(device=device)
        sc_cols = (self.in_features // 32 + 3) // 4 * 4
        sc_rows = (self.out_features + 127) // 128 * 128
        if block_scale.numel() != sc_rows * sc_cols:
            error_msgs.append(f"{prefix}weight_scale has {block_scale.numel()} entries, the tiled layout of a "
                              f"[{self.out_features}, {self.in_features}] weight has {sc_rows * sc_cols}")
            return
        if data.dtype != torch.float8_e4m3fn:
            data = data.view(torch.float8_e4m3fn)
        params = TensorCoreMXFP8Layout.Params(scale=_as_e8m0(block_scale.reshape(sc_rows, sc_cols).contiguous()),
                                              orig_dtype=self.compute_dtype,
                                              orig_shape=(self.out_features, self.in_features))
        self.weight = nn.Parameter(QuantizedTensor(data.contiguous(), MXFP8, params), requires_grad=False)
        self._load_plain_entries(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs,
                                 {prefix + "weight"})

    @classmethod
    def from_linear(cls, linear: nn.Linear) -> "MXFP8Linear":
        w = linear.weight.detach()
        new = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, device=w.device, dtype=w.dtype)
        new.weight = nn.Parameter(QuantizedTensor.from_float(w.contiguous(), MXFP8), requires_grad=False)
        if linear.bias is not None:
            new.bias = nn.Parameter(linear.bias.detach().to(w.dtype), requires_grad=False)
        return new

    def _quantize_input(self, x: torch.Tensor) -> QuantizedTensor:
        return QuantizedTensor.from_float(x, MXFP8)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Dense CUDA activations take the one-call path (quantize and GEMM enqueued by a single library
        call, same bits); everything else the layout path."""
        w = self.weight
        if not isinstance(x, QuantizedTensor) and w is not None and x.dim() >= 2 and x.shape[-1] % 32 == 0 and \
                x.dtype in (torch.bfloat16, torch.float16, torch.float32) and not getattr(w._params, "transposed", False):
            backend = direct_backend(x, w._qdata, self.bias)
            if backend is not None:
                shape = x.shape
                x2 = x.reshape(-1, shape[-1])
                if not x2.is_contiguous():
                    x2 = x2.contiguous()
                try:
                    y = backend.linear_mxfp8_from_float(x2, w._qdata, w._params.scale, bias=self.bias, out_dtype=x.dtype)
                    strict_status_check("MXFP8Linear")
                    if y.shape[1] != self.out_features:  # weight rows padded to the block size
                        y = y[:, :self.out_features]
                    return y if len(shape) == 2 else y.reshape(*shape[:-1], self.out_features)
                except (RuntimeError, TypeError, AssertionError):
                    if strict_mode():
                        raise
        return super().forward(x)


class NVFP4MLP(nn.Module):
    """``fc2(gelu_tanh(fc1(x)))`` on two ``NVFP4Linear`` layers.

    When ``fc2`` carries a static ``input_scale`` (checkpoint key of the reference's layer,
    samples/nvfp4_linear.py:39-74), the first GEMM's epilogue applies the activation and quantizes the
    hidden tensor against that scale: the dense hidden tensor is never written and the separate GELU,
    tensor-scale and quantize kernels disappear.  Bit-identical to running
    ``fc1`` -> GELU -> ``quantize_nvfp4(h, input_scale)`` -> ``fc2`` one after the other.  Without
    the static scale the layers run unfused with a dynamic scale; ``calibrate`` derives a static
    scale from a sample (amax / 2688, the rule the dynamic path applies per call).
    """

    def __init__(self, fc1: NVFP4Linear, fc2: NVFP4Linear) -> None:
        super().__init__()
        if fc1.out_features != fc2.in_features:
            raise ValueError(f"fc1 produces {fc1.out_features} features, fc2 takes {fc2.in_features}")
        self.fc1 = fc1
        self.fc2 = fc2

    @torch.no_grad()
    def calibrate(self, x: torch.Tensor) -> torch.Tensor:
        """Set ``fc2.input_scale`` from the hidden tensor this input produces; returns the scale."""
        from .backends import cuda as backend
        h = torch.nn.functional.gelu(self.fc1(x), approximate="tanh")
        scale = backend.nvfp4_tensor_scale(h.reshape(-1, h.shape[-1]).contiguous()).reshape(())
        self.fc2.input_scale = nn.Parameter(scale.to(torch.float32), requires_grad=False)
        return scale

    def fusable(self) -> bool:
        return self.fc2.input_scale is not None and self.fc1.out_features % 64 == 0 and \
            self.fc1.compute_dtype in (torch.bfloat16, torch.float16)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.fusable():
            return self.fc2(torch.nn.functional.gelu(self.fc1(x), approximate="tanh"))
        from .backends import cuda as backend
        shape = None
        if isinstance(x, QuantizedTensor):
            xq = x
        else:
            shape = x.shape
            if x.dim() != 2:
                x = x.reshape(-1, shape[-1])
            xq = self.fc1.quantize_input(x)
        rows = xq._params.orig_shape[0]
        w1, w2 = self.fc1.weight, self.fc2.weight
        dtype = self.fc1.compute_dtype
        _, codes, block_scales = backend.linear_nvfp4_fused(
            xq._qdata, w1._qdata, xq._params.scale, w1._params.scale, xq._params.block_scale, w1._params.block_scale,
            bias=self.fc1.bias, activation="gelu_tanh", out_dtype=dtype, requant_scale=self.fc2.input_scale,
            return_dense=False)
        y = backend.scaled_mm_nvfp4(codes, w2._qdata, self.fc2.input_scale, w2._params.scale, block_scales,
                                    w2._params.block_scale, bias=self.fc2.bias, out_dtype=dtype)
        if y.shape[0] != rows:
            y = y[:rows]
        if shape is not None and len(shape) != 2:
            y = y.reshape(*shape[:-1], self.fc2.out_features)
        return y


_LAYERS = {"nvfp4": NVFP4Linear, "mxfp8": MXFP8Linear, NVFP4: NVFP4Linear, MXFP8: MXFP8Linear}


def patch_model(model: nn.Module, layout: str = "nvfp4", min_features: int = 64,
                skip_names: Iterable[str] | None = None) -> tuple[nn.Module, dict]:
    """Replace the ``nn.Linear`` layers of ``model`` in place by quantized ones.

    Skipped: layers whose qualified name contains one of ``skip_names``, layers with a feature
    dimension below ``min_features`` or not a multiple of the layout's block (16 / 32), and layers
    not on a CUDA device.  Returns the model and a report ``{"patched": [...], "skipped": {name: reason}}``.
    """
    layer_cls = _LAYERS[layout]
    block = 16 if layer_cls is NVFP4Linear else 32
    skip = list(skip_names or [])
    report = {"patched": [], "skipped": {}}

    def visit(module: nn.Module, prefix: str) -> None:
        for name, child in list(module.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if isinstance(child, nn.Linear):
                if any(s in full for s in skip):
                    report["skipped"][full] = "name matches a skip pattern"
                elif min(child.in_features, child.out_features) < min_features:
                    report["skipped"][full] = f"smaller than {min_features} features"
                elif child.in_features % block != 0:
                    report["skipped"][full] = f"in_features not a multiple of {block}"
                elif not child.weight.is_cuda:
                    report["skipped"][full] = "weight is not on a CUDA device"
                else:
                    setattr(module, name, layer_cls.from_linear(child))
                    report["patched"].append(full)
            else:
                visit(child, full)

    visit(model, "")
    return model, report


def quantize_state_dict(state_dict: dict, layout: str = "nvfp4", device="cuda", keys: Iterable[str] | None = None,
                        min_features: int = 64) -> dict:
    """Offline weight quantizer: returns a copy of ``state_dict`` in which every 2-D ``*.weight``
    (or the entries named by ``keys``) is replaced by the checkpoint keys of the quantized layer
    (``weight`` + ``weight_scale`` [+ ``weight_scale_2``]).  Block scales are stored as uint8."""
    layout_name = NVFP4 if _LAYERS[layout] is NVFP4Linear else MXFP8
    block = 16 if layout_name == NVFP4 else 32
    wanted = set(keys) if keys is not None else None
    out = {}
    for k, v in state_dict.items():
        take = (k in wanted) if wanted is not None else (
            k.endswith("weight") and isinstance(v, torch.Tensor) and v.dim() == 2 and v.is_floating_point() and
            min(v.shape) >= min_features and v.shape[1] % block == 0)
        if not take:
            out[k] = v
            continue
        q = QuantizedTensor.from_float(v.to(device).contiguous(), layout_name)
        for name, t in q.state_dict(k).items():
            out[name] = (t.view(torch.uint8) if t.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu) and
                         name.endswith("_scale") else t).cpu()
    return out
