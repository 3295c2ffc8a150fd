"""Host-side behaviour of the tensor layer that needs no GPU: shape math, wrapper metadata,
flatten / unflatten, generic aten handlers, and loud failure without a CUDA backend."""
from __future__ import annotations

import pytest
import torch

import comfy_kitchen as ck
from comfy_kitchen.tensor import (QuantizedTensor, TensorCoreMXFP8Layout, TensorCoreNVFP4Layout, get_layout_class)


def _fake_nvfp4(rows=32, cols=64, orig=None, dtype=torch.bfloat16):
    orig = orig or (rows, cols)
    qdata = torch.zeros(rows, cols // 2, dtype=torch.uint8)
    params = TensorCoreNVFP4Layout.Params(
        scale=torch.tensor(0.5, dtype=torch.float64), orig_dtype=dtype, orig_shape=orig,
        block_scale=torch.zeros(128, 4, dtype=torch.uint8).view(torch.float8_e4m3fn))
    return QuantizedTensor(qdata, "TensorCoreNVFP4Layout", params)


def test_shape_math_matches_reference_contract():
    # reference tests/test_tensor.py:78-102 and :1134-1156
    assert TensorCoreNVFP4Layout.get_padded_shape((129, 130)) == (144, 144)
    assert TensorCoreNVFP4Layout.get_storage_shape((129, 130)) == (144, 72)
    assert TensorCoreNVFP4Layout.get_logical_shape_from_storage((144, 72)) == (144, 144)
    assert TensorCoreMXFP8Layout.get_padded_shape((129, 130)) == (160, 160)
    assert TensorCoreMXFP8Layout.get_storage_shape((129, 130)) == (160, 160)
    with pytest.raises(ValueError):
        TensorCoreNVFP4Layout.get_padded_shape((2, 3, 4))
    with pytest.raises(ValueError):
        TensorCoreNVFP4Layout.quantize(torch.zeros(2, 16, 16))
    with pytest.raises(ValueError):
        TensorCoreMXFP8Layout.quantize(torch.zeros(2, 32, 32))
    assert TensorCoreNVFP4Layout.MIN_SM_VERSION == (10, 0) and TensorCoreMXFP8Layout.MIN_SM_VERSION == (10, 0)
    assert get_layout_class("TensorCoreNVFP4Layout") is TensorCoreNVFP4Layout


def test_wrapper_metadata_and_scale_normalisation():
    qt = _fake_nvfp4(144, 144, orig=(129, 130))
    assert tuple(qt.shape) == (129, 130) and qt.dtype == torch.bfloat16
    assert qt.storage_shape == (144, 72) and qt.storage_dtype == torch.uint8
    assert qt.padded_shape == (144, 144) and qt.is_padded
    assert qt.nbytes == 144 * 72
    assert qt.params.scale.dtype == torch.float32  # normalised to fp32 on construction
    assert set(qt.state_dict("w")) == {"w", "w_scale", "w_scale_2"}
    assert "TensorCoreNVFP4Layout" in repr(qt)


def test_generic_handlers_keep_the_subclass():
    qt = _fake_nvfp4()
    for other in (qt.detach(), qt.clone(), torch.empty_like(qt)):
        assert isinstance(other, QuantizedTensor) and tuple(other.shape) == tuple(qt.shape)
    assert qt.clone()._qdata.data_ptr() != qt._qdata.data_ptr()
    as_half = qt.to(torch.float16)
    assert isinstance(as_half, QuantizedTensor) and as_half.dtype == torch.float16 and qt.dtype == torch.bfloat16
    assert qt.to(torch.bfloat16) is qt
    dst = _fake_nvfp4()
    src = _fake_nvfp4()
    src._qdata.fill_(7)
    dst.copy_(src)
    assert int(dst._qdata[0, 0]) == 7
    with pytest.raises(TypeError):
        dst.copy_(torch.zeros(32, 64))


def test_transpose_is_a_flag_flip():
    # reference tests/test_tensor.py:1062-1075
    qt = _fake_nvfp4(32, 64)
    t = qt.t()
    assert isinstance(t, QuantizedTensor) and tuple(t.shape) == (64, 32)
    assert t._params.transposed and not qt._params.transposed
    assert t._qdata.data_ptr() == qt._qdata.data_ptr()
    assert not t.t()._params.transposed


def test_flatten_unflatten_round_trip():
    qt = _fake_nvfp4(144, 144, orig=(129, 130))
    names, ctx = qt.__tensor_flatten__()
    assert names[0] == "_qdata" and "_param_block_scale" in names and "_param_scale" in names
    inner = {n: getattr(qt, n) for n in names}
    back = QuantizedTensor.__tensor_unflatten__(inner, ctx, None, None)
    assert tuple(back.shape) == (129, 130) and back._layout_cls == "TensorCoreNVFP4Layout"
    assert back._params.block_scale is qt._params.block_scale


def test_no_cpu_implementation_behind_the_layouts():
    x = torch.randn(32, 64, dtype=torch.bfloat16)
    with pytest.raises(ck.NoCapableBackendError):
        QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout")
    with pytest.raises(ck.NoCapableBackendError):
        QuantizedTensor.from_float(x, "TensorCoreMXFP8Layout")
    if not torch.cuda.is_available():
        with pytest.raises(ck.NoCapableBackendError):
            _fake_nvfp4().dequantize()
