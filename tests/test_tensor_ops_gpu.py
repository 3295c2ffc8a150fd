"""QuantizedTensor as a tensor: construction, shapes, device / dtype moves, copies, shape ops.

The behaviours the reference pins for its wrapper subclass and the two block-scaled layouts
(tests/test_tensor.py:66-109 and :1123-1166 layouts, :111-372 wrapper, :410-455 capability queries,
:456-482 copy validation, :483-528 params, :1046-1122 and :1284-1334 shape ops), on real quantized
data.  Dequantized values are compared with the CPU oracle bit for bit instead of with allclose.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch
from gpu_util import bits

from oracle import ck_oracle as oc

pytestmark = pytest.mark.gpu
NVFP4, MXFP8 = "TensorCoreNVFP4Layout", "TensorCoreMXFP8Layout"
LAYOUTS = [NVFP4, MXFP8]
BLOCK = {NVFP4: 16, MXFP8: 32}


@pytest.fixture(scope="module")
def T(cuda_device):
    import comfy_kitchen
    from comfy_kitchen import tensor

    assert comfy_kitchen.list_backends()["cuda"]["available"]
    return tensor


def _x(cuda_device, rows=128, cols=256, scale=4.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * scale).bfloat16().to(cuda_device)


def _oracle_dequantize(layout, qt, out_dtype="float32"):
    """Values of the whole (padded) storage by the CPU oracle, computed in ``out_dtype`` as the
    reference does and returned as float32."""
    if layout == NVFP4:
        return oc.dequantize_nvfp4(bits(qt._qdata), np.float32(qt.params.scale.item()), bits(qt.params.block_scale),
                                   out_dtype=out_dtype)
    return oc.dequantize_mxfp8(bits(qt._qdata), bits(qt.params.scale), out_dtype=out_dtype)


@pytest.mark.parametrize("layout", LAYOUTS)
def test_from_float_shapes_and_round_trip(T, cuda_device, layout):
    QT = T.QuantizedTensor
    b = BLOCK[layout]
    x = _x(cuda_device)
    qt = QT.from_float(x, layout)
    assert isinstance(qt, QT) and qt.layout_cls is T.get_layout_class(layout)
    assert tuple(qt.shape) == (128, 256) and qt.padded_shape == (128, 256) and not qt.is_padded
    assert qt.storage_shape == ((128, 128) if layout == NVFP4 else (128, 256))
    dq = qt.dequantize()
    assert dq.dtype == torch.bfloat16 and tuple(dq.shape) == (128, 256)
    want = torch.from_numpy(_oracle_dequantize(layout, qt, "bfloat16")).bfloat16()
    assert torch.equal(dq.cpu(), want)
    tol = 0.5 if layout == NVFP4 else 0.1  # the formats' own error, as in the reference's round-trip tests
    assert torch.allclose(dq.float(), x.float(), rtol=tol, atol=tol)

    # unaligned: rows and columns padded to the block size, logical shape kept
    xu = _x(cuda_device, 129, 130, seed=1)
    qu = QT.from_float(xu, layout)
    pad = lambda n: (n + b - 1) // b * b  # noqa: E731
    assert tuple(qu.shape) == (129, 130) and qu.is_padded and qu.padded_shape == (pad(129), pad(130))
    assert qu.storage_shape == ((pad(129), pad(130) // 2) if layout == NVFP4 else (pad(129), pad(130)))
    du = qu.dequantize()
    assert tuple(du.shape) == (129, 130)
    full = torch.from_numpy(_oracle_dequantize(layout, qu, "bfloat16")).bfloat16()
    assert torch.equal(du.cpu(), full[:129, :130])
    lay = T.get_layout_class(layout)
    assert lay.get_padded_shape((129, 130)) == (pad(129), pad(130))
    assert lay.get_storage_shape((129, 130)) == qu.storage_shape
    with pytest.raises((ValueError, AssertionError, RuntimeError)):
        QT.from_float(torch.randn(4, 32, 64, device=cuda_device, dtype=torch.bfloat16), layout)  # 2-D only


@pytest.mark.parametrize("layout", LAYOUTS)
def test_detach_clone_contiguous_repr(T, cuda_device, layout):
    QT = T.QuantizedTensor
    qt = QT.from_float(_x(cuda_device, 64, 64), layout)
    d = qt.detach()
    assert isinstance(d, QT) and d._qdata is not qt._qdata and d._qdata.data_ptr() == qt._qdata.data_ptr()
    c = qt.clone()
    assert isinstance(c, QT) and c._qdata.data_ptr() != qt._qdata.data_ptr() and torch.equal(bytes_of(c), bytes_of(qt))
    assert qt.is_contiguous() and isinstance(qt.contiguous(), QT)
    assert qt.params is qt._params
    r = repr(qt)
    assert "QuantizedTensor" in r and layout in r and "64" in r


def bytes_of(qt):
    return qt._qdata.view(torch.uint8)


@pytest.mark.parametrize("layout", LAYOUTS)
def test_device_and_dtype_moves(T, cuda_device, layout):
    QT = T.QuantizedTensor
    qt = QT.from_float(_x(cuda_device, 64, 64, 5.0), layout)
    on_cpu = qt.to("cpu")
    assert isinstance(on_cpu, QT) and on_cpu._qdata.device.type == "cpu" and on_cpu.params.scale.device.type == "cpu"
    if layout == NVFP4:
        assert on_cpu.params.block_scale.device.type == "cpu"
    back = on_cpu.to(cuda_device)
    assert back._qdata.device.type == "cuda" and back.params.scale.device.type == "cuda"
    assert torch.equal(back.dequantize(), qt.dequantize())

    # a dtype change re-labels the logical dtype; the stored bytes are untouched
    as_f32 = qt.float()
    assert isinstance(as_f32, QT) and as_f32.params.orig_dtype == torch.float32 and qt.params.orig_dtype == torch.bfloat16
    assert torch.equal(bytes_of(as_f32), bytes_of(qt))
    assert as_f32.dequantize().dtype == torch.float32
    assert qt.half().params.orig_dtype == torch.float16
    both = qt.to("cpu", dtype=torch.float32)
    assert both._qdata.device.type == "cpu" and both.params.orig_dtype == torch.float32
    forced = qt.to(torch.float32, copy=True)
    assert forced._qdata.dtype == qt._qdata.dtype and forced._qdata.data_ptr() != qt._qdata.data_ptr()
    assert forced.params.orig_dtype == torch.float32 and torch.equal(bytes_of(forced), bytes_of(qt))
    same = qt.to(copy=True)
    assert same._qdata.data_ptr() != qt._qdata.data_ptr() and same.params.orig_dtype == qt.params.orig_dtype
    # the dequantized fp32 values are the oracle's, exactly
    want = torch.from_numpy(_oracle_dequantize(layout, qt))
    assert torch.equal(as_f32.dequantize().cpu(), want)


@pytest.mark.parametrize("layout", LAYOUTS)
def test_empty_like_and_copy(T, cuda_device, layout):
    QT = T.QuantizedTensor
    qt = QT.from_float(_x(cuda_device, 64, 64), layout)
    e = torch.empty_like(qt)
    assert isinstance(e, QT) and tuple(e.shape) == (64, 64) and e._qdata.dtype == qt._qdata.dtype
    e32 = torch.empty_like(qt, dtype=torch.float32)
    assert e32._qdata.dtype == qt._qdata.dtype and e32.params.orig_dtype == torch.float32
    ecpu = torch.empty_like(qt, device="cpu")
    assert ecpu._qdata.device.type == "cpu"
    # the allocate-then-copy pattern of weight loaders keeps the logical dtype of the destination
    r = torch.empty_like(qt, dtype=torch.float16, device=cuda_device)
    r.copy_(qt)
    assert isinstance(r, QT) and r.params.orig_dtype == torch.float16 and r.dequantize().dtype == torch.float16
    assert torch.equal(bytes_of(r), bytes_of(qt))
    assert torch.equal(r.dequantize().cpu(), torch.from_numpy(_oracle_dequantize(layout, qt, "float16")).half())
    with pytest.raises(TypeError):
        r.copy_(torch.zeros(64, 64, device=cuda_device, dtype=torch.bfloat16))
    other = MXFP8 if layout == NVFP4 else NVFP4
    with pytest.raises((TypeError, ValueError, RuntimeError)):
        r.copy_(QT.from_float(_x(cuda_device, 64, 64), other))


@pytest.mark.parametrize("layout", LAYOUTS)
def test_params_records(T, cuda_device, layout):
    qt = T.QuantizedTensor.from_float(_x(cuda_device, 64, 64), layout)
    p = qt.params
    assert isinstance(p, T.BaseLayoutParams)
    moved = p.to_device("cpu")
    cloned = p.clone()
    fields = ["scale"] + (["block_scale"] if layout == NVFP4 else [])
    for f in fields:
        assert getattr(moved, f).device.type == "cpu" and getattr(p, f).device.type == "cuda"
        assert getattr(cloned, f).data_ptr() != getattr(p, f).data_ptr()
        assert torch.equal(getattr(cloned, f).reshape(-1).view(torch.uint8), getattr(p, f).reshape(-1).view(torch.uint8))
    assert cloned.orig_dtype == p.orig_dtype and tuple(cloned.orig_shape) == tuple(p.orig_shape)


def test_capability_queries(T, cuda_device):
    cap = T.get_cuda_capability()
    assert cap is not None and cap >= (10, 0)
    for layout in LAYOUTS:
        lay = T.get_layout_class(layout)
        assert lay.MIN_SM_VERSION == (10, 0)
        req = lay.get_requirements()
        assert req["min_sm_version"] == (10, 0)
        assert isinstance(lay.supports_fast_matmul(), bool) and lay.supports_fast_matmul() == (cap >= req["min_sm_version"])


@pytest.mark.parametrize("layout", LAYOUTS)
def test_shape_ops(T, cuda_device, layout):
    """view / reshape leave the subclass (dense result of the dequantized tensor); t() is a flag."""
    QT = T.QuantizedTensor
    qt = QT.from_float(_x(cuda_device, 32, 128), layout)
    dense = qt.dequantize()
    v = qt.view(16, 256)
    assert not isinstance(v, QT) and tuple(v.shape) == (16, 256) and torch.equal(v, dense.view(16, 256))
    r = qt.reshape(64, 64)
    assert not isinstance(r, QT) and torch.equal(r, dense.reshape(64, 64))
    t = qt.t()
    assert isinstance(t, QT) and tuple(t.shape) == (128, 32) and t.params.transposed is True
    assert t._qdata.data_ptr() == qt._qdata.data_ptr()
    assert torch.equal(t.dequantize(), dense.t())
    tt = t.t()
    assert isinstance(tt, QT) and tuple(tt.shape) == (32, 128) and tt.params.transposed is False
    assert torch.equal(tt.dequantize(), dense)
