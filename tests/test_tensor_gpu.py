"""F.linear / mm / addmm interception on QuantizedTensors, on the GPU.

Mirrors the intents of the reference's tests/test_tensor.py:877-1334 and
tests/test_integration.py:63-164, with the stricter numerical bar of this build: the fast
path must match the oracle GEMM contract (1e-3 relative norm on identical quantized
operands) instead of rtol/atol 0.3.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from gpu_util import bits

from oracle import ck_oracle as oc

pytestmark = pytest.mark.gpu
LAYOUTS = ["TensorCoreNVFP4Layout", "TensorCoreMXFP8Layout"]


@pytest.fixture(scope="module")
def qt_mod(cuda_device):
    import comfy_kitchen
    from comfy_kitchen import tensor

    assert comfy_kitchen.list_backends()["cuda"]["available"]
    return tensor


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).norm() / b.float().norm())


def _oracle_linear(layout, qx, qw, bias):
    if layout == "TensorCoreNVFP4Layout":
        ref = oc.scaled_mm_nvfp4(bits(qx._qdata), bits(qw._qdata), np.float32(qx.params.scale.item()),
                                 np.float32(qw.params.scale.item()), bits(qx.params.block_scale),
                                 bits(qw.params.block_scale), bias=None if bias is None else bias.float().cpu().numpy())
    else:
        ref = oc.scaled_mm_mxfp8(bits(qx._qdata), bits(qw._qdata), bits(qx.params.scale), bits(qw.params.scale),
                                 bias=None if bias is None else bias.float().cpu().numpy())
    return torch.from_numpy(ref)


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_fast_path(qt_mod, cuda_device, layout, with_bias, monkeypatch):
    monkeypatch.setenv("CK_STRICT", "1")  # the fast path must not silently fall back
    g = torch.Generator(device="cpu").manual_seed(11)
    x = torch.randn(256, 512, generator=g).bfloat16().to(cuda_device)
    w = (torch.randn(384, 512, generator=g) * 0.02).bfloat16().to(cuda_device)
    b = (torch.randn(384, generator=g) * 0.01).bfloat16().to(cuda_device) if with_bias else None
    qx = qt_mod.QuantizedTensor.from_float(x, layout)
    qw = qt_mod.QuantizedTensor.from_float(w, layout)
    # aten.linear reaches the subclass un-decomposed under inference mode (how inference
    # frameworks call it); in grad mode PyTorch splits it into t + mm / addmm first
    with torch.inference_mode():
        y = F.linear(qx, qw, b)
    assert not isinstance(y, qt_mod.QuantizedTensor) and y.dtype == torch.bfloat16 and tuple(y.shape) == (256, 384)
    ref = _oracle_linear(layout, qx, qw, b).to(torch.bfloat16)
    assert _rel(y.cpu(), ref) <= 1e-3
    if b is None or layout == "TensorCoreMXFP8Layout":
        assert torch.equal(F.linear(qx, qw, b), y)  # the decomposed form hits the same kernel
    # and it is a faithful quantized linear: close to the dense result on the dequantized operands
    dense = F.linear(qx.dequantize(), qw.dequantize(), b)
    assert _rel(y, dense) < 2e-2


@pytest.mark.parametrize("layout", LAYOUTS)
def test_padded_shapes(qt_mod, cuda_device, layout, monkeypatch):
    # reference tests/test_tensor.py:919-939: 49 x 81 input, 113 x 81 weight
    monkeypatch.setenv("CK_STRICT", "1")
    g = torch.Generator(device="cpu").manual_seed(12)
    x = torch.randn(49, 81, generator=g).bfloat16().to(cuda_device)
    w = torch.randn(113, 81, generator=g).bfloat16().to(cuda_device)
    qx = qt_mod.QuantizedTensor.from_float(x, layout)
    qw = qt_mod.QuantizedTensor.from_float(w, layout)
    assert qx.is_padded and tuple(qx.shape) == (49, 81)
    y = F.linear(qx, qw)
    assert tuple(y.shape) == (49, 113)
    dense = F.linear(qx.dequantize(), qw.dequantize())
    assert tuple(qx.dequantize().shape) == (49, 81)
    assert _rel(y, dense) < 2e-2


@pytest.mark.parametrize("layout", LAYOUTS)
def test_fallbacks_equal_dense_on_dequantized(qt_mod, cuda_device, layout):
    # reference tests/test_tensor.py:941-986: one-sided quantization and untransposed mm fall back exactly
    g = torch.Generator(device="cpu").manual_seed(13)
    x = torch.randn(64, 128, generator=g).bfloat16().to(cuda_device)
    w = torch.randn(96, 128, generator=g).bfloat16().to(cuda_device)
    qw = qt_mod.QuantizedTensor.from_float(w, layout)
    assert torch.equal(F.linear(x, qw), F.linear(x, qw.dequantize()))
    qx = qt_mod.QuantizedTensor.from_float(x, layout)
    w2 = torch.randn(128, 96, generator=g).bfloat16().to(cuda_device)
    qw2 = qt_mod.QuantizedTensor.from_float(w2, layout)
    assert torch.equal(torch.mm(qx, qw2), torch.mm(qx.dequantize(), qw2.dequantize()))
    # shape ops dequantize
    assert torch.equal(qx.reshape(128, 64), qx.dequantize().reshape(128, 64))


@pytest.mark.parametrize("layout", LAYOUTS)
def test_mm_with_deferred_transpose_and_addmm(qt_mod, cuda_device, layout, monkeypatch):
    monkeypatch.setenv("CK_STRICT", "1")
    g = torch.Generator(device="cpu").manual_seed(14)
    x = torch.randn(128, 256, generator=g).bfloat16().to(cuda_device)
    w = (torch.randn(192, 256, generator=g) * 0.05).bfloat16().to(cuda_device)
    b = torch.randn(192, generator=g).bfloat16().to(cuda_device)
    qx = qt_mod.QuantizedTensor.from_float(x, layout)
    qw = qt_mod.QuantizedTensor.from_float(w, layout)
    y_lin = F.linear(qx, qw)
    y_mm = torch.mm(qx, qw.t())
    assert torch.equal(y_lin, y_mm)  # same kernel, same operands
    y_addmm = torch.addmm(b, qx, qw.t())
    with torch.inference_mode():
        y_lin_bias = F.linear(qx, qw, b)
    assert torch.equal(y_addmm, y_lin_bias)  # fused path for both layouts (reference mxfp8.py:179-208)
    # F.linear with a bias in grad mode is decomposed into t + addmm before the subclass sees it:
    # it must stay on the tensor-core path (CK_STRICT would raise on a failed fast path; the
    # dequantize fallback would give different bits)
    assert torch.equal(F.linear(qx, qw, b), y_lin_bias)
    # b without a deferred transpose is not the kernel's layout: dense fallback, exact
    # (reference tests/test_tensor.py:1010-1025)
    qwt = qt_mod.QuantizedTensor.from_float(w.t().contiguous(), layout)
    assert torch.equal(torch.addmm(b, qx, qwt), torch.addmm(b, qx.dequantize(), qwt.dequantize()))
    # dequantize of a transposed tensor
    assert torch.equal(qw.t().dequantize(), qw.dequantize().t())


@pytest.mark.parametrize("layout", LAYOUTS)
def test_device_moves_and_state_dict(qt_mod, cuda_device, layout):
    g = torch.Generator(device="cpu").manual_seed(15)
    w = torch.randn(64, 128, generator=g).bfloat16().to(cuda_device)
    qw = qt_mod.QuantizedTensor.from_float(w, layout)
    cpu = qw.to("cpu")
    assert isinstance(cpu, qt_mod.QuantizedTensor) and cpu._qdata.device.type == "cpu"
    back = cpu.to(cuda_device)
    assert torch.equal(back.dequantize(), qw.dequantize())
    sd = qw.state_dict("layer.weight")
    if layout == "TensorCoreNVFP4Layout":
        assert set(sd) == {"layer.weight", "layer.weight_scale", "layer.weight_scale_2"}
        # rebuild from the serialised tensors (pre-quantized weights)
        params = qt_mod.TensorCoreNVFP4Layout.Params(scale=sd["layer.weight_scale_2"], orig_dtype=torch.bfloat16,
                                                     orig_shape=(64, 128), block_scale=sd["layer.weight_scale"])
        rebuilt = qt_mod.QuantizedTensor(sd["layer.weight"], layout, params)
        assert torch.equal(rebuilt.dequantize(), qw.dequantize())
    else:
        assert set(sd) == {"layer.weight", "layer.weight_scale"}


def test_static_scale_model_under_cuda_graph(qt_mod, cuda_device, monkeypatch):
    """quantize(x, static scale) -> linear -> GELU -> quantize(h, static scale) -> linear, captured
    in a CUDA graph on a side stream; replays are bit-identical (reference tests/test_integration.py:63-164)."""
    monkeypatch.setenv("CK_STRICT", "1")
    L = "TensorCoreNVFP4Layout"
    g = torch.Generator(device="cpu").manual_seed(16)
    w1 = qt_mod.QuantizedTensor.from_float((torch.randn(256, 128, generator=g) * 0.05).bfloat16().to(cuda_device), L)
    w2 = qt_mod.QuantizedTensor.from_float((torch.randn(128, 256, generator=g) * 0.05).bfloat16().to(cuda_device), L)
    s_in = torch.tensor(4.0 / 2688.0, device=cuda_device)
    s_hid = torch.tensor(8.0 / 2688.0, device=cuda_device)

    def model(x):
        h = F.gelu(F.linear(qt_mod.QuantizedTensor.from_float(x, L, scale=s_in), w1), approximate="tanh")
        return F.linear(qt_mod.QuantizedTensor.from_float(h, L, scale=s_hid), w2)

    x = torch.randn(64, 128, generator=g).bfloat16().to(cuda_device)
    eager = model(x)
    side = torch.cuda.Stream()
    static_x = x.clone()
    with torch.cuda.stream(side):
        model(static_x)  # warm-up outside capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            static_y = model(static_x)
    graph.replay()
    torch.cuda.synchronize()
    first = static_y.clone()
    assert torch.equal(first, eager)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_y, first)
    static_x.copy_(x * 0.5)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_y, model(x * 0.5))


# ------------------------------------------------------------------------------------------ torch.compile
class _TwoLayerModel(torch.nn.Module):
    """quantize(x, static scale) -> linear -> GELU -> quantize(h, static scale) -> linear: the model of
    the reference's integration tests (tests/test_integration.py:14-53)."""

    def __init__(self, qt_mod, layout, device):
        super().__init__()
        g = torch.Generator(device="cpu").manual_seed(21)
        self.layout = layout
        self.qt = qt_mod
        self.w1 = qt_mod.QuantizedTensor.from_float((torch.randn(128, 64, generator=g) * 0.05).bfloat16().to(device), layout)
        self.w2 = qt_mod.QuantizedTensor.from_float((torch.randn(32, 128, generator=g) * 0.05).bfloat16().to(device), layout)
        self.b1 = (torch.randn(128, generator=g) * 0.01).bfloat16().to(device)
        self.input_scale = torch.tensor(48.0 / 2688.0, device=device)
        self.hidden_scale = torch.tensor(96.0 / 2688.0, device=device)

    def _q(self, t, scale):
        if self.layout == "TensorCoreNVFP4Layout":
            return self.qt.QuantizedTensor.from_float(t, self.layout, scale=scale)
        return self.qt.QuantizedTensor.from_float(t, self.layout)

    def forward(self, x):
        h = F.gelu(F.linear(self._q(x, self.input_scale), self.w1, self.b1))
        return F.linear(self._q(h, self.hidden_scale), self.w2)


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("compile_backend", ["aot_eager", "inductor"])
def test_torch_compile_matches_eager_and_is_deterministic(qt_mod, cuda_device, layout, compile_backend, monkeypatch):
    """torch.compile of a quantized model gives the eager-mode output (rtol/atol 1e-3) and the same
    bits on every run (reference tests/test_integration.py:169-215).  The custom ops trace through
    their fake kernels; under the compiler linear(x, w, b) arrives as t + addmm / mm."""
    monkeypatch.setenv("CK_STRICT", "1")
    torch._dynamo.reset()
    model = _TwoLayerModel(qt_mod, layout, cuda_device)
    x = torch.randn(16, 64, generator=torch.Generator(device="cpu").manual_seed(22)).bfloat16().to(cuda_device)
    with torch.no_grad():
        ref = model(x)
        compiled = torch.compile(model, backend=compile_backend)
        outs = [compiled(x).clone() for _ in range(3)]
    assert outs[0].shape == ref.shape and outs[0].dtype == ref.dtype
    torch.testing.assert_close(outs[0].float(), ref.float(), rtol=1e-3, atol=1e-3)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_mm_of_compile_decomposition_hits_kernel(qt_mod, cuda_device, monkeypatch):
    """mm(a, b.t()) - what torch.compile makes of linear(a, b) - runs the tensor-core kernel and meets
    the GEMM contract against the oracle (reference tests/test_tensor.py:988-1008, there rtol 0.3)."""
    monkeypatch.setenv("CK_STRICT", "1")
    g = torch.Generator(device="cpu").manual_seed(23)
    a = torch.randn(32, 64, generator=g).bfloat16().to(cuda_device)
    b = torch.randn(128, 64, generator=g).bfloat16().to(cuda_device)
    for layout in LAYOUTS:
        qa = qt_mod.QuantizedTensor.from_float(a, layout)
        qb = qt_mod.QuantizedTensor.from_float(b, layout)
        got = torch.mm(qa, qb.t())
        ref = _oracle_linear(layout, qa, qb, None).to(torch.bfloat16).float()
        assert _rel(got.cpu(), ref) <= 1e-3


# ------------------------------------------------------------------------------------------ error path
def test_strict_mode_reports_a_kernel_wait_that_gave_up(qt_mod, cuda_device, monkeypatch):
    """A launch returns 0 before its kernel runs; a bounded wait that gives up only sets a device
    status word.  With CK_STRICT=1 the layouts read it after the call chain and raise.  The word is
    set from the host here (no kernel is made to fail)."""
    from comfy_kitchen.backends import cuda as backend

    lib = backend.load_library()
    g = torch.Generator(device="cpu").manual_seed(24)
    x = qt_mod.QuantizedTensor.from_float(torch.randn(32, 64, generator=g).bfloat16().to(cuda_device), LAYOUTS[0])
    w = qt_mod.QuantizedTensor.from_float(torch.randn(64, 64, generator=g).bfloat16().to(cuda_device), LAYOUTS[0])
    backend.check_device_status("clean start")  # nothing pending
    assert lib.ck_debug_set_gemm_status(1) == 0
    with pytest.raises(RuntimeError, match="gave up"):
        backend.check_device_status("test")
    backend.check_device_status("cleared by the read")
    monkeypatch.setenv("CK_STRICT", "1")
    assert lib.ck_debug_set_gemm_status(1) == 0
    with pytest.raises(RuntimeError, match="gave up"), torch.inference_mode():
        F.linear(x, w)
    monkeypatch.setenv("CK_STRICT", "0")
    assert lib.ck_debug_set_gemm_status(1) == 0
    with torch.inference_mode():
        F.linear(x, w)  # not strict: the call chain does not look at the status word
    with pytest.raises(RuntimeError, match="gave up"):
        backend.check_device_status("explicit check")
