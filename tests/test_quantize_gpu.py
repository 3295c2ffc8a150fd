"""GPU parity of the sm_100a quantizers: bit-exact against the golden fixtures and the oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import golden_names, load_golden
from gpu_util import as_f32, bits, dit_activation, dit_weight, layout_scale, tensor_from_golden

from oracle import ck_oracle as oc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ck(cuda_device):
    import comfy_kitchen

    info = comfy_kitchen.list_backends()["cuda"]
    assert info["available"], f"cuda backend not loaded: {info['unavailable_reason']}"
    return comfy_kitchen


def _scale_tensor(v, device):
    return torch.tensor(float(v), dtype=torch.float32, device=device)


# ------------------------------------------------------------------------------------------ golden
@pytest.mark.parametrize("name", golden_names("nvfp4_"))
def test_nvfp4_golden(ck, cuda_device, name):
    d = load_golden(name)
    x = tensor_from_golden(d, cuda_device)
    q, s = ck.quantize_nvfp4(x, _scale_tensor(d["scale"], cuda_device), pad_16x=bool(d["pad"]), hi_first=bool(d["hi_first"]))
    assert q.dtype == torch.uint8 and s.dtype == torch.float8_e4m3fn
    assert tuple(q.shape) == d["codes"].shape and tuple(s.shape) == d["scales"].shape
    np.testing.assert_array_equal(bits(s), d["scales"])
    np.testing.assert_array_equal(bits(q), d["codes"])


@pytest.mark.parametrize("name", golden_names("mxfp8_"))
def test_mxfp8_golden(ck, cuda_device, name):
    d = load_golden(name)
    x = tensor_from_golden(d, cuda_device)
    q, s = ck.quantize_mxfp8(x, pad_32x=bool(d["pad"]))
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float8_e8m0fnu
    assert tuple(q.shape) == d["data"].shape and tuple(s.shape) == d["scales"].shape
    np.testing.assert_array_equal(bits(s), d["scales"])
    np.testing.assert_array_equal(bits(q), d["data"])


# ------------------------------------------------------------------------------------------ oracle, seeded
NVFP4_SHAPES = [(16, 16), (16, 64), (128, 64), (129, 128), (33, 65), (1, 17), (300, 272), (512, 1024), (1024, 2048),
                (256, 3072), (144, 4112)]


@pytest.mark.parametrize("shape", NVFP4_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_nvfp4_matches_oracle(ck, cuda_device, shape, dtype):
    g = torch.Generator(device="cpu").manual_seed(shape[0] * 7919 + shape[1])
    x = (torch.randn(*shape, generator=g) * 4).to(dtype)
    scale = layout_scale(x)
    pad = shape[0] % 16 != 0 or shape[1] % 16 != 0
    q, s = ck.quantize_nvfp4(x.to(cuda_device), scale.to(cuda_device), pad_16x=pad)
    rq, rs = oc.quantize_nvfp4(as_f32(x), np.float32(scale.item()), pad_16x=pad)
    np.testing.assert_array_equal(bits(s), rs)
    np.testing.assert_array_equal(bits(q), rq)


MXFP8_SHAPES = [(32, 32), (32, 128), (128, 128), (129, 130), (65, 96), (1, 33), (300, 288), (512, 1024), (1024, 2048),
                (256, 3072)]


@pytest.mark.parametrize("shape", MXFP8_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_mxfp8_matches_oracle(ck, cuda_device, shape, dtype):
    g = torch.Generator(device="cpu").manual_seed(shape[0] * 104729 + shape[1])
    x = (torch.randn(*shape, generator=g) * 4).to(dtype)
    pad = shape[0] % 32 != 0 or shape[1] % 32 != 0
    q, s = ck.quantize_mxfp8(x.to(cuda_device), pad_32x=pad)
    rq, rs = oc.quantize_mxfp8(as_f32(x), pad_32x=pad)
    np.testing.assert_array_equal(bits(s), rs)
    np.testing.assert_array_equal(bits(q), rq)


def test_nvfp4_lo_first_is_nibble_swap(ck, cuda_device):
    # reference tests/test_qdq.py:277-310
    x = dit_activation(256, 512).to(cuda_device)
    sc = layout_scale(x)
    q_default, s_default = ck.quantize_nvfp4(x, sc)
    q_hi, s_hi = ck.quantize_nvfp4(x, sc, hi_first=True)
    q_lo, s_lo = ck.quantize_nvfp4(x, sc, hi_first=False)
    assert torch.equal(q_default, q_hi) and torch.equal(s_default.view(torch.uint8), s_hi.view(torch.uint8))
    assert torch.equal(ck.swap_nibbles(q_hi), q_lo)
    assert torch.equal(s_hi.view(torch.uint8), s_lo.view(torch.uint8))


# ------------------------------------------------------------------------------------------ full size
def test_dit_projection_operands_full_size(ck, cuda_device):
    """x [4096,3072] with x20 outliers and W [3072,3072] ~N(0,0.02): both formats, bit-exact against the oracle."""
    for t in (dit_activation(4096, 3072), dit_weight(3072, 3072)):
        sc = layout_scale(t)
        q, s = ck.quantize_nvfp4(t.to(cuda_device), sc.to(cuda_device))
        rq, rs = oc.quantize_nvfp4(as_f32(t), np.float32(sc.item()))
        np.testing.assert_array_equal(bits(s), rs)
        np.testing.assert_array_equal(bits(q), rq)
        q8, s8 = ck.quantize_mxfp8(t.to(cuda_device))
        rq8, rs8 = oc.quantize_mxfp8(as_f32(t))
        np.testing.assert_array_equal(bits(s8), rs8)
        np.testing.assert_array_equal(bits(q8), rq8)


def test_fast_quotient_equals_ieee_division(ck, cuda_device):
    """The reciprocal-FMA quotient and the IEEE division kernel must agree on every byte.

    Size-independent property checked on 64 Mi elements spread over many magnitudes and
    global scales, including scales that saturate or underflow the block scale.
    """
    from comfy_kitchen.backends import cuda as backend

    lib = backend.load_library()
    g = torch.Generator(device="cuda").manual_seed(1234)
    try:
        for i, gs in enumerate([1.0, 3.1e-4, 0.0123, 7.7, 1e-6, 513.0, 2.0 ** -20, 1.0 / 3.0]):
            x = torch.randn(4096, 2048, generator=g, device=cuda_device)
            x = (x * torch.exp2(torch.randint(-12, 12, (4096, 1), generator=g, device=cuda_device).float())).bfloat16()
            if i % 2:
                x[::7, ::3] = -0.0
            sc = torch.tensor(gs if i else layout_scale(x).item(), dtype=torch.float32, device=cuda_device)
            lib.ck_debug_set_exact_division(0)
            q_fast, s_fast = ck.quantize_nvfp4(x, sc)
            lib.ck_debug_set_exact_division(1)
            q_div, s_div = ck.quantize_nvfp4(x, sc)
            assert torch.equal(s_fast.view(torch.uint8), s_div.view(torch.uint8))
            assert torch.equal(q_fast, q_div), f"fast quotient differs from IEEE division at global scale {gs}"
    finally:
        lib.ck_debug_set_exact_division(0)


def test_quotients_at_rounding_thresholds(ck, cuda_device):
    """Elements placed exactly on, and one bf16 step around, every E2M1 rounding boundary of their block."""
    thresholds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    rows = []
    for blk_scale in [1.0, 0.5, 1.5, 0.875, 20.0, 0.015625]:
        row = torch.zeros(16)
        row[0] = 6.0 * blk_scale  # fixes the block scale
        row[1:8] = thresholds * blk_scale
        row[8:15] = -thresholds * blk_scale
        rows.append(row)
    base = torch.stack(rows).bfloat16()
    nonzero = base != 0  # stepping the bits of 0.0 down would make a NaN
    up = torch.where(nonzero, (base.view(torch.int16) + 1).view(torch.bfloat16), base)
    down = torch.where(nonzero, (base.view(torch.int16) - 1).view(torch.bfloat16), base)
    x = torch.cat([base, up, down], dim=0)
    x = torch.cat([x, torch.zeros(16 - x.shape[0] % 16, 16, dtype=torch.bfloat16)], dim=0) if x.shape[0] % 16 else x
    for gs in [1.0, 1.0 / 3.0, 0.0071]:
        q, s = ck.quantize_nvfp4(x.to(cuda_device), torch.tensor(gs, device=cuda_device))
        rq, rs = oc.quantize_nvfp4(as_f32(x), np.float32(gs))
        np.testing.assert_array_equal(bits(s), rs)
        np.testing.assert_array_equal(bits(q), rq)


def test_rejects_bad_inputs(ck, cuda_device):
    x3 = torch.zeros(2, 16, 16, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(RuntimeError):  # NoCapableBackendError is a RuntimeError (reference tests/test_constraints.py:311-323)
        ck.quantize_nvfp4(x3, torch.ones((), device=cuda_device))
    with pytest.raises(RuntimeError):
        ck.quantize_nvfp4(torch.zeros(16, 16, dtype=torch.bfloat16), torch.ones(()))  # CPU tensor: no CPU fallback
    with pytest.raises(AssertionError):
        ck.quantize_nvfp4(torch.zeros(16, 24, dtype=torch.bfloat16, device=cuda_device), torch.ones((), device=cuda_device))
    with pytest.raises(AssertionError):
        ck.quantize_mxfp8(torch.zeros(32, 48, dtype=torch.bfloat16, device=cuda_device))


# ------------------------------------------------------------------------------------------ dynamic tensor scale
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 1), (16, 16), (33, 65), (256, 3072), (4096, 3072), (1000, 8193)])
def test_dynamic_tensor_scale_matches_layout_expression(ck, cuda_device, dtype, shape):
    """amax(|x|) / (448*6) in x's dtype, then float32 (reference tensor/nvfp4.py:64-69), evaluated on the CPU."""
    from comfy_kitchen.backends import cuda as backend

    g = torch.Generator(device="cpu").manual_seed(shape[0] + shape[1])
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    want = (torch.amax(x.abs()) / (448.0 * 6.0)).to(torch.float32)
    xd = x.to(cuda_device)
    for _ in range(3):  # the scratch buffer is left clean by every call
        got = backend.nvfp4_tensor_scale(xd)
        assert got.dtype == torch.float32 and got.dim() == 0
        assert got.cpu().view(torch.int32).item() == want.view(torch.int32).item()
    # a tensor whose maximum sits in the very last element, and an unaligned view
    y = torch.zeros(shape, dtype=dtype)
    y.view(-1)[-1] = -7.0
    assert backend.nvfp4_tensor_scale(y.to(cuda_device)).item() == (torch.amax(y.abs()) / 2688.0).float().item()
    if x.numel() > 3:
        sl = xd.view(-1)[1:]  # 2- or 4-byte aligned only
        want_sl = (torch.amax(x.view(-1)[1:].abs()) / 2688.0).to(torch.float32)
        assert backend.nvfp4_tensor_scale(sl).cpu().view(torch.int32).item() == want_sl.view(torch.int32).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_dynamic_tensor_scale_against_the_device_evaluation_of_the_expression(ck, cuda_device, dtype):
    """The kernel pins the IEEE division of the expression (what torch computes on the CPU).  torch's
    CUDA kernel for ``tensor / python_scalar`` multiplies by a float32 reciprocal instead, which can land
    one unit in the last place of x's dtype away: the two evaluations agree to that, and are usually
    identical."""
    from comfy_kitchen.backends import cuda as backend

    same = 0
    for seed in range(40):
        g = torch.Generator(device="cpu").manual_seed(1000 + seed)
        x = (torch.randn(64, 128, generator=g) * (0.1 + seed)).to(dtype)
        xd = x.to(cuda_device)
        got = backend.nvfp4_tensor_scale(xd)
        dev = (torch.amax(xd.abs()) / (448.0 * 6.0)).to(torch.float32)
        cpu = (torch.amax(x.abs()) / (448.0 * 6.0)).to(torch.float32)
        assert got.cpu().view(torch.int32).item() == cpu.view(torch.int32).item()
        step = torch.finfo(dtype).eps * abs(cpu.item())  # one unit in the last place of x's dtype, at most
        assert abs(got.item() - dev.item()) <= step
        same += int(got.item() == dev.item())
    assert same >= 30


def test_layout_uses_the_dynamic_scale_kernel(ck, cuda_device):
    from comfy_kitchen.tensor import QuantizedTensor

    x = dit_activation(512, 1024).to(cuda_device)
    qt = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout")
    want = layout_scale(x.cpu())
    assert qt.params.scale.cpu().view(torch.int32).item() == want.view(torch.int32).item()
    rq, rs = oc.quantize_nvfp4(as_f32(x), np.float32(want.item()))
    np.testing.assert_array_equal(bits(qt._qdata), rq)
    np.testing.assert_array_equal(bits(qt.params.block_scale), rs)
