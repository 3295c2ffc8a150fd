"""Fused NVFP4 linear epilogue (activation + re-quantize for the next layer), on the GPU.

Parity contract: the re-quantized codes and scale bytes are bit-identical to
quantize_nvfp4 applied to the dense output the same kernel produces (checked against the
oracle and against the stand-alone CUDA quantizer), and the dense output matches the
unfused sequence linear -> round to bf16 -> GELU(tanh) -> round to bf16 within bf16
rounding (the tanh of the two implementations may differ in the last fp32 bit).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from gpu_util import as_f32, bits, layout_scale

from oracle import ck_oracle as oc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(cuda_device):
    import comfy_kitchen as ck
    from comfy_kitchen.backends import cuda as backend

    assert ck.list_backends()["cuda"]["available"]
    return ck, backend


def _setup(ck, dev, m, n, k, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(m, k, generator=g).bfloat16().to(dev)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(dev)
    bias = (torch.randn(n, generator=g) * 0.01).bfloat16().to(dev)
    sx, sw = layout_scale(x), layout_scale(w)
    qx, bsx = ck.quantize_nvfp4(x, sx)
    qw, bsw = ck.quantize_nvfp4(w, sw)
    return qx, bsx, sx, qw, bsw, sw, bias


@pytest.mark.parametrize("shape", [(128, 128, 256), (256, 384, 512), (200, 320, 288), (1024, 1024, 512), (4608, 1536, 256)])
@pytest.mark.parametrize("activation", [None, "gelu_tanh"])
def test_fused_requant_equals_quantizer_on_its_own_output(env, cuda_device, shape, activation, monkeypatch):
    ck, backend = env
    m, n, k = shape
    qx, bsx, sx, qw, bsw, sw, bias = _setup(ck, cuda_device, m, n, k, seed=m + n + k)
    rq_scale = torch.tensor(0.0045, device=cuda_device)
    for config in (1, 3, 4):
        monkeypatch.setenv("CK_GEMM_CONFIG", str(config))
        h, codes, scales = backend.linear_nvfp4_fused(qx, qw, sx, sw, bsx, bsw, bias=bias, activation=activation,
                                                      requant_scale=rq_scale)
        assert h.dtype == torch.bfloat16 and tuple(h.shape) == (m, n)
        assert tuple(codes.shape) == (m, n // 2) and tuple(scales.shape) == ((m + 127) // 128 * 128, n // 16)
        # 1. against the oracle quantizer on the kernel's own dense output
        rq, rs = oc.quantize_nvfp4(as_f32(h), np.float32(rq_scale.item()))
        np.testing.assert_array_equal(bits(scales), rs)
        np.testing.assert_array_equal(bits(codes), rq)
        # 2. against the stand-alone CUDA quantizer
        q2, s2 = ck.quantize_nvfp4(h, rq_scale, pad_16x=(m % 16 != 0))
        assert torch.equal(q2[:m], codes) and torch.equal(s2.view(torch.uint8), scales.view(torch.uint8))
        # 3. the dense output against the unfused sequence
        y = ck.scaled_mm_nvfp4(qx, qw, sx, sw, bsx, bsw, bias=bias, out_dtype=torch.bfloat16)
        ref = F.gelu(y, approximate="tanh") if activation else y
        if activation is None:
            assert torch.equal(h, ref)
        else:
            diff = (h.float() - ref.float()).abs()
            ulp = torch.maximum(ref.float().abs(), torch.tensor(1e-3, device=cuda_device)) * 2.0 ** -7
            assert bool((diff <= ulp).all()), "fused GELU differs from torch's by more than one bf16 step"
            assert float((diff > 0).float().mean()) < 0.01
        # requant only (no dense output) gives the same codes
        _, codes_only, scales_only = backend.linear_nvfp4_fused(qx, qw, sx, sw, bsx, bsw, bias=bias, activation=activation,
                                                                requant_scale=rq_scale, return_dense=False)
        assert torch.equal(codes_only, codes) and torch.equal(scales_only.view(torch.uint8), scales.view(torch.uint8))


def test_mlp_pair_fused_matches_unfused(env, cuda_device):
    """fc1 -> GELU -> re-quantize (fused) -> fc2 equals the unfused chain that quantizes the dense hidden."""
    ck, backend = env
    dev = cuda_device
    g = torch.Generator(device="cpu").manual_seed(3)
    m, d, hdim = 512, 256, 1024
    x = torch.randn(m, d, generator=g).bfloat16().to(dev)
    w1 = (torch.randn(hdim, d, generator=g) * 0.05).bfloat16().to(dev)
    w2 = (torch.randn(d, hdim, generator=g) * 0.02).bfloat16().to(dev)
    sx, s1, s2 = layout_scale(x), layout_scale(w1), layout_scale(w2)
    qx, bsx = ck.quantize_nvfp4(x, sx)
    q1, b1 = ck.quantize_nvfp4(w1, s1)
    q2, b2 = ck.quantize_nvfp4(w2, s2)
    h_scale = torch.tensor(0.004, device=dev)
    h, hc, hs = backend.linear_nvfp4_fused(qx, q1, sx, s1, bsx, b1, activation="gelu_tanh", requant_scale=h_scale)
    y_fused = ck.scaled_mm_nvfp4(hc, q2, h_scale, s2, hs, b2)
    hq, hqs = ck.quantize_nvfp4(h, h_scale)
    y_unfused = ck.scaled_mm_nvfp4(hq, q2, h_scale, s2, hqs, b2)
    assert torch.equal(y_fused, y_unfused)


def test_rejects_bad_requests(env, cuda_device):
    ck, backend = env
    qx, bsx, sx, qw, bsw, sw, bias = _setup(ck, cuda_device, 128, 136, 256, seed=1)
    with pytest.raises(AssertionError):
        backend.linear_nvfp4_fused(qx, qw, sx, sw, bsx, bsw, requant_scale=torch.tensor(0.01, device=cuda_device))
