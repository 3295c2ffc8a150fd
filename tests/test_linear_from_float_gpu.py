"""The one-call NVFP4 linear on a dense activation (quantize -> GEMM inside one library call)
against the separate calls and the oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch
from gpu_util import as_f32, bits, dit_activation, dit_weight, layout_scale

from oracle import ck_oracle_c as occ
from oracle import ck_oracle as oc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(cuda_device):
    import comfy_kitchen as ck
    from comfy_kitchen.backends import cuda as backend

    assert ck.list_backends()["cuda"]["available"]
    return ck, backend


@pytest.mark.parametrize("shape", [(128, 128, 256), (48, 136, 192), (300, 520, 544), (1024, 768, 1024)])
@pytest.mark.parametrize("dynamic", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_one_call_equals_separate_calls(env, cuda_device, shape, dynamic, dtype):
    ck, backend = env
    m, n, k = shape
    g = torch.Generator(device="cpu").manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).to(dtype).to(cuda_device)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(cuda_device)
    bias = (torch.randn(n, generator=g) * 0.01).bfloat16().to(cuda_device)
    sw = layout_scale(w)
    qw, bsw = ck.quantize_nvfp4(w, sw)
    sx = None if dynamic else layout_scale(x)
    for _ in range(2):  # second call: the workspace (and the scale kernel's scratch in it) is reused
        y = backend.linear_nvfp4_from_float(x, qw, sw, bsw, bias=bias, x_scale=sx, out_dtype=torch.bfloat16)
        sx_ref = backend.nvfp4_tensor_scale(x) if dynamic else sx
        qx, bsx = ck.quantize_nvfp4(x, sx_ref)
        ref = ck.scaled_mm_nvfp4(qx, qw, sx_ref, sw, bsx, bsw, bias=bias, out_dtype=torch.bfloat16)
        assert torch.equal(y, ref)
    backend.check_device_status("linear_nvfp4_from_float")


def test_full_size_projection_against_oracle(env, cuda_device):
    """x [4096,3072] with outliers, W [3072,3072], bias: the one-call path against the CPU oracle chain
    quantize -> dequantize -> fp32 matmul (1e-3 relative norm, reference rounded to bf16)."""
    ck, backend = env
    x = dit_activation(4096, 3072)
    w = dit_weight(3072, 3072)
    bias = (torch.randn(3072, generator=torch.Generator(device="cpu").manual_seed(2)) * 0.01).bfloat16()
    sx, sw = layout_scale(x), layout_scale(w)
    qw, bsw = ck.quantize_nvfp4(w.to(cuda_device), sw.to(cuda_device))
    y = backend.linear_nvfp4_from_float(x.to(cuda_device), qw, sw.to(cuda_device), bsw, bias=bias.to(cuda_device),
                                        x_scale=sx.to(cuda_device), out_dtype=torch.bfloat16)
    impl = occ if occ.available() else oc
    rqx, rbsx = impl.quantize_nvfp4(as_f32(x), np.float32(sx.item()))
    ref = impl.scaled_mm_nvfp4(rqx, bits(qw), np.float32(sx.item()), np.float32(sw.item()), rbsx, bits(bsw), bias=as_f32(bias))
    ref = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
    got = y.float().cpu().numpy()
    err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert err <= 1e-3, f"relative error {err:.3e}"


def test_rejects_bad_arguments(env, cuda_device):
    ck, backend = env
    lib = backend.load_library()
    assert lib.ck_linear_nvfp4_from_float_workspace_bytes(128, 48, 0) == 0  # K not a multiple of 32
    need = lib.ck_linear_nvfp4_from_float_workspace_bytes(128, 256, 1)
    assert need > 128 * 128 + 128 * 16
    x = torch.zeros(128, 256, dtype=torch.bfloat16, device=cuda_device)
    small = torch.zeros(256, dtype=torch.uint8, device=cuda_device)
    rc = lib.ck_linear_nvfp4_from_float(x.data_ptr(), 2, None, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 0,
                                        x.data_ptr(), 2, 128, 128, 256, small.data_ptr(), small.numel(), None)
    assert rc != 0 and b"workspace" in lib.ck_last_error()


@pytest.mark.parametrize("shape", [(128, 128, 256), (48, 136, 192), (300, 520, 544), (4096, 3072, 3072)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_mxfp8_one_call_equals_separate_calls(env, cuda_device, shape, dtype):
    ck, backend = env
    m, n, k = shape
    g = torch.Generator(device="cpu").manual_seed(m + n + k + 1)
    x = torch.randn(m, k, generator=g).to(dtype).to(cuda_device)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(cuda_device)
    bias = (torch.randn(n, generator=g) * 0.01).bfloat16().to(cuda_device)
    qw, bsw = ck.quantize_mxfp8(w)
    for _ in range(2):
        y = backend.linear_mxfp8_from_float(x, qw, bsw, bias=bias, out_dtype=torch.bfloat16)
        qx, bsx = ck.quantize_mxfp8(x)
        ref = ck.scaled_mm_mxfp8(qx, qw, bsx, bsw, bias=bias, out_dtype=torch.bfloat16)
        assert torch.equal(y, ref)
    backend.check_device_status("linear_mxfp8_from_float")
    lib = backend.load_library()
    assert lib.ck_linear_mxfp8_from_float_workspace_bytes(128, 48) == 0  # K not a multiple of 32
    assert lib.ck_linear_mxfp8_from_float(x.data_ptr(), 2, qw.data_ptr(), bsw.data_ptr(), None, 2, y.data_ptr(), 2, m, n, k,
                                          None, 0, None) != 0  # no workspace
