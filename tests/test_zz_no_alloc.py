"""The allocation-free tensor-scale entry point, called through the C ABI.

Some callers cannot pass a scratch buffer because they are not allowed to allocate device
memory where they call from (inside a stream capture, inside a host application that owns
all device memory, in a latency-critical serving loop).  `ck_nvfp4_tensor_scale_noalloc`
serves them from a fixed array inside the library.  This test checks that it returns
exactly what the scratch-taking entry point returns, twice in a row (the array is shared
and keeps the previous call's contents), and that it refuses inputs beyond its limit.
Collected last on purpose: a failure here cannot hide the result of any other test.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMENTS = 16384 * 8192


@pytest.fixture(scope="module")
def lib(cuda_device):
    from comfy_kitchen.backends import cuda as backend

    return backend.load_library()


def _with_scratch(lib, x: torch.Tensor) -> torch.Tensor:
    n = x.numel()
    need = lib.ck_nvfp4_tensor_scale_scratch_bytes(n)
    scratch = torch.zeros(need, dtype=torch.uint8, device=x.device)
    out = torch.empty((), dtype=torch.float32, device=x.device)
    rc = lib.ck_nvfp4_tensor_scale(x.data_ptr(), 2, n, out.data_ptr(), scratch.data_ptr(), need,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ck_last_error()
    return out


def _no_alloc(lib, x: torch.Tensor) -> torch.Tensor:
    out = torch.empty((), dtype=torch.float32, device=x.device)
    rc = lib.ck_nvfp4_tensor_scale_noalloc(x.data_ptr(), 2, x.numel(), out.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ck_last_error()
    return out


def test_no_alloc_entry_point_matches_scratch_entry_point(lib, cuda_device):
    g = torch.Generator(device="cpu").manual_seed(2024)
    big = (torch.randn(4096, 3072, generator=g) * 2).bfloat16().to(cuda_device)
    small = (torch.randn(33, 65, generator=g) * 9).bfloat16().to(cuda_device)   # fewer blocks than the call before
    for x in (big, small, big):
        want = _with_scratch(lib, x)
        first = _no_alloc(lib, x)
        second = _no_alloc(lib, x)   # the shared array still holds the first call's partials
        torch.cuda.synchronize()
        assert first.view(torch.int32).item() == want.view(torch.int32).item()
        assert second.view(torch.int32).item() == want.view(torch.int32).item()
        # and both agree with the layout's expression evaluated on the host
        ref = (torch.amax(x.cpu().abs()) / (448.0 * 6.0)).to(torch.float32)
        assert first.cpu().view(torch.int32).item() == ref.view(torch.int32).item()


def test_no_alloc_entry_point_refuses_oversized_input(lib, cuda_device):
    x = torch.zeros(16, dtype=torch.bfloat16, device=cuda_device)
    out = torch.empty((), dtype=torch.float32, device=cuda_device)
    rc = lib.ck_nvfp4_tensor_scale_noalloc(x.data_ptr(), 2, MAX_ELEMENTS + 1, out.data_ptr(), None)
    assert rc == 1
    msg = lib.ck_last_error().decode()
    assert "exceed" in msg and str(MAX_ELEMENTS) in msg
