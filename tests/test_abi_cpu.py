"""The C-ABI library builds, loads without a GPU and exports every declared symbol."""
from __future__ import annotations

import ctypes
import os
import re

import pytest
from conftest import PKG_DIR, ROOT

HEADER = os.path.join(ROOT, "include", "ck_b200.h")


@pytest.fixture(scope="module")
def lib_path():
    import importlib.util

    spec = importlib.util.spec_from_file_location("ck_build", os.path.join(PKG_DIR, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def declared_symbols() -> list[str]:
    text = open(HEADER).read()
    names = re.findall(r"CK_API\s+[\w\s\*]+?\b(ck_\w+)\s*\(", text)
    assert len(names) >= 7
    return names


def test_every_declared_symbol_is_exported(lib_path):
    lib = ctypes.CDLL(lib_path)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/ck_b200.h but not exported"


def test_version_and_error_string(lib_path):
    lib = ctypes.CDLL(lib_path)
    lib.ck_last_error.restype = ctypes.c_char_p
    header_version = int(re.search(r"#define CK_ABI_VERSION (\d+)", open(HEADER).read()).group(1))
    assert lib.ck_abi_version() == header_version
    assert isinstance(lib.ck_last_error(), bytes)


def test_argument_validation_needs_no_gpu(lib_path):
    """Bad arguments are rejected on the host before any CUDA call."""
    lib = ctypes.CDLL(lib_path)
    lib.ck_last_error.restype = ctypes.c_char_p
    P, L, I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.ck_quantize_nvfp4.argtypes = [P, I, P, P, P, L, L, L, L, I, P]
    assert lib.ck_quantize_nvfp4(None, 2, None, None, None, 16, 16, 16, 16, 1, None) == 1
    assert b"null" in lib.ck_last_error()
    fake = ctypes.c_void_p(0x1000)
    # 24 columns cannot be a 16-padded shape
    assert lib.ck_quantize_nvfp4(fake, 2, fake, fake, fake, 16, 24, 16, 24, 1, None) == 1
    # unknown dtype code
    assert lib.ck_quantize_nvfp4(fake, 9, fake, fake, fake, 16, 32, 16, 32, 1, None) == 1
    lib.ck_quantize_mxfp8.argtypes = [P, I, P, P, L, L, L, L, P]
    assert lib.ck_quantize_mxfp8(fake, 2, fake, fake, 32, 48, 32, 48, None) == 1


def test_python_package_reports_backends_without_gpu(lib_path):
    import torch

    import comfy_kitchen as ck

    info = ck.list_backends()
    assert {"cuda", "eager", "triton"} <= set(info)
    assert not info["eager"]["available"] and not info["triton"]["available"]
    if not torch.cuda.is_available():
        assert not info["cuda"]["available"]
        with pytest.raises(ck.NoCapableBackendError):
            ck.quantize_nvfp4(torch.zeros(16, 16, dtype=torch.bfloat16), torch.ones((), dtype=torch.float32))
