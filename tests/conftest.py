"""Shared test configuration: path set-up, the ``gpu`` marker and fixture loading."""
from __future__ import annotations

import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "comfy-kitchen_b200")
GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")

for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def golden_names(prefix: str) -> list[str]:
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz")))
    assert names, f"no golden fixtures with prefix {prefix!r}"
    return names


def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def golden_input_f32(d: dict) -> np.ndarray:
    """Input of a quantizer fixture as exact float32 values."""
    kind = str(d["x_dtype"])
    x = d["x"]
    if kind == "bfloat16":
        return (x.astype(np.uint32) << np.uint32(16)).view(np.float32)
    if kind == "float16":
        return x.view(np.float16).astype(np.float32)
    return x.astype(np.float32)


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
