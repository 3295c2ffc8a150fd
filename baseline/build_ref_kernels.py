"""Compile the reference's own Blackwell quantizer kernels into baseline/_ref/libref_quant.so.

    python baseline/build_ref_kernels.py [--reference /path/to/comfy-kitchen] [--force]

These are the "kernels to beat" on the same GPU: the reference project's
comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu (launch_quantize_nvfp4_kernel, :323-384) and
ops/quantize_mxfp8.cu (launch_quantize_mxfp8_kernel, :148-208) with their three headers
(float_utils.cuh, utils.cuh, dtype_dispatch.cuh).  They are compiled from where they lie in a
checkout of the reference - nothing is copied into this repository - with the reference's own
nvcc flags (backends/cuda/CMakeLists.txt:69-79: -O3 --use_fast_math, extended lambdas, relaxed
constexpr) for sm_100a, static CUDA runtime.  The output directory is git-ignored.  bench.py
loads the library if it exists and times the two launchers beside this build's kernels; without
a checkout of the reference nothing is built and bench.py reports the entries as unavailable.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libref_quant.so")
DEFAULT_REFERENCE = os.environ.get("CK_REFERENCE", "/root/reference")
SOURCES = ("ops/quantize_nvfp4.cu", "ops/quantize_mxfp8.cu")


def build(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    cuda_dir = os.path.join(reference, "comfy_kitchen", "backends", "cuda")
    srcs = [os.path.join(cuda_dir, s) for s in SOURCES]
    if not all(os.path.exists(s) for s in srcs):
        return LIB if os.path.exists(LIB) else None
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--use_fast_math", "-std=c++17",
           "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
           "-I", cuda_dir, "-o", LIB, *srcs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("compiling the reference quantizer kernels failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force) or "reference checkout not found: nothing built")
