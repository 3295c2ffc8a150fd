"""The numpy oracle must reproduce the reference's eager outputs bit for bit.

The fixtures under tests/golden/ were produced by the reference's own eager
implementation (see tests/golden/make_golden.py); this file pins the oracle to
them, so that the GPU parity tests can trust the oracle at any size.
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import pytest
from conftest import GOLDEN_DIR, golden_input_f32, golden_names, load_golden

from oracle import ck_oracle as oc


@pytest.mark.parametrize("name", golden_names("nvfp4_"))
def test_quantize_nvfp4_matches_reference(name):
    d = load_golden(name)
    codes, scales = oc.quantize_nvfp4(golden_input_f32(d), d["scale"], pad_16x=bool(d["pad"]), hi_first=bool(d["hi_first"]))
    assert codes.shape == d["codes"].shape and scales.shape == d["scales"].shape
    np.testing.assert_array_equal(scales, d["scales"])
    np.testing.assert_array_equal(codes, d["codes"])


def _golden_as_f32(bits16: np.ndarray, kind: str) -> np.ndarray:
    if kind == "bfloat16":
        return oc.bf16_bits_to_f32(bits16)
    return bits16.view(np.float16).astype(np.float32)


@pytest.mark.parametrize("name", golden_names("nvfp4_"))
def test_dequantize_nvfp4_matches_reference(name):
    d = load_golden(name)
    deq = oc.dequantize_nvfp4(d["codes"], d["scale"], d["scales"], hi_first=bool(d["hi_first"]))
    np.testing.assert_array_equal(deq.view(np.uint32), d["deq"].view(np.uint32))
    for key, kind in (("deq_bf16", "bfloat16"), ("deq_f16", "float16")):
        got = oc.dequantize_nvfp4(d["codes"], d["scale"], d["scales"], hi_first=bool(d["hi_first"]), out_dtype=kind)
        np.testing.assert_array_equal(got.view(np.uint32), _golden_as_f32(d[key], kind).view(np.uint32))


@pytest.mark.parametrize("name", golden_names("mxfp8_"))
def test_quantize_mxfp8_matches_reference(name):
    d = load_golden(name)
    data, scales = oc.quantize_mxfp8(golden_input_f32(d), pad_32x=bool(d["pad"]))
    assert data.shape == d["data"].shape and scales.shape == d["scales"].shape
    np.testing.assert_array_equal(scales, d["scales"])
    np.testing.assert_array_equal(data, d["data"])


@pytest.mark.parametrize("name", golden_names("mxfp8_"))
def test_dequantize_mxfp8_matches_reference(name):
    d = load_golden(name)
    deq = oc.dequantize_mxfp8(d["data"], d["scales"])
    np.testing.assert_array_equal(deq.view(np.uint32), d["deq"].view(np.uint32))
    for key, kind in (("deq_bf16", "bfloat16"), ("deq_f16", "float16")):
        got = oc.dequantize_mxfp8(d["data"], d["scales"], out_dtype=kind)
        np.testing.assert_array_equal(got.view(np.uint32), _golden_as_f32(d[key], kind).view(np.uint32))


@pytest.mark.parametrize("name", golden_names("swizzle_"))
def test_swizzle_matches_reference(name):
    d = load_golden(name)
    blocked = oc.to_blocked(d["inp"])
    np.testing.assert_array_equal(blocked, d["blocked"])
    rows, cols = d["inp"].shape
    np.testing.assert_array_equal(oc.from_blocked(blocked, rows, cols), d["inp"])


def test_hi_first_is_a_nibble_swap():
    # reference tests/test_qdq.py:292-310: lo-first output == nibble-swapped hi-first output
    hi = load_golden("nvfp4_bf16_48x96_hi_first")
    lo = load_golden("nvfp4_bf16_48x96_lo_first")
    np.testing.assert_array_equal(((hi["codes"] << 4) | (hi["codes"] >> 4)).astype(np.uint8), lo["codes"])
    np.testing.assert_array_equal(hi["scales"], lo["scales"])


@pytest.mark.parametrize("name", golden_names("gemm_nvfp4_"))
def test_gemm_nvfp4_contract(name):
    d = load_golden(name)
    out = oc.scaled_mm_nvfp4(d["qa"], d["qb"], d["sa"], d["sb"], d["bsa"], d["bsb"],
                             bias=oc.bf16_bits_to_f32(d["bias"]) if "bias" in d else None)
    ref = d["ref"]
    # same dequantized operands; only the fp32 summation order of the matmul may differ
    assert np.linalg.norm(out - ref) / np.linalg.norm(ref) <= 1e-6


@pytest.mark.parametrize("name", golden_names("gemm_mxfp8_"))
def test_gemm_mxfp8_contract(name):
    d = load_golden(name)
    out = oc.scaled_mm_mxfp8(d["qa"], d["qb"], d["bsa"], d["bsb"],
                             bias=oc.bf16_bits_to_f32(d["bias"]) if "bias" in d else None)
    ref = d["ref"]
    assert np.linalg.norm(out - ref) / np.linalg.norm(ref) <= 1e-6


def test_large_case_digests():
    """Operands of the CPU-runnable linear ([256,3072] and [3072,3072], seed 0): digests of all four outputs."""
    import torch

    with open(os.path.join(GOLDEN_DIR, "large_digests.json")) as f:
        dig = json.load(f)
    g0 = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(256, 3072, generator=g0).bfloat16()
    w = (torch.randn(3072, 3072, generator=g0) * 0.02).bfloat16()
    for nm, t in (("x", x), ("w", w)):
        bits = t.view(torch.int16).numpy().view(np.uint16)
        if hashlib.sha256(bits.tobytes()).hexdigest() != dig[nm]["input_sha256"]:
            pytest.skip("torch's CPU generator produced different inputs than when the digests were frozen")
        xf = oc.bf16_bits_to_f32(bits)
        codes, scales = oc.quantize_nvfp4(xf, np.float32(dig[nm]["scale"]))
        assert hashlib.sha256(codes.tobytes()).hexdigest() == dig[nm]["nvfp4_codes_sha256"]
        assert hashlib.sha256(scales.tobytes()).hexdigest() == dig[nm]["nvfp4_scales_sha256"]
        data, e8 = oc.quantize_mxfp8(xf)
        assert hashlib.sha256(data.tobytes()).hexdigest() == dig[nm]["mxfp8_data_sha256"]
        assert hashlib.sha256(e8.tobytes()).hexdigest() == dig[nm]["mxfp8_scales_sha256"]
