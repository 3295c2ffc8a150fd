"""The C restatement (oracle/ck_oracle.c) against the same golden vectors as the numpy oracle,
and against the numpy oracle on random tensors with edge blocks."""
from __future__ import annotations

import numpy as np
import pytest
from conftest import golden_input_f32, golden_names, load_golden

from oracle import ck_oracle as oc
from oracle import ck_oracle_c as occ

pytestmark = pytest.mark.skipif(not occ.available(), reason="no C compiler for oracle/ck_oracle.c")


@pytest.mark.parametrize("name", golden_names("nvfp4_"))
def test_quantize_and_dequantize_nvfp4_match_reference(name):
    d = load_golden(name)
    codes, scales = occ.quantize_nvfp4(golden_input_f32(d), d["scale"], pad_16x=bool(d["pad"]), hi_first=bool(d["hi_first"]))
    np.testing.assert_array_equal(scales, d["scales"])
    np.testing.assert_array_equal(codes, d["codes"])
    deq = occ.dequantize_nvfp4(d["codes"], d["scale"], d["scales"], hi_first=bool(d["hi_first"]))
    np.testing.assert_array_equal(deq.view(np.uint32), d["deq"].view(np.uint32))


@pytest.mark.parametrize("name", golden_names("mxfp8_"))
def test_quantize_and_dequantize_mxfp8_match_reference(name):
    d = load_golden(name)
    data, scales = occ.quantize_mxfp8(golden_input_f32(d), pad_32x=bool(d["pad"]))
    np.testing.assert_array_equal(scales, d["scales"])
    np.testing.assert_array_equal(data, d["data"])
    deq = occ.dequantize_mxfp8(d["data"], d["scales"])
    np.testing.assert_array_equal(deq.view(np.uint32), d["deq"].view(np.uint32))


@pytest.mark.parametrize("shape", [(129, 128), (33, 80), (256, 3072), (1, 32)])
def test_c_equals_numpy_on_random_tensors(shape):
    rng = np.random.default_rng(shape[0] * 7 + shape[1])
    x = rng.standard_normal(shape).astype(np.float32)
    x[rng.random(shape) < 0.01] *= 30.0
    x[rng.random(shape) < 0.05] = 0.0
    x[0, :16] = -0.0
    x = oc.bf16_bits_to_f32(oc.f32_to_bf16_bits(x))
    gs = np.float32(np.abs(x).max() / 2688.0)
    a, b = oc.quantize_nvfp4(x, gs, pad_16x=True), occ.quantize_nvfp4(x, gs, pad_16x=True)
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])
    a, b = oc.quantize_mxfp8(x, pad_32x=True), occ.quantize_mxfp8(x, pad_32x=True)
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])
    np.testing.assert_array_equal(oc.f32_to_bf16_bits(x * np.float32(1.0009765625)), occ.f32_to_bf16_bits(x * np.float32(1.0009765625)))


@pytest.mark.parametrize("name", golden_names("gemm_nvfp4_"))
def test_gemm_contract_matches_reference(name):
    d = load_golden(name)
    out = occ.scaled_mm_nvfp4(d["qa"], d["qb"], d["sa"], d["sb"], d["bsa"], d["bsb"],
                              bias=oc.bf16_bits_to_f32(d["bias"]) if "bias" in d else None)
    ref = d["ref"]
    # same dequantized operands; only the fp32 summation order of the matmul may differ
    assert np.linalg.norm(out - ref) / np.linalg.norm(ref) <= 1e-6
