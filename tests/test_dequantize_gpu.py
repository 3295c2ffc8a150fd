"""GPU parity of the dequantizers: bit-exact against the golden fixtures and the oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import golden_names, load_golden
from gpu_util import bits, dit_activation, layout_scale

from oracle import ck_oracle as oc

pytestmark = pytest.mark.gpu
DTYPES = [(torch.float32, "float32", "deq"), (torch.bfloat16, "bfloat16", "deq_bf16"), (torch.float16, "float16", "deq_f16")]


@pytest.fixture(scope="module")
def ck(cuda_device):
    import comfy_kitchen

    assert comfy_kitchen.list_backends()["cuda"]["available"]
    return comfy_kitchen


def _as_bits32(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy().view(np.uint32)


def _golden_f32(a: np.ndarray, kind: str) -> np.ndarray:
    if kind == "float32":
        return a
    if kind == "bfloat16":
        return oc.bf16_bits_to_f32(a)
    return a.view(np.float16).astype(np.float32)


@pytest.mark.parametrize("name", golden_names("nvfp4_"))
@pytest.mark.parametrize("dtype,kind,key", DTYPES)
def test_nvfp4_golden(ck, cuda_device, name, dtype, kind, key):
    d = load_golden(name)
    q = torch.from_numpy(d["codes"]).to(cuda_device)
    s = torch.from_numpy(d["scales"]).to(cuda_device).view(torch.float8_e4m3fn)
    out = ck.dequantize_nvfp4(q, torch.tensor(float(d["scale"]), device=cuda_device), s, dtype, hi_first=bool(d["hi_first"]))
    assert out.dtype == dtype and tuple(out.shape) == (d["codes"].shape[0], d["codes"].shape[1] * 2)
    np.testing.assert_array_equal(_as_bits32(out), _golden_f32(d[key], kind).view(np.uint32))


@pytest.mark.parametrize("name", golden_names("mxfp8_"))
@pytest.mark.parametrize("dtype,kind,key", DTYPES)
def test_mxfp8_golden(ck, cuda_device, name, dtype, kind, key):
    d = load_golden(name)
    q = torch.from_numpy(d["data"]).to(cuda_device).view(torch.float8_e4m3fn)
    s = torch.from_numpy(d["scales"]).to(cuda_device).view(torch.float8_e8m0fnu)
    out = ck.dequantize_mxfp8(q, s, dtype)
    got, want = _as_bits32(out), _golden_f32(d[key], kind).view(np.uint32)
    finite = np.isfinite(_golden_f32(d[key], kind))  # out-of-domain blocks decode to NaN payloads
    np.testing.assert_array_equal(got[finite], want[finite])


@pytest.mark.parametrize("dtype,kind,key", DTYPES)
def test_round_trip_full_size(ck, cuda_device, dtype, kind, key):
    """[4096,3072] activation: quantize -> dequantize equals the oracle's dequantization, both formats."""
    x = dit_activation(4096, 3072).to(cuda_device)
    sc = layout_scale(x)
    q, s = ck.quantize_nvfp4(x, sc)
    out = ck.dequantize_nvfp4(q, sc, s, dtype)
    ref = oc.dequantize_nvfp4(bits(q), np.float32(sc.item()), bits(s), out_dtype=kind)
    np.testing.assert_array_equal(_as_bits32(out), ref.view(np.uint32))
    q8, s8 = ck.quantize_mxfp8(x)
    out8 = ck.dequantize_mxfp8(q8, s8, dtype)
    ref8 = oc.dequantize_mxfp8(bits(q8), bits(s8), out_dtype=kind)
    np.testing.assert_array_equal(_as_bits32(out8), ref8.view(np.uint32))
    # quantization error bound of the formats: relative error of the round trip
    err = (out.float() - x.float()).norm() / x.float().norm()
    err8 = (out8.float() - x.float()).norm() / x.float().norm()
    assert err < 0.15 and err8 < 0.05
