"""Regenerate the golden fixtures in this directory from the reference's eager code.

Run once, on a machine that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It imports the reference package from that path, runs its eager (pure torch,
CPU) implementations on seeded inputs, and stores inputs and outputs as raw
bytes in ``*.npz`` files next to this script, plus ``large_digests.json`` with
SHA-256 digests for cases too big to store.  Nothing else in the repository
imports the reference; tests only read the files written here.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as a numpy array (bf16/fp16 -> uint16, fp8 -> uint8)."""
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.float8_e5m2):
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def _layout_scale(x: torch.Tensor) -> torch.Tensor:
    # the dynamic scale of the NVFP4 layout: computed in x's dtype, then fp32
    return (torch.amax(x.abs()) / (448.0 * 6.0)).to(torch.float32)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    import comfy_kitchen as ck  # the reference

    ck.set_backend_priority(["eager"])
    from comfy_kitchen.float_utils import to_blocked

    out: dict[str, dict] = {}

    def nvfp4_case(name, x, scale=None, pad=False, hi_first=True):
        scale = _layout_scale(x) if scale is None else torch.tensor(scale, dtype=torch.float32)
        q, s = ck.quantize_nvfp4(x, scale, pad_16x=pad, hi_first=hi_first)
        deq = ck.dequantize_nvfp4(q, scale, s, torch.float32, hi_first=hi_first)
        out[name] = dict(
            x=_bits(x), x_dtype=str(x.dtype).replace("torch.", ""), scale=np.float32(scale.item()),
            pad=pad, hi_first=hi_first, codes=_bits(q), scales=_bits(s), deq=_bits(deq),
            deq_bf16=_bits(ck.dequantize_nvfp4(q, scale, s, torch.bfloat16, hi_first=hi_first)),
            deq_f16=_bits(ck.dequantize_nvfp4(q, scale, s, torch.float16, hi_first=hi_first)),
        )
        return q, s, scale

    def mxfp8_case(name, x, pad=False):
        q, s = ck.quantize_mxfp8(x, pad_32x=pad)
        deq = ck.dequantize_mxfp8(q, s, torch.float32)
        out[name] = dict(
            x=_bits(x), x_dtype=str(x.dtype).replace("torch.", ""), pad=pad,
            data=_bits(q), scales=_bits(s), deq=_bits(deq),
            deq_bf16=_bits(ck.dequantize_mxfp8(q, s, torch.bfloat16)),
            deq_f16=_bits(ck.dequantize_mxfp8(q, s, torch.float16)),
        )
        return q, s

    g = torch.Generator(device="cpu").manual_seed(42)

    # ---------------- NVFP4: shapes the reference's own tests use (scaled down) ------------
    nvfp4_case("nvfp4_bf16_64x128", (torch.randn(64, 128, generator=g) * 4).bfloat16())
    nvfp4_case("nvfp4_bf16_129x128_pad", (torch.randn(129, 128, generator=g) * 4).bfloat16(), pad=True)
    nvfp4_case("nvfp4_bf16_33x65_pad", (torch.randn(33, 65, generator=g) * 4).bfloat16(), pad=True)
    x = (torch.randn(48, 96, generator=g) * 4).bfloat16()
    nvfp4_case("nvfp4_bf16_48x96_lo_first", x, hi_first=False)
    nvfp4_case("nvfp4_bf16_48x96_hi_first", x, hi_first=True)
    nvfp4_case("nvfp4_fp16_32x64", (torch.randn(32, 64, generator=g) * 4).half())
    nvfp4_case("nvfp4_fp32_32x64", torch.randn(32, 64, generator=g) * 4)
    # activation-like data with sparse x20 outliers and a small-variance weight
    xo = torch.randn(160, 256, generator=g)
    mask = torch.rand(160, 256, generator=g) < 0.001
    nvfp4_case("nvfp4_bf16_160x256_outliers", torch.where(mask, xo * 20, xo).bfloat16())
    nvfp4_case("nvfp4_bf16_144x320_weight", (torch.randn(144, 320, generator=g) * 0.02).bfloat16())
    # static (calibrated) scale instead of the dynamic one
    nvfp4_case("nvfp4_bf16_32x64_static_scale", torch.randn(32, 64, generator=g).bfloat16(), scale=48.0 / 2688.0)

    # ---------------- NVFP4: hand-built edge blocks ------------------------------------------
    edge = torch.zeros(16, 64)
    # row 0: one x1000 outlier sets the global scale; rows 1-3 probe scale underflow
    edge[0, 0] = 1000.0
    edge[1, :16] = 1e-4
    edge[1, 16:32] = -2e-3
    edge[2, :16] = -3e-3
    edge[2, 16:32] = 3e-3
    # row 3: every rounding tie of the E2M1 grid (scale 1 * global) and signed zeros
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    edge[3, :16] = ties * (1000.0 / 6.0 / 448.0 * 32)  # some non-trivial block scale
    edge[4, :16] = ties
    edge[5, :16] = torch.tensor([6.0, -0.0, 0.0, -0.1, 0.1, -0.24, 0.26, 7.0, -7.0, 5.01, 4.99, 0.74, 0.76, -1e-6, 1e-6, 3.0])
    # row 6: a block that is exactly zero next to one that is not
    edge[6, 16:32] = 2.0
    # rows 7..15: decreasing magnitudes to walk the E4M3 scale through its subnormals
    for r in range(7, 16):
        edge[r, :] = torch.randn(64, generator=g) * (10.0 ** (-(r - 6) * 0.6))
    nvfp4_case("nvfp4_bf16_edge_blocks", edge.bfloat16())
    # scale saturation: global scale deliberately too small for the data
    nvfp4_case("nvfp4_bf16_saturating_scale", (torch.randn(16, 64, generator=g) * 4).bfloat16(), scale=1e-4)
    # block-scale rounding exactly at E4M3 ties and at the 2^-10 underflow tie
    gs = 0.5
    sat = torch.zeros(16, 32)
    for r, s_target in enumerate([2.0 ** -10, 2.0 ** -10 * 1.0001, 2.0 ** -9, 1.5 * 2.0 ** -9, 17.0, 19.0, 21.0, 23.0,
                                  1.0625, 1.1875, 0.0166015625, 448.0, 447.0, 463.0, 2.0 ** -6, 0.017578125]):
        sat[r, 0] = s_target * gs * 6.0
        sat[r, 1:16] = torch.linspace(-1, 1, 15) * s_target * gs * 6.0
    nvfp4_case("nvfp4_fp32_scale_ties", sat, scale=gs)

    # ---------------- MXFP8 ----------------------------------------------------------------------
    mxfp8_case("mxfp8_bf16_64x128", (torch.randn(64, 128, generator=g) * 4).bfloat16())
    mxfp8_case("mxfp8_bf16_65x96_pad", (torch.randn(65, 96, generator=g) * 4).bfloat16(), pad=True)
    mxfp8_case("mxfp8_fp16_32x64", (torch.randn(32, 64, generator=g) * 4).half())
    mxfp8_case("mxfp8_fp32_32x64", torch.randn(32, 64, generator=g) * 4)
    mxfp8_case("mxfp8_bf16_160x256_outliers", torch.where(mask, xo * 20, xo).bfloat16())
    mxfp8_case("mxfp8_bf16_144x320_weight", (torch.randn(144, 320, generator=g) * 0.02).bfloat16())
    medge = torch.zeros(16, 64)
    medge[0, :4] = torch.tensor([80.0, -1e-6, 1e-6, -0.0])
    medge[1, :32] = 448.0           # amax/448 exactly a power of two
    medge[1, 32:] = 449.0
    medge[2, :32] = 1.75            # 1.75/448 = 2^-8 exactly
    medge[2, 32:] = 1.7578125       # next bf16 above
    medge[3, :32] = torch.linspace(-3, 3, 32)
    medge[4, 32:] = -5e-5
    for r in range(5, 16):
        medge[r, :] = torch.randn(64, generator=g) * (10.0 ** ((r - 10) * 1.5))
    mxfp8_case("mxfp8_bf16_edge_blocks", medge.bfloat16())

    # ---------------- swizzle -------------------------------------------------------------------
    sw_in = (torch.arange(300 * 10, dtype=torch.int64) % 251).to(torch.uint8).reshape(300, 10)
    out["swizzle_300x10"] = dict(inp=_bits(sw_in), blocked=_bits(to_blocked(sw_in, flatten=False)))
    sw_in2 = (torch.arange(128 * 4, dtype=torch.int64) % 256).to(torch.uint8).reshape(128, 4)
    out["swizzle_128x4"] = dict(inp=_bits(sw_in2), blocked=_bits(to_blocked(sw_in2, flatten=False)))

    # ---------------- GEMM contract: eager dequantize -> fp32 matmul (+bias) ---------------------
    def gemm_nvfp4(name, m, n, k, with_bias):
        a = torch.randn(m, k, generator=g).bfloat16()
        b = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
        bias = (torch.randn(n, generator=g) * 0.01).bfloat16() if with_bias else None
        sa, sb = _layout_scale(a), _layout_scale(b)
        qa, bsa = ck.quantize_nvfp4(a, sa)
        qb, bsb = ck.quantize_nvfp4(b, sb)
        ref = ck.dequantize_nvfp4(qa, sa, bsa, torch.float32) @ ck.dequantize_nvfp4(qb, sb, bsb, torch.float32).t()
        if bias is not None:
            ref = ref + bias.float()
        d = dict(a=_bits(a), b=_bits(b), sa=np.float32(sa.item()), sb=np.float32(sb.item()),
                 qa=_bits(qa), qb=_bits(qb), bsa=_bits(bsa), bsb=_bits(bsb), ref=_bits(ref))
        if bias is not None:
            d["bias"] = _bits(bias)
        out[name] = d

    def gemm_mxfp8(name, m, n, k, with_bias):
        a = torch.randn(m, k, generator=g).bfloat16()
        b = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
        bias = (torch.randn(n, generator=g) * 0.01).bfloat16() if with_bias else None
        qa, bsa = ck.quantize_mxfp8(a)
        qb, bsb = ck.quantize_mxfp8(b)
        ref = ck.dequantize_mxfp8(qa, bsa, torch.float32) @ ck.dequantize_mxfp8(qb, bsb, torch.float32).t()
        if bias is not None:
            ref = ref + bias.float()
        d = dict(a=_bits(a), b=_bits(b), qa=_bits(qa), qb=_bits(qb), bsa=_bits(bsa), bsb=_bits(bsb), ref=_bits(ref))
        if bias is not None:
            d["bias"] = _bits(bias)
        out[name] = d

    gemm_nvfp4("gemm_nvfp4_128x256x256_bias", 128, 256, 256, True)
    gemm_nvfp4("gemm_nvfp4_48x136x192", 48, 136, 192, False)
    gemm_mxfp8("gemm_mxfp8_128x256x256_bias", 128, 256, 256, True)
    gemm_mxfp8("gemm_mxfp8_64x136x160", 64, 136, 160, False)

    for name, d in out.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)

    # ---------------- large case: the CPU-runnable linear (x [256,3072], W [3072,3072], seed 0), digests only ----
    g0 = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(256, 3072, generator=g0).bfloat16()
    w = (torch.randn(3072, 3072, generator=g0) * 0.02).bfloat16()
    digests = {"torch": torch.__version__, "how": "torch.Generator('cpu').manual_seed(0); x=randn(256,3072).bfloat16(); "
               "w=(randn(3072,3072)*0.02).bfloat16(); scale=(amax(|t|)/(448*6)) in bf16 then float32"}
    for nm, t in (("x", x), ("w", w)):
        s = _layout_scale(t)
        q, bs = ck.quantize_nvfp4(t, s)
        q8, bs8 = ck.quantize_mxfp8(t)
        digests[nm] = {
            "input_sha256": hashlib.sha256(_bits(t).tobytes()).hexdigest(),
            "scale": float(s.item()),
            "nvfp4_codes_sha256": hashlib.sha256(_bits(q).tobytes()).hexdigest(),
            "nvfp4_scales_sha256": hashlib.sha256(_bits(bs).tobytes()).hexdigest(),
            "mxfp8_data_sha256": hashlib.sha256(_bits(q8).tobytes()).hexdigest(),
            "mxfp8_scales_sha256": hashlib.sha256(_bits(bs8).tobytes()).hexdigest(),
        }
    with open(os.path.join(HERE, "large_digests.json"), "w") as f:
        json.dump(digests, f, indent=1)
    print(f"wrote {len(out)} fixtures + large_digests.json to {HERE}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
