"""CPU oracle for the quantized-linear path (TEST INFRASTRUCTURE, not product).

This module restates, in plain numpy, the arithmetic of the reference's eager
backend for the four hot-path operators and their helpers.  It exists only so
that tests, the smoke check and the bench's CPU-baseline leg can check or time
something that is independent of the CUDA kernels.  The shipped package never
imports it.

Parity status: PINNED.  Every function here is checked bit for bit against
outputs of the reference's own eager implementation, frozen as fixtures under
``tests/golden/`` by ``tests/golden/make_golden.py``.

Conventions
-----------
* bf16 / fp16 inputs are passed as ``float32`` arrays holding the exactly
  representable values (the conversion is lossless), so every operation below
  is IEEE binary32 with round-to-nearest-even unless stated.
* E4M3 / E8M0 / E2M1 results are returned as raw ``uint8`` bit patterns.

Reference files followed (paths inside the reference project):
  comfy_kitchen/backends/eager/quantization.py:115-160  quantize_nvfp4
  comfy_kitchen/backends/eager/quantization.py:171-219  dequantize_nvfp4
  comfy_kitchen/backends/eager/quantization.py:257-324  quantize_mxfp8
  comfy_kitchen/backends/eager/quantization.py:327-364  dequantize_mxfp8
  comfy_kitchen/float_utils.py:37-150                   E4M3 round trip, E2M1 cast
  comfy_kitchen/float_utils.py:253-260                  nibble packing
  comfy_kitchen/float_utils.py:292-352                  128x4 scale swizzle
  comfy_kitchen/float_utils.py:376-382                  E8M0 decode
"""
from __future__ import annotations

import numpy as np

F4_E2M1_MAX = np.float32(6.0)
F8_E4M3_MAX = np.float32(448.0)
E8M0_BIAS = 127

#: value of every 4-bit E2M1 code (comfy_kitchen/backends/eager/quantization.py:163-166)
E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=np.float32,
)


def roundup(x: int, m: int) -> int:
    return (x + m - 1) // m * m


# --------------------------------------------------------------------------- #
# input helpers
# --------------------------------------------------------------------------- #
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 bit patterns -> the same values as float32."""
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round-to-nearest-even (finite inputs)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)


# --------------------------------------------------------------------------- #
# small-float casts
# --------------------------------------------------------------------------- #
def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """float32 -> float8_e4m3fn bits, round-to-nearest-even, subnormals kept.

    Same result as ``x.to(torch.float8_e4m3fn)`` for |x| <= 448, which is the
    only range the quantizers feed it (float_utils.py:37-38 and
    eager/quantization.py:141-142, 314-315).  Larger magnitudes saturate to
    0x7E and NaN maps to 0x7F; neither is reachable from in-domain inputs.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    sign = ((bits >> np.uint32(24)) & np.uint32(0x80)).astype(np.uint8)
    mag = bits & np.uint32(0x7FFFFFFF)
    a = mag.view(np.float32)
    # normal numbers: keep 3 mantissa bits, ties to even, re-bias 127 -> 7
    r = mag + np.uint32(0x7FFFF) + ((mag >> np.uint32(20)) & np.uint32(1))
    code_n = (r >> np.uint32(20)).astype(np.int64) - ((127 - 7) << 3)
    # below 2^-6 the grid is uniform with step 2^-9 (8 rounds up into 0x08)
    with np.errstate(invalid="ignore", over="ignore"):
        code_s = np.rint(a * np.float32(512.0))
    code_s = np.where(np.isfinite(code_s), code_s, 0).astype(np.int64)
    code = np.where(a >= np.float32(2.0 ** -6), code_n, code_s)
    code = np.minimum(code, 0x7E)
    code = np.where(np.isnan(a), 0x7F, code)
    return (code.astype(np.uint8) | sign).astype(np.uint8)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    """float8_e4m3fn bits -> float32 (0x7F / 0xFF decode to NaN)."""
    b = np.asarray(b, dtype=np.uint8)
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 0x7).astype(np.float32)
    normal = np.ldexp(np.float32(1.0) + m / np.float32(8.0), e - 7)
    sub = np.ldexp(m / np.float32(8.0), -6)
    v = np.where(e == 0, sub, normal).astype(np.float32)
    v = np.where((b & 0x7F) == 0x7F, np.float32(np.nan), v)
    return np.where(b & 0x80, -v, v).astype(np.float32)


def f32_to_e2m1(y: np.ndarray) -> np.ndarray:
    """float32 in [-6, 6] -> 4-bit E2M1 code (sign in bit 3), ties to even.

    Restates the result of ``_f32_to_floatx_unpacked(y, 2, 1)``
    (float_utils.py:41-150) as decision thresholds: the representable
    magnitudes are 0, .5, 1, 1.5, 2, 3, 4, 6 and a midpoint goes to the
    neighbour whose mantissa bit is 0.  The sign bit of ``y`` is copied even
    when the magnitude rounds to zero (float_utils.py:141-148).
    """
    y = np.ascontiguousarray(y, dtype=np.float32)
    neg = (y.view(np.uint32) >> np.uint32(31)).astype(np.uint8)
    a = np.abs(y)
    code = (
        (a > 0.25).astype(np.uint8)
        + (a >= 0.75)
        + (a > 1.25)
        + (a >= 1.75)
        + (a > 2.5)
        + (a >= 3.5)
        + (a > 5.0)
    ).astype(np.uint8)
    return (code | (neg << 3)).astype(np.uint8)


def e8m0_to_f32(e: np.ndarray) -> np.ndarray:
    """E8M0 byte -> float32 2^(e-127); byte 0 decodes to 0.0 (float_utils.py:376-382)."""
    e = np.asarray(e, dtype=np.uint8)
    return (e.astype(np.uint32) << np.uint32(23)).view(np.float32)


# --------------------------------------------------------------------------- #
# packing and scale swizzle
# --------------------------------------------------------------------------- #
def pack_fp4(codes: np.ndarray, hi_first: bool = True) -> np.ndarray:
    """[R, C] 4-bit codes -> [R, C/2] bytes (float_utils.py:253-260)."""
    even, odd = codes[..., 0::2], codes[..., 1::2]
    if hi_first:
        return ((even << 4) | odd).astype(np.uint8)
    return ((odd << 4) | even).astype(np.uint8)


def unpack_fp4(packed: np.ndarray, hi_first: bool = True) -> np.ndarray:
    """Inverse of :func:`pack_fp4` (float_utils.py:263-274)."""
    hi, lo = packed >> 4, packed & 0xF
    pair = (hi, lo) if hi_first else (lo, hi)
    return np.stack(pair, axis=-1).reshape(*packed.shape[:-1], -1).astype(np.uint8)


def swizzled_offsets(rows: int, cols: int) -> np.ndarray:
    """Byte offset of logical scale (r, c) inside the 128x4-tiled scale buffer.

    The buffer has roundup(rows,128) * roundup(cols,4) bytes.  Each tile of 128
    rows x 4 columns occupies 512 contiguous bytes stored as 32 rows of 16
    bytes: row r of the tile lands at (r % 32) * 16 + (r // 32) * 4 + c
    (float_utils.py:303-326; backends/cuda/float_utils.cuh:110-125).
    """
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(cols, dtype=np.int64)[None, :]
    col_tiles = (cols + 3) // 4
    tile = (r // 128) * col_tiles + (c // 4)
    return tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (c % 4)


def to_blocked(scales: np.ndarray) -> np.ndarray:
    """[R, C] bytes -> swizzled [roundup(R,128), roundup(C,4)] bytes, zero padded."""
    rows, cols = scales.shape
    out = np.zeros(roundup(rows, 128) * roundup(cols, 4), dtype=scales.dtype)
    out[swizzled_offsets(rows, cols).ravel()] = scales.ravel()
    return out.reshape(roundup(rows, 128), roundup(cols, 4))


def from_blocked(blocked: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Inverse of :func:`to_blocked` restricted to the logical [rows, cols] window."""
    return blocked.reshape(-1)[swizzled_offsets(rows, cols)]


def _pad2d(x: np.ndarray, mult: int) -> np.ndarray:
    rows, cols = x.shape
    pr, pc = roundup(rows, mult), roundup(cols, mult)
    if (pr, pc) == (rows, cols):
        return x
    out = np.zeros((pr, pc), dtype=x.dtype)
    out[:rows, :cols] = x
    return out


# --------------------------------------------------------------------------- #
# NVFP4
# --------------------------------------------------------------------------- #
def quantize_nvfp4(x, per_tensor_scale, pad_16x: bool = False, hi_first: bool = True):
    """NVFP4 quantization (eager/quantization.py:115-160).

    x: float32 [M, K] holding the input's exact values; per_tensor_scale: the
    fp32 global scale.  Returns (packed codes uint8 [M', K'/2], E4M3 scale
    bytes uint8 [roundup(M',128), roundup(K'/16,4)] in the swizzled layout).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim != 2:
        raise ValueError("quantize_nvfp4 expects a 2-D input")
    g = np.float32(per_tensor_scale)
    if pad_16x:
        x = _pad2d(x, 16)
    rows, cols = x.shape
    if cols % 16:
        raise ValueError("columns must be a multiple of 16 unless pad_16x is set")
    xb = x.reshape(rows, cols // 16, 16)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        amax = np.max(np.abs(xb), axis=-1)                     # :137-138
        s = (amax / F4_E2M1_MAX) / g                           # :139-140 two true divisions
        s = np.minimum(s, F8_E4M3_MAX)                         # :141
        s8 = f32_to_e4m3(s)                                    # :142
        total = g * e4m3_to_f32(s8)                            # :143
        dead = total == 0                                      # :146
        safe = np.where(dead, np.float32(1.0), total)          # :147
        y = xb / safe[..., None]                               # :149
        y = np.where(dead[..., None], np.float32(0.0), y)      # :150
        y = np.clip(y, -F4_E2M1_MAX, F4_E2M1_MAX)              # :154
    codes = f32_to_e2m1(y.reshape(rows, cols))                 # :157
    return pack_fp4(codes, hi_first), to_blocked(s8)           # :158-159


def round_to_dtype(x: np.ndarray, out_dtype: str) -> np.ndarray:
    """float32 values rounded (nearest-even) to "float32" | "float16" | "bfloat16", returned as float32."""
    x = np.asarray(x, dtype=np.float32)
    if out_dtype == "float32":
        return x
    if out_dtype == "float16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if out_dtype == "bfloat16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    raise ValueError(out_dtype)


def dequantize_nvfp4(packed, per_tensor_scale, blocked_scales, hi_first: bool = True, out_dtype: str = "float32"):
    """NVFP4 -> values of ``out_dtype`` (returned as float32), eager/quantization.py:171-219.

    The reference does the arithmetic in the output dtype: the tensor scale and the
    block scale are cast to it, multiplied (:211), and the product scales the code
    value (:214); each product of two output-dtype numbers is exact in float32, so
    rounding the float32 product reproduces the output-dtype multiplication.
    """
    codes = unpack_fp4(np.asarray(packed, dtype=np.uint8), hi_first)
    rows, cols = codes.shape
    s8 = from_blocked(np.asarray(blocked_scales, dtype=np.uint8), rows, cols // 16)
    ts = round_to_dtype(np.float32(per_tensor_scale), out_dtype)
    total = round_to_dtype(ts * e4m3_to_f32(s8), out_dtype)    # :211
    vals = E2M1_VALUES[codes].reshape(rows, cols // 16, 16)
    return round_to_dtype((vals * total[..., None]).reshape(rows, cols), out_dtype)


# --------------------------------------------------------------------------- #
# MXFP8
# --------------------------------------------------------------------------- #
def _ceil_log2_biased(r: np.ndarray) -> np.ndarray:
    """clamp(ceil(log2(r)) + 127, 0, 254) for positive float32 r, by exponent bits.

    eager/quantization.py:298-300 evaluates ``ceil(log2(r))`` in float32.  For
    r = amax/448 with amax a bf16 or fp16 number the quotient is either an
    exact power of two or at least 5e-4 away (relative) from one, so the
    float32 logarithm cannot round across an integer and this integer form is
    bit-identical.  For float32 inputs within rounding distance of a power of
    two the reference's result depends on its log2 routine; that sliver is
    outside the pinned domain.
    """
    bits = np.ascontiguousarray(r, dtype=np.float32).view(np.uint32)
    e = ((bits >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int32)
    frac = (bits & np.uint32(0x7FFFFF)) != 0
    # subnormal r (exponent field 0) is below 2^-126: result clamps to <= 1
    biased = np.where(e == 0, np.where(frac, 1, 0), e + frac)
    return np.clip(biased, 0, 254).astype(np.uint8)


def quantize_mxfp8(x, pad_32x: bool = False):
    """MXFP8 quantization (eager/quantization.py:257-324).

    Returns (E4M3 data bytes uint8 [M', K'], E8M0 scale bytes uint8
    [roundup(M',128), roundup(K'/32,4)] in the swizzled layout).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim != 2:
        raise ValueError("quantize_mxfp8 expects a 2-D input")       # :276
    if pad_32x:
        x = _pad2d(x, 32)                                            # :279-285
    rows, cols = x.shape
    if cols % 32:
        raise ValueError("K dimension must be divisible by 32")      # :287
    xb = x.reshape(rows, cols // 32, 32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        amax = np.max(np.abs(xb), axis=-1)                           # :292
        need = amax / F8_E4M3_MAX                                    # :294
        need = np.maximum(need, np.float32(2.0 ** -127))             # :295
        e = _ceil_log2_biased(need)                                  # :298-302
        scale = e8m0_to_f32(e)                                       # :303
        dead = amax == 0                                             # :306
        scale = np.where(dead, np.float32(1.0), scale)               # :307
        y = xb / scale[..., None]                                    # :310
        y = np.where(dead[..., None], np.float32(0.0), y)            # :311
        y = np.clip(y, -F8_E4M3_MAX, F8_E4M3_MAX)                    # :314
    data = f32_to_e4m3(y.reshape(rows, cols))                        # :315
    e = np.where(dead, 0, e).astype(np.uint8)                        # :318
    return data, to_blocked(e)                                       # :322-324


def dequantize_mxfp8(data, blocked_scales, out_dtype: str = "float32"):
    """MXFP8 -> values of ``out_dtype`` (returned as float32), eager/quantization.py:327-364:
    float32 product, then one cast."""
    data = np.asarray(data, dtype=np.uint8)
    rows, cols = data.shape
    e = from_blocked(np.asarray(blocked_scales, dtype=np.uint8), rows, cols // 32)
    vals = e4m3_to_f32(data).reshape(rows, cols // 32, 32)
    with np.errstate(invalid="ignore"):
        prod = (vals * e8m0_to_f32(e)[..., None]).reshape(rows, cols).astype(np.float32)
    return round_to_dtype(prod, out_dtype)


# --------------------------------------------------------------------------- #
# GEMM reference: dequantize -> fp32 matmul (the contract for scaled_mm_*)
# --------------------------------------------------------------------------- #
def scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b,
                    bias=None, hi_first: bool = True):
    """float32 [M, N] = deq(a) @ deq(b).T + bias.

    The reference's eager ``scaled_mm_nvfp4`` (eager/quantization.py:222-246)
    hands the operands to ``torch.nn.functional.scaled_mm`` (PyTorch, pinned
    only as torch>=2.5 / >=2.10 for this API: scaled_mm_v2.py:7-53), which has
    no CPU kernel.  The parity contract is therefore the eager dequantizers
    followed by a float32 matmul, which is also what the tensor layer does
    when it falls back (tensor/nvfp4.py:262-264).
    """
    da = dequantize_nvfp4(a, tensor_scale_a, block_scale_a, hi_first)
    db = dequantize_nvfp4(b, tensor_scale_b, block_scale_b, hi_first)
    out = da @ db.T
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float32)[None, :]
    return out.astype(np.float32)


def scaled_mm_mxfp8(a, b, block_scale_a, block_scale_b, bias=None):
    """float32 [M, N] = deq(a) @ deq(b).T + bias (eager/quantization.py:367-402)."""
    out = dequantize_mxfp8(a, block_scale_a) @ dequantize_mxfp8(b, block_scale_b).T
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float32)[None, :]
    return out.astype(np.float32)
