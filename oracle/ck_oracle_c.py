"""ctypes front end of oracle/ck_oracle.c with the calling conventions of oracle/ck_oracle.py.

TEST INFRASTRUCTURE - not part of the product (see the header of ck_oracle.c).  The library is
built on first use by oracle/build.py; ``available()`` says whether that worked (gcc present).
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import build as _build

_lib = None
_error = None


def _load():
    global _lib, _error
    if _lib is not None or _error is not None:
        return _lib
    try:
        lib = ctypes.CDLL(_build.build())
        P, L, I, F = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        lib.ck_oracle_quantize_nvfp4.argtypes = [P, L, L, L, L, F, I, P, P]
        lib.ck_oracle_dequantize_nvfp4.argtypes = [P, P, F, L, L, I, P]
        lib.ck_oracle_quantize_mxfp8.argtypes = [P, L, L, L, L, P, P]
        lib.ck_oracle_dequantize_mxfp8.argtypes = [P, P, L, L, P]
        lib.ck_oracle_f32_to_bf16.argtypes = [P, L, P]
        for name in ("ck_oracle_quantize_nvfp4", "ck_oracle_dequantize_nvfp4", "ck_oracle_quantize_mxfp8",
                     "ck_oracle_dequantize_mxfp8", "ck_oracle_f32_to_bf16"):
            getattr(lib, name).restype = None
        lib.ck_oracle_threads.restype = I
        lib.ck_oracle_set_threads.argtypes = [I]
        lib.ck_oracle_set_threads.restype = None
        _lib = lib
    except Exception as e:  # noqa: BLE001 - no compiler, no library: callers fall back to numpy
        _error = f"{type(e).__name__}: {e}"
    return _lib


def available() -> bool:
    return _load() is not None


def threads() -> int:
    return int(_load().ck_oracle_threads())


def set_threads(n: int) -> None:
    """Use ``n`` OpenMP threads in the row loops from now on, whatever OMP_NUM_THREADS said at start-up."""
    _load().ck_oracle_set_threads(int(n))


def _roundup(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def quantize_nvfp4(x, per_tensor_scale, pad_16x: bool = False, hi_first: bool = True):
    lib = _load()
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    rp, cp = (_roundup(rows, 16), _roundup(cols, 16)) if pad_16x else (rows, cols)
    if cp % 16:
        raise ValueError("K dimension must be divisible by 16")
    codes = np.empty((rp, cp // 2), dtype=np.uint8)
    scales = np.empty((_roundup(rp, 128), _roundup(cp // 16, 4)), dtype=np.uint8)
    lib.ck_oracle_quantize_nvfp4(_ptr(x), rows, cols, rp, cp, ctypes.c_float(float(np.float32(per_tensor_scale))),
                                 int(hi_first), _ptr(codes), _ptr(scales))
    return codes, scales


def dequantize_nvfp4(packed, per_tensor_scale, blocked_scales, hi_first: bool = True) -> np.ndarray:
    lib = _load()
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(blocked_scales, dtype=np.uint8)
    rows, half = packed.shape
    out = np.empty((rows, half * 2), dtype=np.float32)
    lib.ck_oracle_dequantize_nvfp4(_ptr(packed), _ptr(scales), ctypes.c_float(float(np.float32(per_tensor_scale))), rows,
                                   half * 2, int(hi_first), _ptr(out))
    return out


def quantize_mxfp8(x, pad_32x: bool = False):
    lib = _load()
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    rp, cp = (_roundup(rows, 32), _roundup(cols, 32)) if pad_32x else (rows, cols)
    if cp % 32:
        raise ValueError("K dimension must be divisible by 32")
    data = np.empty((rp, cp), dtype=np.uint8)
    scales = np.empty((_roundup(rp, 128), _roundup(cp // 32, 4)), dtype=np.uint8)
    lib.ck_oracle_quantize_mxfp8(_ptr(x), rows, cols, rp, cp, _ptr(data), _ptr(scales))
    return data, scales


def dequantize_mxfp8(data, blocked_scales) -> np.ndarray:
    lib = _load()
    data = np.ascontiguousarray(data, dtype=np.uint8)
    scales = np.ascontiguousarray(blocked_scales, dtype=np.uint8)
    rows, cols = data.shape
    out = np.empty((rows, cols), dtype=np.float32)
    lib.ck_oracle_dequantize_mxfp8(_ptr(data), _ptr(scales), rows, cols, _ptr(out))
    return out


def f32_to_bf16_bits(x) -> np.ndarray:
    lib = _load()
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib.ck_oracle_f32_to_bf16(_ptr(x), x.size, _ptr(out))
    return out


def scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b, bias=None) -> np.ndarray:
    """The GEMM contract: dequantize both operands to float32, float32 matmul (BLAS), alpha, bias."""
    da = dequantize_nvfp4(a, 1.0, block_scale_a)
    db = dequantize_nvfp4(b, 1.0, block_scale_b)
    out = (da @ db.T) * (np.float32(tensor_scale_a) * np.float32(tensor_scale_b))
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float32)[None, :]
    return out.astype(np.float32)
