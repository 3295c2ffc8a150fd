"""The ``cuda`` backend: thin Python wrappers over the sm_100a C-ABI library.

Each wrapper has the name and keyword arguments of the reference's wrapper in
comfy_kitchen/backends/cuda/__init__.py (quantize_nvfp4 :215-265, quantize_mxfp8
:303-336, scaled_mm_nvfp4 :339-463), allocates the outputs with torch, and passes raw
device pointers, sizes and the current stream through ``ctypes``.  Nothing here
computes: if the library is missing the backend is marked unavailable and every
operator raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

from comfy_kitchen.float_utils import roundup
from comfy_kitchen.ops import DTYPE_TO_CODE

__all__ = [
    "quantize_nvfp4",
    "quantize_mxfp8",
    "dequantize_nvfp4",
    "dequantize_mxfp8",
    "scaled_mm_nvfp4",
    "scaled_mm_mxfp8",
    "linear_nvfp4_fused",
    "linear_nvfp4_from_float",
    "linear_mxfp8_from_float",
    "nvfp4_tensor_scale",
    "check_device_status",
]

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
_DEFAULT_LIB = os.path.join(_PKG_ROOT, "lib", "libck_b200.so")
ABI_VERSION = 1

_lib = None
_lib_error: str | None = None

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64

# symbol -> argument types (return type is int unless listed in _RESTYPE)
_SIGNATURES = {
    "ck_abi_version": [],
    "ck_last_error": [],
    "ck_device_supported": [_I],
    "ck_debug_set_exact_division": [_I],
    "ck_quantize_nvfp4": [_P, _I, _P, _P, _P, _L, _L, _L, _L, _I, _P],
    "ck_quantize_mxfp8": [_P, _I, _P, _P, _L, _L, _L, _L, _P],
    "ck_scaled_mm_nvfp4": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _L, _L, _L, _P],
    "ck_scaled_mm_mxfp8": [_P, _P, _P, _P, _P, _I, _P, _I, _L, _L, _L, _P],
    "ck_gemm_status": [_P],
    "ck_debug_set_gemm_status": [_I],
    "ck_scaled_mm_workspace_bytes": [_I, _L, _L, _L],
    "ck_scaled_mm_nvfp4_ws": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _L, _L, _L, _P, _L, _P],
    "ck_scaled_mm_mxfp8_ws": [_P, _P, _P, _P, _P, _I, _P, _I, _L, _L, _L, _P, _L, _P],
    "ck_nvfp4_tensor_scale_scratch_bytes": [_L],
    "ck_nvfp4_tensor_scale": [_P, _I, _L, _P, _P, _L, _P],
    "ck_nvfp4_tensor_scale_noalloc": [_P, _I, _L, _P, _P],
    "ck_linear_nvfp4_fused": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _I, _P, _P, _P, _L, _L, _L, _P],
    "ck_linear_nvfp4_from_float_workspace_bytes": [_L, _L, _I],
    "ck_linear_nvfp4_from_float": [_P, _I, _P, _P, _P, _P, _P, _I, _P, _I, _L, _L, _L, _P, _L, _P],
    "ck_linear_mxfp8_from_float_workspace_bytes": [_L, _L],
    "ck_linear_mxfp8_from_float": [_P, _I, _P, _P, _P, _I, _P, _I, _L, _L, _L, _P, _L, _P],
    "ck_scaled_mm_nvfp4_allgather": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _L, _L, _L, _L, _L, _P],
    "ck_scaled_mm_mxfp8_allgather": [_P, _P, _P, _P, _P, _I, _P, _I, _I, _L, _L, _L, _L, _L, _P],
    "ck_peer_barrier": [_P, _I, _I, ctypes.c_uint32, _P],
    "ck_peer_barrier_bounded": [_P, _I, _I, ctypes.c_uint32, ctypes.c_uint32, _P],
    "ck_peer_status": [_P],
    "ck_dequantize_nvfp4": [_P, _P, _P, _P, _I, _L, _L, _I, _P],
    "ck_dequantize_mxfp8": [_P, _P, _P, _I, _L, _L, _P],
}
_RESTYPE = {"ck_last_error": ctypes.c_char_p, "ck_nvfp4_tensor_scale_scratch_bytes": ctypes.c_int64,
            "ck_scaled_mm_workspace_bytes": ctypes.c_int64, "ck_linear_nvfp4_from_float_workspace_bytes": ctypes.c_int64,
            "ck_linear_mxfp8_from_float_workspace_bytes": ctypes.c_int64}


def library_path() -> str:
    """Path of the shared library: ``$CK_LIB`` if set, else ``lib/libck_b200.so`` next to the package."""
    return os.environ.get("CK_LIB", _DEFAULT_LIB)


def load_library():
    """Load the C-ABI library once and declare its signatures.  Raises RuntimeError when it cannot."""
    global _lib, _lib_error
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        _lib_error = f"C-ABI library not found at {path} (build it with comfy-kitchen_b200/build.py)"
        raise RuntimeError(_lib_error)
    try:
        lib = ctypes.CDLL(path)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPE.get(name, _I)
        got = lib.ck_abi_version()
        if got != ABI_VERSION:
            raise RuntimeError(f"ABI version {got} != expected {ABI_VERSION}")
    except (OSError, AttributeError, RuntimeError) as e:
        _lib_error = f"cannot load {path}: {e}"
        raise RuntimeError(_lib_error) from e
    _lib = lib
    return lib


def is_loaded() -> bool:
    """True once the C-ABI library has been loaded in this process (never tries to load it)."""
    return _lib is not None


def _check(rc: int, what: str):
    if rc != 0:
        msg = _lib.ck_last_error()
        raise RuntimeError(f"{what} failed (code {rc}): {msg.decode() if msg else 'unknown error'}")


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on_device(device):
    """Context that makes ``device`` current for the library call; no device switch (several
    microseconds of host time per call) when it already is."""
    if not isinstance(device, torch.device):
        device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    index = device.index
    if index is None or index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _plain(t):
    return t.data if isinstance(t, torch.nn.Parameter) else t


def _scalar_f32(t: torch.Tensor, device, what: str) -> torch.Tensor:
    t = _plain(t)
    if t.numel() != 1:
        raise ValueError(f"{what} must hold exactly one value")
    if t.dtype != torch.float32 or t.device != device:
        t = t.to(device=device, dtype=torch.float32)
    return t.reshape(1)


# ------------------------------------------------------------------------------------------
# quantizers
# ------------------------------------------------------------------------------------------
def quantize_nvfp4(x: torch.Tensor, per_tensor_scale: torch.Tensor, epsilon: float = 0.0, pad_16x: bool = False,
                   hi_first: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16/f16/f32 [M, K] -> (uint8 [M', K'/2] codes, float8_e4m3fn swizzled block scales).

    ``epsilon`` is accepted for signature compatibility and unused, as in the reference.
    The scale tensor is allocated uninitialised: the kernel writes its padding as zeros.
    """
    lib = load_library()
    x = _plain(x)
    assert x.is_contiguous(), "Input tensor must be contiguous"
    rows, cols = x.shape
    if pad_16x:
        out_rows, out_cols = roundup(rows, 16), roundup(cols, 16)
    else:
        # rows are unconstrained, as in the eager implementation the results are pinned to
        out_rows, out_cols = rows, cols
        assert out_cols % 16 == 0, f"num_cols must be divisible by 16, got {out_cols}"
    scale = _scalar_f32(per_tensor_scale, x.device, "per_tensor_scale")
    qx = torch.empty((out_rows, out_cols // 2), device=x.device, dtype=torch.uint8)
    sx = torch.empty((roundup(out_rows, 128), roundup(out_cols // 16, 4)), device=x.device, dtype=torch.uint8)
    with _on_device(x.device):
        _check(lib.ck_quantize_nvfp4(_ptr(x), DTYPE_TO_CODE[x.dtype], _ptr(scale), _ptr(qx), _ptr(sx), rows, cols,
                                     out_rows, out_cols, int(bool(hi_first)), _stream(x.device)), "quantize_nvfp4")
    return qx, sx.view(torch.float8_e4m3fn)


def quantize_mxfp8(x: torch.Tensor, pad_32x: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16/f16/f32 [M, K] -> (float8_e4m3fn [M', K'], float8_e8m0fnu swizzled block scales)."""
    lib = load_library()
    x = _plain(x)
    assert x.is_contiguous(), "Input tensor must be contiguous"
    rows, cols = x.shape
    if pad_32x:
        out_rows, out_cols = roundup(rows, 32), roundup(cols, 32)
    else:
        out_rows, out_cols = rows, cols
        assert out_cols % 32 == 0, f"num_cols must be divisible by 32, got {out_cols}"
    qx = torch.empty((out_rows, out_cols), device=x.device, dtype=torch.uint8)
    sx = torch.empty((roundup(out_rows, 128), roundup(out_cols // 32, 4)), device=x.device, dtype=torch.uint8)
    with _on_device(x.device):
        _check(lib.ck_quantize_mxfp8(_ptr(x), DTYPE_TO_CODE[x.dtype], _ptr(qx), _ptr(sx), rows, cols, out_rows,
                                     out_cols, _stream(x.device)), "quantize_mxfp8")
    return qx.view(torch.float8_e4m3fn), sx.view(torch.float8_e8m0fnu)


_scale_scratch: dict = {}


def _scale_scratch_for(device, stream: int, need: int) -> torch.Tensor:
    """The zeroed scratch buffer of the tensor-scale kernel for this device and stream, at least
    ``need`` bytes.  An outgrown buffer is kept alive: a captured CUDA graph may still point at it."""
    key = (device, stream)
    scratch = _scale_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        if scratch is not None:
            _retired_workspaces.append(scratch)
        # 1 MiB covers 2^33 elements: growth (an allocation and a memset) is a first-call event
        scratch = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _scale_scratch[key] = scratch
    return scratch


def nvfp4_tensor_scale(x: torch.Tensor) -> torch.Tensor:
    """0-d float32 tensor ``amax(|x|) / (448 * 6)`` (division in x's dtype), computed by one kernel.

    The value the NVFP4 layout derives for a dynamically scaled tensor
    (comfy_kitchen/tensor/nvfp4.py:64-69 of the reference).  The kernel's scratch buffer is
    cached per (device, stream) and zeroed once when it is created.
    """
    lib = load_library()
    x = _plain(x)
    assert x.is_contiguous(), "Input tensor must be contiguous"
    n = x.numel()
    stream = _stream(x.device)
    scratch = _scale_scratch_for(x.device, stream, lib.ck_nvfp4_tensor_scale_scratch_bytes(n))
    out = torch.empty((), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        _check(lib.ck_nvfp4_tensor_scale(_ptr(x), DTYPE_TO_CODE[x.dtype], n, _ptr(out), _ptr(scratch), scratch.numel(),
                                         stream), "nvfp4_tensor_scale")
    return out


def dequantize_nvfp4(qx: torch.Tensor, per_tensor_scale: torch.Tensor, block_scales: torch.Tensor,
                     output_type: torch.dtype = torch.bfloat16, hi_first: bool = True) -> torch.Tensor:
    """uint8 [M, K/2] codes + swizzled E4M3 scales + fp32 tensor scale -> [M, K] of ``output_type``."""
    lib = load_library()
    qx, block_scales = _plain(qx), _plain(block_scales)
    assert qx.is_contiguous() and block_scales.is_contiguous(), "Input tensor must be contiguous"
    rows, packed = qx.shape
    cols = packed * 2
    assert cols % 16 == 0, f"num_cols must be divisible by 16, got {cols}"
    assert tuple(block_scales.shape) == (roundup(rows, 128), roundup(cols // 16, 4)), "Invalid scale shape"
    scale = _scalar_f32(per_tensor_scale, qx.device, "per_tensor_scale")
    out = torch.empty((rows, cols), device=qx.device, dtype=output_type)
    with _on_device(qx.device):
        _check(lib.ck_dequantize_nvfp4(_ptr(qx), _ptr(scale), _ptr(block_scales), _ptr(out), DTYPE_TO_CODE[output_type],
                                       rows, cols, int(bool(hi_first)), _stream(qx.device)), "dequantize_nvfp4")
    return out


def dequantize_mxfp8(qx: torch.Tensor, block_scales: torch.Tensor,
                     output_type: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """float8_e4m3fn [M, K] + swizzled E8M0 scales -> [M, K] of ``output_type``."""
    lib = load_library()
    qx, block_scales = _plain(qx), _plain(block_scales)
    assert qx.is_contiguous() and block_scales.is_contiguous(), "Input tensor must be contiguous"
    rows, cols = qx.shape
    assert cols % 32 == 0, f"num_cols must be divisible by 32, got {cols}"
    assert tuple(block_scales.shape) == (roundup(rows, 128), roundup(cols // 32, 4)), "Invalid scale shape"
    out = torch.empty((rows, cols), device=qx.device, dtype=output_type)
    with _on_device(qx.device):
        _check(lib.ck_dequantize_mxfp8(_ptr(qx), _ptr(block_scales), _ptr(out), DTYPE_TO_CODE[output_type], rows, cols,
                                       _stream(qx.device)), "dequantize_mxfp8")
    return out


# ------------------------------------------------------------------------------------------
# GEMMs
# ------------------------------------------------------------------------------------------
def _bias_args(bias, n: int, device):
    if bias is None or bias.numel() == 0:
        return None, 0, None
    bias = _plain(bias)
    assert bias.dtype in DTYPE_TO_CODE and DTYPE_TO_CODE[bias.dtype] <= 2, "bias must be f32, f16 or bf16"
    assert bias.numel() == n, f"bias must have {n} elements"
    bias = bias.contiguous()
    if bias.device != device:
        bias = bias.to(device)
    return bias.data_ptr(), DTYPE_TO_CODE[bias.dtype], bias


def scaled_mm_nvfp4(a: torch.Tensor, b: torch.Tensor, tensor_scale_a: torch.Tensor, tensor_scale_b: torch.Tensor,
                    block_scale_a: torch.Tensor, block_scale_b: torch.Tensor, bias: torch.Tensor | None = None,
                    out_dtype: torch.dtype | None = None, alpha: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] = (deq(a) @ deq(b).T) * (tensor_scale_a * tensor_scale_b) + bias.

    a: uint8 [M, K/2], b: uint8 [N, K/2]; block scales in the swizzled layout.  ``alpha``
    overrides the product of the tensor scales when given, as in the reference wrapper.
    """
    lib = load_library()
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    out_dtype = out_dtype or torch.bfloat16
    m, ka = a.shape
    n, kb = b.shape
    assert ka == kb, "Matrix dimensions do not match"
    k = 2 * ka
    assert n % 8 == 0, "B tensor must have 8 alignment in N dimension"
    assert block_scale_a.dtype == block_scale_b.dtype == torch.float8_e4m3fn, "NVFP4 block scales must be float8_e4m3fn"
    sk = roundup(k // 16, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    assert a.is_contiguous() and b.is_contiguous() and block_scale_a.is_contiguous() and block_scale_b.is_contiguous()
    dev = a.device
    tsa = _scalar_f32(tensor_scale_a, dev, "tensor_scale_a")
    tsb = _scalar_f32(tensor_scale_b, dev, "tensor_scale_b")
    alpha_t = None if alpha is None else _scalar_f32(alpha, dev, "alpha")
    bias_ptr, bias_code, bias_keep = _bias_args(bias, n, dev)
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    with _on_device(dev):
        ws_ptr, ws_bytes = _gemm_workspace(lib, False, m, n, k, dev)
        _check(lib.ck_scaled_mm_nvfp4_ws(_ptr(a), _ptr(b), _ptr(block_scale_a), _ptr(block_scale_b), _ptr(tsa), _ptr(tsb),
                                         _ptr(alpha_t), bias_ptr, bias_code, _ptr(out), DTYPE_TO_CODE[out_dtype], m, n, k,
                                         ws_ptr, ws_bytes, _stream(dev)), "scaled_mm_nvfp4")
    del bias_keep
    return out


_gemm_workspaces: dict = {}
_retired_workspaces: list = []  # outgrown buffers stay alive: a captured CUDA graph may still point at them


def _gemm_workspace(lib, is_mxfp8: bool, m: int, n: int, k: int, device):
    """(pointer, bytes) of the split-K workspace for this shape on the current stream, or (None, 0).

    The library decides (few activation rows, or few output tiles and a long K); the buffer is
    cached per device and stream and only ever grows, so steady-state calls allocate nothing."""
    need = int(lib.ck_scaled_mm_workspace_bytes(int(is_mxfp8), m, n, k))
    if need == 0:
        return None, 0
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _gemm_workspaces.get(key)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _retired_workspaces.append(ws)
        # zero-filled: the head of the workspace holds arrival counters that must start at zero
        # (every call leaves them at zero again)
        ws = torch.zeros(max(need, 1 << 22), dtype=torch.uint8, device=device)
        _gemm_workspaces[key] = ws
    return ws.data_ptr(), ws.numel()


def _pointer_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def scaled_mm_nvfp4_allgather(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b, out_ptrs, n_total: int,
                              col_offset: int, bias=None, out_dtype: torch.dtype = torch.bfloat16, alpha=None) -> None:
    """This rank's [M, N_local] block of a column-sharded NVFP4 GEMM, stored by the epilogue into every
    rank's [M, n_total] buffer (``out_ptrs``: device addresses valid in this process) at ``col_offset``.
    Launch only; the caller runs :func:`peer_barrier` behind it."""
    lib = load_library()
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    m, ka = a.shape
    n, kb = b.shape
    assert ka == kb, "Matrix dimensions do not match"
    k = 2 * ka
    sk = roundup(k // 16, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    assert a.is_contiguous() and b.is_contiguous() and block_scale_a.is_contiguous() and block_scale_b.is_contiguous()
    dev = a.device
    tsa = _scalar_f32(tensor_scale_a, dev, "tensor_scale_a")
    tsb = _scalar_f32(tensor_scale_b, dev, "tensor_scale_b")
    alpha_t = None if alpha is None else _scalar_f32(alpha, dev, "alpha")
    bias_ptr, bias_code, bias_keep = _bias_args(bias, n, dev)
    arr = _pointer_array(out_ptrs)
    with _on_device(dev):
        _check(lib.ck_scaled_mm_nvfp4_allgather(_ptr(a), _ptr(b), _ptr(block_scale_a), _ptr(block_scale_b), _ptr(tsa),
                                                _ptr(tsb), _ptr(alpha_t), bias_ptr, bias_code, arr, len(out_ptrs),
                                                DTYPE_TO_CODE[out_dtype], m, n, k, n_total, col_offset, _stream(dev)),
               "scaled_mm_nvfp4_allgather")
    del bias_keep


def scaled_mm_mxfp8_allgather(a, b, block_scale_a, block_scale_b, out_ptrs, n_total: int, col_offset: int, bias=None,
                              out_dtype: torch.dtype = torch.bfloat16) -> None:
    """MXFP8 counterpart of :func:`scaled_mm_nvfp4_allgather`."""
    lib = load_library()
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    m, k = a.shape
    n, kb = b.shape
    assert k == kb, "Matrix dimensions do not match"
    assert a.is_contiguous() and b.is_contiguous() and block_scale_a.is_contiguous() and block_scale_b.is_contiguous()
    dev = a.device
    bias_ptr, bias_code, bias_keep = _bias_args(bias, n, dev)
    arr = _pointer_array(out_ptrs)
    with _on_device(dev):
        _check(lib.ck_scaled_mm_mxfp8_allgather(_ptr(a), _ptr(b), _ptr(block_scale_a), _ptr(block_scale_b), bias_ptr,
                                                bias_code, arr, len(out_ptrs), DTYPE_TO_CODE[out_dtype], m, n, k, n_total,
                                                col_offset, _stream(dev)), "scaled_mm_mxfp8_allgather")
    del bias_keep


def peer_barrier(flag_ptrs, rank: int, epoch: int, device, max_polls: int | None = None) -> None:
    """Launch the cross-GPU barrier kernel on the current stream of ``device`` (see ck_peer_barrier).
    ``max_polls`` (about 0.5 us each, at most 2**26) replaces the default bound of about a second."""
    lib = load_library()
    arr = _pointer_array(flag_ptrs)
    with _on_device(device):
        if max_polls is None:
            _check(lib.ck_peer_barrier(arr, rank, len(flag_ptrs), epoch & 0xFFFFFFFF, _stream(device)), "peer_barrier")
        else:
            _check(lib.ck_peer_barrier_bounded(arr, rank, len(flag_ptrs), epoch & 0xFFFFFFFF, int(max_polls),
                                               _stream(device)), "peer_barrier")


def peer_status() -> int:
    """Synchronise and return the barrier status word (0 = all barriers completed); clears it."""
    lib = load_library()
    v = ctypes.c_int(0)
    _check(lib.ck_peer_status(ctypes.byref(v)), "peer_status")
    return v.value


def check_device_status(what: str = "kernel") -> None:
    """Raise RuntimeError if a bounded wait inside a GEMM kernel or the cross-GPU barrier gave up
    since the last check.  A launch returns 0 long before its kernel runs, so this is the only
    way to learn of such a failure; it synchronises the device, hence it is not called on the hot
    path (the layouts call it after each call chain when ``CK_STRICT=1``, never during graph
    capture)."""
    lib = load_library()
    g, b = ctypes.c_int(0), ctypes.c_int(0)
    _check(lib.ck_gemm_status(ctypes.byref(g)), "gemm_status")
    _check(lib.ck_peer_status(ctypes.byref(b)), "peer_status")
    if g.value != 0:
        raise RuntimeError(f"{what}: a wait inside a GEMM kernel gave up (device status {g.value}); the result is invalid")
    if b.value != 0:
        raise RuntimeError(f"{what}: rank {b.value - 1} did not arrive at the cross-GPU barrier in time; the result is invalid")


_linear_workspaces: dict = {}


def linear_nvfp4_from_float(x: torch.Tensor, w_codes: torch.Tensor, w_scale: torch.Tensor, w_block_scales: torch.Tensor,
                            bias: torch.Tensor | None = None, x_scale: torch.Tensor | None = None,
                            out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """NVFP4 linear on a dense activation in one library call: (dynamic scale ->) quantize -> GEMM.

    ``x`` [M, K] float; ``w_codes`` uint8 [N, K/2] with its tiled E4M3 ``w_block_scales`` and fp32
    ``w_scale``; ``x_scale`` a static per-tensor scale or None for ``amax(|x|)/2688``.  Same bits
    as ``quantize_nvfp4`` followed by ``scaled_mm_nvfp4``.  The quantized activation goes to a
    workspace cached per device and stream (grow-only; outgrown buffers are kept alive because a
    captured CUDA graph may still point at them)."""
    lib = load_library()
    x, w_codes, w_block_scales = _plain(x), _plain(w_codes), _plain(w_block_scales)
    assert x.dim() == 2 and x.is_contiguous(), "x must be a contiguous 2-D tensor"
    m, k = x.shape
    n, kb = w_codes.shape
    assert 2 * kb == k, "Matrix dimensions do not match"
    assert k % 32 == 0 and n % 8 == 0, "K must be a multiple of 32 and N of 8"
    assert tuple(w_block_scales.shape) == (roundup(n, 128), roundup(k // 16, 4)), "Invalid B scale shape"
    dev = x.device
    out_dtype = out_dtype or (x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16)
    sw = _scalar_f32(w_scale, dev, "w_scale")
    sx = None if x_scale is None else _scalar_f32(x_scale, dev, "x_scale")
    bias_ptr, bias_code, bias_keep = _bias_args(bias, n, dev)
    need = int(lib.ck_linear_nvfp4_from_float_workspace_bytes(m, k, int(sx is None)))
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    ws = _linear_workspaces.get(key)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)
        _linear_workspaces[key] = ws
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    with _on_device(dev):
        _check(lib.ck_linear_nvfp4_from_float(_ptr(x), DTYPE_TO_CODE[x.dtype], _ptr(sx), _ptr(w_codes), _ptr(w_block_scales),
                                              _ptr(sw), bias_ptr, bias_code, _ptr(out), DTYPE_TO_CODE[out_dtype], m, n, k,
                                              ws.data_ptr(), ws.numel(), _stream(dev)), "linear_nvfp4_from_float")
    del bias_keep
    return out


def linear_mxfp8_from_float(x: torch.Tensor, w_data: torch.Tensor, w_block_scales: torch.Tensor,
                            bias: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """MXFP8 linear on a dense activation in one library call: quantize -> GEMM.  ``x`` [M, K] float;
    ``w_data`` float8_e4m3fn [N, K] with its tiled E8M0 ``w_block_scales``.  Same bits as
    ``quantize_mxfp8`` followed by ``scaled_mm_mxfp8``; the quantized activation goes to a workspace
    cached per device and stream."""
    lib = load_library()
    x, w_data, w_block_scales = _plain(x), _plain(w_data), _plain(w_block_scales)
    assert x.dim() == 2 and x.is_contiguous(), "x must be a contiguous 2-D tensor"
    m, k = x.shape
    n, kb = w_data.shape
    assert kb == k, "Matrix dimensions do not match"
    assert k % 32 == 0 and n % 8 == 0, "K must be a multiple of 32 and N of 8"
    assert tuple(w_block_scales.shape) == (roundup(n, 128), roundup(k // 32, 4)), "Invalid B scale shape"
    assert w_data.is_contiguous() and w_block_scales.is_contiguous()
    dev = x.device
    out_dtype = out_dtype or (x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16)
    bias_ptr, bias_code, bias_keep = _bias_args(bias, n, dev)
    need = int(lib.ck_linear_mxfp8_from_float_workspace_bytes(m, k))
    key = (dev, torch.cuda.current_stream(dev).cuda_stream, "mxfp8")  # not shared with the NVFP4 path (its zeroed head)
    ws = _linear_workspaces.get(key)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=dev)
        _linear_workspaces[key] = ws
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    with _on_device(dev):
        _check(lib.ck_linear_mxfp8_from_float(_ptr(x), DTYPE_TO_CODE[x.dtype], _ptr(w_data), _ptr(w_block_scales), bias_ptr,
                                              bias_code, _ptr(out), DTYPE_TO_CODE[out_dtype], m, n, k, ws.data_ptr(),
                                              ws.numel(), _stream(dev)), "linear_mxfp8_from_float")
    del bias_keep
    return out


ACTIVATIONS = {None: 0, "none": 0, "gelu_tanh": 1}


def linear_nvfp4_fused(a: torch.Tensor, b: torch.Tensor, tensor_scale_a: torch.Tensor, tensor_scale_b: torch.Tensor,
                       block_scale_a: torch.Tensor, block_scale_b: torch.Tensor, bias: torch.Tensor | None = None,
                       activation: str | None = None, out_dtype: torch.dtype | None = None,
                       requant_scale: torch.Tensor | None = None, return_dense: bool = True):
    """NVFP4 linear whose epilogue applies ``activation`` and, when ``requant_scale`` (a static
    per-tensor scale) is given, quantizes the result to NVFP4 for the next layer.

    Returns ``(h, codes, block_scales)``: ``h`` is the dense [M, N] output (None when
    ``return_dense`` is False), ``codes`` / ``block_scales`` are what
    ``quantize_nvfp4(h, requant_scale)`` would return (None without ``requant_scale``).
    No counterpart in the reference, which runs the three steps as separate kernels.
    """
    lib = load_library()
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    out_dtype = out_dtype or torch.bfloat16
    m, ka = a.shape
    n, kb = b.shape
    assert ka == kb, "Matrix dimensions do not match"
    k = 2 * ka
    sk = roundup(k // 16, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    assert activation in ACTIVATIONS, f"unknown activation {activation!r}"
    assert return_dense or requant_scale is not None, "nothing to compute"
    dev = a.device
    tsa = _scalar_f32(tensor_scale_a, dev, "tensor_scale_a")
    tsb = _scalar_f32(tensor_scale_b, dev, "tensor_scale_b")
    bias_ptr, bias_code, bias_keep = _bias_args(bias, n, dev)
    out = torch.empty((m, n), dtype=out_dtype, device=dev) if return_dense else None
    codes = scales = rq = None
    if requant_scale is not None:
        assert n % 64 == 0, "re-quantized output needs N % 64 == 0"
        rq = _scalar_f32(requant_scale, dev, "requant_scale")
        codes = torch.empty((m, n // 2), dtype=torch.uint8, device=dev)
        scales = torch.empty((roundup(m, 128), n // 16), dtype=torch.uint8, device=dev)
    with _on_device(dev):
        _check(lib.ck_linear_nvfp4_fused(_ptr(a), _ptr(b), _ptr(block_scale_a), _ptr(block_scale_b), _ptr(tsa), _ptr(tsb),
                                         None, bias_ptr, bias_code, ACTIVATIONS[activation], _ptr(out),
                                         DTYPE_TO_CODE[out_dtype], _ptr(codes), _ptr(scales), _ptr(rq), m, n, k,
                                         _stream(dev)), "linear_nvfp4_fused")
    del bias_keep
    return out, codes, None if scales is None else scales.view(torch.float8_e4m3fn)


def scaled_mm_mxfp8(a: torch.Tensor, b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                    bias: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """out[M, N] = deq(a) @ deq(b).T + bias with E4M3 data [M, K] / [N, K] and E8M0 1x32 block scales."""
    lib = load_library()
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    out_dtype = out_dtype or torch.bfloat16
    m, k = a.shape
    n, kb = b.shape
    assert k == kb, "Matrix dimensions do not match"
    assert n % 8 == 0, "B tensor must have 8 alignment in N dimension"
    sk = roundup(k // 32, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    assert a.is_contiguous() and b.is_contiguous() and block_scale_a.is_contiguous() and block_scale_b.is_contiguous()
    dev = a.device
    bias_ptr, bias_code, bias_keep = _bias_args(bias, n, dev)
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    with _on_device(dev):
        ws_ptr, ws_bytes = _gemm_workspace(lib, True, m, n, k, dev)
        _check(lib.ck_scaled_mm_mxfp8_ws(_ptr(a), _ptr(b), _ptr(block_scale_a), _ptr(block_scale_b), bias_ptr, bias_code,
                                         _ptr(out), DTYPE_TO_CODE[out_dtype], m, n, k, ws_ptr, ws_bytes, _stream(dev)),
               "scaled_mm_mxfp8")
    del bias_keep
    return out


# ------------------------------------------------------------------------------------------
# registration
# ------------------------------------------------------------------------------------------
def _build_constraints() -> dict:
    from comfy_kitchen.constraints import DivisibleBy, ExactDims, FunctionConstraints, ParamConstraint

    cuda_only = frozenset({"cuda"})
    floats = frozenset({torch.float32, torch.float16, torch.bfloat16})
    f32 = frozenset({torch.float32})
    blackwell = (10, 0)
    return {
        "quantize_nvfp4": FunctionConstraints(
            params={"x": ParamConstraint(dtypes=floats, shape_rules=(ExactDims(2),)),
                    "per_tensor_scale": ParamConstraint(dtypes=f32)},
            default_devices=cuda_only, min_compute_capability=blackwell),
        "quantize_mxfp8": FunctionConstraints(
            params={"x": ParamConstraint(dtypes=floats, shape_rules=(ExactDims(2),))},
            default_devices=cuda_only, min_compute_capability=blackwell),
        "dequantize_nvfp4": FunctionConstraints(
            params={"qx": ParamConstraint(dtypes=frozenset({torch.uint8}), shape_rules=(ExactDims(2),)),
                    "per_tensor_scale": ParamConstraint(dtypes=f32),
                    "block_scales": ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn})),
                    "output_type": ParamConstraint(dtypes=floats)},
            default_devices=cuda_only, min_compute_capability=blackwell),
        "dequantize_mxfp8": FunctionConstraints(
            params={"qx": ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn}), shape_rules=(ExactDims(2), DivisibleBy(1, 32))),
                    "block_scales": ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                    "output_type": ParamConstraint(dtypes=floats)},
            default_devices=cuda_only, min_compute_capability=blackwell),
        "scaled_mm_nvfp4": FunctionConstraints(
            params={"a": ParamConstraint(dtypes=frozenset({torch.uint8}), shape_rules=(ExactDims(2), DivisibleBy(1, 16))),
                    "b": ParamConstraint(dtypes=frozenset({torch.uint8}), shape_rules=(ExactDims(2), DivisibleBy(1, 16))),
                    "tensor_scale_a": ParamConstraint(dtypes=f32),
                    "tensor_scale_b": ParamConstraint(dtypes=f32),
                    "block_scale_a": ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn})),
                    "block_scale_b": ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn})),
                    "out_dtype": ParamConstraint(dtypes=floats)},
            default_devices=cuda_only, min_compute_capability=blackwell),
        "scaled_mm_mxfp8": FunctionConstraints(
            params={"a": ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn}), shape_rules=(ExactDims(2), DivisibleBy(1, 32))),
                    "b": ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn}), shape_rules=(ExactDims(2), DivisibleBy(1, 32))),
                    "block_scale_a": ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                    "block_scale_b": ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                    "out_dtype": ParamConstraint(dtypes=floats)},
            default_devices=cuda_only, min_compute_capability=blackwell),
    }


def _register():
    import sys

    from comfy_kitchen.registry import registry

    try:
        load_library()
    except RuntimeError as e:
        registry.mark_unavailable("cuda", str(e))
        return
    if not torch.cuda.is_available():
        registry.mark_unavailable("cuda", "CUDA not available on this system")
        return
    registry.register("cuda", sys.modules[__name__], _build_constraints())


_register()
