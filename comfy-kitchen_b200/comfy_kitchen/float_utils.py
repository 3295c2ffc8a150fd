"""Format constants and layout helpers shared by the operators and the tensor layouts.

Only the helpers the quantized-linear path exposes are kept from the reference's
comfy_kitchen/float_utils.py: the numeric limits (:17-29), ``roundup`` (:32-34),
``swap_nibbles`` (:277-289) and the scale-factor swizzle ``to_blocked`` /
``from_blocked`` (:292-352).  The swizzle is written here as one gather with the
closed-form tile offset instead of a pad/permute chain.
"""
from __future__ import annotations

import torch

F4_E2M1_MAX = 6.0
F4_E2M1_EPS = 0.5
F8_E4M3_MAX = 448.0
F8_E4M3_EPS = 0.125
F8_E5M2_MAX = 57344.0
F8_E5M2_EPS = 0.0625
E8M0_BIAS = 127


def roundup(x: int, multiple: int) -> int:
    return (x + multiple - 1) // multiple * multiple


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def swap_nibbles(packed: torch.Tensor) -> torch.Tensor:
    """0xAB -> 0xBA in every byte: converts between the two FP4 nibble orders."""
    return ((packed << 4) | (packed >> 4)).to(torch.uint8)


def _swizzle_index(rows: int, cols: int, device) -> torch.Tensor:
    """Flat offset of logical scale (r, c) inside the 128x4-tiled buffer, as an [rows, cols] int64 tensor."""
    r = torch.arange(rows, device=device, dtype=torch.int64).unsqueeze(1)
    c = torch.arange(cols, device=device, dtype=torch.int64).unsqueeze(0)
    tile = (r // 128) * ceil_div(cols, 4) + (c // 4)
    return tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (c % 4)


def to_blocked(input_matrix: torch.Tensor, flatten: bool = True) -> torch.Tensor:
    """[H, W] scale matrix -> 128x4-tiled layout of roundup(H,128) x roundup(W,4) entries, zero padded."""
    rows, cols = input_matrix.shape
    pr, pc = roundup(rows, 128), roundup(cols, 4)
    raw = input_matrix.view(torch.uint8) if input_matrix.element_size() == 1 and input_matrix.dtype != torch.uint8 else input_matrix
    out = torch.zeros(pr * pc, device=raw.device, dtype=raw.dtype)
    out[_swizzle_index(rows, cols, raw.device).reshape(-1)] = raw.reshape(-1)
    out = out.view(input_matrix.dtype)
    return out if flatten else out.reshape(pr, pc)


def from_blocked(blocked_matrix: torch.Tensor, num_rows: int, num_cols: int) -> torch.Tensor:
    """Inverse of :func:`to_blocked`: the logical [num_rows, num_cols] window of a tiled scale buffer."""
    raw = blocked_matrix.view(torch.uint8) if blocked_matrix.element_size() == 1 and blocked_matrix.dtype != torch.uint8 else blocked_matrix
    out = raw.reshape(-1)[_swizzle_index(num_rows, num_cols, raw.device)]
    return out.view(blocked_matrix.dtype)
