"""Helpers shared by the GPU parity tests (torch tensor <-> raw bits, seeded inputs)."""
from __future__ import annotations

import numpy as np
import torch


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as numpy (bf16/f16 -> uint16, 1-byte floats -> uint8)."""
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.element_size() == 1:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def as_f32(t: torch.Tensor) -> np.ndarray:
    """Exact float32 values of a float tensor."""
    return t.detach().float().cpu().numpy()


def tensor_from_golden(d: dict, device) -> torch.Tensor:
    kind = str(d["x_dtype"])
    x = d["x"]
    if kind == "bfloat16":
        return torch.from_numpy(x.view(np.int16).copy()).view(torch.bfloat16).to(device)
    if kind == "float16":
        return torch.from_numpy(x.view(np.int16).copy()).view(torch.float16).to(device)
    return torch.from_numpy(x.astype(np.float32)).to(device)


def layout_scale(x: torch.Tensor) -> torch.Tensor:
    """Dynamic per-tensor scale of the NVFP4 layout: amax/(448*6) in x's dtype, then float32."""
    return (torch.amax(x.abs()) / (448.0 * 6.0)).to(torch.float32)


def dit_activation(m: int, k: int, seed: int = 0, outliers: bool = True) -> torch.Tensor:
    """CPU bf16 [m, k] ~ N(0,1) with 0.1 % of the entries scaled x20 (the DiT-projection input)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    if outliers:
        x = torch.where(torch.rand(m, k, generator=g) < 0.001, x * 20, x)
    return x.bfloat16()


def dit_weight(n: int, k: int, seed: int = 1, std: float = 0.02) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(n, k, generator=g) * std).bfloat16()
