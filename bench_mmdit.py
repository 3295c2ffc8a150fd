"""Random-init MMDiT-shaped stack for the data-parallel full-model measurement.

A workload generator, not a model port: the reference ships no model, so this is a minimal
two-stream / one-stream transformer written from the dimensions alone (hidden 3072, 24 heads of
128, 19 double-stream + 38 single-stream blocks, MLP ratio 4, 4096 image + 512 text tokens).
Every ``nn.Linear`` of the blocks is created, quantized to NVFP4 and released layer by layer
(``comfy_kitchen.modules.NVFP4Linear``: dynamic activation scale, quantize kernel, tcgen05 GEMM
with bias); attention is ``torch`` SDPA in bf16; no positional encoding (not on the measured
path).  Parameter count of the linears at full size: 19 x 36 h^2 + 38 x 15 h^2 = 11.84 B.
Element-wise glue is kept to one pass where torch offers it (addcmul for modulation and gated
residuals).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class MMDiTConfig:
    hidden: int = 3072
    heads: int = 24
    double_blocks: int = 19
    single_blocks: int = 38
    mlp_ratio: int = 4
    img_tokens: int = 4096
    txt_tokens: int = 512

    @property
    def linear_params(self) -> int:
        h2 = self.hidden * self.hidden
        r = self.mlp_ratio
        per_stream = (3 + 1 + 2 * r + 6) * h2
        single = ((3 + r) + (1 + r) + 3) * h2
        return self.double_blocks * 2 * per_stream + self.single_blocks * single

    def linear_flops(self, batch: int) -> float:
        """2 x parameters x tokens for the token-wise linears; the modulation linears see one row per sample."""
        h2 = self.hidden * self.hidden
        r = self.mlp_ratio
        tokens = batch * (self.img_tokens + self.txt_tokens)
        tokenwise = self.double_blocks * (3 + 1 + 2 * r) * h2 + self.single_blocks * ((3 + r) + (1 + r)) * h2
        per_sample = self.double_blocks * 2 * 6 * h2 + self.single_blocks * 3 * h2
        return 2.0 * tokenwise * tokens + 2.0 * per_sample * batch

    def attention_flops(self, batch: int) -> float:
        s = self.img_tokens + self.txt_tokens
        return (self.double_blocks + self.single_blocks) * 4.0 * s * s * self.hidden * batch


def _qlinear(i: int, o: int, device, gen, make_linear):
    """A dense layer with N(0, 0.02) weights, handed to ``make_linear`` (quantizer) and released."""
    lin = nn.Linear(i, o, bias=True, device=device, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_((torch.randn(o, i, device=device, generator=gen) * 0.02).to(torch.bfloat16))
        lin.bias.zero_()
    return make_linear(lin)


def _modulate(x, shift, scale):
    # layer_norm(x) * (1 + scale) + shift in one pass over the tokens
    return torch.addcmul(shift.unsqueeze(1), F.layer_norm(x, x.shape[-1:]), (1 + scale).unsqueeze(1))


def _attention(q, k, v, heads):
    b, s, h = q.shape
    d = h // heads
    q, k, v = (t.reshape(b, s, heads, d).transpose(1, 2) for t in (q, k, v))
    o = F.scaled_dot_product_attention(q, k, v)
    return o.transpose(1, 2).reshape(b, s, h)


def _mlp(fc1, fc2):
    """fc2(gelu(fc1(x))): quantized NVFP4 layers get the module that can fuse the middle steps into
    fc1's epilogue once fc2 has a static input scale (``calibrate_hidden_scales``)."""
    try:
        from comfy_kitchen.modules import NVFP4Linear, NVFP4MLP
        if isinstance(fc1, NVFP4Linear) and isinstance(fc2, NVFP4Linear):
            return NVFP4MLP(fc1, fc2)
    except ImportError:
        pass
    return lambda x: fc2(F.gelu(fc1(x), approximate="tanh"))


class _Stream(nn.Module):
    def __init__(self, cfg: MMDiTConfig, device, gen, make_linear):
        super().__init__()
        h = cfg.hidden
        self.mod = _qlinear(h, 6 * h, device, gen, make_linear)
        self.qkv = _qlinear(h, 3 * h, device, gen, make_linear)
        self.proj = _qlinear(h, h, device, gen, make_linear)
        self.fc1 = _qlinear(h, cfg.mlp_ratio * h, device, gen, make_linear)
        self.fc2 = _qlinear(cfg.mlp_ratio * h, h, device, gen, make_linear)
        self.mlp = _mlp(self.fc1, self.fc2)


class DoubleBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, device, gen, make_linear):
        super().__init__()
        self.heads = cfg.heads
        self.img = _Stream(cfg, device, gen, make_linear)
        self.txt = _Stream(cfg, device, gen, make_linear)

    def forward(self, img, txt, vec):
        parts = []
        for x, st in ((txt, self.txt), (img, self.img)):
            m = st.mod(F.silu(vec)).chunk(6, dim=-1)
            parts.append((x, st, m, st.qkv(_modulate(x, m[0], m[1])).chunk(3, dim=-1)))
        q = torch.cat([p[3][0] for p in parts], dim=1)
        k = torch.cat([p[3][1] for p in parts], dim=1)
        v = torch.cat([p[3][2] for p in parts], dim=1)
        attn = _attention(q, k, v, self.heads)
        outs, start = [], 0
        for x, st, m, _ in parts:
            a = attn[:, start:start + x.shape[1]]
            start += x.shape[1]
            x = torch.addcmul(x, m[2].unsqueeze(1), st.proj(a))
            x = torch.addcmul(x, m[5].unsqueeze(1), st.mlp(_modulate(x, m[3], m[4])))
            outs.append(x)
        return outs[1], outs[0]


class SingleBlock(nn.Module):
    """One-stream block: attention and MLP branches read the same modulated input and are merged by
    the second projection.  The fused weights [h -> 3h + 4h] and [h + 4h -> h] are kept as their
    column / row blocks (same parameters and FLOPs), so that no split or concatenation copy of the
    wide hidden tensor is needed and the activation is quantized once for both input projections."""

    def __init__(self, cfg: MMDiTConfig, device, gen, make_linear):
        super().__init__()
        h, r = cfg.hidden, cfg.mlp_ratio
        self.heads, self.h = cfg.heads, h
        self.mod = _qlinear(h, 3 * h, device, gen, make_linear)
        self.linear1_qkv = _qlinear(h, 3 * h, device, gen, make_linear)
        self.linear1_mlp = _qlinear(h, r * h, device, gen, make_linear)
        self.linear2_attn = _qlinear(h, h, device, gen, make_linear)
        self.linear2_mlp = _qlinear(r * h, h, device, gen, make_linear)
        self.mlp = _mlp(self.linear1_mlp, self.linear2_mlp)

    def forward(self, x, vec):
        shift, scale, gate = self.mod(F.silu(vec)).chunk(3, dim=-1)
        xin = _modulate(x, shift, scale)
        quantize = getattr(self.linear1_qkv, "quantize_input", None)
        if quantize is not None:  # quantized layers: one activation quantization feeds both projections
            b, s_, _ = xin.shape
            xq = quantize(xin.reshape(b * s_, self.h))
            q, k, v = self.linear1_qkv(xq).reshape(b, s_, 3 * self.h).chunk(3, dim=-1)
            mlp = self.mlp(xq).reshape(b, s_, -1)
        else:
            q, k, v = self.linear1_qkv(xin).chunk(3, dim=-1)
            mlp = self.mlp(xin)
        attn = _attention(q, k, v, self.heads)
        return torch.addcmul(x, gate.unsqueeze(1), self.linear2_attn(attn) + mlp)


class MMDiTStack(nn.Module):
    def __init__(self, cfg: MMDiTConfig, device, make_linear, seed: int = 0):
        super().__init__()
        gen = torch.Generator(device=device).manual_seed(seed)
        self.cfg = cfg
        self.double_stream = nn.ModuleList([DoubleBlock(cfg, device, gen, make_linear) for _ in range(cfg.double_blocks)])
        self.single_stream = nn.ModuleList([SingleBlock(cfg, device, gen, make_linear) for _ in range(cfg.single_blocks)])

    def forward(self, img, txt, vec):
        for blk in self.double_stream:
            img, txt = blk(img, txt, vec)
        x = torch.cat([txt, img], dim=1)
        for blk in self.single_stream:
            x = blk(x, vec)
        return x[:, txt.shape[1]:]


def calibrate_hidden_scales(model: nn.Module, img, txt, vec) -> int:
    """One forward in which every fusable MLP records a static scale for its hidden tensor from the
    activations it sees (amax / 2688, what the dynamic path computes per call); later forwards then
    run those MLPs with GELU and the hidden tensor's quantization inside the first GEMM's epilogue.
    Returns the number of MLPs switched."""
    from comfy_kitchen.modules import NVFP4MLP
    mlps = [m for m in model.modules() if isinstance(m, NVFP4MLP)]
    hooks = [m.register_forward_pre_hook(lambda mod, args: (mod.calibrate(args[0]), None)[1]) for m in mlps]
    try:
        with torch.inference_mode():
            model(img, txt, vec)
    finally:
        for h in hooks:
            h.remove()
    return sum(1 for m in mlps if m.fusable())


def make_inputs(cfg: MMDiTConfig, batch: int, device, seed: int = 0):
    gen = torch.Generator(device=device).manual_seed(seed + 1)
    kw = dict(device=device, generator=gen)
    img = torch.randn(batch, cfg.img_tokens, cfg.hidden, **kw).to(torch.bfloat16)
    txt = torch.randn(batch, cfg.txt_tokens, cfg.hidden, **kw).to(torch.bfloat16)
    vec = torch.randn(batch, cfg.hidden, **kw).to(torch.bfloat16)
    return img, txt, vec
