"""Offline weight quantizer: turn the dense linear weights of a checkpoint into the keys the
quantized layers load.

    python comfy-kitchen_b200/quantize_checkpoint.py IN.pt OUT.pt [--layout nvfp4|mxfp8]
        [--min-features 64] [--skip PATTERN ...] [--only KEY ...] [--device cuda:0] [--dry-run]

IN is a ``torch.save``d state dict (or a dict holding one under ``state_dict`` / ``model``).  Every
2-D floating-point ``*.weight`` whose dimensions are at least ``--min-features`` and whose input
dimension is a multiple of the layout's block (16 / 32) is replaced by

    <name>            packed E2M1 codes (uint8)           | E4M3 bytes (MXFP8)
    <name>_scale      block scales in the tiled layout (uint8 bytes)
    <name>_scale_2    fp32 per-tensor scale (NVFP4 only)

which is what ``comfy_kitchen.modules.NVFP4Linear`` / ``MXFP8Linear`` load, and the key set the
reference's sample layer reads (samples/nvfp4_linear.py:39-74).  The quantization runs the
library's kernels, so it needs the GPU; ``--dry-run`` only lists what would be converted (no GPU,
no output file).
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def select_keys(state_dict: dict, block: int, min_features: int, skip: list[str], only: list[str] | None) -> list[str]:
    """Names of the entries that will be quantized, in checkpoint order."""
    import torch

    if only:
        missing = [k for k in only if k not in state_dict]
        if missing:
            raise KeyError(f"not in the checkpoint: {missing}")
        return list(only)
    keys = []
    for k, v in state_dict.items():
        if not (k.endswith("weight") and isinstance(v, torch.Tensor) and v.dim() == 2 and v.is_floating_point()):
            continue
        if min(v.shape) < min_features or v.shape[1] % block != 0 or any(p in k for p in skip):
            continue
        keys.append(k)
    return keys


def unwrap(obj):
    """The state dict inside what ``torch.load`` returned, and a function that puts a new one back."""
    for name in ("state_dict", "model"):
        if isinstance(obj, dict) and isinstance(obj.get(name), dict):
            def put(new, _obj=obj, _name=name):
                out = dict(_obj)
                out[_name] = new
                return out
            return obj[name], put
    return obj, (lambda new: new)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("src")
    ap.add_argument("dst", nargs="?")
    ap.add_argument("--layout", default="nvfp4", choices=["nvfp4", "mxfp8"])
    ap.add_argument("--min-features", type=int, default=64)
    ap.add_argument("--skip", nargs="*", default=[], help="substrings of names to leave dense")
    ap.add_argument("--only", nargs="*", default=None, help="exact names to quantize (overrides the rules)")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    import torch

    loaded = torch.load(a.src, map_location="cpu", weights_only=True)
    sd, put_back = unwrap(loaded)
    block = 16 if a.layout == "nvfp4" else 32
    keys = select_keys(sd, block, a.min_features, a.skip, a.only)
    dense = sum(sd[k].numel() * sd[k].element_size() for k in keys)
    per_elem = 0.5625 if a.layout == "nvfp4" else 1.03125
    print(f"{len(keys)} of {len(sd)} entries -> {a.layout}: {dense / 1e6:.1f} MB dense, "
          f"~{sum(sd[k].numel() for k in keys) * per_elem / 1e6:.1f} MB quantized")
    for k in keys:
        print(f"  {k} {tuple(sd[k].shape)} {sd[k].dtype}")
    if a.dry_run:
        return 0
    if not a.dst:
        ap.error("an output path is needed unless --dry-run is given")
    from comfy_kitchen.modules import quantize_state_dict

    out = quantize_state_dict(sd, layout=a.layout, device=a.device, keys=keys)
    torch.save(put_back(out), a.dst)
    print(f"wrote {a.dst}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
