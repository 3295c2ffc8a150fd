"""Host logic of the column-sharded linear, exercised with two gloo ranks on CPU.

The local GEMM is replaced by the oracle's dequantize -> fp32 matmul (tests may use the
oracle); what is under test is the shard arithmetic, the slicing of the tiled scale
tensor and the reassembly of the all-gathered column blocks.
"""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from comfy_kitchen import sharded


def test_shard_bounds():
    assert sharded.shard_bounds(3072, 8, 0) == (0, 384)
    assert sharded.shard_bounds(3072, 8, 7) == (2688, 3072)
    assert sharded.shard_bounds(15360, 8, 3) == (5760, 7680)
    for n in (3072, 12288, 15360):
        for g in (1, 2, 4, 8):
            spans = [sharded.shard_bounds(n, g, r) for r in range(g)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(s % 128 == 0 and e % 128 == 0 for s, e in spans)
    with pytest.raises(ValueError):
        sharded.shard_bounds(3072 + 128, 8, 0)
    with pytest.raises(ValueError):
        sharded.shard_bounds(1024, 4, 4)


def test_scale_slices_are_valid_tiled_tensors():
    from oracle import ck_oracle as oc

    rng = np.random.default_rng(0)
    logical = rng.integers(0, 255, size=(512, 12), dtype=np.uint8)
    blocked = torch.from_numpy(oc.to_blocked(logical))
    for start, end in ((0, 256), (256, 512), (128, 256)):
        piece = sharded.slice_block_scales(blocked, start, end).contiguous().numpy()
        np.testing.assert_array_equal(piece, oc.to_blocked(logical[start:end]))
    with pytest.raises(ValueError):
        sharded.slice_block_scales(blocked, 64, 256)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    from oracle import ck_oracle as oc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        m, n, k = 48, 512, 128
        x = torch.randn(m, k, generator=g).bfloat16()
        w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
        bias = torch.randn(n, generator=g).bfloat16()
        sx = np.float32((x.abs().amax() / 2688.0).float().item())
        sw = np.float32((w.abs().amax() / 2688.0).float().item())
        qx, bsx = oc.quantize_nvfp4(x.float().numpy(), sx)
        qw, bsw = oc.quantize_nvfp4(w.float().numpy(), sw)

        def local_mm(a, b, tsa, tsb, bsa, bsb, bias=None, out_dtype=None):
            y = oc.scaled_mm_nvfp4(a.numpy(), b.numpy(), np.float32(tsa.item()), np.float32(tsb.item()), bsa.numpy(),
                                   bsb.numpy(), bias=None if bias is None else bias.float().numpy())
            return torch.from_numpy(y)

        shard = sharded.ShardedQuantizedWeight.from_full(torch.from_numpy(qw), torch.from_numpy(bsw), torch.tensor(sw),
                                                         bias, world, rank)
        assert shard.qdata.shape[0] == n // world and shard.block_scale.shape[0] == n // world
        y = sharded.sharded_linear_nvfp4(torch.from_numpy(qx), torch.tensor(sx), torch.from_numpy(bsx), shard,
                                         out_dtype=torch.float32, local_mm=local_mm)
        full = oc.scaled_mm_nvfp4(qx, qw, sx, sw, bsx, bsw, bias=bias.float().numpy())
        np.testing.assert_allclose(y.numpy(), full, rtol=1e-5, atol=1e-5)
        # M == 1 takes the copy-free branch
        y1 = sharded.gather_columns(torch.full((1, 4), float(rank)), 4 * world)
        assert y1.tolist() == [[float(r) for r in range(world) for _ in range(4)]]
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_linear_matches_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
