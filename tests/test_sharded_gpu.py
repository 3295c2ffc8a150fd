"""Column-sharded GEMM with the all-gather fused into the epilogue.

Single-GPU cases drive the multi-destination / strided store path of the kernel with all
destinations on one device; the two-GPU case (skipped on a one-GPU machine) runs one process
per GPU over NCCL with peer-mapped result buffers and compares with the unsharded GEMM.
"""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def ck(cuda_device):
    import comfy_kitchen

    info = comfy_kitchen.list_backends()["cuda"]
    assert info["available"], f"cuda backend not loaded: {info['unavailable_reason']}"
    return comfy_kitchen


def _operands(m, n, k, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    bias = (torch.randn(n, generator=g) * 0.01).bfloat16()
    return x, w, bias


@pytest.mark.parametrize("shape", [(256, 512, 256), (4096, 1024, 512), (300, 768, 320)])
@pytest.mark.parametrize("kind", ["nvfp4", "mxfp8"])
def test_two_destinations_on_one_gpu(ck, cuda_device, shape, kind):
    """world = 2 emulated on one device: each 'rank' stores its column block into both result
    matrices; both must equal the unsharded GEMM bit for bit, and columns outside a rank's block
    must stay untouched by it."""
    from comfy_kitchen import sharded
    from comfy_kitchen.backends import cuda as backend

    m, n, k = shape
    x, w, bias = _operands(m, n, k, seed=m + n + k)
    x, w, bias = x.to(cuda_device), w.to(cuda_device), bias.to(cuda_device)
    if kind == "nvfp4":
        sx = (x.abs().amax() / 2688).float()
        sw = (w.abs().amax() / 2688).float()
        qx, bsx = ck.quantize_nvfp4(x, sx, pad_16x=(m % 16 != 0))
        qw, bsw = ck.quantize_nvfp4(w, sw)
        full = ck.scaled_mm_nvfp4(qx, qw, sx, sw, bsx, bsw, bias=bias, out_dtype=torch.bfloat16)
    else:
        qx, bsx = ck.quantize_mxfp8(x, pad_32x=(m % 32 != 0))
        qw, bsw = ck.quantize_mxfp8(w)
        full = ck.scaled_mm_mxfp8(qx, qw, bsx, bsw, bias=bias, out_dtype=torch.bfloat16)
    mp = qx.shape[0]
    outs = [torch.full((mp, n), 7.0, dtype=torch.bfloat16, device=cuda_device) for _ in range(2)]
    ptrs = [o.data_ptr() for o in outs]
    for rank in range(2):
        shard = sharded.ShardedQuantizedWeight.from_full(qw, bsw, sw if kind == "nvfp4" else None, bias, 2, rank)
        if kind == "nvfp4":
            backend.scaled_mm_nvfp4_allgather(qx, shard.qdata, sx, shard.tensor_scale, bsx, shard.block_scale, ptrs, n,
                                              shard.start, bias=shard.bias)
        else:
            backend.scaled_mm_mxfp8_allgather(qx, shard.qdata, bsx, shard.block_scale, ptrs, n, shard.start, bias=shard.bias)
        if rank == 0:
            torch.cuda.synchronize()
            for o in outs:  # the other rank's columns are still the fill value
                assert torch.all(o[:, shard.end:] == 7.0)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o.view(torch.int16), full.view(torch.int16))


def test_peer_barrier_single_rank_and_timeout_status(ck, cuda_device):
    """world = 1 passes at once; a barrier whose partner never signals gives up after its bounded wait
    and reports the missing rank instead of hanging (the context stays usable)."""
    from comfy_kitchen.backends import cuda as backend

    flags = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    backend.peer_barrier([flags.data_ptr()], 0, 1, cuda_device)
    assert backend.peer_status() == 0
    assert int(flags[0].item()) == 1
    # two "ranks" whose flag arrays live on this device; rank 1 never launches
    f0 = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    f1 = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    backend.peer_barrier([f0.data_ptr(), f1.data_ptr()], 0, 1, cuda_device)
    assert backend.peer_status() == 2  # 1 + rank 1
    assert int(f1[0].item()) == 1      # rank 0's own signal did reach rank 1's array
    x = torch.ones(4, device=cuda_device)
    assert float((x + 1).sum().item()) == 8.0


def _two_gpu_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    sys.path.insert(0, os.path.join(ROOT, "comfy-kitchen_b200"))
    import torch.distributed as dist

    import comfy_kitchen as ck
    from comfy_kitchen import sharded
    from comfy_kitchen.backends import cuda as backend

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        m, n, k = 2048, 3072, 1024
        x, w, bias = _operands(m, n, k, seed=11)
        x, w, bias = x.to(dev), w.to(dev), bias.to(dev)
        sx = (x.abs().amax() / 2688).float()
        sw = (w.abs().amax() / 2688).float()
        qx, bsx = ck.quantize_nvfp4(x, sx)
        qw, bsw = ck.quantize_nvfp4(w, sw)
        full = ck.scaled_mm_nvfp4(qx, qw, sx, sw, bsx, bsw, bias=bias, out_dtype=torch.bfloat16)
        shard = sharded.ShardedQuantizedWeight.from_full(qw, bsw, sw, bias, world, rank)
        peers = sharded.PeerOutput(m, n, torch.bfloat16, dev)
        ok = True
        for it in range(3):
            y = sharded.sharded_linear_nvfp4_fused(qx, sx, bsx, shard, peers)
            ok = ok and bool(torch.equal(y.view(torch.int16), full.view(torch.int16)))
        # the NCCL path gives the same matrix
        y2 = sharded.sharded_linear_nvfp4(qx, sx, bsx, shard)
        ok = ok and bool(torch.equal(y2.view(torch.int16), full.view(torch.int16)))
        status = backend.peer_status()
        results[rank] = (ok, status)
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_allgather_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = 29500 + (os.getpid() % 2000)
        procs = [ctx.Process(target=_two_gpu_worker, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("a rank did not finish in time")
            assert p.exitcode == 0
        for r in range(world):
            ok, status = results[r]
            assert ok, f"rank {r}: sharded result differs from the unsharded GEMM"
            assert status == 0, f"rank {r}: barrier status {status}"
