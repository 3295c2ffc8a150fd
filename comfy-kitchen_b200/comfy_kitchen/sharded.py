"""Column-sharded quantized linear across the GPUs of one node.

The reference has no multi-device code.  The quantized-linear path shards in one natural
way for a single large GEMM: the output columns (rows of the weight) are independent, so
rank r of g keeps ``W[r*N/g : (r+1)*N/g, :]`` - packed codes, its own tiled block-scale
tensor and its bias slice - computes ``y[:, shard]`` from the full (replicated) quantized
activation, and the shards are put together with one all-gather over NVLink.  Shard
boundaries fall on multiples of 128 weight rows so that each shard's block scales are whole
tiles of the 128x4 layout.

One process per GPU (``torch.distributed``, backend ``nccl``; ``gloo`` works for the host
logic on CPU).  Nothing here computes: the local GEMM is ``comfy_kitchen.scaled_mm_*`` (or a
caller-supplied function with the same meaning), the exchange is
``all_gather_into_tensor``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist

from .float_utils import roundup

SHARD_GRANULE = 128  # weight rows per scale tile


def shard_bounds(n: int, world: int, rank: int, granule: int = SHARD_GRANULE) -> tuple[int, int]:
    """[start, end) of the weight rows rank ``rank`` owns: equal shards, every boundary a multiple of ``granule``.

    Raises ValueError when ``n`` does not split that way (the caller pads N or uses fewer ranks).
    """
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % (world * granule) != 0:
        raise ValueError(f"N={n} does not split into {world} shards of whole {granule}-row scale tiles")
    per = n // world
    return rank * per, (rank + 1) * per


def slice_block_scales(block_scales: torch.Tensor, start: int, end: int) -> torch.Tensor:
    """Rows [start, end) of a tiled scale tensor [roundup(N,128), C]; both bounds multiples of 128.

    In the tiled layout a 128-row group is a contiguous run of ``C/4`` 512-byte tiles, so the
    slice is a contiguous view that is itself a valid tiled tensor for the shard.
    """
    if start % SHARD_GRANULE or end % SHARD_GRANULE:
        raise ValueError("scale tensors can only be cut at multiples of 128 rows")
    return block_scales[start:end]


@dataclass
class ShardedQuantizedWeight:
    """This rank's slice of a quantized [N, K] weight."""

    qdata: torch.Tensor          # [N/g, K/2] uint8 (NVFP4) or [N/g, K] float8_e4m3fn (MXFP8)
    block_scale: torch.Tensor    # tiled scales of the shard
    tensor_scale: torch.Tensor | None   # fp32 per-tensor scale (NVFP4), None for MXFP8
    bias: torch.Tensor | None    # [N/g] or None
    n_total: int
    start: int
    end: int

    @classmethod
    def from_full(cls, qdata, block_scale, tensor_scale, bias, world: int, rank: int) -> "ShardedQuantizedWeight":
        """Cut rank ``rank``'s shard out of a fully quantized weight (all ranks hold the same full tensors)."""
        n = qdata.shape[0]
        start, end = shard_bounds(n, world, rank)
        return cls(qdata=qdata[start:end].contiguous(),
                   block_scale=slice_block_scales(block_scale, start, end).contiguous(),
                   tensor_scale=tensor_scale, bias=None if bias is None else bias[start:end].contiguous(),
                   n_total=n, start=start, end=end)


def gather_columns(local: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """All-gather the [M, N/g] column blocks of every rank into the full [M, N] matrix (on every rank).

    The collective fills a [g, M, N/g] buffer (rank-major, what NCCL produces without extra
    copies on its side); one permute-copy lays it out as [M, N].  For M == 1 the buffer
    already is the result.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local
    m, n_local = local.shape
    if n_local * world != n_total:
        raise ValueError(f"shards of {n_local} columns on {world} ranks do not make {n_total}")
    staged = torch.empty((world, m, n_local), dtype=local.dtype, device=local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(staged, local.contiguous(), group=group)
    else:  # gloo (CPU tests of the host logic) has no flat all-gather
        dist.all_gather([staged[r] for r in range(world)], local.contiguous(), group=group)
    if m == 1:
        return staged.reshape(1, n_total)
    return staged.permute(1, 0, 2).reshape(m, n_total)


def sharded_linear_nvfp4(qx: torch.Tensor, x_scale: torch.Tensor, x_block_scale: torch.Tensor,
                         weight: ShardedQuantizedWeight, out_dtype: torch.dtype = torch.bfloat16, group=None,
                         local_mm: Callable | None = None, gather: bool = True) -> torch.Tensor:
    """y[M, N] = linear(x, W) with W column-sharded: local NVFP4 GEMM on this rank's shard, then all-gather.

    ``qx`` / ``x_block_scale`` / ``x_scale`` are the full quantized activation (identical on every
    rank).  ``local_mm`` defaults to ``comfy_kitchen.scaled_mm_nvfp4``; ``gather=False`` returns
    the local [M, N/g] block (GEMM-only timing).
    """
    if local_mm is None:
        import comfy_kitchen as ck

        local_mm = ck.scaled_mm_nvfp4
    y_local = local_mm(qx, weight.qdata, x_scale, weight.tensor_scale, x_block_scale, weight.block_scale,
                       bias=weight.bias, out_dtype=out_dtype)
    return gather_columns(y_local, weight.n_total, group) if gather else y_local


def sharded_linear_mxfp8(qx: torch.Tensor, x_block_scale: torch.Tensor, weight: ShardedQuantizedWeight,
                         out_dtype: torch.dtype = torch.bfloat16, group=None, local_mm: Callable | None = None,
                         gather: bool = True) -> torch.Tensor:
    """MXFP8 counterpart of :func:`sharded_linear_nvfp4`."""
    if local_mm is None:
        import comfy_kitchen as ck

        local_mm = ck.scaled_mm_mxfp8
    y_local = local_mm(qx, weight.qdata, x_block_scale, weight.block_scale, bias=weight.bias, out_dtype=out_dtype)
    return gather_columns(y_local, weight.n_total, group) if gather else y_local


class PeerOutput:
    """Result buffers [M, N] of every rank, mapped into every process, for the GEMM whose epilogue
    does the all-gather itself.

    Allocation goes through ``torch.distributed._symmetric_memory`` (one process per GPU, NCCL
    group): ``buffers`` result matrices used round-robin plus one array of barrier flags.  A
    result may be read after :meth:`barrier` has run behind the GEMM on the same stream; with two
    or more buffers a rank can still be reading result i while its peers already write result
    i + 1.  Multicast mappings are not needed (all stores are plain peer stores).

    The barrier's wait is bounded (about a second; ``first_barrier_seconds`` for the first one,
    when ranks can be far apart because of module loading and first-call set-up).  A barrier that
    gave up leaves a partly written result and an error status on the device, nothing else:
    **a result is valid only if** :meth:`check` **passes** - call it wherever the host reads
    results or at the end of a step (it synchronises the device).
    """

    def __init__(self, m: int, n_total: int, dtype: torch.dtype, device, group=None, buffers: int = 2,
                 first_barrier_seconds: float = 20.0):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.m, self.n_total, self.dtype, self.device = m, n_total, dtype, device
        self.tensors, self.ptrs, self._handles = [], [], []
        for _ in range(buffers):
            t = symm.empty((m, n_total), dtype=dtype, device=device)
            h = symm.rendezvous(t, self.group)
            self.tensors.append(t)
            self.ptrs.append([int(p) for p in h.buffer_ptrs])
            self._handles.append(h)
        self.flags = symm.empty((64,), dtype=torch.int32, device=device)
        self.flags.zero_()
        fh = symm.rendezvous(self.flags, self.group)
        self._handles.append(fh)
        self.flag_ptrs = [int(p) for p in fh.buffer_ptrs]
        self.epoch = 0
        self.turn = 0
        self._first_polls = max(1, min(1 << 26, int(first_barrier_seconds * 2e6)))  # ~0.5 us per poll
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # every rank's flags are zero before anyone signals

    def next_buffer(self) -> tuple[torch.Tensor, list[int]]:
        i = self.turn % len(self.tensors)
        self.turn += 1
        return self.tensors[i], self.ptrs[i]

    def barrier(self) -> None:
        """Launch the bounded cross-GPU barrier on the current stream."""
        from .backends import cuda as backend

        self.epoch += 1
        backend.peer_barrier(self.flag_ptrs, self.rank, self.epoch, self.device,
                             max_polls=self._first_polls if self.epoch == 1 else None)

    def check(self) -> None:
        """Synchronise the device and raise RuntimeError if any barrier (or GEMM wait) since the
        last check gave up - the results produced in between are then incomplete."""
        from .backends import cuda as backend

        backend.check_device_status("sharded linear with fused all-gather")


def sharded_linear_nvfp4_fused(qx: torch.Tensor, x_scale: torch.Tensor, x_block_scale: torch.Tensor,
                               weight: ShardedQuantizedWeight, peers: PeerOutput,
                               out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """y[M, N] = linear(x, W), W column-sharded, with the all-gather done by the GEMM epilogue: every
    output tile is stored straight into all ranks' result buffers over NVLink while the tensor cores
    work on the next tile, followed by one cross-GPU barrier.  Returns this rank's full [M, N] result
    (a view of one of ``peers``' buffers, valid in stream order)."""
    from .backends import cuda as backend

    out, ptrs = peers.next_buffer()
    backend.scaled_mm_nvfp4_allgather(qx, weight.qdata, x_scale, weight.tensor_scale, x_block_scale, weight.block_scale,
                                      ptrs, weight.n_total, weight.start, bias=weight.bias, out_dtype=out_dtype)
    peers.barrier()
    return out


def sharded_linear_mxfp8_fused(qx: torch.Tensor, x_block_scale: torch.Tensor, weight: ShardedQuantizedWeight,
                               peers: PeerOutput, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """MXFP8 counterpart of :func:`sharded_linear_nvfp4_fused`."""
    from .backends import cuda as backend

    out, ptrs = peers.next_buffer()
    backend.scaled_mm_mxfp8_allgather(qx, weight.qdata, x_block_scale, weight.block_scale, ptrs, weight.n_total,
                                      weight.start, bias=weight.bias, out_dtype=out_dtype)
    peers.barrier()
    return out


def padded_scale_rows(n: int) -> int:
    return roundup(n, SHARD_GRANULE)
