#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--case CASE]

One *step* is one NVFP4 linear of the single-DiT-projection workload
(x bf16 [4096,3072] with 0.1 % x20 outliers, W bf16 [3072,3072] ~N(0,0.02)
pre-quantized, bias bf16): ``quantize_nvfp4(x)`` followed by ``scaled_mm_nvfp4`` with
bias into a bf16 [4096,3072] output.  ``value`` is 2*M*N*K / step time in TFLOP/s with
the inputs resident in HBM; every step uses a different x / W / output buffer out of a
ring whose total size exceeds the L2 cache.  With --gpus N (launched under torchrun) each
rank runs the same step on its own data (the batch shards data-parallel, no collective
on the data path), and the value is the aggregate over ranks.

Other cases time one kernel alone (used for profiling and the per-kernel rooflines):
quantize_nvfp4, quantize_mxfp8, dequantize_nvfp4, dequantize_mxfp8, tensor_scale, gemm_nvfp4,
gemm_mxfp8, linear_mxfp8; or another workload: mlp_pair (fc1 + GELU + re-quantize + fc2),
sharded_gemm (N column-sharded over the ranks, fused all-gather vs NCCL), mmdit (full-model
harness, batch split over the ranks).

The JSON line also carries: ``e2e`` (the same step through the public Python API with
host buffers: pinned-host x -> device, linear, bf16 result -> host), ``roofline`` for the
dominant kernel (the GEMM), ``roofline_quantize``, ``cpu_baseline`` (the CPU oracle of the
same path timed on the host cores, rank 0 of a one-GPU run only), ``clocks`` sampled during the timed region, and
``gpu_launches``.

--impl reference times the CPU restatement of the reference's eager path (oracle/) on the
host cores for the same metric.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "comfy-kitchen_b200"))
sys.path.insert(0, ROOT)

M, N, K = 4096, 3072, 3072
WORKLOAD = "single DiT projection: x bf16 [4096,3072] ~N(0,1) + 0.1% x20 outliers, W bf16 [3072,3072] ~N(0,0.02), bias bf16; NVFP4 quantize(x) + scaled_mm + bias -> bf16"
METRIC = "nvfp4_linear_tflops"
NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_FP8_TFLOPS = 4500.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------------------------
# clocks sampling
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._proc = None
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        # one long-running nvidia-smi that prints a row every 50 ms
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                           "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                          stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        for raw in self._proc.stdout:
            row = [c.strip() for c in raw.strip().split(",")]
            if len(row) == 6:
                self.samples.append(row)
            if self._stop.is_set():
                break

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        proc = getattr(self, "_proc", None)
        if proc is not None:
            proc.terminate()  # the exact child this object started
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(float(s[0])) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(float(self.samples[0][1])), "reasons": reasons,
                "samples": len(mhz)}


# --------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's eager path, timed on the host
# --------------------------------------------------------------------------------------------
def cpu_linear_once(rows: int, seed: int = 0) -> tuple[float, int, str]:
    """One NVFP4 linear on `rows` rows of the workload through the CPU oracle: the C restatement
    (OpenMP row loops) when it could be built, else the numpy one; the float32 matmul of the GEMM
    contract is BLAS either way.  Returns (seconds, rows, which)."""
    import numpy as np
    import torch

    from oracle import ck_oracle as oc
    from oracle import ck_oracle_c as occ

    impl, which = (occ, "C/OpenMP oracle") if occ.available() else (oc, "numpy oracle")
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(rows, K, generator=g)
    x = torch.where(torch.rand(rows, K, generator=g) < 0.001, x * 20, x).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.01).bfloat16().float().numpy()
    sx = np.float32((x.abs().amax() / 2688.0).float().item())
    sw = np.float32((w.abs().amax() / 2688.0).float().item())
    xf, wf = x.float().numpy(), w.float().numpy()
    qw, bsw = impl.quantize_nvfp4(wf, sw)  # weights are pre-quantized: not timed
    t0 = time.perf_counter()
    qx, bsx = impl.quantize_nvfp4(xf, sx)
    out = impl.scaled_mm_nvfp4(qx, qw, sx, sw, bsx, bsw, bias=bias)
    impl.f32_to_bf16_bits(out)
    return time.perf_counter() - t0, rows, which


def cpu_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference_arm(args) -> dict:
    """--impl reference: the CPU port of the reference's eager path, all host threads, bounded sample per step."""
    import torch

    torch.set_num_threads(cpu_threads())
    rows = 1024  # bounded sample of the 4096-row workload per step
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_linear_once(rows)
    times = []
    which = ""
    for _ in range(args.steps):
        dt, _, which = cpu_linear_once(rows)
        times.append(dt)
    per_step = sum(times) / len(times)
    tflops = 2.0 * rows * N * K / per_step / 1e12
    sample = f"{rows} of {M} rows per step (quantize_nvfp4(x) + dequantize->fp32 matmul + bias -> bf16), {which}, BLAS matmul"
    return {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": M, "N": N, "K": K},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
class Workload:
    """Device buffers of the step, as a ring of `ring` independent (x, W, out) sets."""

    def __init__(self, torch, ck, device, rows: int, ring: int, seed: int):
        self.torch, self.rows, self.ring, self.device = torch, rows, ring, device
        g = torch.Generator(device="cpu").manual_seed(seed)
        x = torch.randn(rows, K, generator=g)
        x = torch.where(torch.rand(rows, K, generator=g) < 0.001, x * 20, x).bfloat16()
        w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
        self.bias = (torch.randn(N, generator=g) * 0.01).bfloat16().to(device)
        self.x_host = x.pin_memory()
        self.x = [x.to(device) if i == 0 else torch.roll(x, i, 0).to(device) for i in range(ring)]
        self.sx = (x.abs().amax() / 2688.0).float().to(device).reshape(1)
        self.sw = (w.abs().amax() / 2688.0).float().to(device).reshape(1)
        wd = w.to(device)
        self.w_bf16 = wd
        # pre-quantized weights, `ring` copies so that successive steps do not share L2 lines
        qw, bsw = ck.quantize_nvfp4(wd, self.sw)
        self.qw = [qw.clone() for _ in range(ring)]
        self.bsw = [bsw.view(torch.uint8).clone() for _ in range(ring)]
        qw8, bsw8 = ck.quantize_mxfp8(wd)
        self.qw8 = [qw8.view(torch.uint8).clone() for _ in range(ring)]
        self.bsw8 = [bsw8.view(torch.uint8).clone() for _ in range(ring)]
        u8 = dict(dtype=torch.uint8, device=device)
        rp = (rows + 127) // 128 * 128
        self.qx = [torch.empty(rows, K // 2, **u8) for _ in range(ring)]
        self.bsx = [torch.empty(rp, K // 16, **u8) for _ in range(ring)]
        self.qx8 = [torch.empty(rows, K, **u8) for _ in range(ring)]
        self.bsx8 = [torch.empty(rp, K // 32, **u8) for _ in range(ring)]
        self.out = [torch.empty(rows, N, dtype=torch.bfloat16, device=device) for _ in range(ring)]
        self.dyn_scale = torch.empty((), dtype=torch.float32, device=device)
        self.scale_scratch = torch.zeros(1 << 20, dtype=torch.uint8, device=device)

    def ring_bytes(self) -> int:
        per = self.x[0].numel() * 2 + self.qw[0].numel() + self.bsw[0].numel() + self.out[0].numel() * 2 + \
            self.qx[0].numel() + self.bsx[0].numel()
        return per * self.ring


def _tensor_scale(lib, wl, i, st):
    j = i % wl.ring
    rc = lib.ck_nvfp4_tensor_scale(wl.x[j].data_ptr(), 2, wl.rows * K, wl.dyn_scale.data_ptr(), wl.scale_scratch.data_ptr(),
                                   wl.scale_scratch.numel(), st)
    assert rc == 0, lib.ck_last_error()


def make_steps(lib, wl: Workload, case: str):
    """Returns (launch(i, stream) -> None, kernels per step, flops per step, algorithmic bytes per step)."""
    rows = wl.rows
    p = lambda t: t.data_ptr()  # noqa: E731
    flops = 2.0 * rows * N * K
    q4_bytes = 2 * rows * K + rows * K // 2 + ((rows + 127) // 128 * 128) * (K // 16) + 4
    q8_bytes = 2 * rows * K + rows * K + ((rows + 127) // 128 * 128) * (K // 32)

    def q4(i, st):
        j = i % wl.ring
        rc = lib.ck_quantize_nvfp4(p(wl.x[j]), 2, p(wl.sx), p(wl.qx[j]), p(wl.bsx[j]), rows, K, rows, K, 1, st)
        assert rc == 0, lib.ck_last_error()

    def q8(i, st):
        j = i % wl.ring
        rc = lib.ck_quantize_mxfp8(p(wl.x[j]), 2, p(wl.qx8[j]), p(wl.bsx8[j]), rows, K, rows, K, st)
        assert rc == 0, lib.ck_last_error()

    def g4(i, st):
        j = i % wl.ring
        rc = lib.ck_scaled_mm_nvfp4(p(wl.qx[j]), p(wl.qw[j]), p(wl.bsx[j]), p(wl.bsw[j]), p(wl.sx), p(wl.sw), None,
                                    p(wl.bias), 2, p(wl.out[j]), 2, rows, N, K, st)
        assert rc == 0, lib.ck_last_error()

    def g8(i, st):
        j = i % wl.ring
        rc = lib.ck_scaled_mm_mxfp8(p(wl.qx8[j]), p(wl.qw8[j]), p(wl.bsx8[j]), p(wl.bsw8[j]), p(wl.bias), 2,
                                    p(wl.out[j]), 2, rows, N, K, st)
        assert rc == 0, lib.ck_last_error()

    dq4_bytes = rows * K // 2 + ((rows + 127) // 128 * 128) * (K // 16) + 4 + 2 * rows * K
    dq8_bytes = rows * K + ((rows + 127) // 128 * 128) * (K // 32) + 2 * rows * K

    def dq4(i, st):  # dequantizes what q4 of the same ring slot produced, into the x buffer of the next slot
        j = i % wl.ring
        rc = lib.ck_dequantize_nvfp4(p(wl.qx[j]), p(wl.sx), p(wl.bsx[j]), p(wl.deq[j]), 2, rows, K, 1, st)
        assert rc == 0, lib.ck_last_error()

    def dq8(i, st):
        j = i % wl.ring
        rc = lib.ck_dequantize_mxfp8(p(wl.qx8[j]), p(wl.bsx8[j]), p(wl.deq[j]), 2, rows, K, st)
        assert rc == 0, lib.ck_last_error()

    if case.startswith("dequantize"):
        wl.deq = [wl.torch.empty(rows, K, dtype=wl.torch.bfloat16, device=wl.device) for _ in range(wl.ring)]
        for j in range(wl.ring):  # operands of the timed kernel
            (q4 if "nvfp4" in case else q8)(j, wl.torch.cuda.current_stream().cuda_stream)
        wl.torch.cuda.synchronize()

    table = {
        "dequantize_nvfp4": (dq4, 1, None, dq4_bytes),
        "dequantize_mxfp8": (dq8, 1, None, dq8_bytes),
        "linear": (lambda i, st: (q4(i, st), g4(i, st)), 2, flops, None),
        "linear_mxfp8": (lambda i, st: (q8(i, st), g8(i, st)), 2, flops, None),
        "tensor_scale": (lambda i, st: _tensor_scale(lib, wl, i, st), 1, None, 2 * rows * K + 4),
        "quantize_nvfp4": (q4, 1, None, q4_bytes),
        "quantize_mxfp8": (q8, 1, None, q8_bytes),
        "gemm_nvfp4": (g4, 1, flops, None),
        "gemm_mxfp8": (g8, 1, flops, None),
    }
    return table[case]


def time_steps(torch, launch, steps: int, warmup: int, use_graph: bool, dist=None) -> float:
    """Device time in ms of `steps` launches after `warmup`, CUDA events on the launch stream.

    With use_graph the steps are captured once into a CUDA graph (removes host launch
    gaps between the short kernels) and the timed region is one replay."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        st = stream.cuda_stream
        for i in range(warmup):
            launch(i, st)
        stream.synchronize()
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(steps):
                    launch(warmup + i, st)
            graph.replay()  # one untimed replay: graph upload
            stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record(stream)
        if use_graph:
            graph.replay()
        else:
            for i in range(steps):
                launch(warmup + i, st)
        e1.record(stream)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        return e0.elapsed_time(e1)


def run_e2e(torch, ck, wl: Workload, steps: int, warmup: int, dist=None) -> dict:
    """The step through the public API with host buffers: H2D of x, linear, D2H of the bf16 result.

    Every step does all three inside the timed region.  Steps are issued round-robin on three
    streams (each step stays in order on its own stream), so the copy of one step's input, the
    kernels of another and the read-back of a third overlap, as a serving loop would run them."""
    dev = wl.device
    qw, bsw = wl.qw[0], wl.bsw[0].view(torch.float8_e4m3fn)
    lanes = 3
    streams = [torch.cuda.Stream() for _ in range(lanes)]
    out_host = [torch.empty(wl.rows, N, dtype=torch.bfloat16).pin_memory() for _ in range(lanes)]

    def step(i):
        lane = i % lanes
        with torch.cuda.stream(streams[lane]):
            x = wl.x_host.to(dev, non_blocking=True)
            qx, bsx = ck.quantize_nvfp4(x, wl.sx)
            y = ck.scaled_mm_nvfp4(qx, qw, wl.sx, wl.sw, bsx, bsw, bias=wl.bias, out_dtype=torch.bfloat16)
            out_host[lane].copy_(y, non_blocking=True)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    main = torch.cuda.current_stream()
    e0.record(main)
    for st in streams:
        st.wait_event(e0)
    for i in range(steps):
        step(i)
    for st in streams:
        main.wait_stream(st)
    e1.record(main)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    return {"ms": ms, "h2d": wl.x_host.numel() * 2, "d2h": out_host[0].numel() * 2, "lanes": lanes}


def run_sharded_gemm(args, torch, ck, dist, device, rank, world, clocks_cls, local_rank) -> dict | None:
    """NVFP4 GEMM with N column-sharded over the ranks and an NCCL all-gather of the bf16 output.

    Strong scaling: the problem is fixed, each rank computes y[:, shard].  Two timings: the local
    GEMM alone (aggregate TFLOP/s scales with the ranks) and GEMM + all-gather (bounded by the
    NVLink bytes each rank receives: (g-1)/g * 2*M*N)."""
    from comfy_kitchen import sharded

    m, n, k = (int(v) for v in args.shape.split(","))
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(m, k, generator=g).bfloat16().to(device)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(device)
    sx = (x.abs().amax() / 2688.0).float()
    sw = (w.abs().amax() / 2688.0).float()
    qx, bsx = ck.quantize_nvfp4(x, sx)
    qw, bsw = ck.quantize_nvfp4(w, sw)
    shard = sharded.ShardedQuantizedWeight.from_full(qw, bsw, sw, None, world, rank)
    del w, qw, bsw

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # The fused path (epilogue stores into every rank's peer-mapped result + one barrier kernel)
    # needs torch's symmetric memory; when that is unavailable only the NCCL path is timed.
    peers, fused_error = None, None
    if dist is not None and world > 1:
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            peers = sharded.PeerOutput(m, n, torch.bfloat16, device, buffers=2)
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            fused_error = f"{type(e).__name__}: {e}"[:200]
    with clocks_cls(local_rank) as clocks:
        ms_gemm = timed(lambda: sharded.sharded_linear_nvfp4(qx, sx, bsx, shard, gather=False), args.steps, args.warmup)
        ms_nccl = timed(lambda: sharded.sharded_linear_nvfp4(qx, sx, bsx, shard), args.steps, args.warmup)
        ms_fused = None
        if peers is not None:
            ms_fused = timed(lambda: sharded.sharded_linear_nvfp4_fused(qx, sx, bsx, shard, peers), args.steps, args.warmup)
    y = sharded.sharded_linear_nvfp4(qx, sx, bsx, shard)
    y_local = sharded.sharded_linear_nvfp4(qx, sx, bsx, shard, gather=False)
    ok = bool(torch.equal(y[:, shard.start:shard.end], y_local)) and tuple(y.shape) == (m, n)
    fused_ok, barrier_status = None, None
    if peers is not None:
        from comfy_kitchen.backends import cuda as backend

        yf = sharded.sharded_linear_nvfp4_fused(qx, sx, bsx, shard, peers)
        fused_ok = bool(torch.equal(yf, y))
        barrier_status = backend.peer_status()
    ms_full = ms_fused if ms_fused is not None else ms_nccl
    if rank != 0:
        return None
    flops = 2.0 * m * n * k
    recv = (world - 1) / world * 2.0 * m * n
    return {
        "metric": "sharded_nvfp4_gemm_tflops", "value": flops / (ms_full * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_full, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"NVFP4 GEMM M={m} N={n} K={k}, N column-sharded over {world} GPUs, all-gather of the bf16 "
                               + ("output fused into the GEMM epilogue (peer stores over NVLink + barrier kernel)"
                                  if ms_fused is not None else "output by NCCL"),
                   "M": m, "N": n, "K": k},
        "gemm_only": {"ms": ms_gemm, "aggregate_tflops": flops / (ms_gemm * 1e-3) / 1e12},
        "nccl_all_gather": {"ms_gemm_plus_gather": ms_nccl, "tflops": flops / (ms_nccl * 1e-3) / 1e12,
                            "bytes_received_per_gpu": recv,
                            "gbs_per_gpu": (recv / ((ms_nccl - ms_gemm) * 1e-3) / 1e9) if ms_nccl > ms_gemm else None},
        "fused_all_gather": None if ms_fused is None else {
            "ms": ms_fused, "tflops": flops / (ms_fused * 1e-3) / 1e12, "equals_nccl_result": fused_ok,
            "barrier_status": barrier_status,
            # roofline of the fused kernel: the slower of tensor time and the bytes this GPU must push
            "nvlink_floor_ms": recv / 770.0e9 * 1e3, "nvlink_peak_gbs": 770.0,
            "frac_of_floor": max(recv / 770.0e9 * 1e3, ms_gemm) / ms_fused},
        "fused_unavailable": fused_error,
        "gathered_equals_local": ok, "clocks": clocks.summary(), "gpu_launches": args.steps * (2 if ms_fused is not None else 1),
    }


def run_mlp_pair(args, torch, ck, backend, device, clocks_cls, local_rank) -> dict:
    """DiT MLP pair: x [4608,3072] -> fc1 [12288,3072] -> GELU(tanh) -> NVFP4 -> fc2 [3072,12288] -> bf16.

    Pre-quantized NVFP4 weights; the hidden activation is re-quantized with a static
    (calibrated once) per-tensor scale.  Fused: quantize(x), fc1 with the GELU + re-quantize
    epilogue (no dense hidden is written), fc2.  Unfused: quantize(x), fc1, torch GELU,
    quantize(h), fc2 - the reference's sequence of kernels."""
    import torch.nn.functional as F

    m, d, hdim = (args.rows or 4608), 3072, 12288
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(m, d, generator=g).bfloat16().to(device)
    w1 = (torch.randn(hdim, d, generator=g) * 0.02).bfloat16().to(device)
    w2 = (torch.randn(d, hdim, generator=g) * 0.01).bfloat16().to(device)
    sx = (x.abs().amax() / 2688.0).float()
    s1 = (w1.abs().amax() / 2688.0).float()
    s2 = (w2.abs().amax() / 2688.0).float()
    q1, b1 = ck.quantize_nvfp4(w1, s1)
    q2, b2 = ck.quantize_nvfp4(w2, s2)
    del w1, w2
    # calibrate the hidden scale once from an unfused pass
    qx, bsx = ck.quantize_nvfp4(x, sx)
    h = F.gelu(ck.scaled_mm_nvfp4(qx, q1, sx, s1, bsx, b1), approximate="tanh")
    sh = (h.abs().amax() / 2688.0).float()
    del h

    def fused():
        qx, bsx = ck.quantize_nvfp4(x, sx)
        _, hc, hs = backend.linear_nvfp4_fused(qx, q1, sx, s1, bsx, b1, activation="gelu_tanh", requant_scale=sh,
                                               return_dense=False)
        return ck.scaled_mm_nvfp4(hc, q2, sh, s2, hs, b2)

    def unfused():
        qx, bsx = ck.quantize_nvfp4(x, sx)
        h = F.gelu(ck.scaled_mm_nvfp4(qx, q1, sx, s1, bsx, b1), approximate="tanh")
        hq, hqs = ck.quantize_nvfp4(h, sh)
        return ck.scaled_mm_nvfp4(hq, q2, sh, s2, hqs, b2)

    if args.case == "fc1_fused":
        # the fused kernel alone, launched from the host (profiling case)
        qx, bsx = ck.quantize_nvfp4(x, sx)

        def fc1():
            return backend.linear_nvfp4_fused(qx, q1, sx, s1, bsx, b1, activation="gelu_tanh", requant_scale=sh,
                                              return_dense=False)

        for _ in range(args.warmup):
            fc1()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fc1()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        fl = 2.0 * m * d * hdim
        return {"metric": "fc1_fused_tflops", "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
                "config": {"workload": f"fc1 of the DiT MLP pair with the GELU + NVFP4 re-quantize epilogue, M={m} N={hdim} K={d}",
                           "cuda_graph": False}, "gpu_launches": args.steps}

    def timed(fn):
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(args.warmup):
                fn()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(args.steps):
                    fn()
            graph.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.steps

    with clocks_cls(local_rank) as clocks:
        ms_fused = timed(fused)
        ms_unfused = timed(unfused)
    rel = float((fused().float() - unfused().float()).norm() / unfused().float().norm())
    flops = 2.0 * 2 * m * d * hdim
    return {
        "metric": "nvfp4_mlp_pair_tflops", "value": flops / (ms_fused * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_fused, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "DiT MLP pair: x [4608,3072] -> fc1 [12288,3072] + GELU-tanh + NVFP4 re-quantize in the epilogue -> fc2 [3072,12288] -> bf16",
                   "cuda_graph": True, "l2": "hidden activation (28 MB NVFP4) and weights (42 MB) exceed nothing: L2-resident between kernels, as in a real layer"},
        "unfused": {"ms_per_step": ms_unfused, "tflops": flops / (ms_unfused * 1e-3) / 1e12,
                    "sequence": "quantize, fc1, torch gelu, quantize, fc2"},
        "fused_vs_unfused_rel_diff": rel, "clocks": clocks.summary(), "gpu_launches": args.steps * 3,
    }


def run_gemm_sweep(args, torch, ck, device) -> dict:
    """NVFP4 GEMM over the sweep of config 4 on one GPU: M in {1, 16, 256, 4096, 16384} x
    (K, N) in {(3072, 3072), (3072, 12288), (12288, 3072), (3072, 15360)}, bf16 output, through
    ``ck.scaled_mm_nvfp4`` (split-K workspace path included), 20 launches per CUDA-graph replay,
    operands L2-resident where they fit."""
    rows = []
    gen = torch.Generator(device="cpu").manual_seed(0)
    for (k, n) in ((3072, 3072), (3072, 12288), (12288, 3072), (3072, 15360)):
        w = (torch.randn(n, k, generator=gen) * 0.02).bfloat16().to(device)
        sw = (w.abs().amax() / 2688.0).float()
        qw, bsw = ck.quantize_nvfp4(w, sw)
        del w
        for m in (1, 16, 256, 4096, 16384):
            x = torch.randn(m, k, generator=gen).bfloat16().to(device)
            sx = (x.abs().amax() / 2688.0).float()
            qx, bsx = ck.quantize_nvfp4(x, sx, pad_16x=(m % 16 != 0))

            def f():
                return ck.scaled_mm_nvfp4(qx, qw, sx, sw, bsx, bsw)

            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(3):
                    f()
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(20):
                        f()
                graph.replay()
                stream.synchronize()
                best = 1e9
                for _ in range(3):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    graph.replay()
                    e1.record(stream)
                    torch.cuda.synchronize()
                    best = min(best, e0.elapsed_time(e1) / 20)
            rows.append({"M": m, "N": n, "K": k, "us": best * 1e3, "tflops": 2.0 * m * n * k / (best * 1e-3) / 1e12})
    big = [r for r in rows if r["M"] >= 4096]
    return {"metric": "nvfp4_gemm_sweep_tflops", "value": sum(r["tflops"] for r in big) / len(big), "unit": "TFLOP/s",
            "n_gpus": 1, "steps": 20, "warmup": 3, "ms_per_step": sum(r["us"] for r in rows) * 1e-3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "NVFP4 GEMM sweep of config 4 on one GPU (value = mean TFLOP/s of the M >= 4096 shapes)"},
            "shapes": rows, "gpu_launches": 20 * len(rows)}


def run_mmdit(args, torch, dist, device, rank, world, clocks_cls, local_rank) -> dict | None:
    """Random-init MMDiT-shaped stack, every block linear through NVFP4 QuantizedTensors, batch 8 split
    data-parallel over the ranks (strong scaling, no collective inside the forward)."""
    import bench_mmdit as mm
    from comfy_kitchen.modules import NVFP4Linear

    cfg = mm.MMDiTConfig()
    if args.mmdit_blocks:
        d, s_ = (int(v) for v in args.mmdit_blocks.split(","))
        cfg.double_blocks, cfg.single_blocks = d, s_
    total_batch = args.mmdit_batch
    if total_batch % world != 0:
        raise SystemExit(f"--case mmdit splits a batch of {total_batch}: the GPU count must divide it")
    batch = total_batch // world
    use_graph = not args.no_graph
    with torch.inference_mode():
        model = mm.MMDiTStack(cfg, device, NVFP4Linear.from_linear, seed=0)
        img, txt, vec = mm.make_inputs(cfg, batch, device, seed=rank)
        steps, warmup = min(args.steps, 8), min(max(args.warmup, 1), 3)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                out = model(img, txt, vec)
            stream.synchronize()
            graph = None
            if use_graph:
                # static shapes: the whole forward (every kernel of the library is launch-only) is
                # captured once and replayed, which takes the per-layer host work off the step
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        out = model(img, txt, vec)
                    graph.replay()
                    stream.synchronize()
                except Exception as e:  # noqa: BLE001 - reported in the JSON line
                    graph, use_graph = None, f"capture failed: {type(e).__name__}: {e}"[:160]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with clocks_cls(local_rank) as clocks:
                if dist is not None:
                    dist.barrier()
                torch.cuda.synchronize()
                e0.record(stream)
                for _ in range(steps):
                    if graph is not None:
                        graph.replay()
                    else:
                        out = model(img, txt, vec)
                e1.record(stream)
                torch.cuda.synchronize()
                if dist is not None:
                    dist.barrier()
        finite = bool(torch.isfinite(out.float()).all().item())
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank != 0:
        return None
    tokens = total_batch * (cfg.img_tokens + cfg.txt_tokens)
    # kernels of the library per forward: (tensor scale + quantize + GEMM) per linear; a single-stream
    # block quantizes its input once for its two input projections
    n_kernels = cfg.double_blocks * 10 * 3 + cfg.single_blocks * 13
    return {
        "metric": "mmdit_forward_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 linears (e2m1 x ue4m3, fp32 accumulate), bf16 attention", "data": "synthetic",
        "config": {"workload": f"random-init MMDiT-shaped stack: hidden {cfg.hidden}, {cfg.heads} heads, {cfg.double_blocks} double + "
                               f"{cfg.single_blocks} single blocks, {cfg.img_tokens}+{cfg.txt_tokens} tokens, batch {total_batch} "
                               f"split over {world} GPU(s); dynamic activation scales",
                   "linear_params": cfg.linear_params, "batch_per_gpu": batch, "cuda_graph": use_graph},
        "linear_tflops": cfg.linear_flops(total_batch) / (ms * 1e-3) / 1e12,
        "attention_tflops_in_step": cfg.attention_flops(total_batch) / (ms * 1e-3) / 1e12,
        "output_finite": finite, "clocks": clocks.summary(), "gpu_launches": steps * n_kernels,
    }


def run_gpu_arm(args) -> dict | None:
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist  # type: ignore[no-redef]

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the hot path has no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    device = torch.device(f"cuda:{local_rank}")

    import comfy_kitchen as ck
    from comfy_kitchen.backends import cuda as backend

    info = ck.list_backends()["cuda"]
    if not info["available"]:
        raise SystemExit(f"cuda backend unavailable: {info['unavailable_reason']}")
    lib = backend.load_library()
    peaks, peak_kind = load_peaks()
    if args.case == "gemm_sweep":
        return run_gemm_sweep(args, torch, ck, device) if rank == 0 else None
    if args.case in ("mlp_pair", "fc1_fused"):
        return run_mlp_pair(args, torch, ck, backend, device, ClockSampler, local_rank) if rank == 0 else None
    if args.case == "sharded_gemm":
        line = run_sharded_gemm(args, torch, ck, dist, device, rank, world, ClockSampler, local_rank)
        if dist is not None:
            dist.destroy_process_group()
        return line
    if args.case == "mmdit":
        line = run_mmdit(args, torch, dist, device, rank, world, ClockSampler, local_rank)
        if dist is not None:
            dist.destroy_process_group()
        return line

    rows = args.rows or M
    ring = args.ring
    wl = Workload(torch, ck, device, rows, ring, seed=rank)
    launch, kernels_per_step, flops, alg_bytes = make_steps(lib, wl, args.case)
    use_graph = not args.no_graph

    with ClockSampler(local_rank) as clocks:
        ms = time_steps(torch, launch, args.steps, args.warmup, use_graph, dist)
        # per-kernel timings for the rooflines (same buffers, each kernel alone)
        extra = {}
        if args.case == "linear" and not args.skip_extras:
            for name in ("gemm_nvfp4", "quantize_nvfp4", "gemm_mxfp8", "quantize_mxfp8"):
                l2, _, fl2, by2 = make_steps(lib, wl, name)
                extra[name] = (time_steps(torch, l2, args.steps, args.warmup, use_graph, dist) / args.steps, fl2, by2)
        # keep the sampler running long enough to see the clocks under load
        t_end = time.time() + 0.6
        spin_stream = torch.cuda.Stream()
        with torch.cuda.stream(spin_stream):
            i = 0
            while time.time() < t_end:
                launch(i, spin_stream.cuda_stream)
                i += 1
                if i % 64 == 0:
                    spin_stream.synchronize()
            spin_stream.synchronize()
    status = ctypes.c_int(0)
    lib.ck_gemm_status(ctypes.byref(status))
    if status.value != 0:
        raise SystemExit("GEMM kernel reported a wait that gave up (device status word set); timing invalid")

    e2e = None
    if args.case == "linear" and not args.skip_extras:
        e2e = run_e2e(torch, ck, wl, max(3, min(args.steps, 20)), 3, dist)
        e2e["steps"] = max(3, min(args.steps, 20))

    # max over ranks of the device time
    if dist is not None:
        t = torch.tensor([ms, e2e["ms"] / e2e["steps"] if e2e else 0.0], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0].item())
        if e2e:
            e2e["ms"] = float(t[1].item()) * e2e["steps"]
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return None

    ms_per_step = ms / args.steps
    line = {
        "metric": METRIC if args.case == "linear" else args.case,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
        "config": {"workload": WORKLOAD if rows == M else f"{args.case} on {rows} rows of the DiT projection operands",
                   "M": rows, "N": N, "K": K, "case": args.case, "per_rank": "one replica of the step per GPU (batch data-parallel)",
                   "l2": f"ring of {ring} independent buffer sets, {wl.ring_bytes() / 1e6:.0f} MB in total (> 126 MB L2)",
                   "cuda_graph": use_graph},
        "clocks": clocks.summary(),
        "gpu_launches": args.steps * kernels_per_step,
    }
    if flops is not None:
        line["value"] = world * flops / (ms_per_step * 1e-3) / 1e12
        line["unit"] = "TFLOP/s"
        line["dtype"] = "mxfp8 (e4m3 x ue8m0, fp32 accumulate)" if "mxfp8" in args.case else "nvfp4 (e2m1 x ue4m3, fp32 accumulate)"
    else:
        line["value"] = world * alg_bytes / (ms_per_step * 1e-3) / 1e9
        line["unit"] = "GB/s"
        line["dtype"] = "bf16 -> " + ("e4m3 + ue8m0" if "mxfp8" in args.case else "e2m1 + ue4m3")

    fp4_peak = 4.0 * peaks["bf16_tflops"]
    fp8_peak = 2.0 * peaks["bf16_tflops"]

    # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised
    # under profiles/.  The quantizers were captured at 32768 rows (their traffic is proportional
    # to the rows: per-row figures); the GEMMs at the 4096-row workload itself (operand reads; the
    # output is still in L2 when the kernel ends).
    def ncu_traffic(kernel):
        per_row = {"quantize_nvfp4": (201.498368e6 + 40.577536e6) / 32768, "dequantize_nvfp4": (56.629504e6 + 143.971584e6) / 32768, "quantize_mxfp8": (201.338880e6 + 74.617600e6) / 32768}
        fixed_4096 = {"scaled_mm_nvfp4": 12.437248e6 + 1.536e3, "scaled_mm_mxfp8": 22.758144e6 + 81.664e3}
        key = kernel.replace("gemm_", "scaled_mm_")
        if key in per_row:
            return per_row[key] * rows
        if key in fixed_4096 and rows == M:
            return fixed_4096[key]
        return None

    def tensor_roofline(ms_launch, fl, peak, nominal, kernel):
        ach = fl / (ms_launch * 1e-3) / 1e12
        return {"kernel": kernel, "bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "peak_basis": f"{'4' if nominal == NOMINAL_FP4_TFLOPS else '2'} x bf16_tflops of {peak_kind} peaks",
                "frac_of_nominal": ach / nominal, "nominal_peak": nominal, "traffic": ncu_traffic(kernel),
                "us_per_launch": ms_launch * 1e3}

    def hbm_roofline(ms_launch, by, kernel):
        ach = by / (ms_launch * 1e-3) / 1e9
        return {"kernel": kernel, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "peak_basis": f"hbm_gbs of {peak_kind} peaks", "traffic": ncu_traffic(kernel),
                "algorithmic_bytes": by, "us_per_launch": ms_launch * 1e3}

    if args.case == "linear" and extra:
        line["roofline"] = tensor_roofline(extra["gemm_nvfp4"][0], extra["gemm_nvfp4"][1], fp4_peak, NOMINAL_FP4_TFLOPS, "scaled_mm_nvfp4")
        line["roofline_quantize"] = hbm_roofline(extra["quantize_nvfp4"][0], extra["quantize_nvfp4"][2], "quantize_nvfp4")
        line["roofline_mxfp8"] = {
            "gemm": tensor_roofline(extra["gemm_mxfp8"][0], extra["gemm_mxfp8"][1], fp8_peak, NOMINAL_FP8_TFLOPS, "scaled_mm_mxfp8"),
            "quantize": hbm_roofline(extra["quantize_mxfp8"][0], extra["quantize_mxfp8"][2], "quantize_mxfp8"),
        }
    elif flops is not None and args.case.startswith("gemm"):
        is8 = "mxfp8" in args.case
        line["roofline"] = tensor_roofline(ms_per_step, flops, fp8_peak if is8 else fp4_peak,
                                           NOMINAL_FP8_TFLOPS if is8 else NOMINAL_FP4_TFLOPS, args.case)
    elif alg_bytes is not None:
        line["roofline"] = hbm_roofline(ms_per_step, alg_bytes, args.case)

    if e2e:
        per = e2e["ms"] / e2e["steps"]
        line["e2e"] = {"value": world * 2.0 * rows * N * K / (per * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": per,
                       "api": "comfy_kitchen.quantize_nvfp4 + comfy_kitchen.scaled_mm_nvfp4 (pinned host x in, bf16 result out)",
                       "steps_in_flight": e2e.get("lanes", 1)}
    if args.case == "linear" and not args.skip_extras and not args.no_cpu_baseline and world == 1:
        import torch as _t

        _t.set_num_threads(cpu_threads())
        sample_rows = 1024
        cpu_linear_once(256)
        dt, _, which = cpu_linear_once(sample_rows)
        line["cpu_baseline"] = {
            "value": 2.0 * sample_rows * N * K / dt / 1e12, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
            "sample": f"{sample_rows} of {M} rows, one step: {which} quantize_nvfp4(x) + dequantize->fp32 BLAS matmul + bias",
            "seconds": dt}
    if dist is not None:
        dist.destroy_process_group()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--case", default="linear",
                    choices=["linear", "linear_mxfp8", "tensor_scale", "quantize_nvfp4", "quantize_mxfp8", "dequantize_nvfp4",
                             "dequantize_mxfp8", "gemm_nvfp4", "gemm_mxfp8",
                             "sharded_gemm", "gemm_sweep", "mlp_pair", "fc1_fused", "mmdit"])
    ap.add_argument("--mmdit-blocks", default="", help="double,single block counts of --case mmdit (default 19,38)")
    ap.add_argument("--mmdit-batch", type=int, default=8, help="total batch of --case mmdit, split over the GPUs")
    ap.add_argument("--shape", default="16384,15360,3072", help="M,N,K of --case sharded_gemm")
    ap.add_argument("--rows", type=int, default=0, help="override M (profiling of one kernel on a different size)")
    ap.add_argument("--ring", type=int, default=8, help="independent buffer sets cycled through (L2 defeat)")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--skip-extras", action="store_true", help="only the timed case: no per-kernel, e2e or CPU legs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        print(json.dumps(run_reference_arm(args)), flush=True)
        return
    line = run_gpu_arm(args)
    if line is not None:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
