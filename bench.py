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

The K steps are captured once into a CUDA graph; the graph is replayed back to back for about
half a second with a CUDA-event pair around every replay, and the step time is the median replay
divided by K (SM clocks are sampled while those replays run).

The JSON line also carries: ``fused`` (the same step through the one-call entry point
``ck_linear_nvfp4_from_float``), ``e2e`` (the step through the public Python API with host
buffers: pinned-host x -> device, linear, bf16 result -> host) with the floor of the bare copies,
``roofline`` for the dominant kernel (the GEMM), ``roofline_quantize``, ``vs_ref_kernels`` (the
reference's own sm_100 quantizer kernels from baseline/_ref and cuBLASLt through
``torch.nn.functional.scaled_mm``, timed in the same harness on the same operands),
``cpu_baseline`` (the CPU oracle of the same path timed on the host cores, rank 0 of a one-GPU run
only), ``clocks`` and ``gpu_launches``; ``extra`` holds the workloads that shard - the
column-sharded GEMM with its all-gather (fused into the epilogue vs NCCL) and the MMDiT-shaped
stack with the batch split over the ranks - measured inside the same process group.

--impl reference times the CPU restatement of the reference's eager path (oracle/) on the
host cores for the same metric and workload.
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


def bench_config(ring: int = 8) -> dict:
    """The ``config`` object of the JSON line - identical in the GPU arm and the CPU reference arm."""
    return {"workload": WORKLOAD, "M": M, "N": N, "K": K,
            "l2": f"GPU arm: every step uses another of {ring} independent buffer sets (x, W, scales, out; > 126 MB L2 in total)",
            "timing": "GPU arm: K steps captured in one CUDA graph, replayed back to back for ~0.5 s, median replay / K; "
                      "CPU arm: mean of K full steps"}


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


def use_all_host_threads() -> int:
    """Give every thread pool of the CPU arm (torch, BLAS under numpy, OpenMP in the C oracle) the cores
    this process may run on, whatever OMP_NUM_THREADS a launcher exported (torchrun sets it to 1)."""
    import torch

    from oracle import ck_oracle_c as occ

    n = cpu_threads()
    torch.set_num_threads(n)
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=n)
    except Exception:  # noqa: BLE001 - without threadpoolctl the BLAS pool keeps its start-up size
        pass
    if occ.available():
        occ.set_threads(n)
    return n


def run_reference_arm(args) -> dict:
    """--impl reference: the CPU port of the reference's eager path on all host threads, full 4096-row steps."""
    cores = use_all_host_threads()
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_linear_once(M)
    times = []
    which = ""
    for _ in range(args.steps):
        dt, _, which = cpu_linear_once(M)
        times.append(dt)
    per_step = sum(times) / len(times)
    tflops = 2.0 * M * N * K / per_step / 1e12
    sample = f"all {M} rows per step (quantize_nvfp4(x) + dequantize->fp32 matmul + bias -> bf16), {which}, BLAS matmul"
    return {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": bench_config(args.ring),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
class Workload:
    """Device buffers of the step, as a ring of `ring` independent (x, W, out) sets."""

    def __init__(self, torch, ck, lib, device, rows: int, ring: int, seed: int):
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
        # workspaces of the one-call linear (quantized activation of the step), one per ring slot
        need = int(lib.ck_linear_nvfp4_from_float_workspace_bytes(rows, K, 0))
        self.onecall_ws = [torch.zeros(need, **u8) for _ in range(ring)]

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

    def onecall(i, st):  # quantize(x) + GEMM enqueued by one library call
        j = i % wl.ring
        rc = lib.ck_linear_nvfp4_from_float(p(wl.x[j]), 2, p(wl.sx), p(wl.qw[j]), p(wl.bsw[j]), p(wl.sw), p(wl.bias), 2,
                                            p(wl.out[j]), 2, rows, N, K, p(wl.onecall_ws[j]), wl.onecall_ws[j].numel(), st)
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

    def copy_floor(i, st):  # a device copy that moves the quantizer's bytes: 2 B/element in, 0.5625 B/element out
        j = i % wl.ring
        wl.copy_dst[j].copy_(wl.copy_src[j], non_blocking=True)

    if case.startswith("dequantize"):
        wl.deq = [wl.torch.empty(rows, K, dtype=wl.torch.bfloat16, device=wl.device) for _ in range(wl.ring)]
        for j in range(wl.ring):  # operands of the timed kernel
            (q4 if "nvfp4" in case else q8)(j, wl.torch.cuda.current_stream().cuda_stream)
        wl.torch.cuda.synchronize()
    if case == "copy_floor":
        # torch's device-to-device copy of half of the quantizer's traffic each way (read n bytes, write n
        # bytes, 2n = the quantizer's algorithmic bytes): what a plain copy kernel of the same size achieves
        n = q4_bytes // 2
        wl.copy_src = [wl.torch.empty(n, dtype=wl.torch.uint8, device=wl.device) for _ in range(wl.ring)]
        wl.copy_dst = [wl.torch.empty(n, dtype=wl.torch.uint8, device=wl.device) for _ in range(wl.ring)]

    table = {
        "dequantize_nvfp4": (dq4, 1, None, dq4_bytes),
        "dequantize_mxfp8": (dq8, 1, None, dq8_bytes),
        "linear": (lambda i, st: (q4(i, st), g4(i, st)), 2, flops, None),
        "linear_onecall": (onecall, 2, flops, None),
        "linear_mxfp8": (lambda i, st: (q8(i, st), g8(i, st)), 2, flops, None),
        "tensor_scale": (lambda i, st: _tensor_scale(lib, wl, i, st), 1, None, 2 * rows * K + 4),
        "quantize_nvfp4": (q4, 1, None, q4_bytes),
        "quantize_mxfp8": (q8, 1, None, q8_bytes),
        "gemm_nvfp4": (g4, 1, flops, None),
        "gemm_mxfp8": (g8, 1, flops, None),
        "copy_floor": (copy_floor, 1, None, q4_bytes),
    }
    return table[case]


def time_replays(torch, launch, steps: int, warmup: int, use_graph: bool = True, dist=None, min_seconds: float = 0.5,
                 min_replays: int = 11, max_replays: int = 4000) -> dict:
    """Device time of `steps` launches, CUDA events on the launch stream.

    The steps are captured once into a CUDA graph (no host launch gaps between the short kernels).
    The graph is replayed back to back, each replay bracketed by its own event pair, until about
    `min_seconds` of device time have passed (at least `min_replays` times); returns the median, the
    best and the number of replays, in ms per replay.  Without a graph the launches of one "replay"
    are issued from the host."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        st = stream.cuda_stream
        for i in range(warmup):
            launch(i, st)
        stream.synchronize()
        graph = None
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(steps):
                    launch(warmup + i, st)

        def one():
            if graph is not None:
                graph.replay()
            else:
                for i in range(steps):
                    launch(warmup + i, st)

        for _ in range(3):  # untimed: graph upload, caches of the launch path
            one()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        one()
        e1.record(stream)
        stream.synchronize()
        est = max(e0.elapsed_time(e1), 1e-3)
        replays = int(min(max_replays, max(min_replays, min_seconds * 1e3 / est)))
        events = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        events[0].record(stream)
        for r in range(replays):
            one()
            events[r + 1].record(stream)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        times = sorted(events[r].elapsed_time(events[r + 1]) for r in range(replays))
    return {"median_ms": times[len(times) // 2], "best_ms": times[0], "replays": replays}


def bind_to_gpu_numa(torch, local_rank: int) -> dict:
    """Restrict this process to the cores of the NUMA node its GPU hangs off (if the node is known and
    the process is allowed on it), so that pinned host buffers are allocated next to the GPU and the
    ranks of one box do not all stage through node 0.  Returns what was found, for the JSON line."""
    info = {"numa_node": None, "cpus_before": cpu_threads(), "bound": False}
    try:
        props = torch.cuda.get_device_properties(local_rank)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if allowed and allowed != os.sched_getaffinity(0):
            os.sched_setaffinity(0, allowed)
            info["bound"] = True
        info["cpus_after"] = cpu_threads()
    except (OSError, AttributeError, ValueError):
        pass
    return info


def run_e2e(torch, ck, wl: Workload, steps: int, warmup: int, dist=None) -> dict:
    """The step through the public API with host buffers: H2D of x, linear, D2H of the bf16 result.

    Every step does all three inside the timed region.  Steps are issued round-robin on three
    streams (each step stays in order on its own stream), so the copy of one step's input, the
    kernels of another and the read-back of a third overlap, as a serving loop would run them.
    ``floor`` is the same loop with the copies only (same pinned buffers, same three streams): what
    the host link allows, whatever the kernels cost."""
    dev = wl.device
    qw, bsw = wl.qw[0], wl.bsw[0].view(torch.float8_e4m3fn)
    lanes = 3
    streams = [torch.cuda.Stream() for _ in range(lanes)]
    out_host = [torch.empty(wl.rows, N, dtype=torch.bfloat16).pin_memory() for _ in range(lanes)]
    x_dev = [torch.empty(wl.rows, K, dtype=torch.bfloat16, device=dev) for _ in range(lanes)]
    y_dev = [torch.empty(wl.rows, N, dtype=torch.bfloat16, device=dev) for _ in range(lanes)]

    def step(i):
        lane = i % lanes
        with torch.cuda.stream(streams[lane]):
            x = wl.x_host.to(dev, non_blocking=True)
            qx, bsx = ck.quantize_nvfp4(x, wl.sx)
            y = ck.scaled_mm_nvfp4(qx, qw, wl.sx, wl.sw, bsx, bsw, bias=wl.bias, out_dtype=torch.bfloat16)
            out_host[lane].copy_(y, non_blocking=True)

    def copies_only(i):
        lane = i % lanes
        with torch.cuda.stream(streams[lane]):
            x_dev[lane].copy_(wl.x_host, non_blocking=True)
            out_host[lane].copy_(y_dev[lane], non_blocking=True)

    def timed(fn):
        for i in range(warmup):
            fn(i)
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
            fn(i)
        for st in streams:
            main.wait_stream(st)
        e1.record(main)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    ms = timed(step)
    floor_ms = timed(copies_only)
    return {"ms": ms, "floor_ms": floor_ms, "h2d": wl.x_host.numel() * 2, "d2h": out_host[0].numel() * 2, "lanes": lanes}


# --------------------------------------------------------------------------------------------
# same-box baselines: the reference's own sm_100 kernels and cuBLASLt
# --------------------------------------------------------------------------------------------
REF_QUANT_LIB = os.path.join(ROOT, "baseline", "_ref", "libref_quant.so")


def reference_kernel_baselines(torch, lib, wl: Workload, steps: int, warmup: int, ours: dict) -> dict:
    """The kernels the reference ships for Blackwell, timed on the same GPU, in the same ring / graph
    harness, on the same operands as this build's kernels:

    * its quantizers (launch_quantize_nvfp4_kernel, ops/quantize_nvfp4.cu:323-335, and
      launch_quantize_mxfp8_kernel, ops/quantize_mxfp8.cu:148-157), compiled from a checkout of the
      reference by baseline/build_ref_kernels.py (kernel alone; the reference's wrapper also zero-fills
      the scale tensor before every call, cuda/__init__.py:242-244);
    * its GEMM library call: cuBLASLt block-scaled matmul through torch.nn.functional.scaled_mm, which
      is what the reference's eager path runs on a GPU (scaled_mm_v2.py:40-53) and the same cuBLASLt
      algorithm family its cuda backend calls (ops/cublas_gemm_nvfp4.cu:256-272).
    `ours` maps the same four names to this build's microseconds per launch."""
    rows = wl.rows
    res: dict = {}

    def entry(name, us, note=None):
        e = {"ref_us": us, "ours_us": ours.get(name), "speedup": (us / ours[name]) if ours.get(name) else None}
        if note:
            e["note"] = note
        res[name] = e

    # --- quantizers
    if os.path.exists(REF_QUANT_LIB):
        try:
            ref = ctypes.CDLL(REF_QUANT_LIB)
            P, L, I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
            ref.launch_quantize_nvfp4_kernel.argtypes = [P, P, P, P, L, L, L, L, ctypes.c_float, I, ctypes.c_bool, P]
            ref.launch_quantize_nvfp4_kernel.restype = None
            ref.launch_quantize_mxfp8_kernel.argtypes = [P, P, P, L, L, L, L, I, P]
            ref.launch_quantize_mxfp8_kernel.restype = None

            def rq4(i, st):
                j = i % wl.ring
                ref.launch_quantize_nvfp4_kernel(wl.x[j].data_ptr(), wl.sx.data_ptr(), wl.qx[j].data_ptr(),
                                                 wl.bsx[j].data_ptr(), rows, K, rows, K, 0.0, 2, True, st)

            def rq8(i, st):
                j = i % wl.ring
                ref.launch_quantize_mxfp8_kernel(wl.x[j].data_ptr(), wl.qx8[j].data_ptr(), wl.bsx8[j].data_ptr(), rows, K,
                                                 rows, K, 2, st)

            for name, fn in (("quantize_nvfp4", rq4), ("quantize_mxfp8", rq8)):
                t = time_replays(torch, fn, steps, warmup, min_seconds=0.1)
                entry(name, t["median_ms"] / steps * 1e3, "reference kernel alone (its wrapper adds a memset of the scale tensor)")
        except (OSError, AttributeError) as e:
            res["quantize_nvfp4"] = res["quantize_mxfp8"] = {"unavailable": f"{type(e).__name__}: {e}"[:160]}
    else:
        res["quantize_nvfp4"] = res["quantize_mxfp8"] = {
            "unavailable": "baseline/_ref/libref_quant.so not built (baseline/build_ref_kernels.py needs a checkout of the reference)"}
    # the quantizers above overwrote the activations of the ring with the reference's codes: restore ours
    st0 = torch.cuda.current_stream().cuda_stream
    q4 = make_steps(lib, wl, "quantize_nvfp4")[0]
    q8 = make_steps(lib, wl, "quantize_mxfp8")[0]
    for j in range(wl.ring):
        q4(j, st0)
        q8(j, st0)
    torch.cuda.synchronize()

    # --- cuBLASLt through torch
    try:
        from torch.nn.functional import ScalingType, SwizzleType, scaled_mm

        f4, e4m3, e8m0 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn, torch.float8_e8m0fnu

        def cublas4(i, st):
            j = i % wl.ring
            return scaled_mm(wl.qx[j].view(f4), wl.qw[j].view(f4).t(),
                             scale_a=[wl.bsx[j].view(e4m3).view(-1), wl.sx], scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                             scale_b=[wl.bsw[j].view(e4m3).view(-1), wl.sw], scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                             swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
                             swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
                             bias=wl.bias, output_dtype=torch.bfloat16)

        def cublas8(i, st):
            j = i % wl.ring
            return scaled_mm(wl.qx8[j].view(e4m3), wl.qw8[j].view(e4m3).t(),
                             scale_a=wl.bsx8[j].view(e8m0), scale_recipe_a=ScalingType.BlockWise1x32,
                             scale_b=wl.bsw8[j].view(e8m0), scale_recipe_b=ScalingType.BlockWise1x32,
                             swizzle_a=SwizzleType.SWIZZLE_32_4_4, swizzle_b=SwizzleType.SWIZZLE_32_4_4,
                             bias=wl.bias, output_dtype=torch.bfloat16)

        g4 = make_steps(lib, wl, "gemm_nvfp4")[0]
        g8 = make_steps(lib, wl, "gemm_mxfp8")[0]
        for name, fn, mine in (("cublaslt_nvfp4", cublas4, g4), ("cublaslt_mxfp8", cublas8, g8)):
            try:
                y_ref = fn(0, st0)
                mine(0, st0)
                torch.cuda.synchronize()
                same = bool(torch.equal(y_ref, wl.out[0]))
                # inside the graph every launch allocates its output from the graph's private pool, as
                # torch does for any op that returns a new tensor
                t = time_replays(torch, fn, steps, warmup, min_seconds=0.1)
                entry(name, t["median_ms"] / steps * 1e3, "torch.nn.functional.scaled_mm (cuBLASLt), output allocated by torch")
                res[name]["bit_identical_to_ours"] = same
            except Exception as e:  # noqa: BLE001 - reported in the JSON line
                res[name] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    except ImportError as e:
        res["cublaslt_nvfp4"] = res["cublaslt_mxfp8"] = {"unavailable": f"torch.nn.functional.scaled_mm: {e}"[:160]}
    return res


# --------------------------------------------------------------------------------------------
# workloads that shard: column-sharded GEMM + all-gather, MMDiT stack with the batch split
# --------------------------------------------------------------------------------------------
def measure_peer_copy_gbs(torch, dist, peers, device, rank, world) -> float | None:
    """GB/s of a plain copy from the next rank's result buffer (peer memory over NVLink) into local
    memory, the largest buffer at hand, CUDA events, best of 5: the measured stand-in for the NVLink
    peak a rank's incoming tiles are bounded by."""
    try:
        handle = peers._handles[0]
        src = handle.get_buffer((rank + 1) % world, tuple(peers.tensors[0].shape), peers.dtype)
        dst = torch.empty_like(peers.tensors[0])
        best = 0.0
        for _ in range(5):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dst.copy_(src)
            e1.record()
            torch.cuda.synchronize()
            best = max(best, dst.numel() * dst.element_size() / (e0.elapsed_time(e1) * 1e-3) / 1e9)
        t = torch.tensor([best], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item())
    except Exception:  # noqa: BLE001 - the figure is optional
        return None


def run_sharded_gemm(args, torch, ck, dist, device, rank, world, clocks_cls, local_rank) -> dict | None:
    """NVFP4 GEMM with N column-sharded over the ranks and the all-gather of the bf16 output.

    Strong scaling: the problem is fixed, each rank computes y[:, shard].  Three timings, each a CUDA
    graph of `iters` back-to-back calls replayed for ~0.3 s (median replay): the local GEMM alone,
    GEMM + NCCL all-gather, and the GEMM whose epilogue stores every tile into all ranks' results over
    NVLink + the barrier kernel.  The NVLink floor uses the peer-copy bandwidth measured in this run."""
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
    del w, qw, bsw, x
    iters = 10

    def timed(fn, use_graph=True):
        t = time_replays(torch, lambda i, st: fn(), iters, 3, use_graph=use_graph, dist=dist, min_seconds=0.3)
        v = torch.tensor([t["median_ms"] / iters], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    # The fused path (epilogue stores into every rank's peer-mapped result + one barrier kernel)
    # needs torch's symmetric memory; when that is unavailable only the NCCL path is timed.
    peers, fused_error, peer_gbs = None, None, None
    if dist is not None and world > 1:
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            peers = sharded.PeerOutput(m, n, torch.bfloat16, device, buffers=2)
            peer_gbs = measure_peer_copy_gbs(torch, dist, peers, device, rank, world)
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            fused_error = f"{type(e).__name__}: {e}"[:200]
    with clocks_cls(local_rank) as clocks:
        ms_gemm = timed(lambda: sharded.sharded_linear_nvfp4(qx, sx, bsx, shard, gather=False))
        # NCCL inside a captured graph works with torch's process groups; fall back to host launches if not
        try:
            ms_nccl = timed(lambda: sharded.sharded_linear_nvfp4(qx, sx, bsx, shard)) if world > 1 else ms_gemm
            nccl_graph = True
        except Exception:  # noqa: BLE001
            ms_nccl = timed(lambda: sharded.sharded_linear_nvfp4(qx, sx, bsx, shard), use_graph=False)
            nccl_graph = False
        ms_fused = None
        if peers is not None:
            # the barrier's epoch is a launch argument: a captured graph would replay a stale epoch, so
            # the fused path is launched from the host (one GEMM + one barrier kernel per call)
            ms_fused = timed(lambda: sharded.sharded_linear_nvfp4_fused(qx, sx, bsx, shard, peers), use_graph=False)
    y = sharded.sharded_linear_nvfp4(qx, sx, bsx, shard)
    y_local = sharded.sharded_linear_nvfp4(qx, sx, bsx, shard, gather=False)
    ok = bool(torch.equal(y[:, shard.start:shard.end], y_local)) and tuple(y.shape) == (m, n)
    fused_ok, barrier_status = None, None
    if peers is not None:
        yf = sharded.sharded_linear_nvfp4_fused(qx, sx, bsx, shard, peers)
        fused_ok = bool(torch.equal(yf, y))
        try:
            peers.check()
            barrier_status = 0
        except RuntimeError as e:
            barrier_status = str(e)[:160]
        flag = torch.tensor([1 if (fused_ok and barrier_status == 0) else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) != 1:
            raise SystemExit(f"rank {rank}: fused all-gather result differs from the NCCL result or a barrier gave up "
                             f"(equal={fused_ok}, status={barrier_status})")
    ms_full = ms_fused if ms_fused is not None else ms_nccl
    if rank != 0:
        return None
    flops = 2.0 * m * n * k
    recv = (world - 1) / world * 2.0 * m * n
    link = peer_gbs or 770.0
    floor_ms = recv / (link * 1e9) * 1e3
    return {
        "metric": "sharded_nvfp4_gemm_tflops", "value": flops / (ms_full * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": iters, "warmup": 3, "ms_per_step": ms_full, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"NVFP4 GEMM M={m} N={n} K={k}, N column-sharded over {world} GPUs, all-gather of the bf16 "
                               + ("output fused into the GEMM epilogue (peer stores over NVLink + barrier kernel)"
                                  if ms_fused is not None else "output by NCCL"),
                   "M": m, "N": n, "K": k},
        "gemm_only": {"ms": ms_gemm, "aggregate_tflops": flops / (ms_gemm * 1e-3) / 1e12, "cuda_graph": True},
        "nccl_all_gather": {"ms_gemm_plus_gather": ms_nccl, "tflops": flops / (ms_nccl * 1e-3) / 1e12,
                            "bytes_received_per_gpu": recv, "cuda_graph": nccl_graph,
                            "gbs_per_gpu": (recv / ((ms_nccl - ms_gemm) * 1e-3) / 1e9) if ms_nccl > ms_gemm else None},
        "fused_all_gather": None if ms_fused is None else {
            "ms": ms_fused, "tflops": flops / (ms_fused * 1e-3) / 1e12, "equals_nccl_result": fused_ok,
            "barrier_status": barrier_status, "speedup_vs_nccl": ms_nccl / ms_fused,
            # roofline of the fused kernel: the slower of tensor time and the bytes this GPU must receive
            "nvlink_floor_ms": floor_ms, "nvlink_peak_gbs": link,
            "nvlink_peak_basis": "peer copy measured in this run" if peer_gbs else "770 GB/s, earlier measurement on this pool",
            "bound": "nvlink" if floor_ms > ms_gemm else "tensor",
            "frac_of_floor": max(floor_ms, ms_gemm) / ms_fused},
        "fused_unavailable": fused_error,
        "gathered_equals_local": ok, "clocks": clocks.summary(), "gpu_launches": iters * (2 if ms_fused is not None else 1),
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
    """NVFP4 GEMM over the sweep on one GPU: M in {1, 16, 256, 4096, 16384} x (K, N) in {(3072, 3072),
    (3072, 12288), (12288, 3072), (3072, 15360)}, bf16 output, through ``ck.scaled_mm_nvfp4`` (workspace
    paths included).  Each shape: a CUDA graph of 20 launches that cycle through enough copies of the
    weight to exceed the L2 cache, median of 11 replays.  Rows with M <= 256 are weight streaming: they
    are read against the HBM roofline (0.5625 (M K + N K) + 2 M N bytes), the others against the tensor peak."""
    peaks, peak_kind = load_peaks()
    rows = []
    gen = torch.Generator(device="cpu").manual_seed(0)
    for (k, n) in ((3072, 3072), (3072, 12288), (12288, 3072), (3072, 15360)):
        w = (torch.randn(n, k, generator=gen) * 0.02).bfloat16().to(device)
        sw = (w.abs().amax() / 2688.0).float()
        qw0, bsw0 = ck.quantize_nvfp4(w, sw)
        del w
        copies = max(2, min(48, -(-160_000_000 // (qw0.numel() + bsw0.numel()))))
        qw = [qw0.clone() for _ in range(copies)]
        bsw = [bsw0.clone() for _ in range(copies)]
        for m in (1, 16, 256, 4096, 16384):
            x = torch.randn(m, k, generator=gen).bfloat16().to(device)
            sx = (x.abs().amax() / 2688.0).float()
            qx, bsx = ck.quantize_nvfp4(x, sx, pad_16x=(m % 16 != 0))

            def f(i, st):
                return ck.scaled_mm_nvfp4(qx, qw[i % copies], sx, sw, bsx, bsw[i % copies])

            t = time_replays(torch, f, 20, 3, min_seconds=0.0, min_replays=11)
            us = t["median_ms"] / 20 * 1e3
            row = {"M": m, "N": n, "K": k, "us": us, "tflops": 2.0 * m * n * k / (us * 1e-6) / 1e12, "weight_copies": copies}
            if not args.no_ref_kernels and qx.shape[0] == m:
                # the same launches through cuBLASLt (torch.nn.functional.scaled_mm), same operands and harness
                try:
                    from torch.nn.functional import ScalingType, SwizzleType, scaled_mm
                    f4, e4m3 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
                    recipe = [ScalingType.BlockWise1x16, ScalingType.TensorWise]
                    swz = [SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE]
                    qx4, bsx1 = qx.view(f4), bsx.view(e4m3).view(-1)
                    qw4 = [q.view(f4).t() for q in qw]
                    bsw1 = [b.view(e4m3).view(-1) for b in bsw]

                    def g(i, st):
                        j = i % copies
                        return scaled_mm(qx4, qw4[j], scale_a=[bsx1, sx], scale_recipe_a=recipe, scale_b=[bsw1[j], sw],
                                         scale_recipe_b=recipe, swizzle_a=swz, swizzle_b=swz, output_dtype=torch.bfloat16)

                    same = bool(torch.equal(g(0, None), f(0, None)))
                    tr = time_replays(torch, g, 20, 3, min_seconds=0.0, min_replays=11)
                    row["cublaslt_us"] = tr["median_ms"] / 20 * 1e3
                    row["cublaslt_bit_identical"] = same
                except Exception as e:  # noqa: BLE001 - shapes the library refuses are reported, not fatal
                    row["cublaslt_unavailable"] = f"{type(e).__name__}: {e}"[:120]
            if m <= 256:
                by = 0.5625 * (m * k + n * k) + 2.0 * m * n
                row.update({"bound": "hbm", "algorithmic_bytes": by, "gbs": by / (us * 1e-6) / 1e9,
                            "frac": by / (us * 1e-6) / 1e9 / peaks["hbm_gbs"]})
            else:
                row.update({"bound": "tensor", "frac": row["tflops"] / (4.0 * peaks["bf16_tflops"]),
                            "frac_of_nominal": row["tflops"] / NOMINAL_FP4_TFLOPS})
            rows.append(row)
    big = [r for r in rows if r["M"] >= 4096]
    return {"metric": "nvfp4_gemm_sweep_tflops", "value": sum(r["tflops"] for r in big) / len(big), "unit": "TFLOP/s",
            "n_gpus": 1, "steps": 20, "warmup": 3, "ms_per_step": sum(r["us"] for r in rows) * 1e-3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "NVFP4 GEMM sweep on one GPU (value = mean TFLOP/s of the M >= 4096 shapes)",
                       "l2": "launches cycle through copies of the weight that exceed the L2 cache in total",
                       "peaks": peak_kind},
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
    steps, warmup = min(args.steps, 8), min(max(args.warmup, 1), 3)

    def timed_forward(model, img, txt, vec):
        """(ms per forward on this rank, clock record, output finite, graph used or why not)"""
        use_graph = not args.no_graph
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
            # one more untimed forward gives the step's length: the timed region is made at least ~0.7 s
            # long (the same count on every rank), so that the clock sampler sees it at every N
            e0.record(stream)
            if graph is not None:
                graph.replay()
            else:
                out = model(img, txt, vec)
            e1.record(stream)
            stream.synchronize()
            est = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
            if dist is not None:
                dist.all_reduce(est, op=dist.ReduceOp.MAX)
            n_steps = int(min(64, max(steps, -(-700.0 // max(float(est.item()), 1e-3)))))
            with clocks_cls(local_rank) as clocks:
                if dist is not None:
                    dist.barrier()
                torch.cuda.synchronize()
                e0.record(stream)
                for _ in range(n_steps):
                    if graph is not None:
                        graph.replay()
                    else:
                        out = model(img, txt, vec)
                e1.record(stream)
                torch.cuda.synchronize()
                if dist is not None:
                    dist.barrier()
        finite = bool(torch.isfinite(out.float()).all().item())
        del graph, out
        return e0.elapsed_time(e1) / n_steps, clocks, finite, use_graph, n_steps

    with torch.inference_mode():
        model = mm.MMDiTStack(cfg, device, NVFP4Linear.from_linear, seed=0)
        img, txt, vec = mm.make_inputs(cfg, batch, device, seed=rank)
        ms_local, clocks, finite, use_graph, timed_steps = timed_forward(model, img, txt, vec)
        # second pass: static scales for the MLPs' hidden tensors (fc2.input_scale, calibrated on this
        # input), so that GELU and the hidden tensor's quantization run inside fc1's epilogue
        fused_mlps = mm.calibrate_hidden_scales(model, img, txt, vec)
        ms_static_local, clocks_static, finite_static, _, _ = timed_forward(model, img, txt, vec)
    del model
    torch.cuda.empty_cache()
    attn_ms = attention_only_ms(torch, cfg, batch, device)
    t = torch.tensor([ms_local, attn_ms, ms_static_local], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, attn_ms, ms_static = float(t[0].item()), float(t[1].item()), float(t[2].item())
    if rank != 0:
        return None
    tokens = total_batch * (cfg.img_tokens + cfg.txt_tokens)
    # kernels of the library per forward: (tensor scale + quantize + GEMM) per linear; a single-stream
    # block quantizes its input once for its two input projections
    n_kernels = cfg.double_blocks * 10 * 3 + cfg.single_blocks * 13
    return {
        "metric": "mmdit_forward_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": timed_steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 linears (e2m1 x ue4m3, fp32 accumulate), bf16 attention", "data": "synthetic",
        "config": {"workload": f"random-init MMDiT-shaped stack: hidden {cfg.hidden}, {cfg.heads} heads, {cfg.double_blocks} double + "
                               f"{cfg.single_blocks} single blocks, {cfg.img_tokens}+{cfg.txt_tokens} tokens, batch {total_batch} "
                               f"split over {world} GPU(s); dynamic activation scales",
                   "linear_params": cfg.linear_params, "batch_per_gpu": batch, "cuda_graph": use_graph},
        "attention_only_ms": attn_ms, "share_outside_attention": max(0.0, 1.0 - attn_ms / ms),
        "linear_tflops": cfg.linear_flops(total_batch) / (ms * 1e-3) / 1e12,
        "linear_tflops_outside_attention": cfg.linear_flops(total_batch) / (max(ms - attn_ms, 1e-6) * 1e-3) / 1e12,
        "attention_tflops_in_step": cfg.attention_flops(total_batch) / (ms * 1e-3) / 1e12,
        "output_finite": finite, "clocks": clocks.summary(), "gpu_launches": timed_steps * n_kernels,
        "static_hidden_scales": {
            "ms_per_step": ms_static, "value": tokens / (ms_static * 1e-3), "unit": "tokens/s", "fused_mlps": fused_mlps,
            "what": "same stack after one calibration forward: every MLP's second layer has a static input scale, so "
                    "GELU and the hidden tensor's NVFP4 quantization run inside the first GEMM's epilogue "
                    "(ck_linear_nvfp4_fused) instead of as GELU + tensor-scale + quantize kernels",
            "output_finite": finite_static, "clocks": clocks_static.summary(),
        },
    }


def attention_only_ms(torch, cfg, batch: int, device) -> float:
    """Device time of the stack's attention calls alone (bf16 SDPA over all tokens, one call per block),
    replayed from a CUDA graph: what of a forward is not the quantized-linear path."""
    import bench_mmdit as mm

    s_ = cfg.img_tokens + cfg.txt_tokens
    q, k, v = (torch.randn(batch, s_, cfg.hidden, device=device).to(torch.bfloat16) for _ in range(3))
    blocks = cfg.double_blocks + cfg.single_blocks
    with torch.inference_mode():
        t = time_replays(torch, lambda i, st: mm._attention(q, k, v, cfg.heads), blocks, 1, min_seconds=0.0, min_replays=3)
    return t["median_ms"]


def load_ncu_traffic() -> dict:
    """dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
    profiles/ (profiles/ncu_traffic.json: bytes and the row count each capture ran at)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


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
    numa = bind_to_gpu_numa(torch, local_rank)  # before any pinned allocation

    import comfy_kitchen as ck
    from comfy_kitchen.backends import cuda as backend

    info = ck.list_backends()["cuda"]
    if not info["available"]:
        raise SystemExit(f"cuda backend unavailable: {info['unavailable_reason']}")
    lib = backend.load_library()
    peaks, peak_kind = load_peaks()

    def finish(line):
        if dist is not None:
            dist.destroy_process_group()
        return line

    if args.case == "gemm_sweep":
        return finish(run_gemm_sweep(args, torch, ck, device) if rank == 0 else None)
    if args.case in ("mlp_pair", "fc1_fused"):
        return finish(run_mlp_pair(args, torch, ck, backend, device, ClockSampler, local_rank) if rank == 0 else None)
    if args.case == "sharded_gemm":
        return finish(run_sharded_gemm(args, torch, ck, dist, device, rank, world, ClockSampler, local_rank))
    if args.case == "mmdit":
        return finish(run_mmdit(args, torch, dist, device, rank, world, ClockSampler, local_rank))

    rows = args.rows or M
    ring = args.ring
    wl = Workload(torch, ck, lib, device, rows, ring, seed=rank)
    launch, kernels_per_step, flops, alg_bytes = make_steps(lib, wl, args.case)
    use_graph = not args.no_graph
    full = args.case == "linear" and not args.skip_extras

    with ClockSampler(local_rank) as clocks:
        timing = time_replays(torch, launch, args.steps, args.warmup, use_graph, dist)
        # per-kernel timings for the rooflines and the one-call path (same buffers, each alone)
        extra = {}
        if full:
            # The one-call path, timed exactly like the headline step (same replay time, same ring).
            l2, _, fl2, by2 = make_steps(lib, wl, "linear_onecall")
            t2 = time_replays(torch, l2, args.steps, args.warmup, use_graph, dist)
            extra["linear_onecall"] = (t2["median_ms"] / args.steps, fl2, by2, t2["best_ms"] / args.steps)
            # Each kernel alone: the median of 11 replays of the K-launch graph (a few ms in all - the
            # kernel "timed alone", to be read against the burst peak; the GPU idles for 0.75 s before each
            # pass so that the load of the pass before has left its power average) and, for the GEMM, also
            # the median over ~0.2 s of back-to-back replays (the GPU settles under its power cap: sustained peak).
            for name in ("gemm_nvfp4", "quantize_nvfp4", "gemm_mxfp8", "quantize_mxfp8", "copy_floor"):
                l2, _, fl2, by2 = make_steps(lib, wl, name)
                torch.cuda.synchronize()
                time.sleep(0.75)
                t2 = time_replays(torch, l2, args.steps, args.warmup, use_graph, dist, min_seconds=0.0, min_replays=11)
                extra[name] = (t2["median_ms"] / args.steps, fl2, by2, t2["best_ms"] / args.steps)
            l2 = make_steps(lib, wl, "gemm_nvfp4")[0]
            sustained_gemm_ms = time_replays(torch, l2, args.steps, args.warmup, use_graph, dist, min_seconds=0.2)["median_ms"] / args.steps
    status = ctypes.c_int(0)
    lib.ck_gemm_status(ctypes.byref(status))
    if status.value != 0:
        raise SystemExit("GEMM kernel reported a wait that gave up (device status word set); timing invalid")

    ref_kernels = None
    if full and world == 1 and not args.no_ref_kernels:
        ours = {"quantize_nvfp4": extra["quantize_nvfp4"][0] * 1e3, "quantize_mxfp8": extra["quantize_mxfp8"][0] * 1e3,
                "cublaslt_nvfp4": extra["gemm_nvfp4"][0] * 1e3, "cublaslt_mxfp8": extra["gemm_mxfp8"][0] * 1e3}
        ref_kernels = reference_kernel_baselines(torch, lib, wl, args.steps, args.warmup, ours)

    e2e = None
    if full:
        e2e = run_e2e(torch, ck, wl, max(3, min(args.steps, 20)), 3, dist)
        e2e["steps"] = max(3, min(args.steps, 20))

    # max over ranks of the device time
    ms = timing["median_ms"]
    if dist is not None:
        t = torch.tensor([ms, e2e["ms"] / e2e["steps"] if e2e else 0.0, e2e["floor_ms"] / e2e["steps"] if e2e else 0.0],
                         device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0].item())
        if e2e:
            e2e["ms"] = float(t[1].item()) * e2e["steps"]
            e2e["floor_ms"] = float(t[2].item()) * e2e["steps"]

    # the workloads that shard, inside the same process group
    shard_extra = {}
    ring_mb = wl.ring_bytes() / 1e6
    if full and not args.no_shard_extras:
        del wl.x, wl.out  # the ring is not needed any more: leave the memory to the big shapes
        torch.cuda.empty_cache()
        sub = argparse.Namespace(**vars(args))
        sub.shape = "16384,15360,3072"
        try:
            shard_extra["sharded_gemm"] = run_sharded_gemm(sub, torch, ck, dist, device, rank, world, ClockSampler, local_rank)
        except SystemExit:
            raise
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            shard_extra["sharded_gemm"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        torch.cuda.empty_cache()
        if args.mmdit_batch % world == 0:
            sub.steps, sub.warmup = 3, 1
            try:
                shard_extra["mmdit"] = run_mmdit(sub, torch, dist, device, rank, world, ClockSampler, local_rank)
            except Exception as e:  # noqa: BLE001
                shard_extra["mmdit"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    if rank != 0:
        return finish(None)

    ms_per_step = ms / args.steps
    config = bench_config(ring) if (rows == M and args.case == "linear") else {
        "workload": f"{args.case} on {rows} rows of the DiT projection operands", "M": rows, "N": N, "K": K,
        "l2": f"ring of {ring} independent buffer sets", "cuda_graph": use_graph}
    line = {
        "metric": METRIC if args.case == "linear" else args.case,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
        "config": config,
        "harness": {"case": args.case, "per_rank": "one replica of the step per GPU (batch data-parallel)",
                    "ring_mb": ring_mb, "cuda_graph": use_graph, "replays": timing["replays"],
                    "best_ms_per_step": timing["best_ms"] / args.steps, "numa": numa},
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
    captures = load_ncu_traffic()

    def ncu_traffic(kernel):
        c = captures.get(kernel.replace("gemm_", "scaled_mm_"))
        if not c:
            return None
        total = c["dram_bytes_read"] + c["dram_bytes_write"]
        if c.get("scales_with") == "rows":
            return total / c["rows"] * rows
        return total if c["rows"] == rows else None

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

    if full:
        line["roofline"] = tensor_roofline(extra["gemm_nvfp4"][0], extra["gemm_nvfp4"][1], fp4_peak, NOMINAL_FP4_TFLOPS, "scaled_mm_nvfp4")
        line["roofline"]["timing"] = "median of 11 replays of a graph of K launches after 0.75 s of idling (kernel alone, a few ms): read against the burst peak"
        line["roofline"]["best_us_per_launch"] = extra["gemm_nvfp4"][3] * 1e3
        sus_peak = 4.0 * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        sus = extra["gemm_nvfp4"][1] / (sustained_gemm_ms * 1e-3) / 1e12
        line["roofline"]["sustained"] = {"us_per_launch": sustained_gemm_ms * 1e3, "achieved": sus, "peak": sus_peak,
                                         "frac": sus / sus_peak,
                                         "timing": "median over ~0.2 s of back-to-back replays, against 4 x the sustained bf16 peak"}
        line["roofline_quantize"] = hbm_roofline(extra["quantize_nvfp4"][0], extra["quantize_nvfp4"][2], "quantize_nvfp4")
        floor = hbm_roofline(extra["copy_floor"][0], extra["copy_floor"][2], "copy_floor")
        line["roofline_quantize"]["device_copy_of_the_same_bytes"] = {
            "us_per_launch": floor["us_per_launch"], "gbs": floor["achieved"], "frac_of_peak": floor["frac"],
            "quantizer_vs_copy": floor["us_per_launch"] / line["roofline_quantize"]["us_per_launch"]}
        line["roofline_mxfp8"] = {
            "gemm": tensor_roofline(extra["gemm_mxfp8"][0], extra["gemm_mxfp8"][1], fp8_peak, NOMINAL_FP8_TFLOPS, "scaled_mm_mxfp8"),
            "quantize": hbm_roofline(extra["quantize_mxfp8"][0], extra["quantize_mxfp8"][2], "quantize_mxfp8"),
        }
        oc_ms = extra["linear_onecall"][0]
        line["fused"] = {"value": world * flops / (oc_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": oc_ms,
                         "api": "ck_linear_nvfp4_from_float: quantize(x) + GEMM enqueued by one library call "
                                "(programmatic dependent launch between the kernels, quantized activation in a caller workspace)",
                         "separate_calls_ms_per_step": ms_per_step}
    elif flops is not None and args.case.startswith("gemm"):
        is8 = "mxfp8" in args.case
        line["roofline"] = tensor_roofline(ms_per_step, flops, fp8_peak if is8 else fp4_peak,
                                           NOMINAL_FP8_TFLOPS if is8 else NOMINAL_FP4_TFLOPS, args.case)
    elif alg_bytes is not None:
        line["roofline"] = hbm_roofline(ms_per_step, alg_bytes, args.case)

    if ref_kernels is not None:
        line["vs_ref_kernels"] = ref_kernels
    if e2e:
        per = e2e["ms"] / e2e["steps"]
        floor_per = e2e["floor_ms"] / e2e["steps"]
        line["e2e"] = {"value": world * 2.0 * rows * N * K / (per * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": per,
                       "api": "comfy_kitchen.quantize_nvfp4 + comfy_kitchen.scaled_mm_nvfp4 (pinned host x in, bf16 result out)",
                       "steps_in_flight": e2e.get("lanes", 1),
                       "floor_ms": floor_per, "frac_of_floor": floor_per / per,
                       "floor": "the same loop with the two pinned copies only (same buffers, same three streams)",
                       "host_link_gbs_at_floor": (e2e["h2d"] + e2e["d2h"]) / (floor_per * 1e-3) / 1e9}
    if shard_extra:
        line["extra"] = shard_extra
    if full and not args.no_cpu_baseline and world == 1:
        cores = use_all_host_threads()
        cpu_linear_once(256)
        dt, _, which = cpu_linear_once(M)
        line["cpu_baseline"] = {
            "value": 2.0 * M * N * K / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"all {M} rows, one step: {which} quantize_nvfp4(x) + dequantize->fp32 BLAS matmul + bias",
            "seconds": dt}
    return finish(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--case", default="linear",
                    choices=["linear", "linear_onecall", "linear_mxfp8", "tensor_scale", "quantize_nvfp4", "quantize_mxfp8",
                             "dequantize_nvfp4", "dequantize_mxfp8", "gemm_nvfp4", "gemm_mxfp8", "copy_floor",
                             "sharded_gemm", "gemm_sweep", "mlp_pair", "fc1_fused", "mmdit"])
    ap.add_argument("--mmdit-blocks", default="", help="double,single block counts of --case mmdit (default 19,38)")
    ap.add_argument("--mmdit-batch", type=int, default=8, help="total batch of --case mmdit, split over the GPUs")
    ap.add_argument("--shape", default="16384,15360,3072", help="M,N,K of --case sharded_gemm")
    ap.add_argument("--rows", type=int, default=0, help="override M (profiling of one kernel on a different size)")
    ap.add_argument("--ring", type=int, default=8, help="independent buffer sets cycled through (L2 defeat)")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--skip-extras", action="store_true", help="only the timed case: no per-kernel, e2e, sharded or CPU legs")
    ap.add_argument("--no-shard-extras", action="store_true", help="skip the sharded-GEMM and MMDiT legs of the default run")
    ap.add_argument("--no-ref-kernels", action="store_true", help="skip the reference-kernel / cuBLASLt baselines")
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
