"""Per-role timeline of the block-scaled GEMM kernel (tuning aid).

    python comfy-kitchen_b200/gemm_timeline.py build [--stages]   # cross-compiles; no GPU needed
    python comfy-kitchen_b200/gemm_timeline.py run [M,N,K] [--ring 8] [--verbose]

``build`` compiles csrc/*.cu with -DCK_GEMM_TRACE into lib/libck_b200_trace.so: the same
kernels, with the SM cycle counter recorded at fixed points of each role's per-tile loop (kept in
shared memory, written out when the CTA is done: the kernel then runs within ~1 % of the
production build) and the global nanosecond timer at CTA entry, after set-up, after the
dependency wait and at the end.  ``--stages`` adds per-stage stamps of the MMA warp, stored to
global memory as they are taken (they slow the kernel by several per cent and stall behind the
epilogue's stores; printed by ``run --verbose``).  ``run`` replays a CUDA graph of 16 back-to-back NVFP4 GEMM launches over a ring of
operand sets (so that operands come from DRAM, as in the benchmark), reads the buffers back and
prints, for the last launches: when CTAs entered / passed the dependency wait / finished, the
SM clock the counters imply, and for a few CTAs the cycle at which each tile's first and last
stage landed, its accumulator was handed over, drained and stored.  The figures quoted in
profiles/scaled_mm_nvfp4_pair_*.md come from this tool.  The instrumented library is never
loaded by the package unless CK_LIB points at it.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
TRACE_LIB = os.path.join(HERE, "lib", "libck_b200_trace.so")
OBJ_DIR = os.path.join(HERE, "build", "trace")


def build(stages: bool = False) -> str:
    sys.path.insert(0, HERE)
    import build as base  # the production build recipe: same flags plus the trace macro

    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(os.path.dirname(TRACE_LIB), exist_ok=True)
    nvcc = base._nvcc()
    procs, objs = [], []
    for src in base._sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        macros = ["-DCK_GEMM_TRACE"] + (["-DCK_GEMM_TRACE_STAGES"] if stages else [])
        procs.append(subprocess.Popen([nvcc, *base.NVCC_FLAGS, *macros, "-c", src, "-o", obj],
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            print(out)
            raise RuntimeError("nvcc failed")
    subprocess.run([nvcc, "-shared", "-o", TRACE_LIB, *objs, "-cudart", "static", "-Xcompiler", "-fPIC"], check=True)
    return TRACE_LIB


def run(shape: str, ring: int, verbose: bool) -> None:
    os.environ["CK_LIB"] = TRACE_LIB
    sys.path.insert(0, HERE)
    import numpy as np
    import torch

    import comfy_kitchen as ck
    from comfy_kitchen.backends import cuda as be

    lib = be.load_library()
    dev = torch.device("cuda:0")
    m, n, k = (int(v) for v in shape.split(","))
    x = torch.randn(m, k, device=dev).bfloat16()
    w = (torch.randn(n, k, device=dev) * 0.02).bfloat16()
    bias = (torch.randn(n, device=dev) * 0.01).bfloat16()
    sa = (x.abs().amax() / 2688).float()
    sb = (w.abs().amax() / 2688).float()
    qa0, bsa0 = ck.quantize_nvfp4(x, sa, pad_16x=(m % 16 != 0))
    qb0, bsb0 = ck.quantize_nvfp4(w, sb)
    mp = qa0.shape[0]
    qa, bsa = [qa0.clone() for _ in range(ring)], [bsa0.clone() for _ in range(ring)]
    qb, bsb = [qb0.clone() for _ in range(ring)], [bsb0.clone() for _ in range(ring)]
    out = [torch.empty(mp, n, dtype=torch.bfloat16, device=dev) for _ in range(ring)]

    need = int(lib.ck_scaled_mm_workspace_bytes(0, mp, n, k))
    ws = torch.zeros(max(need, 16), dtype=torch.uint8, device=dev)
    small = m <= 32  # the weight-streaming path lives in its own translation unit, with its own buffers
    suffix = "_smallm" if small else ""

    def launch(i, st):
        j = i % ring
        rc = lib.ck_scaled_mm_nvfp4_ws(qa[j].data_ptr(), qb[j].data_ptr(), bsa[j].data_ptr(), bsb[j].data_ptr(), sa.data_ptr(),
                                       sb.data_ptr(), None, bias.data_ptr(), 2, out[j].data_ptr(), 2, mp, n, k,
                                       ws.data_ptr() if need else None, need, st)
        assert rc == 0, lib.ck_last_error()

    side = torch.cuda.Stream()
    launches = 16
    with torch.cuda.stream(side):
        for i in range(3):
            launch(i, side.cuda_stream)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(launches):
                launch(i, side.cuda_stream)
        for _ in range(60):  # ~20 ms: lets the SM clock ramp up before the replay that is kept
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        g.replay()
        e1.record(side)
        torch.cuda.synchronize()
        print(f"graph replay of {launches} launches: {e0.elapsed_time(e1) * 1e3 / launches:.2f} us per launch (instrumented build)")

    # ---- per launch and CTA: global timer and SM clock at entry / set-up done / dependency wait done / end
    stamps = np.zeros((8, 160, 4, 2), dtype=np.int64)
    trace3 = getattr(lib, "ck_debug_trace3" + suffix)
    trace3.argtypes = [ctypes.c_void_p]
    assert trace3(stamps.ctypes.data) == 0
    ncta = int((stamps[0, :, 0, 0] != 0).sum())
    b = stamps[:, :ncta]
    order = np.argsort(b[:, :, 0, 0].min(axis=1))  # the ring holds the last 8 launches
    t0 = b[order[0], :, 0, 0].min()
    names = ["entry", "setup_done", "dep_wait_done", "body_done"]
    prev_end = None
    print(f"{ncta} CTAs; times in us from the first entry of the oldest launch kept")
    for l in order:
        gt = b[l, :, :, 0] - t0
        clk = b[l, :, :, 1]
        mhz = (clk[:, 3] - clk[:, 0]) / np.maximum(1, b[l, :, 3, 0] - b[l, :, 0, 0]) * 1e3
        s = "  ".join(f"{nm} {gt[:, i].min() / 1e3:.2f}/{np.median(gt[:, i]) / 1e3:.2f}/{gt[:, i].max() / 1e3:.2f}" for i, nm in enumerate(names))
        s += f" | SM clock {np.median(mhz):.0f} MHz"
        if prev_end is not None:
            s += f" | period {(gt[:, 3].max() - prev_end) / 1e3:.2f} us"
        prev_end = gt[:, 3].max()
        print(f"launch: (min/median/max) {s}")
    last = order[-1]

    # ---- per tile (SM clock, last launch)
    tiles = np.zeros((160, 40, 16), dtype=np.int64)
    trace = getattr(lib, "ck_debug_trace" + suffix)
    trace.argtypes = [ctypes.c_void_p]
    assert trace(tiles.ctypes.data) == 0
    slots = ["mma:acc_wait", "mma:acc_free", "mma:first_stage", "mma:last_stage", "tma:first", "tma:last", "epi:wait", "epi:acc_full",
             "epi:drained", "epi:done", "epi:loop", "epi:box0_free", "epi:chunk0", "epi:chunk1", "epi:box1_free", "epi:store0"]
    body = (b[last, :, 3, 0] - b[last, :, 2, 0]) / 1e3
    slowest = int(np.argmax(body))
    print(f"body (dependency wait done -> end) per CTA: min {body.min():.2f} us, median {np.median(body):.2f}, max {body.max():.2f} (CTA {slowest})")
    for cta in sorted({0, ncta // 2 - ncta // 2 % 2, ncta - 2, slowest}):
        if cta < 0 or cta >= ncta:
            continue
        base = b[last, cta, 0, 1]
        print(f"--- CTA {cta}: cycles since its entry; set-up done {b[last, cta, 1, 1] - base}, dependency wait done "
              f"{b[last, cta, 2, 1] - base}, body done {b[last, cta, 3, 1] - base}")
        for t in range(12):  # the kernel keeps the stamps of its first 12 tiles (low 32 bits of the counter)
            row = tiles[cta, t]
            if not row.any():
                break
            print(f"  tile {t}: " + "  ".join(f"{nm}={(int(v) - int(base)) & 0xFFFFFFFF}" for nm, v in zip(slots, row) if v))
    if verbose and not small:
        per_stage = np.zeros((160, 4, 64), dtype=np.int64)
        lib.ck_debug_trace2.argtypes = [ctypes.c_void_p]
        assert lib.ck_debug_trace2(per_stage.ctypes.data) == 0
        if not per_stage.any():
            print("(no per-stage stamps: build with --stages)")
            return
        nst = min(48, 3 * ((k // 2 + 127) // 128))
        w_ = per_stage[0, 2, :nst] - per_stage[0, 1, :nst]
        iss = per_stage[0, 3, :nst] - per_stage[0, 2, :nst]
        per = np.diff(per_stage[0, 2, :nst])
        print("CTA 0, MMA warp per stage: cycles waiting for the stage | issuing | stage period")
        print("  wait  :", [int(v) for v in w_])
        print("  issue :", [int(v) for v in iss])
        print("  period:", [int(v) for v in per])


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("command", choices=["build", "run"])
    ap.add_argument("shape", nargs="?", default="4096,3072,3072")
    ap.add_argument("--ring", type=int, default=8)
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--stages", action="store_true", help="build: also record per-stage stamps of the MMA warp")
    a = ap.parse_args()
    if a.command == "build":
        print(build(a.stages))
    else:
        run(a.shape, a.ring, a.verbose)
