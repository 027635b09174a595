"""Per-phase timeline of the Q4 streaming kernel inside a replayed CUDA graph (diagnostic).

    python -m makepad_b200.build --trace        # builds libmpq_trace.so (here or on the GPU box)
    python -m makepad_b200.timeline [--layers 3] [--m 1]

Runs `layers` 7B-shape decode layers (QKV, O, gate+up, down; distinct weights) as one CUDA graph with
programmatic dependent launch, exactly as the benchmark's stack does, using the diagnostic build of the
library in which thread 0 of every CTA stamps %globaltimer when it has
  0 started, 1 computed its runs, 2 issued its first ring copies, 3 returned from griddepcontrol.wait,
  4 staged the activation, 5 drained its own run, 6 passed the CTA barrier, 7 merged and stored its tiles,
and warp 0 counts the cycles of its run: in total, waiting for its copies, and in the warp barrier + refill.
Prints, per launch of the last layers, min / median / max over CTAs of each stamp in microseconds since
the first stamp, so that the gaps between launches and the phases inside one can be read off.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os

import numpy as np

NAMES = ["start", "runs", "issued", "waited", "staged", "drained", "synced", "merged"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--m", type=int, default=1)
    args = ap.parse_args()
    import torch
    from . import _lib, build
    _lib.LIB_PATH = build.build(trace=True)          # before the first load: this process uses the diagnostic library
    from .decode_stack import SHAPES_7B, random_q4_weight_on_device
    from .quant_linear import Context
    ctx = Context(0)
    ws, shapes = [], []
    for layer in range(args.layers):
        for j, (_, N, K) in enumerate(SHAPES_7B):
            ws.append(random_q4_weight_on_device(ctx, N, K, layer * 4 + j))
            shapes.append((N, K))
    n = len(ws)
    assert n <= 32, "the trace ring holds 64 launches: at most 8 layers"
    xs = [torch.randn(args.m, K, device="cuda") for (_, K) in shapes]
    ys = [torch.empty(args.m, N, device="cuda") for (N, _) in shapes]
    side = torch.cuda.Stream()

    def run_all():
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for w, x, y in zip(ws, xs, ys):
            ctx.check(ctx.lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(x.data_ptr()), args.m, C.c_void_p(y.data_ptr()), s))

    with torch.cuda.stream(side):
        run_all()                                   # launches 0 .. n-1 (eager: allocates the scratch)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        run_all()                                   # launches n .. 2n-1: these trace slots are what the replays fill
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    lib = ctx.lib
    lib.mpq_debug_trace.restype = C.c_void_p
    lib.mpq_debug_trace.argtypes = [C.POINTER(C.c_int32)]
    count = C.c_int32()
    ptr = lib.mpq_debug_trace(C.byref(count))
    arr = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint64)), shape=(64, 1024, 16)).copy()
    t0 = None
    prev_done = None
    for i in range(max(0, n - 8), n):
        slot = (n + i) % 64
        N, K = shapes[i]
        nct = int((arr[slot, :, 0] > 0).sum())
        a = arr[slot, :nct, :8].astype(np.int64)
        cyc = arr[slot, :nct, 8:13].astype(np.int64)
        if t0 is None:
            t0 = a[:, 0].min()
        a = a - t0
        cols = " ".join(f"{nm} {a[:, k].min() / 1e3:.2f}/{np.median(a[:, k]) / 1e3:.2f}/{a[:, k].max() / 1e3:.2f}" for k, nm in enumerate(NAMES))
        gap = "" if prev_done is None else f" | last CTA done -> previous launch's last done: {(a[:, 7].max() - prev_done) / 1e3:.2f} us"
        print(f"launch {i} {N}x{K} M={args.m} ctas {nct}: {cols}{gap}")
        ng = np.maximum(cyc[:, 3], 1)
        print(f"    warp 0 of each CTA, cycles (median over CTAs): whole run {np.median(cyc[:, 0]):.0f} for {np.median(ng):.0f} groups = "
              f"{np.median(cyc[:, 0] / ng):.0f} per group; waiting for copies {np.median(cyc[:, 1] / ng):.0f} per group; "
              f"warp barrier + refill {np.median(cyc[:, 2] / ng):.0f} per group; first group {np.median(cyc[:, 4]):.0f}")
        prev_done = a[:, 7].max()
    ctx.check(lib.mpq_context_poll_status(ctx.h))


if __name__ == "__main__":
    main()
