#!/usr/bin/env python
"""Benchmark of the block-quantised linear hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the 7B-shape decode layer stack, M = 1 -- 32 layers of Q4
projections (QKV 4096->12288, O 4096->4096, gate+up 4096->2*11008, down
11008->4096), 3.64 GB of weights resident in HBM, one step = one token = 128
dependent launches replayed as a CUDA graph.  Metric: decode tokens/s of the
linear stack; the roofline object reports the same run as HBM GB/s.

Synthetic data: weights and activations are drawn on the GPU with the
distributions the task configuration states (codes uniform in [-8,7], fp16
scales |N(0,1)|*0.02, activations N(0,1)); there is no dataset in this path.

--impl reference times the CPU restatement of the same path (the reference
snapshot holds no implementation of it, so the oracle port is the only CPU
arm there is) on all host threads, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one q4_stream_kernel launch / its algorithmic bytes, from an ncu
# capture of the 22016 x 4096 projection (the weights are streamed exactly once, evict-first)
TRAFFIC_OVER_ALGORITHMIC = 1.007
Q_CLOCKS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path = gpu_index, None, f"/tmp/mpq_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={Q_CLOCKS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, power = [], set(), []
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); out["sm_max_mhz"] = float(f[2]); power.append(float(f[3]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["power_w_max"] = max(power) if power else None
        out["reasons"], out["samples"] = sorted(reasons), len(sm)
        return out


def cpu_arm(steps: int, warmup: int, threads: int):
    """tokens/s of the CPU restatement: each step is ONE layer (4 projections, 1/32 of a token)."""
    import numpy as np
    from makepad_b200 import synth
    from makepad_b200.decode_stack import SHAPES_7B
    from oracle import oracle as orc
    orc.build()
    ws = [synth.q4_weight(N, K, seed=0, stream=j) + (synth.activations(1, K, seed=0, stream=j),)
          for j, (_, N, K) in enumerate(SHAPES_7B)]
    def layer():
        for codes, scales, x in ws:
            orc.q4_matmul_f32(codes, scales, x, threads=threads)
    for _ in range(warmup):
        layer()
    t0 = time.perf_counter()
    for _ in range(steps):
        layer()
    dt = (time.perf_counter() - t0) / steps
    return 1.0 / (32 * dt), dt


def _time_graph(torch, enqueue, stream, reps):
    """Median-free simple timing: capture `enqueue` as a graph, replay `reps` times between CUDA events (us per replay)."""
    with torch.cuda.stream(stream):
        enqueue(); enqueue()
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        enqueue()
    g.replay(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def _time_stack(torch, st, reps):
    """us per replay of a captured stack, CUDA events on its stream."""
    for _ in range(3):
        st.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st.stream):
        e0.record()
        for _ in range(reps):
            st.step()
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def ceilings(ctx):
    """Measured ceilings: read-only HBM streaming over 4 GiB, and the FP4 tensor pipe issuing MMAs with nothing in its way."""
    import ctypes as C
    import torch
    out = {}
    n = 4 << 30
    buf = torch.empty(n, dtype=torch.uint8, device="cuda")
    buf.random_(0, 256)
    sink = torch.zeros(4, dtype=torch.int32, device="cuda")
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        ctx.check(ctx.lib.mpq_probe_hbm_read(ctx.h, C.c_void_p(buf.data_ptr()), n, C.c_void_p(sink.data_ptr()), s))
    torch.cuda.synchronize()
    ts = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.check(ctx.lib.mpq_probe_hbm_read(ctx.h, C.c_void_p(buf.data_ptr()), n, C.c_void_p(sink.data_ptr()), s))
        e1.record(); torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    out["hbm_read_only_gbs"] = n / (min(ts) * 1e-3) / 1e9
    del buf
    torch.cuda.empty_cache()
    flop = C.c_double()
    mmas = 16384
    for _ in range(2):
        ctx.check(ctx.lib.mpq_probe_fp4_mma(ctx.h, mmas, C.byref(flop), s))
    torch.cuda.synchronize()
    ts = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.check(ctx.lib.mpq_probe_fp4_mma(ctx.h, mmas, C.byref(flop), s))
        e1.record(); torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    out["fp4_mma_only_tflops"] = flop.value / (min(ts) * 1e-3) / 1e12
    out["fp4_mma_only_note"] = f"{mmas} tcgen05.mma kind::mxf4nvf4 128x224x64 per SM, operands resident, best of 5"
    # issue rate of small fp16 MMAs (what the Q4 tcgen05 kernel is built around): SM cycles per MMA of 128 x n x 16
    cyc = C.c_double()
    issue = {}
    for n_cols in (32, 64):
        for issuers in (1, 2, 4):
            ctx.check(ctx.lib.mpq_probe_f16_mma(ctx.h, n_cols, issuers, 4096, C.byref(cyc)))
            issue[f"n{n_cols}_issuers{issuers}"] = round(cyc.value, 1)
    out["f16_mma_cycles_per_mma"] = issue
    out["f16_mma_note"] = "tcgen05.mma kind::f16 128 x n x 16, A in tensor memory, 4096 per issuing thread; the pipe needs n/2 cycles per MMA"
    return out


def extras(ctx, peak):
    """The other configurations of the task, measured in the same run (N = 1): single Q4 matvec (config 0),
    small-M verify batches (config 2), NVFP4 prefill GEMM (config 3), the 70B-shape FFN on one GPU (config 4)."""
    import ctypes as C
    import torch
    import makepad_b200
    from makepad_b200.decode_stack import DecodeStack, SHAPES_70B_FFN, q4_bytes, random_q4_weight_on_device
    out = ceilings(ctx)
    read_peak = out["hbm_read_only_gbs"]
    side = torch.cuda.Stream()
    # config 0: 4096 x 4096, M = 1; 43 distinct copies so that every launch misses L2
    ws = [random_q4_weight_on_device(ctx, 4096, 4096, 1000 + i) for i in range(43)]
    x = torch.randn(1, 4096, device="cuda"); y = torch.empty(1, 4096, device="cuda")
    def enq():
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for w in ws:
            ctx.check(ctx.lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(x.data_ptr()), 1, C.c_void_p(y.data_ptr()), s))
    us = _time_graph(torch, enq, side, 10) / len(ws)
    b = q4_bytes(4096, 4096, 1)
    out["q4_matvec_4096x4096_m1"] = {"us": us, "gbs": b / us / 1e3, "frac_of_hbm_peak": b / us / 1e3 / peak,
                                     "frac_of_read_only_peak": b / us / 1e3 / read_peak, "frac_of_nominal_8tbs": b / us / 1e3 / 8000.0}
    for w in ws:
        w.destroy()
    # config 2: small-M verify batches on the 7B shapes (4 layers of distinct weights = 455 MB > L2)
    small = {}
    for M in (1, 2, 4, 8, 16):
        st = DecodeStack(ctx, layers=4, M=M, seed=7).capture()
        us_layer = _time_stack(torch, st, 20) / 4
        small[f"M={M}"] = {"us_per_layer": us_layer, "gbs": st.bytes_per_step / 4 / us_layer / 1e3, "launches_per_layer": st.launches_per_step // 4}
        st.destroy()
    for k in small:
        small[k]["time_vs_m1"] = small[k]["us_per_layer"] / small["M=1"]["us_per_layer"]
    out["q4_small_m_7b_layer"] = small
    # config 4 on one GPU: 70B-shape FFN at both batch widths (two copies of each weight: 793 MB per pass)
    for M in (1, 64):
        st = DecodeStack(ctx, layers=2, M=M, shapes=SHAPES_70B_FFN, seed=9).capture()
        us_ffn = _time_stack(torch, st, 20 if M == 1 else 5) / 2
        gbs = st.bytes_per_step / 2 / us_ffn / 1e3
        out[f"q4_70b_ffn_m{M}"] = {"us_per_ffn": us_ffn, "gbs": gbs, "frac_of_hbm_peak": gbs / peak, "frac_of_read_only_peak": gbs / read_peak,
                                   "launches_per_ffn": st.launches_per_step // 2}
        st.destroy()
    out["q4_70b_ffn_m64"]["time_vs_m1"] = out["q4_70b_ffn_m64"]["us_per_ffn"] / out["q4_70b_ffn_m1"]["us_per_ffn"]
    # config 3: NVFP4 prefill GEMM 2048 x 4096 x 14336 -> bf16, L2 flushed between launches
    M, N, K = 2048, 14336, 4096
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    bq = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    # scale factors as the configuration states them: e4m3(|N(0,1)| * 0.1)
    sfa = (torch.randn((M, K // 16), device="cuda", generator=g).abs() * 0.1).to(torch.float8_e4m3fn).view(torch.uint8)
    sfb = (torch.randn((N, K // 16), device="cuda", generator=g).abs() * 0.1).to(torch.float8_e4m3fn).view(torch.uint8)
    w = makepad_b200.Nvfp4Weight(ctx, bq.cpu().numpy(), sfb.cpu().numpy(), 1.0)
    lin = makepad_b200.QuantLinear(w)
    c = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        lin((a, sfa, 1.0), out=c)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(15):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); lin((a, sfa, 1.0), out=c); e1.record(); torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    us = ts[len(ts) // 2]
    tf = 2.0 * M * N * K / us / 1e6
    out["nvfp4_gemm_2048x4096x14336"] = {"us": us, "tflops": tf, "frac_of_nominal_dense_fp4_9pf": tf / 9000.0,
                                         "frac_of_measured_mma_only": tf / out["fp4_mma_only_tflops"],
                                         "note": "one mpq_nvfp4_gemm_forward call; L2 flushed between launches; scales e4m3(|N(0,1)|*0.1)"}
    w.destroy()
    return out


def one_kernel(spec: str, reps: int):
    """`--one q4:NxK:M` or `--one nvfp4:MxNxK`: a few launches of one operator on seeded synthetic data (four weight copies
    for Q4, so that launches miss L2), event-timed; the command the ncu captures under profiles/ run."""
    import ctypes as C
    import torch
    import makepad_b200
    from makepad_b200.decode_stack import q4_bytes, random_q4_weight_on_device
    kind, dims = spec.split(":", 1)
    ctx = makepad_b200.Context(0)
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if kind == "q4":
        shape, M = dims.split(":")
        N, K = (int(v) for v in shape.split("x"))
        M = int(M)
        ws = [random_q4_weight_on_device(ctx, N, K, 100 + i) for i in range(4)]
        x = torch.randn(M, K, device="cuda"); y = torch.empty(M, N, device="cuda")
        def run():
            for w in ws:
                ctx.check(ctx.lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(x.data_ptr()), M, C.c_void_p(y.data_ptr()), s))
        work, unit = q4_bytes(N, K, M) * len(ws), "GB/s"
    else:
        M, N, K = (int(v) for v in dims.split("x"))
        g = torch.Generator(device="cuda"); g.manual_seed(3)
        a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device="cuda", generator=g)
        bq = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda", generator=g)
        sfa = (torch.randn((M, K // 16), device="cuda", generator=g).abs() * 0.1).to(torch.float8_e4m3fn).view(torch.uint8)
        sfb = (torch.randn((N, K // 16), device="cuda", generator=g).abs() * 0.1).to(torch.float8_e4m3fn).view(torch.uint8)
        w = makepad_b200.Nvfp4Weight(ctx, bq.cpu().numpy(), sfb.cpu().numpy(), 1.0)
        lin = makepad_b200.QuantLinear(w)
        c = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        def run():
            lin((a, sfa, 1.0), out=c)
        work, unit = 2.0 * M * N * K, "TFLOP/s"
    run(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record(); torch.cuda.synchronize()
    ctx.check(ctx.lib.mpq_context_poll_status(ctx.h))
    us = e0.elapsed_time(e1) * 1e3 / reps
    print(json.dumps({"one": spec, "us_per_pass": us, "rate": work / us / (1e3 if unit == "GB/s" else 1e6), "unit": unit, "launches": ctx.launches}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="mpq", choices=["mpq", "reference"])
    ap.add_argument("--cpu-steps", type=int, default=20)
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations (config 0, 2, 3, 4 on one GPU)")
    ap.add_argument("--one", default=None, help="q4:NxK:M or nvfp4:MxNxK: run only this operator a few times (for profiler captures)")
    ap.add_argument("--one-reps", type=int, default=2)
    args = ap.parse_args()
    if args.one:
        return one_kernel(args.one, args.one_reps)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    threads = os.cpu_count() or 1
    config = {"workload": "7B-shape Q4 decode layer stack (configs[1]): 32 x {QKV 12288x4096, O 4096x4096, gate+up 22016x4096, "
                          "down 4096x11008}, M=1, fp32 activations",
              "l2": "weights (3.64 GB per step) exceed L2 (126 MB): every launch streams from HBM, no flush needed",
              "parallelism": f"tp{args.gpus}" if args.gpus > 1 else "single GPU"}

    if args.impl == "reference":
        if rank != 0:
            return
        steps = max(1, min(args.steps, 40))
        toks, dt = cpu_arm(steps, max(1, min(args.warmup, 3)), threads)
        sample = f"{steps} timed steps of ONE layer (4 projections, 113.8 MB of Q4 weights = 1/32 token) on {threads} threads"
        print(json.dumps({
            "impl": "reference", "metric": "q4_decode_tokens_per_s_7b_linear_stack", "value": toks, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": dt * 32 * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "cpu_baseline": {"value": toks, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": toks, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement (oracle port) of the path; the reference snapshot holds no implementation of it"}))
        return

    import torch
    import makepad_b200
    from makepad_b200.decode_stack import DecodeStack

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
        from makepad_b200.tensor_parallel import TpDecodeStack
        ctx = makepad_b200.Context(local_rank)
        stack = TpDecodeStack(ctx, rank, world, keep_layer0=True).capture()
    else:
        dist = None
        ctx = makepad_b200.Context(local_rank)
        stack = DecodeStack(ctx, layers=32, M=1).capture()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    # ---- device-resident arm
    for _ in range(max(3, args.warmup)):
        stack.step()
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stack.stream):
        e0.record()
        for _ in range(args.steps):
            stack.step()
        e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    # ---- end-to-end arm: host activations in, host result out, every step
    for _ in range(3):
        stack.step_host()
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(10, args.steps // 4)
    for _ in range(e2e_steps):
        stack.step_host()
    barrier()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([ms, e2e_s * 1e3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
        e2e_s = e2e_ms / 1e3
    ctx.check(ctx.lib.mpq_context_poll_status(ctx.h))
    import types
    stack_facts = types.SimpleNamespace(launches_per_step=stack.launches_per_step, bytes_per_step=stack.bytes_per_step,
                                        kernel_name=stack.kernel_name, h2d_bytes_per_step=stack.h2d_bytes_per_step,
                                        d2h_bytes_per_step=stack.d2h_bytes_per_step)
    tp_extra = None
    if dist is not None:
        # Correctness evidence for the sharded run, outside every timed region: the first layer's outputs of the stack
        # just timed against the CPU checker (column slices on every rank, the fused row-parallel sums on rank 0).
        from oracle import oracle as orc
        if rank == 0:
            orc.build()
        dist.barrier()
        parity = stack.parity_of_layer0(orc)
        tp_extra = {"parity": parity}
    if dist is not None and not args.no_extra:
        # configuration 4: the 70B-shape FFN layer tensor-parallel over the same ranks, M = 1 and M = 64; enough copies
        # of the layer that each rank's weights exceed L2
        stack.destroy()
        del stack
        torch.cuda.empty_cache()
        from makepad_b200.decode_stack import q4_bytes as _qb
        per_rank = sum(_qb(N, K, 1) for (_, N, K, _) in TpDecodeStack.LAYOUT_70B_FFN) / world
        copies = max(2, int(400e6 // per_rank) + 1)
        copies += copies & 1                 # a replayed graph must hold an even number of calls per exchange
        for Mb in (1, 64):
            ffn = TpDecodeStack(ctx, rank, world, layers=copies, M=Mb, seed=11, layout=TpDecodeStack.LAYOUT_70B_FFN,
                                keep_layer0=True).capture()
            for _ in range(3):
                ffn.step()
            barrier()
            reps = 20 if Mb == 1 else 5
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(ffn.stream):
                f0.record()
                for _ in range(reps):
                    ffn.step()
                f1.record()
            barrier()
            t = torch.tensor([f0.elapsed_time(f1)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us_ffn = float(t.item()) * 1e3 / reps / copies
            par = ffn.parity_of_layer0(orc)
            tp_extra[f"q4_70b_ffn_m{Mb}_tp"] = {"us_per_ffn": us_ffn, "gbs_whole_job": ffn.bytes_per_step / copies / us_ffn / 1e3, "copies": copies,
                                                 "n_gpus": world, "row_parallel_sum": "in-kernel exchange" if ffn.use_fused else "NCCL all-reduce",
                                                 "parity": par}
            ctx.check(ctx.lib.mpq_context_poll_status(ctx.h))
            ffn.destroy()
            del ffn
            torch.cuda.empty_cache()
        stack = None
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    ms_per_step = ms / args.steps
    toks = 1e3 / ms_per_step
    peak, peak_src = measured_peak()
    if stack is None:
        stack = stack_facts
    launches = stack.launches_per_step
    bytes_per_launch = stack.bytes_per_step / launches / max(1, world) if world > 1 else stack.bytes_per_step / launches
    achieved = stack.bytes_per_step / max(1, world) / (ms_per_step * 1e-3) / 1e9      # per GPU
    out = {
        "metric": "q4_decode_tokens_per_s_7b_linear_stack", "value": toks, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "effective_hbm_gbs": stack.bytes_per_step / (ms_per_step * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "kernel": stack.kernel_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": bytes_per_launch, "avg_launch_us": ms_per_step * 1e3 / launches,
                     "traffic": bytes_per_launch * TRAFFIC_OVER_ALGORITHMIC,
                     "traffic_note": "ncu dram bytes of one launch scaled by algorithmic bytes (traffic grows in proportion)"},
        "e2e": {"value": e2e_steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": stack.h2d_bytes_per_step,
                "d2h_bytes_per_step": stack.d2h_bytes_per_step, "ms_per_step": e2e_s * 1e3 / e2e_steps},
        "gpu_launches": launches * args.steps,
        "clocks": clocks,
    }
    if tp_extra is not None:
        out["extra"] = tp_extra
    if world == 1 and not args.no_extra:
        # the same graph replayed for at least two seconds, with the SM clock sampled beside it
        reps = max(200, int(2.2e3 / ms_per_step))
        sampler2 = ClockSampler(local_rank)
        sampler2.start()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stack.stream):
            s0.record()
            for _ in range(reps):
                stack.step()
            s1.record()
        torch.cuda.synchronize()
        sus_ms = s0.elapsed_time(s1) / reps
        clk2 = sampler2.stop()
        sustained = {"steps": reps, "seconds": sus_ms * reps / 1e3, "tokens_per_s": 1e3 / sus_ms, "frac_of_hbm_peak": stack.bytes_per_step / (sus_ms * 1e-3) / 1e9 / peak,
                     "sm_mhz_median": clk2["sm_mhz"], "reasons": clk2["reasons"], "samples": clk2["samples"],
                     "tokens_per_s_per_ghz": (1e3 / sus_ms) / (clk2["sm_mhz"] / 1e3) if clk2["sm_mhz"] else None}
        stack.destroy()
        del stack
        torch.cuda.empty_cache()
        out["extra"] = extras(ctx, peak)
        out["extra"]["sustained"] = sustained
        out["roofline"]["frac_of_read_only_peak"] = achieved / out["extra"]["hbm_read_only_gbs"]
        out["roofline"]["frac_of_nominal_8tbs"] = achieved / 8000.0
        ctx.check(ctx.lib.mpq_context_poll_status(ctx.h))
    if world == 1:
        toks_cpu, dt = cpu_arm(args.cpu_steps, 2, threads)
        out["cpu_baseline"] = {"value": toks_cpu, "unit": "tokens/s", "cores": threads, "kind": "port",
                               "sample": f"{args.cpu_steps} timed passes over ONE layer (4 projections, 113.8 MB, 1/32 token), "
                                         f"{dt * 1e3:.1f} ms per layer"}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
