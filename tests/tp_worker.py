"""Multi-GPU worker for the tensor-parallel tests: run under torchrun, one rank per GPU.

Checks, against the unsharded CPU oracle on the same seeded inputs:
  column-parallel (slices and NCCL all-gather), row-parallel with the fused in-kernel sum over ranks,
  row-parallel with the NCCL all-reduce, and that both row-parallel paths agree.
Prints "TP_WORKER_OK <rank>" on success.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import makepad_b200  # noqa: E402
from makepad_b200 import _lib, synth  # noqa: E402
from makepad_b200.tensor_parallel import ColumnParallelLinear, Exchange, RowParallelLinear, TpDecodeStack  # noqa: E402
from oracle import oracle as orc  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    ctx = makepad_b200.Context(local)
    ex = Exchange(ctx, rank, world, max_floats=4 * 8192)
    TOL = 1e-3
    for (N, K) in [(1024, 2048), (8192, 3584 * world), (4096, 11008 if 11008 % (32 * world) == 0 else 4096)]:
        codes, scales = synth.q4_weight(N, K, seed=7)
        for M in (1, 3, 4, 8):
            x = synth.activations(M, K, seed=8)
            ref = orc.q4_matmul_f64(codes, scales, x)
            xd = torch.from_numpy(x).cuda()
            # column-parallel
            col = ColumnParallelLinear(ctx, codes, scales, rank, world, gather=True)
            y = col(xd)
            torch.cuda.synchronize()
            assert orc.rel_err(y.cpu().numpy(), ref)[1] < TOL, ("column", N, K, M)
            # row-parallel: fused and NCCL
            a, b = rank * (K // world), (rank + 1) * (K // world)
            xs = xd[:, a:b].contiguous()
            row = RowParallelLinear(ctx, codes, scales, rank, world, exchange=ex)
            y_fused = row(xs)                      # fused for M <= 4, NCCL otherwise
            y_nccl = row(xs, fused=False)
            torch.cuda.synchronize()
            ctx.check(ctx.lib.mpq_context_poll_status(ctx.h))
            assert orc.rel_err(y_fused.cpu().numpy(), ref)[1] < TOL, ("row fused", N, K, M)
            assert orc.rel_err(y_nccl.cpu().numpy(), ref)[1] < TOL, ("row nccl", N, K, M)
            rms = float(np.sqrt(np.mean(ref * ref)))
            assert (y_fused - y_nccl).abs().max().item() < 1e-5 * rms
            # every rank holds the same bits after the fused sum (fixed rank order)
            gathered = [torch.empty_like(y_fused) for _ in range(world)]
            dist.all_gather(gathered, y_fused)
            assert all(torch.equal(gathered[0], g) for g in gathered)
            # repeated calls (both halves of the exchange) stay correct
            for _ in range(3):
                y2 = row(xs)
            torch.cuda.synchronize()
            assert torch.equal(y2, y_fused)
            col.w.destroy(); row.w.destroy()
    # the sharded decode stack: graph replay is deterministic and finite
    st = TpDecodeStack(ctx, rank, world, layers=2).capture()
    st.step(); torch.cuda.synchronize()
    y1 = st.y.clone()
    st.step(); st.step(); torch.cuda.synchronize()
    assert torch.equal(y1, st.y) and torch.isfinite(st.y).all()
    ctx.check(ctx.lib.mpq_context_poll_status(ctx.h))
    dist.barrier()
    print(f"TP_WORKER_OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
