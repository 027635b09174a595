"""Tensor-parallel Q4 linears: one process per GPU, torch.distributed for the plumbing.

Column-parallel: rank r keeps output rows [r*N/g, (r+1)*N/g) of W; outputs are
slices, gathered only when the consumer needs the whole vector.
Row-parallel: rank r keeps K-slice [r*K/g, (r+1)*K/g); the partial outputs are
summed over ranks -- inside the GEMV kernel, through peer stores into an
exchange buffer (libmpq), or with NCCL as the baseline path.

The reference snapshot has nothing distributed; the partitioning follows the
task configuration (gate/up column-split, down row-split + all-reduce).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .decode_stack import SHAPES_7B, q4_bytes, random_q4_weight_on_device
from .quant_linear import Context, MpqError, Q4Weight


def shard_range(total: int, rank: int, world: int, multiple: int = 1):
    """[begin, end) of rank's contiguous equal share; the share must be a multiple of `multiple`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} / world {world}")
    if total % (world * multiple):
        raise ValueError(f"{total} does not split into {world} shares that are multiples of {multiple}")
    n = total // world
    return rank * n, (rank + 1) * n


def shard_q4(codes: np.ndarray, scales: np.ndarray, mode: int, rank: int, world: int):
    """The canonical arrays of one rank's shard (host-side view of what the library keeps)."""
    N, K = codes.shape[0], codes.shape[1] * 2
    if mode == _lib.TP_COLUMN:
        a, b = shard_range(N, rank, world)
        return codes[a:b], scales[a:b]
    if mode == _lib.TP_ROW:
        a, b = shard_range(K, rank, world, 32)
        return codes[:, a // 2:b // 2], scales[:, a // 32:b // 32]
    return codes, scales


class Exchange:
    """A buffer on every rank that every rank can write (see include/mpq.h)."""

    def __init__(self, ctx: Context, rank: int, world: int, max_floats: int, group=None):
        self.ctx, self.rank, self.world = ctx, rank, world
        h = C.c_void_p()
        ctx.check(ctx.lib.mpq_exchange_create(ctx.h, rank, world, max_floats, C.byref(h)))
        self.h = h
        if world > 1:
            import torch.distributed as dist
            mine = (C.c_uint8 * 64)()
            st = ctx.lib.mpq_exchange_ipc_handle(self.h, mine)
            if st != _lib.OK:
                raise MpqError(st, "cudaIpcGetMemHandle failed")
            handles = [None] * world
            dist.all_gather_object(handles, bytes(mine), group=group)
            blob = (C.c_uint8 * (64 * world)).from_buffer_copy(b"".join(handles))
            st = ctx.lib.mpq_exchange_attach(self.h, blob)
            if st != _lib.OK:
                raise MpqError(st, "cudaIpcOpenMemHandle failed (is peer access available between the GPUs?)")
            dist.barrier(group=group)

    def set_wait_limit(self, polls: int):
        self.ctx.check(self.ctx.lib.mpq_exchange_set_wait_limit(self.h, polls))

    def destroy(self):
        if self.h:
            self.ctx.lib.mpq_exchange_destroy(self.h)
            self.h = None


class ColumnParallelLinear:
    """y[:, shard] = x . W[shard]^T; gather=True returns the whole y on every rank (NCCL all-gather)."""

    def __init__(self, ctx: Context, codes, scales, rank: int, world: int, gather: bool = False, group=None):
        self.w = Q4Weight(ctx, codes, scales, _lib.TP_COLUMN, rank, world)
        self.ctx, self.rank, self.world, self.gather, self.group = ctx, rank, world, gather, group

    def forward(self, x):
        import torch
        ctx, w = self.ctx, self.w
        x2 = x.reshape(-1, w.K)
        y = torch.empty((x2.shape[0], w.N), dtype=torch.float32, device=x.device)
        ctx.check(ctx.lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(x2.data_ptr()), x2.shape[0], C.c_void_p(y.data_ptr()),
                                                C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        if not self.gather or self.world == 1:
            return y
        import torch.distributed as dist
        parts = torch.empty((self.world, x2.shape[0], w.N), dtype=torch.float32, device=x.device)
        dist.all_gather_into_tensor(parts, y, group=self.group)
        return parts.permute(1, 0, 2).reshape(x2.shape[0], self.world * w.N)

    __call__ = forward


class RowParallelLinear:
    """y = sum over ranks of x[:, shard] . W[:, shard]^T.

    With an exchange and M <= 4 the sum is fused into the kernel (peer stores over
    NVLink); otherwise the partial output is reduced with NCCL.
    """

    def __init__(self, ctx: Context, codes, scales, rank: int, world: int, exchange: Exchange | None = None, group=None):
        self.w = Q4Weight(ctx, codes, scales, _lib.TP_ROW, rank, world)
        self.ctx, self.rank, self.world, self.ex, self.group = ctx, rank, world, exchange, group

    def forward(self, x_shard, fused: bool | None = None):
        import torch
        ctx, w = self.ctx, self.w
        x2 = x_shard.reshape(-1, w.K)
        M = x2.shape[0]
        y = torch.empty((M, w.N), dtype=torch.float32, device=x_shard.device)
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        use_fused = (self.ex is not None and M <= 4) if fused is None else fused
        if use_fused:
            st = ctx.lib.mpq_q4_linear_forward_allreduce(ctx.h, w.h, self.ex.h, C.c_void_p(x2.data_ptr()), M, C.c_void_p(y.data_ptr()), s)
            if st != _lib.ERR_UNSUPPORTED:
                ctx.check(st)
                return y
        ctx.check(ctx.lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(x2.data_ptr()), M, C.c_void_p(y.data_ptr()), s))
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(y, group=self.group)
        return y

    __call__ = forward


class TpDecodeStack:
    """The 7B-shape decode stack sharded over `world` GPUs: QKV and gate+up column-split, O and down
    row-split with the sum over ranks fused into the kernel.  Same interface as DecodeStack."""

    # (name, N, K, mode)
    LAYOUT = (("qkv", 12288, 4096, _lib.TP_COLUMN), ("o", 4096, 4096, _lib.TP_ROW),
              ("gate_up", 22016, 4096, _lib.TP_COLUMN), ("down", 4096, 11008, _lib.TP_ROW))
    # the 70B-shape FFN: gate+up 8192 -> 2 x 28672 column-split, down 28672 -> 8192 row-split + sum over ranks
    LAYOUT_70B_FFN = (("gate_up", 57344, 8192, _lib.TP_COLUMN), ("down", 8192, 28672, _lib.TP_ROW))

    def __init__(self, ctx: Context, rank: int, world: int, layers: int = 32, M: int = 1, seed: int = 0, fused: bool = True,
                 layout=None, keep_layer0: bool = False):
        import torch
        self.ctx, self.rank, self.world, self.layers, self.M, self.fused = ctx, rank, world, layers, M, fused
        if layout is not None:
            self.LAYOUT = tuple(layout)
        self.dev = torch.device(f"cuda:{ctx.device}")
        row_n = max([N for (_, N, _, mode) in self.LAYOUT if mode == _lib.TP_ROW] + [1])
        self.ex = Exchange(ctx, rank, world, max_floats=M * row_n) if fused else None
        self.weights, self.modes = [], []
        for layer in range(layers):
            for j, (_, N, K, mode) in enumerate(self.LAYOUT):
                n, k = (N // world, K) if mode == _lib.TP_COLUMN else (N, K // world)
                if mode == _lib.TP_ROW and (K // world) % 32:
                    raise ValueError(f"K={K} does not split into {world} multiples of 32")
                self.weights.append(random_q4_weight_on_device(ctx, n, k, seed + 1000 * rank + layer * len(self.LAYOUT) + j,
                                                               keep_canonical=keep_layer0 and layer == 0))
                self.modes.append(mode)
        self.x_off, self.y_off, xo, yo = [], [], 0, 0
        for w in self.weights:
            self.x_off.append(xo)
            self.y_off.append(yo)
            xo += M * w.K
            yo += M * w.N
        g = torch.Generator(device=self.dev)
        g.manual_seed(seed + 100003 + rank)
        self.x = torch.randn(xo, dtype=torch.float32, device=self.dev, generator=g)
        self.y = torch.empty(yo, dtype=torch.float32, device=self.dev)
        self.x_host = torch.empty(xo, dtype=torch.float32).pin_memory()
        self.x_host.copy_(self.x)
        self.y_last_host = torch.empty(M * self.weights[-1].N, dtype=torch.float32).pin_memory()
        self.stream = torch.cuda.Stream(device=self.dev)
        self.graph = None
        self.bytes_per_step = layers * sum(q4_bytes(N, K, M) for (_, N, K, _) in self.LAYOUT)     # whole job
        self.launches_per_step = layers * len(self.LAYOUT)
        self.kernel_name = "q4_stream_kernel"
        self.use_fused = fused and M <= 4       # the in-kernel sum over ranks covers M <= 4; wider batches reduce with NCCL

    def _enqueue(self):
        import torch
        import torch.distributed as dist
        s = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        lib, ctx = self.ctx.lib, self.ctx
        for i, w in enumerate(self.weights):
            xp = C.c_void_p(self.x.data_ptr() + 4 * self.x_off[i])
            yp = C.c_void_p(self.y.data_ptr() + 4 * self.y_off[i])
            if self.modes[i] == _lib.TP_ROW and self.world > 1:
                if self.use_fused:
                    ctx.check(lib.mpq_q4_linear_forward_allreduce(ctx.h, w.h, self.ex.h, xp, self.M, yp, s))
                else:
                    ctx.check(lib.mpq_q4_linear_forward(ctx.h, w.h, xp, self.M, yp, s))
                    dist.all_reduce(self.y[self.y_off[i]:self.y_off[i] + self.M * w.N])
            else:
                ctx.check(lib.mpq_q4_linear_forward(ctx.h, w.h, xp, self.M, yp, s))

    def capture(self):
        import torch
        import torch.distributed as dist
        with torch.cuda.stream(self.stream):
            self._enqueue()
            before = self.ctx.launches
            self._enqueue()
            self.launches_per_step = self.ctx.launches - before
        self.stream.synchronize()
        if self.world > 1:
            dist.barrier()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream):
            self._enqueue()
        return self

    def step(self):
        self.graph.replay()

    def parity_of_layer0(self, orc, nrows: int = 256):
        """Outputs of the first layer (after a step) against the CPU checker, on `nrows` sampled output rows per
        projection.  Column-parallel projections: each rank checks its own slice.  Row-parallel ones: the ranks'
        canonical shards and activations are gathered on rank 0, which checks the summed output and that every
        rank holds the same bits.  Returns {"max_floored", "max_strict", "ok"} on rank 0, None elsewhere; needs
        keep_layer0=True.  Not part of any timed region."""
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        worst_fl, worst_st, same = 0.0, 0.0, True
        for i in range(len(self.LAYOUT)):
            w = self.weights[i]
            x = self.x[self.x_off[i]:self.x_off[i] + self.M * w.K].view(self.M, w.K).cpu().numpy()
            y = self.y[self.y_off[i]:self.y_off[i] + self.M * w.N].view(self.M, w.N)
            rows = np.unique(np.random.default_rng(i).choice(w.N, min(nrows, w.N), replace=False))
            got = y[:, torch.from_numpy(rows).to(y.device)].cpu().numpy()
            if self.modes[i] == _lib.TP_COLUMN or self.world == 1:
                ref = orc.q4_matmul_f64(w.codes_host[rows], w.scales_host[rows], x)
                st, fl = orc.rel_err(got, ref)
                local = (st, fl, True)
            else:
                parts = [None] * self.world
                dist.all_gather_object(parts, (w.codes_host[rows], w.scales_host[rows], x, got))
                if self.rank == 0:
                    ref = sum(orc.q4_matmul_f64(c, s_, x_) for (c, s_, x_, _) in parts)
                    st, fl = orc.rel_err(got, ref)
                    local = (st, fl, all(np.array_equal(parts[0][3], g) for (_, _, _, g) in parts))
                else:
                    local = (0.0, 0.0, True)
            allv = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(allv, local)
            else:
                allv = [local]
            worst_st = max([worst_st] + [a[0] for a in allv])
            worst_fl = max([worst_fl] + [a[1] for a in allv])
            same = same and all(a[2] for a in allv)
        if self.rank != 0:
            return None
        return {"max_floored": worst_fl, "max_strict": worst_st, "ranks_hold_same_bits": same, "ok": bool(worst_fl < 1e-3 and same),
                "checked": f"layer 0, {nrows} sampled output rows per projection, against the CPU checker (binary64)"}

    def step_host(self):
        import torch
        with torch.cuda.stream(self.stream):
            self.x.copy_(self.x_host, non_blocking=True)
            self.graph.replay()
            last = self.weights[-1]
            self.y_last_host.copy_(self.y[self.y_off[-1]:self.y_off[-1] + self.M * last.N], non_blocking=True)
        self.stream.synchronize()
        return self.y_last_host

    @property
    def h2d_bytes_per_step(self) -> int:
        return self.x.numel() * 4

    @property
    def d2h_bytes_per_step(self) -> int:
        return self.y_last_host.numel() * 4

    def destroy(self):
        """Free the graph, the weights and the exchange (every rank calls it at the same point)."""
        import torch
        torch.cuda.synchronize()
        self.graph = None
        for w in self.weights:
            w.destroy()
        self.weights = []
        if self.ex is not None:
            self.ex.destroy()
            self.ex = None
