"""The 7B-shape decode layer stack: 32 layers of Q4 projections driven as one CUDA graph.

Per layer: QKV 4096->12288, O 4096->4096, gate+up 4096->2*11008, down 11008->4096.
Only the block-quantised linear operators are in scope (attention, norms and the
activation function between them are not), so the chain is shape-only: every
projection reads its own activation buffer.  The launches are nevertheless
issued in stream order with programmatic dependent launch, exactly as a real
decode step would issue them: each kernel prefetches its weights early and
reads its activation only after the previous kernel has completed.

torch owns the buffers, the stream and the graph; every operator runs in libmpq.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .quant_linear import Context, MpqError

SHAPES_7B = (("qkv", 12288, 4096), ("o", 4096, 4096), ("gate_up", 22016, 4096), ("down", 4096, 11008))
SHAPES_70B_FFN = (("gate_up", 57344, 8192), ("down", 8192, 28672))


def q4_bytes(N: int, K: int, M: int = 1) -> int:
    """Algorithmic bytes of one Q4 linear: codes + fp16 scales + fp32 activations in and out."""
    return N * K // 2 + (N * K // 32) * 2 + 4 * M * K + 4 * M * N


class _DevWeight:
    def __init__(self, ctx: Context, h, N, K):
        self.ctx, self.h, self.N, self.K = ctx, h, N, K

    def destroy(self):
        if self.h:
            self.ctx.lib.mpq_weight_destroy(self.h)
            self.h = None


def random_q4_weight_on_device(ctx: Context, N: int, K: int, seed: int, keep_canonical: bool = False):
    """Q4 weight with the configured distributions (codes uniform in [-8,7], scale = fp16(|z|*0.02)),
    drawn on the GPU with torch's generator and repacked by the library."""
    import torch
    g = torch.Generator(device=f"cuda:{ctx.device}")
    g.manual_seed(seed)
    codes = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=g.device, generator=g)
    z = torch.randn((N, K // 32), dtype=torch.float32, device=g.device, generator=g)
    scales = (z.abs() * 0.02).to(torch.float16).view(torch.int16)
    h = C.c_void_p()
    ctx.check(ctx.lib.mpq_q4_weight_create_dev(ctx.h, N, K, C.c_void_p(codes.data_ptr()), C.c_void_p(scales.data_ptr()),
                                               C.byref(h)))
    w = _DevWeight(ctx, h, N, K)
    if keep_canonical:
        w.codes_host = codes.cpu().numpy()
        w.scales_host = scales.cpu().numpy().view(np.uint16)
    return w


class DecodeStack:
    """`layers` x len(shapes) Q4 projections with M activation rows, captured as one CUDA graph."""

    def __init__(self, ctx: Context, layers: int = 32, M: int = 1, shapes=SHAPES_7B, seed: int = 0, keep_layer0: bool = False):
        import torch
        self.ctx, self.layers, self.M, self.shapes = ctx, layers, M, shapes
        self.dev = torch.device(f"cuda:{ctx.device}")
        self.weights = []
        for layer in range(layers):
            for j, (_, N, K) in enumerate(shapes):
                self.weights.append(random_q4_weight_on_device(ctx, N, K, seed + layer * len(shapes) + j,
                                                               keep_canonical=keep_layer0 and layer == 0))
        # one activation slab and one output slab for the whole step; projection i uses slice i
        self.x_off, self.y_off, xo, yo = [], [], 0, 0
        for layer in range(layers):
            for (_, N, K) in shapes:
                self.x_off.append(xo)
                self.y_off.append(yo)
                xo += M * K
                yo += M * N
        g = torch.Generator(device=self.dev)
        g.manual_seed(seed + 100003)
        self.x = torch.randn(xo, dtype=torch.float32, device=self.dev, generator=g)
        self.y = torch.empty(yo, dtype=torch.float32, device=self.dev)
        self.x_host = torch.empty(xo, dtype=torch.float32).pin_memory()
        self.x_host.copy_(self.x)
        last = self.weights[-1]
        self.y_last_host = torch.empty(M * last.N, dtype=torch.float32).pin_memory()
        self.stream = torch.cuda.Stream(device=self.dev)
        self.graph = None
        self.bytes_per_step = layers * sum(q4_bytes(N, K, M) for (_, N, K) in shapes)
        self.launches_per_step = None          # counted by the library while the step is enqueued (capture())
        self.kernel_name = ("q4_stream_kernel" if M == 1 else
                            "q4_stream_kernel (up to 4 rows of a short K) / q4_rect_kernel (up to 16 rows) / q4_umma_kernel (from 17 rows)")

    def _enqueue(self, first: int = 0, last: int = None):
        import torch
        s = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        lib, ctx = self.ctx.lib, self.ctx
        for i, w in enumerate(self.weights):
            if i < first or (last is not None and i >= last):
                continue
            xp = self.x.data_ptr() + 4 * self.x_off[i]
            yp = self.y.data_ptr() + 4 * self.y_off[i]
            ctx.check(lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(xp), self.M, C.c_void_p(yp), s))

    def capture(self):
        """Warm up (first calls allocate the library's scratch) and capture the step as a graph."""
        import torch
        with torch.cuda.stream(self.stream):
            self._enqueue()
            before = self.ctx.launches
            self._enqueue()
            self.launches_per_step = self.ctx.launches - before
        self.stream.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream):
            self._enqueue()
        # The host-to-host step as one graph of its own: the layers' inputs are copied up in three parts (layer 0; layers
        # 1..3; the rest), each part on a second stream beside the launches of the part before it, so that only the first
        # 93 KB are waited for; the last output is read back at the end.
        n0 = len(self.shapes)
        bounds = sorted({0, min(1, self.layers), min(4, self.layers), self.layers})          # in layers
        parts = [(bounds[i] * n0, bounds[i + 1] * n0) for i in range(len(bounds) - 1)]         # in projections
        xend = lambda j: self.x_off[j] if j < len(self.weights) else self.x.numel()
        side = torch.cuda.Stream(device=self.dev)
        last = self.weights[-1]
        self.graph_host = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_host, stream=self.stream):
            cur = torch.cuda.current_stream(self.dev)
            a0, a1 = xend(parts[0][0]), xend(parts[0][1])
            self.x[a0:a1].copy_(self.x_host[a0:a1], non_blocking=True)
            for k, (p0, p1) in enumerate(parts):
                if k + 1 < len(parts):                               # the next part's inputs travel while this part runs
                    b0, b1 = xend(parts[k + 1][0]), xend(parts[k + 1][1])
                    side.wait_stream(cur)
                    with torch.cuda.stream(side):
                        self.x[b0:b1].copy_(self.x_host[b0:b1], non_blocking=True)
                self._enqueue(p0, p1)
                if k + 1 < len(parts):
                    cur.wait_stream(side)
            self.y_last_host.copy_(self.y[self.y_off[-1]:self.y_off[-1] + self.M * last.N], non_blocking=True)
        return self

    def step(self):
        """One decode step with activations already resident in HBM (enqueue only)."""
        self.graph.replay()

    def step_host(self):
        """One decode step from HOST activations to a HOST result: pinned H2D of every projection's input (in three parts,
        each copied beside the launches of the part before it), the 128 launches, D2H of the last projection's output,
        synchronise."""
        import torch
        with torch.cuda.stream(self.stream):
            self.graph_host.replay()
        self.stream.synchronize()
        return self.y_last_host

    @property
    def h2d_bytes_per_step(self) -> int:
        return self.x.numel() * 4

    @property
    def d2h_bytes_per_step(self) -> int:
        return self.y_last_host.numel() * 4

    def output(self, i: int):
        w = self.weights[i]
        return self.y[self.y_off[i]:self.y_off[i] + self.M * w.N].view(self.M, w.N)

    def input(self, i: int):
        w = self.weights[i]
        return self.x[self.x_off[i]:self.x_off[i] + self.M * w.K].view(self.M, w.K)

    def destroy(self):
        for w in self.weights:
            w.destroy()
        self.weights = []
