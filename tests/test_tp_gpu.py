"""Tensor-parallel Q4 linears on the GPU: the fused exchange path on one GPU (world 1, and a peer
that never answers), and the real multi-rank path on 2+ GPUs when the box has them."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from makepad_b200 import _lib, synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world1_exchange_path_equals_plain_forward(ctx, orc):
    import torch
    import makepad_b200
    from makepad_b200.tensor_parallel import Exchange, RowParallelLinear
    codes, scales = synth.q4_weight(1000, 2048, seed=21)
    ex = Exchange(ctx, 0, 1, max_floats=4 * 1000)
    row = RowParallelLinear(ctx, codes, scales, 0, 1, exchange=ex)
    plain = makepad_b200.QuantLinear(row.w)
    for M in (1, 2, 4):
        x = torch.from_numpy(synth.activations(M, 2048, seed=22)).cuda()
        for _ in range(3):                                   # both halves of the buffer, slots cleared after use
            y = row(x)
        y0 = plain(x)
        torch.cuda.synchronize()
        assert torch.equal(y, y0)
        assert orc.rel_err(y.cpu().numpy(), orc.q4_matmul_f64(codes, scales, x.cpu().numpy()))[1] < 1e-3
    assert ctx.lib.mpq_context_poll_status(ctx.h) == _lib.OK
    # M > 4 is refused by the fused entry point (the host class falls back to the collective path)
    x = torch.zeros((5, 2048), device="cuda")
    y = torch.zeros((5, 1000), device="cuda")
    assert ctx.lib.mpq_q4_linear_forward_allreduce(ctx.h, row.w.h, ex.h, x.data_ptr(), 5, y.data_ptr(), None) == _lib.ERR_UNSUPPORTED
    assert ctx.lib.mpq_q4_linear_forward_allreduce(ctx.h, row.w.h, ex.h, x.data_ptr(), 4, y.data_ptr(), None) == _lib.OK
    # capacity check
    big = synth.q4_weight(4100, 64, seed=1)
    import makepad_b200 as m
    wbig = m.Q4Weight(ctx, *big)
    assert ctx.lib.mpq_q4_linear_forward_allreduce(ctx.h, wbig.h, ex.h, x.data_ptr(), 1, y.data_ptr(), None) == _lib.ERR_UNSUPPORTED
    ex.destroy()


def test_allreduce_output_guard_regions_untouched(ctx):
    import torch
    from makepad_b200.tensor_parallel import Exchange, RowParallelLinear
    N, K, M = 1000, 2048, 3
    codes, scales = synth.q4_weight(N, K, seed=23)
    ex = Exchange(ctx, 0, 1, max_floats=M * N)
    row = RowParallelLinear(ctx, codes, scales, 0, 1, exchange=ex)
    buf = torch.full((M * N + 512,), 321.0, device="cuda")
    y = buf[256:256 + M * N]
    x = torch.from_numpy(synth.activations(M, K, seed=24)).cuda()
    for _ in range(2):
        ctx.check(ctx.lib.mpq_q4_linear_forward_allreduce(ctx.h, row.w.h, ex.h, x.data_ptr(), M, y.data_ptr(), None))
    torch.cuda.synchronize()
    assert (buf[:256] == 321.0).all() and (buf[256 + M * N:] == 321.0).all() and not (y == 321.0).any()
    ex.destroy()


def test_odd_number_of_captured_calls_is_reported(ctx):
    """A replayed graph must hold an even number of calls on one exchange (they alternate between the halves of
    the buffer); the library counts the calls of a stream capture and reports an odd count."""
    import torch
    from makepad_b200.tensor_parallel import Exchange, RowParallelLinear
    lib = ctx.lib
    codes, scales = synth.q4_weight(256, 512, seed=25)
    ex = Exchange(ctx, 0, 1, max_floats=256)
    row = RowParallelLinear(ctx, codes, scales, 0, 1, exchange=ex)
    x = torch.from_numpy(synth.activations(1, 512, seed=26)).cuda()
    y = torch.empty((1, 256), device="cuda")
    side = torch.cuda.Stream()

    def enqueue(n):
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for _ in range(n):
            ctx.check(lib.mpq_q4_linear_forward_allreduce(ctx.h, row.w.h, ex.h, x.data_ptr(), 1, y.data_ptr(), s))

    with torch.cuda.stream(side):
        enqueue(2)                                       # eager calls are not counted
    side.synchronize()
    assert lib.mpq_exchange_graph_check(ex.h) == _lib.OK
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        enqueue(3)
    assert lib.mpq_exchange_graph_check(ex.h) == _lib.ERR_STATE      # odd: reported, and cleared by the check
    assert lib.mpq_exchange_graph_check(ex.h) == _lib.OK
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=side):
        enqueue(1)
    # without the check, the next forward call reports it
    with torch.cuda.stream(side):
        st = lib.mpq_q4_linear_forward_allreduce(ctx.h, row.w.h, ex.h, x.data_ptr(), 1, y.data_ptr(), C.c_void_p(side.cuda_stream))
    assert st == _lib.ERR_STATE and b"odd number" in lib.mpq_last_error(ctx.h)
    assert lib.mpq_exchange_graph_check(ex.h) == _lib.ERR_STATE
    g3 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g3, stream=side):
        enqueue(4)
    assert lib.mpq_exchange_graph_check(ex.h) == _lib.OK
    g3.replay(); g3.replay()
    torch.cuda.synchronize()
    assert lib.mpq_context_poll_status(ctx.h) == _lib.OK
    del g, g2, g3
    ex.destroy()


def test_two_contexts_in_one_process_on_two_devices(orc):
    """Kernel attributes are per device: a second context on another GPU of the same process must work too."""
    import torch
    import makepad_b200
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    codes, scales = synth.q4_weight(512, 4096, seed=27)
    x = synth.activations(2, 4096, seed=28)
    ref = orc.q4_matmul_f64(codes, scales, x)
    for dev in (0, 1):
        c = makepad_b200.Context(dev)
        w = makepad_b200.Q4Weight(c, codes, scales)
        with torch.cuda.device(dev):
            xd = torch.from_numpy(x).to(f"cuda:{dev}")
            y = makepad_b200.QuantLinear(w)(xd)
            torch.cuda.synchronize(dev)
        assert orc.rel_err(y.cpu().numpy(), ref)[1] < 1e-3
        w.destroy()
        c.close()


def test_exchange_call_order_and_arguments(ctx):
    lib = ctx.lib
    h = C.c_void_p()
    assert lib.mpq_exchange_create(ctx.h, 0, 9, 1024, C.byref(h)) == _lib.ERR_INVALID_ARG
    assert lib.mpq_exchange_create(ctx.h, 2, 2, 1024, C.byref(h)) == _lib.ERR_INVALID_ARG
    assert lib.mpq_exchange_create(ctx.h, 0, 2, 0, C.byref(h)) == _lib.ERR_SHAPE
    assert lib.mpq_exchange_create(ctx.h, 0, 2, 4096, C.byref(h)) == _lib.OK
    import torch
    import makepad_b200
    codes, scales = synth.q4_weight(64, 128, seed=2)
    w = makepad_b200.Q4Weight(ctx, codes, scales)
    x = torch.zeros(128, device="cuda"); y = torch.zeros(64, device="cuda")
    # used before the peers were attached
    assert lib.mpq_q4_linear_forward_allreduce(ctx.h, w.h, h, x.data_ptr(), 1, y.data_ptr(), None) == _lib.ERR_STATE
    assert lib.mpq_exchange_set_wait_limit(h, 0) == _lib.ERR_INVALID_ARG
    assert lib.mpq_exchange_destroy(h) == _lib.OK
    assert lib.mpq_exchange_destroy(None) == _lib.ERR_INVALID_ARG


def test_silent_peer_times_out_and_is_reported():
    """Rank 0 of a world of 2 whose peer never writes: the bounded wait runs out, the kernel returns, the
    status word says so, and the context stays usable.  The 'peer' is a second buffer on the same GPU
    that nothing fills; no kernel waits on another kernel here."""
    import torch
    import makepad_b200
    ctx = makepad_b200.Context(0)
    lib = ctx.lib
    h = C.c_void_p()
    assert lib.mpq_exchange_create(ctx.h, 0, 2, 4096, C.byref(h)) == _lib.OK
    nbytes = C.c_int64()
    lib.mpq_exchange_buffer(h, None, C.byref(nbytes))
    peer = torch.zeros(nbytes.value, dtype=torch.uint8, device="cuda")
    ptrs = (C.c_void_p * 2)(None, peer.data_ptr())
    assert lib.mpq_exchange_attach_pointers(h, ptrs) == _lib.OK
    assert lib.mpq_exchange_attach_pointers(h, ptrs) == _lib.ERR_STATE
    assert lib.mpq_exchange_set_wait_limit(h, 2000) == _lib.OK
    codes, scales = synth.q4_weight(256, 512, seed=3)
    w = makepad_b200.Q4Weight(ctx, codes, scales, _lib.TP_ROW, 0, 2)
    x = torch.from_numpy(synth.activations(1, 256, seed=3)).cuda()
    y = torch.zeros((1, 256), device="cuda")
    assert lib.mpq_q4_linear_forward_allreduce(ctx.h, w.h, h, x.data_ptr(), 1, y.data_ptr(), None) == _lib.OK
    torch.cuda.synchronize()
    assert lib.mpq_context_poll_status(ctx.h) == _lib.ERR_PEER_TIMEOUT
    assert b"wait ran out" in lib.mpq_last_error(ctx.h)
    assert lib.mpq_context_poll_status(ctx.h) == _lib.OK             # cleared by the first poll
    # the rank's own partial did reach the "peer": 256 tagged pairs in slot 0 of the half this launch used
    assert int(peer.view(torch.int32)[1::2].sum().item()) == 256
    # the context still works
    w2 = makepad_b200.Q4Weight(ctx, codes, scales)
    x2 = torch.from_numpy(synth.activations(1, 512, seed=4)).cuda()
    y2 = makepad_b200.QuantLinear(w2)(x2)
    torch.cuda.synchronize()
    assert torch.isfinite(y2).all() and lib.mpq_context_poll_status(ctx.h) == _lib.OK
    lib.mpq_exchange_destroy(h)
    ctx.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_ranks(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29500 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("TP_WORKER_OK") == world
