"""The allocation-free Q4 entry point, for hosts that must not let the library allocate (a fixed memory
budget, a thread that may not enter the CUDA allocator): its scratch is a static device array inside the
library.  Called through the C ABI twice in a row, it must give exactly what the ordinary entry point
gives.  This file is collected last, so a run that stops at the first failure has run everything else.
"""
import ctypes as C

import numpy as np
import pytest

from makepad_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_the_ordinary_one(orc):
    import torch
    import makepad_b200
    ctx = makepad_b200.Context(0)           # a fresh context: the ordinary path's scratch is not even allocated yet
    lib = ctx.lib
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # (1024, 11008) and (1000, 2112) have too few rows for whole tiles per CTA: their row tiles straddle the runs of
    # several CTAs, whose partial sums meet in the static array (the other shapes never touch it)
    for (N, K) in [(4096, 4096), (1024, 11008), (1000, 2112), (4096, 11008)]:
        codes, scales = synth.q4_weight(N, K, seed=31)
        w = makepad_b200.Q4Weight(ctx, codes, scales)
        for M in (1, 3, 4, 7, 20):                                   # M > 4 runs as several launches
            x = torch.from_numpy(synth.activations(M, K, seed=32)).cuda()
            outs = []
            for _ in range(2):                                       # two calls in a row share the static array
                y = torch.full((M, N), float("nan"), device="cuda")
                ctx.check(lib.mpq_q4_linear_forward_static(ctx.h, w.h, C.c_void_p(x.data_ptr()), M, C.c_void_p(y.data_ptr()),
                                                           C.c_void_p(status.data_ptr()), s))
                outs.append(y)
            want = torch.empty((M, N), device="cuda")
            ctx.check(lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(x.data_ptr()), M, C.c_void_p(want.data_ptr()), s))
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            ref = orc.q4_matmul_f64(codes, scales, x.cpu().numpy())
            assert torch.equal(outs[0], outs[1])                     # the second call found the array as clean as the first
            if M == 1 or (M <= 4 and M * K < 16384):                 # the ordinary entry point streams too (one row; several rows
                assert torch.equal(outs[0], want)                    # of a short K): the same kernel, the same runs, the same bits
            else:                                                    # other kernels there: equal to rounding
                rms = float(np.sqrt(np.mean(ref * ref)))
                assert (outs[0] - want).abs().max().item() < 2e-5 * rms
            assert orc.rel_err(want.cpu().numpy(), ref)[1] < 1e-3
            assert orc.rel_err(outs[0].cpu().numpy(), ref)[1] < 1e-3
        w.destroy()
    # NULL status pointer is accepted; bad arguments are rejected like the ordinary entry point's
    codes, scales = synth.q4_weight(64, 128, seed=33)
    w = makepad_b200.Q4Weight(ctx, codes, scales)
    x = torch.zeros(128, device="cuda"); y = torch.zeros(64, device="cuda")
    assert lib.mpq_q4_linear_forward_static(ctx.h, w.h, C.c_void_p(x.data_ptr()), 1, C.c_void_p(y.data_ptr()), None, s) == _lib.OK
    assert lib.mpq_q4_linear_forward_static(ctx.h, w.h, C.c_void_p(x.data_ptr() + 4), 1, C.c_void_p(y.data_ptr()), None, s) == _lib.ERR_ALIGN
    assert lib.mpq_q4_linear_forward_static(ctx.h, w.h, None, 1, C.c_void_p(y.data_ptr()), None, s) == _lib.ERR_INVALID_ARG
    torch.cuda.synchronize()
    # no allocation: with every buffer made beforehand, the device's free memory is the same after a series of calls
    codes, scales = synth.q4_weight(1024, 11008, seed=34)
    w2 = makepad_b200.Q4Weight(ctx, codes, scales)
    x = torch.from_numpy(synth.activations(6, 11008, seed=35)).cuda()
    y = torch.empty((6, 1024), device="cuda")
    ctx.check(lib.mpq_q4_linear_forward_static(ctx.h, w2.h, C.c_void_p(x.data_ptr()), 6, C.c_void_p(y.data_ptr()), None, s))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for M in (1, 2, 4, 6):
        ctx.check(lib.mpq_q4_linear_forward_static(ctx.h, w2.h, C.c_void_p(x.data_ptr()), M, C.c_void_p(y.data_ptr()), None, s))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    # with no status pointer, a timeout would be recorded in the array's own status word, which the context's poll reads
    assert lib.mpq_context_poll_status(ctx.h) == _lib.OK
    ctx.close()
