"""SwiGLU between the gate+up and the down projection: the stand-alone kernel against a binary64 reference (a
transcendental: tolerance 4 fp32 ulps of the result, stated below), and the fused forms (Q4 down projection with the
SwiGLU in its activation staging, NVFP4 quantisation with the SwiGLU in front) against the unfused chain, bit for bit."""
import ctypes as C

import numpy as np
import pytest

from makepad_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def _gate_up(M, F, seed, scale=3.0):
    """Activations of the gate+up projection: N(0,1) times `scale`; with 3 silu runs through its whole shape
    (about -0.28 at its minimum, linear for large g, 0 for very negative g)."""
    return (synth.activations(M, 2 * F, seed=seed) * scale).astype(np.float32)


@pytest.mark.parametrize("M,F", [(1, 11008), (3, 2112), (64, 4096)])
def test_swiglu_against_binary64(ctx, orc, M, F):
    import makepad_b200
    torch = _torch()
    gu = _gate_up(M, F, 31)
    gu[0, :8] = [0.0, -0.0, 100.0, -100.0, 88.0, -88.0, 1e-30, -1e-30]       # ends of the exponential's range
    h = makepad_b200.swiglu(ctx, torch.from_numpy(gu).cuda()).cpu().numpy()
    ref = orc.swiglu_f64(gu)
    # tolerance: expf (<= 2 ulp), one correctly rounded division, one multiplication: 4 ulp of the fp32 result; and
    # 2^-120 |up| absolute, because the fp32 exponential overflows for gate < -88.7, where silu is below 1e-36 and comes out as -0
    ulp = np.spacing(np.abs(ref).astype(np.float32)).astype(np.float64)
    allowed = 4 * ulp + 2.0 ** -120 * np.abs(gu[:, F:].astype(np.float64))
    err = np.abs(h.astype(np.float64) - ref)
    assert np.all(err <= allowed), float(np.max(err / allowed))
    assert np.isfinite(h).all()
    assert ctx.lib.mpq_swiglu(ctx.h, None, M, F, None, None) == _lib.ERR_INVALID_ARG
    x = torch.zeros(16, device="cuda")
    assert ctx.lib.mpq_swiglu(ctx.h, C.c_void_p(x.data_ptr()), 1, 6, C.c_void_p(x.data_ptr()), None) == _lib.ERR_SHAPE


@pytest.mark.parametrize("N,K", [(4096, 11008), (1000, 2112)])
def test_q4_down_projection_with_fused_swiglu(ctx, orc, N, K):
    """Fused (M <= 4: inside the streaming kernel's staging) and unfused (larger M) forms give the bits of
    mpq_swiglu followed by mpq_q4_linear_forward, and agree with the binary64 chain to the Q4 tolerance."""
    import makepad_b200
    torch = _torch()
    codes, scales = synth.q4_weight(N, K, seed=32)
    w = makepad_b200.Q4Weight(ctx, codes, scales)
    lin = makepad_b200.QuantLinear(w)
    for M in (1, 2, 4, 7, 40):
        gu = _gate_up(M, K, 33 + M, scale=1.0)
        gud = torch.from_numpy(gu).cuda()
        y = lin.forward_swiglu(gud)
        y2 = lin(makepad_b200.swiglu(ctx, gud))
        torch.cuda.synchronize()
        assert torch.equal(y, y2), (N, K, M)
        ref = orc.q4_matmul_f64(codes, scales, orc.swiglu_f64(gu))
        rep = orc.err_report(y.cpu().numpy(), ref)
        # The activation carries up to 4 ulp of SwiGLU error and is heavier-tailed than N(0,1) (its largest element is
        # about 13 times its rms, against 4.2), and the kernel's error scales with that ratio: 3e-3 floored relative and
        # 5e-5 of the output rms here, against 1e-3 and 2e-5 for the N(0,1) activations of the plain forward tests.
        assert rep["floored_1e-2_rms"] < 3e-3 and rep["max_abs_over_rms"] < 5e-5, (N, K, M, rep)
    w.destroy()
    assert ctx.lib.mpq_context_poll_status(ctx.h) == _lib.OK


@pytest.mark.parametrize("M,F", [(5, 4096), (128, 14336)])
def test_nvfp4_quantisation_with_fused_swiglu(ctx, orc, M, F):
    """codes and scale bytes equal those of quantising mpq_swiglu's output, which the checker's quantiser reproduces."""
    import makepad_b200
    torch = _torch()
    gu = _gate_up(M, F, 41)
    gud = torch.from_numpy(gu).cuda()
    h = makepad_b200.swiglu(ctx, gud)
    for ts in (1.0, 0.37):
        c1, s1 = makepad_b200.nvfp4_quantize(ctx, gud, ts, swiglu_fused=True)
        c2, s2 = makepad_b200.nvfp4_quantize(ctx, h, ts)
        torch.cuda.synchronize()
        assert torch.equal(c1, c2) and torch.equal(s1, s2)
        want_c, want_s = orc.nvfp4_quantize(h.cpu().numpy(), ts)
        assert np.array_equal(c1.cpu().numpy(), want_c) and np.array_equal(s1.cpu().numpy(), want_s)
    # bf16 input: converted to fp32 first, then the same arithmetic
    gub = gud.to(torch.bfloat16)
    c3, s3 = makepad_b200.nvfp4_quantize(ctx, gub, 1.0, swiglu_fused=True)
    c4, s4 = makepad_b200.nvfp4_quantize(ctx, makepad_b200.swiglu(ctx, gub.float()), 1.0)
    torch.cuda.synchronize()
    assert torch.equal(c3, c4) and torch.equal(s3, s4)
