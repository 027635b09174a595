"""Parity of the NVFP4 tcgen05 GEMM (through the C ABI) with the CPU oracle.

Tolerance (from the task statement): dequantised values bit-exact; bf16 outputs
within max relative error 2e-2 per element.  Products of e2m1 codes and e4m3
scales are exact and the tensor core accumulates in fp32, so in practice the
only difference from the oracle is the final bf16 rounding: the test also
requires agreement within one bf16 ulp of the binary64-accumulated value.
"""
import ctypes as C
import os

import numpy as np
import pytest

from makepad_b200 import _lib, synth

pytestmark = pytest.mark.gpu
TOL = 2e-2
GOLD = os.path.join(os.path.dirname(__file__), "golden", "nvfp4_small.npz")


def _gemm(ctx, a, sfa, ta, b, sfb, tb):
    import torch
    import makepad_b200
    w = makepad_b200.Nvfp4Weight(ctx, b, sfb, tb)
    y = makepad_b200.QuantLinear(w)((torch.from_numpy(a).cuda(), torch.from_numpy(sfa).cuda(), ta))
    torch.cuda.synchronize()
    assert ctx.lib.mpq_context_poll_status(ctx.h) == _lib.OK
    out = y.view(torch.int16).cpu().numpy().view(np.uint16)
    w.destroy()
    return out


def _check(orc, got_bits, c32):
    got = orc.bf16_bits_to_f32(got_bits).astype(np.float64)
    ref = c32.astype(np.float64)
    strict, floored = orc.rel_err(got, ref)
    assert floored < TOL, (strict, floored)
    # within one bf16 ulp of the exact value (2^-8 relative), plus fp32 accumulation noise
    rms = np.sqrt(np.mean(ref * ref)) + 1e-30
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -8 + 1e-5 * rms)


@pytest.mark.parametrize("R,K", [(1, 16), (5, 48), (224, 256), (300, 4096)])
def test_dequant_bit_exact(ctx, orc, R, K):
    import torch
    codes, sf = synth.nvfp4_tensor(R, K, seed=R + K)
    out = torch.empty((R, K), dtype=torch.float32, device="cuda")
    cd, sd = torch.from_numpy(codes).cuda(), torch.from_numpy(sf).cuda()
    for ts in (1.0, 0.37):
        ctx.check(ctx.lib.mpq_nvfp4_dequantize(ctx.h, R, K, cd.data_ptr(), sd.data_ptr(), C.c_float(ts), out.data_ptr(), None))
        torch.cuda.synchronize()
        want = orc.nvfp4_dequantize(codes, sf, ts)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_dequant_every_code_and_scale(ctx, orc):
    import torch
    # 16 codes x all 127 finite non-negative scales (and the negative ones too)
    sfb = np.arange(256, dtype=np.uint8)
    sfb = sfb[(sfb & 0x7F) != 0x7F]
    codes = synth.pack_nibbles(np.tile(np.arange(16, dtype=np.uint8), (len(sfb), 1)))
    sf = sfb[:, None].copy()
    out = torch.empty((len(sfb), 16), dtype=torch.float32, device="cuda")
    cd, sd = torch.from_numpy(codes).cuda(), torch.from_numpy(sf).cuda()
    ctx.check(ctx.lib.mpq_nvfp4_dequantize(ctx.h, len(sfb), 16, cd.data_ptr(), sd.data_ptr(), C.c_float(1.0), out.data_ptr(), None))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), orc.nvfp4_dequantize(codes, sf, 1.0).view(np.uint32))


def test_weight_export_bit_exact(ctx, orc):
    import makepad_b200
    b, sfb = synth.nvfp4_tensor(448, 512, seed=3)
    w = makepad_b200.Nvfp4Weight(ctx, b, sfb, 0.25)
    assert np.array_equal(w.dequantize().cpu().numpy().view(np.uint32), orc.nvfp4_dequantize(b, sfb, 0.25).view(np.uint32))


@pytest.mark.parametrize("M,N,K", [(128, 224, 256), (128, 224, 1024), (256, 448, 512), (384, 672, 2048),
                                   (100, 200, 320), (1, 8, 32), (129, 232, 288), (2048, 224, 4096)])
def test_gemm_matches_oracle(ctx, orc, M, N, K):
    a, sfa = synth.nvfp4_tensor(M, K, seed=M, stream=0)
    b, sfb = synth.nvfp4_tensor(N, K, seed=M, stream=1)
    c32, c16 = orc.nvfp4_gemm(a, sfa, 0.5, b, sfb, 3.0)
    got = _gemm(ctx, a, sfa, 0.5, b, sfb, 3.0)
    _check(orc, got, c32)
    # the rounding itself agrees with the oracle's on nearly every element (ties in fp32 accumulation order aside)
    assert np.mean(got == c16) > 0.99


@pytest.mark.parametrize("kernel", ["single"])
@pytest.mark.parametrize("M,N,K", [(128, 224, 256), (256, 448, 512), (100, 200, 320), (1, 8, 32), (640, 672, 2048),
                                   (300, 224, 4096), (1200, 2912, 1024)])
def test_single_cta_kernel_matches_oracle(ctx, orc, kernel, M, N, K):
    """The one-CTA-per-tile kernel, used where clusters of two cannot be scheduled (MPQ_FP4_KERNEL=single), computes the same GEMM."""
    a, sfa = synth.nvfp4_tensor(M, K, seed=M + 2, stream=0)
    b, sfb = synth.nvfp4_tensor(N, K, seed=M + 2, stream=1)
    c32, c16 = orc.nvfp4_gemm(a, sfa, 0.5, b, sfb, 3.0)
    os.environ["MPQ_FP4_KERNEL"] = kernel
    try:
        got = _gemm(ctx, a, sfa, 0.5, b, sfb, 3.0)
    finally:
        del os.environ["MPQ_FP4_KERNEL"]
    _check(orc, got, c32)
    assert np.mean(got == c16) > 0.99


def test_many_tiles_per_cta_deterministic(ctx, orc):
    """More tiles than CTA pairs (every pair runs several tiles back to back) and K % 256 != 0 (re-tiled activation scales):
    equal to the oracle and bit-identical between runs and between the two kernels."""
    M, N, K = 1536, 224 * 40, 1056
    a, sfa = synth.nvfp4_tensor(M, K, seed=11, stream=0)
    b, sfb = synth.nvfp4_tensor(N, K, seed=11, stream=1)
    c32, _ = orc.nvfp4_gemm(a, sfa, 1.0, b, sfb, 1.0)
    got = _gemm(ctx, a, sfa, 1.0, b, sfb, 1.0)
    _check(orc, got, c32)
    for _ in range(3):
        assert np.array_equal(_gemm(ctx, a, sfa, 1.0, b, sfb, 1.0), got)
    os.environ["MPQ_FP4_KERNEL"] = "single"
    try:
        assert np.array_equal(_gemm(ctx, a, sfa, 1.0, b, sfb, 1.0), got)
    finally:
        del os.environ["MPQ_FP4_KERNEL"]


def test_known_answers(ctx, orc):
    M, N, K = 128, 224, 256
    one = lambda R: synth.pack_nibbles(np.full((R, K), 2, dtype=np.uint8))
    sf1 = lambda R: np.full((R, K // 16), 0x38, dtype=np.uint8)
    got = orc.bf16_bits_to_f32(_gemm(ctx, one(M), sf1(M), 1.0, one(N), sf1(N), 1.0))
    assert np.all(got == float(K))
    # zero scales zero their blocks; +-0 codes contribute nothing
    z = np.zeros((M, K // 16), dtype=np.uint8)
    assert np.all(orc.bf16_bits_to_f32(_gemm(ctx, one(M), z, 1.0, one(N), sf1(N), 1.0)) == 0.0)
    negzero = synth.pack_nibbles(np.full((M, K), 8, dtype=np.uint8))
    assert np.all(orc.bf16_bits_to_f32(_gemm(ctx, negzero, sf1(M), 1.0, one(N), sf1(N), 1.0)) == 0.0)
    # max magnitudes: 6 * 448 on both sides, K = 256 terms: 256 * (6*448)^2 = 1.85e9 fits fp32 and bf16
    six = lambda R: synth.pack_nibbles(np.full((R, K), 7, dtype=np.uint8))
    big = lambda R: np.full((R, K // 16), 0x7E, dtype=np.uint8)
    got = orc.bf16_bits_to_f32(_gemm(ctx, six(M), big(M), 1.0, six(N), big(N), 1.0))
    want = orc.bf16_bits_to_f32(orc.f32_to_bf16(np.array([256.0 * (6 * 448.0) ** 2], dtype=np.float32)))[0]
    assert np.all(got == want)


def test_golden_vectors(ctx, orc):
    g = np.load(GOLD)
    n = len([k for k in g.files if k.endswith("_sfa")])
    for i in range(n):
        got = _gemm(ctx, g[f"fp4_{i}_a"], g[f"fp4_{i}_sfa"], 1.0, g[f"fp4_{i}_b"], g[f"fp4_{i}_sfb"], 1.0)
        _check(orc, got, g[f"fp4_{i}_c32"])


def test_prefill_shape_rows_against_oracle(ctx, orc):
    """Configuration 3 at full size (2048 x 4096 x 14336); the oracle checks a sample of 48 rows of A."""
    import torch
    import makepad_b200
    M, N, K = 2048, 14336, 4096
    a, sfa = synth.nvfp4_tensor(M, K, seed=0, stream=0)
    b, sfb = synth.nvfp4_tensor(N, K, seed=0, stream=1)
    w = makepad_b200.Nvfp4Weight(ctx, b, sfb, 1.0)
    lin = makepad_b200.QuantLinear(w)
    ad, sd = torch.from_numpy(a).cuda(), torch.from_numpy(sfa).cuda()
    y = lin((ad, sd, 1.0))
    y2 = lin((ad, sd, 1.0))
    torch.cuda.synchronize()
    assert ctx.lib.mpq_context_poll_status(ctx.h) == _lib.OK
    assert torch.equal(y, y2)                                         # deterministic
    rows = np.random.default_rng(0).choice(M, 48, replace=False)
    c32, _ = orc.nvfp4_gemm(a[rows], sfa[rows], 1.0, b, sfb, 1.0)
    got = y[torch.from_numpy(rows).cuda()].view(torch.int16).cpu().numpy().view(np.uint16)
    _check(orc, got, c32)
    # size-independent property at full size: scaling A's tensor scale by 2 doubles every output exactly
    y3 = lin((ad, sd, 2.0))
    torch.cuda.synchronize()
    assert torch.equal(y3.float(), 2.0 * y.float())


def test_error_statuses(ctx):
    import torch
    lib = ctx.lib
    b, sfb = synth.nvfp4_tensor(224, 256, seed=1)
    h = C.c_void_p()
    assert lib.mpq_nvfp4_weight_create(ctx.h, 224, 240, b.ctypes.data, sfb.ctypes.data, C.c_float(1.0), C.byref(h)) == _lib.ERR_SHAPE
    assert lib.mpq_nvfp4_weight_create(ctx.h, 220, 256, b.ctypes.data, sfb.ctypes.data, C.c_float(1.0), C.byref(h)) == _lib.ERR_SHAPE
    assert lib.mpq_nvfp4_weight_create(ctx.h, 224, 256, None, sfb.ctypes.data, C.c_float(1.0), C.byref(h)) == _lib.ERR_INVALID_ARG
    assert lib.mpq_nvfp4_weight_create(ctx.h, 224, 256, b.ctypes.data, sfb.ctypes.data, C.c_float(1.0), C.byref(h)) == _lib.OK
    a = torch.zeros(128 * 128 + 16, dtype=torch.uint8, device="cuda")
    c = torch.zeros(128 * 224, dtype=torch.bfloat16, device="cuda")
    assert lib.mpq_nvfp4_gemm_forward(ctx.h, h, a.data_ptr() + 1, a.data_ptr(), C.c_float(1.0), 128, c.data_ptr(), None) == _lib.ERR_ALIGN
    assert lib.mpq_nvfp4_gemm_forward(ctx.h, h, a.data_ptr(), a.data_ptr(), C.c_float(1.0), 0, c.data_ptr(), None) == _lib.ERR_SHAPE
    assert lib.mpq_nvfp4_gemm_forward(ctx.h, h, None, a.data_ptr(), C.c_float(1.0), 128, c.data_ptr(), None) == _lib.ERR_INVALID_ARG
    # a Q4 entry point refuses an NVFP4 weight
    x = torch.zeros(256, device="cuda")
    assert lib.mpq_q4_linear_forward(ctx.h, h, x.data_ptr(), 1, x.data_ptr(), None) == _lib.ERR_INVALID_ARG
    assert lib.mpq_weight_destroy(h) == _lib.OK


def test_output_guard_regions_untouched(ctx):
    """TMA tile stores clip at the tensor's edge: nothing is written outside C, for M and N off the tile grid."""
    import torch
    import makepad_b200
    M, N, K = 130, 232, 288
    a, sfa = synth.nvfp4_tensor(M, K, seed=21, stream=0)
    b, sfb = synth.nvfp4_tensor(N, K, seed=21, stream=1)
    w = makepad_b200.Nvfp4Weight(ctx, b, sfb, 1.0)
    buf = torch.full((M * N + 4096,), 7.0, dtype=torch.bfloat16, device="cuda")
    c = buf[2048:2048 + M * N].view(M, N)
    for kernel in (None, "single"):
        buf.fill_(7.0)
        if kernel:
            os.environ["MPQ_FP4_KERNEL"] = kernel
        try:
            makepad_b200.QuantLinear(w)((torch.from_numpy(a).cuda(), torch.from_numpy(sfa).cuda(), 1.0), out=c)
            torch.cuda.synchronize()
        finally:
            os.environ.pop("MPQ_FP4_KERNEL", None)
        assert (buf[:2048] == 7.0).all() and (buf[2048 + M * N:] == 7.0).all()
    assert ctx.lib.mpq_context_poll_status(ctx.h) == _lib.OK
    w.destroy()


def test_error_metrics_strict_and_floored(ctx, orc):
    """Strict and floored (1e-2 and 1e-3 of the rms) maxima of the bf16 output against the exact value: all three are
    bounded by the bf16 rounding (2^-8), because the products are exact and the accumulation is fp32."""
    a, sfa = synth.nvfp4_tensor(256, 1024, seed=5, stream=0)
    b, sfb = synth.nvfp4_tensor(448, 1024, seed=5, stream=1)
    c32, _ = orc.nvfp4_gemm(a, sfa, 1.0, b, sfb, 1.0)
    got = orc.bf16_bits_to_f32(_gemm(ctx, a, sfa, 1.0, b, sfb, 1.0)).astype(np.float64)
    rep = orc.err_report(got, c32.astype(np.float64))
    print(f"NVFP4 256x448x1024: {rep}")
    assert rep["floored_1e-2_rms"] < TOL and rep["floored_1e-3_rms"] < TOL


def test_weight_export_reads_the_tiled_scales(ctx, orc):
    """The weight keeps its scale factors only in the tiled order the GEMM consumes; the export un-tiles them, so a
    bit-exact export proves the tiling pass (rows and K off the tile grid included)."""
    import makepad_b200
    for (N, K) in [(448, 512), (232, 288), (1000, 4096), (8, 32)]:
        b, sfb = synth.nvfp4_tensor(N, K, seed=N + K)
        w = makepad_b200.Nvfp4Weight(ctx, b, sfb, 0.5)
        assert np.array_equal(w.dequantize().cpu().numpy().view(np.uint32), orc.nvfp4_dequantize(b, sfb, 0.5).view(np.uint32))
        w.destroy()


@pytest.mark.parametrize("M,K", [(1, 16), (7, 48), (200, 512), (2048, 4096)])
def test_activation_quantisation_bit_exact(ctx, orc, M, K):
    """fp32 and bf16 activations -> NVFP4 on the GPU: the same bytes as the CPU checker, and usable as the GEMM's A."""
    import torch
    rng = np.random.default_rng(M + K)
    x = (rng.standard_normal((M, K)) * rng.uniform(1e-3, 50, size=(M, 1))).astype(np.float32)
    x[0, :16] = 0                                                    # an all-zero block
    if M > 1:
        x[1, :4] = [448 * 6 * 2, -1e-9, 0.25, 0.75]                  # saturation, underflow, ties
    for ts in (1.0, 0.37):
        for bf16 in (0, 1):
            xd = torch.from_numpy(x).cuda()
            if bf16:
                xd = xd.to(torch.bfloat16)
                want_c, want_s = orc.nvfp4_quantize(xd.float().cpu().numpy(), ts)
            else:
                want_c, want_s = orc.nvfp4_quantize(x, ts)
            codes = torch.empty((M, K // 2), dtype=torch.uint8, device="cuda")
            sf = torch.empty((M, K // 16), dtype=torch.uint8, device="cuda")
            ctx.check(ctx.lib.mpq_nvfp4_quantize_activations(ctx.h, C.c_void_p(xd.data_ptr()), bf16, M, K, C.c_float(ts),
                                                             C.c_void_p(codes.data_ptr()), C.c_void_p(sf.data_ptr()), None))
            torch.cuda.synchronize()
            assert np.array_equal(sf.cpu().numpy(), want_s)
            assert np.array_equal(codes.cpu().numpy(), want_c)
    assert ctx.lib.mpq_nvfp4_quantize_activations(ctx.h, C.c_void_p(xd.data_ptr()), 0, M, 24, C.c_float(1.0), C.c_void_p(codes.data_ptr()),
                                                  C.c_void_p(sf.data_ptr()), None) == _lib.ERR_SHAPE


def test_quantise_then_gemm(ctx, orc):
    """The prefill chain: quantise fp32 activations on the GPU, feed them to the GEMM; equal to the checker's chain."""
    import torch
    import makepad_b200
    M, N, K = 256, 448, 1024
    x = synth.activations(M, K, seed=17)
    b, sfb = synth.nvfp4_tensor(N, K, seed=17, stream=1)
    xd = torch.from_numpy(x).cuda()
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device="cuda")
    sf = torch.empty((M, K // 16), dtype=torch.uint8, device="cuda")
    ctx.check(ctx.lib.mpq_nvfp4_quantize_activations(ctx.h, C.c_void_p(xd.data_ptr()), 0, M, K, C.c_float(1.0), C.c_void_p(codes.data_ptr()),
                                                     C.c_void_p(sf.data_ptr()), None))
    w = makepad_b200.Nvfp4Weight(ctx, b, sfb, 1.0)
    y = makepad_b200.QuantLinear(w)((codes, sf, 1.0))
    torch.cuda.synchronize()
    a_c, a_s = orc.nvfp4_quantize(x, 1.0)
    c32, _ = orc.nvfp4_gemm(a_c, a_s, 1.0, b, sfb, 1.0)
    _check(orc, y.view(torch.int16).cpu().numpy().view(np.uint16), c32)
    w.destroy()
