"""Known-answer tests and golden vectors for the Q4 half of the oracle."""
import os

import numpy as np

from makepad_b200 import synth

GOLD = os.path.join(os.path.dirname(__file__), "golden", "q4_small.npz")


def _f16(x):
    return np.asarray(x, dtype=np.float16).view(np.uint16)


def test_kat_all_ones(orc):
    # every code 1, every scale 1.0: y = sum(x)
    N, K = 4, 64
    codes = synth.q4_codes_from_ints(np.ones((N, K), dtype=np.int64))
    scales = np.full((N, K // 32), _f16(1.0), dtype=np.uint16)
    x = np.arange(K, dtype=np.float32)[None, :]
    assert np.array_equal(orc.q4_dequantize(codes, scales), np.ones((N, K), dtype=np.float32))
    assert np.array_equal(orc.q4_matmul_f64(codes, scales, x), np.full((1, N), K * (K - 1) / 2))
    assert np.array_equal(orc.q4_matmul_f32(codes, scales, x), np.full((1, N), K * (K - 1) / 2, dtype=np.float32))


def test_kat_nibble_order_and_sign(orc):
    # one row: element 0 = -8 (low nibble of byte 0), element 1 = 7 (high nibble), element 33 = 3 in block 1
    c = np.zeros((1, 64), dtype=np.int64)
    c[0, 0], c[0, 1], c[0, 33] = -8, 7, 3
    codes = synth.q4_codes_from_ints(c)
    assert codes[0, 0] == 0x78 and codes[0, 16] == 0x30
    scales = np.array([[_f16(0.5), _f16(2.0)]], dtype=np.uint16)
    w = orc.q4_dequantize(codes, scales)
    assert w[0, 0] == -4.0 and w[0, 1] == 3.5 and w[0, 33] == 6.0 and np.count_nonzero(w) == 3
    x = np.zeros((2, 64), dtype=np.float32)
    x[0, 0], x[0, 1], x[1, 33] = 1.0, 2.0, -1.5
    assert np.array_equal(orc.q4_matmul_f64(codes, scales, x), np.array([[3.0], [-9.0]]))


def test_dequant_product_is_exact_in_fp32(orc):
    # fp16 scale (11-bit significand) times a 4-bit integer never rounds in binary32
    codes, scales = synth.q4_weight(64, 256, seed=5)
    w = orc.q4_dequantize(codes, scales).astype(np.float64)
    lo, hi = (codes & 0xF).astype(np.int64), (codes >> 4).astype(np.int64)
    c = np.empty((64, 256), dtype=np.int64)
    c[:, 0::2], c[:, 1::2] = (lo ^ 8) - 8, (hi ^ 8) - 8
    s = np.repeat(scales.view(np.float16).astype(np.float64), 32, axis=1)
    assert np.array_equal(w, s * c)


def test_matmul_against_numpy(orc):
    codes, scales = synth.q4_weight(96, 320, seed=6)
    x = synth.activations(7, 320, seed=6)
    w = orc.q4_dequantize(codes, scales).astype(np.float64)
    want = x.astype(np.float64) @ w.T
    got = orc.q4_matmul_f64(codes, scales, x)
    assert np.abs(got - want).max() <= 1e-12 * np.abs(want).max()
    strict, floored = orc.rel_err(orc.q4_matmul_f32(codes, scales, x), want)
    assert floored < 1e-4
    assert np.array_equal(orc.q4_matmul_f32(codes, scales, x, threads=1), orc.q4_matmul_f32(codes, scales, x, threads=5))


def test_golden_vectors(orc):
    g = np.load(GOLD)
    n = len([k for k in g.files if k.endswith("_codes")])
    assert n >= 4
    for i in range(n):
        codes, scales, x = g[f"q4_{i}_codes"], g[f"q4_{i}_scales"], g[f"q4_{i}_x"]
        assert np.array_equal(orc.q4_dequantize(codes, scales).view(np.uint32), g[f"q4_{i}_deq"].view(np.uint32))
        assert np.array_equal(orc.q4_matmul_f64(codes, scales, x, threads=1), g[f"q4_{i}_y64"])


def test_config0_shapes_and_bytes(orc):
    # the CPU-runnable configuration: 4096 x 4096, M = 1, seed 0 (a 256-row slice keeps the test quick)
    codes, scales = synth.q4_weight(4096, 4096, seed=0)
    assert codes.nbytes + scales.nbytes == 9_437_184
    x = synth.activations(1, 4096, seed=0)
    y64 = orc.q4_matmul_f64(codes[:256], scales[:256], x)
    y32 = orc.q4_matmul_f32(codes[:256], scales[:256], x)
    assert orc.rel_err(y32, y64)[1] < 1e-4
