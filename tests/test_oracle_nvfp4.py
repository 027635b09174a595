"""Known-answer tests and golden vectors for the NVFP4 half of the oracle."""
import os

import numpy as np
import torch

from makepad_b200 import synth

GOLD = os.path.join(os.path.dirname(__file__), "golden", "nvfp4_small.npz")


def test_kat_unit_scales(orc):
    # codes all 1.0 (nibble 2), scales 1.0 (0x38): C = K
    M, N, K = 2, 3, 32
    a = synth.pack_nibbles(np.full((M, K), 2, dtype=np.uint8))
    b = synth.pack_nibbles(np.full((N, K), 2, dtype=np.uint8))
    sfa = np.full((M, K // 16), 0x38, dtype=np.uint8)
    sfb = np.full((N, K // 16), 0x38, dtype=np.uint8)
    c32, c16 = orc.nvfp4_gemm(a, sfa, 1.0, b, sfb, 1.0)
    assert np.array_equal(c32, np.full((M, N), 32.0, dtype=np.float32))
    assert np.array_equal(orc.bf16_bits_to_f32(c16), c32)
    c32, _ = orc.nvfp4_gemm(a, sfa, 0.5, b, sfb, 3.0)
    assert np.array_equal(c32, np.full((M, N), 48.0, dtype=np.float32))


def test_kat_block_scales_and_signs(orc):
    # A row: block 0 all +6 (0x7) scale 2.0 (0x40); block 1 all -0.5 (0x9) scale 0.25 (0x28)
    # B row: all 1.5 (0x3), scales 1.0 / 4.0 (0x48)
    K = 32
    a = synth.pack_nibbles(np.array([[7] * 16 + [9] * 16], dtype=np.uint8))
    b = synth.pack_nibbles(np.full((1, K), 3, dtype=np.uint8))
    sfa = np.array([[0x40, 0x28]], dtype=np.uint8)
    sfb = np.array([[0x38, 0x48]], dtype=np.uint8)
    c32, _ = orc.nvfp4_gemm(a, sfa, 1.0, b, sfb, 1.0)
    assert c32[0, 0] == 16 * 6 * 1.5 * 2.0 * 1.0 + 16 * (-0.5) * 1.5 * 0.25 * 4.0


def test_zero_scale_zeroes_block(orc):
    a = synth.pack_nibbles(np.full((1, 16), 7, dtype=np.uint8))
    c32, _ = orc.nvfp4_gemm(a, np.array([[0]], dtype=np.uint8), 1.0, a, np.array([[0x38]], dtype=np.uint8), 1.0)
    assert c32[0, 0] == 0.0


def test_gemm_against_numpy_and_torch_bf16(orc):
    M, N, K = 24, 40, 192
    a, sfa = synth.nvfp4_tensor(M, K, seed=7, stream=0)
    b, sfb = synth.nvfp4_tensor(N, K, seed=7, stream=1)
    A = orc.nvfp4_dequantize(a, sfa, 1.0).astype(np.float64)
    B = orc.nvfp4_dequantize(b, sfb, 1.0).astype(np.float64)
    want = A @ B.T
    c32, c16 = orc.nvfp4_gemm(a, sfa, 1.0, b, sfb, 1.0)
    assert np.abs(c32 - want).max() <= 1e-6 * np.abs(want).max()
    bf = torch.from_numpy(c32).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(c16, bf)


def test_golden_vectors(orc):
    g = np.load(GOLD)
    n = len([k for k in g.files if k.endswith("_sfa")])
    assert n >= 2
    for i in range(n):
        a, sfa, b, sfb = g[f"fp4_{i}_a"], g[f"fp4_{i}_sfa"], g[f"fp4_{i}_b"], g[f"fp4_{i}_sfb"]
        c32, c16 = orc.nvfp4_gemm(a, sfa, 1.0, b, sfb, 1.0, threads=1)
        assert np.array_equal(c32.view(np.uint32), g[f"fp4_{i}_c32"].view(np.uint32))
        assert np.array_equal(c16, g[f"fp4_{i}_c16"])
        assert np.array_equal(orc.nvfp4_dequantize(b, sfb, 1.0).view(np.uint32), g[f"fp4_{i}_deq_b"].view(np.uint32))


def test_activation_quantisation_known_answers_and_bounds():
    """orc_nvfp4_quantize: hand-checked blocks, and the error bound of the format on random data."""
    from oracle import oracle as orc
    orc.build()
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, :16] = [6, -6, 3, 1.5, 0.5, 0.25, 0.26, -0.74, 0.75, 1.25, 1.26, 2.5, 2.6, 5.0, 5.1, 0]
    codes, sf = orc.nvfp4_quantize(x, 1.0)
    assert sf[0, 0] == 0x38 and sf[0, 1] == 0                      # amax 6 -> scale 1.0 (e4m3 0x38); the all-zero block -> 0
    nib = np.stack([codes[0, :8] & 0xF, codes[0, :8] >> 4], axis=1).reshape(-1)
    # ties go to the even mantissa: 0.25 -> 0, 0.75 -> 1.0, 1.25 -> 1.0, 2.5 -> 2, 5.0 -> 4
    assert list(nib) == [7, 15, 5, 3, 1, 0, 1, 9, 2, 2, 3, 4, 5, 6, 7, 0]
    assert not codes[0, 8:].any()
    # scale rounding and saturation
    x2 = np.full((1, 16), 448.0 * 6 * 4, dtype=np.float32)
    c2, s2 = orc.nvfp4_quantize(x2, 1.0)
    assert s2[0, 0] == 0x7E and (c2 == 0x77).all()                 # scale saturates at 448, codes at 6
    rng = np.random.default_rng(3)
    x3 = (rng.standard_normal((8, 256)) * rng.uniform(0.01, 100, size=(8, 1))).astype(np.float32)
    for ts in (1.0, 0.37):
        c3, s3 = orc.nvfp4_quantize(x3, ts)
        back = orc.nvfp4_dequantize(c3, s3, ts)
        amax = np.abs(x3.reshape(8, 16, 16)).max(axis=2, keepdims=True)
        err = np.abs(back - x3).reshape(8, 16, 16)
        # e2m1 steps are at most 2 (between 4 and 6) in units of amax/6 (scale rounding adds < 1/16): error <= ~amax/6 * 1.07
        assert (err <= amax / 6 * 1.07 + 1e-12).all()
