"""Pins the oracle's number conversions against independent implementations
(numpy float16, torch bfloat16 / float8_e4m3fn) over their whole code spaces."""
import numpy as np
import torch

from makepad_b200 import synth


def test_f16_decode_all_codes(orc):
    bits = np.arange(65536, dtype=np.uint16)
    got = orc.f16_to_f32(bits)
    want = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    assert np.isnan(got[nan]).all()


def test_f16_encode_rne(orc):
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e10, -1e10, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 2.0 ** -14,
                  np.inf, -np.inf], dtype=np.float32),
        # every exact tie between adjacent fp16 values in a band
        (np.arange(1024, 2048, dtype=np.float32) + 0.5) * np.float32(2.0 ** -10),
    ])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(orc.f32_to_f16(x), want)


def test_bf16_encode_matches_torch(orc):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(300000) * 10.0 ** rng.integers(-20, 20, 300000)).astype(np.float32)
    x = np.concatenate([x, np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, np.inf, -np.inf, 3.3895e38], dtype=np.float32)])
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.f32_to_bf16(x), want)


def test_e4m3_decode_all_codes(orc):
    b = np.arange(256, dtype=np.uint8)
    got = orc.e4m3_to_f32(b)
    want = torch.from_numpy(b).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    nan = np.isnan(want)
    assert list(np.nonzero(nan)[0]) == [0x7F, 0xFF]
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    assert np.isnan(got[nan]).all()
    assert got[0x7E] == 448.0 and got[0x01] == 2.0 ** -9 and got[0x08] == 2.0 ** -6


def test_e4m3_encode_matches_torch_in_range(orc):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(300000) * 10.0 ** rng.integers(-4, 3, 300000)).astype(np.float32)
    x = x[np.abs(x) <= 448.0]
    vals = orc.e4m3_to_f32(np.arange(0x7F, dtype=np.uint8))
    ties = ((vals[:-1].astype(np.float64) + vals[1:].astype(np.float64)) / 2).astype(np.float32)   # exact midpoints
    x = np.concatenate([x, ties, -ties, vals, np.array([0.0, 1e-9, 447.9, 448.0], dtype=np.float32)])
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = orc.f32_to_e4m3(x)
    # +-0 may differ in sign handling of tiny negatives: compare decoded values and the bytes where non-zero
    assert np.array_equal(orc.e4m3_to_f32(got), orc.e4m3_to_f32(want))
    assert np.array_equal(got & 0x7F, want & 0x7F)


def test_e4m3_encode_saturates(orc):
    x = np.array([449.0, 464.0, 1e6, np.inf, -1e6], dtype=np.float32)
    assert list(orc.f32_to_e4m3(x)) == [0x7E, 0x7E, 0x7E, 0x7E, 0xFE]
    assert orc.f32_to_e4m3(np.array([np.nan], dtype=np.float32))[0] & 0x7F == 0x7F


def test_synth_e4m3_encoder_agrees_with_oracle(orc):
    rng = np.random.default_rng(3)
    x = np.abs(rng.standard_normal(100000)).astype(np.float32) * np.float32(0.1)
    assert np.array_equal(synth.e4m3_encode_nonneg(x), orc.f32_to_e4m3(x))


def test_e2m1_table_and_round_trip(orc):
    assert list(orc.E2M1_VALUES[:8]) == [0, .5, 1, 1.5, 2, 3, 4, 6]
    assert np.array_equal(orc.E2M1_VALUES[8:], -orc.E2M1_VALUES[:8])
    # decode through the dequantiser: one row of the 16 codes, scale byte 0x38 = 1.0
    codes = synth.pack_nibbles(np.arange(16, dtype=np.uint8)[None, :])
    out = orc.nvfp4_dequantize(codes, np.array([[0x38]], dtype=np.uint8), 1.0)
    assert np.array_equal(out[0].view(np.uint32), orc.E2M1_VALUES.view(np.uint32))
    # encode: every representable value maps to itself; ties go to the even mantissa
    enc = orc.f32_to_e2m1(orc.E2M1_VALUES)
    assert list(enc) == list(range(16))
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 100.0], dtype=np.float32)
    assert list(orc.f32_to_e2m1(ties)) == [0, 2, 2, 4, 4, 6, 6, 7, 7]
