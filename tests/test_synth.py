import numpy as np

from makepad_b200 import synth


def test_streams_are_deterministic_and_independent():
    a = synth.q4_weight(64, 128, seed=0, stream=0)
    b = synth.q4_weight(64, 128, seed=0, stream=0)
    c = synth.q4_weight(64, 128, seed=0, stream=1)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    assert not np.array_equal(a[0], c[0])
    assert not np.array_equal(synth.activations(1, 128, 0, 0), synth.activations(1, 128, 1, 0))


def test_q4_distribution():
    codes, scales = synth.q4_weight(256, 4096, seed=0)
    lo, hi = (codes & 0xF).astype(np.int32), (codes >> 4).astype(np.int32)
    c = np.concatenate([((lo ^ 8) - 8).ravel(), ((hi ^ 8) - 8).ravel()])
    assert c.min() == -8 and c.max() == 7
    counts = np.bincount(c + 8, minlength=16) / c.size
    assert np.abs(counts - 1 / 16).max() < 2e-3
    s = scales.view(np.float16).astype(np.float64)
    assert (s >= 0).all()
    assert abs(s.mean() - 0.02 * np.sqrt(2 / np.pi)) < 2e-4          # E|z| = sqrt(2/pi)


def test_activation_moments():
    x = synth.activations(4, 65536, seed=0).astype(np.float64)
    assert abs(x.mean()) < 0.01 and abs(x.std() - 1.0) < 0.01


def test_nvfp4_distribution():
    codes, sf = synth.nvfp4_tensor(128, 4096, seed=0)
    nib = np.concatenate([(codes & 0xF).ravel(), (codes >> 4).ravel()])
    counts = np.bincount(nib, minlength=16) / nib.size
    assert np.abs(counts - 1 / 16).max() < 3e-3                      # all 16 patterns, +-0 included
    assert sf.max() < 0x7F and (sf == 0).any()                       # finite; some scales round to zero
