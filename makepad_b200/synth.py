"""Seeded synthetic inputs in the canonical (interchange) formats.

The task configuration fixes the distributions (Q4 codes uniform in [-8,7],
fp16 scales |N(0,1)|*0.02, activations N(0,1); NVFP4 codes uniform over the 16
e2m1 patterns, e4m3 scales from |N(0,1)|*0.1) and "seed 0", but names no
generator; the reference snapshot has none for this path.  This module defines
one: a counter-based splitmix64 stream per (seed, stream id), so any tensor can
be regenerated independently of the order of calls.

Canonical layouts
  Q4     codes  u8[N][K/2]   element 2j = low nibble of byte j, 2j+1 = high nibble,
                             nibble = two's-complement 4-bit integer
         scales u16[N][K/32] IEEE binary16 bits, block b covers k in [32b, 32b+32)
  NVFP4  codes  u8[R][K/2]   same nibble order, nibble = e2m1 (S.EE.M)
         sf     u8[R][K/16]  e4m3 (finite-only) bits, non-negative
"""
from __future__ import annotations

import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)


def _splitmix64(ctr: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = ctr + _GOLD
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _stream(seed: int, stream: int, n: int) -> np.ndarray:
    """n 64-bit words of the stream (seed, stream)."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([np.uint64(seed) * np.uint64(0xD1342543DE82EF95) + np.uint64(stream)], dtype=np.uint64))[0]
        return _splitmix64(base + np.arange(n, dtype=np.uint64) * np.uint64(2) + np.uint64(1))


def uniform_nibbles(seed: int, stream: int, n: int) -> np.ndarray:
    """n values uniform in 0..15 (one 64-bit word yields 16 of them)."""
    words = _stream(seed, stream, (n + 15) // 16)
    sh = (np.arange(16, dtype=np.uint64) * np.uint64(4))[None, :]
    return ((words[:, None] >> sh) & np.uint64(0xF)).astype(np.uint8).reshape(-1)[:n]


def normal(seed: int, stream: int, n: int) -> np.ndarray:
    """n draws of N(0,1) in float64 (Box-Muller on two 53-bit uniforms per value)."""
    w = _stream(seed, stream, 2 * n)
    u1 = ((w[0::2] >> np.uint64(11)).astype(np.float64) + 1.0) * (1.0 / 9007199254740992.0)
    u2 = (w[1::2] >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def pack_nibbles(nib: np.ndarray) -> np.ndarray:
    """[R][K] nibbles (0..15) -> [R][K/2] bytes, element 2j in the low nibble."""
    nib = np.asarray(nib, dtype=np.uint8)
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).astype(np.uint8)


def q4_weight(N: int, K: int, seed: int = 0, stream: int = 0):
    """(codes u8[N][K/2], scales u16[N][K/32]): codes uniform in [-8,7], scale = fp16(|z|*0.02)."""
    assert K % 32 == 0
    nib = uniform_nibbles(seed, 3 * stream, N * K).reshape(N, K)      # nibble = code & 0xF, uniform
    z = normal(seed, 3 * stream + 1, N * (K // 32)).reshape(N, K // 32)
    scales = (np.abs(z) * 0.02).astype(np.float32).astype(np.float16).view(np.uint16)
    return pack_nibbles(nib), np.ascontiguousarray(scales)


def q4_codes_from_ints(c: np.ndarray) -> np.ndarray:
    """[N][K] integers in [-8,7] -> packed canonical codes."""
    c = np.asarray(c)
    assert c.min() >= -8 and c.max() <= 7
    return pack_nibbles((c & 0xF).astype(np.uint8))


def activations(M: int, K: int, seed: int = 0, stream: int = 0) -> np.ndarray:
    """fp32 [M][K] ~ N(0,1)."""
    return normal(seed, 3 * stream + 2, M * K).astype(np.float32).reshape(M, K)


_E4M3_LUT = None


def _e4m3_positive_values() -> np.ndarray:
    """fp32 values of the e4m3 bytes 0x00..0x7E (finite, non-negative, ascending)."""
    global _E4M3_LUT
    if _E4M3_LUT is None:
        b = np.arange(0x7F, dtype=np.int64)
        e, m = b >> 3, b & 7
        _E4M3_LUT = np.where(e == 0, m * 2.0 ** -9, (8 + m) * 2.0 ** (e - 10)).astype(np.float64)
    return _E4M3_LUT


def e4m3_encode_nonneg(x: np.ndarray) -> np.ndarray:
    """Round non-negative floats to e4m3 bytes: nearest, ties to even, saturating at 448."""
    lut = _e4m3_positive_values()
    x = np.minimum(np.asarray(x, dtype=np.float64), 448.0)
    hi = np.clip(np.searchsorted(lut, x, side="left"), 1, len(lut) - 1)
    lo = hi - 1
    dlo, dhi = x - lut[lo], lut[hi] - x
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    return np.where(pick_hi, hi, lo).astype(np.uint8)


def nvfp4_tensor(R: int, K: int, seed: int = 0, stream: int = 0):
    """(codes u8[R][K/2], sf u8[R][K/16]): codes uniform over the 16 e2m1 patterns, sf = e4m3(|z|*0.1)."""
    assert K % 16 == 0
    nib = uniform_nibbles(seed, 3 * stream, R * K).reshape(R, K)
    z = normal(seed, 3 * stream + 1, R * (K // 16)).reshape(R, K // 16)
    sf = e4m3_encode_nonneg(np.abs(z).astype(np.float32).astype(np.float64) * np.float64(np.float32(0.1)))
    return pack_nibbles(nib), np.ascontiguousarray(sf)
