"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE -- parity unpinned).

The makepad/makepad snapshot holds no implementation of the block-quantised
linear path, so ``mpq_oracle.c`` restates the formats as the task configuration
words them; see the header of that file.  Only tests, the smoke check and the
benchmark's CPU-baseline leg may import this module.  The shipped library never
does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liborc.so")
_lib = None


def _host_signature() -> str:
    """What the binary was built for: it is compiled with -march=native, so a copy built on another machine
    (it travels with the tree) must not be reused on this one."""
    import hashlib
    import platform
    try:
        with open("/proc/cpuinfo") as f:
            lines = [ln for ln in f if ln.startswith(("model name", "flags"))][:2]
    except OSError:
        lines = []
    return hashlib.sha1((platform.machine() + "".join(lines)).encode()).hexdigest()


def build(force: bool = False) -> str:
    """Compile ``mpq_oracle.c`` into ``liborc.so`` beside it (gcc, a second or two), on the machine that runs it."""
    src, mark = os.path.join(_HERE, "mpq_oracle.c"), os.path.join(_HERE, "liborc.host")
    sig = _host_signature()
    try:
        built_for = open(mark).read().strip()
    except OSError:
        built_for = ""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src) or built_for != sig:
        subprocess.check_call(["make", "-C", _HERE, "-B", "liborc.so"], stdout=subprocess.DEVNULL)
        with open(mark, "w") as f:
            f.write(sig + "\n")
    return _LIB_PATH


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
    return _lib


def _conv(name, src, sdt, ddt, sct, dct):
    src = np.ascontiguousarray(src, dtype=sdt)
    out = np.empty(src.shape, dtype=ddt)
    getattr(lib(), name)(_p(src, sct), _p(out, dct), C.c_int64(src.size))
    return out


def f16_to_f32(bits):
    return _conv("orc_f16_to_f32_n", bits, np.uint16, np.float32, C.c_uint16, C.c_float)


def f32_to_f16(x):
    return _conv("orc_f32_to_f16_n", x, np.float32, np.uint16, C.c_float, C.c_uint16)


def f32_to_bf16(x):
    return _conv("orc_f32_to_bf16_n", x, np.float32, np.uint16, C.c_float, C.c_uint16)


def e4m3_to_f32(b):
    return _conv("orc_e4m3_to_f32_n", b, np.uint8, np.float32, C.c_uint8, C.c_float)


def f32_to_e4m3(x):
    return _conv("orc_f32_to_e4m3_n", x, np.float32, np.uint8, C.c_float, C.c_uint8)


def f32_to_e2m1(x):
    return _conv("orc_f32_to_e2m1_n", x, np.float32, np.uint8, C.c_float, C.c_uint8)


E2M1_VALUES = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def bf16_bits_to_f32(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _check_q4(codes, scales, N, K):
    assert K % 32 == 0 and codes.shape == (N, K // 2) and scales.shape == (N, K // 32)
    assert codes.dtype == np.uint8 and scales.dtype == np.uint16


def q4_dequantize(codes, scales):
    N, K = codes.shape[0], codes.shape[1] * 2
    codes = np.ascontiguousarray(codes); scales = np.ascontiguousarray(scales)
    _check_q4(codes, scales, N, K)
    out = np.empty((N, K), dtype=np.float32)
    lib().orc_q4_dequantize(C.c_int64(N), C.c_int64(K), _p(codes, C.c_uint8), _p(scales, C.c_uint16), _p(out, C.c_float))
    return out


def q4_matmul_f64(codes, scales, X, threads=0):
    """Y[M,N] in binary64: the arbiter of the tolerance tests."""
    N, K = codes.shape[0], codes.shape[1] * 2
    codes = np.ascontiguousarray(codes); scales = np.ascontiguousarray(scales)
    _check_q4(codes, scales, N, K)
    X = np.ascontiguousarray(X, dtype=np.float32).reshape(-1, K)
    Y = np.empty((X.shape[0], N), dtype=np.float64)
    lib().orc_q4_matmul_f64(C.c_int64(X.shape[0]), C.c_int64(N), C.c_int64(K), _p(codes, C.c_uint8),
                            _p(scales, C.c_uint16), _p(X, C.c_float), _p(Y, C.c_double),
                            C.c_int(threads or os.cpu_count() or 1))
    return Y


def q4_matmul_f32(codes, scales, X, threads=0):
    """The fp32 CPU path (dequantise, fp32 multiply-accumulate): the timed baseline."""
    N, K = codes.shape[0], codes.shape[1] * 2
    codes = np.ascontiguousarray(codes); scales = np.ascontiguousarray(scales)
    _check_q4(codes, scales, N, K)
    X = np.ascontiguousarray(X, dtype=np.float32).reshape(-1, K)
    Y = np.empty((X.shape[0], N), dtype=np.float32)
    lib().orc_q4_matmul_f32(C.c_int64(X.shape[0]), C.c_int64(N), C.c_int64(K), _p(codes, C.c_uint8),
                            _p(scales, C.c_uint16), _p(X, C.c_float), _p(Y, C.c_float),
                            C.c_int(threads or os.cpu_count() or 1))
    return Y


def nvfp4_dequantize(codes, sf, tscale=1.0):
    R, K = codes.shape[0], codes.shape[1] * 2
    codes = np.ascontiguousarray(codes, dtype=np.uint8); sf = np.ascontiguousarray(sf, dtype=np.uint8)
    assert K % 16 == 0 and sf.shape == (R, K // 16)
    out = np.empty((R, K), dtype=np.float32)
    lib().orc_nvfp4_dequantize(C.c_int64(R), C.c_int64(K), _p(codes, C.c_uint8), _p(sf, C.c_uint8),
                               C.c_float(tscale), _p(out, C.c_float))
    return out


def nvfp4_quantize(x, tscale=1.0):
    """fp32 [R][K] -> (codes u8 [R][K/2], sf u8 [R][K/16]); see orc_nvfp4_quantize."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, K = x.shape
    assert K % 16 == 0
    codes = np.empty((R, K // 2), dtype=np.uint8)
    sf = np.empty((R, K // 16), dtype=np.uint8)
    lib().orc_nvfp4_quantize(C.c_int64(R), C.c_int64(K), _p(x, C.c_float), C.c_float(tscale), _p(codes, C.c_uint8), _p(sf, C.c_uint8))
    return codes, sf


def swiglu_f64(gate_up):
    """[M][2F] = [gate | up] -> silu(gate) * up in binary64, silu(g) = g / (1 + exp(-g)): the reference the GPU's fp32
    SwiGLU is held against (a transcendental: checked to a tolerance, not to the bit)."""
    gu = np.asarray(gate_up, dtype=np.float64)
    F = gu.shape[1] // 2
    g, u = gu[:, :F], gu[:, F:]
    with np.errstate(over="ignore"):
        return g / (1.0 + np.exp(-g)) * u


def nvfp4_gemm(a, sfa, ta, b, sfb, tb, threads=0):
    """Returns (C fp32 [M,N], C bf16 bits [M,N]); B is stored [N][K/2]."""
    M, K = a.shape[0], a.shape[1] * 2
    N = b.shape[0]
    a = np.ascontiguousarray(a, dtype=np.uint8); b = np.ascontiguousarray(b, dtype=np.uint8)
    sfa = np.ascontiguousarray(sfa, dtype=np.uint8); sfb = np.ascontiguousarray(sfb, dtype=np.uint8)
    assert b.shape == (N, K // 2) and sfa.shape == (M, K // 16) and sfb.shape == (N, K // 16)
    c32 = np.empty((M, N), dtype=np.float32)
    c16 = np.empty((M, N), dtype=np.uint16)
    lib().orc_nvfp4_gemm(C.c_int64(M), C.c_int64(N), C.c_int64(K), _p(a, C.c_uint8), _p(sfa, C.c_uint8), C.c_float(ta),
                         _p(b, C.c_uint8), _p(sfb, C.c_uint8), C.c_float(tb), _p(c32, C.c_float), _p(c16, C.c_uint16),
                         C.c_int(threads or os.cpu_count() or 1))
    return c32, c16


def rel_err(got, ref64, floor=1e-2):
    """(strict, floored) max relative error against a binary64 reference.

    strict  = max |got-ref| / |ref|                       (ill-conditioned where ref is near 0)
    floored = max |got-ref| / max(|ref|, floor*rms(ref))  (the pass/fail criterion)

    The outputs are zero-mean sums, so some land arbitrarily close to 0 and the
    strict ratio is unbounded for ANY finite-precision implementation: the plain
    fp32 CPU path itself reaches 1e-3 strict on a 512x4096 matrix with 33 rows.
    The floor of 1% of the output rms keeps the per-element test meaningful.
    """
    got = np.asarray(got, dtype=np.float64); ref = np.asarray(ref64, dtype=np.float64)
    d = np.abs(got - ref)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    with np.errstate(divide="ignore", invalid="ignore"):
        strict = np.where(ref != 0, d / np.abs(ref), np.where(d == 0, 0.0, np.inf))
    fl = np.maximum(np.abs(ref), floor * rms)
    floored = np.where(fl > 0, d / np.where(fl > 0, fl, 1), np.where(d == 0, 0.0, np.inf))
    return (float(strict.max()) if d.size else 0.0, float(floored.max()) if d.size else 0.0)


def err_report(got, ref64):
    """Every error figure the parity tests quote, in one dict: the strict maximum, the floored maxima with the
    floor at 1e-2 and at 1e-3 of the output rms, and the largest absolute error as a fraction of the rms."""
    ref = np.asarray(ref64, dtype=np.float64)
    strict, fl2 = rel_err(got, ref, floor=1e-2)
    _, fl3 = rel_err(got, ref, floor=1e-3)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    d = float(np.abs(np.asarray(got, dtype=np.float64) - ref).max()) if ref.size else 0.0
    return {"strict": strict, "floored_1e-2_rms": fl2, "floored_1e-3_rms": fl3, "max_abs_over_rms": d / rms if rms > 0 else 0.0}
