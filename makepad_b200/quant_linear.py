"""Host-side mirror of the operator interface, on top of the C ABI.

The reference snapshot has no operator/tensor API for this path, so the names
follow the task configuration (Q4 weight, NVFP4 weight, quantised linear) and
the error behaviour follows the reference's FFI idiom: a loader that returns an
error instead of panicking (platform/src/os/linux/module_loader.rs:9-33) and
Result-style failures, here ``MpqError`` carrying the library's status code.

torch is used only as the owner of device buffers and streams; every operator
runs inside libmpq.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib


class MpqError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"mpq status {status}: {text}")
        self.status = status


def _np_ptr(a: np.ndarray):
    return C.c_void_p(a.ctypes.data)


class Context:
    """One per (process, GPU)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        st = self.lib.mpq_context_create(device, C.byref(h))
        if st != _lib.OK:
            raise MpqError(st, self.lib.mpq_status_string(st).decode())
        self.h = h
        self.device = device

    def check(self, st: int):
        if st != _lib.OK:
            raise MpqError(st, f"{self.lib.mpq_status_string(st).decode()}: {self.lib.mpq_last_error(self.h).decode()}")

    def info(self) -> _lib.DeviceInfo:
        d = _lib.DeviceInfo()
        self.check(self.lib.mpq_context_info(self.h, C.byref(d)))
        return d

    @property
    def launches(self) -> int:
        return int(self.lib.mpq_context_launch_count(self.h))

    def close(self):
        if self.h:
            self.lib.mpq_context_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _Weight:
    def __init__(self, ctx: Context, h):
        self.ctx, self.h = ctx, h
        n, k, f = C.c_int64(), C.c_int64(), C.c_int32()
        ctx.check(ctx.lib.mpq_weight_shape(h, C.byref(n), C.byref(k), C.byref(f)))
        self.N, self.K, self.fmt = n.value, k.value, f.value

    @property
    def device_bytes(self) -> int:
        return int(self.ctx.lib.mpq_weight_device_bytes(self.h))

    def dequantize(self):
        """Exact fp32 [N][K] export read back from the device layout (torch tensor on the GPU)."""
        import torch
        out = torch.empty((self.N, self.K), dtype=torch.float32, device=f"cuda:{self.ctx.device}")
        self.ctx.check(self.ctx.lib.mpq_weight_dequantize(self.ctx.h, self.h, C.c_void_p(out.data_ptr()),
                                                          C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out

    def save(self, path: str):
        """Write the weight as it lies in device memory (a cache file: see load_weight)."""
        self.ctx.check(self.ctx.lib.mpq_weight_save(self.ctx.h, self.h, str(path).encode()))

    def destroy(self):
        if self.h:
            self.ctx.lib.mpq_weight_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def load_weight(ctx: Context, path: str) -> "_Weight":
    """Load a device-layout file written by ``_Weight.save``: no repack pass.  Raises MpqError with status
    ERR_FORMAT when the file was written for another layout (or is damaged): rebuild from the canonical arrays."""
    h = C.c_void_p()
    ctx.check(ctx.lib.mpq_weight_load(ctx.h, str(path).encode(), C.byref(h)))
    w = _Weight(ctx, h)
    if w.fmt == _lib.FMT_NVFP4:
        info = _lib.FileInfo()
        ctx.check(ctx.lib.mpq_file_info(str(path).encode(), C.byref(info)))
        w.tensor_scale = float(info.tensor_scale)
    return w


def save_canonical(path: str, fmt: int, codes: np.ndarray, scales: np.ndarray, tensor_scale: float = 1.0):
    """Write the interchange arrays of a weight (no GPU needed)."""
    lib = _lib.load()
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint16 if fmt == _lib.FMT_Q4 else np.uint8)
    st = lib.mpq_canonical_save(str(path).encode(), fmt, codes.shape[0], codes.shape[1] * 2, _np_ptr(codes), _np_ptr(scales), C.c_float(tensor_scale))
    if st != _lib.OK:
        raise MpqError(st, lib.mpq_status_string(st).decode())


def load_canonical(path: str):
    """-> (fmt, codes, scales, tensor_scale) of a canonical file (no GPU needed)."""
    lib = _lib.load()
    info = _lib.FileInfo()
    st = lib.mpq_file_info(str(path).encode(), C.byref(info))
    if st == _lib.OK and info.kind != _lib.FILE_CANONICAL:
        st = _lib.ERR_FORMAT
    if st != _lib.OK:
        raise MpqError(st, lib.mpq_status_string(st).decode())
    codes = np.empty((info.N, info.K // 2), dtype=np.uint8)
    scales = np.empty((info.N, info.K // 32), dtype=np.uint16) if info.fmt == _lib.FMT_Q4 else np.empty((info.N, info.K // 16), dtype=np.uint8)
    ts = C.c_float()
    st = lib.mpq_canonical_load(str(path).encode(), _np_ptr(codes), codes.nbytes, _np_ptr(scales), scales.nbytes, C.byref(ts))
    if st != _lib.OK:
        raise MpqError(st, lib.mpq_status_string(st).decode())
    return info.fmt, codes, scales, float(ts.value)


class Q4Weight(_Weight):
    """Q4 weight: codes u8[N][K/2] + fp16-bit scales u16[N][K/32] (canonical), repacked on the GPU."""

    def __init__(self, ctx: Context, codes: np.ndarray, scales: np.ndarray, tp_mode: int = _lib.TP_NONE, rank: int = 0,
                 world: int = 1):
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.uint16)
        if codes.ndim != 2 or scales.ndim != 2:
            raise MpqError(_lib.ERR_SHAPE, "codes and scales must be 2-D")
        N, K = codes.shape[0], codes.shape[1] * 2
        if scales.shape != (N, K // 32) or K % 32:
            raise MpqError(_lib.ERR_SHAPE, f"scales shape {scales.shape} does not match codes {codes.shape}")
        h = C.c_void_p()
        ctx.check(ctx.lib.mpq_q4_weight_create(ctx.h, N, K, _np_ptr(codes), _np_ptr(scales), tp_mode, rank, world, C.byref(h)))
        super().__init__(ctx, h)


class Nvfp4Weight(_Weight):
    """NVFP4 weight B: codes u8[N][K/2], e4m3 scale bytes u8[N][K/16], fp32 tensor scale."""

    def __init__(self, ctx: Context, codes: np.ndarray, sf: np.ndarray, tensor_scale: float = 1.0):
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        sf = np.ascontiguousarray(sf, dtype=np.uint8)
        N, K = codes.shape[0], codes.shape[1] * 2
        if sf.shape != (N, K // 16):
            raise MpqError(_lib.ERR_SHAPE, f"sf shape {sf.shape} does not match codes {codes.shape}")
        h = C.c_void_p()
        ctx.check(ctx.lib.mpq_nvfp4_weight_create(ctx.h, N, K, _np_ptr(codes), _np_ptr(sf), C.c_float(tensor_scale), C.byref(h)))
        super().__init__(ctx, h)
        self.tensor_scale = float(tensor_scale)


class QuantLinear:
    """y = x . W^T for a quantised weight.

    Q4:    x fp32 [M][K] (torch CUDA tensor or numpy host array) -> fp32 [M][N]
    NVFP4: x = (codes u8 [M][K/2], sf u8 [M][K/16], tensor_scale) on the GPU -> bf16 [M][N]
    """

    def __init__(self, weight: _Weight):
        self.w = weight
        self.ctx = weight.ctx

    def forward(self, x, out=None):
        import torch
        w, ctx = self.w, self.ctx
        if w.fmt == _lib.FMT_Q4:
            if isinstance(x, np.ndarray):                      # host path: copies inside the library
                x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, w.K)
                y = np.empty((x.shape[0], w.N), dtype=np.float32) if out is None else out
                ctx.check(ctx.lib.mpq_q4_linear_forward_host(ctx.h, w.h, _np_ptr(x), x.shape[0], _np_ptr(y)))
                return y
            if x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
                raise MpqError(_lib.ERR_INVALID_ARG, "x must be a contiguous fp32 CUDA tensor")
            x2 = x.reshape(-1, w.K)
            y = torch.empty((x2.shape[0], w.N), dtype=torch.float32, device=x.device) if out is None else out
            ctx.check(ctx.lib.mpq_q4_linear_forward(ctx.h, w.h, C.c_void_p(x2.data_ptr()), x2.shape[0],
                                                    C.c_void_p(y.data_ptr()),
                                                    C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            return y
        codes, sf, ts = x
        M = codes.shape[0]
        y = torch.empty((M, w.N), dtype=torch.bfloat16, device=codes.device) if out is None else out
        ctx.check(ctx.lib.mpq_nvfp4_gemm_forward(ctx.h, w.h, C.c_void_p(codes.data_ptr()), C.c_void_p(sf.data_ptr()),
                                                 C.c_float(ts), M, C.c_void_p(y.data_ptr()),
                                                 C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return y

    __call__ = forward

    def forward_swiglu(self, gate_up, out=None):
        """Q4 only: y = (silu(gate) * up) . W^T for gate_up fp32 [M][2K] = [gate | up] on the GPU (the down projection of a
        feed-forward block with the SwiGLU fused into the kernel's activation staging)."""
        import torch
        w, ctx = self.w, self.ctx
        if w.fmt != _lib.FMT_Q4:
            raise MpqError(_lib.ERR_INVALID_ARG, "forward_swiglu is for Q4 weights")
        if gate_up.dtype != torch.float32 or not gate_up.is_cuda or not gate_up.is_contiguous():
            raise MpqError(_lib.ERR_INVALID_ARG, "gate_up must be a contiguous fp32 CUDA tensor")
        g2 = gate_up.reshape(-1, 2 * w.K)
        y = torch.empty((g2.shape[0], w.N), dtype=torch.float32, device=gate_up.device) if out is None else out
        ctx.check(ctx.lib.mpq_q4_linear_forward_swiglu(ctx.h, w.h, C.c_void_p(g2.data_ptr()), g2.shape[0], C.c_void_p(y.data_ptr()),
                                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return y


def swiglu(ctx: Context, gate_up):
    """silu(gate) * up for gate_up fp32 [M][2F] = [gate | up] on the GPU -> fp32 [M][F]."""
    import torch
    M, F2 = gate_up.shape
    out = torch.empty((M, F2 // 2), dtype=torch.float32, device=gate_up.device)
    ctx.check(ctx.lib.mpq_swiglu(ctx.h, C.c_void_p(gate_up.data_ptr()), M, F2 // 2, C.c_void_p(out.data_ptr()),
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return out


def nvfp4_quantize(ctx: Context, x, tensor_scale: float = 1.0, swiglu_fused: bool = False):
    """fp32 or bf16 [M][K] on the GPU -> (codes u8 [M][K/2], sf u8 [M][K/16]) ready to be the GEMM's A.  With swiglu_fused
    the input is [M][2K] = [gate | up] and silu(gate) * up is what gets quantised."""
    import torch
    M = x.shape[0]
    K = x.shape[1] // 2 if swiglu_fused else x.shape[1]
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty((M, K // 16), dtype=torch.uint8, device=x.device)
    fn = ctx.lib.mpq_nvfp4_quantize_swiglu if swiglu_fused else ctx.lib.mpq_nvfp4_quantize_activations
    ctx.check(fn(ctx.h, C.c_void_p(x.data_ptr()), 1 if x.dtype == torch.bfloat16 else 0, M, K, C.c_float(tensor_scale),
                 C.c_void_p(codes.data_ptr()), C.c_void_p(sf.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return codes, sf
