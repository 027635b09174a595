"""ctypes binding of libmpq.so (the C ABI in include/mpq.h).

The library is the product; this module only loads it.  A missing library is a
hard error: there is no Python or CPU fallback for any operator.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmpq.so")

OK = 0
ERR_INVALID_ARG, ERR_SHAPE, ERR_ALIGN, ERR_CUDA, ERR_UNSUPPORTED, ERR_PEER_TIMEOUT, ERR_STATE = -1, -2, -3, -4, -5, -6, -7
ERR_FORMAT, ERR_IO = -8, -9
FILE_CANONICAL, FILE_DEVICE = 1, 2
FMT_Q4, FMT_NVFP4 = 1, 2
TP_NONE, TP_COLUMN, TP_ROW = 0, 1, 2


class DeviceInfo(C.Structure):
    _fields_ = [("device", C.c_int32), ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("l2_bytes", C.c_int64), ("total_mem_bytes", C.c_int64), ("sm_clock_khz", C.c_int32),
                ("mem_clock_khz", C.c_int32)]


class FileInfo(C.Structure):
    _fields_ = [("kind", C.c_int32), ("fmt", C.c_int32), ("layout_version", C.c_int32), ("reserved", C.c_int32),
                ("N", C.c_int64), ("K", C.c_int64), ("bytes_a", C.c_int64), ("bytes_b", C.c_int64),
                ("tensor_scale", C.c_float), ("reserved2", C.c_int32)]


_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); mirrors include/mpq.h one to one
SIGNATURES = {
    "mpq_context_create": (_i32, [_i32, _pp]),
    "mpq_context_destroy": (_i32, [_vp]),
    "mpq_context_info": (_i32, [_vp, C.POINTER(DeviceInfo)]),
    "mpq_status_string": (C.c_char_p, [_i32]),
    "mpq_last_error": (C.c_char_p, [_vp]),
    "mpq_context_launch_count": (_i64, [_vp]),
    "mpq_context_poll_status": (_i32, [_vp]),
    "mpq_q4_weight_create": (_i32, [_vp, _i64, _i64, _vp, _vp, _i32, _i32, _i32, _pp]),
    "mpq_q4_weight_create_dev": (_i32, [_vp, _i64, _i64, _vp, _vp, _pp]),
    "mpq_nvfp4_weight_create": (_i32, [_vp, _i64, _i64, _vp, _vp, _f32, _pp]),
    "mpq_weight_shape": (_i32, [_vp, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i32)]),
    "mpq_weight_dequantize": (_i32, [_vp, _vp, _vp, _vp]),
    "mpq_weight_device_bytes": (_i64, [_vp]),
    "mpq_weight_destroy": (_i32, [_vp]),
    "mpq_q4_linear_forward": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp]),
    "mpq_q4_linear_forward_static": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp]),
    "mpq_q4_linear_forward_host": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "mpq_exchange_create": (_i32, [_vp, _i32, _i32, _i64, _pp]),
    "mpq_exchange_ipc_handle": (_i32, [_vp, _vp]),
    "mpq_exchange_attach": (_i32, [_vp, _vp]),
    "mpq_exchange_attach_pointers": (_i32, [_vp, _pp]),
    "mpq_exchange_buffer": (_i32, [_vp, _pp, C.POINTER(_i64)]),
    "mpq_exchange_set_wait_limit": (_i32, [_vp, C.c_uint32]),
    "mpq_exchange_graph_check": (_i32, [_vp]),
    "mpq_exchange_destroy": (_i32, [_vp]),
    "mpq_q4_linear_forward_allreduce": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "mpq_nvfp4_gemm_forward": (_i32, [_vp, _vp, _vp, _vp, _f32, _i64, _vp, _vp]),
    "mpq_nvfp4_dequantize": (_i32, [_vp, _i64, _i64, _vp, _vp, _f32, _vp, _vp]),
    "mpq_nvfp4_quantize_activations": (_i32, [_vp, _vp, _i32, _i64, _i64, _f32, _vp, _vp, _vp]),
    "mpq_nvfp4_quantize_swiglu": (_i32, [_vp, _vp, _i32, _i64, _i64, _f32, _vp, _vp, _vp]),
    "mpq_swiglu": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "mpq_q4_linear_forward_swiglu": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp]),
    "mpq_file_info": (_i32, [C.c_char_p, C.POINTER(FileInfo)]),
    "mpq_canonical_save": (_i32, [C.c_char_p, _i32, _i64, _i64, _vp, _vp, _f32]),
    "mpq_canonical_load": (_i32, [C.c_char_p, _vp, _i64, _vp, _i64, C.POINTER(_f32)]),
    "mpq_weight_save": (_i32, [_vp, _vp, C.c_char_p]),
    "mpq_weight_load": (_i32, [_vp, C.c_char_p, _pp]),
    "mpq_probe_hbm_read": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "mpq_probe_fp4_mma": (_i32, [_vp, _i32, C.POINTER(C.c_double), _vp]),
    "mpq_probe_f16_mma": (_i32, [_vp, _i32, _i32, _i32, C.POINTER(C.c_double)]),
}

_lib = None


def load() -> C.CDLL:
    """Load libmpq.so from the package directory; raise if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m makepad_b200.build` "
                               "(there is no fallback implementation)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError here = header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
