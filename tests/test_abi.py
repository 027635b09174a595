"""The C-ABI library loads and exports exactly what include/mpq.h declares (no compute calls)."""
import ctypes
import os
import re

from makepad_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "mpq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(mpq_[a-z0-9_]+)\s*\(", text))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    lib = ctypes.CDLL(path)
    names = _header_symbols()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), f"{n} declared in mpq.h but not exported"


def test_python_binding_covers_the_header():
    assert set(_lib.SIGNATURES) == _header_symbols()
    _lib.load()


def test_status_strings_and_null_handles():
    lib = _lib.load()
    assert lib.mpq_status_string(0) == b"ok"
    for code in range(-7, 0):
        assert lib.mpq_status_string(code) not in (b"ok", b"unknown status")
    assert lib.mpq_status_string(-99) == b"unknown status"
    # bad handles are rejected before any CUDA call
    assert lib.mpq_context_destroy(None) == _lib.ERR_INVALID_ARG
    assert lib.mpq_weight_destroy(None) == _lib.ERR_INVALID_ARG
    assert lib.mpq_q4_linear_forward(None, None, None, 1, None, None) == _lib.ERR_INVALID_ARG
    assert lib.mpq_context_launch_count(None) == -1


def test_product_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "makepad_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".rs")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("no Python or CPU fallback", ""), f"{f} mentions the oracle"
