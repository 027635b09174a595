"""Builds libmpq.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

`python -m makepad_b200.build [-v] [--trace]`; --trace builds the diagnostic variant libmpq_trace.so
(-DMPQ_TRACE: the Q4 streaming kernel stamps its phases, see makepad_b200/timeline.py).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmpq.so")
LIB_TRACE = os.path.join(HERE, "libmpq_trace.so")
SOURCES = ["mpq.cu", "nvfp4_gemm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _stale(lib: str) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "mpq.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    lib = LIB_TRACE if trace else LIB
    if not force and not _stale(lib):
        return lib
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", "_trace.o" if trace else ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if trace:
            cmd.insert(1, "-DMPQ_TRACE")
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        subprocess.check_call(cmd)
        objs.append(obj)
    subprocess.check_call([nvcc, "-shared", "-o", lib, *objs])
    return lib


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
