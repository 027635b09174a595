"""Host-side logic of the library that needs no GPU: the per-device bookkeeping that guards settings CUDA
keeps per device (kernel attributes, symbol addresses), compiled with g++ from the header the library uses."""
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include "per_device.h"
#include <cstdio>
int main()
{
    mpq::PerDeviceOnce once;
    int bad = 0;
    // nothing is configured at the start, on any device
    for (int d = 0; d < mpq::PerDeviceOnce::MAX_DEVICES; ++d) bad += !once.needs(d);
    // configuring device 0 leaves device 1 unconfigured (the fault a per-process flag has)
    once.mark(0);
    bad += once.needs(0);
    bad += !once.needs(1);
    once.mark(1);
    bad += once.needs(1);
    bad += !once.needs(2);
    // indices outside the table are always (re)configured and never written
    bad += !once.needs(-1);
    bad += !once.needs(mpq::PerDeviceOnce::MAX_DEVICES);
    once.mark(-1);
    once.mark(mpq::PerDeviceOnce::MAX_DEVICES + 5);
    bad += !once.needs(-1);
    bad += !once.needs(mpq::PerDeviceOnce::MAX_DEVICES + 5);
    // two independent instances (two kernels) do not share state
    mpq::PerDeviceOnce other;
    bad += !other.needs(0);
    std::printf("%d\n", bad);
    return bad;
}
"""


def test_per_device_flags_are_per_device():
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = os.path.join(tmp, "t.cpp"), os.path.join(tmp, "t")
        open(src, "w").write(PROGRAM)
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "makepad_b200", "csrc"), src, "-o", exe])
        out = subprocess.run([exe], capture_output=True, text=True)
        assert out.returncode == 0 and out.stdout.strip() == "0", out.stdout + out.stderr


def test_no_per_process_flag_guards_a_per_device_setting():
    """Every cudaFuncSetAttribute in the library sits behind PerDeviceOnce, none behind a plain static bool."""
    csrc = os.path.join(ROOT, "makepad_b200", "csrc")
    for f in os.listdir(csrc):
        if f.endswith((".cu", ".cuh")):
            text = open(os.path.join(csrc, f)).read()
            assert "static bool configured" not in text, f
