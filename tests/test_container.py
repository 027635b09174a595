"""The weight container: canonical files round-trip on the CPU; device-layout files round-trip on the GPU
without a repack pass and are refused when damaged or written for another layout."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from makepad_b200 import _lib, synth


def test_canonical_roundtrip_needs_no_gpu(tmp_path):
    import makepad_b200
    codes, scales = synth.q4_weight(96, 256, seed=1)
    p = str(tmp_path / "w.q4c")
    makepad_b200.save_canonical(p, _lib.FMT_Q4, codes, scales)
    fmt, c2, s2, ts = makepad_b200.load_canonical(p)
    assert fmt == _lib.FMT_Q4 and np.array_equal(c2, codes) and np.array_equal(s2, scales) and ts == 1.0
    b, sfb = synth.nvfp4_tensor(64, 128, seed=2)
    p2 = str(tmp_path / "w.fp4c")
    makepad_b200.save_canonical(p2, _lib.FMT_NVFP4, b, sfb, 0.25)
    fmt, c3, s3, ts = makepad_b200.load_canonical(p2)
    assert fmt == _lib.FMT_NVFP4 and np.array_equal(c3, b) and np.array_equal(s3, sfb) and ts == 0.25
    info = _lib.FileInfo()
    assert _lib.load().mpq_file_info(p2.encode(), C.byref(info)) == _lib.OK
    assert (info.kind, info.N, info.K, info.bytes_a, info.bytes_b) == (_lib.FILE_CANONICAL, 64, 128, 64 * 64, 64 * 8)


def test_canonical_files_are_validated(tmp_path):
    import makepad_b200
    lib = _lib.load()
    codes, scales = synth.q4_weight(32, 64, seed=3)
    p = str(tmp_path / "w.q4c")
    makepad_b200.save_canonical(p, _lib.FMT_Q4, codes, scales)
    raw = bytearray(open(p, "rb").read())
    info = _lib.FileInfo()
    # a flipped payload byte: the checksum catches it
    bad = bytearray(raw); bad[200] ^= 0x40
    open(p, "wb").write(bad)
    with pytest.raises(makepad_b200.MpqError) as e:
        makepad_b200.load_canonical(p)
    assert e.value.status == _lib.ERR_FORMAT
    # truncated, wrong magic, future container version
    open(p, "wb").write(raw[:-1])
    assert lib.mpq_file_info(p.encode(), C.byref(info)) == _lib.ERR_FORMAT
    bad = bytearray(raw); bad[0] ^= 1
    open(p, "wb").write(bad)
    assert lib.mpq_file_info(p.encode(), C.byref(info)) == _lib.ERR_FORMAT
    bad = bytearray(raw); struct.pack_into("<I", bad, 4, 99)
    open(p, "wb").write(bad)
    assert lib.mpq_file_info(p.encode(), C.byref(info)) == _lib.ERR_FORMAT
    assert lib.mpq_file_info(str(tmp_path / "missing").encode(), C.byref(info)) == _lib.ERR_IO
    # capacity and shape checks
    open(p, "wb").write(raw)
    small = np.empty(8, dtype=np.uint8)
    assert lib.mpq_canonical_load(p.encode(), small.ctypes.data, small.nbytes, small.ctypes.data, small.nbytes, None) == _lib.ERR_SHAPE
    assert lib.mpq_canonical_save(p.encode(), _lib.FMT_Q4, 32, 48, codes.ctypes.data, scales.ctypes.data, C.c_float(1.0)) == _lib.ERR_SHAPE


@pytest.mark.gpu
def test_device_layout_roundtrip(ctx, orc, tmp_path):
    import torch
    import makepad_b200
    codes, scales = synth.q4_weight(1000, 2112, seed=4)
    w = makepad_b200.Q4Weight(ctx, codes, scales)
    p = str(tmp_path / "w.q4d")
    w.save(p)
    before = ctx.launches
    w2 = makepad_b200.load_weight(ctx, p)
    assert ctx.launches == before                                  # no repack kernel ran
    assert (w2.N, w2.K, w2.fmt) == (1000, 2112, _lib.FMT_Q4) and w2.device_bytes == w.device_bytes
    assert np.array_equal(w2.dequantize().cpu().numpy().view(np.uint32), orc.q4_dequantize(codes, scales).view(np.uint32))
    x = torch.from_numpy(synth.activations(3, 2112, seed=5)).cuda()
    assert torch.equal(makepad_b200.QuantLinear(w)(x), makepad_b200.QuantLinear(w2)(x))
    # NVFP4
    b, sfb = synth.nvfp4_tensor(448, 512, seed=6)
    w4 = makepad_b200.Nvfp4Weight(ctx, b, sfb, 0.5)
    p4 = str(tmp_path / "w.fp4d")
    w4.save(p4)
    w5 = makepad_b200.load_weight(ctx, p4)
    assert w5.tensor_scale == 0.5
    assert np.array_equal(w5.dequantize().cpu().numpy().view(np.uint32), orc.nvfp4_dequantize(b, sfb, 0.5).view(np.uint32))
    a, sfa = synth.nvfp4_tensor(200, 512, seed=7)
    ad, sd = torch.from_numpy(a).cuda(), torch.from_numpy(sfa).cuda()
    assert torch.equal(makepad_b200.QuantLinear(w4)((ad, sd, 1.0)).view(torch.int16), makepad_b200.QuantLinear(w5)((ad, sd, 1.0)).view(torch.int16))
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_stale_or_damaged_cache_files_are_refused(ctx, tmp_path):
    import makepad_b200
    codes, scales = synth.q4_weight(64, 128, seed=8)
    w = makepad_b200.Q4Weight(ctx, codes, scales)
    p = str(tmp_path / "w.q4d")
    w.save(p)
    raw = bytearray(open(p, "rb").read())
    h = C.c_void_p()
    for mutate in ("layout", "payload", "truncate", "canonical"):
        bad = bytearray(raw)
        if mutate == "layout":
            struct.pack_into("<I", bad, 16, 1)                     # an older layout version
        elif mutate == "payload":
            bad[128 + 77] ^= 0x01
        elif mutate == "truncate":
            bad = bad[:-16]
        else:
            makepad_b200.save_canonical(p, _lib.FMT_Q4, codes, scales)
            bad = bytearray(open(p, "rb").read())
        open(p, "wb").write(bad)
        assert ctx.lib.mpq_weight_load(ctx.h, p.encode(), C.byref(h)) == _lib.ERR_FORMAT, mutate
        assert not h.value
    assert ctx.lib.mpq_weight_load(ctx.h, str(tmp_path / "nope").encode(), C.byref(h)) == _lib.ERR_IO
