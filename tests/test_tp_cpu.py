"""Host-side logic of the tensor-parallel layer on CPU: shard ranges, and -- as two gloo ranks -- that the
sharded computation (column slices gathered, row partials summed in rank order) equals the unsharded oracle."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges():
    from makepad_b200.tensor_parallel import shard_range
    assert shard_range(57344, 3, 8) == (21504, 28672)
    assert shard_range(28672, 7, 8, 32) == (25088, 28672)
    assert shard_range(11008, 1, 8, 32) == (1376, 2752)                  # 43 blocks of 32 per rank
    with pytest.raises(ValueError):
        shard_range(4096, 0, 3)
    with pytest.raises(ValueError):
        shard_range(4096 + 32, 0, 8, 32)
    with pytest.raises(ValueError):
        shard_range(64, 2, 2)


def test_shard_q4_slices_blocks_consistently():
    from makepad_b200 import _lib, synth
    from makepad_b200.tensor_parallel import shard_q4
    codes, scales = synth.q4_weight(64, 256, seed=1)
    c, s = shard_q4(codes, scales, _lib.TP_ROW, 1, 4)
    assert c.shape == (64, 32) and s.shape == (64, 2)
    assert np.array_equal(c, codes[:, 32:64]) and np.array_equal(s, scales[:, 2:4])
    c, s = shard_q4(codes, scales, _lib.TP_COLUMN, 3, 4)
    assert np.array_equal(c, codes[48:]) and np.array_equal(s, scales[48:])


def _rank_main(rank, world, port, ok):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from makepad_b200 import _lib, synth
    from makepad_b200.tensor_parallel import shard_q4, shard_range
    from oracle import oracle as orc
    N, K, M = 96, 512, 3
    codes, scales = synth.q4_weight(N, K, seed=5)
    x = synth.activations(M, K, seed=6)
    ref = orc.q4_matmul_f64(codes, scales, x, threads=1)
    # column-parallel: each rank's slice, gathered
    c, s = shard_q4(codes, scales, _lib.TP_COLUMN, rank, world)
    part = torch.from_numpy(orc.q4_matmul_f64(c, s, x, threads=1))
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    good = np.array_equal(torch.cat(parts, dim=1).numpy(), ref)
    # row-parallel: partial sums added in rank order
    c, s = shard_q4(codes, scales, _lib.TP_ROW, rank, world)
    a, b = shard_range(K, rank, world, 32)
    partial = torch.from_numpy(orc.q4_matmul_f64(c, s, x[:, a:b], threads=1))
    parts = [torch.empty_like(partial) for _ in range(world)]
    dist.all_gather(parts, partial)
    total = parts[0].clone()
    for p in parts[1:]:
        total += p
    good = good and np.allclose(total.numpy(), ref, rtol=1e-12, atol=1e-12)
    ok[rank] = 1 if good else 0
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_oracle():
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_rank_main, args=(world, 29611, ok), nprocs=world, join=True)
    assert list(ok) == [1] * world
