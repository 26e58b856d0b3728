"""The N>1 host logic, on CPU with two gloo ranks: each rank computes its column shard of a (reduced) config-3
mul with the oracle into its slice of the full column-major destination, the shards are all-gathered in
place exactly as bench.py does over NCCL, and every rank must end up with the unsharded result."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import util
from ruy_b200 import cases
from ruy_b200.sharding import column_shard, mul_range


def test_ranges_cover_everything_once():
    for n, world in ((16384, 8), (10, 4), (3, 8), (0, 2)):
        got = []
        for r in range(world):
            first, count = mul_range(n, r, world)
            got.extend(range(first, first + count))
        assert got == list(range(n))
    assert [column_shard(8192, r, 8) for r in range(8)] == [(1024 * r, 1024) for r in range(8)]
    with pytest.raises(ValueError):
        column_shard(10, 0, 4)


def test_column_shards_equal_slices_of_the_whole():
    whole = cases.config3(rows=64, depth=96, cols=512, dst="int8")
    for rank in range(2):
        first, count = column_shard(512, rank, 2)
        part = cases.config3(rows=64, depth=96, cols=512, dst="int8", col_begin=first, col_count=count)
        assert np.array_equal(part.lhs, whole.lhs) and np.array_equal(part.bias, whole.bias)
        assert np.array_equal(part.rhs, whole.rhs.reshape(512, 96)[first:first + count].reshape(-1))
    # config 2: a shard is the corresponding slice of the whole job
    all_muls = cases.config2(n=40, seed=0)
    first, count = mul_range(40, 1, 3)
    shard = cases.config2(n=40, seed=0, first=first, count=count)
    for a, b in zip(all_muls[first:first + count], shard):
        assert a.name == b.name and np.array_equal(a.lhs, b.lhs) and np.array_equal(a.rhs, b.rhs)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rows, depth, cols = 48, 160, 256
    first, count = column_shard(cols, rank, world)
    case = cases.config3(rows=rows, depth=depth, cols=cols, dst="int8", col_begin=first, col_count=count)
    full = torch.zeros(rows * cols, dtype=torch.int8)
    mine = full[first * rows:(first + count) * rows]
    mine.copy_(torch.from_numpy(np.ascontiguousarray(util.run_oracle(case).T).reshape(-1)))   # column-major shard
    dist.all_gather_into_tensor(full, mine.clone())
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gather_the_full_destination(tmp_path):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    whole = cases.config3(rows=48, depth=160, cols=256, dst="int8")
    want = np.ascontiguousarray(util.run_oracle(whole).T).reshape(-1)
    for rank in range(world):
        assert np.array_equal(np.load(tmp_path / f"rank{rank}.npy"), want)
