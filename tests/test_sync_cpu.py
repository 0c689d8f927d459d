"""Multi-rank host logic on CPU: two gloo ranks shard a batch, exchange per-channel moment
records with an all-gather and merge them in rank order; the result must equal the oracle's
statistics of the whole batch.  (The GPU path does the same merge on the device.)"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from anode_b200 import sync
from oracle import bn_oracle as o
from tests.util import assert_close, make_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, shape, axis, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d = make_inputs(shape, seed=31, loc=0.5, scale=2.0)
    lo, hi = sync.shard_range(shape[axis], rank, world)
    idx = [slice(None)] * len(shape); idx[axis] = slice(lo, hi)
    local = np.ascontiguousarray(d["x"][tuple(idx)])
    rec = torch.from_numpy(sync.local_moments(local))            # [C, 3] float64
    gathered = [torch.empty_like(rec) for _ in range(world)]
    dist.all_gather(gathered, rec)
    n, mean, m2 = sync.merge_moments(torch.stack(gathered).numpy())
    np.save(os.path.join(out_dir, "r%d.npy" % rank), np.stack([n, mean, m2 / n + 1e-5]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("shape,axis,world", [((8, 5, 6, 6), 0, 2), ((7, 3, 4, 4), 0, 2), ((2, 4, 6, 4, 4), 2, 2), ((9, 4, 3, 3), 0, 3)])
def test_two_rank_merge_equals_global_statistics(tmp_path, shape, axis, world):
    port = 29000 + (os.getpid() + hash((shape, axis)) % 500) % 2000
    mp.spawn(_worker, args=(world, port, shape, axis, str(tmp_path)), nprocs=world, join=True)
    d = make_inputs(shape, seed=31, loc=0.5, scale=2.0)
    mean = o.batch_mean(d["x"]); var = o.batch_var(d["x"], mean, 1e-5)
    results = [np.load(os.path.join(str(tmp_path), "r%d.npy" % r)) for r in range(world)]
    for r in results:
        assert (r == results[0]).all()                 # every rank ends with bit-identical statistics
        assert_close(r[1], mean, "mean"); assert_close(r[2], var, "var")
        assert (r[0] == d["x"].size / shape[1]).all()


def test_shard_range_partitions_exactly():
    for extent in (1, 7, 8, 2048, 128):
        for world in (1, 2, 3, 4, 8):
            got = [sync.shard_range(extent, r, world) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == extent
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [b - a for a, b in got]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sync.shard_range(8, 2, 2)
