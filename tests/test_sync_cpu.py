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


# ---- failure detection on the host (no GPU): ranks that disagree, a rank that never arrives ----------

def _mismatch_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from anode_b200._lib import AnodeError
    sync.check_same_on_every_rank([64, 3136], "dims")            # agreeing ranks pass
    try:
        sync.check_same_on_every_rank([64 if rank == 0 else 32], "channel count")
        msg = "no error"
    except AnodeError as e:
        msg = "code %d" % e.code
    with open(os.path.join(out_dir, "r%d.txt" % rank), "w") as f:
        f.write(msg)
    dist.barrier()
    dist.destroy_process_group()


def test_mismatched_channel_count_is_refused_on_every_rank(tmp_path):
    port = 29100 + os.getpid() % 1500
    mp.spawn(_mismatch_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(os.path.join(str(tmp_path), "r%d.txt" % r)).read() == "code -5"


def _absent_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from anode_b200._lib import AnodeError
    import datetime
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    if rank == 1:
        # this rank dies before the rendezvous: it connects to the store and leaves without announcing itself
        return
    import time
    t0 = time.time()
    try:
        sync.wait_for_ranks(store, world, rank, "layer0", timeout_s=1.5)
        msg = "no error"
    except AnodeError as e:
        msg = "code %d after %.1f s" % (e.code, time.time() - t0)
    with open(os.path.join(out_dir, "r%d.txt" % rank), "w") as f:
        f.write(msg)


def test_rank_that_never_arrives_becomes_an_error_not_a_wait(tmp_path):
    port = 29300 + os.getpid() % 1500
    mp.spawn(_absent_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    msg = open(os.path.join(str(tmp_path), "r0.txt")).read()
    assert msg.startswith("code -5 after"), msg
    assert float(msg.split()[3]) < 10.0


def _present_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import datetime
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    sync.wait_for_ranks(store, world, rank, "layer0", timeout_s=10.0)
    with open(os.path.join(out_dir, "r%d.txt" % rank), "w") as f:
        f.write("ok")
    if rank == 0:      # keep the store alive until the other rank has read it
        store.wait(["done/1"], datetime.timedelta(seconds=10))
    else:
        store.set("done/1", "1")


def test_rendezvous_passes_when_every_rank_arrives(tmp_path):
    port = 29500 + os.getpid() % 1500
    mp.spawn(_present_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all(open(os.path.join(str(tmp_path), "r%d.txt" % r)).read() == "ok" for r in range(2))
