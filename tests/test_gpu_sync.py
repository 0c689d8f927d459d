"""Synchronized batch-norm on real GPUs through the C ABI.  world = 1 runs everywhere; the
2-rank case needs two visible GPUs (one process per GPU, NCCL) and is skipped otherwise.
Parity definition: the G-way result equals the oracle on the concatenated global batch."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import bn_oracle as o
from tests.util import check_layer, make_inputs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, shape, axis, out_dir, dist_kind, exchange):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from anode_b200 import ops, sync
    d = make_inputs(shape, seed=41, dist=dist_kind, loc=0.5 if dist_kind == "normal" else 0.0,
                    scale=2.0 if dist_kind == "normal" else 4.0)
    lo, hi = sync.shard_range(shape[axis], rank, world)
    idx = [slice(None)] * len(shape); idx[axis] = slice(lo, hi)
    x = torch.from_numpy(np.ascontiguousarray(d["x"][tuple(idx)])).cuda()
    dy = torch.from_numpy(np.ascontiguousarray(d["dy"][tuple(idx)])).cuda()
    per_channel = int(np.prod(shape)) // shape[1]          # shards may be uneven: the global count is stated
    layer = ops.SyncBatchNormRelu(shape[1], epsilon=1e-5, avg_rate=0.1, exchange=exchange, global_count=per_channel)
    assert layer.launches_per_step == (2 if (exchange or world == 1) else 6)
    layer.gamma.copy_(torch.from_numpy(d["gamma"])); layer.beta.copy_(torch.from_numpy(d["beta"]))
    # twice on one workspace, other data the first time: nothing of a step may reach the next one
    for xs, dys in ((x * 2.0 + 1.0, dy * 0.5), (x, dy)):
        layer.avg_mean.zero_(); layer.avg_var.fill_(1.0)
        y = layer.forward(xs)
        dx = layer.backward(dys)
    torch.cuda.synchronize()
    assert layer.status() == 0
    # the same step with the shard in page-locked host memory, through the one-call host-buffer entry point
    hx, hdy = x.cpu().pin_memory(), dy.cpu().pin_memory()
    hy, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
    layer.avg_mean.zero_(); layer.avg_var.fill_(1.0)
    blocks = layer.step_from_host(hx, hdy, hy, hdx, chunk_channels=max(1, shape[1] // 3))
    torch.cuda.synchronize()
    assert blocks >= 1 and layer.host_step_status() == 0
    tol = lambda a, b: bool(((a - b).abs() <= 1e-5 + 1e-4 * b.abs()).all())
    assert tol(hy, y.cpu()) and tol(hdx, dx.cpu()), "host-buffer step differs from the device step"
    # the gradient all-reduce that shares the communicator (SumSpmdOp's role)
    grad = torch.full((1000,), float(rank + 1), device="cuda")
    layer.comm.allreduce_sum(grad)
    torch.cuda.synchronize()
    assert (grad == world * (world + 1) / 2).all()
    np.savez(os.path.join(out_dir, "r%d.npz" % rank), y=y.cpu().numpy(), dx=dx.cpu().numpy(),
             mean=layer.mean.cpu().numpy(), var=layer.var.cpu().numpy(), run_mean=layer.avg_mean.cpu().numpy(),
             run_var=layer.avg_var.cpu().numpy(), dgamma=layer.dgamma.cpu().numpy(), dbeta=layer.dbeta.cpu().numpy())
    dist.barrier()
    layer.comm.destroy()
    dist.destroy_process_group()


CASES = [((16, 8, 28, 28), 0, "normal"), ((8, 4, 8, 16, 16), 2, "normal"), ((32, 64, 7, 7), 0, "student3"),
         ((6, 3, 5, 5), 0, "normal"),
         ((48, 12, 56, 56), 0, "normal"),      # long rows: the slice-resident kernel with the exchange inside
         ((19, 6, 56, 56), 0, "normal"),       # uneven shards (19 samples over 2, 4 or 8 ranks)
         ((8, 4, 16, 64, 64), 2, "normal"),    # depth slabs of a volume
         ((23, 5, 9, 9), 0, "normal")]         # scalar path, uneven shards: reduce kernel, exchange kernel, apply kernel


def _run(tmp_path, world, shape, axis, dist_kind, exchange=True):
    if shape[axis] < world:
        pytest.skip("fewer items along the sharded axis than ranks")
    port = 30000 + (os.getpid() * 7 + hash((shape, axis, world)) % 997) % 3000
    mp.spawn(_worker, args=(world, port, shape, axis, str(tmp_path), dist_kind, exchange), nprocs=world, join=True)
    d = make_inputs(shape, seed=41, dist=dist_kind, loc=0.5 if dist_kind == "normal" else 0.0,
                    scale=2.0 if dist_kind == "normal" else 4.0)
    truth = o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    parts = [np.load(os.path.join(str(tmp_path), "r%d.npz" % r)) for r in range(world)]
    got = {k: parts[0][k] for k in ("mean", "var", "run_mean", "run_var", "dgamma", "dbeta")}
    for p in parts[1:]:
        for k in got:
            assert (p[k] == got[k]).all(), k      # identical on every rank, bit for bit
    got["y"] = np.concatenate([p["y"] for p in parts], axis=axis)
    got["dx"] = np.concatenate([p["dx"] for p in parts], axis=axis)
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "world %d " % world)


@pytest.mark.parametrize("shape,axis,dist_kind", CASES)
def test_sync_world1_matches_oracle(tmp_path, shape, axis, dist_kind):
    _run(tmp_path, 1, shape, axis, dist_kind)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", [True, False], ids=["in-kernel-exchange", "nccl-all-gather"])
@pytest.mark.parametrize("shape,axis,dist_kind", CASES)
def test_sync_world2_matches_oracle(tmp_path, shape, axis, dist_kind, exchange):
    _run(tmp_path, 2, shape, axis, dist_kind, exchange)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
@pytest.mark.parametrize("shape,axis,dist_kind", CASES)
def test_sync_world4_matches_oracle(tmp_path, shape, axis, dist_kind):
    _run(tmp_path, 4, shape, axis, dist_kind, True)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs eight GPUs")
@pytest.mark.parametrize("shape,axis,dist_kind", CASES)
def test_sync_world8_matches_oracle(tmp_path, shape, axis, dist_kind):
    _run(tmp_path, 8, shape, axis, dist_kind, True)


# ---- the residual-block epilogue across GPUs -----------------------------------------------------------

def _residual_worker(rank, world, port, shape, axis, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from anode_b200 import ops, sync
    d = make_inputs(shape, seed=43, loc=0.3, scale=1.5)
    res_h = np.random.default_rng(44).standard_normal(shape).astype(np.float32)
    lo, hi = sync.shard_range(shape[axis], rank, world)
    idx = [slice(None)] * len(shape); idx[axis] = slice(lo, hi)
    cut = lambda a: torch.from_numpy(np.ascontiguousarray(a[tuple(idx)])).cuda()
    x, dy, res = cut(d["x"]), cut(d["dy"]), cut(res_h)
    layer = ops.SyncBatchNormRelu(shape[1], epsilon=1e-5, avg_rate=0.1, global_count=int(np.prod(shape)) // shape[1])
    layer.gamma.copy_(torch.from_numpy(d["gamma"])); layer.beta.copy_(torch.from_numpy(d["beta"]))
    for _ in range(2):      # twice on one workspace
        layer.avg_mean.zero_(); layer.avg_var.fill_(1.0)
        y = layer.forward_add(x, res)
        dx, dres = layer.backward_add(dy, dresidual=torch.empty_like(x))
    torch.cuda.synchronize()
    assert layer.status() == 0
    np.savez(os.path.join(out_dir, "r%d.npz" % rank), y=y.cpu().numpy(), dx=dx.cpu().numpy(), dres=dres.cpu().numpy(),
             mean=layer.mean.cpu().numpy(), var=layer.var.cpu().numpy(), run_mean=layer.avg_mean.cpu().numpy(),
             run_var=layer.avg_var.cpu().numpy(), dgamma=layer.dgamma.cpu().numpy(), dbeta=layer.dbeta.cpu().numpy())
    dist.barrier()
    layer.comm.destroy()
    dist.destroy_process_group()


RESIDUAL_CASES = [((24, 6, 56, 56), 0),      # long rows: the slice-resident kernel, exchange inside
                  ((32, 64, 7, 7), 0),       # short rows: the cluster kernel, exchange inside
                  ((10, 3, 5, 5), 0)]        # scalar path: reduce kernel, exchange kernel, apply kernel


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("shape,axis", RESIDUAL_CASES)
def test_sync_residual_epilogue_matches_oracle(tmp_path, shape, axis, world):
    from tests.util import assert_close, assert_sum_close
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    port = 33000 + (os.getpid() * 5 + hash((shape, world)) % 997) % 3000
    mp.spawn(_residual_worker, args=(world, port, shape, axis, str(tmp_path)), nprocs=world, join=True)
    d = make_inputs(shape, seed=43, loc=0.3, scale=1.5)
    res_h = np.random.default_rng(44).standard_normal(shape).astype(np.float32)
    truth = o.bn_add_act_fwd_bwd_f64(d["x"], res_h, d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"], neg_slope=0.0)
    parts = [np.load(os.path.join(str(tmp_path), "r%d.npz" % r)) for r in range(world)]
    c = shape[1]
    bs = (1, c) + (1,) * (len(shape) - 2)
    pre = ((d["x"].astype(np.float64) - truth["mean"].reshape(bs)) / np.sqrt(truth["var"]).reshape(bs)
           * d["gamma"].astype(np.float64).reshape(bs) + d["beta"].astype(np.float64).reshape(bs) + res_h)
    skip = np.abs(pre) < 1e-5
    for k in ("mean", "var", "run_mean", "run_var"):
        for p in parts:
            assert (p[k] == parts[0][k]).all(), k
        assert_close(parts[0][k], truth[k], k)
    cat = lambda k: np.concatenate([p[k] for p in parts], axis=axis)
    assert_close(cat("y"), truth["y"], "y", skip=skip)
    assert_close(cat("dx"), truth["dx"], "dx", skip=skip)
    assert_close(cat("dres"), truth["dresidual"], "dresidual", skip=skip)
    assert_sum_close(parts[0]["dgamma"], truth["dgamma"], "dgamma")
    assert_sum_close(parts[0]["dbeta"], truth["dbeta"], "dbeta")
