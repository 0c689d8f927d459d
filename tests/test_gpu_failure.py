"""Failure detection on the device, in the form that cannot hurt a GPU: a synchronized call whose peer
never writes its records.  One process, one GPU, an exchange-only communicator that claims two ranks
with both exchange buffers in local memory; the wait limit is set to 20 ms, so the kernel's bounded
wait runs out, the status word says so, the kernel drains and returns, and after a re-initialisation
the same workspace serves a normal call.  Nothing here faults, traps or spins without bound."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import bn_oracle as o
from tests.util import check_layer, make_inputs

pytestmark = pytest.mark.gpu

WAIT_STATS, WAIT_PEER, ABORTED = 1, 2, 4


@pytest.fixture
def short_waits():
    from anode_b200 import ops
    ops.set_wait_limit_ms(20)
    yield ops
    ops.set_wait_limit_ms(1500)
    ops.set_kernel("auto")


@pytest.mark.parametrize("kernel,shape", [("tiled", (16, 8, 56, 56)), ("resident", (16, 8, 56, 56)), ("cluster", (32, 64, 7, 7)),
                                          ("plain", (6, 3, 5, 5))])
def test_wait_for_an_absent_peer_runs_out_and_the_workspace_recovers(short_waits, kernel, shape):
    ops = short_waits
    from anode_b200 import _lib, sync
    lib = _lib.load()
    ops.set_kernel(kernel)
    d = make_inputs(shape, seed=81, loc=0.5, scale=2.0)
    x = torch.from_numpy(d["x"]).cuda(); dy = torch.from_numpy(d["dy"]).cuda()
    c = shape[1]
    comm = sync.SyncComm.exchange_only(0, 2)
    nbytes = int(lib.anode_gpu_sync_exchange_bytes(c, 2))
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    comm.attach_exchange_pointers(bufs, c)
    layer = ops.SyncBatchNormRelu(c, comm=comm, global_count=2 * x.numel() // c)
    layer.gamma.copy_(torch.from_numpy(d["gamma"])); layer.beta.copy_(torch.from_numpy(d["beta"]))
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    layer.forward(x)
    t1.record()
    torch.cuda.synchronize()
    status = layer.status()
    assert status & WAIT_PEER, status
    if kernel in ("tiled", "resident"):
        assert status & ABORTED, status
    assert t0.elapsed_time(t1) < 1000.0          # the 20 ms bound, not the default 1.5 s, and certainly no hang
    # this rank's own record did reach "the peer" (a local buffer here): the exchange itself works
    assert int(bufs[1].view(torch.int64).ne(0).sum()) > 0
    comm.destroy()
    # recovery: re-initialise the workspace, then a normal (one-GPU) call on it is right again
    ops.set_wait_limit_ms(1500)
    ws = layer._ws
    ws.reset()
    torch.cuda.synchronize()
    assert ws.status() == 0
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    rm = torch.from_numpy(d["run_mean"]).cuda(); rv = torch.from_numpy(d["run_var"]).cuda()
    dg = torch.zeros(c, device="cuda"); db = torch.zeros(c, device="cuda")
    y = torch.empty_like(x); dx = torch.empty_like(x)
    axes = list(range(x.dim() - 2))
    ops.BatchNormalize2dFusedOp.apply(axes, 1e-5, 0.1, x, y, mean, var, rm, rv, layer.gamma, layer.beta, True, ws)
    ops.BatchNormalize2dBwdFusedOp.apply(axes, dy, x, mean, var, dx, layer.gamma, layer.beta, dg, db, True, ops.WriteCap.Assign, ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    got = dict(y=y.cpu().numpy(), dx=dx.cpu().numpy(), mean=mean.cpu().numpy(), var=var.cpu().numpy(), run_mean=rm.cpu().numpy(),
               run_var=rv.cpu().numpy(), dgamma=dg.cpu().numpy(), dbeta=db.cpu().numpy())
    truth = o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "after recovery ")


def test_exchange_only_communicator_refuses_what_it_cannot_do():
    from anode_b200 import _lib, sync
    lib = _lib.load()
    comm = sync.SyncComm.exchange_only(1, 2)
    buf = torch.zeros(8, device="cuda")
    # no NCCL behind it: the gradient all-reduce is refused, nothing is enqueued
    assert lib.anode_gpu_sync_allreduce_sum_f32(comm.handle, ctypes.c_void_p(buf.data_ptr()), 8, None) == -5
    # no exchange attached yet: a synchronized call is refused as well
    ws = torch.zeros(int(lib.anode_gpu_sync_batch_norm_workspace_bytes(64, 4, 2, 2)), dtype=torch.uint8, device="cuda")
    x = torch.zeros(2, 4, 8, 8, device="cuda"); v = torch.zeros(4, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32(64, 4, 2, 1e-5, 0.1, 1, p(x), None, None, p(x), p(v), p(v), None, None,
                                                               comm.handle, p(ws), ws.numel(), None, None)
    assert rc == -5
    torch.cuda.synchronize()
    comm.destroy()
