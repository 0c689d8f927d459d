"""Forward + backward with the tensors in host memory (channel blocks, copies overlapped with the
kernels), through the C ABI, against the oracle and against the device-resident entry points."""
import numpy as np
import pytest
import torch

from oracle import bn_oracle as o
from tests.util import check_layer, make_inputs

pytestmark = pytest.mark.gpu


def pinned(a):
    t = torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    return t


def run_host_step(d, chunk, in_place=False):
    from anode_b200 import ops
    c = d["x"].shape[1]
    layer = ops.FusedBatchNormRelu(c, epsilon=1e-5, avg_rate=0.1)
    layer.gamma.copy_(torch.from_numpy(d["gamma"])); layer.beta.copy_(torch.from_numpy(d["beta"]))
    hx, hdy = pinned(d["x"]), pinned(d["dy"])
    hy = hx if in_place else torch.full(hx.shape, float("nan")).pin_memory()
    hdx = hdy if in_place else torch.full(hx.shape, float("nan")).pin_memory()
    blocks = layer.step_from_host(hx, hdy, hy, hdx, chunk_channels=chunk)
    assert layer.host_step_status() == 0          # synchronises
    got = dict(y=hy.numpy().copy(), dx=hdx.numpy().copy(), mean=layer.mean.cpu().numpy(), var=layer.var.cpu().numpy(),
               run_mean=layer.avg_mean.cpu().numpy(), run_var=layer.avg_var.cpu().numpy(),
               dgamma=layer.dgamma.cpu().numpy(), dbeta=layer.dbeta.cpu().numpy())
    return got, blocks, layer


@pytest.mark.parametrize("shape,chunk,want_blocks", [
    ((8, 24, 20, 20), 8, 3),        # equal blocks
    ((8, 24, 20, 20), 10, 3),       # last block smaller: tiled differently, same workspace
    ((8, 24, 20, 20), 0, 6),        # library's choice: at least four blocks
    ((8, 24, 20, 20), 24, 1),       # one block: plain 1-D copies
    ((16, 40, 7, 7), 12, 4),        # short rows (segments regime), ragged tail
    ((3, 5, 9, 13), 4, 2),          # odd sizes: scalar kernels on the blocks
    ((2, 6, 8, 16, 16), 4, 2),      # NCDHW
])
def test_host_step_matches_oracle(shape, chunk, want_blocks):
    d = make_inputs(shape, seed=21, loc=0.5, scale=2.0)
    got, blocks, _ = run_host_step(d, chunk)
    assert blocks == want_blocks
    truth = o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "host step ")


def test_host_step_in_place_and_repeated_with_new_data():
    shape = (32, 16, 56, 56)
    layer_stats = None
    for step in range(2):
        d = make_inputs(shape, seed=30 + step, loc=0.2 * step, scale=1.0 + step)
        got, _, _ = run_host_step(d, 4, in_place=True)
        truth = o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
        check_layer(got, truth, d["x"], d["gamma"], d["beta"], "in place, step %d " % step)


def test_host_step_equals_device_resident_calls():
    from anode_b200 import ops
    shape = (16, 12, 28, 28)
    d = make_inputs(shape, seed=5)
    got, _, _ = run_host_step(d, 12)           # one block: the same problem as the resident call
    layer = ops.FusedBatchNormRelu(shape[1])
    layer.gamma.copy_(torch.from_numpy(d["gamma"])); layer.beta.copy_(torch.from_numpy(d["beta"]))
    x = torch.from_numpy(d["x"]).cuda(); dy = torch.from_numpy(d["dy"]).cuda()
    y = layer.forward(x); dx = layer.backward(dy)
    torch.cuda.synchronize()
    assert (y.cpu().numpy() == got["y"]).all() and (dx.cpu().numpy() == got["dx"]).all()
    assert (layer.mean.cpu().numpy() == got["mean"]).all() and (layer.dgamma.cpu().numpy() == got["dgamma"]).all()


def test_host_step_argument_errors():
    from anode_b200 import ops
    layer = ops.FusedBatchNormRelu(4)
    good = torch.zeros(2, 4, 3, 3).pin_memory()
    with pytest.raises(ValueError):
        layer.step_from_host(good.cuda(), good, good, good)
    with pytest.raises(ValueError):
        layer.step_from_host(good[:, :2], good, good, good)
