"""Inference-mode batch-norm fused with its activation, through the C ABI, against float64 and
against the legacy two-kernel route (normalize, then positive_clip)."""
import numpy as np
import pytest
import torch

from tests.util import assert_close, make_inputs, random_shapes

pytestmark = pytest.mark.gpu


def truth(x, mean, var, gamma, beta, slope):
    c = x.shape[1]
    bs = (1, c) + (1,) * (x.ndim - 2)
    g = np.ones(c) if gamma is None else gamma.astype(np.float64)
    b = np.zeros(c) if (gamma is None or beta is None) else beta.astype(np.float64)
    t = (x.astype(np.float64) - mean.astype(np.float64).reshape(bs)) / np.sqrt(var.astype(np.float64)).reshape(bs)
    t = t * g.reshape(bs) + b.reshape(bs)
    return t, t * np.where(t > 0, 1.0, slope)


@pytest.mark.parametrize("shape,slope,affine", [
    ((32, 64, 28, 28), 0.0, True),
    ((16, 8, 56, 56), 0.1, True),          # leaky ReLU
    ((64, 96, 7, 7), 0.0, True),           # a 16-byte column spans two channels
    ((5, 3, 7, 7), 0.0, True),             # odd sizes: scalar path
    ((2, 4, 16, 32, 32), 1.0, False),      # NCDHW, no activation, no affine
    ((1, 1, 1, 1), 0.0, False),
    ((3, 70000, 1, 1), 0.01, True),        # dim0 = 1: every element its own channel
] + [(s, [0.0, 0.1, 1.0][i % 3], i % 2 == 0) for i, s in enumerate(random_shapes(32, 12, max_elems=1e6))])
def test_infer_matches_float64(shape, slope, affine):
    from anode_b200 import ops
    d = make_inputs(shape, seed=3, loc=0.5, scale=2.0, affine=affine)
    rng = np.random.default_rng(4)
    c = shape[1]
    mean = rng.normal(0.5, 0.2, c).astype(np.float32)
    var = rng.uniform(2.0, 6.0, c).astype(np.float32)
    x = torch.from_numpy(d["x"]).cuda()
    y = torch.full_like(x, float("nan"))
    g = None if d["gamma"] is None else torch.from_numpy(d["gamma"]).cuda()
    b = None if d["beta"] is None else torch.from_numpy(d["beta"]).cuda()
    axes = list(range(x.dim() - 2))
    ops.BatchNormalize2dActInferOp.apply(axes, x, torch.from_numpy(mean).cuda(), torch.from_numpy(var).cuda(), y, g, b, slope)
    torch.cuda.synchronize()
    pre, want = truth(d["x"], mean, var, d["gamma"], d["beta"], slope)
    assert_close(y.cpu().numpy(), want, "y", skip=np.abs(pre) < 1e-5)


def test_infer_equals_legacy_normalize_then_clip_and_runs_in_place():
    from anode_b200 import ops
    shape = (8, 6, 20, 20)
    d = make_inputs(shape, seed=9, affine=False)
    x = torch.from_numpy(d["x"]).cuda()
    c = shape[1]
    mean = torch.linspace(-0.2, 0.2, c, device="cuda")
    var = torch.linspace(0.8, 1.6, c, device="cuda")
    # the reference's route: BatchNormalize2dOp with the running statistics, then PositiveClipOp
    y_ref = torch.empty_like(x)
    ops.BatchNormalize2dOp.apply([0, 1], x, mean, var, y_ref)
    ops.PositiveClipOp.apply(y_ref, y_ref)
    ops.BatchNormalize2dActInferOp.apply([0, 1], x, mean, var, x)      # in place
    torch.cuda.synchronize()
    # rsqrtf in the legacy kernel against divide + square root here: a few ulp
    assert_close(x.cpu().numpy(), y_ref.cpu().numpy().astype(np.float64), "in place vs legacy", rtol=1e-5, atol=1e-6)


def test_layer_infer_uses_running_averages():
    from anode_b200 import ops
    shape = (16, 12, 28, 28)
    d = make_inputs(shape, seed=6)
    layer = ops.FusedBatchNormRelu(shape[1])
    layer.gamma.copy_(torch.from_numpy(d["gamma"])); layer.beta.copy_(torch.from_numpy(d["beta"]))
    x = torch.from_numpy(d["x"]).cuda()
    layer.forward(x)                                   # moves the running averages
    y = layer.infer(x)
    torch.cuda.synchronize()
    _, want = truth(d["x"], layer.avg_mean.cpu().numpy(), layer.avg_var.cpu().numpy(), d["gamma"], d["beta"], 0.0)
    assert_close(y.cpu().numpy(), want, "infer", skip=np.abs(want) < 1e-5)
