"""Each kernel behind the fused calls, forced with anode_gpu_batch_norm_fused_set_kernel, against the
float64 oracle on the shapes it is built for (plain layer, leaky ReLU, no affine, residual epilogue),
and the workspace contract across problems."""
import numpy as np
import pytest
import torch

from oracle import bn_oracle as o
from tests.test_gpu_fused import dev, host, run_fused
from tests.util import assert_close, assert_sum_close, check_layer, make_inputs

pytestmark = pytest.mark.gpu

KIND = {"tiled": 1, "cluster": 2, "resident": 3, "plain": 4}


@pytest.fixture(scope="module")
def ops():
    from anode_b200 import ops
    return ops


@pytest.fixture
def forced(ops):
    """Sets a kernel preference for one test and restores the automatic choice afterwards."""
    def use(name):
        ops.set_kernel(name)
    yield use
    ops.set_kernel("auto")


def kinds(ops, shape):
    from anode_b200 import _lib
    x = torch.empty(shape, device="meta")
    d0, c, n = ops.dims_of(x)
    f = _lib.load().anode_gpu_batch_norm_fused_kernel_kind
    return f(d0, c, n, 0), f(d0, c, n, 1)


RESIDENT_SHAPES = [
    (16, 8, 56, 56),        # one row per piece, every slice resident
    (64, 8, 56, 56),
    (2048, 2, 56, 56),      # slices larger than the ring: resident and streamed pieces
    (4, 3, 16, 64, 64),     # rows split into parts (a volume)
    (64, 16, 14, 14),       # short rows: several rows per piece
    (300, 5, 4, 17),        # 68 floats per row, 32 rows per piece, ragged last piece
    (1, 3, 64, 64),         # one sample
]


@pytest.mark.parametrize("shape", RESIDENT_SHAPES)
def test_resident_kernel_matches_float64(ops, forced, shape):
    forced("resident")
    assert kinds(ops, shape) == (3, 3)
    d = make_inputs(shape, seed=61, loc=0.5, scale=2.0)
    got, ws = run_fused(ops, d)
    truth = o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "resident %r " % (shape,))
    # a second and third launch on the same workspace (the records carry the launch's sequence number)
    for _ in range(2):
        again, _ = run_fused(ops, d, ws=ws)
        for k in ("y", "dx", "mean", "var", "dgamma", "dbeta"):
            assert (again[k] == got[k]).all(), k


@pytest.mark.parametrize("name,shape", [("tiled", (16, 8, 56, 56)), ("tiled", (8, 6, 112, 112)), ("cluster", (32, 64, 28, 28)),
                                        ("cluster", (64, 96, 7, 7)), ("plain", (16, 8, 56, 56)), ("plain", (5, 3, 7, 7)),
                                        ("resident", (8, 6, 112, 112))])
def test_forced_kernel_matches_float64(ops, forced, name, shape):
    forced(name)
    assert kinds(ops, shape) == (KIND[name], KIND[name])
    d = make_inputs(shape, seed=62, loc=0.3, scale=1.5)
    got, _ = run_fused(ops, d)
    truth = o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "%s %r " % (name, shape))


@pytest.mark.parametrize("shape", [(16, 8, 56, 56), (64, 16, 14, 14)])
@pytest.mark.parametrize("slope,affine", [(0.1, True), (1.0, False)])
def test_resident_kernel_general_activation(ops, forced, shape, slope, affine):
    forced("resident")
    d = make_inputs(shape, seed=63, loc=0.3, scale=1.5, affine=affine)
    x = dev(d["x"]); dy = dev(d["dy"]); g = dev(d["gamma"]); b = dev(d["beta"])
    c = shape[1]
    axes = list(range(x.dim() - 2))
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    rm = dev(d["run_mean"]); rv = dev(d["run_var"])
    dg = torch.zeros(c, device="cuda") if affine else None
    db = torch.zeros(c, device="cuda") if affine else None
    y = torch.empty_like(x); dx = torch.empty_like(x)
    ws = ops.Workspace(*ops.dims_of(x), x.device)
    ops.BatchNormalize2dFusedOp.apply(axes, 1e-5, 0.1, x, y, mean, var, rm, rv, g, b, workspace=ws, neg_slope=slope)
    ops.BatchNormalize2dBwdFusedOp.apply(axes, dy, x, mean, var, dx, g, b, dg, db, workspace=ws, neg_slope=slope)
    assert ws.status() == 0
    got = dict(y=host(y), dx=host(dx), mean=host(mean), var=host(var), run_mean=host(rm), run_var=host(rv),
               dgamma=host(dg), dbeta=host(db))
    truth = o.bn_act_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"], neg_slope=slope)
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "slope %g " % slope)


@pytest.mark.parametrize("shape", [(32, 6, 56, 56), (2048, 2, 56, 56), (64, 16, 14, 14), (4, 3, 16, 64, 64)])
def test_resident_kernel_residual_epilogue(ops, forced, shape):
    """y = relu(bn(x) + shortcut) and its adjoint on long rows: a third tensor in every slot."""
    forced("resident")
    d = make_inputs(shape, seed=64, loc=0.3, scale=1.5)
    res_h = np.random.default_rng(65).standard_normal(shape).astype(np.float32)
    x = dev(d["x"]); dy = dev(d["dy"]); res = dev(res_h); g = dev(d["gamma"]); b = dev(d["beta"])
    c = shape[1]
    axes = list(range(x.dim() - 2))
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    rm = dev(d["run_mean"]); rv = dev(d["run_var"])
    dg = torch.zeros(c, device="cuda"); db = torch.zeros(c, device="cuda")
    y = torch.empty_like(x); dx = torch.empty_like(x); dres = torch.empty_like(x)
    ws = ops.Workspace(*ops.dims_of(x), x.device)
    ops.BatchNormalize2dAddActFusedOp.apply(axes, 1e-5, 0.1, x, res, y, mean, var, rm, rv, g, b, 0.0, ws)
    ops.BatchNormalize2dAddActFusedOp.adjoint(axes, dy, x, y, mean, var, dx, dres, g, b, dg, db, 0.0, workspace=ws)
    assert ws.status() == 0
    truth = o.bn_add_act_fwd_bwd_f64(d["x"], res_h, d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"], neg_slope=0.0)
    bs = (1, c) + (1,) * (len(shape) - 2)
    pre = ((d["x"].astype(np.float64) - truth["mean"].reshape(bs)) / np.sqrt(truth["var"]).reshape(bs)
           * d["gamma"].astype(np.float64).reshape(bs) + d["beta"].astype(np.float64).reshape(bs) + res_h)
    skip = np.abs(pre) < 1e-5
    for k, t in (("mean", mean), ("var", var), ("run_mean", rm), ("run_var", rv)):
        assert_close(host(t), truth[k], k)
    assert_close(host(y), truth["y"], "y", skip=skip)
    assert_close(host(dx), truth["dx"], "dx", skip=skip)
    assert_close(host(dres), truth["dresidual"], "dresidual", skip=skip)
    assert_sum_close(host(dg), truth["dgamma"], "dgamma")
    assert_sum_close(host(db), truth["dbeta"], "dbeta")
    # without the optional shortcut gradient
    dx2 = torch.empty_like(x)
    ops.BatchNormalize2dAddActFusedOp.adjoint(axes, dy, x, y, mean, var, dx2, None, g, b, dg, db, 0.0, workspace=ws)
    assert ws.status() == 0 and (host(dx2) == host(dx)).all()


@pytest.mark.parametrize("name", ["tiled", "resident"])
def test_one_buffer_serves_two_problems_when_reinitialised_in_between(ops, forced, name):
    """A workspace belongs to one problem; handing the same memory to another problem is allowed after
    anode_gpu_batch_norm_fused_workspace_init.  Alternates two shapes served by the same kernel."""
    forced(name)
    shapes = [(16, 8, 56, 56), (32, 8, 56, 56)]
    data = [make_inputs(s, seed=70 + i, loc=0.5, scale=2.0) for i, s in enumerate(shapes)]
    truth = [o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"]) for d in data]
    big = max((ops.Workspace(*ops.dims_of(torch.empty(s, device="meta")), "cuda") for s in shapes), key=lambda w: w.bytes)
    for rnd in range(2):
        for s, d, t in zip(shapes, data, truth):
            big.reset()
            got, _ = run_fused(ops, d, ws=big)
            check_layer(got, t, d["x"], d["gamma"], d["beta"], "round %d %r " % (rnd, s))
