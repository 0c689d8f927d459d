"""Fused forward / backward kernels against the oracle, through the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import bn_oracle as o
from tests.util import assert_close, assert_sum_close, check_layer, make_inputs

pytestmark = pytest.mark.gpu


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    if t is None:
        return None
    torch.cuda.synchronize()
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def ops():
    from anode_b200 import ops
    return ops


def run_fused(ops, d, eps=1e-5, rate=0.1, relu=True, ws=None):
    x = dev(d["x"]); dy = dev(d["dy"])
    c = x.shape[1]
    axes = list(range(x.dim() - 2))
    g, b = dev(d["gamma"]), dev(d["beta"])
    rm, rv = dev(d["run_mean"]), dev(d["run_var"])
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    y = torch.full_like(x, float("nan")); dx = torch.full_like(x, float("nan"))
    dg = torch.zeros(c, device="cuda") if g is not None else None
    db = torch.zeros(c, device="cuda") if g is not None else None
    d0, cc, n = ops.dims_of(x)
    ws = ws or ops.Workspace(d0, cc, n, x.device)
    ops.BatchNormalize2dFusedOp.apply(axes, eps, rate, x, y, mean, var, rm, rv, g, b, relu, ws)
    ops.BatchNormalize2dBwdFusedOp.apply(axes, dy, x, mean, var, dx, g, b, dg, db, relu, ops.WriteCap.Assign, ws)
    assert ws.status() == 0
    return dict(y=host(y), dx=host(dx), mean=host(mean), var=host(var), run_mean=host(rm), run_var=host(rv),
                dgamma=host(dg), dbeta=host(db)), ws


CASES = [
    # shape, dist, loc, scale, affine        (regime the planner picks)
    ((32, 64, 28, 28), "normal", 0.0, 1.0, True),      # config 1 of the benchmark; rows, 128-bit
    ((8, 6, 112, 112), "normal", 0.5, 2.0, True),      # config 2 geometry, fewer samples/channels
    ((16, 8, 56, 56), "normal", 0.0, 1.0, True),       # config 3 geometry
    ((2, 4, 16, 32, 32), "normal", 0.0, 1.0, True),    # config 4 geometry (NCDHW slab)
    ((64, 96, 7, 7), "student3", 0.0, 4.0, True),      # config 5 geometry; segments regime
    ((5, 3, 7, 7), "normal", 0.5, 2.0, True),          # C*dim0 odd: scalar rows
    ((3, 2, 1, 1), "normal", 0.0, 1.0, False),
    ((1, 1, 1, 1), "normal", 0.0, 1.0, False),
    ((7, 5, 9, 13), "normal", 3.0, 0.5, True),         # odd everything, mean >> sigma
    ((4, 4, 33, 35), "normal", 100.0, 0.1, True),      # |mean|/sigma = 1000: cancellation stress
    ((2, 3, 200, 204), "normal", 0.0, 1.0, True),      # long rows split into pieces
    ((33, 260, 3, 5), "normal", 0.0, 1.0, True),       # segments, ragged last channel block
    ((4, 8, 4, 4), "normal", 0.0, 1.0, False),         # segments with aligned tiny rows
    ((2, 4, 3, 6, 8), "normal", 0.0, 1.0, True),
]


@pytest.mark.parametrize("shape,dist,loc,scale,affine", CASES)
def test_fused_layer_matches_oracle(ops, shape, dist, loc, scale, affine):
    d = make_inputs(shape, seed=7, dist=dist, loc=loc, scale=scale, affine=affine)
    got, _ = run_fused(ops, d)
    args = (d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    truth = o.bn_relu_fwd_bwd_f64(*args)
    atol = 1e-5
    if abs(loc) > 100 * scale:
        # Conditioning, not the kernel: the mean is returned (and re-read by the backward pass) as
        # f32, so xhat = (x - mean)/sigma carries half an ulp of |mean| divided by sigma, times gamma.
        atol = 1e-5 + 1.5 * float(np.spacing(np.float32(abs(loc)))) / scale
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "vs f64 ", atol_elem=atol, check_sums=atol == 1e-5)
    if abs(loc) <= 10 * scale:
        # the literal f32 restatement of the reference's kernel chain (it is itself inaccurate
        # when |mean| >> sigma, so that case is checked against float64 only)
        lit = o.bn_relu_fwd_bwd_f32(*args)
        check_layer(got, lit, d["x"], d["gamma"], d["beta"], "vs literal ")


def test_no_relu_no_affine_equals_plain_normalize(ops):
    d = make_inputs((6, 5, 12, 12), seed=8, affine=False)
    got, _ = run_fused(ops, d, relu=False)
    mean = o.batch_mean(d["x"]); var = o.batch_var(d["x"], mean, 1e-5)
    assert_close(got["y"], o.batch_norm(d["x"], mean, var), "y")
    # without ReLU the adjoint is the reference's seven-kernel chain on dy itself
    dvar = o.batch_norm_bwd_var(d["dy"], d["x"], mean, var)
    dmean = o.batch_var_bwd_mean(dvar, d["x"], mean, dmean=o.batch_norm_bwd_mean(d["dy"], var))
    dx = o.batch_mean_bwd(dmean, d["x"].shape,
                          dx=o.batch_var_bwd(dvar, d["x"], mean, dx=o.batch_norm_bwd(d["dy"], var)))
    assert_close(got["dx"], dx, "dx")


def test_workspace_reuse_inplace_and_accumulate(ops):
    shape = (8, 6, 20, 20)
    d = make_inputs(shape, seed=10, loc=0.5, scale=2.0)
    first, ws = run_fused(ops, d)
    again, _ = run_fused(ops, d, ws=ws)          # same workspace, no re-initialisation
    for k in first:
        assert (first[k] == again[k]).all(), k   # deterministic, bit for bit
    # in place: y over x, dx over dy
    x = dev(d["x"]); dy = dev(d["dy"]); x_keep = x.clone()
    c = shape[1]
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    g, b = dev(d["gamma"]), dev(d["beta"])
    ops.BatchNormalize2dFusedOp.apply([0, 1], 1e-5, 0.1, x, x, mean, var, None, None, g, b, True, ws)
    assert (host(x) == first["y"]).all()
    ops.BatchNormalize2dBwdFusedOp.apply([0, 1], dy, x_keep, mean, var, dy, g, b, None, None, True,
                                         ops.WriteCap.Assign, ws)
    assert (host(dy) == first["dx"]).all()
    # accumulate: dx_old + dx
    old = torch.ones_like(x_keep)
    ops.BatchNormalize2dBwdFusedOp.apply([0, 1], dev(d["dy"]), x_keep, mean, var, old, g, b, None, None, True,
                                         ops.WriteCap.Accumulate, ws)
    assert_close(host(old), 1.0 + first["dx"].astype(np.float64), "accumulate", rtol=1e-6, atol=1e-6)
    assert ws.status() == 0


def test_consecutive_steps_with_new_data_share_one_workspace(ops):
    """Training: the same layer and workspace, different data every step.  The two directions tile
    this shape differently, so state either of them leaves in the workspace must not reach the other
    (or its own next launch)."""
    shape = (64, 32, 56, 56)
    ws = None
    for step in range(3):
        d = make_inputs(shape, seed=100 + step, loc=0.3 * step, scale=1.0 + step)
        got, ws = run_fused(ops, d, ws=ws)
        truth = o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"],
                                      d["gamma"], d["beta"])
        check_layer(got, truth, d["x"], d["gamma"], d["beta"], what="step %d " % step)


def test_misaligned_pointers_take_the_scalar_path(ops):
    shape = (4, 4, 8, 8)
    d = make_inputs(shape, seed=12)
    n = int(np.prod(shape))
    bufx = torch.zeros(n + 1, device="cuda"); bufd = torch.zeros(n + 1, device="cuda")
    bufx[1:] = dev(d["x"]).flatten(); bufd[1:] = dev(d["dy"]).flatten()
    d2 = dict(d)
    got_ref, _ = run_fused(ops, d)
    x = bufx[1:].view(shape); dy = bufd[1:].view(shape)      # 4-byte aligned only
    c = shape[1]
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    y = torch.empty(n + 1, device="cuda")[1:].view(shape); dx = torch.empty(n + 1, device="cuda")[1:].view(shape)
    g, b = dev(d["gamma"]), dev(d["beta"])
    ws = ops.Workspace(*ops.dims_of(x), x.device)
    ops.BatchNormalize2dFusedOp.apply([0, 1], 1e-5, 0.1, x, y, mean, var, None, None, g, b, True, ws)
    ops.BatchNormalize2dBwdFusedOp.apply([0, 1], dy, x, mean, var, dx, g, b, None, None, True,
                                         ops.WriteCap.Assign, ws)
    assert_close(host(y), got_ref["y"], "y", rtol=1e-6, atol=1e-6)
    assert_close(host(dx), got_ref["dx"], "dx", rtol=1e-5, atol=1e-6)
    del d2


def test_argument_errors(ops):
    from anode_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(2, 2, 2, 2, device="cuda")
    v = torch.zeros(2, device="cuda")
    ws = ops.Workspace(4, 2, 2, x.device)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(4, 2, 2, 1e-5, 0.1, 1, None, None, None, p(x), p(v),
                                                                p(v), None, None, ws.ptr, ws.bytes, None, None)
    assert rc == -1
    rc = lib.anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(0, 2, 2, 1e-5, 0.1, 1, p(x), None, None, p(x), p(v),
                                                                p(v), None, None, ws.ptr, ws.bytes, None, None)
    assert rc == -2
    rc = lib.anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(4, 2, 2, 1e-5, 0.1, 1, p(x), None, None, p(x), p(v),
                                                                p(v), None, None, ws.ptr, 16, None, None)
    assert rc == -3
    with pytest.raises(ValueError):
        ops.BatchMean2dOp.apply([1, 0], x, v)


@pytest.mark.parametrize("shape", [(16, 8, 56, 56), (64, 96, 7, 7), (5, 3, 7, 7)])    # tiled, cluster and plain kernels
@pytest.mark.parametrize("slope", [0.1, 1.0, 0.0])
def test_general_activation_matches_float64(ops, shape, slope):
    """Leaky ReLU (flat_map.cu:44-69) fused like the ReLU: t*(t > 0 ? 1 : slope)."""
    d = make_inputs(shape, seed=17, loc=0.3, scale=1.5)
    x = dev(d["x"]); dy = dev(d["dy"]); g = dev(d["gamma"]); b = dev(d["beta"])
    c = shape[1]
    axes = list(range(x.dim() - 2))
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    rm = dev(d["run_mean"]); rv = dev(d["run_var"])
    dg = torch.zeros(c, device="cuda"); db = torch.zeros(c, device="cuda")
    y = torch.empty_like(x); dx = torch.empty_like(x)
    ws = ops.Workspace(*ops.dims_of(x), x.device)
    ops.BatchNormalize2dFusedOp.apply(axes, 1e-5, 0.1, x, y, mean, var, rm, rv, g, b, workspace=ws, neg_slope=slope)
    ops.BatchNormalize2dBwdFusedOp.apply(axes, dy, x, mean, var, dx, g, b, dg, db, workspace=ws, neg_slope=slope)
    assert ws.status() == 0
    got = dict(y=host(y), dx=host(dx), mean=host(mean), var=host(var), run_mean=host(rm), run_var=host(rv),
               dgamma=host(dg), dbeta=host(db))
    truth = o.bn_act_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"],
                                 neg_slope=slope)
    check_layer(got, truth, d["x"], d["gamma"], d["beta"], "slope %g " % slope)
    if slope == 0.0:      # the same launch as relu = 1
        ref, _ = run_fused(ops, d)
        assert (ref["y"] == got["y"]).all() and (ref["dx"] == got["dx"]).all()


@pytest.mark.parametrize("shape", [(16, 8, 56, 56), (64, 96, 7, 7), (5, 3, 7, 7), (2, 4, 8, 16, 16)])
@pytest.mark.parametrize("slope", [0.0, 0.1])
def test_residual_epilogue_matches_float64(ops, shape, slope):
    """y = act(bn(x) + residual) and its adjoint (mask from the saved y, dresidual = dy*mask)."""
    d = make_inputs(shape, seed=19, loc=0.3, scale=1.5)
    res_h = np.random.default_rng(20).standard_normal(shape).astype(np.float32)
    x = dev(d["x"]); dy = dev(d["dy"]); res = dev(res_h); g = dev(d["gamma"]); b = dev(d["beta"])
    c = shape[1]
    axes = list(range(x.dim() - 2))
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    rm = dev(d["run_mean"]); rv = dev(d["run_var"])
    dg = torch.zeros(c, device="cuda"); db = torch.zeros(c, device="cuda")
    y = torch.empty_like(x); dx = torch.empty_like(x); dres = torch.empty_like(x)
    ws = ops.Workspace(*ops.dims_of(x), x.device)
    ops.BatchNormalize2dAddActFusedOp.apply(axes, 1e-5, 0.1, x, res, y, mean, var, rm, rv, g, b, slope, ws)
    ops.BatchNormalize2dAddActFusedOp.adjoint(axes, dy, x, y, mean, var, dx, dres, g, b, dg, db, slope, workspace=ws)
    assert ws.status() == 0
    truth = o.bn_add_act_fwd_bwd_f64(d["x"], res_h, d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"],
                                     neg_slope=slope)
    got = dict(y=host(y), dx=host(dx), mean=host(mean), var=host(var), run_mean=host(rm), run_var=host(rv),
               dgamma=host(dg), dbeta=host(db))
    # elements whose pre-activation is within 1e-5 of zero may take either side of the mask
    bs = (1, c) + (1,) * (len(shape) - 2)
    pre = ((d["x"].astype(np.float64) - truth["mean"].reshape(bs)) / np.sqrt(truth["var"]).reshape(bs)
           * d["gamma"].astype(np.float64).reshape(bs) + d["beta"].astype(np.float64).reshape(bs) + res_h)
    skip = np.abs(pre) < 1e-5
    assert skip.mean() < 1e-3
    for k in ("mean", "var", "run_mean", "run_var"):
        assert_close(got[k], truth[k], k)
    assert_close(got["y"], truth["y"], "y", skip=skip)
    assert_close(got["dx"], truth["dx"], "dx", skip=skip)
    assert_close(host(dres), truth["dresidual"], "dresidual", skip=skip)
    assert_sum_close(got["dgamma"], truth["dgamma"], "dgamma")
    assert_sum_close(got["dbeta"], truth["dbeta"], "dbeta")
