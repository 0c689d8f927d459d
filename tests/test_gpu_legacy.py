"""The reference's own entry points (same names and signatures) on the GPU, one by one,
against the literal CPU oracle.  Every call goes through the C ABI via anode_b200.ops."""
import numpy as np
import pytest
import torch

from oracle import bn_oracle as o
from tests.util import assert_close, assert_sum_close, make_inputs, random_shapes

pytestmark = pytest.mark.gpu

SHAPES = [(32, 64, 28, 28), (5, 3, 7, 7), (3, 2, 1, 1), (2, 4, 3, 6, 8), (7, 5, 9, 13), (1, 1, 1, 1),
          (64, 40, 7, 7), (2, 3, 64, 66)] + random_shapes(31, 12, max_elems=4e5)      # and a dozen nobody picked by hand


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def ops():
    from anode_b200 import ops
    return ops


@pytest.mark.parametrize("shape", SHAPES)
def test_forward_kernels(ops, shape):
    d = make_inputs(shape, seed=3, loc=0.5, scale=2.0)
    x = d["x"]
    axes = list(range(len(shape) - 2))
    c = shape[1]
    tx = dev(x)
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    ops.BatchMean2dOp.apply(axes, tx, mean)
    ops.BatchVariance2dOp.apply(axes, 1e-5, tx, mean, var)
    want_mean = o.batch_mean(x)
    assert_close(host(mean), want_mean, "mean")
    # variance measured around the oracle's mean so the two kernels are checked separately
    ops.BatchVariance2dOp.apply(axes, 1e-5, tx, dev(want_mean), var)
    want_var = o.batch_var(x, want_mean, 1e-5)
    assert_close(host(var), want_var, "var")
    y = torch.empty_like(tx)
    ops.BatchNormalize2dOp.apply(axes, tx, dev(want_mean), dev(want_var), y)
    want_y = o.batch_norm(x, want_mean, want_var)
    assert_close(host(y), want_y, "normalize")
    r = torch.empty_like(tx)
    ops.PositiveClipOp.apply(y, r)
    assert (host(r) == o.positive_clip(host(y))).all()
    ops.PositiveClipOp.apply(y, y)          # in place
    assert (host(y) == host(r)).all()


@pytest.mark.parametrize("shape", SHAPES)
def test_backward_kernels_assign_and_accumulate(ops, shape):
    d = make_inputs(shape, seed=4, loc=-0.25, scale=1.5)
    x, dy = d["x"], d["dy"]
    axes = list(range(len(shape) - 2))
    c = shape[1]
    mean = o.batch_mean(x); var = o.batch_var(x, mean, 1e-5)
    y = o.positive_clip(o.batch_norm(x, mean, var))
    tx, tdy, tmean, tvar, ty = dev(x), dev(dy), dev(mean), dev(var), dev(y)
    A, ACC = ops.WriteCap.Assign, ops.WriteCap.Accumulate
    rng = np.random.default_rng(9)
    old_c = rng.standard_normal(c).astype(np.float32)
    old_x = rng.standard_normal(shape).astype(np.float32)

    dz = torch.empty_like(tx)
    ops.PositiveClipBwdOp.apply(tdy, ty, dz)
    want_dz = o.positive_clip_bwd(dy, y)
    assert (host(dz) == want_dz).all()
    j = torch.empty_like(tx)
    ops.FlatJoinOp.apply(tdy, ty, j)
    assert (host(j) == want_dz).all()

    for cap, old in ((A, None), (ACC, old_c)):
        out = torch.zeros(c, device="cuda") if old is None else dev(old)
        ops.BatchNormalize2dBwdVarianceOp.apply(axes, dz, tx, tmean, tvar, out, cap)
        assert_sum_close(host(out), o.batch_norm_bwd_var(want_dz, x, mean, var, dvar=old), "bwd_var")
        out = torch.zeros(c, device="cuda") if old is None else dev(old)
        xhat = o.batch_norm(x, mean, var)
        ops.BatchNormalize2dBwdVarianceOp.apply_v2(axes, dz, dev(xhat), tvar, out, cap)
        assert_sum_close(host(out), o.batch_norm_bwd_var_v2(want_dz, xhat, var, dvar=old), "bwd_var_v2")
        out = torch.zeros(c, device="cuda") if old is None else dev(old)
        ops.BatchNormalize2dBwdMeanOp.apply(axes, dz, tvar, out, cap)
        assert_sum_close(host(out), o.batch_norm_bwd_mean(want_dz, var, dmean=old), "bwd_mean")
        dvar = o.batch_norm_bwd_var(want_dz, x, mean, var)
        out = torch.zeros(c, device="cuda") if old is None else dev(old)
        ops.BatchVariance2dBwdMeanOp.apply(axes, dev(dvar), tx, tmean, out, cap)
        # this term is rounding noise around zero (sum of x-mean); compare on the scale of dvar
        want = o.batch_var_bwd_mean(dvar, x, mean, dmean=old)
        assert_close(host(out), want, "var_bwd_mean", atol=1e-5 + 1e-5 * float(np.abs(dvar).max()))

    dvar = o.batch_norm_bwd_var(want_dz, x, mean, var)
    dmean = o.batch_norm_bwd_mean(want_dz, var)
    for cap, old in ((A, None), (ACC, old_x)):
        out = torch.empty_like(tx) if old is None else dev(old)
        ops.BatchNormalize2dBwdOp.apply(axes, dz, tvar, out, cap)
        assert_close(host(out), o.batch_norm_bwd(want_dz, var, dx=old), "norm_bwd")
        out = torch.empty_like(tx) if old is None else dev(old)
        ops.BatchVariance2dBwdOp.apply(axes, dev(dvar), tx, tmean, out, cap)
        assert_close(host(out), o.batch_var_bwd(dvar, x, mean, dx=old), "var_bwd")
        out = torch.empty_like(tx) if old is None else dev(old)
        ops.BatchMean2dBwdOp.apply(axes, dev(dmean), tx, out, cap)
        assert_close(host(out), o.batch_mean_bwd(dmean, shape, dx=old), "mean_bwd")


def test_online_average_known_answer(ops):
    # reference tests/test_gpu.rs:561-593
    x = torch.ones(1024, device="cuda"); y = torch.zeros(1024, device="cuda")
    ops.OnlineAverageOp.apply(0.25, x, y)
    assert (host(y) == np.float32(0.25)).all()
    ops.OnlineAverageOp.apply(0.25, x, y)
    assert (host(y) == np.float32(0.4375)).all()


@pytest.mark.parametrize("shape", [(32, 64, 28, 28), (5, 3, 7, 7), (2, 4, 3, 6, 8)])
def test_front_end_composition(ops, shape):
    """batch_normalize_2d/3d + relu forward and the seven-kernel adjoint, as the reference's
    graph would run them, against the literal oracle of the whole layer."""
    d = make_inputs(shape, seed=6, loc=0.5, scale=2.0, affine=False)
    x, dy = d["x"], d["dy"]
    axes = list(range(len(shape) - 2))
    want = o.bn_relu_fwd_bwd_f32(x, dy, 1e-5, 0.1, d["run_mean"], d["run_var"])
    tx = dev(x)
    fn = ops.batch_normalize_2d if len(shape) == 4 else ops.batch_normalize_3d
    y, mean, var, am, av = fn(tx, axes, True, 0.1, 1e-5, dev(d["run_mean"]), dev(d["run_var"]))
    ops.relu(y, inplace=True)
    dz = torch.empty_like(tx)
    ops.PositiveClipBwdOp.apply(dev(dy), y, dz)
    dx, _, _ = ops.batch_normalize_adjoint(axes, dz, tx, mean, var)
    from tests.util import check_layer
    got = dict(y=host(y), dx=host(dx), mean=host(mean), var=host(var), run_mean=host(am), run_var=host(av))
    check_layer(got, want, x, None, None)
    # inference branch: normalizes with the running averages (src/ops.rs:1010-1011)
    y2, *_ = fn(tx, axes, False, 0.0, 1e-5, am.clone(), av.clone())
    assert_close(host(y2), o.batch_norm(x, host(am), host(av)), "online=false")
