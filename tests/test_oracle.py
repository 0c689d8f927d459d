"""The CPU oracle against its pins: the reference's running-average known-answer test, the
float64 restatements, and the committed golden vectors produced by the reference's kernels."""
import glob
import os

import numpy as np
import pytest

from oracle import bn_oracle as o
from tests.util import assert_close, assert_sum_close, check_layer, make_inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_online_average_known_answer():
    # reference tests/test_gpu.rs:561-593: y0 = 0, x = 1, rate 0.25 -> 0.25, then 0.4375 (exact)
    x = np.ones(1024, np.float32)
    y = np.zeros(1024, np.float32)
    y = o.online_average(0.25, x, y)
    assert (y == np.float32(0.25)).all()
    y = o.online_average(0.25, x, y)
    assert (y == np.float32(0.4375)).all()


@pytest.mark.parametrize("shape,affine", [((32, 64, 28, 28), True), ((32, 64, 28, 28), False),
                                          ((5, 3, 7, 7), True), ((2, 4, 3, 5, 6), True), ((1, 1, 1, 1), False)])
def test_literal_matches_float64(shape, affine):
    d = make_inputs(shape, seed=1, loc=0.5, scale=2.0, affine=affine)
    args = (d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    truth = o.bn_relu_fwd_bwd_f64(*args)
    check_layer(o.bn_relu_fwd_bwd_f32(*args), truth, d["x"], d["gamma"], d["beta"], "tree ")
    check_layer(o.bn_relu_fwd_bwd_f32(*args, block_sz=0), truth, d["x"], d["gamma"], d["beta"], "fast ")
    # the C float64 code and the independent numpy restatement agree to rounding
    nt = o.numpy_truth(*args)
    for k in ("y", "dx", "mean", "var", "run_mean", "run_var"):
        np.testing.assert_allclose(truth[k], nt[k], rtol=1e-10, atol=1e-10)


def test_heavy_tail_literal_matches_float64():
    d = make_inputs((64, 16, 7, 7), seed=5, dist="student3", scale=4.0)
    args = (d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    check_layer(o.bn_relu_fwd_bwd_f32(*args), o.bn_relu_fwd_bwd_f64(*args), d["x"], d["gamma"], d["beta"])


def test_single_kernels_compose_to_the_layer():
    """The per-kernel oracle functions, chained by hand in the reference's order, reproduce the
    whole-layer function bit for bit (same code path), and Accumulate adds to the old value."""
    d = make_inputs((6, 5, 4, 4), seed=2, affine=False)
    x, dy = d["x"], d["dy"]
    whole = o.bn_relu_fwd_bwd_f32(x, dy, 1e-5, 0.1, d["run_mean"], d["run_var"])
    mean = o.batch_mean(x)
    var = o.batch_var(x, mean, 1e-5)
    y = o.positive_clip(o.batch_norm(x, mean, var))
    dz = o.positive_clip_bwd(dy, y)
    dvar = o.batch_norm_bwd_var(dz, x, mean, var)
    dmean = o.batch_var_bwd_mean(dvar, x, mean, dmean=o.batch_norm_bwd_mean(dz, var))
    dx = o.batch_mean_bwd(dmean, x.shape, dx=o.batch_var_bwd(dvar, x, mean, dx=o.batch_norm_bwd(dz, var)))
    assert (mean == whole["mean"]).all() and (var == whole["var"]).all()
    assert (y == whole["y"]).all() and (dx == whole["dx"]).all()
    # v2 form of dvar (uses the saved normalized output) agrees with the x form
    xhat = o.batch_norm(x, mean, var)
    assert_sum_close(o.batch_norm_bwd_var_v2(dz, xhat, var), dvar, "dvar v2")
    base = np.full(5, 3.0, np.float32)
    acc = o.batch_norm_bwd_var(dz, x, mean, var, dvar=base)
    np.testing.assert_allclose(acc, base + dvar, rtol=1e-6)


def test_relu_edge_values():
    x = np.array([-1.0, -0.0, 0.0, 2.5, np.inf], np.float32)
    y = o.positive_clip(x)
    assert y[3] == 2.5 and y[4] == np.inf and y[0] == 0 and np.signbit(y[0])   # x*(x>0): -0 for negatives
    assert np.isnan(o.positive_clip(np.array([-np.inf, np.nan], np.float32))).all()
    dz = o.positive_clip_bwd(np.array([1.0, 2.0, 3.0], np.float32), np.array([0.0, -1.0, 4.0], np.float32))
    assert (dz == np.array([0.0, 0.0, 3.0], np.float32)).all()


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz"))))
def test_golden_vectors_from_reference_kernels(path):
    """Golden vectors were produced by the reference's own CUDA kernels on a B200
    (tests/golden/make_golden.py).  mean and var are reductions of exactly rounded terms in a
    fixed tree, so the literal oracle must reproduce them bit for bit; y and dx go through the
    device's approximate rsqrtf, so they get a tolerance of a few ulp."""
    g = np.load(path)
    x, dy = g["x"], g["dy"]
    block = int(g["block_sz"])
    lit = o.bn_relu_fwd_bwd_f32(x, dy, float(g["eps"]), float(g["avg_rate"]), g["run_mean0"], g["run_var0"],
                                block_sz=block)
    assert (lit["mean"] == g["mean"]).all(), "mean not bit-exact"
    assert (lit["var"] == g["var"]).all(), "var not bit-exact"
    for k in ("run_mean", "run_var"):
        assert_close(lit[k], g[k], k, rtol=1e-6, atol=1e-7)
    for k in ("y", "dx"):
        assert_close(lit[k], g[k], k, rtol=2e-6, atol=2e-6)


def test_golden_vectors_present():
    assert glob.glob(os.path.join(GOLDEN, "ref_*.npz")), "tests/golden/ref_*.npz missing"


def test_leaky_relu_literal_and_float64_variants_agree():
    """The leaky-ReLU functors of the reference (flat_map.cu:44-69) and the float64 layer with a
    negative slope: C against the independent numpy restatement, and slope 0 against the ReLU layer."""
    x = np.array([-2.0, -0.0, 0.0, 0.5, 3.0], np.float32)
    y = o.leaky_relu(0.1, x)
    assert np.allclose(y, [-0.2, -0.0, 0.0, 0.5, 3.0])
    dx = o.leaky_relu_bwd(0.1, np.ones_like(x), y)
    assert np.allclose(dx, [0.1, 0.1, 0.1, 1.0, 1.0])
    d = make_inputs((6, 5, 4, 3), seed=12, loc=0.3, scale=1.5)
    args = (d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
    for slope in (0.0, 0.1, 1.0):
        c = o.bn_act_fwd_bwd_f64(*args, neg_slope=slope)
        n = o.numpy_truth(*args, neg_slope=slope)
        for k in c:
            assert np.allclose(c[k], n[k], rtol=1e-9, atol=1e-11), (slope, k)
    relu = o.bn_relu_fwd_bwd_f64(*args)
    zero = o.bn_act_fwd_bwd_f64(*args, neg_slope=0.0)
    for k in relu:
        assert (relu[k] == zero[k]).all(), k


def test_residual_epilogue_oracle_against_numpy():
    """y = act(bn(x) + residual); dresidual = dy*mask; everything else as in the plain layer with dz."""
    d = make_inputs((6, 5, 4, 3), seed=13, loc=0.3, scale=1.5)
    res = np.random.default_rng(14).standard_normal(d["x"].shape).astype(np.float32)
    for slope in (0.0, 0.2):
        got = o.bn_add_act_fwd_bwd_f64(d["x"], res, d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"],
                                       neg_slope=slope)
        c = d["x"].shape[1]
        bs = (1, c, 1, 1)
        x64 = d["x"].astype(np.float64)
        mean = x64.mean(axis=(0, 2, 3)); var = x64.var(axis=(0, 2, 3)) + 1e-5
        xhat = (x64 - mean.reshape(bs)) / np.sqrt(var).reshape(bs)
        pre = xhat * d["gamma"].astype(np.float64).reshape(bs) + d["beta"].astype(np.float64).reshape(bs) + res
        mask = np.where(pre > 0, 1.0, slope)
        dz = d["dy"].astype(np.float64) * mask
        assert np.allclose(got["y"], pre * mask, rtol=1e-9, atol=1e-11)
        assert np.allclose(got["dresidual"], dz, rtol=1e-12, atol=0)
        assert np.allclose(got["dbeta"], dz.sum(axis=(0, 2, 3)), rtol=1e-9, atol=1e-10)
        assert np.allclose(got["dgamma"], (dz * xhat).sum(axis=(0, 2, 3)), rtol=1e-9, atol=1e-9)
        M = x64.size / c
        dzg = dz * d["gamma"].astype(np.float64).reshape(bs)
        r = (1.0 / np.sqrt(var)).reshape(bs)
        dx = r * (dzg - dzg.sum(axis=(0, 2, 3)).reshape(bs) / M - xhat * (dzg * xhat).sum(axis=(0, 2, 3)).reshape(bs) / M)
        assert np.allclose(got["dx"], dx, rtol=1e-8, atol=1e-10)
