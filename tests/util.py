"""Shared helpers of the test-suite: seeded inputs of the benchmark configurations and the
tolerance rules.

Tolerance (the parity bar of this path): |got - want| <= 1e-5 + 1e-4*|want| on y, dx, mean,
var and the running statistics.  Two refinements, both stated where used:
  * elements whose pre-activation gamma*xhat+beta is within 1e-5 of zero are skipped in y/dx:
    there the ReLU mask legitimately depends on the last bit of the statistics;
  * per-channel sums (dgamma, dbeta) are compared with atol = 1e-5 + 1e-4*rms(want), since a
    sum of M terms that happens to cancel has no meaningful relative error.
"""
import numpy as np

RTOL, ATOL = 1e-4, 1e-5


def make_inputs(shape, seed, dist="normal", loc=0.0, scale=1.0, affine=True):
    """x, dy, gamma, beta, run_mean, run_var as the benchmark configurations define them:
    x ~ N(loc, scale) or scale*Student-t(3); dy ~ N(0,1); gamma ~ U(0.5,1.5); beta ~ U(-0.1,0.1);
    running mean 0, running variance 1."""
    rng = np.random.default_rng(seed)
    if dist == "normal":
        x = rng.standard_normal(shape, dtype=np.float32) * np.float32(scale) + np.float32(loc)
    elif dist == "student3":
        x = (rng.standard_t(3, size=shape) * scale).astype(np.float32)
    else:
        raise ValueError(dist)
    dy = rng.standard_normal(shape, dtype=np.float32)
    c = shape[1]
    gamma = rng.uniform(0.5, 1.5, c).astype(np.float32) if affine else None
    beta = rng.uniform(-0.1, 0.1, c).astype(np.float32) if affine else None
    return dict(x=x, dy=dy, gamma=gamma, beta=beta,
                run_mean=np.zeros(c, np.float32), run_var=np.ones(c, np.float32))


def close(got, want, rtol=RTOL, atol=ATOL):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return np.abs(got - want) <= atol + rtol * np.abs(want)


def assert_close(got, want, what, rtol=RTOL, atol=ATOL, skip=None):
    ok = close(got, want, rtol, atol)
    if skip is not None:
        ok = ok | skip
    if not ok.all():
        got = np.asarray(got, dtype=np.float64)
        want = np.asarray(want, dtype=np.float64)
        bad = np.argwhere(~ok)
        i = tuple(bad[0])
        raise AssertionError("%s: %d of %d elements off; first at %s: got %r want %r (max abs diff %g)" % (
            what, len(bad), ok.size, i, got[i], want[i], np.abs(got - want)[~ok].max()))


def assert_sum_close(got, want, what):
    want = np.asarray(want, dtype=np.float64)
    rms = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
    assert_close(got, want, what, rtol=RTOL, atol=ATOL + RTOL * rms)


def borderline(truth, x, gamma, beta, tol=1e-5):
    """Elements whose pre-activation is within tol of zero (mask undecidable in f32)."""
    c = x.shape[1]
    bs = (1, c) + (1,) * (x.ndim - 2)
    mean = np.asarray(truth["mean"], np.float64).reshape(bs)
    r = 1.0 / np.sqrt(np.asarray(truth["var"], np.float64)).reshape(bs)
    g = np.ones(c) if gamma is None else gamma.astype(np.float64)
    b = np.zeros(c) if (gamma is None or beta is None) else beta.astype(np.float64)
    ybn = (x.astype(np.float64) - mean) * r * g.reshape(bs) + b.reshape(bs)
    return np.abs(ybn) < tol


def check_layer(got, truth, x, gamma, beta, what="", atol_elem=ATOL, check_sums=True):
    """Compares one layer's outputs (dict of numpy arrays) with an oracle's.  `atol_elem`
    replaces the absolute tolerance on y and dx for deliberately ill-conditioned inputs, where
    `check_sums=False` also drops dgamma/dbeta (a single undecidable ReLU mask moves them by |dy|)."""
    skip = borderline(truth, x, gamma, beta, tol=atol_elem)
    assert x.size < 10000 or skip.mean() < 1e-3
    for k in ("mean", "var", "run_mean", "run_var"):
        if got.get(k) is not None and truth.get(k) is not None:
            assert_close(got[k], truth[k], what + k)
    assert_close(got["y"], truth["y"], what + "y", skip=skip, atol=atol_elem)
    assert_close(got["dx"], truth["dx"], what + "dx", skip=skip, atol=atol_elem)
    if gamma is not None and check_sums:
        assert_sum_close(got["dgamma"], truth["dgamma"], what + "dgamma")
        assert_sum_close(got["dbeta"], truth["dbeta"], what + "dbeta")


def check_layer_own_mask(d, got, what="", eps=1e-5, residual=None, slope=0.0):
    """Compares a fused layer's outputs with a float64 computation that takes the layer's OWN ReLU decisions
    (y > 0) wherever the pre-activation lies within 1e-5 of zero, and insists on the exact decision everywhere
    else.  Unlike check_layer it can therefore hold dgamma, dbeta and dx to the usual tolerance on any input:
    one undecidable mask moves the two sums by |dy| and, through them, every dx of the channel.
    `residual` is the shortcut tensor of the residual epilogue (y = act(bn(x) + residual); got["dresidual"] is
    checked when present), `slope` the activation's slope below zero (> 0 or exactly 0).
    Returns the number of decisions that differ from the float64 ones."""
    x = d["x"].astype(np.float64)
    dy = d["dy"].astype(np.float64)
    c = x.shape[1]
    ax = (0,) + tuple(range(2, x.ndim))
    bs = (1, c) + (1,) * (x.ndim - 2)
    m = x.size // c
    g = np.ones(c) if d["gamma"] is None else d["gamma"].astype(np.float64)
    b = np.zeros(c) if d["gamma"] is None else d["beta"].astype(np.float64)
    mean = x.mean(axis=ax)
    var = x.var(axis=ax) + eps
    r = 1.0 / np.sqrt(var)
    xhat = (x - mean.reshape(bs)) * r.reshape(bs)
    ybn = xhat * g.reshape(bs) + b.reshape(bs)
    if residual is not None:
        ybn = ybn + residual.astype(np.float64)
    mask = got["y"] > 0
    flips = mask != (ybn > 0)
    assert not (flips & (np.abs(ybn) >= 1e-5)).any(), what + "a ReLU decision differs away from zero"
    assert_close(got["mean"], mean, what + "mean")
    assert_close(got["var"], var, what + "var")
    act = np.where(mask, 1.0, slope)
    assert_close(got["y"], ybn * act, what + "y")
    dz = dy * act
    if got.get("dresidual") is not None:
        assert_close(got["dresidual"], dz, what + "dresidual")
    s1 = dz.sum(axis=ax)
    s2 = (dz * xhat).sum(axis=ax)
    dx = (g * r).reshape(bs) * (dz - s1.reshape(bs) / m - xhat * s2.reshape(bs) / m)
    # conditioning, not the kernel: the backward pass works from the f32 mean, which moves xhat by half an ulp of
    # |mean| over sigma; and dx is a sum of f32 terms of the size of gamma/sigma * |dz|
    cond = float(np.max(np.abs(mean) * r)) * 2e-7
    mag = float(np.max(np.abs(g * r))) * float(np.max(np.abs(dz))) * 1.2e-7
    assert_close(got["dx"], dx, what + "dx", atol=ATOL + cond + mag)
    if d["gamma"] is not None:
        rms1 = float(np.sqrt(np.mean(s1 * s1)))
        rms2 = float(np.sqrt(np.mean(s2 * s2)))
        assert_close(got["dbeta"], s1, what + "dbeta", atol=ATOL + RTOL * rms1)
        assert_close(got["dgamma"], s2, what + "dgamma", atol=ATOL + RTOL * rms2 + cond * float(np.abs(dz).sum(axis=ax).max()))
    return int(flips.sum())


def random_case(rng, max_elems=3e6):
    """A random problem shape (N, C, spatial...): tiny, ragged and long unaligned rows, the networks' feature maps,
    odd channel counts, one to a few hundred samples."""
    mode = int(rng.integers(0, 4))
    nd = int(rng.choice([1, 2, 2, 3]))
    if mode == 0:
        sp = [int(rng.integers(1, 9)) for _ in range(nd)]                  # tiny rows
    elif mode == 1:
        sp = [int(rng.integers(1, 40)) for _ in range(nd)]
    elif mode == 2:
        sp = [int(rng.choice([7, 14, 28, 56, 112, 8, 16, 32, 64]))] * 2      # the networks' feature maps
    else:
        sp = [int(rng.integers(1, 6)), int(rng.integers(50, 3000))]         # long, mostly unaligned rows
    dim0 = int(np.prod(sp))
    c = int(rng.choice([1, 2, 3, 4, 5, 8, 16, 31, 64, 96, 130, 260]))
    n = int(min(max(1, int(max_elems // (dim0 * c))), rng.choice([1, 2, 3, 5, 8, 16, 33, 64, 100, 257, 513])))
    while n * dim0 < 16:        # a handful of elements per channel is a conditioning exercise, not a kernel test
        n *= 2
    return (n, c) + tuple(sp)


def random_shapes(seed, count, max_elems=3e6):
    rng = np.random.default_rng(seed)
    return [random_case(rng, max_elems) for _ in range(count)]
