"""Pins against the reference's own CUDA kernels (compiled unmodified into oracle/_ref):
 1. the literal CPU oracle reproduces them (bit for bit where the arithmetic is exactly
    rounded), which is what entitles the oracle to judge everything else;
 2. the fused kernels agree with them at the benchmark's full single-GPU size, compared on
    the device, plus a CPU-oracle check on a subset of channels (channels are independent)."""
import numpy as np
import pytest
import torch

from oracle import bn_oracle as o
from oracle import ref_gpu
from tests.util import assert_close, check_layer, make_inputs

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_gpu.available(), reason="oracle/_ref not built")]


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("shape,block", [((32, 64, 28, 28), 1024), ((5, 3, 7, 7), 256), ((2, 4, 3, 6, 8), 512),
                                         ((16, 8, 56, 56), 1024)])
def test_literal_oracle_reproduces_reference_kernels(shape, block):
    d = make_inputs(shape, seed=21, loc=0.5, scale=2.0, affine=False)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cfg = ref_gpu.KernelConfig(block, 32 * sms)
    r = ref_gpu.bn_relu_fwd_bwd(dev(d["x"]), dev(d["dy"]), 1e-5, 0.1, dev(d["run_mean"]), dev(d["run_var"]), cfg=cfg)
    torch.cuda.synchronize()
    r = {k: v.cpu().numpy() for k, v in r.items()}
    lit = o.bn_relu_fwd_bwd_f32(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], block_sz=block)
    assert (lit["mean"] == r["mean"]).all()      # same tree, exactly rounded adds and one divide
    assert (lit["var"] == r["var"]).all()
    assert_close(lit["y"], r["y"], "y", rtol=2e-6, atol=2e-6)       # rsqrtf is approximate on the device
    assert_close(lit["dx"], r["dx"], "dx", rtol=2e-5, atol=2e-6)


def _fused(ops, x, dy, rm, rv, gamma=None, beta=None):
    c = x.shape[1]
    axes = list(range(x.dim() - 2))
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    y = torch.empty_like(x); dx = torch.empty_like(x)
    ws = ops.Workspace(*ops.dims_of(x), x.device)
    ops.BatchNormalize2dFusedOp.apply(axes, 1e-5, 0.1, x, y, mean, var, rm, rv, gamma, beta, True, ws)
    ops.BatchNormalize2dBwdFusedOp.apply(axes, dy, x, mean, var, dx, gamma, beta, None, None, True,
                                         ops.WriteCap.Assign, ws)
    assert ws.status() == 0
    return dict(y=y, dx=dx, mean=mean, var=var, run_mean=rm, run_var=rv)


FULL = [  # the benchmark's shapes: whole (what one GPU runs alone) and as one GPU of eight sees them
    ("cfg3", (2048, 256, 56, 56), "normal", 0.0, 1.0),
    ("cfg5", (1024, 2048, 7, 7), "student3", 0.0, 4.0),
    ("cfg2", (256, 64, 112, 112), "normal", 0.5, 2.0),
    ("cfg3/8", (256, 256, 56, 56), "normal", 0.0, 1.0),
    ("cfg4/8", (4, 32, 16, 128, 128), "normal", 0.0, 1.0),
    ("cfg5/8", (128, 2048, 7, 7), "student3", 0.0, 4.0),
]


@pytest.mark.parametrize("name,shape,dist,loc,scale", FULL)
def test_fused_matches_reference_kernels_full_size(name, shape, dist, loc, scale):
    from anode_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(1234)
    if dist == "normal":
        x = torch.randn(shape, device="cuda", generator=g) * scale + loc
    else:
        # Student-t(3) = Z / sqrt(chi2_3 / 3)
        z = torch.randn(shape, device="cuda", generator=g)
        chi = sum(torch.randn(shape, device="cuda", generator=g) ** 2 for _ in range(3))
        x = (z / torch.sqrt(chi / 3.0)) * scale
        del z, chi
    dy = torch.randn(shape, device="cuda", generator=g)
    c = shape[1]
    rm = torch.zeros(c, device="cuda"); rv = torch.ones(c, device="cuda")
    ref = ref_gpu.bn_relu_fwd_bwd(x, dy, 1e-5, 0.1, rm.clone(), rv.clone())
    got = _fused(ops, x, dy, rm.clone(), rv.clone())
    torch.cuda.synchronize()
    for k in ("mean", "var", "run_mean", "run_var"):
        assert_close(got[k].cpu().numpy(), ref[k].cpu().numpy(), name + " " + k)
    # elementwise on the device: |a-b| <= 1e-5 + 1e-4|b|, skipping elements whose pre-activation
    # is within 1e-5 of zero (mask undecidable in f32)
    step = max(1, int(128e6 // (x.numel() // c)))          # channels per pass: bounds the temporaries
    nskip = 0
    for c0 in range(0, c, step):
        sl = slice(c0, c0 + step)
        cb = (1, -1) + (1,) * (len(shape) - 2)
        xhat = (x[:, sl] - ref["mean"][sl].view(cb)) * torch.rsqrt(ref["var"][sl].view(cb))
        skip = xhat.abs() < 1e-5
        nskip += int(skip.sum())
        for k in ("y", "dx"):
            diff = (got[k][:, sl] - ref[k][:, sl]).abs()
            bad = (diff > 1e-5 + 1e-4 * ref[k][:, sl].abs()) & ~skip
            assert int(bad.sum()) == 0, "%s %s: %d elements off, max diff %g" % (name, k, int(bad.sum()), float(diff.max()))
        del xhat, skip
    assert nskip < 1e-3 * x.numel()
    # CPU oracle (float64) on four channels
    idx = [0, 1, c // 2, c - 1]
    sub = dict(x=x[:, idx].contiguous().cpu().numpy(), dy=dy[:, idx].contiguous().cpu().numpy())
    truth = o.bn_relu_fwd_bwd_f64(sub["x"], sub["dy"], 1e-5, 0.1, np.zeros(4, np.float32), np.ones(4, np.float32))
    part = {k: got[k][:, idx].contiguous().cpu().numpy() for k in ("y", "dx")}
    part.update({k: got[k][idx].cpu().numpy() for k in ("mean", "var", "run_mean", "run_var")})
    check_layer(part, truth, sub["x"], None, None, name + " subset ")


def test_round_trip_properties_full_size():
    """Size-independent properties at the benchmark's full size: the normalized output has
    zero mean / unit variance per channel, and dx is orthogonal to 1 and to xhat per channel
    (the two directions batch-norm's Jacobian projects out)."""
    from anode_b200 import ops
    shape = (256, 64, 112, 112)
    g = torch.Generator(device="cuda"); g.manual_seed(99)
    x = torch.randn(shape, device="cuda", generator=g) * 2.0 + 0.5
    dy = torch.randn(shape, device="cuda", generator=g)
    c = shape[1]
    mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
    y = torch.empty_like(x); dx = torch.empty_like(x)
    ws = ops.Workspace(*ops.dims_of(x), x.device)
    ops.BatchNormalize2dFusedOp.apply([0, 1], 1e-5, 0.1, x, y, mean, var, None, None, None, None, False, ws)
    ops.BatchNormalize2dBwdFusedOp.apply([0, 1], dy, x, mean, var, dx, None, None, None, None, False,
                                         ops.WriteCap.Assign, ws)
    M = x.numel() // c
    ym = y.double().mean(dim=(0, 2, 3)); yv = (y.double() ** 2).mean(dim=(0, 2, 3))
    assert float(ym.abs().max()) < 1e-5
    assert float((yv - 1.0).abs().max()) < 1e-4
    s1 = dx.double().sum(dim=(0, 2, 3)); s2 = (dx.double() * y.double()).sum(dim=(0, 2, 3))
    scale = float(dx.abs().mean()) * M
    assert float(s1.abs().max()) < 1e-5 * scale and float(s2.abs().max()) < 1e-5 * scale
    assert ws.status() == 0
