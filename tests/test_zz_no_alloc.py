"""The forward entry point that brings its own scratch (a fixed array inside the library, for
callers that cannot allocate: anode's fixed op argument list has no workspace slot, and code
inside a memory-pool transaction must not call cudaMalloc).  It is called through the C ABI on
shapes served by kernels that really keep state in the array (the tiled and the plain kernel; the
cluster kernel needs none), back to back and alternating, so that every call finds the leftovers of
a different problem; each result is compared with the workspace-taking entry point on the same
inputs and with the float64 oracle."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import bn_oracle as o
from tests.util import assert_close, borderline, make_inputs

pytestmark = pytest.mark.gpu


def p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def run_both(lib, ops, d, eps, rate):
    x = torch.from_numpy(d["x"]).cuda()
    g, b = torch.from_numpy(d["gamma"]).cuda(), torch.from_numpy(d["beta"]).cuda()
    c = x.shape[1]
    d0, cc, n = ops.dims_of(x)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = {}
    for which in ("workspace", "static"):
        y = torch.full_like(x, float("nan"))
        mean = torch.zeros(c, device="cuda"); var = torch.zeros(c, device="cuda")
        rm = torch.zeros(c, device="cuda"); rv = torch.ones(c, device="cuda")
        if which == "workspace":
            ws = ops.Workspace(d0, cc, n, x.device)
            rc = lib.anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(
                d0, cc, n, eps, rate, 1, p(x), p(g), p(b), p(y), p(mean), p(var), p(rm), p(rv),
                ws.ptr, ws.bytes, None, stream)
        else:
            rc = lib.anode_gpu_batch_norm_relu_fused_fwd_static_3d1_packed_f32(
                d0, cc, n, eps, rate, 1, p(x), p(g), p(b), p(y), p(mean), p(var), p(rm), p(rv), None, stream)
        assert rc == 0, (which, rc)
        torch.cuda.synchronize()
        if which == "static":
            st = ctypes.c_uint32(99)
            assert lib.anode_gpu_batch_norm_fused_static_status(stream, ctypes.byref(st)) == 0 and st.value == 0
        out[which] = {k: v.cpu().numpy() for k, v in dict(y=y, mean=mean, var=var, run_mean=rm, run_var=rv).items()}
    return out


def test_static_scratch_forward_matches_workspace_forward_and_oracle():
    from anode_b200 import _lib, ops
    lib = _lib.load()
    kind = lib.anode_gpu_batch_norm_fused_kernel_kind
    # tiled kernel, plain kernel, cluster kernel, and two more tiled problems with other tile plans
    shapes = [(16, 8, 56, 56), (5, 3, 7, 7), (16, 8, 28, 28), (64, 8, 56, 56), (8, 6, 112, 112)]
    served = {kind(*ops.dims_of(torch.empty(s, device="meta")), 0) for s in shapes}
    assert {1, 2, 4} <= served, served          # ANODE_KERNEL_TILED, _CLUSTER, _PLAIN: two of them use the array
    data = {s: make_inputs(s, seed=51 + i, loc=0.5, scale=2.0) for i, s in enumerate(shapes)}
    truth = {s: o.bn_relu_fwd_bwd_f64(d["x"], d["dy"], 1e-5, 0.1, d["run_mean"], d["run_var"], d["gamma"], d["beta"])
             for s, d in data.items()}
    # each problem twice in a row, then all of them again: every call finds another plan's leftovers
    for shape in shapes + shapes[::-1]:
        d = data[shape]
        for _ in range(2):
            out = run_both(lib, ops, d, 1e-5, 0.1)
            skip = borderline(truth[shape], d["x"], d["gamma"], d["beta"])
            for k in ("mean", "var", "run_mean", "run_var", "y"):
                sk = skip if k == "y" else None
                assert_close(out["static"][k], out["workspace"][k], "%r %s vs workspace call" % (shape, k), skip=sk)   # 1e-4 rel / 1e-5 abs
                assert_close(out["static"][k], truth[shape][k], "%r %s vs oracle" % (shape, k), skip=sk)


def test_static_scratch_rejects_problems_beyond_its_size():
    from anode_b200 import _lib
    lib = _lib.load()
    # 4.2e9 elements in 256000 odd rows: the plain kernel serves it and keeps 32 bytes per tile in its
    # scratch, twice the built-in 4 MiB (checked on the host first: the call must be refused, not run)
    d0, c, n = 16385, 256, 1000
    assert lib.anode_gpu_batch_norm_fused_kernel_kind(d0, c, n, 0) == 4      # ANODE_KERNEL_PLAIN
    plan = (ctypes.c_uint32 * 15)()
    assert lib.anode_gpu_batch_norm_fused_plan(d0, c, n, 1, 0, 0, 0, plan, 15) == 0
    assert plan[13] + (plan[14] << 32) > (4 << 20)
    x = torch.zeros(16, device="cuda")       # never touched: the call is refused before any launch
    v = torch.zeros(c, device="cuda")
    rc = lib.anode_gpu_batch_norm_relu_fused_fwd_static_3d1_packed_f32(
        d0, c, n, 1e-5, 0.1, 1, p(x), None, None, p(x), p(v), p(v), None, None, None, None)
    assert rc == -7
    torch.cuda.synchronize()
