"""The forward entry point that brings its own scratch (a fixed array inside the library, for
callers that cannot allocate: anode's fixed op argument list has no workspace slot, and code
inside a memory-pool transaction must not call cudaMalloc).  It is called twice in a row
through the C ABI and each result is compared with the workspace-taking entry point on the
same inputs.  The second call finds whatever the first one left in the shared array."""
import ctypes

import numpy as np
import pytest
import torch

from tests.util import assert_close, make_inputs

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
        out[which] = {k: v.cpu().numpy() for k, v in dict(y=y, mean=mean, var=var, run_mean=rm, run_var=rv).items()}
    return out


def test_static_scratch_forward_matches_workspace_forward_twice():
    from anode_b200 import _lib, ops
    lib = _lib.load()
    # two different problems back to back: the second finds the first one's leftovers in the array
    for shape, seed in (((16, 8, 28, 28), 51), ((32, 64, 7, 7), 52), ((16, 8, 28, 28), 53)):
        d = make_inputs(shape, seed=seed, loc=0.5, scale=2.0)
        for _ in range(2):
            out = run_both(lib, ops, d, 1e-5, 0.1)
            for k in ("mean", "var", "run_mean", "run_var", "y"):
                assert_close(out["static"][k], out["workspace"][k], "%r %s" % (shape, k))   # 1e-4 rel / 1e-5 abs


def test_static_scratch_rejects_problems_beyond_its_size():
    from anode_b200 import _lib
    lib = _lib.load()
    # 2^31 elements in rows of four floats need far more per-tile scratch than the built-in 4 MiB
    d0, c, n = 4, 1 << 19, 1 << 10
    assert lib.anode_gpu_batch_norm_fused_workspace_bytes(d0, c, n) > (4 << 20)
    x = torch.zeros(16, device="cuda")       # never touched: the call must be refused before any launch
    v = torch.zeros(1 << 19, device="cuda")
    rc = lib.anode_gpu_batch_norm_relu_fused_fwd_static_3d1_packed_f32(
        d0, c, n, 1e-5, 0.1, 1, p(x), None, None, p(x), p(v), p(v), None, None, None, None)
    assert rc == -7
    torch.cuda.synchronize()
