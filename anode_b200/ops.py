"""Host-side mirror of anode's batch-norm / ReLU operator surface, on top of the C ABI.

The reference builds a graph of ops whose `apply` closures each enqueue one kernel
(src/ops_gpu.rs:3690-5860 batch-norm, :7864-7940 and :8414-8755 ReLU); this module keeps the
op names, the argument meaning and the Assign/Accumulate write capability, but evaluates
eagerly on torch CUDA tensors (torch is used for device memory and streams only).

Arrays: a contiguous f32 tensor [N, C, *spatial] is the reference's
GPUDeviceOuterBatchArray3d/4d of size [W, H, (D,) C] + batch; per-channel vectors are
GPUDeviceArray1d of length C.  `axes` is [0, 1] for 2-D and [0, 1, 2] for 3-D data, the only
values the reference accepts (src/ops_gpu.rs:3736 `assert_eq!([0, 1], axes)`).
"""
import ctypes
import enum

import torch

from . import _lib
from ._lib import AnodeError, KernelConfig, check  # noqa: F401  (re-exported)


class WriteCap(enum.Enum):
    """src/lib.rs:1809-1820: first writer assigns, later writers accumulate."""
    Assign = 0
    Accumulate = 1


_DEFAULT_CFG = KernelConfig(1024, 148 * 32)


def _cfg(cfg):
    return ctypes.byref(cfg if cfg is not None else _DEFAULT_CFG)


def _stream(stream):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def _hp(t):
    """Pointer to a host tensor's data."""
    return ctypes.c_void_p(t.data_ptr())


def _p(t):
    if t is None:
        return None
    if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        # the reference only implements packed arrays too (src/ops_gpu.rs:3777-3779)
        raise ValueError("expected a contiguous float32 CUDA tensor")
    return ctypes.c_void_p(t.data_ptr())


def dims_of(x, axes=None):
    """[N, C, *spatial] -> (dim0, dim1, dim2) as the apply closures compute them
    (src/ops_gpu.rs:3764-3766 for 2-D, :4911-4913 for 3-D)."""
    if axes is not None:
        want = list(range(x.dim() - 2))
        if list(axes) != want:
            raise ValueError("axes must be %r for a %d-D batch array" % (want, x.dim() - 2))
    d0 = 1
    for s in x.shape[2:]:
        d0 *= int(s)
    return d0, int(x.shape[1]), int(x.shape[0])


def _call(name, *args):
    getattr(_lib.load(), name)(*args)


def _dims(x):
    d0, c, n = dims_of(x)
    return ctypes.c_uint32(d0), ctypes.c_uint32(c), ctypes.c_uint32(n)


# --------------------------------------------------------------------------------------------
# The reference's nine batch-norm ops (2-D and 3-D share the kernels; src/ops_gpu.rs:4858-5860).
# Each `apply` enqueues exactly one kernel, like the reference's closure of the same op.
# --------------------------------------------------------------------------------------------

class BatchMean2dOp:
    """src/ops_gpu.rs:3690-3800.  Accumulate is `unimplemented!()` there and rejected here."""
    @staticmethod
    def apply(axes, x, mean, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(x, axes)
        if cap is not WriteCap.Assign:
            raise NotImplementedError("BatchMean2dOp: Accumulate (unimplemented in the reference)")
        _call("anode_gpu_batch_mean_3d1_packed_f32", *_dims(x), _p(x), _p(mean), _cfg(cfg), _stream(stream))
        return mean


class BatchMean2dBwdOp:
    """src/ops_gpu.rs:3803-3911."""
    @staticmethod
    def apply(axes, dmean, x, dx, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(x, axes)
        name = "anode_gpu_batch_mean_bwd_3d1_packed_f32" if cap is WriteCap.Assign else \
            "anode_gpu_batch_mean_bwd_3d1_packed_accumulate_f32"
        _call(name, *_dims(x), _p(dmean), _p(dx), _cfg(cfg), _stream(stream))
        return dx


class BatchVariance2dOp:
    """src/ops_gpu.rs:3913-4010.  The stored variance includes epsilon."""
    @staticmethod
    def apply(axes, epsilon, x, mean, var, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(x, axes)
        if cap is not WriteCap.Assign:
            raise NotImplementedError("BatchVariance2dOp: Accumulate (unimplemented in the reference)")
        _call("anode_gpu_batch_var_3d1_packed_f32", *_dims(x), ctypes.c_float(epsilon), _p(x), _p(mean),
              _p(var), _cfg(cfg), _stream(stream))
        return var


class BatchVariance2dBwdOp:
    """src/ops_gpu.rs:4012-4130."""
    @staticmethod
    def apply(axes, dvar, x, mean, dx, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(x, axes)
        name = "anode_gpu_batch_var_bwd_3d1_packed_f32" if cap is WriteCap.Assign else \
            "anode_gpu_batch_var_bwd_3d1_packed_accumulate_f32"
        _call(name, *_dims(x), _p(dvar), _p(x), _p(mean), _p(dx), _cfg(cfg), _stream(stream))
        return dx


class BatchVariance2dBwdMeanOp:
    """src/ops_gpu.rs:4132-4247."""
    @staticmethod
    def apply(axes, dvar, x, mean, dmean, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(x, axes)
        name = "anode_gpu_batch_var_bwd_mean_3d1_packed_f32" if cap is WriteCap.Assign else \
            "anode_gpu_batch_var_bwd_mean_3d1_packed_accumulate_f32"
        _call(name, *_dims(x), _p(dvar), _p(x), _p(mean), _p(dmean), _cfg(cfg), _stream(stream))
        return dmean


class BatchNormalize2dOp:
    """src/ops_gpu.rs:4249-4362."""
    @staticmethod
    def apply(axes, x, mean, var, y, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(x, axes)
        if cap is not WriteCap.Assign:
            raise NotImplementedError("BatchNormalize2dOp: Accumulate (unimplemented in the reference)")
        _call("anode_gpu_batch_norm_3d1_packed_f32", *_dims(x), _p(x), _p(mean), _p(var), _p(y),
              _cfg(cfg), _stream(stream))
        return y


class BatchNormalize2dBwdOp:
    """src/ops_gpu.rs:4364-4474."""
    @staticmethod
    def apply(axes, dy, var, dx, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(dy, axes)
        name = "anode_gpu_batch_norm_bwd_3d1_packed_f32" if cap is WriteCap.Assign else \
            "anode_gpu_batch_norm_bwd_3d1_packed_accumulate_f32"
        _call(name, *_dims(dy), _p(dy), _p(var), _p(dx), _cfg(cfg), _stream(stream))
        return dx


class BatchNormalize2dBwdMeanOp:
    """src/ops_gpu.rs:4476-4584."""
    @staticmethod
    def apply(axes, dy, var, dmean, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(dy, axes)
        name = "anode_gpu_batch_norm_bwd_mean_3d1_packed_f32" if cap is WriteCap.Assign else \
            "anode_gpu_batch_norm_bwd_mean_3d1_packed_accumulate_f32"
        _call(name, *_dims(dy), _p(dy), _p(var), _p(dmean), _cfg(cfg), _stream(stream))
        return dmean


class BatchNormalize2dBwdVarianceOp:
    """src/ops_gpu.rs:4586-4736; `apply_v2` is build_device_f32_op_v2 (:4738), which reads the
    saved normalized output instead of x."""
    @staticmethod
    def apply(axes, dy, x, mean, var, dvar, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(x, axes)
        name = "anode_gpu_batch_norm_bwd_var_3d1_packed_f32" if cap is WriteCap.Assign else \
            "anode_gpu_batch_norm_bwd_var_3d1_packed_accumulate_f32"
        _call(name, *_dims(x), _p(dy), _p(x), _p(mean), _p(var), _p(dvar), _cfg(cfg), _stream(stream))
        return dvar

    @staticmethod
    def apply_v2(axes, dy, y, var, dvar, cap=WriteCap.Assign, cfg=None, stream=None):
        dims_of(y, axes)
        name = "anode_gpu_batch_norm_bwd_var_v2_3d1_packed_f32" if cap is WriteCap.Assign else \
            "anode_gpu_batch_norm_bwd_var_v2_3d1_packed_accumulate_f32"
        _call(name, *_dims(y), _p(dy), _p(y), _p(var), _p(dvar), _cfg(cfg), _stream(stream))
        return dvar


# The 3-D ops call the same entry points with dim0 = W*H*D (src/ops_gpu.rs:4911-4913).
BatchMean3dOp, BatchMean3dBwdOp = BatchMean2dOp, BatchMean2dBwdOp
BatchVariance3dOp, BatchVariance3dBwdOp, BatchVariance3dBwdMeanOp = \
    BatchVariance2dOp, BatchVariance2dBwdOp, BatchVariance2dBwdMeanOp
BatchNormalize3dOp, BatchNormalize3dBwdOp = BatchNormalize2dOp, BatchNormalize2dBwdOp
BatchNormalize3dBwdMeanOp, BatchNormalize3dBwdVarianceOp = BatchNormalize2dBwdMeanOp, BatchNormalize2dBwdVarianceOp


class OnlineAverageOp:
    """src/ops_gpu.rs:6034-6077: y <- y + rate*(x - y), in place on y."""
    @staticmethod
    def apply(avg_rate, x, y, cfg=None, stream=None):
        check(_lib.load().anode_gpu_online_average_f32(ctypes.c_uint32(x.numel()), ctypes.c_float(avg_rate),
                                                       _p(x), _p(y), _cfg(cfg), _stream(stream)),
              "anode_gpu_online_average_f32")
        return y


class PositiveClipOp:
    """ReLU, src/ops_gpu.rs:8414-8497 (PositiveClipFlatMap<f32>::apply, :7864-7880); `y is x`
    is the in-place form of PositiveClipClobberOp (:8584-8671)."""
    @staticmethod
    def apply(x, y, cfg=None, stream=None):
        _call("anode_gpu_positive_clip_flat_map_f32", ctypes.c_uint32(x.numel()), _p(x), _p(y),
              _cfg(cfg), _stream(stream))
        return y


class PositiveClipBwdOp:
    """src/ops_gpu.rs:8499-8582: dx = dy * (y > 0); `dx is dy` is the clobber form (:8673-8755)."""
    @staticmethod
    def apply(dy, y, dx, cfg=None, stream=None):
        _call("anode_gpu_positive_clip_flat_map_bwd_f32", ctypes.c_uint32(dy.numel()), _p(dy), _p(y), _p(dx),
              _cfg(cfg), _stream(stream))
        return dx


class FlatJoinOp:
    """src/ops_gpu.rs:8169-8261: y = x1 * step(x2) (routines_gpu/flat_join.cu:50-60)."""
    @staticmethod
    def apply(x1, x2, y, cfg=None, stream=None):
        _call("anode_gpu_M1_copy_map_M2_unit_step_map_R_product_reduce_flat_join_f32",
              ctypes.c_uint32(x1.numel()), _p(x1), _p(x2), _p(y), _cfg(cfg), _stream(stream))
        return y


# --------------------------------------------------------------------------------------------
# Front-end compositions (src/ops.rs:983-1056) and their adjoints, kernel by kernel.
# --------------------------------------------------------------------------------------------

def batch_normalize_2d(x, axes, online, avg_rate, epsilon, avg_mean=None, avg_var=None, cfg=None, stream=None):
    """`x.batch_normalize_2d(axes, online, avg_rate, epsilon)` of src/ops.rs:999-1014.

    Returns (y, mean, var, avg_mean, avg_var).  avg_mean / avg_var are the running averages
    (zeros when not given, as `zeros_like(...)` in the reference) and are updated in place.
    online=True normalizes with the batch statistics, online=False with the running ones
    (`switch(online, avg, batch)`, src/ops.rs:1671-1674).
    """
    c = x.shape[1]
    mean = torch.zeros(c, device=x.device, dtype=torch.float32)
    var = torch.zeros(c, device=x.device, dtype=torch.float32)
    if avg_mean is None:
        avg_mean = torch.zeros_like(mean)
    if avg_var is None:
        avg_var = torch.zeros_like(var)
    BatchMean2dOp.apply(axes, x, mean, cfg=cfg, stream=stream)
    BatchVariance2dOp.apply(axes, epsilon, x, mean, var, cfg=cfg, stream=stream)
    OnlineAverageOp.apply(avg_rate, mean, avg_mean, cfg=cfg, stream=stream)
    OnlineAverageOp.apply(avg_rate, var, avg_var, cfg=cfg, stream=stream)
    y = torch.empty_like(x)
    if online:
        BatchNormalize2dOp.apply(axes, x, mean, var, y, cfg=cfg, stream=stream)
    else:
        BatchNormalize2dOp.apply(axes, x, avg_mean, avg_var, y, cfg=cfg, stream=stream)
    return y, mean, var, avg_mean, avg_var


def batch_normalize_3d(x, axes, online, avg_rate, epsilon, avg_mean=None, avg_var=None, cfg=None, stream=None):
    """src/ops.rs:1043-1055; same kernels with dim0 = W*H*D."""
    return batch_normalize_2d(x, axes, online, avg_rate, epsilon, avg_mean, avg_var, cfg, stream)


def batch_normalize_adjoint(axes, dy_bn, x, mean, var, cfg=None, stream=None):
    """Adjoint of the training-mode composition with respect to x, as the reference's Sink
    evaluates it: BatchNormalize2dOp.adjoint emits (adj_x, adj_mean, adj_var)
    (src/ops_gpu.rs:4344-4352), BatchVariance2dOp.adjoint (adj_x, adj_mean) (:3997-4003),
    BatchMean2dOp.adjoint adj_x (:3787-3791); the first contribution to a variable is written
    with Assign and later ones with Accumulate (src/lib.rs:2160-2165).  Seven kernels."""
    c = x.shape[1]
    dvar = torch.zeros(c, device=x.device, dtype=torch.float32)
    dmean = torch.zeros(c, device=x.device, dtype=torch.float32)
    dx = torch.empty_like(x)
    kw = dict(cfg=cfg, stream=stream)
    BatchNormalize2dBwdVarianceOp.apply(axes, dy_bn, x, mean, var, dvar, WriteCap.Assign, **kw)
    BatchNormalize2dBwdMeanOp.apply(axes, dy_bn, var, dmean, WriteCap.Assign, **kw)
    BatchVariance2dBwdMeanOp.apply(axes, dvar, x, mean, dmean, WriteCap.Accumulate, **kw)
    BatchNormalize2dBwdOp.apply(axes, dy_bn, var, dx, WriteCap.Assign, **kw)
    BatchVariance2dBwdOp.apply(axes, dvar, x, mean, dx, WriteCap.Accumulate, **kw)
    BatchMean2dBwdOp.apply(axes, dmean, x, dx, WriteCap.Accumulate, **kw)
    return dx, dmean, dvar


def relu(x, inplace=False, cfg=None, stream=None):
    """`.positive_clip()` / `.relu()` and `.positive_clip_inplace()` (src/ops.rs:1199-1222)."""
    y = x if inplace else torch.empty_like(x)
    return PositiveClipOp.apply(x, y, cfg=cfg, stream=stream)


# --------------------------------------------------------------------------------------------
# Fused ops: BatchNormalize{2,3}dFusedOp / BatchNormalize{2,3}dBwdFusedOp, declared but never
# built by the reference (src/ops.rs:105-106).  One kernel per direction.
# --------------------------------------------------------------------------------------------

KERNELS = {"auto": 0, "tiled": 1, "cluster": 2, "resident": 3, "plain": 4}


def set_kernel(name):
    """Process-wide kernel preference of the fused calls (anode_gpu_batch_norm_fused_set_kernel):
    'auto', 'tiled', 'cluster', 'resident' or 'plain'.  For tests and measurements."""
    check(_lib.load().anode_gpu_batch_norm_fused_set_kernel(KERNELS[name]), "anode_gpu_batch_norm_fused_set_kernel")


def set_wait_limit_ms(ms):
    """Bound of the in-kernel waits (anode_gpu_batch_norm_fused_set_wait_limit_ms)."""
    check(_lib.load().anode_gpu_batch_norm_fused_set_wait_limit_ms(int(ms)), "anode_gpu_batch_norm_fused_set_wait_limit_ms")


class Workspace:
    """Caller-owned scratch of the fused kernels (the C ABI allocates nothing)."""

    def __init__(self, dim0, dim1, dim2, device):
        lib = _lib.load()
        self.bytes = int(lib.anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2))
        if self.bytes == 0:
            raise AnodeError(-2, "anode_gpu_batch_norm_fused_workspace_bytes")
        self.buf = torch.empty(self.bytes, dtype=torch.uint8, device=device)
        check(lib.anode_gpu_batch_norm_fused_workspace_init(
            ctypes.c_void_p(self.buf.data_ptr()), self.bytes, _stream(None)), "workspace_init")
        self.key = (dim0, dim1, dim2)

    @property
    def ptr(self):
        return ctypes.c_void_p(self.buf.data_ptr())

    def status(self, stream=None):
        st = ctypes.c_uint32(0)
        check(_lib.load().anode_gpu_batch_norm_fused_status(self.ptr, _stream(stream), ctypes.byref(st)),
              "anode_gpu_batch_norm_fused_status")
        return st.value

    def reset(self, stream=None):
        check(_lib.load().anode_gpu_batch_norm_fused_workspace_init(self.ptr, self.bytes, _stream(stream)),
              "workspace_init")


class BatchNormalize2dFusedOp:
    """Forward: statistics, running averages, normalize, affine, ReLU in one launch."""
    @staticmethod
    def apply(axes, epsilon, avg_rate, x, y, mean, var, avg_mean=None, avg_var=None, gamma=None, beta=None,
              relu=True, workspace=None, cfg=None, stream=None, neg_slope=None):
        d0, c, n = dims_of(x, axes)
        ws = workspace if workspace is not None else Workspace(d0, c, n, x.device)
        if neg_slope is not None:      # general activation t*(t > 0 ? 1 : neg_slope), e.g. leaky ReLU
            check(_lib.load().anode_gpu_batch_norm_act_fused_fwd_3d1_packed_f32(
                d0, c, n, ctypes.c_float(epsilon), ctypes.c_float(avg_rate), ctypes.c_float(neg_slope),
                _p(x), _p(gamma), _p(beta), _p(y), _p(mean), _p(var), _p(avg_mean), _p(avg_var),
                ws.ptr, ws.bytes, _cfg(cfg), _stream(stream)),
                "anode_gpu_batch_norm_act_fused_fwd_3d1_packed_f32")
            return y
        check(_lib.load().anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(
            d0, c, n, ctypes.c_float(epsilon), ctypes.c_float(avg_rate), int(bool(relu)),
            _p(x), _p(gamma), _p(beta), _p(y), _p(mean), _p(var), _p(avg_mean), _p(avg_var),
            ws.ptr, ws.bytes, _cfg(cfg), _stream(stream)),
            "anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32")
        return y


class BatchNormalize2dBwdFusedOp:
    """Backward: ReLU mask, both channel reductions, dgamma/dbeta and dx in one launch."""
    @staticmethod
    def apply(axes, dy, x, mean, var, dx, gamma=None, beta=None, dgamma=None, dbeta=None, relu=True,
              cap=WriteCap.Assign, workspace=None, cfg=None, stream=None, neg_slope=None):
        d0, c, n = dims_of(x, axes)
        ws = workspace if workspace is not None else Workspace(d0, c, n, x.device)
        if neg_slope is not None:
            check(_lib.load().anode_gpu_batch_norm_act_fused_bwd_3d1_packed_f32(
                d0, c, n, ctypes.c_float(neg_slope), int(cap is WriteCap.Accumulate),
                _p(dy), _p(x), _p(mean), _p(var), _p(gamma), _p(beta), _p(dx), _p(dgamma), _p(dbeta),
                ws.ptr, ws.bytes, _cfg(cfg), _stream(stream)),
                "anode_gpu_batch_norm_act_fused_bwd_3d1_packed_f32")
            return dx
        check(_lib.load().anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32(
            d0, c, n, int(bool(relu)), int(cap is WriteCap.Accumulate),
            _p(dy), _p(x), _p(mean), _p(var), _p(gamma), _p(beta), _p(dx), _p(dgamma), _p(dbeta),
            ws.ptr, ws.bytes, _cfg(cfg), _stream(stream)),
            "anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32")
        return dx


class BatchNormalize2dAddActFusedOp:
    """Residual-block epilogue y = act(bn(x) + residual) and its adjoint (mask from the saved y,
    dresidual = dy*mask), examples/run_imagenet_mpi.rs:191-195, 224-226."""
    @staticmethod
    def apply(axes, epsilon, avg_rate, x, residual, y, mean, var, avg_mean=None, avg_var=None, gamma=None, beta=None,
              neg_slope=0.0, workspace=None, cfg=None, stream=None):
        d0, c, n = dims_of(x, axes)
        ws = workspace if workspace is not None else Workspace(d0, c, n, x.device)
        check(_lib.load().anode_gpu_batch_norm_add_act_fused_fwd_3d1_packed_f32(
            d0, c, n, ctypes.c_float(epsilon), ctypes.c_float(avg_rate), ctypes.c_float(neg_slope),
            _p(x), _p(residual), _p(gamma), _p(beta), _p(y), _p(mean), _p(var), _p(avg_mean), _p(avg_var),
            ws.ptr, ws.bytes, _cfg(cfg), _stream(stream)), "anode_gpu_batch_norm_add_act_fused_fwd_3d1_packed_f32")
        return y

    @staticmethod
    def adjoint(axes, dy, x, y, mean, var, dx, dresidual=None, gamma=None, beta=None, dgamma=None, dbeta=None,
                neg_slope=0.0, cap=WriteCap.Assign, workspace=None, cfg=None, stream=None):
        d0, c, n = dims_of(x, axes)
        ws = workspace if workspace is not None else Workspace(d0, c, n, x.device)
        check(_lib.load().anode_gpu_batch_norm_add_act_fused_bwd_3d1_packed_f32(
            d0, c, n, ctypes.c_float(neg_slope), int(cap is WriteCap.Accumulate),
            _p(dy), _p(x), _p(y), _p(mean), _p(var), _p(gamma), _p(beta), _p(dx), _p(dresidual), _p(dgamma), _p(dbeta),
            ws.ptr, ws.bytes, _cfg(cfg), _stream(stream)), "anode_gpu_batch_norm_add_act_fused_bwd_3d1_packed_f32")
        return dx, dresidual


BatchNormalize3dFusedOp, BatchNormalize3dBwdFusedOp = BatchNormalize2dFusedOp, BatchNormalize2dBwdFusedOp


class BatchNormalize2dActInferOp:
    """Inference: batch-norm with given (running) statistics and the activation after it in one pass.
    neg_slope 0 = ReLU (positive_clip), 1 = none, c = leaky ReLU (flat_map.cu:44-52)."""
    @staticmethod
    def apply(axes, x, mean, var, y, gamma=None, beta=None, neg_slope=0.0, cfg=None, stream=None):
        d0, c, n = dims_of(x, axes)
        check(_lib.load().anode_gpu_batch_norm_act_infer_3d1_packed_f32(
            d0, c, n, ctypes.c_float(neg_slope), _p(x), _p(mean), _p(var), _p(gamma), _p(beta), _p(y),
            _cfg(cfg), _stream(stream)), "anode_gpu_batch_norm_act_infer_3d1_packed_f32")
        return y


BatchNormalize3dActInferOp = BatchNormalize2dActInferOp


class FusedBatchNormRelu:
    """A batch-norm + ReLU layer that keeps its own buffers (statistics, running averages,
    workspace), so that a training loop makes two calls per step: forward(x) and backward(dy)."""

    def __init__(self, channels, epsilon=1e-5, avg_rate=0.1, affine=True, relu=True, device="cuda"):
        dev = torch.device(device)
        self.epsilon, self.avg_rate, self.relu = float(epsilon), float(avg_rate), bool(relu)
        self.gamma = torch.ones(channels, device=dev) if affine else None
        self.beta = torch.zeros(channels, device=dev) if affine else None
        self.avg_mean = torch.zeros(channels, device=dev)
        self.avg_var = torch.ones(channels, device=dev)
        self.mean = torch.zeros(channels, device=dev)
        self.var = torch.zeros(channels, device=dev)
        self.dgamma = torch.zeros(channels, device=dev) if affine else None
        self.dbeta = torch.zeros(channels, device=dev) if affine else None
        self._ws = None
        self._staging = None
        self._dev = None
        self._x = None

    launches_per_step = 2      # one forward kernel, one backward kernel

    def _workspace(self, x):
        key = dims_of(x)
        if self._ws is None or self._ws.key != key:
            self._ws = Workspace(*key, x.device)
        return self._ws

    def status(self):
        """Device status word of the last launches (0 = clean); synchronises the stream."""
        return 0 if self._ws is None else self._ws.status()

    def step_from_host(self, hx, hdy, hy, hdx, chunk_channels=0):
        """One forward + backward with x, dy, y, dx in (page-locked) host memory.  The layer is
        processed in blocks of channels, so that copies to the device, both kernels and copies back
        overlap; everything is enqueued when the call returns and the current stream ends after
        the last copy.  Returns the number of channel blocks (each is two kernel launches)."""
        for t in (hx, hdy, hy, hdx):
            if t.is_cuda or not t.is_contiguous() or t.dtype != torch.float32:
                raise ValueError("step_from_host takes contiguous float32 host tensors")
        d0, c, n = dims_of(hx)
        lib = _lib.load()
        need = int(lib.anode_gpu_batch_norm_host_step_staging_bytes(d0, c, n, int(chunk_channels)))
        if need == 0:
            raise AnodeError(-2, "anode_gpu_batch_norm_host_step_staging_bytes")
        dev = self.mean.device
        if self._staging is None or self._staging.numel() < need:
            self._staging = None
            self._staging = torch.empty(need, dtype=torch.uint8, device=dev)
        check(lib.anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32(
            d0, c, n, ctypes.c_float(self.epsilon), ctypes.c_float(self.avg_rate), int(self.relu),
            _hp(hx), _hp(hdy), _p(self.gamma), _p(self.beta), _hp(hy), _hp(hdx),
            _p(self.mean), _p(self.var), _p(self.avg_mean), _p(self.avg_var), _p(self.dgamma), _p(self.dbeta),
            ctypes.c_void_p(self._staging.data_ptr()), need, int(chunk_channels), _cfg(None), _stream(None)),
            "anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32")
        return self.host_step_blocks(d0, c, n, chunk_channels)

    @staticmethod
    def host_step_blocks(d0, c, n, chunk_channels=0):
        """Channel blocks step_from_host cuts a [d0, c, n] layer into."""
        return int(_lib.load().anode_gpu_batch_norm_host_step_blocks(d0, c, n, int(chunk_channels)))

    def host_step_status(self):
        """Status word of the last step_from_host (0 = clean); synchronises the stream."""
        if self._staging is None:
            return 0
        out = ctypes.c_uint32(0)
        check(_lib.load().anode_gpu_batch_norm_fused_status(
            ctypes.c_void_p(self._staging.data_ptr()), _stream(None), ctypes.byref(out)), "status")
        return int(out.value)

    def infer(self, x, out=None):
        """Evaluation mode: normalize with the running averages, then the activation."""
        axes = list(range(x.dim() - 2))
        y = out if out is not None else torch.empty_like(x)
        return BatchNormalize2dActInferOp.apply(axes, x, self.avg_mean, self.avg_var, y, self.gamma, self.beta,
                                                0.0 if self.relu else 1.0)

    def forward(self, x, out=None):
        axes = list(range(x.dim() - 2))
        y = out if out is not None else torch.empty_like(x)
        BatchNormalize2dFusedOp.apply(axes, self.epsilon, self.avg_rate, x, y, self.mean, self.var,
                                      self.avg_mean, self.avg_var, self.gamma, self.beta, self.relu,
                                      self._workspace(x))
        self._x = x
        return y

    def backward(self, dy, out=None):
        x = self._x
        axes = list(range(x.dim() - 2))
        dx = out if out is not None else torch.empty_like(x)
        BatchNormalize2dBwdFusedOp.apply(axes, dy, x, self.mean, self.var, dx, self.gamma, self.beta,
                                         self.dgamma, self.dbeta, self.relu, WriteCap.Assign,
                                         self._workspace(x))
        return dx


class SyncWorkspace(Workspace):
    """Workspace of the synchronized entry points (single-GPU scratch + the gather buffer)."""

    def __init__(self, dim0, dim1, dim2, world, device):
        lib = _lib.load()
        self.bytes = int(lib.anode_gpu_sync_batch_norm_workspace_bytes(dim0, dim1, dim2, world))
        if self.bytes == 0:
            raise AnodeError(-2, "anode_gpu_sync_batch_norm_workspace_bytes")
        self.buf = torch.empty(self.bytes, dtype=torch.uint8, device=device)
        check(lib.anode_gpu_batch_norm_fused_workspace_init(
            ctypes.c_void_p(self.buf.data_ptr()), self.bytes, _stream(None)), "workspace_init")
        self.key = (dim0, dim1, dim2, world)


class SyncBatchNormRelu(FusedBatchNormRelu):
    """FusedBatchNormRelu over a batch sharded across the ranks of `comm` (anode_b200.sync.SyncComm):
    statistics, running averages, dgamma and dbeta are those of the global batch."""

    @property
    def launches_per_step(self):
        """Two kernels per step where a kernel with the exchange inside serves the shape; otherwise, per
        direction, reduce kernel, exchange (or merge) kernel and apply kernel."""
        if self.comm.world == 1:
            return 2
        if getattr(self.comm, "_exchange", None) is None:
            return 6
        if self._x is None:
            return 2
        d0, c, n = dims_of(self._x)
        kind = _lib.load().anode_gpu_batch_norm_fused_kernel_kind
        return sum(1 if kind(d0, c, n, d) != 4 else 3 for d in (0, 1))      # 4: the plain kernel (ANODE_KERNEL_PLAIN)

    def step_from_host(self, hx, hdy, hy, hdx, chunk_channels=0):
        """This rank's shard in (page-locked) host memory, through ONE C-ABI call: channel blocks copied in
        and out on the library's copy streams while the synchronized kernels of the block in between run.
        Returns the number of channel blocks (each is one synchronized forward and one backward)."""
        for t in (hx, hdy, hy, hdx):
            if t.is_cuda or not t.is_contiguous() or t.dtype != torch.float32:
                raise ValueError("step_from_host takes contiguous float32 host tensors")
        d0, c, n = dims_of(hx)
        lib = _lib.load()
        total = self.global_count if self.global_count is not None else d0 * n * self.comm.world
        need = int(lib.anode_gpu_sync_batch_norm_host_step_staging_bytes(d0, c, n, total, self.comm.handle, int(chunk_channels)))
        if need == 0:
            raise AnodeError(-2, "anode_gpu_sync_batch_norm_host_step_staging_bytes")
        if self._staging is None or self._staging.numel() < need:
            self._staging = None
            self._staging = torch.empty(need, dtype=torch.uint8, device=self.mean.device)
        check(lib.anode_gpu_sync_batch_norm_relu_step_host_3d1_packed_f32(
            d0, c, n, ctypes.c_uint64(total), ctypes.c_float(self.epsilon), ctypes.c_float(self.avg_rate), int(self.relu),
            _hp(hx), _hp(hdy), _p(self.gamma), _p(self.beta), _hp(hy), _hp(hdx),
            _p(self.mean), _p(self.var), _p(self.avg_mean), _p(self.avg_var), _p(self.dgamma), _p(self.dbeta),
            self.comm.handle, ctypes.c_void_p(self._staging.data_ptr()), need, int(chunk_channels), _cfg(None), _stream(None)),
            "anode_gpu_sync_batch_norm_relu_step_host_3d1_packed_f32")
        return int(lib.anode_gpu_sync_batch_norm_host_step_blocks(d0, c, n, total, self.comm.handle, int(chunk_channels)))

    def host_step_status(self):
        return FusedBatchNormRelu.host_step_status(self)

    def __init__(self, channels, comm=None, global_count=None, exchange=True, **kw):
        super().__init__(channels, **kw)
        if comm is None:
            from .sync import SyncComm
            from .sync import check_same_on_every_rank
            check_same_on_every_rank([channels], "channel count of the synchronized layer")
            comm = SyncComm.from_torch_distributed()
            if exchange and comm.world > 1:
                comm.attach_exchange(channels)       # one kernel per direction, exchange inside it
        self.comm = comm
        self.global_count = global_count      # elements per channel over all ranks; default: equal shards

    def _workspace(self, x):
        key = dims_of(x) + (self.comm.world,)
        if self._ws is None or self._ws.key != key:
            self._ws = SyncWorkspace(*key, x.device)
        return self._ws

    def forward(self, x, out=None):
        d0, c, n = dims_of(x)
        y = out if out is not None else torch.empty_like(x)
        ws = self._workspace(x)
        check(_lib.load().anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32(
            d0, c, n, ctypes.c_float(self.epsilon), ctypes.c_float(self.avg_rate), int(self.relu),
            _p(x), _p(self.gamma), _p(self.beta), _p(y), _p(self.mean), _p(self.var), _p(self.avg_mean),
            _p(self.avg_var), self.comm.handle, ws.ptr, ws.bytes, _cfg(None), _stream(None)),
            "anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32")
        self._x = x
        return y

    def forward_add(self, x, residual, out=None, neg_slope=0.0):
        """y = act(bn(x) + residual) with statistics over all ranks (the residual-block epilogue)."""
        d0, c, n = dims_of(x)
        y = out if out is not None else torch.empty_like(x)
        ws = self._workspace(x)
        check(_lib.load().anode_gpu_sync_batch_norm_add_act_fwd_3d1_packed_f32(
            d0, c, n, ctypes.c_float(self.epsilon), ctypes.c_float(self.avg_rate), ctypes.c_float(neg_slope),
            _p(x), _p(residual), _p(self.gamma), _p(self.beta), _p(y), _p(self.mean), _p(self.var), _p(self.avg_mean),
            _p(self.avg_var), self.comm.handle, ws.ptr, ws.bytes, _cfg(None), _stream(None)),
            "anode_gpu_sync_batch_norm_add_act_fwd_3d1_packed_f32")
        self._x, self._y = x, y
        return y

    def backward_add(self, dy, out=None, dresidual=None, neg_slope=0.0):
        """Adjoint of forward_add: returns (dx, dresidual); the mask comes from the saved output."""
        x, y = self._x, self._y
        d0, c, n = dims_of(x)
        dx = out if out is not None else torch.empty_like(x)
        ws = self._workspace(x)
        total = self.global_count if self.global_count is not None else d0 * n * self.comm.world
        check(_lib.load().anode_gpu_sync_batch_norm_add_act_bwd_3d1_packed_f32(
            d0, c, n, ctypes.c_uint64(total), ctypes.c_float(neg_slope), 0,
            _p(dy), _p(x), _p(y), _p(self.mean), _p(self.var), _p(self.gamma), _p(self.beta), _p(dx), _p(dresidual),
            _p(self.dgamma), _p(self.dbeta), self.comm.handle, ws.ptr, ws.bytes, _cfg(None), _stream(None)),
            "anode_gpu_sync_batch_norm_add_act_bwd_3d1_packed_f32")
        return dx, dresidual

    def backward(self, dy, out=None):
        x = self._x
        d0, c, n = dims_of(x)
        dx = out if out is not None else torch.empty_like(x)
        ws = self._workspace(x)
        total = self.global_count if self.global_count is not None else d0 * n * self.comm.world
        check(_lib.load().anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32(
            d0, c, n, ctypes.c_uint64(total), int(self.relu), 0,
            _p(dy), _p(x), _p(self.mean), _p(self.var), _p(self.gamma), _p(self.beta), _p(dx),
            _p(self.dgamma), _p(self.dbeta), self.comm.handle, ws.ptr, ws.bytes, _cfg(None), _stream(None)),
            "anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32")
        return dx
