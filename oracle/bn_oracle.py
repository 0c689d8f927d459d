"""Python face of the CPU oracle (test infrastructure, never imported by the library).

`liboracle_bn.so` (built from bn_oracle.c by oracle/Makefile) is loaded with ctypes and
wrapped so that tests can hand it numpy arrays.  Arrays are NCHW / NCDHW, f32, contiguous:
a tensor of shape [N, C, *spatial] is the reference's packed [dim0, dim1, dim2] array with
dim0 = prod(spatial), dim1 = C, dim2 = N (routines_gpu/common.cuh:88-94).

Also holds `numpy_truth`, an independent vectorised float64 restatement of the same layer
used to cross-check the C code.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle_bn.so")
_lib = None

_u32, _f32, _f64, _int = ctypes.c_uint32, ctypes.c_float, ctypes.c_double, ctypes.c_int
_pf = ctypes.POINTER(ctypes.c_float)
_pd = ctypes.POINTER(ctypes.c_double)


def build():
    """Compile the C restatement (gcc only; no GPU needed)."""
    subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        L.oracle_num_threads.restype = _int
        sig = {
            "oracle_batch_mean_f32": [_u32, _u32, _u32, _pf, _pf, _u32],
            "oracle_batch_var_f32": [_u32, _u32, _u32, _f32, _pf, _pf, _pf, _u32],
            "oracle_batch_var_bwd_mean_f32": [_u32, _u32, _u32, _pf, _pf, _pf, _pf, _int, _u32],
            "oracle_batch_norm_bwd_mean_f32": [_u32, _u32, _u32, _pf, _pf, _pf, _int, _u32],
            "oracle_batch_norm_bwd_var_f32": [_u32, _u32, _u32, _pf, _pf, _pf, _pf, _pf, _int, _u32],
            "oracle_batch_norm_bwd_var_v2_f32": [_u32, _u32, _u32, _pf, _pf, _pf, _pf, _int, _u32],
            "oracle_batch_norm_f32": [_u32, _u32, _u32, _pf, _pf, _pf, _pf],
            "oracle_batch_norm_bwd_f32": [_u32, _u32, _u32, _pf, _pf, _pf, _int],
            "oracle_batch_var_bwd_f32": [_u32, _u32, _u32, _pf, _pf, _pf, _pf, _int],
            "oracle_batch_mean_bwd_f32": [_u32, _u32, _u32, _pf, _pf, _int],
            "oracle_positive_clip_f32": [ctypes.c_size_t, _pf, _pf],
            "oracle_positive_clip_bwd_f32": [ctypes.c_size_t, _pf, _pf, _pf],
            "oracle_online_average_f32": [_u32, _f32, _pf, _pf],
            "oracle_bn_relu_fwd_bwd_f32": [_u32, _u32, _u32, _f32, _f32] + [_pf] * 14 + [_u32],
            "oracle_bn_relu_fwd_bwd_f64": [_u32, _u32, _u32, _f64, _f64, _pf, _pf, _pf, _pf] + [_pd] * 8,
            "oracle_bn_act_fwd_bwd_f64": [_u32, _u32, _u32, _f64, _f64, _f64, _pf, _pf, _pf, _pf] + [_pd] * 8,
            "oracle_bn_add_act_fwd_bwd_f64": [_u32, _u32, _u32, _f64, _f64, _f64, _pf, _pf, _pf, _pf, _pf] + [_pd] * 9,
            "oracle_leaky_relu_f32": [ctypes.c_size_t, _f32, _pf, _pf],
            "oracle_leaky_relu_bwd_f32": [ctypes.c_size_t, _f32, _pf, _pf, _pf],
        }
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = None
        _lib = L
    return _lib


def dims_of(shape):
    """[N, C, *spatial] -> (dim0, dim1, dim2) = (prod(spatial), C, N)."""
    n, c = int(shape[0]), int(shape[1])
    d0 = 1
    for s in shape[2:]:
        d0 *= int(s)
    return d0, c, n


def _p(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_pf)


def _pd_(a):
    if a is None:
        return None
    assert a.dtype == np.float64 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_pd)


def num_threads():
    return int(lib().oracle_num_threads())


def f32c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


# ---- single kernels (f32 literal) -------------------------------------------------

def batch_mean(x, block_sz=1024):
    d0, c, n = dims_of(x.shape)
    mean = np.zeros(c, np.float32)
    lib().oracle_batch_mean_f32(d0, c, n, _p(x), _p(mean), block_sz)
    return mean


def batch_var(x, mean, eps, block_sz=1024):
    d0, c, n = dims_of(x.shape)
    var = np.zeros(c, np.float32)
    lib().oracle_batch_var_f32(d0, c, n, eps, _p(x), _p(mean), _p(var), block_sz)
    return var


def batch_norm(x, mean, var):
    d0, c, n = dims_of(x.shape)
    y = np.empty_like(x)
    lib().oracle_batch_norm_f32(d0, c, n, _p(x), _p(mean), _p(var), _p(y))
    return y


def batch_norm_bwd(dy, var, dx=None):
    d0, c, n = dims_of(dy.shape)
    acc = dx is not None
    out = dx.copy() if acc else np.empty_like(dy)
    lib().oracle_batch_norm_bwd_f32(d0, c, n, _p(dy), _p(var), _p(out), int(acc))
    return out


def batch_var_bwd(dvar, x, mean, dx=None):
    d0, c, n = dims_of(x.shape)
    acc = dx is not None
    out = dx.copy() if acc else np.empty_like(x)
    lib().oracle_batch_var_bwd_f32(d0, c, n, _p(dvar), _p(x), _p(mean), _p(out), int(acc))
    return out


def batch_mean_bwd(dmean, shape, dx=None):
    d0, c, n = dims_of(shape)
    acc = dx is not None
    out = dx.copy() if acc else np.empty(shape, np.float32)
    lib().oracle_batch_mean_bwd_f32(d0, c, n, _p(dmean), _p(out), int(acc))
    return out


def batch_var_bwd_mean(dvar, x, mean, dmean=None, block_sz=1024):
    d0, c, n = dims_of(x.shape)
    acc = dmean is not None
    out = dmean.copy() if acc else np.zeros(c, np.float32)
    lib().oracle_batch_var_bwd_mean_f32(d0, c, n, _p(dvar), _p(x), _p(mean), _p(out), int(acc), block_sz)
    return out


def batch_norm_bwd_mean(dy, var, dmean=None, block_sz=1024):
    d0, c, n = dims_of(dy.shape)
    acc = dmean is not None
    out = dmean.copy() if acc else np.zeros(c, np.float32)
    lib().oracle_batch_norm_bwd_mean_f32(d0, c, n, _p(dy), _p(var), _p(out), int(acc), block_sz)
    return out


def batch_norm_bwd_var(dy, x, mean, var, dvar=None, block_sz=1024):
    d0, c, n = dims_of(x.shape)
    acc = dvar is not None
    out = dvar.copy() if acc else np.zeros(c, np.float32)
    lib().oracle_batch_norm_bwd_var_f32(d0, c, n, _p(dy), _p(x), _p(mean), _p(var), _p(out), int(acc), block_sz)
    return out


def batch_norm_bwd_var_v2(dy, y, var, dvar=None, block_sz=1024):
    d0, c, n = dims_of(y.shape)
    acc = dvar is not None
    out = dvar.copy() if acc else np.zeros(c, np.float32)
    lib().oracle_batch_norm_bwd_var_v2_f32(d0, c, n, _p(dy), _p(y), _p(var), _p(out), int(acc), block_sz)
    return out


def positive_clip(x):
    y = np.empty_like(x)
    lib().oracle_positive_clip_f32(x.size, _p(x), _p(y))
    return y


def positive_clip_bwd(dy, y):
    dx = np.empty_like(dy)
    lib().oracle_positive_clip_bwd_f32(dy.size, _p(dy), _p(y), _p(dx))
    return dx


def leaky_relu(c, x):
    """routines_gpu/flat_map.cu:44-52."""
    y = np.empty_like(x)
    lib().oracle_leaky_relu_f32(x.size, c, _p(x), _p(y))
    return y


def leaky_relu_bwd(c, dy, y):
    """routines_gpu/flat_map.cu:61-69."""
    dx = np.empty_like(dy)
    lib().oracle_leaky_relu_bwd_f32(dy.size, c, _p(dy), _p(y), _p(dx))
    return dx


def online_average(rate, x, y):
    out = y.copy()
    lib().oracle_online_average_f32(x.size, rate, _p(x), _p(out))
    return out


# ---- whole layer ------------------------------------------------------------------

def bn_relu_fwd_bwd_f32(x, dy, eps, avg_rate, run_mean, run_var, gamma=None, beta=None, block_sz=1024):
    """f32 literal layer.  Returns dict(y, dx, mean, var, run_mean, run_var, dgamma, dbeta)."""
    d0, c, n = dims_of(x.shape)
    rm, rv = run_mean.astype(np.float32).copy(), run_var.astype(np.float32).copy()
    y, dx = np.empty_like(x), np.empty_like(x)
    mean, var = np.zeros(c, np.float32), np.zeros(c, np.float32)
    dg = np.zeros(c, np.float32) if gamma is not None else None
    db = np.zeros(c, np.float32) if gamma is not None else None
    xhat, dz = np.empty_like(x), np.empty_like(x)
    lib().oracle_bn_relu_fwd_bwd_f32(d0, c, n, eps, avg_rate, _p(x), _p(dy), _p(gamma), _p(beta),
                                     _p(rm), _p(rv), _p(y), _p(dx), _p(mean), _p(var), _p(dg), _p(db),
                                     _p(xhat), _p(dz), block_sz)
    return dict(y=y, dx=dx, mean=mean, var=var, run_mean=rm, run_var=rv, dgamma=dg, dbeta=db)


def bn_relu_fwd_bwd_f64(x, dy, eps, avg_rate, run_mean, run_var, gamma=None, beta=None):
    """float64 truth of the same layer (C implementation)."""
    d0, c, n = dims_of(x.shape)
    rm, rv = run_mean.astype(np.float64).copy(), run_var.astype(np.float64).copy()
    y, dx = np.empty(x.shape, np.float64), np.empty(x.shape, np.float64)
    mean, var = np.zeros(c), np.zeros(c)
    dg, db = np.zeros(c), np.zeros(c)
    lib().oracle_bn_relu_fwd_bwd_f64(d0, c, n, eps, avg_rate, _p(x), _p(dy), _p(gamma), _p(beta),
                                     _pd_(rm), _pd_(rv), _pd_(y), _pd_(dx), _pd_(mean), _pd_(var),
                                     _pd_(dg), _pd_(db))
    return dict(y=y, dx=dx, mean=mean, var=var, run_mean=rm, run_var=rv, dgamma=dg, dbeta=db)


def bn_act_fwd_bwd_f64(x, dy, eps, avg_rate, run_mean, run_var, gamma=None, beta=None, neg_slope=0.0):
    """float64 truth with the activation t*(t > 0 ? 1 : neg_slope) (0: ReLU, c: leaky ReLU, 1: none)."""
    d0, c, n = dims_of(x.shape)
    rm, rv = run_mean.astype(np.float64).copy(), run_var.astype(np.float64).copy()
    y, dx = np.empty(x.shape, np.float64), np.empty(x.shape, np.float64)
    mean, var = np.zeros(c), np.zeros(c)
    dg, db = np.zeros(c), np.zeros(c)
    lib().oracle_bn_act_fwd_bwd_f64(d0, c, n, eps, avg_rate, neg_slope, _p(x), _p(dy), _p(gamma), _p(beta),
                                    _pd_(rm), _pd_(rv), _pd_(y), _pd_(dx), _pd_(mean), _pd_(var),
                                    _pd_(dg), _pd_(db))
    return dict(y=y, dx=dx, mean=mean, var=var, run_mean=rm, run_var=rv, dgamma=dg, dbeta=db)


def bn_add_act_fwd_bwd_f64(x, residual, dy, eps, avg_rate, run_mean, run_var, gamma=None, beta=None, neg_slope=0.0):
    """float64 truth of the residual-block epilogue y = act(bn(x) + residual); also returns dresidual."""
    d0, c, n = dims_of(x.shape)
    rm, rv = run_mean.astype(np.float64).copy(), run_var.astype(np.float64).copy()
    y, dx, dres = (np.empty(x.shape, np.float64) for _ in range(3))
    mean, var = np.zeros(c), np.zeros(c)
    dg, db = np.zeros(c), np.zeros(c)
    lib().oracle_bn_add_act_fwd_bwd_f64(d0, c, n, eps, avg_rate, neg_slope, _p(x), _p(residual), _p(dy), _p(gamma), _p(beta),
                                        _pd_(rm), _pd_(rv), _pd_(y), _pd_(dx), _pd_(dres), _pd_(mean), _pd_(var),
                                        _pd_(dg), _pd_(db))
    return dict(y=y, dx=dx, dresidual=dres, mean=mean, var=var, run_mean=rm, run_var=rv, dgamma=dg, dbeta=db)


def numpy_truth(x, dy, eps, avg_rate, run_mean, run_var, gamma=None, beta=None, neg_slope=0.0):
    """Vectorised float64 restatement, written independently of the C code.

    mean/var: routines_gpu/batch_norm.cu:54,160 (biased, eps folded into var);
    normalize: :333; ReLU and its mask: routines_gpu/flat_map.cu:176-177,191-192;
    dvar/dmean/dx: batch_norm.cu:494-500, 423-429, 259-277, 373, 203, 92.
    """
    x64, dy64 = x.astype(np.float64), dy.astype(np.float64)
    c = x.shape[1]
    ax = (0,) + tuple(range(2, x.ndim))
    bshape = (1, c) + (1,) * (x.ndim - 2)
    M = x64.size / c
    mean = x64.mean(axis=ax)
    xm = x64 - mean.reshape(bshape)
    var = (xm * xm).sum(axis=ax) / M + eps
    r = 1.0 / np.sqrt(var)
    xhat = xm * r.reshape(bshape)
    g = np.ones(c) if gamma is None else gamma.astype(np.float64)
    b = np.zeros(c) if (gamma is None or beta is None) else beta.astype(np.float64)
    ybn = xhat * g.reshape(bshape) + b.reshape(bshape)
    y = np.where(ybn > 0, ybn, neg_slope * ybn)
    dz = np.where(ybn > 0, dy64, neg_slope * dy64)
    dbeta = dz.sum(axis=ax)
    dgamma = (dz * xhat).sum(axis=ax)
    dzg = dz * g.reshape(bshape)
    dvar = (dzg * xm).sum(axis=ax) * (-0.5 * r / var)
    dmean = -r * dzg.sum(axis=ax) + xm.sum(axis=ax) * (-2.0 * dvar) / M
    dx = dzg * r.reshape(bshape) + dvar.reshape(bshape) * xm * 2.0 / M + dmean.reshape(bshape) / M
    rm = run_mean.astype(np.float64)
    rv = run_var.astype(np.float64)
    return dict(y=y, dx=dx, mean=mean, var=var, run_mean=rm + avg_rate * (mean - rm),
                run_var=rv + avg_rate * (var - rv), dgamma=dgamma, dbeta=dbeta)
