"""The reference's own CUDA kernels as a GPU oracle (test infrastructure only).

oracle/_ref/libanode_routines_gpu_ref.so is built by oracle/Makefile from the reference's
unmodified routines_gpu/{batch_norm,flat_map,flat_join}.cu.  This module runs the layer the
way anode's graph does (src/ops.rs:999-1014 forward; src/ops_gpu.rs:4344-4352, 3997-4003,
3787-3791 adjoints; ReLU src/ops_gpu.rs:8414-8582): eleven launches on torch CUDA tensors.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(_HERE, "_ref", "libanode_routines_gpu_ref.so")
_lib = None


class KernelConfig(ctypes.Structure):
    _fields_ = [("block_sz", ctypes.c_uint32), ("max_block_ct", ctypes.c_uint32)]


def available():
    return os.path.exists(REF_SO)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(REF_SO)   # RTLD_LOCAL: its symbols shadow nobody else's
    return _lib


def _call(name, *args):
    fn = getattr(lib(), name)
    fn.restype = None
    conv = []
    for a in args:
        if isinstance(a, torch.Tensor):
            conv.append(ctypes.c_void_p(a.data_ptr()))
        elif isinstance(a, float):
            conv.append(ctypes.c_float(a))
        elif isinstance(a, int):
            conv.append(ctypes.c_uint32(a))
        else:
            conv.append(a)
    fn(*conv)


def default_cfg():
    """block_sz = 1024 threads, max_block_ct = 32 blocks per SM (the values are the caller's
    in anode; only the summation order depends on them)."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    return KernelConfig(1024, 32 * sms)


def bn_relu_fwd_bwd(x, dy, eps, avg_rate, run_mean, run_var, cfg=None, timing=None):
    """Reference kernel sequence (no gamma/beta: the reference has none).  Returns a dict of
    torch tensors: y, dx, mean, var, run_mean, run_var.  With `timing` = (start, stop) CUDA
    events, they are recorded around the eleven launches (running-average update excluded,
    it lives in another crate)."""
    cfg = cfg or default_cfg()
    pc = ctypes.byref(cfg)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    d0 = 1
    for s in x.shape[2:]:
        d0 *= int(s)
    c, n = int(x.shape[1]), int(x.shape[0])
    dev = x.device
    mean = torch.zeros(c, device=dev); var = torch.zeros(c, device=dev)
    dvar = torch.zeros(c, device=dev); dmean = torch.zeros(c, device=dev)
    y = torch.empty_like(x); dz = torch.empty_like(x); dx = torch.empty_like(x)
    if timing:
        timing[0].record()
    _call("anode_gpu_batch_mean_3d1_packed_f32", d0, c, n, x, mean, pc, st)
    _call("anode_gpu_batch_var_3d1_packed_f32", d0, c, n, float(eps), x, mean, var, pc, st)
    _call("anode_gpu_batch_norm_3d1_packed_f32", d0, c, n, x, mean, var, y, pc, st)
    _call("anode_gpu_positive_clip_flat_map_f32", x.numel(), y, y, pc, st)
    _call("anode_gpu_positive_clip_flat_map_bwd_f32", x.numel(), dy, y, dz, pc, st)
    _call("anode_gpu_batch_norm_bwd_var_3d1_packed_f32", d0, c, n, dz, x, mean, var, dvar, pc, st)
    _call("anode_gpu_batch_norm_bwd_mean_3d1_packed_f32", d0, c, n, dz, var, dmean, pc, st)
    _call("anode_gpu_batch_var_bwd_mean_3d1_packed_accumulate_f32", d0, c, n, dvar, x, mean, dmean, pc, st)
    _call("anode_gpu_batch_norm_bwd_3d1_packed_f32", d0, c, n, dz, var, dx, pc, st)
    _call("anode_gpu_batch_var_bwd_3d1_packed_accumulate_f32", d0, c, n, dvar, x, mean, dx, pc, st)
    _call("anode_gpu_batch_mean_bwd_3d1_packed_accumulate_f32", d0, c, n, dmean, dx, pc, st)
    if timing:
        timing[1].record()
    rm = run_mean + avg_rate * (mean - run_mean)    # y <- y + r*(x - y), tests/test_gpu.rs:561-593
    rv = run_var + avg_rate * (var - run_var)
    return dict(y=y, dx=dx, mean=mean, var=var, run_mean=rm, run_var=rv, dmean=dmean, dvar=dvar)
