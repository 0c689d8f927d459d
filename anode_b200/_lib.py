"""ctypes binding of libanode_routines_gpu.so (the C ABI declared in include/anode_routines_gpu.h).

There is no fallback of any kind: if the shared library is missing the import fails with
instructions to build it, and every call goes to the CUDA kernels.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# ANODE_B200_LIB selects another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("ANODE_B200_LIB") or os.path.join(HERE, "libanode_routines_gpu.so")

u32, f32, c_int = ctypes.c_uint32, ctypes.c_float, ctypes.c_int
vp, size_t = ctypes.c_void_p, ctypes.c_size_t


class KernelConfig(ctypes.Structure):
    """routines_gpu/common.cuh:51-67 / src/ffi.rs:28-33."""
    _fields_ = [("block_sz", u32), ("max_block_ct", u32)]


_D = [u32, u32, u32]          # dim0, dim1, dim2
_T = [vp, vp]                 # cfg, stream

# name -> (restype, argtypes); order matches include/anode_routines_gpu.h
SIGNATURES = {
    "anode_gpu_batch_mean_3d1_packed_f32": (None, _D + [vp, vp] + _T),
    "anode_gpu_batch_mean_bwd_3d1_packed_f32": (None, _D + [vp, vp] + _T),
    "anode_gpu_batch_mean_bwd_3d1_packed_accumulate_f32": (None, _D + [vp, vp] + _T),
    "anode_gpu_batch_var_3d1_packed_f32": (None, _D + [f32, vp, vp, vp] + _T),
    "anode_gpu_batch_var_bwd_3d1_packed_f32": (None, _D + [vp, vp, vp, vp] + _T),
    "anode_gpu_batch_var_bwd_3d1_packed_accumulate_f32": (None, _D + [vp, vp, vp, vp] + _T),
    "anode_gpu_batch_var_bwd_mean_3d1_packed_f32": (None, _D + [vp, vp, vp, vp] + _T),
    "anode_gpu_batch_var_bwd_mean_3d1_packed_accumulate_f32": (None, _D + [vp, vp, vp, vp] + _T),
    "anode_gpu_batch_norm_3d1_packed_f32": (None, _D + [vp, vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_3d1_packed_f32": (None, _D + [vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_3d1_packed_accumulate_f32": (None, _D + [vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_mean_3d1_packed_f32": (None, _D + [vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_mean_3d1_packed_accumulate_f32": (None, _D + [vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_var_3d1_packed_f32": (None, _D + [vp, vp, vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_var_3d1_packed_accumulate_f32": (None, _D + [vp, vp, vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_var_v2_3d1_packed_f32": (None, _D + [vp, vp, vp, vp] + _T),
    "anode_gpu_batch_norm_bwd_var_v2_3d1_packed_accumulate_f32": (None, _D + [vp, vp, vp, vp] + _T),
    "anode_gpu_M1_copy_map_M2_unit_step_map_R_product_reduce_flat_join_f32": (None, [u32, vp, vp, vp] + _T),
    "anode_gpu_positive_clip_flat_map_f32": (None, [u32, vp, vp] + _T),
    "anode_gpu_positive_clip_flat_map_bwd_f32": (None, [u32, vp, vp, vp] + _T),
    "anode_gpu_batch_norm_fused_workspace_bytes": (size_t, _D),
    "anode_gpu_batch_norm_fused_workspace_init": (c_int, [vp, size_t, vp]),
    "anode_gpu_batch_norm_fused_status": (c_int, [vp, vp, ctypes.POINTER(u32)]),
    "anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32":
        (c_int, _D + [f32, f32, c_int] + [vp] * 8 + [vp, size_t] + _T),
    "anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32":
        (c_int, _D + [c_int, c_int] + [vp] * 9 + [vp, size_t] + _T),
    "anode_gpu_batch_norm_act_fused_fwd_3d1_packed_f32":
        (c_int, _D + [f32, f32, f32] + [vp] * 8 + [vp, size_t] + _T),
    "anode_gpu_batch_norm_act_fused_bwd_3d1_packed_f32":
        (c_int, _D + [f32, c_int] + [vp] * 9 + [vp, size_t] + _T),
    "anode_gpu_batch_norm_add_act_fused_fwd_3d1_packed_f32":
        (c_int, _D + [f32, f32, f32] + [vp] * 9 + [vp, size_t] + _T),
    "anode_gpu_batch_norm_add_act_fused_bwd_3d1_packed_f32":
        (c_int, _D + [f32, c_int] + [vp] * 11 + [vp, size_t] + _T),
    "anode_gpu_batch_norm_relu_fused_fwd_static_3d1_packed_f32":
        (c_int, _D + [f32, f32, c_int] + [vp] * 8 + _T),
    "anode_gpu_batch_norm_fused_static_status": (c_int, [vp, ctypes.POINTER(u32)]),
    "anode_gpu_batch_norm_host_step_staging_bytes": (size_t, _D + [u32]),
    "anode_gpu_batch_norm_host_step_blocks": (u32, _D + [u32]),
    "anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32":
        (c_int, _D + [f32, f32, c_int] + [vp] * 12 + [vp, size_t, u32] + _T),
    "anode_gpu_batch_norm_act_infer_3d1_packed_f32": (c_int, _D + [f32] + [vp] * 6 + _T),
    "anode_gpu_online_average_f32": (c_int, [u32, f32, vp, vp] + _T),
    "anode_gpu_sync_unique_id_bytes": (size_t, []),
    "anode_gpu_sync_get_unique_id": (c_int, [vp]),
    "anode_gpu_sync_comm_create": (c_int, [vp, c_int, c_int, ctypes.POINTER(vp)]),
    "anode_gpu_sync_comm_destroy": (c_int, [vp]),
    "anode_gpu_sync_comm_create_exchange_only": (c_int, [c_int, c_int, ctypes.POINTER(vp)]),
    "anode_gpu_sync_allreduce_sum_f32": (c_int, [vp, vp, size_t, vp]),
    "anode_gpu_sync_exchange_bytes": (size_t, [u32, c_int]),
    "anode_gpu_sync_comm_attach_exchange": (c_int, [vp, ctypes.POINTER(vp), u32]),
    "anode_gpu_sync_batch_norm_workspace_bytes": (size_t, _D + [c_int]),
    "anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32":
        (c_int, _D + [f32, f32, c_int] + [vp] * 8 + [vp, vp, size_t] + _T),
    "anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32":
        (c_int, _D + [ctypes.c_uint64, c_int, c_int] + [vp] * 9 + [vp, vp, size_t] + _T),
    "anode_gpu_sync_batch_norm_add_act_fwd_3d1_packed_f32":
        (c_int, _D + [f32, f32, f32] + [vp] * 9 + [vp, vp, size_t] + _T),
    "anode_gpu_sync_batch_norm_add_act_bwd_3d1_packed_f32":
        (c_int, _D + [ctypes.c_uint64, f32, c_int] + [vp] * 11 + [vp, vp, size_t] + _T),
    "anode_gpu_sync_batch_norm_host_step_staging_bytes": (size_t, _D + [ctypes.c_uint64, vp, u32]),
    "anode_gpu_sync_batch_norm_host_step_blocks": (u32, _D + [ctypes.c_uint64, vp, u32]),
    "anode_gpu_sync_batch_norm_relu_step_host_3d1_packed_f32":
        (c_int, _D + [ctypes.c_uint64, f32, f32, c_int] + [vp] * 12 + [vp, vp, size_t, u32] + _T),
    "anode_gpu_batch_norm_fused_plan": (c_int, _D + [c_int, u32, u32, u32, ctypes.POINTER(u32), u32]),
    "anode_gpu_batch_norm_fused_plan_walk":
        (c_int, _D + [c_int, u32, u32, u32, u32, u32, ctypes.POINTER(ctypes.c_uint64)]),
    "anode_gpu_batch_norm_segres_geometry": (c_int, _D + [c_int, ctypes.POINTER(u32)]),
    "anode_gpu_batch_norm_tiled_geometry": (c_int, _D + [c_int, ctypes.POINTER(u32)]),
    "anode_gpu_batch_norm_fused_kernel_kind": (c_int, _D + [c_int]),
    "anode_gpu_batch_norm_add_act_fused_kernel_kind": (c_int, _D + [c_int]),
    "anode_gpu_batch_norm_fused_set_wait_limit_ms": (c_int, [u32]),
    "anode_gpu_batch_norm_fused_set_kernel": (c_int, [c_int]),
    "anode_gpu_batch_norm_resident_plan": (c_int, _D + [u32, ctypes.POINTER(u32)]),
    "anode_gpu_batch_norm_resident_schedule":
        (ctypes.c_longlong, _D + [u32, u32, ctypes.POINTER(u32), ctypes.c_uint64]),
    "anode_gpu_batch_norm_fused_plan_tile":
        (c_int, _D + [c_int, u32, u32, u32, ctypes.POINTER(ctypes.c_uint64)]),
}

_lib = None


def load():
    """Loads the library (once) and attaches the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libanode_routines_gpu.so is not built: run `python -m anode_b200.build` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if a declared symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


ERRORS = {
    -1: "ANODE_E_NULL: a required pointer is NULL",
    -2: "ANODE_E_DIMS: a dimension is 0 or the tensor has 2^32 or more elements",
    -3: "ANODE_E_WORKSPACE: workspace missing, misaligned or too small",
    -4: "ANODE_E_LAUNCH: the CUDA runtime refused the launch",
    -5: "ANODE_E_COMM: communicator missing, inconsistent, or NCCL failure",
    -6: "ANODE_E_ALIGN: tensor pointers must be 4-byte aligned",
    -7: "ANODE_E_TOO_LARGE: the problem needs more scratch than the library's built-in array holds",
}


class AnodeError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        super().__init__("%s failed: %s" % (where, ERRORS.get(code, "error %d" % code)))


def check(code, where):
    if code != 0:
        raise AnodeError(code, where)
