"""The C-ABI library loads and exports every symbol that include/anode_routines_gpu.h
declares; argument checks that need no GPU behave."""
import ctypes
import os
import re

from anode_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for header in ("anode_routines_gpu.h", "anode_routines_gpu_diag.h"):
        src = open(os.path.join(ROOT, "include", header)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names |= set(re.findall(r"\b(anode_gpu_\w+)\s*\(", src))
    return sorted(names)


def test_every_exported_symbol_is_declared_in_a_header():
    """Nothing is exported behind the headers' back (nm on the built library)."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line and line.split()[-1].startswith("anode_")}
    assert exported == set(declared_symbols()), sorted(exported ^ set(declared_symbols()))


def test_header_symbols_are_exported_and_bound():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 26
    for n in names:
        assert hasattr(lib, n), n
        assert n in _lib.SIGNATURES, "no ctypes prototype for " + n


def test_reference_symbol_names_are_all_there():
    # the 17 batch-norm symbols + flat join + ReLU pair of the reference's bindgen whitelist
    # (build.rs:65-82, 90, 98-99)
    want = """anode_gpu_batch_mean_3d1_packed_f32 anode_gpu_batch_mean_bwd_3d1_packed_f32
    anode_gpu_batch_mean_bwd_3d1_packed_accumulate_f32 anode_gpu_batch_var_3d1_packed_f32
    anode_gpu_batch_var_bwd_3d1_packed_f32 anode_gpu_batch_var_bwd_3d1_packed_accumulate_f32
    anode_gpu_batch_var_bwd_mean_3d1_packed_f32 anode_gpu_batch_var_bwd_mean_3d1_packed_accumulate_f32
    anode_gpu_batch_norm_3d1_packed_f32 anode_gpu_batch_norm_bwd_3d1_packed_f32
    anode_gpu_batch_norm_bwd_3d1_packed_accumulate_f32 anode_gpu_batch_norm_bwd_mean_3d1_packed_f32
    anode_gpu_batch_norm_bwd_mean_3d1_packed_accumulate_f32 anode_gpu_batch_norm_bwd_var_3d1_packed_f32
    anode_gpu_batch_norm_bwd_var_3d1_packed_accumulate_f32 anode_gpu_batch_norm_bwd_var_v2_3d1_packed_f32
    anode_gpu_batch_norm_bwd_var_v2_3d1_packed_accumulate_f32
    anode_gpu_M1_copy_map_M2_unit_step_map_R_product_reduce_flat_join_f32
    anode_gpu_positive_clip_flat_map_f32 anode_gpu_positive_clip_flat_map_bwd_f32""".split()
    lib = _lib.load()
    for n in want:
        assert hasattr(lib, n), n


def test_workspace_size_and_argument_checks_without_gpu():
    lib = _lib.load()
    assert lib.anode_gpu_batch_norm_fused_workspace_bytes(12544, 64, 256) > 0
    assert lib.anode_gpu_batch_norm_fused_workspace_bytes(0, 64, 256) == 0
    assert lib.anode_gpu_batch_norm_fused_workspace_bytes(1 << 16, 1 << 16, 2) == 0     # 2^33 elements
    # rejected before anything touches a device
    rc = lib.anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(4, 2, 2, 1e-5, 0.1, 1, None, None, None, None, None,
                                                                None, None, None, None, 0, None, None)
    assert rc == -1
    rc = lib.anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32(4, 0, 2, 1, 0, None, None, None, None, None, None,
                                                                None, None, None, None, 0, None, None)
    assert rc == -2
    st = ctypes.c_uint32(7)
    assert lib.anode_gpu_batch_norm_fused_status(None, None, ctypes.byref(st)) == -1


def test_kernel_config_layout():
    # routines_gpu/common.cuh:65-66: two uint32_t, block_sz first
    assert ctypes.sizeof(_lib.KernelConfig) == 8
    assert _lib.KernelConfig.block_sz.offset == 0 and _lib.KernelConfig.max_block_ct.offset == 4
