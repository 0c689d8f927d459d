// UNVERIFIED SOURCE: there is no Rust toolchain (rustc, cargo, bindgen) in the image this library is
// built in, and anode's sibling crates (gpudevicemem, cuda, ...) are not vendored, so this file has never
// been compiled.  It is what `bindgen` would produce from include/anode_routines_gpu.h for the entry
// points that are NOT part of anode's own routines_gpu/lib.h (those keep their names and signatures, so
// anode's existing bindings, src/ffi.rs:21-37 and build.rs:62-119, cover them unchanged).
//
// Where it goes in anode: next to src/ffi.rs, e.g. `pub mod routines_gpu_fused` in src/ffi.rs, or add
// the symbol names below to the bindgen whitelist in build.rs and let it generate the same thing.

#![allow(non_camel_case_types)]
#![allow(non_snake_case)]

use std::os::raw::{c_int, c_void};

use cuda::ffi::runtime::CUstream_st;
use gpudevicemem::ffi::routines_gpu::KernelConfig;

/// Opaque communicator of the synchronized entry points.
#[repr(C)]
pub struct AnodeSyncComm { _private: [u8; 0] }

pub const ANODE_OK: c_int = 0;
pub const ANODE_E_NULL: c_int = -1;
pub const ANODE_E_DIMS: c_int = -2;
pub const ANODE_E_WORKSPACE: c_int = -3;
pub const ANODE_E_LAUNCH: c_int = -4;
pub const ANODE_E_COMM: c_int = -5;
pub const ANODE_E_ALIGN: c_int = -6;
pub const ANODE_E_TOO_LARGE: c_int = -7;
pub const ANODE_ST_WAIT_STATS: u32 = 1;
pub const ANODE_ST_WAIT_PEER: u32 = 2;
pub const ANODE_ST_ABORTED: u32 = 4;
pub const ANODE_KERNEL_AUTO: c_int = 0;
pub const ANODE_KERNEL_TILED: c_int = 1;
pub const ANODE_KERNEL_CLUSTER: c_int = 2;
pub const ANODE_KERNEL_RESIDENT: c_int = 3;
pub const ANODE_KERNEL_PLAIN: c_int = 4;
pub const ANODE_STATIC_SCRATCH_BYTES: usize = 4 << 20;

#[link(name = "anode_routines_gpu")]
extern "C" {
  pub fn anode_gpu_batch_norm_fused_set_kernel(
    kernel: c_int,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_fused_set_wait_limit_ms(
    ms: u32,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_fused_workspace_bytes(
    dim0: u32,
    dim1: u32,
    dim2: u32,
  ) -> usize;
  pub fn anode_gpu_batch_norm_fused_workspace_init(
    workspace: *mut c_void,
    bytes: usize,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_fused_status(
    workspace: *const c_void,
    stream: *mut CUstream_st,
    status: *mut u32,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    epsilon: f32,
    avg_rate: f32,
    relu: c_int,
    x: *const f32,
    gamma: *const f32,
    beta: *const f32,
    y: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    relu: c_int,
    accumulate: c_int,
    dy: *const f32,
    x: *const f32,
    mean: *const f32,
    var: *const f32,
    gamma: *const f32,
    beta: *const f32,
    dx: *mut f32,
    dgamma: *mut f32,
    dbeta: *mut f32,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_act_fused_fwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    epsilon: f32,
    avg_rate: f32,
    neg_slope: f32,
    x: *const f32,
    gamma: *const f32,
    beta: *const f32,
    y: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_act_fused_bwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    neg_slope: f32,
    accumulate: c_int,
    dy: *const f32,
    x: *const f32,
    mean: *const f32,
    var: *const f32,
    gamma: *const f32,
    beta: *const f32,
    dx: *mut f32,
    dgamma: *mut f32,
    dbeta: *mut f32,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_add_act_fused_fwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    epsilon: f32,
    avg_rate: f32,
    neg_slope: f32,
    x: *const f32,
    residual: *const f32,
    gamma: *const f32,
    beta: *const f32,
    y: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_add_act_fused_bwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    neg_slope: f32,
    accumulate: c_int,
    dy: *const f32,
    x: *const f32,
    y: *const f32,
    mean: *const f32,
    var: *const f32,
    gamma: *const f32,
    beta: *const f32,
    dx: *mut f32,
    dresidual: *mut f32,
    dgamma: *mut f32,
    dbeta: *mut f32,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_relu_fused_fwd_static_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    epsilon: f32,
    avg_rate: f32,
    relu: c_int,
    x: *const f32,
    gamma: *const f32,
    beta: *const f32,
    y: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_fused_static_status(
    stream: *mut CUstream_st,
    status: *mut u32,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_host_step_staging_bytes(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    chunk_channels: u32,
  ) -> usize;
  pub fn anode_gpu_batch_norm_host_step_blocks(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    chunk_channels: u32,
  ) -> u32;
  pub fn anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    epsilon: f32,
    avg_rate: f32,
    relu: c_int,
    host_x: *const f32,
    host_dy: *const f32,
    gamma: *const f32,
    beta: *const f32,
    host_y: *mut f32,
    host_dx: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    dgamma: *mut f32,
    dbeta: *mut f32,
    staging: *mut c_void,
    staging_bytes: usize,
    chunk_channels: u32,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_batch_norm_act_infer_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    neg_slope: f32,
    x: *const f32,
    mean: *const f32,
    var: *const f32,
    gamma: *const f32,
    beta: *const f32,
    y: *mut f32,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_online_average_f32(
    len: u32,
    rate: f32,
    x: *const f32,
    y: *mut f32,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_sync_unique_id_bytes(

  ) -> usize;
  pub fn anode_gpu_sync_get_unique_id(
    out: *mut c_void,
  ) -> c_int;
  pub fn anode_gpu_sync_comm_create(
    unique_id: *const c_void,
    rank: c_int,
    world: c_int,
    out: *mut *mut AnodeSyncComm,
  ) -> c_int;
  pub fn anode_gpu_sync_comm_destroy(
    comm: *mut AnodeSyncComm,
  ) -> c_int;
  pub fn anode_gpu_sync_comm_create_exchange_only(
    rank: c_int,
    world: c_int,
    out: *mut *mut AnodeSyncComm,
  ) -> c_int;
  pub fn anode_gpu_sync_allreduce_sum_f32(
    comm: *mut AnodeSyncComm,
    buf: *mut f32,
    len: usize,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_sync_exchange_bytes(
    max_channels: u32,
    world: c_int,
  ) -> usize;
  pub fn anode_gpu_sync_comm_attach_exchange(
    comm: *mut AnodeSyncComm,
    peer_ptrs: *const *mut c_void,
    max_channels: u32,
  ) -> c_int;
  pub fn anode_gpu_sync_batch_norm_workspace_bytes(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    world: c_int,
  ) -> usize;
  pub fn anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    epsilon: f32,
    avg_rate: f32,
    relu: c_int,
    x: *const f32,
    gamma: *const f32,
    beta: *const f32,
    y: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    comm: *mut AnodeSyncComm,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    global_count: u64,
    relu: c_int,
    accumulate: c_int,
    dy: *const f32,
    x: *const f32,
    mean: *const f32,
    var: *const f32,
    gamma: *const f32,
    beta: *const f32,
    dx: *mut f32,
    dgamma: *mut f32,
    dbeta: *mut f32,
    comm: *mut AnodeSyncComm,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_sync_batch_norm_host_step_staging_bytes(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    global_count: u64,
    comm: *mut AnodeSyncComm,
    chunk_channels: u32,
  ) -> usize;
  pub fn anode_gpu_sync_batch_norm_host_step_blocks(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    global_count: u64,
    comm: *mut AnodeSyncComm,
    chunk_channels: u32,
  ) -> u32;
  pub fn anode_gpu_sync_batch_norm_relu_step_host_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    global_count: u64,
    epsilon: f32,
    avg_rate: f32,
    relu: c_int,
    host_x: *const f32,
    host_dy: *const f32,
    gamma: *const f32,
    beta: *const f32,
    host_y: *mut f32,
    host_dx: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    dgamma: *mut f32,
    dbeta: *mut f32,
    comm: *mut AnodeSyncComm,
    staging: *mut c_void,
    staging_bytes: usize,
    chunk_channels: u32,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_sync_batch_norm_add_act_fwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    epsilon: f32,
    avg_rate: f32,
    neg_slope: f32,
    x: *const f32,
    residual: *const f32,
    gamma: *const f32,
    beta: *const f32,
    y: *mut f32,
    mean: *mut f32,
    var: *mut f32,
    run_mean: *mut f32,
    run_var: *mut f32,
    comm: *mut AnodeSyncComm,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
  pub fn anode_gpu_sync_batch_norm_add_act_bwd_3d1_packed_f32(
    dim0: u32,
    dim1: u32,
    dim2: u32,
    global_count: u64,
    neg_slope: f32,
    accumulate: c_int,
    dy: *const f32,
    x: *const f32,
    y: *const f32,
    mean: *const f32,
    var: *const f32,
    gamma: *const f32,
    beta: *const f32,
    dx: *mut f32,
    dresidual: *mut f32,
    dgamma: *mut f32,
    dbeta: *mut f32,
    comm: *mut AnodeSyncComm,
    workspace: *mut c_void,
    workspace_bytes: usize,
    cfg: *const KernelConfig,
    stream: *mut CUstream_st,
  ) -> c_int;
}
