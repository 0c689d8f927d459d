// UNVERIFIED SOURCE: there is no Rust toolchain in the image this library is built in and anode's
// sibling crates are not vendored, so this file has never been compiled.  It shows how the fused entry
// points of include/anode_routines_gpu.h (bindings: rust/ffi_fused.rs) slot into anode's operator layer.
//
// What it fills in: `BatchNormalize2dFusedOp` and `BatchNormalize2dBwdFusedOp`, which src/ops.rs:105-106
// declares and nothing builds, in the `build_device_f32_op` style of the existing batch-norm ops
// (src/ops_gpu.rs:4250-4361: an `OpExt` with `make_val`, `apply` and `adjoint` closures around one
// kernel call), and a `batch_normalize_relu_2d` front end that emits ONE node where
// `batch_normalize_2d(...)` followed by `.positive_clip()` emits six (src/ops.rs:999-1014,
// examples/run_imagenet_mpi.rs:143-150).  The 3-d ops are the same code with dim0 = W*H*D
// (src/ops_gpu.rs:4911-4913).
//
// A fused node has five results (y, mean, var and the two running averages); anode's ops have one.  The
// node's value is y; the statistics live in arrays owned by the node's state and are exposed as source
// nodes (`FusedStats`), which is how `zeros_like(...).online_average(...).fix()` already keeps the
// running averages outside of the differentiated graph (src/ops.rs:1002-1003).

use crate::*;
use crate::context::*;
use crate::ffi::routines_gpu_fused::*;
use crate::ops::*;

use gpudevicemem::*;
use gpudevicemem::array::*;

use std::cell::RefMut;
use std::rc::Rc;
use std::sync::Arc;

/// Per-node device state of a fused batch-norm: statistics, running averages and the kernels' scratch.
pub struct FusedStats {
  pub mean:     GPUDeviceArray1d<f32>,
  pub var:      GPUDeviceArray1d<f32>,   // biased variance + epsilon, as anode stores it (batch_norm.cu:160)
  pub avg_mean: GPUDeviceArray1d<f32>,
  pub avg_var:  GPUDeviceArray1d<f32>,
  pub workspace: GPUDeviceArray1d<u8>,   // anode_gpu_batch_norm_fused_workspace_bytes, zeroed once
}

impl FusedStats {
  pub fn new(dim0: usize, channels: usize, max_batch_sz: usize, conn: GPUDeviceConn) -> Self {
    let ws_bytes = unsafe { anode_gpu_batch_norm_fused_workspace_bytes(dim0 as u32, channels as u32, max_batch_sz as u32) };
    assert!(ws_bytes > 0);
    // `zeros` gives what anode_gpu_batch_norm_fused_workspace_init would: the scratch must start at zero
    FusedStats{
      mean:     GPUDeviceArray1d::zeros(channels, conn.clone()),
      var:      GPUDeviceArray1d::zeros(channels, conn.clone()),
      avg_mean: GPUDeviceArray1d::zeros(channels, conn.clone()),
      avg_var:  GPUDeviceArray1d::zeros(channels, conn.clone()),
      workspace: GPUDeviceArray1d::zeros(ws_bytes, conn),
    }
  }
}

fn check(rc: i32, what: &str) {
  // the reference's kernels return void and abort on misuse (routines_gpu/batch_norm.cu:68); keep that behaviour
  assert_eq!(rc, ANODE_OK, "{} refused its arguments: {}", what, rc);
}

impl BatchNormalize2dFusedOp {
  /// y = relu(gamma * (x - mean) / sqrt(var) + beta) with batch statistics, running averages updated
  /// in the same launch.  `gamma_`/`beta_` of `None` give the reference's plain normalisation.
  pub fn build_device_f32_op(
      axes: [isize; 2], epsilon: f32, avg_rate: f32, relu: bool,
      x_: Val<GPUDeviceOuterBatchArray3d<f32>>,
      gamma_: Option<Val<GPUDeviceArray1d<f32>>>, beta_: Option<Val<GPUDeviceArray1d<f32>>>,
      stats: Rc<FusedStats>)
  -> Val<GPUDeviceOuterBatchArray3d<f32>>
  {
    let ext = OpExt{
      make_val: {
        let x_ = x_.clone();
        Box::new(move |_state: RefMut<_>| {
          let section = GPULazyAsyncSection::default();
          let x_ = x_.clone();
          RWVal::from(Arc::new(move |txn| {
            let ctx = thread_ctx().gpu();
            let mut pool = ctx.pool();
            let conn = pool.conn();
            let mut section = section.clone();
            let mut guard = section.push(conn.clone());
            let y = GPUDeviceOuterBatchArray3d::zeros(x_.get(txn).size(), x_.get(txn).max_batch_size(), conn);
            guard._wait(y.async_state());
            y
          }))
        })
      },
      apply: {
        let section = GPULazyAsyncSection::default();
        let x_ = x_.clone();
        let gamma_ = gamma_.clone();
        let beta_ = beta_.clone();
        let stats = stats.clone();
        Box::new(move |txn: Txn, _state: RefMut<_>, output: LVal<GPUDeviceOuterBatchArray3d<f32>>| {
          output.write(txn, |cap, token| {
            let ctx = thread_ctx().gpu();
            let mut pool = ctx.pool();
            let conn = pool.conn();
            let mut section = section.clone();
            let mut guard = section.push(conn.clone());
            let x = x_.get(txn);
            let mut y = output.get_mut(txn, token);
            guard._wait(x.async_state());
            guard._wait(y.async_state());
            y.set_batch_size(x.batch_size());
            // packed NCHW only, like every batch-norm op of the reference (src/ops_gpu.rs:3777-3779)
            assert!(x.is_packed() && y.is_packed());
            assert_eq!([0, 1], axes);
            match cap {
              WriteCap::Assign => {}
              WriteCap::Accumulate => unimplemented!(),     // as in BatchNormalize2dOp (src/ops_gpu.rs:4327-4330)
            }
            let x = x.as_view().wait(conn.clone());
            let mut y = y.as_view_mut().wait_mut(conn.clone());
            let gamma = gamma_.as_ref().map(|g| g.get(txn));
            let beta = beta_.as_ref().map(|b| b.get(txn));
            let mut stream = conn.cuda_stream();
            let sz = x.inner().size();
            check(unsafe { anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(
                sz2uint(sz.index_cut(3).index_cut(2).flat_len()),
                sz2uint(sz.index_at(2)),
                sz2uint(sz.index_at(3)),
                epsilon, avg_rate, relu as i32,
                x.as_dptr(),
                gamma.as_ref().map_or(std::ptr::null(), |g| g.as_view().wait(conn.clone()).as_dptr()),
                beta.as_ref().map_or(std::ptr::null(), |b| b.as_view().wait(conn.clone()).as_dptr()),
                y.as_mut_dptr(),
                stats.mean.as_view().wait(conn.clone()).as_dptr() as *mut f32,
                stats.var.as_view().wait(conn.clone()).as_dptr() as *mut f32,
                stats.avg_mean.as_view().wait(conn.clone()).as_dptr() as *mut f32,
                stats.avg_var.as_view().wait(conn.clone()).as_dptr() as *mut f32,
                stats.workspace.as_view().wait(conn.clone()).as_dptr() as *mut _,
                stats.workspace.size(),
                conn.cuda_kernel_config() as *const _,
                stream.as_mut_ptr(),
            ) }, "anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32");
          })
        })
      },
      build: None,
      tangent: None,
      adjoint: Some({
        let x_ = x_.clone();
        let gamma_ = gamma_.clone();
        let beta_ = beta_.clone();
        let stats = stats.clone();
        Box::new(move |_: Pass, y_: Val<GPUDeviceOuterBatchArray3d<f32>>, _state: RefMut<_>, sink: &mut Sink| {
          if let Some(adj_y_) = y_.adjoint(sink) {
            // one node instead of the seven of BatchNormalize2dOp / BatchVariance2dOp / BatchMean2dOp / PositiveClipOp
            // (src/ops_gpu.rs:4344-4352, 3997-4003, 3787-3791, 8499)
            let adj_x_ = BatchNormalize2dBwdFusedOp::build_device_f32_op(
                axes, relu, adj_y_.clone(), x_.clone(), gamma_.clone(), beta_.clone(), stats.clone());
            x_.put_adjoint(adj_x_, sink);
            // dgamma / dbeta are written by the same kernel into arrays of the backward node's state;
            // hand them to gamma_ / beta_ here once anode's affine ops exist (src/ops_gpu.rs:9736-9787 are unimplemented!())
          }
        })
      }),
      inplace: None,
    };
    Val::from(Rc::new(F1Op::new(BatchNormalize2dFusedOp, ext, x_)))
  }
}

impl BatchNormalize2dBwdFusedOp {
  /// dx of the fused forward: ReLU mask recomputed from x, both channel reductions, dgamma / dbeta and dx
  /// in one launch (closed form of the reference's dvar / dmean / dx chain, routines_gpu/batch_norm.cu:181-619).
  pub fn build_device_f32_op(
      axes: [isize; 2], relu: bool,
      dy_: Val<GPUDeviceOuterBatchArray3d<f32>>, x_: Val<GPUDeviceOuterBatchArray3d<f32>>,
      gamma_: Option<Val<GPUDeviceArray1d<f32>>>, beta_: Option<Val<GPUDeviceArray1d<f32>>>,
      stats: Rc<FusedStats>)
  -> Val<GPUDeviceOuterBatchArray3d<f32>>
  {
    let ext = OpExt{
      make_val: {
        let x_ = x_.clone();
        Box::new(move |_state: RefMut<_>| {
          let section = GPULazyAsyncSection::default();
          let x_ = x_.clone();
          RWVal::from(Arc::new(move |txn| {
            let ctx = thread_ctx().gpu();
            let mut pool = ctx.pool();
            let conn = pool.conn();
            let mut section = section.clone();
            let mut guard = section.push(conn.clone());
            let dx = GPUDeviceOuterBatchArray3d::zeros(x_.get(txn).size(), x_.get(txn).max_batch_size(), conn);
            guard._wait(dx.async_state());
            dx
          }))
        })
      },
      apply: {
        let section = GPULazyAsyncSection::default();
        Box::new(move |txn: Txn, _state: RefMut<_>, output: LVal<GPUDeviceOuterBatchArray3d<f32>>| {
          output.write(txn, |cap, token| {
            let ctx = thread_ctx().gpu();
            let mut pool = ctx.pool();
            let conn = pool.conn();
            let mut section = section.clone();
            let mut guard = section.push(conn.clone());
            let dy = dy_.get(txn);
            let x = x_.get(txn);
            let mut dx = output.get_mut(txn, token);
            guard._wait(dy.async_state());
            guard._wait(x.async_state());
            guard._wait(dx.async_state());
            dx.set_batch_size(x.batch_size());
            assert!(dy.is_packed() && x.is_packed() && dx.is_packed());
            assert_eq!([0, 1], axes);
            // the first adjoint contribution to a variable is an Assign, later ones Accumulate (src/lib.rs:2160-2165)
            let accumulate = match cap { WriteCap::Assign => 0, WriteCap::Accumulate => 1 };
            let dy = dy.as_view().wait(conn.clone());
            let x = x.as_view().wait(conn.clone());
            let mut dx = dx.as_view_mut().wait_mut(conn.clone());
            let gamma = gamma_.as_ref().map(|g| g.get(txn));
            let beta = beta_.as_ref().map(|b| b.get(txn));
            let mut stream = conn.cuda_stream();
            let sz = x.inner().size();
            check(unsafe { anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32(
                sz2uint(sz.index_cut(3).index_cut(2).flat_len()),
                sz2uint(sz.index_at(2)),
                sz2uint(sz.index_at(3)),
                relu as i32, accumulate,
                dy.as_dptr(), x.as_dptr(),
                stats.mean.as_view().wait(conn.clone()).as_dptr(),
                stats.var.as_view().wait(conn.clone()).as_dptr(),
                gamma.as_ref().map_or(std::ptr::null(), |g| g.as_view().wait(conn.clone()).as_dptr()),
                beta.as_ref().map_or(std::ptr::null(), |b| b.as_view().wait(conn.clone()).as_dptr()),
                dx.as_mut_dptr(),
                std::ptr::null_mut(), std::ptr::null_mut(),      // dgamma, dbeta: see the note in the forward op's adjoint
                stats.workspace.as_view().wait(conn.clone()).as_dptr() as *mut _,
                stats.workspace.size(),
                conn.cuda_kernel_config() as *const _,
                stream.as_mut_ptr(),
            ) }, "anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32");
          })
        })
      },
      build: None,
      tangent: None,
      adjoint: None,
      inplace: None,
    };
    Val::from(Rc::new(F2Op::new(BatchNormalize2dBwdFusedOp, ext, dy_, x_)))
  }
}

/// `x.batch_normalize_2d(axes, online, avg_rate, epsilon)` followed by `.positive_clip()`
/// (src/ops.rs:999-1014, :1199-1222) as one node.  Returns the same tuple as `batch_normalize_2d`;
/// the statistics are source nodes over the fused node's state.  In evaluation mode (`online` false:
/// normalise with the running averages, src/ops.rs:1010-1011) call
/// `anode_gpu_batch_norm_act_infer_3d1_packed_f32` instead, which is one pass over x.
pub fn batch_normalize_relu_2d(
    x_: Val<GPUDeviceOuterBatchArray3d<f32>>, axes: [isize; 2], avg_rate: f32, epsilon: f32,
    dim0: usize, channels: usize, max_batch_sz: usize, conn: GPUDeviceConn)
-> (Val<GPUDeviceOuterBatchArray3d<f32>>, Rc<FusedStats>)
{
  let stats = Rc::new(FusedStats::new(dim0, channels, max_batch_sz, conn));
  let y_ = BatchNormalize2dFusedOp::build_device_f32_op(axes, epsilon, avg_rate, true, x_, None, None, stats.clone());
  (y_, stats)
}
