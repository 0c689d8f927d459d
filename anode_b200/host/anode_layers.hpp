// Compositions and fused operators on top of anode_ops.hpp (included from there).
#pragma once

namespace anode {

// `x.batch_normalize_2d(axes, online, avg_rate, epsilon)` of src/ops.rs:999-1014 (3-D: :1043-1055):
// five launches in the reference's order.  avg_mean / avg_var are the running averages (zeros when
// empty, as `zeros_like(...)` in the reference) and are updated in place; `online` picks the batch
// statistics, otherwise the running ones normalize (`switch(online, avg, batch)`).
struct BatchNormalizeOut { DeviceArray y, mean, var; };
inline BatchNormalizeOut batch_normalize_2d(const DeviceArray &x, const std::vector<int> &axes, bool online, float avg_rate,
                                            float epsilon, DeviceArray &avg_mean, DeviceArray &avg_var, cudaStream_t s = 0)
{
  const Dims d = dims_of(x, axes);
  BatchNormalizeOut o{DeviceArray(x.size()), DeviceArray::zeros({d.dim1}, s), DeviceArray::zeros({d.dim1}, s)};
  if (avg_mean.empty()) avg_mean = DeviceArray::zeros({d.dim1}, s);
  if (avg_var.empty()) avg_var = DeviceArray::zeros({d.dim1}, s);
  BatchMean2dOp::apply(axes, x, o.mean, s);
  BatchVariance2dOp::apply(axes, epsilon, x, o.mean, o.var, s);
  OnlineAverageOp::apply(avg_rate, o.mean, avg_mean, s);
  OnlineAverageOp::apply(avg_rate, o.var, avg_var, s);
  if (online) BatchNormalize2dOp::apply(axes, x, o.mean, o.var, o.y, s);
  else BatchNormalize2dOp::apply(axes, x, avg_mean, avg_var, o.y, s);
  return o;
}
inline BatchNormalizeOut batch_normalize_3d(const DeviceArray &x, const std::vector<int> &axes, bool online, float avg_rate,
                                            float epsilon, DeviceArray &avg_mean, DeviceArray &avg_var, cudaStream_t s = 0)
{
  return batch_normalize_2d(x, axes, online, avg_rate, epsilon, avg_mean, avg_var, s);
}

// Adjoint of the training-mode composition with respect to x, as the reference's sink evaluates it:
// BatchNormalize2dOp's adjoint emits (adj_x, adj_mean, adj_var) (src/ops_gpu.rs:4344-4352),
// BatchVariance2dOp's (adj_x, adj_mean) (:3997-4003), BatchMean2dOp's adj_x (:3787-3791); the first
// contribution to a variable is an Assign, later ones Accumulate (src/lib.rs:2160-2165).  Six launches.
inline DeviceArray batch_normalize_adjoint(const std::vector<int> &axes, const DeviceArray &dy_bn, const DeviceArray &x,
                                           const DeviceArray &mean, const DeviceArray &var, cudaStream_t s = 0)
{
  const Dims d = dims_of(x, axes);
  DeviceArray dvar = DeviceArray::zeros({d.dim1}, s), dmean = DeviceArray::zeros({d.dim1}, s), dx(x.size());
  BatchNormalize2dBwdVarianceOp::apply(axes, dy_bn, x, mean, var, dvar, WriteCap::Assign, s);
  BatchNormalize2dBwdMeanOp::apply(axes, dy_bn, var, dmean, WriteCap::Assign, s);
  BatchVariance2dBwdMeanOp::apply(axes, dvar, x, mean, dmean, WriteCap::Accumulate, s);
  BatchNormalize2dBwdOp::apply(axes, dy_bn, var, dx, WriteCap::Assign, s);
  BatchVariance2dBwdOp::apply(axes, dvar, x, mean, dx, WriteCap::Accumulate, s);
  BatchMean2dBwdOp::apply(axes, dmean, dx, WriteCap::Accumulate, s);
  return dx;
}

// Scratch of the fused operators for one layer shape (zeroed once; the kernels leave it clean).
class Workspace {
 public:
  Workspace() = default;
  Workspace(Dims d, cudaStream_t s = 0) : dims_(d)
  {
    bytes_ = anode_gpu_batch_norm_fused_workspace_bytes(d.dim0, d.dim1, d.dim2);
    if (bytes_ == 0) throw Error(ANODE_E_DIMS, "anode_gpu_batch_norm_fused_workspace_bytes");
    cuda_check(cudaMalloc(&ptr_, bytes_), "cudaMalloc");
    check(anode_gpu_batch_norm_fused_workspace_init(ptr_, bytes_, raw(s)), "anode_gpu_batch_norm_fused_workspace_init");
  }
  Workspace(Workspace &&o) noexcept { *this = std::move(o); }
  Workspace &operator=(Workspace &&o) noexcept
  {
    if (this != &o) { if (ptr_) (void)cudaFree(ptr_); ptr_ = o.ptr_; bytes_ = o.bytes_; dims_ = o.dims_; o.ptr_ = nullptr; o.bytes_ = 0; }
    return *this;
  }
  Workspace(const Workspace &) = delete;
  Workspace &operator=(const Workspace &) = delete;
  ~Workspace() { if (ptr_) (void)cudaFree(ptr_); }
  void *ptr() const { return ptr_; }
  size_t bytes() const { return bytes_; }
  bool fits(Dims d) const { return ptr_ && d.dim0 == dims_.dim0 && d.dim1 == dims_.dim1 && d.dim2 == dims_.dim2; }
  // Device status word (0 = clean); synchronises the stream.
  uint32_t status(cudaStream_t s = 0) const
  {
    uint32_t st = 0;
    check(anode_gpu_batch_norm_fused_status(ptr_, raw(s), &st), "anode_gpu_batch_norm_fused_status");
    return st;
  }

 private:
  void *ptr_ = nullptr;
  size_t bytes_ = 0;
  Dims dims_{0, 0, 0};
};

inline const float *opt(const DeviceArray *a) { return (a && !a->empty()) ? a->ptr() : nullptr; }
inline float *opt(DeviceArray *a) { return (a && !a->empty()) ? a->ptr() : nullptr; }

// The fused operator src/ops.rs:105 declares: statistics, running averages, normalize, optional
// affine and ReLU in one launch.  gamma / beta / avg_* may be null (no affine is the reference's behaviour).
struct BatchNormalize2dFusedOp {
  static void apply(const std::vector<int> &axes, float epsilon, float avg_rate, const DeviceArray &x, DeviceArray &y,
                    DeviceArray &mean, DeviceArray &var, DeviceArray *avg_mean, DeviceArray *avg_var, const DeviceArray *gamma,
                    const DeviceArray *beta, bool relu, Workspace &ws, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes);
    want_len(y, x.len(), "y"); want_len(mean, d.dim1, "mean"); want_len(var, d.dim1, "var");
    check(anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(d.dim0, d.dim1, d.dim2, epsilon, avg_rate, relu ? 1 : 0, x.ptr(), opt(gamma),
                                                             opt(beta), y.ptr(), mean.ptr(), var.ptr(), opt(avg_mean), opt(avg_var),
                                                             ws.ptr(), ws.bytes(), kernel_config(), raw(s)),
          "anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32");
  }
};
// Its adjoint (src/ops.rs:106): ReLU mask, both channel sums, dgamma / dbeta and dx in one launch.
struct BatchNormalize2dBwdFusedOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &dy, const DeviceArray &x, const DeviceArray &mean,
                    const DeviceArray &var, DeviceArray &dx, const DeviceArray *gamma, const DeviceArray *beta, DeviceArray *dgamma,
                    DeviceArray *dbeta, bool relu, WriteCap cap, Workspace &ws, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes);
    want_len(dy, x.len(), "dy"); want_len(dx, x.len(), "dx");
    check(anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32(d.dim0, d.dim1, d.dim2, relu ? 1 : 0, cap == WriteCap::Accumulate ? 1 : 0,
                                                             dy.ptr(), x.ptr(), mean.ptr(), var.ptr(), opt(gamma), opt(beta), dx.ptr(),
                                                             opt(dgamma), opt(dbeta), ws.ptr(), ws.bytes(), kernel_config(), raw(s)),
          "anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32");
  }
};
// Inference: given statistics and the activation after them in one pass (neg_slope 0 = ReLU,
// 1 = none, c = leaky ReLU as routines_gpu/flat_map.cu:44-52).
struct BatchNormalize2dActInferOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &x, const DeviceArray &mean, const DeviceArray &var, DeviceArray &y,
                    const DeviceArray *gamma, const DeviceArray *beta, float neg_slope, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes);
    want_len(y, x.len(), "y");
    check(anode_gpu_batch_norm_act_infer_3d1_packed_f32(d.dim0, d.dim1, d.dim2, neg_slope, x.ptr(), mean.ptr(), var.ptr(), opt(gamma),
                                                        opt(beta), y.ptr(), kernel_config(), raw(s)),
          "anode_gpu_batch_norm_act_infer_3d1_packed_f32");
  }
};
using BatchNormalize3dFusedOp = BatchNormalize2dFusedOp;
using BatchNormalize3dBwdFusedOp = BatchNormalize2dBwdFusedOp;
using BatchNormalize3dActInferOp = BatchNormalize2dActInferOp;

// A batch-norm + ReLU layer that keeps its own buffers, so that a training loop makes two calls
// per step: forward(x, y) and backward(dy, dx) (x is remembered by reference between the two).
class FusedBatchNormRelu {
 public:
  FusedBatchNormRelu(uint32_t channels, float epsilon = 1e-5f, float avg_rate = 0.1f, bool affine = true, bool relu = true)
      : avg_mean(DeviceArray::zeros({channels})), avg_var(DeviceArray::filled({channels}, 1.0f)),
        mean(DeviceArray::zeros({channels})), var(DeviceArray::zeros({channels})),
        epsilon_(epsilon), avg_rate_(avg_rate), relu_(relu)
  {
    if (affine) {
      gamma = DeviceArray::filled({channels}, 1.0f); beta = DeviceArray::zeros({channels});
      dgamma = DeviceArray::zeros({channels}); dbeta = DeviceArray::zeros({channels});
    }
  }
  void forward(const DeviceArray &x, DeviceArray &y, cudaStream_t s = 0)
  {
    const std::vector<int> axes = leading_axes(x);
    workspace_for(dims_of(x, axes), s);
    BatchNormalize2dFusedOp::apply(axes, epsilon_, avg_rate_, x, y, mean, var, &avg_mean, &avg_var, &gamma, &beta, relu_, ws_, s);
    x_ = &x;
  }
  void backward(const DeviceArray &dy, DeviceArray &dx, WriteCap cap = WriteCap::Assign, cudaStream_t s = 0)
  {
    if (!x_) throw Error(ANODE_E_NULL, "backward before forward");
    const std::vector<int> axes = leading_axes(*x_);
    BatchNormalize2dBwdFusedOp::apply(axes, dy, *x_, mean, var, dx, &gamma, &beta, &dgamma, &dbeta, relu_, cap, ws_, s);
  }
  void infer(const DeviceArray &x, DeviceArray &y, cudaStream_t s = 0)
  {
    BatchNormalize2dActInferOp::apply(leading_axes(x), x, avg_mean, avg_var, y, &gamma, &beta, relu_ ? 0.0f : 1.0f, s);
  }
  // x, dy, y, dx in (page-locked) host memory, sizes as `size` ([spatial..., C, N]); copies in both
  // directions overlap the kernels.  Everything is enqueued when the call returns.
  void step_from_host(const std::vector<uint32_t> &size, const float *hx, const float *hdy, float *hy, float *hdx,
                      uint32_t chunk_channels = 0, cudaStream_t s = 0)
  {
    if (size.size() < 3) throw Error(ANODE_E_DIMS, "batch array needs [spatial..., C, N]");
    uint64_t d0 = 1;
    for (size_t i = 0; i + 2 < size.size(); ++i) d0 *= size[i];
    const uint32_t c = size[size.size() - 2], n = size[size.size() - 1];
    const size_t need = anode_gpu_batch_norm_host_step_staging_bytes((uint32_t)d0, c, n, chunk_channels);
    if (need == 0) throw Error(ANODE_E_DIMS, "anode_gpu_batch_norm_host_step_staging_bytes");
    if (need > staging_bytes_) {
      if (staging_) (void)cudaFree(staging_);
      staging_ = nullptr; staging_bytes_ = 0;
      cuda_check(cudaMalloc(&staging_, need), "cudaMalloc");
      staging_bytes_ = need;
    }
    check(anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32((uint32_t)d0, c, n, epsilon_, avg_rate_, relu_ ? 1 : 0, hx, hdy,
                                                                   opt(&gamma), opt(&beta), hy, hdx, mean.ptr(), var.ptr(), avg_mean.ptr(),
                                                                   avg_var.ptr(), opt(&dgamma), opt(&dbeta), staging_, staging_bytes_,
                                                                   chunk_channels, kernel_config(), raw(s)),
          "anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32");
  }
  uint32_t status(cudaStream_t s = 0) const { return ws_.ptr() ? ws_.status(s) : 0u; }
  ~FusedBatchNormRelu() { if (staging_) (void)cudaFree(staging_); }
  FusedBatchNormRelu(const FusedBatchNormRelu &) = delete;
  FusedBatchNormRelu &operator=(const FusedBatchNormRelu &) = delete;

  DeviceArray gamma, beta, avg_mean, avg_var, mean, var, dgamma, dbeta;

 private:
  static std::vector<int> leading_axes(const DeviceArray &x)
  {
    std::vector<int> a;
    for (size_t i = 0; i + 2 < x.size().size(); ++i) a.push_back((int)i);
    return a;
  }
  void workspace_for(Dims d, cudaStream_t s) { if (!ws_.fits(d)) ws_ = Workspace(d, s); }
  float epsilon_, avg_rate_;
  bool relu_;
  Workspace ws_;
  const DeviceArray *x_ = nullptr;
  void *staging_ = nullptr;
  size_t staging_bytes_ = 0;
};

// Communicator of the synchronized entry points (one process per GPU).  `from_unique_id` wraps
// anode_gpu_sync_comm_create (NCCL behind it; the 128-byte id comes from rank 0 by any means, in anode over
// DistProcGroup, src/proc_mpi.rs:27-105); `exchange_only` has no NCCL and works once the world's exchange
// buffers are attached.
class SyncComm {
 public:
  static SyncComm from_unique_id(const void *id, int rank, int world)
  {
    SyncComm c; c.rank_ = rank; c.world_ = world;
    check(anode_gpu_sync_comm_create(id, rank, world, &c.h_), "anode_gpu_sync_comm_create");
    return c;
  }
  static SyncComm exchange_only(int rank, int world)
  {
    SyncComm c; c.rank_ = rank; c.world_ = world;
    check(anode_gpu_sync_comm_create_exchange_only(rank, world, &c.h_), "anode_gpu_sync_comm_create_exchange_only");
    return c;
  }
  // peer_ptrs[r]: rank r's exchange buffer as mapped into this process (anode_gpu_sync_exchange_bytes each, zeroed once)
  void attach_exchange(void *const *peer_ptrs, uint32_t max_channels)
  {
    check(anode_gpu_sync_comm_attach_exchange(h_, peer_ptrs, max_channels), "anode_gpu_sync_comm_attach_exchange");
  }
  // SumSpmdOp's role for gradients (src/ops_gpu.rs:538-545), on the device
  void allreduce_sum(DeviceArray &buf, cudaStream_t s = 0)
  {
    check(anode_gpu_sync_allreduce_sum_f32(h_, buf.ptr(), buf.len(), raw(s)), "anode_gpu_sync_allreduce_sum_f32");
  }
  AnodeSyncComm *handle() const { return h_; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  SyncComm(SyncComm &&o) noexcept : h_(o.h_), rank_(o.rank_), world_(o.world_) { o.h_ = nullptr; }
  SyncComm &operator=(SyncComm &&o) noexcept { if (this != &o) { reset(); h_ = o.h_; rank_ = o.rank_; world_ = o.world_; o.h_ = nullptr; } return *this; }
  SyncComm(const SyncComm &) = delete;
  SyncComm &operator=(const SyncComm &) = delete;
  ~SyncComm() { reset(); }

 private:
  SyncComm() = default;
  void reset() { if (h_) { (void)anode_gpu_sync_comm_destroy(h_); h_ = nullptr; } }
  AnodeSyncComm *h_ = nullptr;
  int rank_ = 0, world_ = 1;
};

// FusedBatchNormRelu over a batch sharded across the ranks of a SyncComm: statistics, running averages,
// dgamma and dbeta are those of the global batch (identical on every rank).  `global_count` is the number
// of elements per channel over all ranks (the M of the formulas); 0 means equal shards.
class SyncBatchNormRelu {
 public:
  SyncBatchNormRelu(SyncComm &comm, uint32_t channels, uint64_t global_count = 0, float epsilon = 1e-5f, float avg_rate = 0.1f,
                    bool affine = true, bool relu = true)
      : avg_mean(DeviceArray::zeros({channels})), avg_var(DeviceArray::filled({channels}, 1.0f)),
        mean(DeviceArray::zeros({channels})), var(DeviceArray::zeros({channels})),
        comm_(comm), global_count_(global_count), epsilon_(epsilon), avg_rate_(avg_rate), relu_(relu)
  {
    if (affine) {
      gamma = DeviceArray::filled({channels}, 1.0f); beta = DeviceArray::zeros({channels});
      dgamma = DeviceArray::zeros({channels}); dbeta = DeviceArray::zeros({channels});
    }
  }
  void forward(const DeviceArray &x, DeviceArray &y, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, leading_axes(x));
    want_len(y, x.len(), "y");
    workspace_for(d, s);
    check(anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32(d.dim0, d.dim1, d.dim2, epsilon_, avg_rate_, relu_ ? 1 : 0, x.ptr(), opt(&gamma),
                                                            opt(&beta), y.ptr(), mean.ptr(), var.ptr(), avg_mean.ptr(), avg_var.ptr(),
                                                            comm_.handle(), ws_, ws_bytes_, kernel_config(), raw(s)),
          "anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32");
    x_ = &x;
  }
  void backward(const DeviceArray &dy, DeviceArray &dx, WriteCap cap = WriteCap::Assign, cudaStream_t s = 0)
  {
    if (!x_) throw Error(ANODE_E_NULL, "backward before forward");
    const Dims d = dims_of(*x_, leading_axes(*x_));
    want_len(dx, x_->len(), "dx");
    const uint64_t total = global_count_ ? global_count_ : (uint64_t)d.dim0 * d.dim2 * (uint64_t)comm_.world();
    check(anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32(d.dim0, d.dim1, d.dim2, total, relu_ ? 1 : 0, cap == WriteCap::Accumulate ? 1 : 0,
                                                            dy.ptr(), x_->ptr(), mean.ptr(), var.ptr(), opt(&gamma), opt(&beta), dx.ptr(),
                                                            opt(&dgamma), opt(&dbeta), comm_.handle(), ws_, ws_bytes_, kernel_config(), raw(s)),
          "anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32");
  }
  uint32_t status(cudaStream_t s = 0) const
  {
    uint32_t st = 0;
    if (ws_) check(anode_gpu_batch_norm_fused_status(ws_, raw(s), &st), "anode_gpu_batch_norm_fused_status");
    return st;
  }
  ~SyncBatchNormRelu() { if (ws_) (void)cudaFree(ws_); }
  SyncBatchNormRelu(const SyncBatchNormRelu &) = delete;
  SyncBatchNormRelu &operator=(const SyncBatchNormRelu &) = delete;

  DeviceArray gamma, beta, avg_mean, avg_var, mean, var, dgamma, dbeta;

 private:
  static std::vector<int> leading_axes(const DeviceArray &x)
  {
    std::vector<int> a;
    for (size_t i = 0; i + 2 < x.size().size(); ++i) a.push_back((int)i);
    return a;
  }
  // a workspace belongs to one problem: a new shape gets a fresh, zeroed one
  void workspace_for(Dims d, cudaStream_t s)
  {
    if (ws_ && d.dim0 == dims_.dim0 && d.dim1 == dims_.dim1 && d.dim2 == dims_.dim2) return;
    if (ws_) { (void)cudaFree(ws_); ws_ = nullptr; }
    ws_bytes_ = anode_gpu_sync_batch_norm_workspace_bytes(d.dim0, d.dim1, d.dim2, comm_.world());
    if (ws_bytes_ == 0) throw Error(ANODE_E_DIMS, "anode_gpu_sync_batch_norm_workspace_bytes");
    cuda_check(cudaMalloc(&ws_, ws_bytes_), "cudaMalloc");
    check(anode_gpu_batch_norm_fused_workspace_init(ws_, ws_bytes_, raw(s)), "anode_gpu_batch_norm_fused_workspace_init");
    dims_ = d;
  }
  SyncComm &comm_;
  uint64_t global_count_;
  float epsilon_, avg_rate_;
  bool relu_;
  void *ws_ = nullptr;
  size_t ws_bytes_ = 0;
  Dims dims_{};
  const DeviceArray *x_ = nullptr;
};

}  // namespace anode
