// Host side of the batch-norm path in C++: the operator interface anode's Rust layer exposes for
// this path (src/ops.rs:983-1056, src/ops_gpu.rs:3690-5860, 6034-6077, 7864-7940, 8414-8760),
// restated over the C ABI of include/anode_routines_gpu.h.  Header-only; link against
// libanode_routines_gpu and the CUDA runtime.
//
// What maps to what:
//   GPUDeviceOuterBatchArray3d<f32> ([W,H,C] + batch) / 4d ([W,H,D,C] + batch)   ->  anode::DeviceArray
//   WriteCap::{Assign, Accumulate} (src/lib.rs:2160-2165)                          ->  anode::WriteCap
//   conn.cuda_kernel_config()                                                      ->  anode::kernel_config()
//   BatchMean2dOp ... PositiveClipBwdOp `apply` closures                           ->  structs with static apply()
//   x.batch_normalize_2d(axes, online, avg_rate, eps) (src/ops.rs:999-1014)        ->  anode::batch_normalize_2d
//   the adjoint wiring of the three ops (src/ops_gpu.rs:3785-3796, 3994-4005, 4340-4357) -> anode::batch_normalize_adjoint
//   BatchNormalize2dFusedOp / BatchNormalize2dBwdFusedOp (declared, never built: src/ops.rs:105-106) -> same names here
// Error behaviour: the reference's entry points return void and `unimplemented!()` on anything
// that is not packed or not over the leading axes; here that is an anode::Error, as is a negative
// return code of the new entry points.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/anode_routines_gpu.h"

namespace anode {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string &what) : std::runtime_error(what + " (code " + std::to_string(c) + ")"), code(c) {}
};
inline void check(int rc, const char *fn) { if (rc != ANODE_OK) throw Error(rc, fn); }
inline void cuda_check(cudaError_t e, const char *what) { if (e != cudaSuccess) throw Error((int)e, std::string(what) + ": " + cudaGetErrorString(e)); }

enum class WriteCap { Assign, Accumulate };

inline CUstream_st *raw(cudaStream_t s) { return reinterpret_cast<CUstream_st *>(s); }

// The launch hint every reference call receives (`conn.cuda_kernel_config()`): 1024 threads,
// 32 blocks per SM.  The kernels here treat it as a hint; the reductions still insist, like the
// reference (routines_gpu/batch_norm.cu:68), on a power-of-two block size.
inline const KernelConfig *kernel_config()
{
  static KernelConfig cfg = [] {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return KernelConfig{1024u, 32u * (uint32_t)sms};
  }();
  return &cfg;
}

// A packed f32 device array; `size` lists the extents fastest-varying first, the last one being
// the outer batch ([W,H,C,N] or [W,H,D,C,N], byte-identical to contiguous NCHW / NCDHW), or a
// plain vector ([C]).  Owns its memory.
class DeviceArray {
 public:
  DeviceArray() = default;
  explicit DeviceArray(std::vector<uint32_t> size) : size_(std::move(size))
  {
    len_ = 1;
    for (uint32_t s : size_) len_ *= s;
    cuda_check(cudaMalloc(&ptr_, bytes() ? bytes() : 4), "cudaMalloc");
  }
  static DeviceArray zeros(std::vector<uint32_t> size, cudaStream_t s = 0)
  {
    DeviceArray a(std::move(size));
    cuda_check(cudaMemsetAsync(a.ptr_, 0, a.bytes(), s), "cudaMemsetAsync");
    return a;
  }
  static DeviceArray filled(std::vector<uint32_t> size, float v, cudaStream_t s = 0)
  {
    DeviceArray a(std::move(size));
    std::vector<float> h(a.len_, v);
    a.copy_from_host(h.data(), s);
    return a;
  }
  static DeviceArray from_host(std::vector<uint32_t> size, const float *h, cudaStream_t s = 0)
  {
    DeviceArray a(std::move(size));
    a.copy_from_host(h, s);
    return a;
  }
  DeviceArray(DeviceArray &&o) noexcept { *this = std::move(o); }
  DeviceArray &operator=(DeviceArray &&o) noexcept
  {
    if (this != &o) { release(); ptr_ = o.ptr_; len_ = o.len_; size_ = std::move(o.size_); o.ptr_ = nullptr; o.len_ = 0; }
    return *this;
  }
  DeviceArray(const DeviceArray &) = delete;
  DeviceArray &operator=(const DeviceArray &) = delete;
  ~DeviceArray() { release(); }

  float *ptr() { return ptr_; }
  const float *ptr() const { return ptr_; }
  size_t len() const { return len_; }
  size_t bytes() const { return len_ * sizeof(float); }
  const std::vector<uint32_t> &size() const { return size_; }
  bool empty() const { return ptr_ == nullptr; }
  void copy_from_host(const float *h, cudaStream_t s = 0)
  {
    cuda_check(cudaMemcpyAsync(ptr_, h, bytes(), cudaMemcpyHostToDevice, s), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  }
  std::vector<float> to_host(cudaStream_t s = 0) const
  {
    std::vector<float> h(len_);
    cuda_check(cudaMemcpyAsync(h.data(), ptr_, bytes(), cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    return h;
  }

 private:
  void release() { if (ptr_) (void)cudaFree(ptr_); ptr_ = nullptr; }
  float *ptr_ = nullptr;
  size_t len_ = 0;
  std::vector<uint32_t> size_;
};

// dim0, dim1, dim2 as the apply closures compute them from `x.inner().size()`:
// index_cut(3).index_cut(2).flat_len(), index_at(2), index_at(3) for [W,H,C,N]
// (src/ops_gpu.rs:3764-3766); the first three extents flattened for [W,H,D,C,N] (:4911-4913).
struct Dims { uint32_t dim0, dim1, dim2; };
inline Dims dims_of(const DeviceArray &x, const std::vector<int> &axes)
{
  const auto &s = x.size();
  if (s.size() < 3) throw Error(ANODE_E_DIMS, "batch array needs [spatial..., C, N]");
  const size_t spatial = s.size() - 2;
  if (axes.size() != spatial) throw Error(ANODE_E_DIMS, "axes must be the leading spatial axes");     // the reference: unimplemented!()
  for (size_t i = 0; i < spatial; ++i)
    if (axes[i] != (int)i) throw Error(ANODE_E_DIMS, "axes must be the leading spatial axes");
  uint64_t d0 = 1;
  for (size_t i = 0; i < spatial; ++i) d0 *= s[i];
  if (d0 == 0 || d0 >> 32) throw Error(ANODE_E_DIMS, "dim0 out of range");
  return Dims{(uint32_t)d0, s[spatial], s[spatial + 1]};
}
inline void want_len(const DeviceArray &a, size_t n, const char *what) { if (a.len() != n) throw Error(ANODE_E_DIMS, std::string(what) + ": wrong length"); }

// ---- the reference's operators, one launch each --------------------------------------------------
#define ANODE_CAP(cap, fn, ...) do { if ((cap) == WriteCap::Accumulate) fn##_accumulate_f32(__VA_ARGS__); else fn##_f32(__VA_ARGS__); } while (0)

// src/ops_gpu.rs:3690 (2-D), :4858 (3-D): mean[c] = sum(x)/M
struct BatchMean2dOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &x, DeviceArray &mean, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes); want_len(mean, d.dim1, "mean");
    anode_gpu_batch_mean_3d1_packed_f32(d.dim0, d.dim1, d.dim2, x.ptr(), mean.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:3803 / :4950: dx (+)= dmean[c]/M
struct BatchMean2dBwdOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &dmean, DeviceArray &dx, WriteCap cap, cudaStream_t s = 0)
  {
    const Dims d = dims_of(dx, axes); want_len(dmean, d.dim1, "dmean");
    ANODE_CAP(cap, anode_gpu_batch_mean_bwd_3d1_packed, d.dim0, d.dim1, d.dim2, dmean.ptr(), dx.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:3913 / :5060: var[c] = sum((x-mean)^2)/M + epsilon
struct BatchVariance2dOp {
  static void apply(const std::vector<int> &axes, float epsilon, const DeviceArray &x, const DeviceArray &mean, DeviceArray &var,
                    cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes); want_len(mean, d.dim1, "mean"); want_len(var, d.dim1, "var");
    anode_gpu_batch_var_3d1_packed_f32(d.dim0, d.dim1, d.dim2, epsilon, x.ptr(), mean.ptr(), var.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:4012 / :5159: dx (+)= dvar[c]*(x-mean[c])*2/M
struct BatchVariance2dBwdOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &dvar, const DeviceArray &x, const DeviceArray &mean,
                    DeviceArray &dx, WriteCap cap, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes); want_len(dx, x.len(), "dx");
    ANODE_CAP(cap, anode_gpu_batch_var_bwd_3d1_packed, d.dim0, d.dim1, d.dim2, dvar.ptr(), x.ptr(), mean.ptr(), dx.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:4132 / :5279: dmean[c] (+)= sum((x-mean[c])*(-2*dvar[c]))/M
struct BatchVariance2dBwdMeanOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &dvar, const DeviceArray &x, const DeviceArray &mean,
                    DeviceArray &dmean, WriteCap cap, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes); want_len(dmean, d.dim1, "dmean");
    ANODE_CAP(cap, anode_gpu_batch_var_bwd_mean_3d1_packed, d.dim0, d.dim1, d.dim2, dvar.ptr(), x.ptr(), mean.ptr(), dmean.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:4249 / :5396: y = (x-mean[c])*rsqrt(var[c])
struct BatchNormalize2dOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &x, const DeviceArray &mean, const DeviceArray &var,
                    DeviceArray &y, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes); want_len(y, x.len(), "y");
    anode_gpu_batch_norm_3d1_packed_f32(d.dim0, d.dim1, d.dim2, x.ptr(), mean.ptr(), var.ptr(), y.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:4364 / :5511: dx (+)= dy*rsqrt(var[c])
struct BatchNormalize2dBwdOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &dy, const DeviceArray &var, DeviceArray &dx, WriteCap cap,
                    cudaStream_t s = 0)
  {
    const Dims d = dims_of(dy, axes); want_len(dx, dy.len(), "dx");
    ANODE_CAP(cap, anode_gpu_batch_norm_bwd_3d1_packed, d.dim0, d.dim1, d.dim2, dy.ptr(), var.ptr(), dx.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:4476 / :5623: dmean[c] (+)= sum(dy)*(-rsqrt(var[c]))
struct BatchNormalize2dBwdMeanOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &dy, const DeviceArray &var, DeviceArray &dmean, WriteCap cap,
                    cudaStream_t s = 0)
  {
    const Dims d = dims_of(dy, axes); want_len(dmean, d.dim1, "dmean");
    ANODE_CAP(cap, anode_gpu_batch_norm_bwd_mean_3d1_packed, d.dim0, d.dim1, d.dim2, dy.ptr(), var.ptr(), dmean.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:4586 / :5733: dvar[c] (+)= sum(dy*(x-mean[c]))*(-0.5*rsqrt(var[c])/var[c]); _v2 from the saved y
struct BatchNormalize2dBwdVarianceOp {
  static void apply(const std::vector<int> &axes, const DeviceArray &dy, const DeviceArray &x, const DeviceArray &mean,
                    const DeviceArray &var, DeviceArray &dvar, WriteCap cap, cudaStream_t s = 0)
  {
    const Dims d = dims_of(x, axes); want_len(dvar, d.dim1, "dvar");
    ANODE_CAP(cap, anode_gpu_batch_norm_bwd_var_3d1_packed, d.dim0, d.dim1, d.dim2, dy.ptr(), x.ptr(), mean.ptr(), var.ptr(), dvar.ptr(), kernel_config(), raw(s));
  }
  static void apply_v2(const std::vector<int> &axes, const DeviceArray &dy, const DeviceArray &y, const DeviceArray &var,
                       DeviceArray &dvar, WriteCap cap, cudaStream_t s = 0)
  {
    const Dims d = dims_of(y, axes); want_len(dvar, d.dim1, "dvar");
    ANODE_CAP(cap, anode_gpu_batch_norm_bwd_var_v2_3d1_packed, d.dim0, d.dim1, d.dim2, dy.ptr(), y.ptr(), var.ptr(), dvar.ptr(), kernel_config(), raw(s));
  }
};
#undef ANODE_CAP
using BatchMean3dOp = BatchMean2dOp;
using BatchMean3dBwdOp = BatchMean2dBwdOp;
using BatchVariance3dOp = BatchVariance2dOp;
using BatchVariance3dBwdOp = BatchVariance2dBwdOp;
using BatchVariance3dBwdMeanOp = BatchVariance2dBwdMeanOp;
using BatchNormalize3dOp = BatchNormalize2dOp;
using BatchNormalize3dBwdOp = BatchNormalize2dBwdOp;
using BatchNormalize3dBwdMeanOp = BatchNormalize2dBwdMeanOp;
using BatchNormalize3dBwdVarianceOp = BatchNormalize2dBwdVarianceOp;

// src/ops_gpu.rs:6034-6077; rule pinned by tests/test_gpu.rs:561-593: y += rate*(x - y)
struct OnlineAverageOp {
  static void apply(float avg_rate, const DeviceArray &x, DeviceArray &y, cudaStream_t s = 0)
  {
    want_len(y, x.len(), "y");
    check(anode_gpu_online_average_f32((uint32_t)x.len(), avg_rate, x.ptr(), y.ptr(), kernel_config(), raw(s)), "anode_gpu_online_average_f32");
  }
};
// src/ops_gpu.rs:8414 (and the in-place PositiveClipClobberOp, :8584): y = x*(x > 0)
struct PositiveClipOp {
  static void apply(const DeviceArray &x, DeviceArray &y, cudaStream_t s = 0)
  {
    want_len(y, x.len(), "y");
    anode_gpu_positive_clip_flat_map_f32((uint32_t)x.len(), x.ptr(), y.ptr(), kernel_config(), raw(s));
  }
};
// src/ops_gpu.rs:8499, :8673: dx = dy*(y > 0)
struct PositiveClipBwdOp {
  static void apply(const DeviceArray &dy, const DeviceArray &y, DeviceArray &dx, cudaStream_t s = 0)
  {
    want_len(dx, dy.len(), "dx");
    anode_gpu_positive_clip_flat_map_bwd_f32((uint32_t)dy.len(), dy.ptr(), y.ptr(), dx.ptr(), kernel_config(), raw(s));
  }
};

}  // namespace anode

#include "anode_layers.hpp"
