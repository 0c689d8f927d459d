// Batch-norm with given statistics fused with the activation that follows it: the inference branch
// of batch_normalize_2d/3d (src/ops.rs:1010-1011: `switch(online, avg_mean, mean)` feeding
// BatchNormalize2dOp, evaluation loop examples/run_imagenet_mpi.rs:841-843) followed by
// positive_clip (routines_gpu/flat_map.cu:172-179) or leaky ReLU (flat_map.cu:44-52), in one pass:
//
//   y = act(gamma[c]*(x - mean[c])*var[c]^-1/2 + beta[c]),   act(t) = t * (t > 0 ? 1 : neg_slope)
//
// (var is what anode stores: biased variance + epsilon.)  One read and one write of the tensor:
// 8 bytes per element, HBM-bound.  A thread owns one 16-byte column of the sample (its channel
// never changes), computes its coefficients once and walks down the samples.
#include "bn_device.cuh"
#include "bn_host.h"

namespace anode_b200 {

constexpr uint32_t kInferThreads = 256;

template <int VEC>
__global__ void __launch_bounds__(kInferThreads) bn_infer_kernel(uint32_t dim0, uint32_t C, uint32_t N, float neg_slope,
                                                                 const float *__restrict__ x, const float *__restrict__ mean,
                                                                 const float *__restrict__ var, const float *__restrict__ gamma,
                                                                 const float *__restrict__ beta, float *y)
{
  const uint64_t per_sample = (uint64_t)C * dim0;                 // floats
  const uint64_t col = ((uint64_t)blockIdx.x * kInferThreads + threadIdx.x) * VEC;
  if (col >= per_sample) return;
  // channel of each of this thread's elements, and its coefficients
  uint32_t c = (uint32_t)(col / dim0), off = (uint32_t)(col - (uint64_t)c * dim0);
  float sc[VEC], sh[VEC], mu[VEC];
  uint32_t prev = 0xffffffffu;
  float s0 = 0.f, b0 = 0.f, m0 = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    if (c != prev) {
      const float g = gamma ? gamma[c] : 1.0f;
      m0 = mean[c]; s0 = g * inv_std(var[c]); b0 = (gamma && beta) ? beta[c] : 0.0f;
      prev = c;
    }
    mu[i] = m0; sc[i] = s0; sh[i] = b0;
    if (++off == dim0) { off = 0; ++c; }
  }
  for (uint32_t n = blockIdx.y; n < N; n += gridDim.y) {
    const size_t at = (size_t)n * per_sample + col;
    Pack<VEC> p = Pack<VEC>::load(x + at);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float t = fmaf(p.v[i] - mu[i], sc[i], sh[i]);
      p.v[i] = t * (t > 0.0f ? 1.0f : neg_slope);
    }
    p.store_stream(y + at);
  }
}

}  // namespace anode_b200

using namespace anode_b200;

extern "C" int anode_gpu_batch_norm_act_infer_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float neg_slope,
    const float *x, const float *mean, const float *var, const float *gamma, const float *beta,
    float *y, const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  const int rc = check_dims(dim0, dim1, dim2);
  if (rc) return rc;
  if (!x || !y || !mean || !var) return ANODE_E_NULL;
  if (!aligned4(x) || !aligned4(y)) return ANODE_E_ALIGN;
  const uint64_t per_sample = (uint64_t)dim1 * dim0;
  const bool vec = aligned16(x) && aligned16(y) && per_sample % 4 == 0;
  const uint64_t cols = vec ? per_sample / 4 : per_sample;
  const uint64_t bx = (cols + kInferThreads - 1) / kInferThreads;
  if (bx > 0x7fffffffull) return ANODE_E_DIMS;
  // enough blocks to fill the device a few times over; the rest of the samples are walked in the loop
  const uint64_t want = (uint64_t)sm_count() * 32;
  uint64_t by = (want + bx - 1) / bx;
  if (by > dim2) by = dim2;
  if (by > 65535) by = 65535;
  if (by < 1) by = 1;
  const dim3 grid((unsigned)bx, (unsigned)by);
  if (vec) bn_infer_kernel<4><<<grid, kInferThreads, 0, stream>>>(dim0, dim1, dim2, neg_slope, x, mean, var, gamma, beta, y);
  else bn_infer_kernel<1><<<grid, kInferThreads, 0, stream>>>(dim0, dim1, dim2, neg_slope, x, mean, var, gamma, beta, y);
  if (cudaGetLastError() != cudaSuccess) return ANODE_E_LAUNCH;
  return ANODE_OK;
}
