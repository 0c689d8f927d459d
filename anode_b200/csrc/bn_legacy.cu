// The reference's own batch-norm / ReLU entry points (routines_gpu/lib.h:32-193, 296-302,
// 344-356), re-implemented for sm_100a with the same names, signatures and results:
//
//   per-channel reductions   one thread-block cluster per channel; 128-bit loads, register
//                            accumulation, warp shuffles, then a distributed-shared-memory
//                            gather of the cluster's block sums, added in a fixed order
//   elementwise kernels      128-bit grid-stride loops; the channel of a vector comes from one
//                            division per four elements instead of two per element
//
// Expressions are kept term for term as the reference writes them (e.g. rsqrtf, the
// "* 2.0f / norm" order), so results differ from its kernels only by summation order.
#include <cooperative_groups.h>

#include "bn_host.h"

namespace cg = cooperative_groups;

namespace anode_b200 {

constexpr int kRedThreads = 512;
constexpr int kClusterMax = 8;

struct Assign { __device__ __forceinline__ static float w(float old, float v) { return v; } static constexpr bool reads = false; };
struct Accumulate { __device__ __forceinline__ static float w(float old, float v) { return old + v; } static constexpr bool reads = true; };

// KIND: 0 x | 1 (x-m)^2 | 2 (x-m)*t | 3 a*t | 4 a*(b-m)*t | 5 -a*b*0.5f/t
template <int KIND>
__device__ __forceinline__ float red_term(float a, float b, float m, float t)
{
  if (KIND == 0) return a;
  if (KIND == 1) return (a - m) * (a - m);
  if (KIND == 2) return (a - m) * t;
  if (KIND == 3) return a * t;
  if (KIND == 4) return a * (b - m) * t;
  return -a * b * 0.5f / t;
}

struct RedArgs {
  uint32_t dim0, C, N;
  float epsilon;
  const float *a, *b;          // streamed tensors (b only for KIND 4, 5)
  const float *p_mean, *p_var, *p_dvar;   // per-channel inputs
  float *out;
};

template <int KIND, int VEC, typename Write>
__global__ void __launch_bounds__(kRedThreads) legacy_reduce_kernel(const RedArgs g)
{
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t cs = cluster.num_blocks(), rank = cluster.block_rank();
  const uint32_t c = blockIdx.x / cs;
  __shared__ double gather[kClusterMax];
  __shared__ double warp_part[kRedThreads / 32];

  float m = 0.f, t = 0.f;
  if (KIND == 1 || KIND == 2 || KIND == 4) m = g.p_mean[c];
  if (KIND == 2) t = -g.p_dvar[c] * 2.0f;                               // batch_norm.cu:255
  if (KIND == 3) t = -rsqrtf(g.p_var[c]);                               // batch_norm.cu:420
  if (KIND == 4) { const float v = g.p_var[c]; t = -0.5f * rsqrtf(v) / v; }   // batch_norm.cu:492
  if (KIND == 5) t = g.p_var[c];

  const uint32_t per_row = g.dim0 / VEC;
  const uint64_t total = (uint64_t)per_row * g.N;
  const uint64_t rs = (uint64_t)g.C * g.dim0;
  const float *pa = g.a + (size_t)c * g.dim0;
  const float *pb = (KIND >= 4) ? g.b + (size_t)c * g.dim0 : nullptr;
  float acc[2] = {0.f, 0.f};
  const uint64_t stride = (uint64_t)cs * kRedThreads;
  for (uint64_t j = (uint64_t)rank * kRedThreads + threadIdx.x; j < total; j += 2 * stride) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint64_t jj = j + u * stride;
      if (jj < total) {
        const uint32_t row = (uint32_t)(jj / per_row), col = (uint32_t)(jj - (uint64_t)row * per_row);
        const size_t off = (size_t)row * rs + (size_t)col * VEC;
        const Pack<VEC> va = Pack<VEC>::load(pa + off);
        Pack<VEC> vb = va;
        if (KIND >= 4) vb = Pack<VEC>::load(pb + off);
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[u] += red_term<KIND>(va.v[i], vb.v[i], m, t);
      }
    }
  }
  double s = (double)acc[0] + (double)acc[1];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double bs = 0.0;
#pragma unroll
    for (int w = 0; w < kRedThreads / 32; ++w) bs += warp_part[w];
    double *dst = cluster.map_shared_rank(gather, 0);      // block 0's shared memory
    dst[rank] = bs;
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    double tot = 0.0;
    for (uint32_t r = 0; r < cs; ++r) tot += gather[r];
    const float sum = (float)tot;
    const float norm = ((float)g.dim0) * ((float)g.N);
    float val;
    if (KIND == 0) val = sum / norm;                       // batch_norm.cu:54
    else if (KIND == 1) val = sum / norm + g.epsilon;      // batch_norm.cu:160
    else if (KIND == 2) val = sum / norm;                  // batch_norm.cu:277
    else val = sum;
    g.out[c] = Write::w(Write::reads ? g.out[c] : 0.f, val);
  }
}

template <int KIND, typename Write>
static void launch_reduce(const RedArgs &g, cudaStream_t stream)
{
  if (g.dim0 == 0 || g.C == 0 || g.N == 0) return;
  const bool vec = (g.dim0 % 4 == 0) && aligned16(g.a) && (KIND < 4 || aligned16(g.b));
  // enough clusters to fill the GPU: C channels x cs blocks, cs a power of two <= 8
  const uint64_t per_channel = (uint64_t)g.dim0 * g.N;
  uint32_t cs = 1;
  while (cs < (uint32_t)kClusterMax && (uint64_t)g.C * cs < 2ull * sm_count() &&
         per_channel / (cs * 2) >= (uint64_t)kRedThreads * 8)
    cs *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g.C * cs);
  cfg.blockDim = dim3(kRedThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (vec) (void)cudaLaunchKernelEx(&cfg, legacy_reduce_kernel<KIND, 4, Write>, g);
  else (void)cudaLaunchKernelEx(&cfg, legacy_reduce_kernel<KIND, 1, Write>, g);
}

// ---- elementwise --------------------------------------------------------------------------
// OP: 0 mean_bwd | 1 var_bwd | 2 norm | 3 norm_bwd | 4 positive_clip | 5 positive_clip_bwd / flat join
struct MapArgs {
  uint32_t dim0, C;
  uint64_t len;
  float norm;
  const float *a, *b;       // streamed inputs
  const float *p0, *p1;     // per-channel inputs
  float *out;
};

template <int OP, int VEC, typename Write>
__global__ void __launch_bounds__(256) legacy_map_kernel(const MapArgs g)
{
  const uint64_t nvec = g.len / VEC;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < nvec; j += stride) {
    const size_t off = (size_t)j * VEC;
    float k0 = 0.f, k1 = 0.f;
    if (OP <= 3) {
      const uint32_t c = (uint32_t)((off / g.dim0) % g.C);    // Index3::Unpack (common.cuh:96-105)
      if (OP == 0) k0 = g.p0[c] / g.norm;                     // dmean[c] / norm1   (batch_norm.cu:92)
      if (OP == 1) { k0 = g.p0[c]; k1 = g.p1[c]; }            // dvar[c], mean[c]   (batch_norm.cu:203)
      if (OP == 2) { k0 = g.p0[c]; k1 = rsqrtf(g.p1[c]); }    // mean[c], rsqrt(var[c]) (batch_norm.cu:333)
      if (OP == 3) k0 = rsqrtf(g.p0[c]);                      // rsqrt(var[c])      (batch_norm.cu:373)
    }
    Pack<VEC> va, vb, vo;
    if (OP != 0) va = Pack<VEC>::load(g.a + off);
    if (OP == 5) vb = Pack<VEC>::load(g.b + off);
    if (Write::reads) vo = Pack<VEC>::load(g.out + off);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float v;
      if (OP == 0) v = k0;
      else if (OP == 1) v = k0 * (va.v[i] - k1) * 2.0f / g.norm;
      else if (OP == 2) v = (va.v[i] - k0) * k1;
      else if (OP == 3) v = va.v[i] * k0;
      else if (OP == 4) v = positive_clip(va.v[i]);
      else v = va.v[i] * (vb.v[i] > 0.0f ? 1.0f : 0.0f);     // flat_map.cu:191-192, flat_join.cu:33-35
      vo.v[i] = Write::w(Write::reads ? vo.v[i] : 0.f, v);
    }
    if (VEC == 4) *reinterpret_cast<float4 *>(g.out + off) = make_float4(vo.v[0], vo.v[1 % VEC], vo.v[2 % VEC], vo.v[3 % VEC]);
    else g.out[off] = vo.v[0];
  }
}

template <int OP, typename Write>
static void launch_map(const MapArgs &g, cudaStream_t stream)
{
  if (g.len == 0) return;
  bool vec = (g.len % 4 == 0) && aligned16(g.out) && (OP == 0 || aligned16(g.a)) && (OP != 5 || aligned16(g.b));
  if (OP <= 3) vec = vec && (g.dim0 % 4 == 0);
  const uint64_t nvec = vec ? g.len / 4 : g.len;
  const uint64_t want = (nvec + 255) / 256;
  const uint32_t cap = sm_count() * 16;
  const uint32_t blocks = (uint32_t)(want < cap ? want : cap);
  if (vec) legacy_map_kernel<OP, 4, Write><<<blocks, 256, 0, stream>>>(g);
  else legacy_map_kernel<OP, 1, Write><<<blocks, 256, 0, stream>>>(g);
}

static void check_cfg(const KernelConfig *cfg)
{
  // The reference's reduce kernels require a power-of-two block size (batch_norm.cu:68).  The
  // kernels here do not depend on it, so a violating hint is simply not used.
  (void)cfg;
}

}  // namespace anode_b200

using namespace anode_b200;

#define ANODE_RED(KIND, WRITE, ...)                                    \
  do {                                                                 \
    check_cfg(cfg);                                                    \
    RedArgs g = {};                                                    \
    g.dim0 = dim0; g.C = dim1; g.N = dim2;                             \
    __VA_ARGS__;                                                       \
    launch_reduce<KIND, WRITE>(g, stream);                             \
  } while (0)

#define ANODE_MAP(OP, WRITE, ...)                                      \
  do {                                                                 \
    MapArgs g = {};                                                    \
    g.dim0 = dim0; g.C = dim1;                                         \
    g.len = (uint64_t)dim0 * dim1 * dim2;                              \
    g.norm = ((float)dim0) * ((float)dim2);                            \
    __VA_ARGS__;                                                       \
    launch_map<OP, WRITE>(g, stream);                                  \
  } while (0)

extern "C" {

void anode_gpu_batch_mean_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *x, float *mean,
                                         const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(0, Assign, g.a = x; g.out = mean); }

void anode_gpu_batch_mean_bwd_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dmean, float *dx,
                                             const KernelConfig *cfg, CUstream_st *stream)
{ (void)cfg; ANODE_MAP(0, Assign, g.p0 = dmean; g.out = dx); }

void anode_gpu_batch_mean_bwd_3d1_packed_accumulate_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dmean,
                                                        float *dx, const KernelConfig *cfg, CUstream_st *stream)
{ (void)cfg; ANODE_MAP(0, Accumulate, g.p0 = dmean; g.out = dx); }

void anode_gpu_batch_var_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, const float *x,
                                        const float *mean, float *var, const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(1, Assign, g.epsilon = epsilon; g.a = x; g.p_mean = mean; g.out = var); }

void anode_gpu_batch_var_bwd_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dvar, const float *x,
                                            const float *mean, float *dx, const KernelConfig *cfg, CUstream_st *stream)
{ (void)cfg; ANODE_MAP(1, Assign, g.a = x; g.p0 = dvar; g.p1 = mean; g.out = dx); }

void anode_gpu_batch_var_bwd_3d1_packed_accumulate_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dvar,
                                                       const float *x, const float *mean, float *dx,
                                                       const KernelConfig *cfg, CUstream_st *stream)
{ (void)cfg; ANODE_MAP(1, Accumulate, g.a = x; g.p0 = dvar; g.p1 = mean; g.out = dx); }

void anode_gpu_batch_var_bwd_mean_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dvar,
                                                 const float *x, const float *mean, float *dmean,
                                                 const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(2, Assign, g.a = x; g.p_mean = mean; g.p_dvar = dvar; g.out = dmean); }

void anode_gpu_batch_var_bwd_mean_3d1_packed_accumulate_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dvar,
                                                            const float *x, const float *mean, float *dmean,
                                                            const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(2, Accumulate, g.a = x; g.p_mean = mean; g.p_dvar = dvar; g.out = dmean); }

void anode_gpu_batch_norm_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *x, const float *mean,
                                         const float *var, float *y, const KernelConfig *cfg, CUstream_st *stream)
{ (void)cfg; ANODE_MAP(2, Assign, g.a = x; g.p0 = mean; g.p1 = var; g.out = y); }

void anode_gpu_batch_norm_bwd_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy, const float *var,
                                             float *dx, const KernelConfig *cfg, CUstream_st *stream)
{ (void)cfg; ANODE_MAP(3, Assign, g.a = dy; g.p0 = var; g.out = dx); }

void anode_gpu_batch_norm_bwd_3d1_packed_accumulate_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy,
                                                        const float *var, float *dx, const KernelConfig *cfg,
                                                        CUstream_st *stream)
{ (void)cfg; ANODE_MAP(3, Accumulate, g.a = dy; g.p0 = var; g.out = dx); }

void anode_gpu_batch_norm_bwd_mean_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy,
                                                  const float *var, float *dmean, const KernelConfig *cfg,
                                                  CUstream_st *stream)
{ ANODE_RED(3, Assign, g.a = dy; g.p_var = var; g.out = dmean); }

void anode_gpu_batch_norm_bwd_mean_3d1_packed_accumulate_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy,
                                                             const float *var, float *dmean, const KernelConfig *cfg,
                                                             CUstream_st *stream)
{ ANODE_RED(3, Accumulate, g.a = dy; g.p_var = var; g.out = dmean); }

void anode_gpu_batch_norm_bwd_var_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy, const float *x,
                                                 const float *mean, const float *var, float *dvar,
                                                 const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(4, Assign, g.a = dy; g.b = x; g.p_mean = mean; g.p_var = var; g.out = dvar); }

void anode_gpu_batch_norm_bwd_var_3d1_packed_accumulate_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy,
                                                            const float *x, const float *mean, const float *var,
                                                            float *dvar, const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(4, Accumulate, g.a = dy; g.b = x; g.p_mean = mean; g.p_var = var; g.out = dvar); }

void anode_gpu_batch_norm_bwd_var_v2_3d1_packed_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy,
                                                    const float *y, const float *var, float *dvar,
                                                    const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(5, Assign, g.a = dy; g.b = y; g.p_var = var; g.out = dvar); }

void anode_gpu_batch_norm_bwd_var_v2_3d1_packed_accumulate_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, const float *dy,
                                                               const float *y, const float *var, float *dvar,
                                                               const KernelConfig *cfg, CUstream_st *stream)
{ ANODE_RED(5, Accumulate, g.a = dy; g.b = y; g.p_var = var; g.out = dvar); }

void anode_gpu_M1_copy_map_M2_unit_step_map_R_product_reduce_flat_join_f32(uint32_t len, const float *x1, const float *x2,
                                                                           float *y, const KernelConfig *cfg,
                                                                           CUstream_st *stream)
{
  (void)cfg;
  const uint32_t dim0 = len, dim1 = 1, dim2 = 1;
  ANODE_MAP(5, Assign, g.a = x1; g.b = x2; g.out = y);
}

void anode_gpu_positive_clip_flat_map_f32(uint32_t len, const float *x, float *y, const KernelConfig *cfg, CUstream_st *stream)
{
  (void)cfg;
  const uint32_t dim0 = len, dim1 = 1, dim2 = 1;
  ANODE_MAP(4, Assign, g.a = x; g.out = y);
}

void anode_gpu_positive_clip_flat_map_bwd_f32(uint32_t len, const float *dy, const float *y, float *dx,
                                              const KernelConfig *cfg, CUstream_st *stream)
{
  (void)cfg;
  const uint32_t dim0 = len, dim1 = 1, dim2 = 1;
  ANODE_MAP(5, Assign, g.a = dy; g.b = y; g.out = dx);
}

}  // extern "C"
