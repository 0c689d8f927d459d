/*
 * CPU oracle for anode's train-mode batch-norm + ReLU path.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are compared
 * against and the timed CPU baseline; nothing in the shipped library calls it.
 *
 * It restates, as plain C loops, the arithmetic of the reference's CUDA kernels
 * (paths are relative to the reference project root):
 *   routines_gpu/batch_norm.cu   the ten batch-norm kernels
 *   routines_gpu/flat_map.cu     positive_clip forward / backward (ReLU)
 *   routines_gpu/flat_join.cu    x1 * step(x2)
 *   routines_gpu/common.cuh      Index2/Index3 packing, Assign/Accumulate writers
 *   routines_gpu/common_reduce.cuh  the shared-memory tree reduction
 *   src/ops.rs:999-1014          batch_normalize_2d composition
 *   tests/test_gpu.rs:561-593    running-average rule  y <- y + r*(x - y)
 *
 * Layout everywhere: element (i0, c, n) of a [dim0, dim1=C, dim2=N] packed array sits at
 * i0 + dim0*(c + dim1*n)  (common.cuh:88-94), i.e. contiguous NCHW / NCDHW.
 *
 * Two flavours:
 *   *_f32   "literal": f32 arithmetic in the reference's own order.  Reductions can
 *           replay the reference's summation tree exactly (block_sz > 0): chunks of
 *           block_sz values are tree-reduced in "shared memory" and thread 0 adds each
 *           chunk total to a serial accumulator (batch_norm.cu:35-53).  With block_sz = 0
 *           a fast blocked summation is used instead (the timed CPU baseline).
 *   *_f64   "truth": the same formulas in double precision.
 *
 * Pinning: the running-average rule is checked against the reference's known-answer
 * test (0 -> 0.25 -> 0.4375 at rate 0.25).  Batch-norm itself has no golden vector in
 * the reference; the literal flavour is pinned by running the reference's own kernels
 * (compiled from its sources into oracle/_ref) on a GPU and comparing.  The gamma/beta
 * affine has no reference implementation at all: parity unpinned for gamma, beta,
 * dgamma, dbeta (they follow the standard composition and are checked against f64).
 *
 * Build: see oracle/Makefile (gcc -O3 -march=x86-64-v3 -fopenmp -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static inline size_t pack3(uint32_t i0, uint32_t dim0, uint32_t c, uint32_t dim1, uint32_t n)
{
  /* common.cuh:88-94 (Index3::Pack) */
  return (size_t)i0 + (size_t)dim0 * ((size_t)c + (size_t)dim1 * (size_t)n);
}

ORACLE_API int oracle_num_threads(void)
{
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------------------
 * Per-channel reduction of term(i) over the fused (i0, n) index, in the reference's order.
 *
 * kind selects the summand (each is one reference kernel's inner expression):
 *   0  x                                   batch_norm.cu:42       (mean)
 *   1  (x-m)*(x-m)                         batch_norm.cu:146-147  (var)
 *   2  (x-m)*t                             batch_norm.cu:259      (var_bwd_mean, t=-2*dvar)
 *   3  dy*t                                batch_norm.cu:423      (norm_bwd_mean, t=-rsqrt(v))
 *   4  dy*(x-m)*t                          batch_norm.cu:494      (norm_bwd_var)
 *   5  -dy*y*0.5f/v                        batch_norm.cu:570      (norm_bwd_var_v2; a=dy, b=y)
 * ---------------------------------------------------------------------------------- */
static inline float term_f32(int kind, const float *a, const float *b, size_t idx, float m, float t)
{
  switch (kind) {
    case 0: return a[idx];
    case 1: { float xi = a[idx]; return (xi - m) * (xi - m); }
    case 2: return (a[idx] - m) * t;
    case 3: return a[idx] * t;
    case 4: return a[idx] * (b[idx] - m) * t;
    default: return -a[idx] * b[idx] * 0.5f / t;
  }
}

static float reduce_channel_f32(int kind, uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t c,
                                const float *a, const float *b, float m, float t,
                                uint32_t block_sz, float *cache)
{
  const size_t fused = (size_t)dim0 * dim2;
  if (block_sz > 0) {
    /* literal replay: batch_norm.cu:35-53 + common_reduce.cuh:22-31 */
    float acc = 0.0f;
    for (size_t base = 0; base < fused; base += block_sz) {
      for (uint32_t th = 0; th < block_sz; ++th) {
        size_t i = base + th;
        if (i < fused) {
          uint32_t i0 = (uint32_t)(i % dim0), i2 = (uint32_t)(i / dim0); /* Index2::Unpack */
          cache[th] = term_f32(kind, a, b, pack3(i0, dim0, c, dim1, i2), m, t);
        } else {
          cache[th] = 0.0f;
        }
      }
      for (uint32_t s = block_sz >> 1; s > 0; s >>= 1)
        for (uint32_t th = 0; th < s; ++th)
          if (s + th < block_sz) cache[th] += cache[s + th];
      acc += cache[0];
    }
    return acc;
  }
  /* fast flavour: 16 interleaved f32 lanes per row, rows added into a double */
  double acc = 0.0;
  for (uint32_t n = 0; n < dim2; ++n) {
    const size_t row = pack3(0, dim0, c, dim1, n);
    float lane[16];
    for (int k = 0; k < 16; ++k) lane[k] = 0.0f;
    uint32_t i0 = 0;
    for (; i0 + 16 <= dim0; i0 += 16)
      for (int k = 0; k < 16; ++k) lane[k] += term_f32(kind, a, b, row + i0 + k, m, t);
    for (; i0 < dim0; ++i0) lane[i0 & 15] += term_f32(kind, a, b, row + i0, m, t);
    float s = 0.0f;
    for (int k = 0; k < 16; ++k) s += lane[k];
    acc += (double)s;
  }
  return (float)acc;
}

static float *alloc_cache(uint32_t block_sz)
{
  return (float *)malloc(sizeof(float) * (block_sz ? block_sz : 1));
}

/* rsqrtf of the reference is the device intrinsic (<= 2 ulp); 1/sqrtf is its CPU stand-in. */
static inline float rsqrt_f32(float v) { return 1.0f / sqrtf(v); }

/* ---- forward statistics ---------------------------------------------------------- */

/* batch_norm.cu:24-57: mean[c] = sum(x) / (dim0*dim2) */
ORACLE_API void oracle_batch_mean_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                      const float *x, float *mean, uint32_t block_sz)
{
  const float norm1 = ((float)dim0) * ((float)dim2);
#pragma omp parallel
  {
    float *cache = alloc_cache(block_sz);
#pragma omp for schedule(dynamic, 1)
    for (uint32_t c = 0; c < dim1; ++c)
      mean[c] = reduce_channel_f32(0, dim0, dim1, dim2, c, x, NULL, 0.f, 0.f, block_sz, cache) / norm1;
    free(cache);
  }
}

/* batch_norm.cu:125-163: var[c] = sum((x-mean)^2) / (dim0*dim2) + epsilon  (biased, eps folded in) */
ORACLE_API void oracle_batch_var_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon,
                                     const float *x, const float *mean, float *var, uint32_t block_sz)
{
  const float norm2 = ((float)dim0) * ((float)dim2);
#pragma omp parallel
  {
    float *cache = alloc_cache(block_sz);
#pragma omp for schedule(dynamic, 1)
    for (uint32_t c = 0; c < dim1; ++c)
      var[c] = reduce_channel_f32(1, dim0, dim1, dim2, c, x, NULL, mean[c], 0.f, block_sz, cache) / norm2 + epsilon;
    free(cache);
  }
}

/* ---- backward reductions (accumulate != 0 selects the AccumulateWrite twin) --------- */

static inline void write_f32(float *dst, float val, int accumulate)
{
  /* common.cuh:171-193 */
  *dst = accumulate ? (*dst + val) : val;
}

/* batch_norm.cu:240-280: dmean[c] (+)= sum((x-mean)*(-2*dvar)) / (dim0*dim2) */
ORACLE_API void oracle_batch_var_bwd_mean_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                              const float *dvar, const float *x, const float *mean,
                                              float *dmean, int accumulate, uint32_t block_sz)
{
  const float norm2 = ((float)dim0) * ((float)dim2);
#pragma omp parallel
  {
    float *cache = alloc_cache(block_sz);
#pragma omp for schedule(dynamic, 1)
    for (uint32_t c = 0; c < dim1; ++c) {
      float dv_term = -dvar[c] * 2.0f;
      float acc = reduce_channel_f32(2, dim0, dim1, dim2, c, x, NULL, mean[c], dv_term, block_sz, cache);
      write_f32(&dmean[c], acc / norm2, accumulate);
    }
    free(cache);
  }
}

/* batch_norm.cu:408-444: dmean[c] (+)= sum(dy * (-rsqrt(var))) */
ORACLE_API void oracle_batch_norm_bwd_mean_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                               const float *dy, const float *var,
                                               float *dmean, int accumulate, uint32_t block_sz)
{
#pragma omp parallel
  {
    float *cache = alloc_cache(block_sz);
#pragma omp for schedule(dynamic, 1)
    for (uint32_t c = 0; c < dim1; ++c) {
      float v_term = -rsqrt_f32(var[c]);
      float acc = reduce_channel_f32(3, dim0, dim1, dim2, c, dy, NULL, 0.f, v_term, block_sz, cache);
      write_f32(&dmean[c], acc, accumulate);
    }
    free(cache);
  }
}

/* batch_norm.cu:476-515: dvar[c] (+)= sum(dy*(x-mean)*(-0.5*rsqrt(var)/var)) */
ORACLE_API void oracle_batch_norm_bwd_var_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                              const float *dy, const float *x, const float *mean,
                                              const float *var, float *dvar, int accumulate,
                                              uint32_t block_sz)
{
#pragma omp parallel
  {
    float *cache = alloc_cache(block_sz);
#pragma omp for schedule(dynamic, 1)
    for (uint32_t c = 0; c < dim1; ++c) {
      float v = var[c];
      float v_term = -0.5f * rsqrt_f32(v) / v;
      float acc = reduce_channel_f32(4, dim0, dim1, dim2, c, dy, x, mean[c], v_term, block_sz, cache);
      write_f32(&dvar[c], acc, accumulate);
    }
    free(cache);
  }
}

/* batch_norm.cu:551-587: dvar[c] (+)= sum(-dy*y*0.5/var), y being the normalized output */
ORACLE_API void oracle_batch_norm_bwd_var_v2_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                                 const float *dy, const float *y, const float *var,
                                                 float *dvar, int accumulate, uint32_t block_sz)
{
#pragma omp parallel
  {
    float *cache = alloc_cache(block_sz);
#pragma omp for schedule(dynamic, 1)
    for (uint32_t c = 0; c < dim1; ++c) {
      float acc = reduce_channel_f32(5, dim0, dim1, dim2, c, dy, y, 0.f, var[c], block_sz, cache);
      write_f32(&dvar[c], acc, accumulate);
    }
    free(cache);
  }
}

/* ---- elementwise kernels --------------------------------------------------------- */

/* batch_norm.cu:314-336: y = (x - mean[c]) * rsqrt(var[c]) */
ORACLE_API void oracle_batch_norm_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                      const float *x, const float *mean, const float *var, float *y)
{
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t n = 0; n < dim2; ++n)
    for (uint32_t c = 0; c < dim1; ++c) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      const float m = mean[c], r = rsqrt_f32(var[c]);
      for (uint32_t i0 = 0; i0 < dim0; ++i0) y[row + i0] = (x[row + i0] - m) * r;
    }
}

/* batch_norm.cu:354-376: dx (+)= dy * rsqrt(var[c]) */
ORACLE_API void oracle_batch_norm_bwd_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                          const float *dy, const float *var, float *dx, int accumulate)
{
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t n = 0; n < dim2; ++n)
    for (uint32_t c = 0; c < dim1; ++c) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      const float r = rsqrt_f32(var[c]);
      for (uint32_t i0 = 0; i0 < dim0; ++i0) write_f32(&dx[row + i0], dy[row + i0] * r, accumulate);
    }
}

/* batch_norm.cu:181-206: dx (+)= dvar[c] * (x - mean[c]) * 2 / (dim0*dim2) */
ORACLE_API void oracle_batch_var_bwd_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                         const float *dvar, const float *x, const float *mean,
                                         float *dx, int accumulate)
{
  const float norm2 = ((float)dim0) * ((float)dim2);
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t n = 0; n < dim2; ++n)
    for (uint32_t c = 0; c < dim1; ++c) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      const float dv = dvar[c], m = mean[c];
      for (uint32_t i0 = 0; i0 < dim0; ++i0)
        write_f32(&dx[row + i0], dv * (x[row + i0] - m) * 2.0f / norm2, accumulate);
    }
}

/* batch_norm.cu:73-95: dx (+)= dmean[c] / (dim0*dim2) */
ORACLE_API void oracle_batch_mean_bwd_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                          const float *dmean, float *dx, int accumulate)
{
  const float norm1 = ((float)dim0) * ((float)dim2);
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t n = 0; n < dim2; ++n)
    for (uint32_t c = 0; c < dim1; ++c) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      const float val = dmean[c] / norm1;
      for (uint32_t i0 = 0; i0 < dim0; ++i0) write_f32(&dx[row + i0], val, accumulate);
    }
}

/* flat_map.cu:172-179: y = x * (float)(x > 0)   (in place allowed) */
ORACLE_API void oracle_positive_clip_f32(size_t len, const float *x, float *y)
{
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < len; ++i) {
    float xi = x[i];
    y[i] = xi * ((float)(xi > 0.0f));
  }
}

/* flat_map.cu:187-194: dx = dy * (float)(y > 0) ; flat_join.cu:28-36 is the same expression
 * with (x1, x2) = (dy, y). */
ORACLE_API void oracle_positive_clip_bwd_f32(size_t len, const float *dy, const float *y, float *dx)
{
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < len; ++i) dx[i] = dy[i] * ((float)(y[i] > 0.0f));
}

/* flat_map.cu:44-52: y = (mask + (1 - mask)*c) * x with mask = (float)(x > 0)   (leaky ReLU) */
ORACLE_API void oracle_leaky_relu_f32(size_t len, float c, const float *x, float *y)
{
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < len; ++i) {
    float xi = x[i];
    float mask = (float)(xi > 0.0f);
    y[i] = (mask + (1.0f - mask) * c) * xi;
  }
}

/* flat_map.cu:61-69: dx = (mask + (1 - mask)*c) * dy with mask = (float)(y > 0) */
ORACLE_API void oracle_leaky_relu_bwd_f32(size_t len, float c, const float *dy, const float *y, float *dx)
{
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < len; ++i) {
    float mask = (float)(y[i] > 0.0f);
    dx[i] = (mask + (1.0f - mask) * c) * dy[i];
  }
}

/* Running statistic update, pinned by tests/test_gpu.rs:561-593: y <- y + r*(x - y). */
ORACLE_API void oracle_online_average_f32(uint32_t len, float rate, const float *x, float *y)
{
  for (uint32_t i = 0; i < len; ++i) y[i] = y[i] + rate * (x[i] - y[i]);
}

/* ---- the whole layer, forward + backward, in the reference's kernel order -------------
 *
 * Forward  (src/ops.rs:999-1014, training branch): mean, var(+eps), running averages,
 *          normalize, [gamma/beta extension], positive_clip.
 * Backward (src/ops_gpu.rs:4344-4352, 3997-4003, 3787-3791; first writer assigns, later
 *          writers accumulate, src/lib.rs:2160-2165):
 *            dz    = dy * (y > 0)
 *            dvar  = norm_bwd_var(dz, x, mean, var)
 *            dmean = norm_bwd_mean(dz, var);  dmean += var_bwd_mean(dvar, x, mean)
 *            dx    = norm_bwd(dz, var);  dx += var_bwd(dvar, x, mean);  dx += mean_bwd(dmean)
 * gamma/beta (both NULL => reference behaviour): y_bn = gamma*xhat + beta;
 *            dbeta = sum(dz), dgamma = sum(dz*xhat), then dz <- gamma*dz.
 * scratch: caller passes two work arrays of the tensor's size (xhat, dz).
 * ---------------------------------------------------------------------------------- */
ORACLE_API void oracle_bn_relu_fwd_bwd_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate,
    const float *x, const float *dy, const float *gamma, const float *beta,
    float *run_mean, float *run_var,             /* in/out [C] */
    float *y, float *dx,                         /* out, tensor-sized */
    float *mean, float *var,                     /* out [C] */
    float *dgamma, float *dbeta,                 /* out [C], may be NULL when gamma is NULL */
    float *xhat, float *dz,                      /* scratch, tensor-sized */
    uint32_t block_sz)
{
  const size_t len = (size_t)dim0 * dim1 * dim2;
  float *dvar = (float *)calloc(dim1, sizeof(float));
  float *dmean = (float *)calloc(dim1, sizeof(float));

  oracle_batch_mean_f32(dim0, dim1, dim2, x, mean, block_sz);
  oracle_batch_var_f32(dim0, dim1, dim2, epsilon, x, mean, var, block_sz);
  oracle_online_average_f32(dim1, avg_rate, mean, run_mean);
  oracle_online_average_f32(dim1, avg_rate, var, run_var);
  oracle_batch_norm_f32(dim0, dim1, dim2, x, mean, var, xhat);
  if (gamma) {
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t n = 0; n < dim2; ++n)
      for (uint32_t c = 0; c < dim1; ++c) {
        const size_t row = pack3(0, dim0, c, dim1, n);
        const float g = gamma[c], b = beta ? beta[c] : 0.0f;
        for (uint32_t i0 = 0; i0 < dim0; ++i0) y[row + i0] = g * xhat[row + i0] + b;
      }
    oracle_positive_clip_f32(len, y, y);
  } else {
    oracle_positive_clip_f32(len, xhat, y);
  }

  oracle_positive_clip_bwd_f32(len, dy, y, dz);
  if (gamma) {
    /* dbeta = sum(dz): kind 3 with t = 1; dgamma = sum(dz*xhat): kind 4 with m = 0, t = 1 */
#pragma omp parallel
    {
      float *cache = alloc_cache(block_sz);
#pragma omp for schedule(dynamic, 1)
      for (uint32_t c = 0; c < dim1; ++c) {
        if (dbeta) dbeta[c] = reduce_channel_f32(3, dim0, dim1, dim2, c, dz, NULL, 0.f, 1.0f, block_sz, cache);
        if (dgamma) dgamma[c] = reduce_channel_f32(4, dim0, dim1, dim2, c, dz, xhat, 0.f, 1.0f, block_sz, cache);
      }
      free(cache);
    }
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t n = 0; n < dim2; ++n)
      for (uint32_t c = 0; c < dim1; ++c) {
        const size_t row = pack3(0, dim0, c, dim1, n);
        const float g = gamma[c];
        for (uint32_t i0 = 0; i0 < dim0; ++i0) dz[row + i0] = g * dz[row + i0];
      }
  }
  oracle_batch_norm_bwd_var_f32(dim0, dim1, dim2, dz, x, mean, var, dvar, 0, block_sz);
  oracle_batch_norm_bwd_mean_f32(dim0, dim1, dim2, dz, var, dmean, 0, block_sz);
  oracle_batch_var_bwd_mean_f32(dim0, dim1, dim2, dvar, x, mean, dmean, 1, block_sz);
  oracle_batch_norm_bwd_f32(dim0, dim1, dim2, dz, var, dx, 0);
  oracle_batch_var_bwd_f32(dim0, dim1, dim2, dvar, x, mean, dx, 1);
  oracle_batch_mean_bwd_f32(dim0, dim1, dim2, dmean, dx, 1);
  free(dvar);
  free(dmean);
}

/* Same layer in double precision (inputs f32, every intermediate and output f64).
 * Channels are independent, so one pass per channel does the whole thing. */
ORACLE_API void oracle_bn_act_fwd_bwd_f64(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, double epsilon, double avg_rate, double neg_slope,
    const float *x, const float *dy, const float *gamma, const float *beta,
    double *run_mean, double *run_var, double *y, double *dx,
    double *mean, double *var, double *dgamma, double *dbeta);

ORACLE_API void oracle_bn_relu_fwd_bwd_f64(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, double epsilon, double avg_rate,
    const float *x, const float *dy, const float *gamma, const float *beta,
    double *run_mean, double *run_var, double *y, double *dx,
    double *mean, double *var, double *dgamma, double *dbeta)
{
  oracle_bn_act_fwd_bwd_f64(dim0, dim1, dim2, epsilon, avg_rate, 0.0, x, dy, gamma, beta, run_mean, run_var, y, dx,
                            mean, var, dgamma, dbeta);
}

/* The same with the activation act(t) = t*(t > 0 ? 1 : neg_slope): 0 is the ReLU above, c the
 * reference's leaky ReLU (flat_map.cu:44-69), 1 no activation. */
ORACLE_API void oracle_bn_add_act_fwd_bwd_f64(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, double epsilon, double avg_rate, double neg_slope,
    const float *x, const float *residual, const float *dy, const float *gamma, const float *beta,
    double *run_mean, double *run_var, double *y, double *dx, double *dresidual,
    double *mean, double *var, double *dgamma, double *dbeta);

ORACLE_API void oracle_bn_act_fwd_bwd_f64(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, double epsilon, double avg_rate, double neg_slope,
    const float *x, const float *dy, const float *gamma, const float *beta,
    double *run_mean, double *run_var, double *y, double *dx,
    double *mean, double *var, double *dgamma, double *dbeta)
{
  oracle_bn_add_act_fwd_bwd_f64(dim0, dim1, dim2, epsilon, avg_rate, neg_slope, x, NULL, dy, gamma, beta, run_mean, run_var,
                                y, dx, NULL, mean, var, dgamma, dbeta);
}

/* With a residual input added before the activation: y = act(bn(x) + residual), the block
 * epilogue of examples/run_imagenet_mpi.rs:191-195, 224-226 (sum, then positive_clip); the sum's
 * adjoint hands dz = dy*mask to both inputs, so dresidual = dz.  residual / dresidual may be NULL. */
ORACLE_API void oracle_bn_add_act_fwd_bwd_f64(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, double epsilon, double avg_rate, double neg_slope,
    const float *x, const float *residual, const float *dy, const float *gamma, const float *beta,
    double *run_mean, double *run_var, double *y, double *dx, double *dresidual,
    double *mean, double *var, double *dgamma, double *dbeta)
{
  const double M = (double)dim0 * (double)dim2;
#pragma omp parallel for schedule(dynamic, 1)
  for (uint32_t c = 0; c < dim1; ++c) {
    double s = 0.0;
    for (uint32_t n = 0; n < dim2; ++n) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      for (uint32_t i0 = 0; i0 < dim0; ++i0) s += (double)x[row + i0];
    }
    const double m = s / M;
    double q = 0.0;
    for (uint32_t n = 0; n < dim2; ++n) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      for (uint32_t i0 = 0; i0 < dim0; ++i0) { double d = (double)x[row + i0] - m; q += d * d; }
    }
    const double v = q / M + epsilon;
    const double r = 1.0 / sqrt(v);
    mean[c] = m; var[c] = v;
    run_mean[c] = run_mean[c] + avg_rate * (m - run_mean[c]);
    run_var[c] = run_var[c] + avg_rate * (v - run_var[c]);
    const double g = gamma ? (double)gamma[c] : 1.0;
    const double b = (gamma && beta) ? (double)beta[c] : 0.0;
    double sdz = 0.0, sdzxh = 0.0;
    for (uint32_t n = 0; n < dim2; ++n) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      for (uint32_t i0 = 0; i0 < dim0; ++i0) {
        double xh = ((double)x[row + i0] - m) * r;
        double yb = g * xh + b + (residual ? (double)residual[row + i0] : 0.0);
        double yy = yb > 0.0 ? yb : neg_slope * yb;
        y[row + i0] = yy;
        double dzz = yb > 0.0 ? (double)dy[row + i0] : neg_slope * (double)dy[row + i0];
        if (dresidual) dresidual[row + i0] = dzz;
        sdz += dzz; sdzxh += dzz * xh;
      }
    }
    if (dbeta) dbeta[c] = sdz;
    if (dgamma) dgamma[c] = sdzxh;
    /* reference order in exact arithmetic: dvar, dmean (incl. the var_bwd_mean term), dx */
    const double dvar = g * sdzxh * (-0.5 * r * r);           /* sum(g dz (x-m)) * (-0.5 r / v) */
    double sxm = 0.0;
    for (uint32_t n = 0; n < dim2; ++n) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      for (uint32_t i0 = 0; i0 < dim0; ++i0) sxm += (double)x[row + i0] - m;
    }
    const double dmean = -r * g * sdz + sxm * (-2.0 * dvar) / M;
    for (uint32_t n = 0; n < dim2; ++n) {
      const size_t row = pack3(0, dim0, c, dim1, n);
      for (uint32_t i0 = 0; i0 < dim0; ++i0) {
        double yb = g * (((double)x[row + i0] - m) * r) + b + (residual ? (double)residual[row + i0] : 0.0);
        double dzz = (yb > 0.0 ? 1.0 : neg_slope) * g * (double)dy[row + i0];
        dx[row + i0] = dzz * r + dvar * ((double)x[row + i0] - m) * 2.0 / M + dmean / M;
      }
    }
  }
}
