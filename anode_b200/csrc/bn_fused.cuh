// The fused batch-norm (+ReLU) kernels: one persistent kernel per direction in which every
// thread block walks its tiles twice, a bounded distance apart (see bn_plan.h):
//
//   reduce pass  forward : per-tile (count, mean, M2) of x              -> workspace partials
//                backward: per-tile sum(dz), sum(dz*(x-mean))           -> workspace partials
//   unit finish  the block that delivers a unit's last partial merges all of them in a fixed
//                order in double precision, writes the per-channel results and coefficients,
//                and raises the unit's ready flag
//   apply pass   forward : y  = relu(gamma*(x-mean)*rstd + beta)
//                backward: dx = A*dz + B*(x-mean) + C0   (closed form of the reference's
//                          dvar / dmean / dx chain, routines_gpu/batch_norm.cu:181-206,
//                          240-280, 354-376, 408-444, 476-515)
//
// The second visit of a tile finds it in L2 when the lookahead window fits there, so the
// tensor crosses HBM once per direction (plus the write).  Correctness never depends on it.
#pragma once
#include <type_traits>

#include "bn_device.cuh"

namespace anode_b200 {

enum : uint32_t { MODE_FUSED = 0, MODE_STATS = 1, MODE_APPLY = 2 };

constexpr uint32_t kSpinLimit = 1u << 20;   // about a second of polling, then give up
constexpr uint32_t kSegMaxFloats = 4 * kThreads * kSegSlots;
constexpr uint32_t kSegMaxChannels = 256;

struct FusedArgs {
  Plan plan;
  const float *x;
  const float *dy;         // backward only
  const float *gamma, *beta;
  const float *mean_in, *var_in;   // backward only
  // residual epilogue (plain kernel only): forward y = act(bn(x) + res); backward takes the mask
  // from the saved output ymask and also writes dres = dy*mask
  const float *res, *ymask;
  float *dres;
  float *out;              // y (forward) or dx (backward)
  float *mean, *var, *run_mean, *run_var;   // forward outputs
  float *dgamma, *dbeta;   // backward outputs
  unsigned char *ws;
  uint64_t ws_capacity;    // bytes of this direction's part of the workspace
  uint32_t *status;        // the workspace's status word (first word of the caller's buffer)
  float epsilon, avg_rate;
  uint32_t relu, accumulate, mode;
  float neg_slope;         // activation t*(t > 0 ? 1 : neg_slope): 0 = ReLU, 1 = none, c = leaky ReLU (flat_map.cu:44-52)
  uint32_t use_rec;        // publish tagged records (the warp-specialised kernel reads them)
  double count_total;      // elements per channel over all participating GPUs
  // cross-GPU exchange inside the kernel (world > 1): xchg[r] is rank r's exchange buffer as
  // mapped into this process (xchg[rank] is local memory); see bn_ring.cuh
  uint32_t rank, world, epoch, xchg_channels;
  unsigned long long *xchg[8];
  long long wait_cycles;   // bound of every in-kernel wait, in SM clock cycles
};

// 1/sqrt(v) as every kernel here computes it (IEEE divide and square root), so that the
// forward pass and the backward pass derive bit-identical scales, hence identical ReLU masks.
// The lowest mantissa bit is forced to one: the value can then never have an all-zero bit
// pattern, which lets a 64-bit (mean, rstd) record double as its own "ready" flag.
__device__ __forceinline__ float inv_std(float v)
{
  return __uint_as_float(__float_as_uint(__fdiv_rn(1.0f, __fsqrt_rn(v))) | 1u);
}

// Tagged per-channel records in the workspace: zero = not ready; written once per launch with a
// release store by the thread that completes the channel, read with acquire loads.
//   forward : (mean, rstd)         rstd has its lowest bit set
//   backward: (B, C0)              C0 gets its lowest bit set
__device__ __forceinline__ unsigned long long pack_rec(float lo, float hi)
{
  return ((unsigned long long)__float_as_uint(hi) << 32) | (unsigned long long)__float_as_uint(lo);
}
__device__ __forceinline__ void st_release_gpu_u64(unsigned long long *p, unsigned long long v)
{
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long *p)
{
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

struct SmemCommon {
  float mom[3 * (kThreads / 32)];
  double dsum[2 * (kThreads / 32)];
  uint32_t last;    // this block delivered the last partial of a unit
  uint32_t go;      // the wait for a unit's statistics succeeded
};
struct SmemSeg {
  float a[kSegMaxFloats];
  float b[kSegMaxFloats];
  float coef[kSegMaxChannels * 5];
};
struct SmemNone {};

__device__ __forceinline__ uint32_t *ws_u32(const FusedArgs &a, uint32_t off) { return reinterpret_cast<uint32_t *>(a.ws + off); }
__device__ __forceinline__ float4 *ws_f4(const FusedArgs &a, uint32_t off) { return reinterpret_cast<float4 *>(a.ws + off); }

// float offset of vector j of a regime-R tile (rows of per_row vectors, row stride rs floats)
template <int VEC>
__device__ __forceinline__ size_t vec_off(const TileRange &tr, uint32_t per_row, uint32_t mul, uint64_t rs, uint32_t j)
{
  if (tr.rows == 1) return (size_t)tr.base + (size_t)j * VEC;
  const uint32_t r = fast_div(j, mul);
  const uint32_t v = j - r * per_row;
  return (size_t)tr.base + (size_t)r * rs + (size_t)v * VEC;
}

// ======================================================================================
// per-channel completion
// ======================================================================================

// Forward: local (count, mean, M2) of channel c is complete.  Executed by one thread.
__device__ __forceinline__ void finish_channel_fwd(const FusedArgs &a, uint32_t c, double n, double mean, double m2)
{
  if (a.mode == MODE_STATS) {
    // the count travels as an exact integer in the first word (a float would round counts above 2^24)
    __stcg(ws_f4(a, a.plan.off_local) + c, make_float4(__uint_as_float((uint32_t)n), (float)mean, (float)m2, 0.f));
    return;
  }
  const float mf = (float)mean;
  const float vf = (float)(m2 / n + (double)a.epsilon);   // biased, epsilon folded in (batch_norm.cu:160)
  const float r = inv_std(vf);
  // What other blocks wait for goes out first; the outputs nobody waits for follow.
  if (a.use_rec) {
    st_release_gpu_u64(reinterpret_cast<unsigned long long *>(a.ws + a.plan.off_rec) + c, pack_rec(mf, r));
  } else {
    const float g = a.gamma ? a.gamma[c] : 1.0f;
    const float bt = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
    __stcg(ws_f4(a, a.plan.off_coef) + 2 * (size_t)c, make_float4(mf, g * r, bt, 0.f));
  }
  a.mean[c] = mf;
  a.var[c] = vf;
  // running statistics: y <- y + rate*(x - y)  (OnlineAverageOp; reference tests/test_gpu.rs:561-593)
  if (a.run_mean) { const float o = a.run_mean[c]; a.run_mean[c] = o + a.avg_rate * (mf - o); }
  if (a.run_var) { const float o = a.run_var[c]; a.run_var[c] = o + a.avg_rate * (vf - o); }
}

// Backward: S1 = sum(dz), S2 = sum(dz*(x-mean)) of channel c over all tiles.  One thread.
__device__ __forceinline__ void finish_channel_bwd(const FusedArgs &a, uint32_t c, double s1, double s2)
{
  if (a.mode == MODE_STATS) {
    __stcg(ws_f4(a, a.plan.off_local) + c, make_float4((float)s1, (float)s2, 0.f, 0.f));
    return;
  }
  const float mf = a.mean_in[c];
  const float r = inv_std(a.var_in[c]);
  const float g = a.gamma ? a.gamma[c] : 1.0f;
  const float bt = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
  const double rs2 = (double)r * s2;                       // sum(dz * xhat)
  const double A = (double)g * (double)r;
  const double invM = 1.0 / a.count_total;
  const float cB = (float)(-A * (double)r * rs2 * invM);
  const float cC = __uint_as_float(__float_as_uint((float)(-A * s1 * invM)) | 1u);   // never all-zero bits
  if (a.use_rec) {
    st_release_gpu_u64(reinterpret_cast<unsigned long long *>(a.ws + a.plan.off_rec) + c, pack_rec(cB, cC));
  } else {
    float4 *coef = ws_f4(a, a.plan.off_coef) + 2 * (size_t)c;
    __stcg(coef, make_float4(mf, g * r, bt, 0.f));
    __stcg(coef + 1, make_float4(cB, cC, 0.f, 0.f));
  }
  if (a.dbeta) a.dbeta[c] = (float)s1;
  if (a.dgamma) a.dgamma[c] = (float)rs2;
}

// Merge the partials of unit u.  Whole block; regime R (one channel, many partials).
template <int DIR>
__device__ __forceinline__ void finish_unit_R(const FusedArgs &a, uint32_t u, SmemCommon &sc)
{
  const Plan &P = a.plan;
  const float4 *part = ws_f4(a, P.off_part) + (size_t)u * P.tiles_per_unit;
  const uint32_t tid = threadIdx.x;
  if (DIR == 0) {
    double sn = 0.0, sm = 0.0;
    for (uint32_t k = tid; k < P.tiles_per_unit; k += kThreads) {
      const float4 p = __ldcg(part + k);
      sn += (double)p.x; sm += (double)p.x * (double)p.y;
    }
    block_sum2<double>(sn, sm, sc.dsum);
    const double mean = sm / sn;
    double sq = 0.0, zero = 0.0;
    for (uint32_t k = tid; k < P.tiles_per_unit; k += kThreads) {
      const float4 p = __ldcg(part + k);
      const double d = (double)p.y - mean;
      sq += (double)p.z + (double)p.x * d * d;
    }
    block_sum2<double>(sq, zero, sc.dsum);
    if (tid == 0) finish_channel_fwd(a, u, sn, mean, sq);
  } else {
    double s1 = 0.0, s2 = 0.0;
    for (uint32_t k = tid; k < P.tiles_per_unit; k += kThreads) {
      const float4 p = __ldcg(part + k);
      s1 += (double)p.x; s2 += (double)p.y;
    }
    block_sum2<double>(s1, s2, sc.dsum);
    if (tid == 0) finish_channel_bwd(a, u, s1, s2);
  }
}

// Regime S: a unit has cw channels and few partials each; one warp per channel.
template <int DIR>
__device__ __forceinline__ void finish_unit_S(const FusedArgs &a, uint32_t u)
{
  const Plan &P = a.plan;
  const uint32_t c0 = u * P.cb;
  const uint32_t cw = (P.C - c0 < P.cb) ? (P.C - c0) : P.cb;
  const float4 *part = ws_f4(a, P.off_part) + (size_t)u * P.tiles_per_unit * P.cb;
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (uint32_t ci = warp; ci < cw; ci += kThreads / 32) {
    if (DIR == 0) {
      double sn = 0.0, sm = 0.0;
      for (uint32_t k = lane; k < P.tiles_per_unit; k += 32) {
        const float4 p = __ldcg(part + (size_t)k * P.cb + ci);
        sn += (double)p.x; sm += (double)p.x * (double)p.y;
      }
      sn = warp_sum_all(sn); sm = warp_sum_all(sm);
      const double mean = sm / sn;
      double sq = 0.0;
      for (uint32_t k = lane; k < P.tiles_per_unit; k += 32) {
        const float4 p = __ldcg(part + (size_t)k * P.cb + ci);
        const double d = (double)p.y - mean;
        sq += (double)p.z + (double)p.x * d * d;
      }
      sq = warp_sum_all(sq);
      if (lane == 0) finish_channel_fwd(a, c0 + ci, sn, mean, sq);
    } else {
      double s1 = 0.0, s2 = 0.0;
      for (uint32_t k = lane; k < P.tiles_per_unit; k += 32) {
        const float4 p = __ldcg(part + (size_t)k * P.cb + ci);
        s1 += (double)p.x; s2 += (double)p.y;
      }
      s1 = warp_sum_all(s1); s2 = warp_sum_all(s2);
      if (lane == 0) finish_channel_bwd(a, c0 + ci, s1, s2);
    }
  }
}

// ======================================================================================
// regime R tiles
// ======================================================================================
constexpr int kUnroll = 4;

template <int VEC>
__device__ __forceinline__ void reduce_fwd_R(const FusedArgs &a, const TileRange &tr, uint32_t t, SmemCommon &sc)
{
  const uint32_t tid = threadIdx.x;
  const uint32_t per_row = tr.len / VEC, nvec = per_row * tr.rows;
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  const uint32_t mul = a.plan.div_mul;
  // Shifted sums: K is this thread's first element, so s and q stay small and q - s^2/n
  // does not cancel catastrophically whatever the channel mean is.
  const uint64_t keep = policy_keep();
  float K = 0.f;
  if (tid < nvec) K = a.x[vec_off<VEC>(tr, per_row, mul, rs, tid)];
  float s = 0.f, q = 0.f;
  for (uint32_t j0 = tid; j0 < nvec; j0 += kThreads * kUnroll) {
    Pack<VEC> v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t j = j0 + u * kThreads;
      if (j < nvec) v[u] = Pack<VEC>::load(a.x + vec_off<VEC>(tr, per_row, mul, rs, j), keep);
      else v[u] = pack_fill<VEC>(K);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int i = 0; i < VEC; ++i) { const float d = v[u].v[i] - K; s += d; q = fmaf(d, d, q); }
  }
  Moments m{0.f, 0.f, 0.f};
  if (tid < nvec) {
    m.n = (float)(((nvec - tid + kThreads - 1) / kThreads) * VEC);
    const float inv = __fdividef(1.0f, m.n);
    m.mean = fmaf(s, inv, K);
    m.m2 = fmaxf(q - s * s * inv, 0.f);
  }
  m = block_merge(m, sc.mom);
  if (tid == 0) __stcg(ws_f4(a, a.plan.off_part) + t, make_float4(m.n, m.mean, m.m2, 0.f));
}

template <int VEC>
__device__ __forceinline__ void apply_fwd_R(const FusedArgs &a, const TileRange &tr)
{
  const uint32_t tid = threadIdx.x;
  const uint32_t per_row = tr.len / VEC, nvec = per_row * tr.rows;
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  const uint32_t mul = a.plan.div_mul;
  const float4 cf = __ldcg(ws_f4(a, a.plan.off_coef) + 2 * (size_t)tr.c0);
  const float mean = cf.x, scale = cf.y, beta = cf.z;
  const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
  const uint64_t drop = policy_drop();
  for (uint32_t j0 = tid; j0 < nvec; j0 += kThreads * kUnroll) {
    Pack<VEC> v[kUnroll];
    size_t off[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t j = j0 + u * kThreads;
      off[u] = vec_off<VEC>(tr, per_row, mul, rs, j < nvec ? j : 0);
      if (j < nvec) v[u] = Pack<VEC>::load(a.x + off[u], drop);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t j = j0 + u * kThreads;
      if (j < nvec) {
        Pack<VEC> r = pack_fill<VEC>(0.f);
        if (a.res) r = Pack<VEC>::load(a.res + off[u]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float yb = fmaf(v[u].v[i] - mean, scale, beta) + r.v[i];
          v[u].v[i] = yb * (yb > 0.0f ? 1.0f : slope);
        }
        v[u].store(a.out + off[u], drop);
      }
    }
  }
}

template <int VEC>
__device__ __forceinline__ void reduce_bwd_R(const FusedArgs &a, const TileRange &tr, uint32_t t, SmemCommon &sc)
{
  const uint32_t tid = threadIdx.x;
  const uint32_t per_row = tr.len / VEC, nvec = per_row * tr.rows;
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  const uint32_t mul = a.plan.div_mul;
  const uint32_t c = tr.c0;
  const float mean = a.mean_in[c];
  const float g = a.gamma ? a.gamma[c] : 1.0f;
  const float beta = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
  const float scale = g * inv_std(a.var_in[c]);
  const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
  const uint64_t keep = policy_keep();
  float s1 = 0.f, s2 = 0.f;
  for (uint32_t j0 = tid; j0 < nvec; j0 += kThreads * kUnroll) {
    Pack<VEC> vx[kUnroll], vd[kUnroll], vy[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t j = j0 + u * kThreads;
      if (j < nvec) {
        const size_t off = vec_off<VEC>(tr, per_row, mul, rs, j);
        vx[u] = Pack<VEC>::load(a.x + off, keep);
        vd[u] = Pack<VEC>::load(a.dy + off, keep);
        if (a.ymask) vy[u] = Pack<VEC>::load(a.ymask + off, keep);
      } else {
        vx[u] = pack_fill<VEC>(mean);
        vd[u] = pack_fill<VEC>(0.f);
        vy[u] = pack_fill<VEC>(0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float d = vx[u].v[i] - mean;
        const float yb = a.ymask ? vy[u].v[i] : fmaf(d, scale, beta);
        // dz = dy * (float)(y > 0)  (routines_gpu/flat_map.cu:191-192)
        const float dz = vd[u].v[i] * (yb > 0.0f ? 1.0f : slope);
        s1 += dz; s2 = fmaf(dz, d, s2);
      }
  }
  block_sum2<float>(s1, s2, sc.mom);
  if (tid == 0) __stcg(ws_f4(a, a.plan.off_part) + t, make_float4(s1, s2, 0.f, 0.f));
}

template <int VEC>
__device__ __forceinline__ void apply_bwd_R(const FusedArgs &a, const TileRange &tr)
{
  const uint32_t tid = threadIdx.x;
  const uint32_t per_row = tr.len / VEC, nvec = per_row * tr.rows;
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  const uint32_t mul = a.plan.div_mul;
  const float4 c0 = __ldcg(ws_f4(a, a.plan.off_coef) + 2 * (size_t)tr.c0);
  const float4 c1 = __ldcg(ws_f4(a, a.plan.off_coef) + 2 * (size_t)tr.c0 + 1);
  const float mean = c0.x, scale = c0.y, beta = c0.z, cB = c1.x, cC = c1.y;
  const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
  const bool acc = a.accumulate != 0;
  const uint64_t drop = policy_drop();
  for (uint32_t j0 = tid; j0 < nvec; j0 += kThreads * kUnroll) {
    Pack<VEC> vx[kUnroll], vd[kUnroll];
    size_t off[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t j = j0 + u * kThreads;
      off[u] = vec_off<VEC>(tr, per_row, mul, rs, j < nvec ? j : 0);
      if (j < nvec) { vx[u] = Pack<VEC>::load(a.x + off[u], drop); vd[u] = Pack<VEC>::load(a.dy + off[u], drop); }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t j = j0 + u * kThreads;
      if (j < nvec) {
        Pack<VEC> o, vy, r;
        if (acc) o = Pack<VEC>::load(a.out + off[u]);
        if (a.ymask) vy = Pack<VEC>::load(a.ymask + off[u], drop);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float d = vx[u].v[i] - mean;
          const float yb = a.ymask ? vy.v[i] : fmaf(d, scale, beta);
          const float dz = vd[u].v[i] * (yb > 0.0f ? 1.0f : slope);
          const float dx = fmaf(scale, dz, fmaf(cB, d, cC));
          o.v[i] = acc ? o.v[i] + dx : dx;
          r.v[i] = dz;
        }
        o.store(a.out + off[u], drop);
        if (a.dres) r.store(a.dres + off[u], drop);
      }
    }
  }
}

// ======================================================================================
// regime S tiles: each thread owns up to kSegSlots float4 positions of the segment and visits
// them in every sample of the tile, so each of its 4*kSegSlots elements always belongs to the
// same channel and per-element accumulators can live in registers.
// ======================================================================================
template <int DIR>
__device__ __forceinline__ void load_coef_S(const FusedArgs &a, const TileRange &tr, SmemSeg &ss, bool from_ws)
{
  // stage (mean, scale, beta[, B, C0]) of the unit's channels in shared memory
  for (uint32_t ci = threadIdx.x; ci < tr.cw; ci += kThreads) {
    const uint32_t c = tr.c0 + ci;
    if (from_ws) {
      const float4 c0 = __ldcg(ws_f4(a, a.plan.off_coef) + 2 * (size_t)c);
      ss.coef[ci * 5 + 0] = c0.x; ss.coef[ci * 5 + 1] = c0.y; ss.coef[ci * 5 + 2] = c0.z;
      if (DIR == 1) {
        const float4 c1 = __ldcg(ws_f4(a, a.plan.off_coef) + 2 * (size_t)c + 1);
        ss.coef[ci * 5 + 3] = c1.x; ss.coef[ci * 5 + 4] = c1.y;
      }
    } else {
      const float g = a.gamma ? a.gamma[c] : 1.0f;
      ss.coef[ci * 5 + 0] = a.mean_in[c];
      ss.coef[ci * 5 + 1] = g * inv_std(a.var_in[c]);
      ss.coef[ci * 5 + 2] = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void reduce_fwd_S(const FusedArgs &a, const TileRange &tr, uint32_t t, SmemSeg &ss)
{
  const uint32_t tid = threadIdx.x;
  const uint32_t seg4 = tr.len / 4;
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  const float *base = a.x + tr.base;
  float K[kSegSlots][4], s[kSegSlots][4], q[kSegSlots][4];
#pragma unroll
  for (int k = 0; k < (int)kSegSlots; ++k) {
    const uint32_t v = tid + k * kThreads;
    Pack<4> p = pack_fill<4>(0.f);
    if (v < seg4) p = Pack<4>::load(base + 4 * (size_t)v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { K[k][i] = p.v[i]; s[k][i] = 0.f; q[k][i] = 0.f; }
  }
  for (uint32_t r0 = 1; r0 < tr.rows; r0 += kUnroll) {
    Pack<4> p[kUnroll][kSegSlots];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int k = 0; k < (int)kSegSlots; ++k) {
        const uint32_t v = tid + k * kThreads;
        if (r0 + u < tr.rows && v < seg4) p[u][k] = Pack<4>::load(base + (size_t)(r0 + u) * rs + 4 * (size_t)v);
        else {
#pragma unroll
          for (int i = 0; i < 4; ++i) p[u][k].v[i] = K[k][i];
        }
      }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int k = 0; k < (int)kSegSlots; ++k)
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float d = p[u][k].v[i] - K[k][i]; s[k][i] += d; q[k][i] = fmaf(d, d, q[k][i]); }
  }
  // per element position: mean and M2 over the tile's samples -> shared memory
  const float nr = (float)tr.rows, inv = __fdividef(1.0f, nr);
  __syncthreads();   // ss.a / ss.b may still be in use by the previous tile's channel pass
#pragma unroll
  for (int k = 0; k < (int)kSegSlots; ++k) {
    const uint32_t v = tid + k * kThreads;
    if (v < seg4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ss.a[4 * v + i] = fmaf(s[k][i], inv, K[k][i]);
        ss.b[4 * v + i] = fmaxf(q[k][i] - s[k][i] * s[k][i] * inv, 0.f);
      }
    }
  }
  __syncthreads();
  // one thread per channel: merge its dim0 positions (equal counts, two passes, fixed order)
  const uint32_t d0 = a.plan.dim0;
  for (uint32_t ci = tid; ci < tr.cw; ci += kThreads) {
    const float *pm = ss.a + ci * d0, *pq = ss.b + ci * d0;
    float sm = 0.f;
    for (uint32_t i = 0; i < d0; ++i) sm += pm[i];
    const float mean = sm / (float)d0;
    float m2 = 0.f, dev = 0.f;
    for (uint32_t i = 0; i < d0; ++i) { const float d = pm[i] - mean; m2 += pq[i]; dev = fmaf(d, d, dev); }
    m2 = fmaf(nr, dev, m2);
    __stcg(ws_f4(a, a.plan.off_part) + (size_t)t * a.plan.cb + ci, make_float4(nr * (float)d0, mean, m2, 0.f));
  }
}

__device__ __forceinline__ void reduce_bwd_S(const FusedArgs &a, const TileRange &tr, uint32_t t, SmemSeg &ss)
{
  const uint32_t tid = threadIdx.x;
  const uint32_t seg4 = tr.len / 4, d0 = a.plan.dim0;
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  __syncthreads();   // previous users of ss.coef / ss.a / ss.b are done
  load_coef_S<1>(a, tr, ss, false);
  float cm[kSegSlots][4], cs[kSegSlots][4], cb[kSegSlots][4], s1[kSegSlots][4], s2[kSegSlots][4];
#pragma unroll
  for (int k = 0; k < (int)kSegSlots; ++k) {
    const uint32_t v = tid + k * kThreads;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t ci = (v < seg4) ? (4 * v + i) / d0 : 0;
      cm[k][i] = ss.coef[ci * 5 + 0]; cs[k][i] = ss.coef[ci * 5 + 1]; cb[k][i] = ss.coef[ci * 5 + 2];
      s1[k][i] = 0.f; s2[k][i] = 0.f;
    }
  }
  const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
  const float *bx = a.x + tr.base, *bd = a.dy + tr.base;
  constexpr int U = 2;
  for (uint32_t r0 = 0; r0 < tr.rows; r0 += U) {
    Pack<4> px[U][kSegSlots], pd[U][kSegSlots], py[U][kSegSlots];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < (int)kSegSlots; ++k) {
        const uint32_t v = tid + k * kThreads;
        if (r0 + u < tr.rows && v < seg4) {
          const size_t off = (size_t)(r0 + u) * rs + 4 * (size_t)v;
          px[u][k] = Pack<4>::load(bx + off); pd[u][k] = Pack<4>::load(bd + off);
          if (a.ymask) py[u][k] = Pack<4>::load(a.ymask + tr.base + off);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) { px[u][k].v[i] = cm[k][i]; pd[u][k].v[i] = 0.f; py[u][k].v[i] = 0.f; }
        }
      }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < (int)kSegSlots; ++k)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float d = px[u][k].v[i] - cm[k][i];
          const float yb = a.ymask ? py[u][k].v[i] : fmaf(d, cs[k][i], cb[k][i]);
          const float dz = pd[u][k].v[i] * (yb > 0.0f ? 1.0f : slope);
          s1[k][i] += dz; s2[k][i] = fmaf(dz, d, s2[k][i]);
        }
  }
#pragma unroll
  for (int k = 0; k < (int)kSegSlots; ++k) {
    const uint32_t v = tid + k * kThreads;
    if (v < seg4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { ss.a[4 * v + i] = s1[k][i]; ss.b[4 * v + i] = s2[k][i]; }
    }
  }
  __syncthreads();
  for (uint32_t ci = tid; ci < tr.cw; ci += kThreads) {
    const float *p1 = ss.a + ci * d0, *p2 = ss.b + ci * d0;
    float t1 = 0.f, t2 = 0.f;
    for (uint32_t i = 0; i < d0; ++i) { t1 += p1[i]; t2 += p2[i]; }
    __stcg(ws_f4(a, a.plan.off_part) + (size_t)t * a.plan.cb + ci, make_float4(t1, t2, 0.f, 0.f));
  }
}

template <int DIR>
__device__ __forceinline__ void apply_S(const FusedArgs &a, const TileRange &tr, SmemSeg &ss)
{
  const uint32_t tid = threadIdx.x;
  const uint32_t seg4 = tr.len / 4, d0 = a.plan.dim0;
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  __syncthreads();   // previous users of ss.coef are done
  load_coef_S<DIR>(a, tr, ss, true);
  float cm[kSegSlots][4], cs[kSegSlots][4], cb[kSegSlots][4], cB[kSegSlots][4], cC[kSegSlots][4];
#pragma unroll
  for (int k = 0; k < (int)kSegSlots; ++k) {
    const uint32_t v = tid + k * kThreads;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t ci = (v < seg4) ? (4 * v + i) / d0 : 0;
      cm[k][i] = ss.coef[ci * 5 + 0]; cs[k][i] = ss.coef[ci * 5 + 1]; cb[k][i] = ss.coef[ci * 5 + 2];
      if (DIR == 1) { cB[k][i] = ss.coef[ci * 5 + 3]; cC[k][i] = ss.coef[ci * 5 + 4]; }
    }
  }
  const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
  const bool acc = a.accumulate != 0;
  const float *bx = a.x + tr.base;
  float *bo = a.out + tr.base;
  constexpr int U = 2;
  for (uint32_t r0 = 0; r0 < tr.rows; r0 += U) {
    Pack<4> px[U][kSegSlots], pd[U][kSegSlots];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < (int)kSegSlots; ++k) {
        const uint32_t v = tid + k * kThreads;
        if (r0 + u < tr.rows && v < seg4) {
          const size_t off = (size_t)(r0 + u) * rs + 4 * (size_t)v;
          px[u][k] = Pack<4>::load(bx + off);
          if (DIR == 1) pd[u][k] = Pack<4>::load(a.dy + tr.base + off);
        }
      }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < (int)kSegSlots; ++k) {
        const uint32_t v = tid + k * kThreads;
        if (r0 + u < tr.rows && v < seg4) {
          const size_t off = (size_t)(r0 + u) * rs + 4 * (size_t)v;
          Pack<4> o, e = pack_fill<4>(0.f), r;       // e: residual (forward) or saved output (backward)
          if (DIR == 1 && acc) o = Pack<4>::load(bo + off);
          if (DIR == 0 && a.res) e = Pack<4>::load(a.res + tr.base + off);
          if (DIR == 1 && a.ymask) e = Pack<4>::load(a.ymask + tr.base + off);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float d = px[u][k].v[i] - cm[k][i];
            const float yb = fmaf(d, cs[k][i], cb[k][i]);
            if (DIR == 0) {
              const float t = yb + e.v[i];
              o.v[i] = t * (t > 0.0f ? 1.0f : slope);
            } else {
              const float t = a.ymask ? e.v[i] : yb;
              const float dz = pd[u][k].v[i] * (t > 0.0f ? 1.0f : slope);
              const float dx = fmaf(cs[k][i], dz, fmaf(cB[k][i], d, cC[k][i]));
              o.v[i] = acc ? o.v[i] + dx : dx;
              r.v[i] = dz;
            }
          }
          o.store_stream(bo + off);
          if (DIR == 1 && a.dres) r.store_stream(a.dres + tr.base + off);
        }
      }
  }
}

// ======================================================================================
// the persistent kernel
// ======================================================================================
template <int VEC, int DIR, int REGIME>
__global__ void __launch_bounds__(kThreads) bn_pipeline_kernel(const FusedArgs a)
{
  __shared__ SmemCommon sc;
  __shared__ typename std::conditional<REGIME == 1, SmemSeg, SmemNone>::type ss;
  const Plan &P = a.plan;
  const uint32_t tid = threadIdx.x, b = blockIdx.x, G = gridDim.x;
  const uint32_t my_tiles = (b < P.total_tiles) ? (P.total_tiles - b + G - 1) / G : 0;
  const uint32_t look = (a.mode == MODE_FUSED) ? P.lookahead_steps : 0;
  const bool do_reduce = a.mode != MODE_APPLY, do_apply = a.mode != MODE_STATS;
  uint32_t *status = a.status;
  uint32_t *done = ws_u32(a, P.off_done), *ready = ws_u32(a, P.off_ready), *applied = ws_u32(a, P.off_applied);

  for (uint32_t s = 0; s < my_tiles + look; ++s) {
    if (do_reduce && s < my_tiles) {
      const uint32_t t = b + s * G;
      const TileRange tr = tile_range(P, t);
      if constexpr (REGIME == 0) {
        if constexpr (DIR == 0) reduce_fwd_R<VEC>(a, tr, t, sc); else reduce_bwd_R<VEC>(a, tr, t, sc);
      } else {
        if constexpr (DIR == 0) reduce_fwd_S(a, tr, t, ss); else reduce_bwd_S(a, tr, t, ss);
      }
      // deliver the partial; the block that delivers a unit's last one completes the unit
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(done + tr.unit, 1u);
        sc.last = (old + 1 == P.tiles_per_unit) ? 1u : 0u;
      }
      __syncthreads();
      if (sc.last) {
        __threadfence();
        if constexpr (REGIME == 0) finish_unit_R<DIR>(a, tr.unit, sc); else finish_unit_S<DIR>(a, tr.unit);
        __syncthreads();
        if (tid == 0) {
          done[tr.unit] = 0;                     // leave the workspace clean for the next launch
          if (a.mode == MODE_FUSED) { __threadfence(); st_release_gpu(ready + tr.unit, 1u); }
        }
      }
    }
    if (do_apply && s >= look) {
      const uint32_t t = b + (s - look) * G;
      const TileRange tr = tile_range(P, t);
      if (a.mode == MODE_FUSED) {
        if (tid == 0) {
          uint32_t ok = 1, it = 0;
          while (ld_acquire_gpu(ready + tr.unit) == 0u) {
            __nanosleep(100);
            ++it;
            if (it > kSpinLimit) { atomicOr(status, ANODE_ST_WAIT_STATS); ok = 0; break; }
            if ((it & 255u) == 0u && ld_relaxed_gpu(status) != 0u) { ok = 0; break; }
          }
          sc.go = ok;
        }
        __syncthreads();
        if (!sc.go) {                          // give up: leave a mark and stop this block
          if (tid == 0) atomicOr(status, ANODE_ST_ABORTED);
          return;
        }
      }
      if constexpr (REGIME == 0) {
        if constexpr (DIR == 0) apply_fwd_R<VEC>(a, tr); else apply_bwd_R<VEC>(a, tr);
      } else {
        apply_S<DIR>(a, tr, ss);
      }
      if (a.mode == MODE_FUSED) {
        // the block that applies a unit's last tile lowers its flags again
        __syncthreads();
        if (tid == 0) {
          const uint32_t old = atomicAdd(applied + tr.unit, 1u);
          if (old + 1 == P.tiles_per_unit) { applied[tr.unit] = 0; ready[tr.unit] = 0; }
        }
      }
    }
  }
}

// ---- shared by the instantiations of the warp-specialised kernel (bn_ring.cuh) and the host ----
constexpr uint32_t kResQ = 4;          // partial mailbox depth
constexpr uint32_t kCoefQ = 4;         // coefficient mailbox depth
constexpr uint32_t kMaxSlots = 8;
constexpr uint32_t kRingCtlBytes = 1024;   // room reserved for the kernel's barrier block (RingCtl)
struct RingGeom {
  uint32_t slots, slot_floats, slot_stride, res_stride, off_res, off_coef, off_slots, smem_bytes;
  float keep_frac;         // fused mode: fraction of the reduce visits' lines loaded with the L2 "keep" priority
};

}  // namespace anode_b200
