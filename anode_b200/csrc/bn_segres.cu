// Fused batch-norm (+activation) for short rows: the "segments" shapes (dim0 < 256 or rows that are
// not 16-byte aligned one by one, e.g. [N, 2048, 7, 7]), where a channel's data is N short runs far
// apart and the tiled kernels spend more time on bookkeeping than on data; also rows of up to 1024
// floats (e.g. 28 x 28) when a channel is small enough to sit in a few blocks' shared memory, and
// the residual-block epilogue on those shapes (a third tensor in the slice).
//
// Decomposition: a unit is a block of cb channels, i.e. per sample one contiguous, 16-byte aligned
// run of L = cb*dim0 floats.  A thread-block CLUSTER of CL blocks owns one unit; block r of the
// cluster takes the samples [r*Rb, (r+1)*Rb) and copies its [Rb x L] slice into shared memory
// (cp.async, 16 bytes per request).  Everything else happens on chip:
//   1. per-column sums over the slice's samples (each thread keeps one float4 column in registers),
//      shifted by the column's first value;
//   2. columns -> channels inside the block (fixed order, double precision);
//   3. the CL block partials are exchanged through distributed shared memory, every block merges
//      them in rank order (bit-identical coefficients everywhere), block 0 writes the channel outputs;
//   4. y (or dx) is computed from the slice still in shared memory and streamed out.
// x (and dy) are read from HBM exactly once, nothing depends on L2 residency, there is no global
// scratch, no flag and no spin-wait: the only synchronisation is the hardware cluster barrier.
// (With several GPUs the per-channel records of the ranks are exchanged between steps 3 and 4 by
// peer stores, and that wait is bounded.  A cluster waits for the peers' records of ITS unit only,
// and the hardware dispatches clusters in index order on every GPU, so the lowest unfinished unit
// anywhere is always being worked on everywhere; should a device ever dispatch differently, the
// bounded wait turns it into a status bit, not a hang.)
// Two blocks share an SM, so one block's copies overlap the other's arithmetic.
//
// Reference kernels this replaces on such shapes: routines_gpu/batch_norm.cu:24-57, 125-163,
// 314-336 (forward) and :181-206, 240-280, 354-376, 408-444, 476-515 (backward), with the ReLU of
// routines_gpu/flat_map.cu:172-194 folded in.
#include <cooperative_groups.h>

#include "bn_device.cuh"
#include "bn_host.h"

namespace cg = cooperative_groups;

namespace anode_b200 {

#ifndef ANODE_SEG_THREADS
#define ANODE_SEG_THREADS 256
#endif
constexpr uint32_t kSegThreads = ANODE_SEG_THREADS;
constexpr uint32_t kSegColFloats = 4 * kSegThreads;      // per-column results of one block (x2 arrays)
constexpr uint32_t kSegMaxCluster = 16;

struct SegGeom {
  uint32_t cb;          // channels per unit
  uint32_t cluster;     // blocks per unit
  uint32_t rows;        // samples per block
  uint32_t units;
  uint32_t off_col, off_coef, off_part, off_stage, stage_bytes, off_dy, off_e, smem_bytes;   // off_e: residual (forward) / saved output (backward)
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc)
{
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long *p)
{
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_u64(unsigned long long *p, unsigned long long v)
{
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// n / d for n < 65536 (see fast_div): the multiplier, computed once per thread
__device__ __forceinline__ uint32_t seg_div_mul(uint32_t d) { return d > 1 ? 0xffffffffu / d + 1u : 0u; }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// The grid has one cluster per unit; a cluster launched with fewer clusters than units walks the
// units cid, cid + clusters, ...
template <int DIR>
__global__ void __launch_bounds__(kSegThreads) bn_segres_kernel(const FusedArgs a, const SegGeom g)
{
  extern __shared__ __align__(16) unsigned char sm[];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster.block_rank();
  const uint32_t csh = (uint32_t)__ffs((int)g.cluster) - 1u;        // the cluster size is a power of two
  const uint32_t cid = blockIdx.x >> csh, ncl = gridDim.x >> csh;
  const uint32_t dim0 = a.plan.dim0, C = a.plan.C, N = a.plan.N;
  const uint32_t n0 = rank * g.rows;
  const uint32_t rows = n0 < N ? ((N - n0 < g.rows) ? (N - n0) : g.rows) : 0;
  const uint64_t rs = (uint64_t)C * dim0;
  const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
  const bool acc = a.accumulate != 0;

  float *colA = reinterpret_cast<float *>(sm + g.off_col), *colB = colA + kSegColFloats;
  float *coef = reinterpret_cast<float *>(sm + g.off_coef);         // 8 floats per channel
  float4 *parts = reinterpret_cast<float4 *>(sm + g.off_part);      // two buffers of one per channel

  // slice of unit u -> stage st, dense [rows][Lw]
  auto issue = [&](uint32_t u) {
    const uint32_t st = 0;
    const uint32_t c0 = u * g.cb, cw = (C - c0 < g.cb) ? (C - c0) : g.cb;
    const uint32_t L4 = cw * dim0 / 4;
    float *sx = reinterpret_cast<float *>(sm + g.off_stage + (size_t)st * g.stage_bytes);
    float *sdy = reinterpret_cast<float *>(sm + g.off_stage + (size_t)st * g.stage_bytes + g.off_dy);
    float *se = reinterpret_cast<float *>(sm + g.off_stage + (size_t)st * g.stage_bytes + g.off_e);
    const float *extra = DIR == 0 ? a.res : a.ymask;       // residual epilogue: third (second) tensor of the slice
    const uint32_t total4 = rows * L4;
    const uint32_t mul = seg_div_mul(L4);
    const uint32_t row = fast_div(tid, mul);
    uint32_t col = tid - row * L4;
    const uint32_t drow = fast_div(kSegThreads, mul), dcol = kSegThreads - drow * L4;
    // float offset of this thread's next piece; advancing by kSegThreads pieces moves drow samples
    // down and dcol pieces right, wrapping into the next sample
    size_t off = (size_t)n0 * rs + (size_t)c0 * dim0 + (size_t)row * rs + 4 * (size_t)col;
    const size_t step = (size_t)drow * rs + 4 * (size_t)dcol, wrap = rs - 4 * (size_t)L4;
#pragma unroll 5
    for (uint32_t i = tid; i < total4; i += kSegThreads) {
      cp_async16(sx + 4 * (size_t)i, a.x + off);
      if (DIR == 1) cp_async16(sdy + 4 * (size_t)i, a.dy + off);
      if (extra) cp_async16(se + 4 * (size_t)i, extra + off);
      off += step; col += dcol;
      if (col >= L4) { col -= L4; off += wrap; }
    }
  };

  for (uint32_t u = cid; u < g.units; u += ncl) {
    const uint32_t st = 0;
    issue(u);
    cp_async_commit();
    const uint32_t c0 = u * g.cb, cw = (C - c0 < g.cb) ? (C - c0) : g.cb;
    const uint32_t Lw = cw * dim0, L4 = Lw / 4;                     // floats / float4s per sample in this unit
    const float *sx = reinterpret_cast<const float *>(sm + g.off_stage + (size_t)st * g.stage_bytes);
    const float *sdy = reinterpret_cast<const float *>(sm + g.off_stage + (size_t)st * g.stage_bytes + g.off_dy);
    const float *se = reinterpret_cast<const float *>(sm + g.off_stage + (size_t)st * g.stage_bytes + g.off_e);
    const bool has_e = (DIR == 0 ? a.res : a.ymask) != nullptr;
    float4 *part = parts + (size_t)st * g.cb;

    if (DIR == 1) {
      // what the mask needs is known before the sums: (mean, gamma*rstd, beta)
      for (uint32_t ci = tid; ci < cw; ci += kSegThreads) {
        const uint32_t c = c0 + ci;
        const float gm = a.gamma ? a.gamma[c] : 1.0f;
        coef[8 * ci + 0] = a.mean_in[c];
        coef[8 * ci + 1] = gm * inv_std(a.var_in[c]);
        coef[8 * ci + 2] = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
      }
    }
    cp_async_wait_all();              // the slice has landed
    __syncthreads();

    // ---- per-column sums.  Thread (grp, v): float4 column v, samples grp, grp+G, ...
    const uint32_t mul_l4 = seg_div_mul(L4), mul_d0 = seg_div_mul(dim0);    // divisions by multiplication from here on
    const uint32_t G = fast_div(kSegThreads, mul_l4);                  // >= 1: L4 <= kSegThreads by construction
    const uint32_t grp = fast_div(tid, mul_l4), v = tid - grp * L4;
    const bool active = grp < G;
    uint32_t ch[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) ch[i] = active ? fast_div(4 * v + i, mul_d0) : 0;
    if (active) {
      const float *px = sx + 4 * (size_t)v;
      if (DIR == 0) {
        float K[4] = {0.f, 0.f, 0.f, 0.f}, s[4] = {0.f, 0.f, 0.f, 0.f}, q[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t cnt = 0;
        if (grp < rows) {
          const float4 p = *reinterpret_cast<const float4 *>(px + (size_t)grp * Lw);
          K[0] = p.x; K[1] = p.y; K[2] = p.z; K[3] = p.w;
        }
        for (uint32_t r = grp; r < rows; r += G) {
          const float4 p = *reinterpret_cast<const float4 *>(px + (size_t)r * Lw);
          const float e[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float d = e[i] - K[i]; s[i] += d; q[i] = fmaf(d, d, q[i]); }
          ++cnt;
        }
        const float inv = cnt ? __fdividef(1.0f, (float)cnt) : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          colA[grp * Lw + 4 * v + i] = fmaf(s[i], inv, K[i]);                         // mean of the column part
          colB[grp * Lw + 4 * v + i] = fmaxf(q[i] - s[i] * s[i] * inv, 0.f);          // its M2
        }
      } else {
        const float *pd = sdy + 4 * (size_t)v, *pe = se + 4 * (size_t)v;
        float cm[4], cs[4], cbt[4], s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; ++i) { cm[i] = coef[8 * ch[i] + 0]; cs[i] = coef[8 * ch[i] + 1]; cbt[i] = coef[8 * ch[i] + 2]; }
        for (uint32_t r = grp; r < rows; r += G) {
          const float4 p = *reinterpret_cast<const float4 *>(px + (size_t)r * Lw);
          const float4 w = *reinterpret_cast<const float4 *>(pd + (size_t)r * Lw);
          float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
          if (has_e) m = *reinterpret_cast<const float4 *>(pe + (size_t)r * Lw);
          const float e[4] = {p.x, p.y, p.z, p.w}, f[4] = {w.x, w.y, w.z, w.w}, ym[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float d = e[i] - cm[i];
            const float yb = has_e ? ym[i] : fmaf(d, cs[i], cbt[i]);      // residual epilogue: the saved output carries the mask
            const float dz = f[i] * (yb > 0.0f ? 1.0f : slope);
            s1[i] += dz; s2[i] = fmaf(dz, d, s2[i]);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { colA[grp * Lw + 4 * v + i] = s1[i]; colB[grp * Lw + 4 * v + i] = s2[i]; }
      }
    }
    __syncthreads();

    // ---- columns -> channels of this block, fixed order, double precision.
    // Level 1: one thread per column folds the row groups (results replace group 0's entries;
    // every column has seen all `rows` samples).  Moments travel as (n, n*mean, M2 + n*mean^2):
    // plain sums in f64, which lose nothing that f32 inputs could have carried.
    const uint32_t Gr = G < rows ? G : rows;
    const uint32_t mul_g = seg_div_mul(G);
    const double inv_rows = rows ? 1.0 / (double)rows : 0.0;
    for (uint32_t col = tid; col < Lw; col += kSegThreads) {
      if (DIR == 0) {
        double t1 = 0.0, t2 = 0.0;
        for (uint32_t gi = 0; gi < Gr; ++gi) {
          const double n = (double)fast_div(rows - gi + G - 1, mul_g), m = (double)colA[gi * Lw + col];
          t1 = fma(n, m, t1); t2 += (double)colB[gi * Lw + col] + n * m * m;
        }
        const double mean = t1 * inv_rows;
        colA[col] = (float)mean; colB[col] = (float)fmax(t2 - t1 * mean, 0.0);
      } else {
        double t1 = 0.0, t2 = 0.0;
        for (uint32_t gi = 0; gi < Gr; ++gi) { t1 += (double)colA[gi * Lw + col]; t2 += (double)colB[gi * Lw + col]; }
        colA[col] = (float)t1; colB[col] = (float)t2;
      }
    }
    __syncthreads();
    // Level 2: one warp per channel over its dim0 columns
    for (uint32_t ci = warp; ci < cw; ci += kSegThreads / 32) {
      double t1 = 0.0, t2 = 0.0;
      for (uint32_t p = lane; p < dim0; p += 32) {
        const double m = (double)colA[ci * dim0 + p], w = (double)colB[ci * dim0 + p];
        if (DIR == 0) { t1 += m; t2 += w + (double)rows * m * m; } else { t1 += m; t2 += w; }
      }
      t1 = warp_sum_all(t1); t2 = warp_sum_all(t2);
      if (lane == 0) {
        if (DIR == 0) {
          const double n = (double)rows * (double)dim0, mean = t1 / (double)dim0;      // equal counts per column
          part[ci] = make_float4((float)n, (float)mean, (float)fmax(t2 - (double)rows * t1 * mean, 0.0), 0.f);
        } else {
          part[ci] = make_float4((float)t1, (float)t2, 0.f, 0.f);
        }
      }
    }
    cluster.sync();

    // ---- fetch the cluster's partials: one remote read per thread, all in flight together, instead of one
    // thread per channel reading rank after rank.  The column arrays are free by now.
    float4 *gath = reinterpret_cast<float4 *>(colA);                   // [channel][rank]
    const bool gathered = cw * g.cluster <= 2 * kSegColFloats / 4;
    if (gathered) {
      for (uint32_t t = tid; t < cw * g.cluster; t += kSegThreads) {
        const uint32_t ci = t >> csh, r = t & (g.cluster - 1u);
        gath[t] = *cluster.map_shared_rank(part + ci, r);
      }
      __syncthreads();
    }
    // ---- merge them in rank order; every block computes the same coefficients
    for (uint32_t ci = tid; ci < cw; ci += kSegThreads) {
      const uint32_t c = c0 + ci;
      const float gm = a.gamma ? a.gamma[c] : 1.0f;
      const float bt = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
      double t0 = 0.0, t1 = 0.0, t2 = 0.0;
#pragma unroll 4
      for (uint32_t r = 0; r < g.cluster; ++r) {
        const float4 p = gathered ? gath[ci * g.cluster + r] : *cluster.map_shared_rank(part + ci, r);
        if (DIR == 0) { const double n = (double)p.x, m = (double)p.y; t0 += n; t1 = fma(n, m, t1); t2 += (double)p.z + n * m * m; }
        else { t1 += (double)p.x; t2 += (double)p.y; }
      }
      if (a.world > 1) {
        // ---- several GPUs: the cluster's block 0 ships this GPU's record of the channel to every
        // rank (plain 8-byte peer stores, each word tagged with the call's sequence number), every
        // block collects the records of all ranks from its own GPU's buffer and merges them in
        // rank order.  Same protocol and buffers as the tiled kernel (bn_ring.cuh, pull_merge_unit).
        const size_t slot = ((((size_t)(a.epoch & 1u)) * a.world) * a.xchg_channels + c) * 4;
        const size_t src_stride = (size_t)a.xchg_channels * 4;
        if (rank == 0) {
          // word 0 of a forward record is the element count as an exact integer
          uint32_t w0, w1, w2;
          if (DIR == 0) { const double mean = t1 / t0; w0 = (uint32_t)t0; w1 = __float_as_uint((float)mean); w2 = __float_as_uint((float)fmax(t2 - t1 * mean, 0.0)); }
          else { w0 = __float_as_uint((float)t1); w1 = __float_as_uint((float)t2); w2 = 0u; }
          const unsigned long long e = (unsigned long long)a.epoch << 32;
          for (uint32_t r = 0; r < a.world; ++r) {
            unsigned long long *dst = a.xchg[r] + slot + a.rank * src_stride;
            st_sys_u64(dst + 0, e | w0);
            st_sys_u64(dst + 1, e | w1);
            st_sys_u64(dst + 2, e | w2);
          }
        }
        t0 = 0.0; t1 = 0.0; t2 = 0.0;
        const long long w_start = clock64();
        for (uint32_t r = 0; r < a.world; ++r) {
          const unsigned long long *src = a.xchg[a.rank] + slot + r * src_stride;
          unsigned long long v0, v1, v2;
          for (;;) {
            v0 = ld_sys_u64(src + 0); v1 = ld_sys_u64(src + 1); v2 = ld_sys_u64(src + 2);
            if ((uint32_t)(v0 >> 32) == a.epoch && (uint32_t)(v1 >> 32) == a.epoch && (uint32_t)(v2 >> 32) == a.epoch) break;
            if (clock64() - w_start > a.wait_cycles) { atomicOr(a.status, ANODE_ST_WAIT_PEER); break; }   // give up, leave a mark
            __nanosleep(200);
          }
          const double f0 = DIR == 0 ? (double)(uint32_t)v0 : (double)__uint_as_float((uint32_t)v0);
          const double f1 = (double)__uint_as_float((uint32_t)v1);
          const double f2 = (double)__uint_as_float((uint32_t)v2);
          if (DIR == 0) { t0 += f0; t1 = fma(f0, f1, t1); t2 += f2 + f0 * f1 * f1; }
          else { t1 += f0; t2 += f1; }
        }
      }
      if (DIR == 0) {
        const double mean = t1 / t0, m2 = fmax(t2 - t1 * mean, 0.0);
        const float mf = (float)mean;
        const float vf = (float)(m2 / t0 + (double)a.epsilon);        // biased, epsilon folded in (batch_norm.cu:160)
        coef[8 * ci + 0] = mf; coef[8 * ci + 1] = gm * inv_std(vf); coef[8 * ci + 2] = bt;
        if (rank == 0) {
          a.mean[c] = mf; a.var[c] = vf;
          if (a.run_mean) { const float o = a.run_mean[c]; a.run_mean[c] = o + a.avg_rate * (mf - o); }
          if (a.run_var) { const float o = a.run_var[c]; a.run_var[c] = o + a.avg_rate * (vf - o); }
        }
      } else {
        const float rstd = inv_std(a.var_in[c]);
        const double rs2 = (double)rstd * t2;                         // sum(dz * xhat)
        const double A = (double)gm * (double)rstd;
        const double invM = 1.0 / a.count_total;
        coef[8 * ci + 3] = (float)(-A * (double)rstd * rs2 * invM);
        coef[8 * ci + 4] = (float)(-A * t1 * invM);
        if (rank == 0) {
          if (a.dbeta) a.dbeta[c] = (float)t1;
          if (a.dgamma) a.dgamma[c] = (float)rs2;
        }
      }
    }
    __syncthreads();
    // This block has read its neighbours' partials: say so now and collect everybody's word at the end of the
    // unit (nobody may overwrite its partials or leave while a neighbour still reads them); the wait is then free.
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    // ---- apply from shared memory, stream the result out
    if (active) {
      float cm[4], cs[4], cbt[4], cB[4], cC[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        cm[i] = coef[8 * ch[i] + 0]; cs[i] = coef[8 * ch[i] + 1]; cbt[i] = coef[8 * ch[i] + 2];
        cB[i] = DIR == 1 ? coef[8 * ch[i] + 3] : 0.f; cC[i] = DIR == 1 ? coef[8 * ch[i] + 4] : 0.f;
      }
      const float *px = sx + 4 * (size_t)v, *pd = sdy + 4 * (size_t)v, *pe = se + 4 * (size_t)v;
      float *po = a.out + (size_t)n0 * rs + (size_t)c0 * dim0 + 4 * (size_t)v;
      float *pr = a.dres ? a.dres + (size_t)n0 * rs + (size_t)c0 * dim0 + 4 * (size_t)v : nullptr;
      for (uint32_t r = grp; r < rows; r += G) {
        const float4 p = *reinterpret_cast<const float4 *>(px + (size_t)r * Lw);
        float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
        if (has_e) m = *reinterpret_cast<const float4 *>(pe + (size_t)r * Lw);
        const float e[4] = {p.x, p.y, p.z, p.w}, ex[4] = {m.x, m.y, m.z, m.w};
        float o[4], dzs[4] = {0.f, 0.f, 0.f, 0.f};
        if (DIR == 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float yb = fmaf(e[i] - cm[i], cs[i], cbt[i]) + ex[i]; o[i] = yb * (yb > 0.0f ? 1.0f : slope); }
        } else {
          const float4 w = *reinterpret_cast<const float4 *>(pd + (size_t)r * Lw);
          const float f[4] = {w.x, w.y, w.z, w.w};
          float old[4] = {0.f, 0.f, 0.f, 0.f};
          if (acc) { const float4 t = *reinterpret_cast<const float4 *>(po + (size_t)r * rs); old[0] = t.x; old[1] = t.y; old[2] = t.z; old[3] = t.w; }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float d = e[i] - cm[i];
            const float yb = has_e ? ex[i] : fmaf(d, cs[i], cbt[i]);
            const float dz = f[i] * (yb > 0.0f ? 1.0f : slope);
            const float dx = fmaf(cs[i], dz, fmaf(cB[i], d, cC[i]));
            o[i] = acc ? old[i] + dx : dx;
            dzs[i] = dz;
          }
        }
        __stcs(reinterpret_cast<float4 *>(po + (size_t)r * rs), make_float4(o[0], o[1], o[2], o[3]));
        if (DIR == 1 && pr) __stcs(reinterpret_cast<float4 *>(pr + (size_t)r * rs), make_float4(dzs[0], dzs[1], dzs[2], dzs[3]));
      }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    __syncthreads();      // this stage, the column arrays and the coefficients may be reused
  }
}

// ---- host side -------------------------------------------------------------------------------

// One unit per cluster and launch; two blocks share an SM, so that one block's copies overlap the
// other's arithmetic.  (A persistent variant with two slices per block was measured slower: what
// limits this kernel is the chain of short dependent phases per unit, which co-resident blocks overlap
// better.)
#ifndef ANODE_SEG_BPS_FWD
#define ANODE_SEG_BPS_FWD 2
#endif
#ifndef ANODE_SEG_BPS_BWD
#define ANODE_SEG_BPS_BWD 2
#endif
constexpr uint32_t kSegBlocksPerSmFwd = ANODE_SEG_BPS_FWD, kSegBlocksPerSmBwd = ANODE_SEG_BPS_BWD;
constexpr uint32_t kSegLongRowCluster = 4;      // long aligned rows are taken when a channel fits this many blocks

// Geometry for direction `dir`, or false when this kernel does not apply: the shape is not a
// "segments" shape, or a unit does not fit the shared memory of one cluster.
static bool seg_geom(uint32_t dim0, uint32_t C, uint32_t N, int dir, bool extra, SegGeom &g)
{
  const uint64_t row_stride = (uint64_t)C * dim0;
  if (row_stride % 4 != 0 || dim0 > 4 * kSegThreads) return false;      // a row must fit one column per thread
  if (dim0 >= 512 && dim0 % 4 != 0) return false;              // long unaligned rows: the plain kernel's case
  uint32_t q = 4; if (dim0 % 2 == 0) q = 2; if (dim0 % 4 == 0) q = 1;      // cb*dim0 must be a multiple of 4
  // the smallest cb that gives runs of at least 512 bytes, within 256 float4 columns and 256 channels
  uint32_t cb = q;
  while ((uint64_t)cb * dim0 < 128 && (uint64_t)(cb + q) * dim0 <= 4 * kSegThreads && cb + q <= 256) cb += q;
  if (cb >= C) cb = C;
  if ((uint64_t)cb * dim0 > 4 * kSegThreads || (cb * dim0) % 4 != 0) return false;
  const uint32_t L = cb * dim0, tensors = (dir == 1 ? 2u : 1u) + (extra ? 1u : 0u);
  const uint32_t per_block = (228u * 1024u) / (dir == 0 ? kSegBlocksPerSmFwd : kSegBlocksPerSmBwd) - 1024u;       // what one of k co-resident blocks may use
  const uint32_t budget = per_block > 227u * 1024u ? 227u * 1024u : per_block;
  g.cb = cb; g.units = ceil_div_u32(C, cb);
  g.off_col = 0;
  g.off_coef = 2 * kSegColFloats * 4;
  g.off_part = g.off_coef + (uint32_t)align_up_u64((uint64_t)cb * 32, 16);
  g.off_stage = g.off_part + (uint32_t)align_up_u64((uint64_t)2 * cb * 16, 128);
  // `tensors` slices, each padded to 128 bytes
  if (g.off_stage + (uint64_t)tensors * ((uint64_t)L * 4 + 128) > budget) return false;
  const uint32_t rows_max = (uint32_t)(((budget - g.off_stage) / tensors - 128) / (L * 4));
  uint32_t cl = 1;
  while (cl < kSegMaxCluster && (uint64_t)cl * rows_max < N) cl *= 2;
  if ((uint64_t)cl * rows_max < N) return false;
  g.cluster = cl;
  g.rows = ceil_div_u32(N, cl);
  const uint32_t slice = (uint32_t)align_up_u64((uint64_t)g.rows * L * 4, 128);
  g.off_dy = slice;                         // within a stage: x, then dy (backward), then the extra tensor
  g.off_e = (dir == 1 ? 2u : 1u) * slice;
  g.stage_bytes = tensors * slice;
  g.smem_bytes = g.off_stage + g.stage_bytes;
  return g.smem_bytes <= budget;
}

// Long aligned rows (256 <= dim0, dim0 % 4 == 0) are also the tiled kernel's shapes.  The cluster
// kernel takes them when a channel is small enough to sit in a few blocks' shared memory: then its
// latency (one short pass, no pipeline to fill and drain) beats the tiled kernel's throughput.
bool segres_preferred(const FusedArgs &a, int dir, bool aligned)
{
  if (!segres_applies(a, dir, aligned)) return false;
  const uint32_t dim0 = a.plan.dim0;
  if (dim0 < 256 || dim0 % 4 != 0) return true;                // short or unaligned rows: always
  SegGeom g;
  const bool extra = (dir == 0 ? a.res : a.ymask) != nullptr;
  if (!seg_geom(dim0, a.plan.C, a.plan.N, dir, extra, g)) return false;
  return g.cluster <= kSegLongRowCluster;
}

bool segres_applies(const FusedArgs &a, int dir, bool aligned)
{
  SegGeom g;
  const bool extra = (dir == 0 ? a.res : a.ymask) != nullptr;
  return aligned && a.mode == MODE_FUSED && seg_geom(a.plan.dim0, a.plan.C, a.plan.N, dir, extra, g);
}

// Launches the segments kernel for a prepared call.  ANODE_E_LAUNCH when the device refuses the
// cluster shape (the caller falls back to the plain kernel).
int launch_segres(FusedArgs &a, int dir, cudaStream_t stream)
{
  SegGeom g;
  if (!seg_geom(a.plan.dim0, a.plan.C, a.plan.N, dir, (dir == 0 ? a.res : a.ymask) != nullptr, g)) return ANODE_E_LAUNCH;
  auto kernel = dir == 0 ? bn_segres_kernel<0> : bn_segres_kernel<1>;
  static std::mutex mu;
  static std::map<std::pair<const void *, uint64_t>, int> fit_cache;     // (kernel, smem | cluster) -> clusters resident at once
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g.units * g.cluster);
  cfg.blockDim = dim3(kSegThreads);
  cfg.dynamicSmemBytes = g.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = g.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int fit = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    (void)cudaGetDevice(&dev);
    const auto key = std::make_pair((const void *)kernel, ((uint64_t)g.smem_bytes << 16) | ((uint64_t)dev << 8) | g.cluster);
    auto it = fit_cache.find(key);
    if (it == fit_cache.end()) {
      int clusters = 0;
      bool ok = cudaFuncSetAttribute((const void *)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024)) == cudaSuccess;
      if (ok && g.cluster > 8)
        ok = cudaFuncSetAttribute((const void *)kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
      if (ok) ok = cudaOccupancyMaxActiveClusters(&clusters, (const void *)kernel, &cfg) == cudaSuccess && clusters > 0;
      if (!ok) { (void)cudaGetLastError(); clusters = 0; }
      it = fit_cache.emplace(key, clusters).first;
    }
    fit = it->second;
  }
  if (fit <= 0) return ANODE_E_LAUNCH;
  cfg.gridDim = dim3(g.units * g.cluster);
  if (cudaLaunchKernelEx(&cfg, kernel, a, g) != cudaSuccess) { (void)cudaGetLastError(); return ANODE_E_LAUNCH; }
  return ANODE_OK;
}

}  // namespace anode_b200

// ---- diagnostics: geometry of the cluster kernel for a shape (no GPU needed) ------------------
// out: applies, cb, cluster, rows per block, units, shared memory bytes
extern "C" int anode_gpu_batch_norm_segres_geometry(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir, uint32_t *out)
{
  using namespace anode_b200;
  if (!out || check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  SegGeom g{};
  const bool ok = seg_geom(dim0, dim1, dim2, dir, false, g);
  out[0] = ok ? 1u : 0u; out[1] = g.cb; out[2] = g.cluster; out[3] = g.rows; out[4] = g.units; out[5] = g.smem_bytes;
  return ANODE_OK;
}
