// Slice-resident fused batch-norm (+activation): every element is loaded from global memory into
// shared memory ONCE per direction, reduced there, kept until its channel's statistics are known,
// normalised in place and written back from shared memory -- all global traffic is bulk
// asynchronous copies (cp.async.bulk, global -> shared and shared -> global).
//
// A channel is spread over a TEAM of thread blocks (one block per SM, see bn_resident_plan.h); each
// block keeps its slice of the channel in a ring of shared-memory slots.  Where a slice is larger
// than the ring, the overflow pieces are streamed: reduced and released, then fetched a second time
// for the apply step (they are loaded with an L2 "keep" hint, everything else with "evict first").
//
// Roles of a block (warp-specialised, all walking the same event sequence, res_walk):
//   loader     issues the bulk loads, as far ahead as free slots allow;
//   consumers  reduce pieces as they land (running sums over the whole slice, in registers) and,
//              later, normalise them in place;
//   storer     issues the bulk stores of normalised pieces and recycles slots;
//   delivery   turns the consumer warps' sums of a channel into ONE partial record in the workspace;
//   coefficient warp  waits for the partial records of all blocks of the team, merges them in a
//              fixed order in double precision (bit-identical on every block; with several GPUs the
//              channel's owner block exchanges per-GPU records with the peers first) and hands the
//              channel's coefficients to the consumers.
// Records carry the launch's sequence number, so nothing in the workspace has to be cleared between
// launches.  Every wait is bounded: a wait that runs out sets a status bit, raises the block's abort
// flag and all roles drain and leave.
//
// Replaces, on long-row shapes: routines_gpu/batch_norm.cu:24-57, 125-163, 314-336 (forward) and
// :181-206, 240-280, 354-376, 408-444, 476-515 (backward) with routines_gpu/flat_map.cu:172-194.
#include "bn_host.h"
#include "bn_resident_plan.h"

namespace anode_b200 {
namespace res {

constexpr uint32_t kResQ = 4;        // partial mailbox depth
constexpr uint32_t kCoefQ = 4;       // coefficient mailbox depth
constexpr uint32_t kCWarps = 8;          // consumer warps (a power of two)
constexpr uint32_t kResThreads = 32 * (kCWarps + 4);     // + loader, storer, delivery and coefficient warps
#ifndef ANODE_RES_BACKOFF_NS
#define ANODE_RES_BACKOFF_NS 64
#endif

struct Ctl {
  unsigned long long full[kResMaxSlots], done[kResMaxSlots], empty[kResMaxSlots];
  unsigned long long res_full[kResQ], res_empty[kResQ], coef_full[kCoefQ], coef_empty[kCoefQ];
  float4 res[kResQ][kCWarps];         // per consumer warp: forward (s, q, K, -), backward (s1, s2, -, -)
  float4 coef[kCoefQ][2];            // (mean, gamma*rstd, beta, -), (B, C0, -, -)
  uint2 ptab[kResMaxPieces];         // per piece of the slice: float offset / 4 inside channel 0, rows << 16 | floats per row
  volatile uint32_t abort;
  volatile uint32_t issued;          // loads of any kind the loader has issued, in schedule order
  uint32_t epoch;
  uint32_t last_block;
};
static_assert(sizeof(Ctl) <= kResCtlBytes, "Ctl outgrew the room reserved for it");

// ---- primitives ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned long long *bar, uint32_t parity)
{
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(s32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try(unsigned long long *bar, uint32_t parity)
{
  uint32_t ok;
  // the last operand lets the hardware keep the thread suspended (up to that many nanoseconds)
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(s32(bar)), "r"(parity), "r"(20000u) : "memory");
  return ok != 0;
}
// Bounded wait, executed by all lanes of a warp alike.  False (abort flag raised) when the barrier did
// not flip in time or another role already gave up.
__device__ __forceinline__ bool warp_wait(unsigned long long *bar, uint32_t parity, Ctl *ctl, uint32_t *status, long long limit)
{
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    // back off: a spinning waiter takes issue slots from the warps that do the work
    __nanosleep(ANODE_RES_BACKOFF_NS);
    if (mbar_try(bar, parity)) return true;
    if (ctl->abort) return false;
    if (clock64() - t0 > limit) {
      if ((threadIdx.x & 31) == 0) { atomicOr(status, ANODE_ST_WAIT_STATS); ctl->abort = 1; }
      return false;
    }
  }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, unsigned long long *bar, uint64_t policy)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(s32(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *dst, uint32_t src, uint32_t bytes, uint64_t policy)
{
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
               ::"l"(dst), "r"(src), "r"(bytes), "l"(policy) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float4 lds128(uint32_t a)
{
  float4 r;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(a) : "memory");
  return r;
}
__device__ __forceinline__ void sts128(uint32_t a, float4 v)
{
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_gpu_u64(const unsigned long long *p)
{
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_gpu_u64(unsigned long long *p, unsigned long long v)
{
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
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

struct ResArgs {
  ResPlan g;
  uint32_t ws_off;          // byte offset of this kernel's records inside the direction's workspace part
};

__device__ __forceinline__ unsigned long long *part_rec(const FusedArgs &a, const ResArgs &ra, uint32_t c, uint32_t b)
{
  return reinterpret_cast<unsigned long long *>(a.ws + ra.ws_off) + ((size_t)c * ra.g.Gt + b) * kResPartWords;
}

struct PieceRef { uint32_t rows, len; size_t off; };     // rows, floats per row, float offset of the piece's first row in channel 0
__device__ __forceinline__ PieceRef piece_ref(const Ctl *ctl, uint32_t t)
{
  const uint2 e = ctl->ptab[t];
  return PieceRef{e.y >> 16, e.y & 0xffffu, (size_t)e.x * 4};
}

// Consumer side of a load: the barrier of a slot tells phases apart by parity only, and consumer warps
// run independently, so a warp could reach the wait for load n of a slot while load n-1 is still in
// flight and mistake the completion of load n-2 (same parity) for its own.  It therefore first waits
// until the loader has issued load number `m` of the schedule (its own), which the loader does only
// after the slot's previous load was consumed and released: from then on the parity is unambiguous.
__device__ __forceinline__ bool wait_load(Ctl *ctl, uint32_t slot, uint32_t par, uint32_t m, uint32_t *status, long long limit)
{
  if ((int)(ctl->issued - m) <= 0) {
    const long long t0 = clock64();
    while ((int)(ctl->issued - m) <= 0) {
      __nanosleep(ANODE_RES_BACKOFF_NS);
      if (ctl->abort) return false;
      if (clock64() - t0 > limit) {
        if ((threadIdx.x & 31) == 0) { atomicOr(status, ANODE_ST_WAIT_STATS); ctl->abort = 1; }
        return false;
      }
    }
  }
  __threadfence_block();
  return warp_wait(&ctl->full[slot], par, ctl, status, limit);
}

// ---- consumer arithmetic ---------------------------------------------------------------------------
// act(t) = t * (t > 0 ? 1 : slope)  (flat_map.cu:44-52, 176-177)
__device__ __forceinline__ float act(float t, float slope) { return t * (t > 0.0f ? 1.0f : slope); }

// One vector (four elements) of the reduce visit.  Forward: sums of (x - K) and (x - K)^2.  Backward:
// sums of dz and dz*(x - mean), dz = dy * (float)(y > 0)  (routines_gpu/flat_map.cu:191-192); with the
// residual epilogue the saved output `vy` carries the sign (the positive_clip adjoint takes it from y).
template <int DIR, bool EXTRA>
__device__ __forceinline__ void reduce_vec(float4 vx, float4 vg, float4 vy, float slope, float K, float rm, float rscale, float rbeta, float &s, float &q)
{
  const float x[4] = {vx.x, vx.y, vx.z, vx.w}, g[4] = {vg.x, vg.y, vg.z, vg.w}, y[4] = {vy.x, vy.y, vy.z, vy.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if constexpr (DIR == 0) {
      const float d = x[e] - K;
      s += d; q = fmaf(d, d, q);
    } else {
      const float d = x[e] - rm;
      const float t = EXTRA ? y[e] : fmaf(d, rscale, rbeta);
      const float z = g[e] * (t > 0.0f ? 1.0f : slope);
      s += z; q = fmaf(z, d, q);
    }
  }
}

// Reduce visit of a piece of nvec vectors at shared address sx (the other tensors in the planes behind
// it).  A lane's vectors are 32 apart; they are taken four, two, one at a time so that the loads of a
// group are all in flight before the arithmetic starts.
template <int DIR, bool EXTRA>
__device__ __forceinline__ void reduce_piece(uint32_t sx, uint32_t plane_bytes, uint32_t nvec, float slope,
                                             float K, float rm, float rscale, float rbeta, float &a0, float &a1, float &b0, float &b1)
{
  constexpr uint32_t kStep = 32 * 16;                 // bytes between a lane's consecutive vectors
  constexpr bool kDy = DIR == 1, kY = DIR == 1 && EXTRA;
  uint32_t v = threadIdx.x & 31;
  uint32_t ax = sx + v * 16;
  const uint32_t p1 = plane_bytes, p2 = 2 * plane_bytes;
  for (; v + 96 < nvec; v += 128, ax += 4 * kStep) {
    const float4 x0 = lds128(ax), x1 = lds128(ax + kStep), x2 = lds128(ax + 2 * kStep), x3 = lds128(ax + 3 * kStep);
    float4 g0 = x0, g1 = x1, g2 = x2, g3 = x3, y0 = x0, y1 = x1, y2 = x2, y3 = x3;
    if constexpr (kDy) { g0 = lds128(ax + p1); g1 = lds128(ax + p1 + kStep); g2 = lds128(ax + p1 + 2 * kStep); g3 = lds128(ax + p1 + 3 * kStep); }
    if constexpr (kY) { y0 = lds128(ax + p2); y1 = lds128(ax + p2 + kStep); y2 = lds128(ax + p2 + 2 * kStep); y3 = lds128(ax + p2 + 3 * kStep); }
    reduce_vec<DIR, EXTRA>(x0, g0, y0, slope, K, rm, rscale, rbeta, a0, b0);
    reduce_vec<DIR, EXTRA>(x1, g1, y1, slope, K, rm, rscale, rbeta, a1, b1);
    reduce_vec<DIR, EXTRA>(x2, g2, y2, slope, K, rm, rscale, rbeta, a0, b0);
    reduce_vec<DIR, EXTRA>(x3, g3, y3, slope, K, rm, rscale, rbeta, a1, b1);
  }
  if (v + 32 < nvec) {
    const float4 x0 = lds128(ax), x1 = lds128(ax + kStep);
    float4 g0 = x0, g1 = x1, y0 = x0, y1 = x1;
    if constexpr (kDy) { g0 = lds128(ax + p1); g1 = lds128(ax + p1 + kStep); }
    if constexpr (kY) { y0 = lds128(ax + p2); y1 = lds128(ax + p2 + kStep); }
    reduce_vec<DIR, EXTRA>(x0, g0, y0, slope, K, rm, rscale, rbeta, a0, b0);
    reduce_vec<DIR, EXTRA>(x1, g1, y1, slope, K, rm, rscale, rbeta, a1, b1);
    v += 64; ax += 2 * kStep;
  }
  if (v < nvec) {
    const float4 x0 = lds128(ax);
    float4 g0 = x0, y0 = x0;
    if constexpr (kDy) g0 = lds128(ax + p1);
    if constexpr (kY) y0 = lds128(ax + p2);
    reduce_vec<DIR, EXTRA>(x0, g0, y0, slope, K, rm, rscale, rbeta, a0, b0);
  }
}

// One vector of the apply visit, in place.  Forward: x <- act(gamma*xhat + beta [+ residual]).  Backward:
// x <- dx = A*dz + B*(x - mean) + C0 and, with the residual epilogue, dy <- dz (the shortcut's gradient).
template <int DIR, bool EXTRA>
__device__ __forceinline__ void apply_vec(uint32_t ax, uint32_t p1, uint32_t p2, float4 vx, float4 vg, float4 ve, float slope,
                                          float mean, float scale, float beta, float cB, float cC)
{
  float x[4] = {vx.x, vx.y, vx.z, vx.w}, g[4] = {vg.x, vg.y, vg.z, vg.w};
  const float ex[4] = {ve.x, ve.y, ve.z, ve.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float d = x[e] - mean;
    const float yb = fmaf(d, scale, beta);
    if constexpr (DIR == 0) {
      x[e] = act(EXTRA ? yb + ex[e] : yb, slope);
    } else {
      const float t = EXTRA ? ex[e] : yb;
      const float dz = g[e] * (t > 0.0f ? 1.0f : slope);
      x[e] = fmaf(scale, dz, fmaf(cB, d, cC));
      g[e] = dz;
    }
  }
  sts128(ax, make_float4(x[0], x[1], x[2], x[3]));
  if constexpr (DIR == 1 && EXTRA) sts128(ax + p1, make_float4(g[0], g[1], g[2], g[3]));
  (void)p2;
}

// Apply visit of a piece: see apply_vec.  Planes: forward x [, residual]; backward x, dy [, saved output].
template <int DIR, bool EXTRA>
__device__ __forceinline__ void apply_piece(uint32_t sx, uint32_t plane_bytes, uint32_t nvec, float slope,
                                            float mean, float scale, float beta, float cB, float cC)
{
  constexpr uint32_t kStep = 32 * 16;
  constexpr bool kDy = DIR == 1;
  uint32_t v = threadIdx.x & 31;
  uint32_t ax = sx + v * 16;
  const uint32_t p1 = plane_bytes, p2 = 2 * plane_bytes;
  const uint32_t pe = DIR == 1 ? p2 : p1;             // where the extra tensor sits
  for (; v + 32 < nvec; v += 64, ax += 2 * kStep) {
    const float4 x0 = lds128(ax), x1 = lds128(ax + kStep);
    float4 g0 = x0, g1 = x1, e0 = x0, e1 = x1;
    if constexpr (kDy) { g0 = lds128(ax + p1); g1 = lds128(ax + p1 + kStep); }
    if constexpr (EXTRA) { e0 = lds128(ax + pe); e1 = lds128(ax + pe + kStep); }
    apply_vec<DIR, EXTRA>(ax, p1, p2, x0, g0, e0, slope, mean, scale, beta, cB, cC);
    apply_vec<DIR, EXTRA>(ax + kStep, p1, p2, x1, g1, e1, slope, mean, scale, beta, cB, cC);
  }
  if (v < nvec) {
    const float4 x0 = lds128(ax);
    float4 g0 = x0, e0 = x0;
    if constexpr (kDy) g0 = lds128(ax + p1);
    if constexpr (EXTRA) e0 = lds128(ax + pe);
    apply_vec<DIR, EXTRA>(ax, p1, p2, x0, g0, e0, slope, mean, scale, beta, cB, cC);
  }
}

// ---- coefficient warp: a channel's statistics ------------------------------------------------------
constexpr int kPullRegs = 5;       // partial records per lane: teams of up to 160 blocks

// Whole warp.  Waits for the records of channel c from all blocks of the team, merges them (and,
// with several GPUs, exchanges the per-GPU record) and returns the coefficients in every lane.
template <int DIR>
__device__ __forceinline__ bool pull_merge(const FusedArgs &a, const ResArgs &ra, Ctl *ctl, uint32_t c, bool owner, float4 &c0, float4 &c1)
{
  const uint32_t lane = threadIdx.x & 31, Gt = ra.g.Gt;
  const unsigned long long *rec = part_rec(a, ra, c, 0);
  const uint32_t epoch = ctl->epoch;
  // inputs that do not depend on the partials: fetch them while waiting
  const float gm = a.gamma ? a.gamma[c] : 1.0f;
  const float bt = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
  float mean_in = 0.f, var_in = 1.f;
  if constexpr (DIR == 1) { mean_in = a.mean_in[c]; var_in = a.var_in[c]; }
  double t0 = 0.0, t1 = 0.0, t2 = 0.0;           // forward: n, mean, M2; backward: -, sum dz, sum dz*(x-mean)
  const long long w0 = clock64();
  const bool local = (a.world <= 1) || owner;    // with several GPUs only the owner needs the local merge
  if (local) {
    unsigned long long r0[kPullRegs], r1[kPullRegs], r2[kPullRegs];
    for (;;) {
      bool all = true;
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        const uint32_t b = lane + 32u * i;
        if (b < Gt) {
          const unsigned long long *p = rec + (size_t)b * kResPartWords;
          r0[i] = ld_gpu_u64(p); r1[i] = ld_gpu_u64(p + 1);
          r2[i] = DIR == 0 ? ld_gpu_u64(p + 2) : r1[i];
          all = all && (uint32_t)(r0[i] >> 32) == epoch && (uint32_t)(r1[i] >> 32) == epoch && (uint32_t)(r2[i] >> 32) == epoch;
        } else { r0[i] = 0; r1[i] = 0; r2[i] = 0; }
      }
      if (__all_sync(0xffffffffu, all)) break;
      __nanosleep(64);
      uint32_t stop = 0;
      if (lane == 0) {
        if (ctl->abort) stop = 1;
        else if (clock64() - w0 > 2 * a.wait_cycles) { atomicOr(a.status, ANODE_ST_WAIT_STATS); ctl->abort = 1; stop = 1; }
      }
      if (__shfl_sync(0xffffffffu, stop, 0)) return false;
    }
    if constexpr (DIR == 0) {
      // two passes from registers: weighted mean, then M2 about it (fixed order: lane-major, then the shuffle tree)
      double sn = 0.0, sm = 0.0;
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        if (lane + 32u * i < Gt) {
          const double n = (double)(uint32_t)r0[i], m = (double)__uint_as_float((uint32_t)r1[i]);
          sn += n; sm = fma(n, m, sm);
        }
      }
      sn = warp_sum_all(sn); sm = warp_sum_all(sm);
      const double mean = sm / sn;
      double sq = 0.0;
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        if (lane + 32u * i < Gt) {
          const double n = (double)(uint32_t)r0[i], m = (double)__uint_as_float((uint32_t)r1[i]);
          const double d = m - mean;
          sq += (double)__uint_as_float((uint32_t)r2[i]) + n * d * d;
        }
      }
      sq = warp_sum_all(sq);
      t0 = sn; t1 = mean; t2 = sq;
    } else {
      double s1 = 0.0, s2 = 0.0;
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        if (lane + 32u * i < Gt) { s1 += (double)__uint_as_float((uint32_t)r0[i]); s2 += (double)__uint_as_float((uint32_t)r1[i]); }
      }
      t1 = warp_sum_all(s1); t2 = warp_sum_all(s2);
    }
  }
  if (a.world > 1) {
    // ---- exchange between GPUs.  A record is three 8-byte words (value in the low half, the call's
    // sequence number in the high half): every word validates itself, so plain peer stores suffice and
    // nothing is ever zeroed; consecutive calls alternate between two buffers.  Word 0 of a forward
    // record is the element count as an exact integer.
    const size_t slot = ((((size_t)(a.epoch & 1u)) * a.world) * a.xchg_channels + c) * 4;
    const size_t src_stride = (size_t)a.xchg_channels * 4;
    if (owner && lane < a.world) {
      const uint32_t w0b = DIR == 0 ? (uint32_t)t0 : __float_as_uint((float)t1);
      const uint32_t w1b = DIR == 0 ? __float_as_uint((float)t1) : __float_as_uint((float)t2);
      const uint32_t w2b = DIR == 0 ? __float_as_uint((float)t2) : 0u;
      unsigned long long *dst = a.xchg[lane] + slot + a.rank * src_stride;       // this rank's place in peer `lane`
      const unsigned long long e = (unsigned long long)a.epoch << 32;
      st_sys_u64(dst + 0, e | w0b); st_sys_u64(dst + 1, e | w1b); st_sys_u64(dst + 2, e | w2b);
    }
    const unsigned long long *mine = a.xchg[a.rank] + slot + (lane < a.world ? lane : 0) * src_stride;
    unsigned long long v0 = 0, v1 = 0, v2 = 0;
    for (;;) {
      bool ok = true;
      if (lane < a.world) {
        v0 = ld_sys_u64(mine); v1 = ld_sys_u64(mine + 1); v2 = ld_sys_u64(mine + 2);
        ok = (uint32_t)(v0 >> 32) == a.epoch && (uint32_t)(v1 >> 32) == a.epoch && (uint32_t)(v2 >> 32) == a.epoch;
      }
      if (__all_sync(0xffffffffu, ok)) break;
      __nanosleep(100);
      uint32_t stop = 0;
      if (lane == 0) {
        if (ctl->abort) stop = 1;
        else if (clock64() - w0 > a.wait_cycles) { atomicOr(a.status, ANODE_ST_WAIT_PEER); ctl->abort = 1; stop = 1; }
      }
      if (__shfl_sync(0xffffffffu, stop, 0)) return false;
    }
    // merge in rank order (lane = rank; the shuffle tree is the same on every GPU: bit-identical statistics)
    const bool live = lane < a.world;
    if constexpr (DIR == 0) {
      const double n = live ? (double)(uint32_t)v0 : 0.0, m = live ? (double)__uint_as_float((uint32_t)v1) : 0.0;
      const double sn = warp_sum_all(n), sm = warp_sum_all(n * m);
      const double mean = sm / sn, d = m - mean;
      const double sq = warp_sum_all(live ? (double)__uint_as_float((uint32_t)v2) + n * d * d : 0.0);
      t0 = sn; t1 = mean; t2 = sq;
    } else {
      t1 = warp_sum_all(live ? (double)__uint_as_float((uint32_t)v0) : 0.0);
      t2 = warp_sum_all(live ? (double)__uint_as_float((uint32_t)v1) : 0.0);
    }
  }
  if constexpr (DIR == 0) {
    const float mf = (float)t1;
    const float vf = (float)(t2 / t0 + (double)a.epsilon);       // biased, epsilon folded in (batch_norm.cu:160)
    c0 = make_float4(mf, gm * inv_std(vf), bt, 0.f);
    c1 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (owner && lane == 0) {
      a.mean[c] = mf; a.var[c] = vf;
      // running statistics: y <- y + rate*(x - y)  (OnlineAverageOp; reference tests/test_gpu.rs:561-593)
      if (a.run_mean) { const float o = a.run_mean[c]; a.run_mean[c] = o + a.avg_rate * (mf - o); }
      if (a.run_var) { const float o = a.run_var[c]; a.run_var[c] = o + a.avg_rate * (vf - o); }
    }
  } else {
    const float r = inv_std(var_in);
    const double rs2 = (double)r * t2;                           // sum(dz * xhat)
    const double A = (double)gm * (double)r;
    const double invM = 1.0 / a.count_total;
    c0 = make_float4(mean_in, gm * r, bt, 0.f);
    c1 = make_float4((float)(-A * (double)r * rs2 * invM), (float)(-A * t1 * invM), 0.f, 0.f);
    if (owner && lane == 0) {
      if (a.dbeta) a.dbeta[c] = (float)t1;
      if (a.dgamma) a.dgamma[c] = (float)rs2;
    }
  }
  return true;
}

// ---- the kernel -------------------------------------------------------------------------------------
template <int DIR, bool EXTRA>
__global__ void __launch_bounds__(kResThreads, 1) bn_resident_kernel(const FusedArgs a, const ResArgs ra)
{
  constexpr uint32_t W = kCWarps;
  extern __shared__ __align__(128) unsigned char sm[];
  Ctl *ctl = reinterpret_cast<Ctl *>(sm);
  const ResPlan &g = ra.g;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t *status = a.status;
  uint32_t *hdr = reinterpret_cast<uint32_t *>(a.ws);      // [3]: launches of this kernel so far, [4]: exit counter
  // a wait that depends on another wait gets the longer bound, so that the status word names the root cause
  const long long limit = 3 * a.wait_cycles;
  const ResBlock rb = res_block(g, blockIdx.x);
  const uint32_t slots0 = s32(sm + kResCtlBytes);

  if (tid == 0) {
    for (uint32_t i = 0; i < g.Q; ++i) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->done[i], 1); mbar_init(&ctl->empty[i], 1); }
    for (uint32_t i = 0; i < kResQ; ++i) { mbar_init(&ctl->res_full[i], W); mbar_init(&ctl->res_empty[i], 1); }
    for (uint32_t i = 0; i < kCoefQ; ++i) { mbar_init(&ctl->coef_full[i], 1); mbar_init(&ctl->coef_empty[i], W); }
    ctl->abort = 0; ctl->last_block = 0; ctl->issued = 0;
    ctl->epoch = hdr[3] + 1u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  for (uint32_t t = tid; t < rb.Tb; t += blockDim.x) {
    const ResPiece pc = res_piece(g, rb.u0 + t);
    ctl->ptab[t] = make_uint2((uint32_t)((((uint64_t)pc.n0 * g.C) * g.dim0 + pc.col0) / 4), (pc.rows << 16) | pc.len);
  }
  __syncthreads();
  const size_t row_stride = (size_t)g.C * g.dim0;        // floats between consecutive samples of a channel

  if (warp < W) {
    // ------------------------------------------------------------------ consumers
    // Piece visits go to the consumer warps in turn: a warp handles a whole piece by itself, so W pieces
    // are being worked on at any time and a visit's fixed costs (barrier, table lookup, loop start) are
    // paid by one warp, not by all of them.
    const float slope = a.neg_slope;
    uint64_t fpar = 0;                       // per slot: parity of the next load to wait for
    uint32_t npub = 0, ncoef = 0, visit = 0, nload = 0;
    uint32_t cur_k = 0xffffffffu;            // channel being reduced
    uint32_t cnt = 0;                        // elements this warp has reduced of the current channel
    float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f, K = 0.f;
    float rm = 0.f, rscale = 1.f, rbeta = 0.f;           // backward: what the mask needs, of the channel being reduced
    float nm = 0.f, nv = 1.f, ng = 1.f, nb = 0.f;        // the same inputs of the next channel, fetched ahead
    float mean = 0.f, scale = 1.f, beta = 0.f, cB = 0.f, cC = 0.f;     // of the channel being applied
    auto fetch = [&](uint32_t k) {
      if constexpr (DIR == 1) {
        if (k < rb.K) {
          const uint32_t c = rb.team + k * g.teams;
          nm = a.mean_in[c]; nv = a.var_in[c];
          ng = a.gamma ? a.gamma[c] : 1.0f;
          nb = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
        }
      }
    };
    fetch(0);
    res_walk(g, rb, [&](const ResEvent &e) -> bool {
      const uint64_t bit = 1ull << e.slot;
      switch (e.kind) {
        case EV_RED_STR:
        case EV_RED_RES: {
          const uint32_t par = (uint32_t)((fpar >> e.slot) & 1ull);
          fpar ^= bit;
          const uint32_t m = nload++;
          if constexpr (DIR == 1) {
            if (e.k != cur_k) { cur_k = e.k; rm = nm; rscale = ng * inv_std(nv); rbeta = nb; fetch(e.k + 1); }
          }
          if ((visit++ & (W - 1)) != warp) return true;
          if (!wait_load(ctl, e.slot, par, m, status, limit)) return false;
          const uint32_t sx = slots0 + e.slot * g.slot_bytes;
          const PieceRef pc = piece_ref(ctl, e.piece);
          const uint32_t nvec = pc.rows * pc.len / 4;
          if constexpr (DIR == 0) {
            // the shift of this warp's sums: the first element it meets in the channel
            if (cnt == 0) K = lds128(sx).x;
          }
          cnt += nvec * 4;
          reduce_piece<DIR, EXTRA>(sx, g.plane_bytes, nvec, slope, K, rm, rscale, rbeta, a0, a1, b0, b1);
          if (e.kind == EV_RED_STR) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->done[e.slot]);
          }
          return true;
        }
        case EV_PUBLISH: {
          const uint32_t q = npub % kResQ, qpar = (npub / kResQ) & 1u; ++npub;
          if (!warp_wait(&ctl->res_empty[q], qpar ^ 1u, ctl, status, limit)) return false;
          const float s = warp_sum(a0 + a1), t = warp_sum(b0 + b1);
          if (lane == 0) { ctl->res[q][warp] = make_float4(s, t, K, __uint_as_float(cnt)); mbar_arrive(&ctl->res_full[q]); }
          a0 = a1 = b0 = b1 = 0.f; cnt = 0;
          return true;
        }
        case EV_NEED_COEF: {
          const uint32_t q = ncoef % kCoefQ, qpar = (ncoef / kCoefQ) & 1u; ++ncoef;
          if (!warp_wait(&ctl->coef_full[q], qpar, ctl, status, limit)) return false;
          const float4 c0 = ctl->coef[q][0], c1 = ctl->coef[q][1];
          mean = c0.x; scale = c0.y; beta = c0.z; cB = c1.x; cC = c1.y;
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->coef_empty[q]);
          return true;
        }
        default: {   // EV_APP_STR, EV_APP_RES
          const uint32_t par = (uint32_t)((fpar >> e.slot) & 1ull);
          uint32_t m = 0;
          if (e.kind == EV_APP_STR) { fpar ^= bit; m = nload++; }
          if ((visit++ & (W - 1)) != warp) return true;
          if (e.kind == EV_APP_STR) {
            if (!wait_load(ctl, e.slot, par, m, status, limit)) return false;
          }
          const uint32_t sx = slots0 + e.slot * g.slot_bytes;
          const PieceRef pc = piece_ref(ctl, e.piece);
          const uint32_t nvec = pc.rows * pc.len / 4;
          apply_piece<DIR, EXTRA>(sx, g.plane_bytes, nvec, slope, mean, scale, beta, cB, cC);
          fence_async_smem();          // the bulk store reads what this thread just wrote
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->done[e.slot]);
          return true;
        }
      }
    });
  } else if (warp == W) {
    // ------------------------------------------------------------------ loader
    const uint64_t keep = policy_keep(), drop = policy_drop();
    uint64_t used = 0, epar = 0, lpar = 0;     // per slot: loaded before; parity of the next `empty` phase; parity of the last load
    uint32_t nload = 0;
    res_walk(g, rb, [&](const ResEvent &e) -> bool {
      if (e.kind != EV_RED_STR && e.kind != EV_RED_RES && e.kind != EV_APP_STR) return true;
      const uint64_t bit = 1ull << e.slot;
      if (used & bit) {
        if (!warp_wait(&ctl->empty[e.slot], (uint32_t)((epar >> e.slot) & 1ull), ctl, status, limit)) return false;
        epar ^= bit;
        lpar ^= bit;
      }
      used |= bit;
      const PieceRef pc = piece_ref(ctl, e.piece);
      const size_t base = pc.off + (size_t)(rb.team + e.k * g.teams) * g.dim0;
      const uint32_t row_bytes = pc.len * 4;
      const uint32_t sx = slots0 + e.slot * g.slot_bytes;
      if (lane == 0) mbar_arrive_expect_tx(&ctl->full[e.slot], row_bytes * pc.rows * g.planes);
      __syncwarp();
      // streamed pieces are asked to stay in L2 until their second visit; everything else is read once
      const uint64_t pol = e.kind == EV_RED_STR ? keep : drop;
      const float *extra = DIR == 0 ? a.res : a.ymask;
      for (uint32_t r = lane; r < pc.rows; r += 32) {
        const size_t off = base + r * row_stride;
        const uint32_t dst = sx + r * row_bytes;
        bulk_g2s(dst, a.x + off, row_bytes, &ctl->full[e.slot], pol);
        if constexpr (DIR == 1) bulk_g2s(dst + g.plane_bytes, a.dy + off, row_bytes, &ctl->full[e.slot], pol);
        if constexpr (EXTRA) bulk_g2s(dst + (DIR == 1 ? 2u : 1u) * g.plane_bytes, extra + off, row_bytes, &ctl->full[e.slot], pol);
      }
      // consumers look at a slot's barrier only once its load has been issued (see wait_load)
      __syncwarp();
      ++nload;
      if (lane == 0) { __threadfence_block(); ctl->issued = nload; }
      return true;
    });
    // after an abort: wait (bounded) for copies that were issued but will not be consumed
    if (ctl->abort && lane == 0) {
      for (uint32_t s = 0; s < g.Q; ++s) {
        if (!((used >> s) & 1ull)) continue;
        const long long t0 = clock64();
        while (!mbar_test(&ctl->full[s], (uint32_t)((lpar >> s) & 1ull)) && clock64() - t0 < limit / 8) {}
      }
    }
  } else if (warp == W + 1) {
    // ------------------------------------------------------------------ storer
    const uint64_t drop = policy_drop();
    uint64_t dpar = 0;                         // per slot: parity of the next `done` phase
    uint32_t pend[2] = {0, 0}, np = 0;         // slots whose store may still be reading shared memory (oldest first)
    auto flush = [&]() {
      bulk_wait_read<0>();
      __syncwarp();
      if (lane == 0) for (uint32_t i = 0; i < np; ++i) mbar_arrive(&ctl->empty[pend[i]]);
      np = 0;
    };
    res_walk(g, rb, [&](const ResEvent &e) -> bool {
      if (e.kind != EV_RED_STR && e.kind != EV_APP_STR && e.kind != EV_APP_RES) return true;
      const uint64_t bit = 1ull << e.slot;
      const uint32_t par = (uint32_t)((dpar >> e.slot) & 1ull);
      if (!mbar_test(&ctl->done[e.slot], par)) {
        // about to sleep: first hand back every slot whose store has been read out, so that nobody
        // waits for a slot this warp is sitting on
        if (np) flush();
        if (!warp_wait(&ctl->done[e.slot], par, ctl, status, limit)) return false;
      }
      dpar ^= bit;
      if (e.kind == EV_RED_STR) {
        if (lane == 0) mbar_arrive(&ctl->empty[e.slot]);
        return true;
      }
      const PieceRef pc = piece_ref(ctl, e.piece);
      const size_t base = pc.off + (size_t)(rb.team + e.k * g.teams) * g.dim0;
      const uint32_t row_bytes = pc.len * 4;
      const uint32_t sx = slots0 + e.slot * g.slot_bytes;
      for (uint32_t r = lane; r < pc.rows; r += 32) {
        bulk_s2g(a.out + base + r * row_stride, sx + r * row_bytes, row_bytes, drop);
        if constexpr (DIR == 1 && EXTRA) { if (a.dres) bulk_s2g(a.dres + base + r * row_stride, sx + g.plane_bytes + r * row_bytes, row_bytes, drop); }
      }
      bulk_commit();
      if (np == 2) {
        // all but the two youngest stores have been read out of shared memory: the oldest slot is free
        bulk_wait_read<2>();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->empty[pend[0]]);
        pend[0] = pend[1]; np = 1;
      }
      pend[np++] = e.slot;
      return true;
    });
    flush();          // shared memory must not be released while a store still reads it
  } else if (warp == W + 2) {
    // ------------------------------------------------------------------ delivery warp
    const unsigned long long tag = (unsigned long long)ctl->epoch << 32;
    uint32_t npub = 0;
    res_walk(g, rb, [&](const ResEvent &e) -> bool {
      if (e.kind != EV_PUBLISH) return true;
      const uint32_t q = npub % kResQ, qpar = (npub / kResQ) & 1u; ++npub;
      if (!warp_wait(&ctl->res_full[q], qpar, ctl, status, limit)) return false;
      const float4 v = lane < W ? ctl->res[q][lane] : make_float4(0.f, 0.f, 0.f, 0.f);
      double r0 = 0.0, r1 = 0.0, r2 = 0.0;
      if constexpr (DIR == 0) {
        // per warp: sums of (x - K) and (x - K)^2 over n elements -> (n, mean, M2); then the usual two
        // passes over the W records (weighted mean, M2 about it), in a fixed order
        const double n = (double)__float_as_uint(v.w), s = (double)v.x, t = (double)v.y;
        const double m = n > 0.0 ? (double)v.z + s / n : 0.0;
        const double m2 = n > 0.0 ? fmax(t - s * s / n, 0.0) : 0.0;
        const double sn = warp_sum_all(n), sm = warp_sum_all(n * m);
        const double mean = sm / sn, d = m - mean;
        r0 = sn; r1 = mean; r2 = warp_sum_all(m2 + n * d * d);
      } else {
        r0 = warp_sum_all((double)v.x); r1 = warp_sum_all((double)v.y);
      }
      if (lane == 0) {
        unsigned long long *rec = part_rec(a, ra, rb.team + e.k * g.teams, rb.b);
        if constexpr (DIR == 0) {
          st_gpu_u64(rec + 0, tag | (uint32_t)r0);
          st_gpu_u64(rec + 1, tag | __float_as_uint((float)r1));
          st_gpu_u64(rec + 2, tag | __float_as_uint((float)r2));
        } else {
          st_gpu_u64(rec + 0, tag | __float_as_uint((float)r0));
          st_gpu_u64(rec + 1, tag | __float_as_uint((float)r1));
        }
        mbar_arrive(&ctl->res_empty[q]);
      }
      return true;
    });
  } else {
    // ------------------------------------------------------------------ coefficient warp
    uint32_t ncoef = 0;
    res_walk(g, rb, [&](const ResEvent &e) -> bool {
      if (e.kind != EV_NEED_COEF) return true;
      const uint32_t q = ncoef % kCoefQ, qpar = (ncoef / kCoefQ) & 1u; ++ncoef;
      if (!warp_wait(&ctl->coef_empty[q], qpar ^ 1u, ctl, status, limit)) return false;
      float4 c0, c1;
      // the channel's owner writes the per-channel outputs (and ships this GPU's record to the peers)
      if (!pull_merge<DIR>(a, ra, ctl, rb.team + e.k * g.teams, rb.b == e.k % g.Gt, c0, c1)) return false;
      if (lane == 0) { ctl->coef[q][0] = c0; ctl->coef[q][1] = c1; mbar_arrive(&ctl->coef_full[q]); }
      return true;
    });
  }

  // ---- leave: the last block out advances the workspace's launch counter
  __syncthreads();
  if (ctl->abort) {
    if (tid == 0) atomicOr(status, ANODE_ST_ABORTED);
    return;
  }
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(hdr + 4, 1u) + 1 == gridDim.x) { hdr[3] = ctl->epoch; hdr[4] = 0; }
  }
}

}  // namespace res

// ---- host side ----------------------------------------------------------------------------------------
static std::atomic<uint32_t> g_wait_ms{1500};

long long wait_limit_cycles()
{
  // device clock64 ticks at the SM clock (about 2 GHz at most): the bound is approximate by design
  return (long long)g_wait_ms.load(std::memory_order_relaxed) * 2000000ll;
}

// Planner inputs, from measurements on B200: bytes of reduce work that should separate the end of a
// channel's reduction from the first use of its statistics, bytes of the streaming ring, and bytes of
// loads in flight ahead of the resident ring's reduce visits.
constexpr uint32_t kResCoverBytes = 48 * 1024, kResStreamBytes = 48 * 1024, kResAheadBytes = 48 * 1024;

static uint32_t res_planes(const FusedArgs &a, int dir) { return (dir == 1 ? 2u : 1u) + ((dir == 0 ? a.res : a.ymask) ? 1u : 0u); }

bool resident_plan_for(uint32_t dim0, uint32_t C, uint32_t N, uint32_t planes, ResPlan &p)
{
  return make_res_plan(dim0, C, N, planes, sm_count(), kResCoverBytes, kResStreamBytes, kResAheadBytes, p);
}

// Bytes the kernel's partial records may take in a direction's workspace part, whatever plan is chosen.
uint64_t resident_ws_bytes(uint32_t dim0, uint32_t C, uint32_t N)
{
  uint64_t need = 0;
  for (uint32_t planes = 1; planes <= 3; ++planes) {
    ResPlan p;
    if (resident_plan_for(dim0, C, N, planes, p) && p.ws_bytes > need) need = p.ws_bytes;
  }
  return need;
}

bool resident_applies(const FusedArgs &a, int dir, bool aligned)
{
  // (accumulating into dx would need a read of dx: the tiled and plain kernels do that)
  if (!aligned || a.mode != MODE_FUSED || a.accumulate) return false;
  if (dir == 0 ? (a.ymask || a.dres) : (a.res != nullptr)) return false;
  if (dir == 1 && a.dres && !a.ymask) return false;
  ResPlan p;
  return resident_plan_for(a.plan.dim0, a.plan.C, a.plan.N, res_planes(a, dir), p);
}

typedef void (*ResKernel)(const FusedArgs, const res::ResArgs);

int launch_resident(FusedArgs &a, int dir, uint64_t ws_off, cudaStream_t stream)
{
  res::ResArgs ra{};
  if (!resident_plan_for(a.plan.dim0, a.plan.C, a.plan.N, res_planes(a, dir), ra.g)) return ANODE_E_LAUNCH;
  if (ws_off + ra.g.ws_bytes > a.ws_capacity) return ANODE_E_WORKSPACE;
  const bool extra = (dir == 0 ? a.res : a.ymask) != nullptr;
  ResKernel k = dir == 0 ? (extra ? res::bn_resident_kernel<0, true> : res::bn_resident_kernel<0, false>)
                         : (extra ? res::bn_resident_kernel<1, true> : res::bn_resident_kernel<1, false>);
  ra.ws_off = (uint32_t)ws_off;
  static std::mutex mu;
  static std::map<std::pair<const void *, int>, int> ready;      // (kernel, device) -> shared-memory attribute set
  {
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    (void)cudaGetDevice(&dev);
    const auto key = std::make_pair((const void *)k, dev);
    if (!ready.count(key)) {
      if (cudaFuncSetAttribute((const void *)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kResSmemBudget) != cudaSuccess) {
        (void)cudaGetLastError();
        return ANODE_E_LAUNCH;
      }
      ready[key] = 1;
    }
  }
  void *params[] = {(void *)&a, (void *)&ra};
  // blocks wait on one another's records: all of them must be resident, which a cooperative launch checks
  if (cudaLaunchCooperativeKernel((const void *)k, dim3(ra.g.grid), dim3(res::kResThreads), params, ra.g.smem_bytes, stream) != cudaSuccess) {
    (void)cudaGetLastError();
    return ANODE_E_LAUNCH;
  }
  return ANODE_OK;
}

}  // namespace anode_b200

using namespace anode_b200;

extern "C" int anode_gpu_batch_norm_fused_set_wait_limit_ms(uint32_t ms)
{
  if (ms == 0) return ANODE_E_DIMS;
  g_wait_ms.store(ms, std::memory_order_relaxed);
  return ANODE_OK;
}

