// Warp-specialised version of the fused batch-norm pipeline for the 128-bit paths.
//
// Same algorithm as bn_fused.cuh (reduce a tile, complete its unit, apply the tile a bounded
// number of steps later), but no consumer thread ever waits on global memory:
//
//   producer warp    walks the block's schedule and streams tiles into a ring of shared-memory
//                    slots with bulk asynchronous copies (cp.async.bulk + mbarrier), tagged
//                    with L2 eviction hints: "keep" for the reduce visit, "drop" for the
//                    apply visit.  The ring keeps HBM requests in flight while everything
//                    else happens.
//   consumer warps   (8) read slots with 128-bit shared loads, accumulate / normalise, write
//                    results with 128-bit streaming stores, and hand partials to the delivery
//                    warp through a shared-memory mailbox.  In regime R every warp works on its
//                    own share of a tile and never synchronises with the other warps.
//   delivery warp    merges the consumer warps' partials of a tile and stores them as ONE tagged
//                    8-byte word per tile in the workspace (no counter, no fence, no atomic).
//   coefficient warp polls, for each upcoming apply visit, the partial words of the visit's
//                    channel until none is zero, merges them in a fixed order in double
//                    precision (every block obtains bit-identical coefficients; with several
//                    GPUs the owner block exchanges per-GPU records with the peers here) and
//                    stages the visit's coefficients in a second mailbox.
//                    (In the three-launch form of the synchronized calls the reduce launch still counts
//                    partials per unit and the apply launch reads prepared coefficients.)
//
// Every wait is bounded: a wait that runs out sets a status bit, raises the block's abort flag
// and all three roles drain and leave.
// This header has no include guard on purpose: it is included once per consumer-warp count, with
// ANODE_RING_NS naming the namespace of the instantiation and ANODE_RING_CONSUMERS the number of
// consumer threads (the forward pass runs best with 8 consumer warps, the backward pass with 16).
#include "bn_fused.cuh"

#if !defined(ANODE_RING_NS) || !defined(ANODE_RING_CONSUMERS)
#error "define ANODE_RING_NS and ANODE_RING_CONSUMERS before including bn_ring.cuh"
#endif
#ifndef ANODE_RING_STORE
#define ANODE_RING_STORE 1      // 0: store with an L2 evict-first hint, 1: st.global.cs, 2: plain store
#endif
#ifndef ANODE_RING_BACKOFF_NS
#define ANODE_RING_BACKOFF_NS 100
#endif
#ifndef ANODE_RING_COPY_BYTES
#define ANODE_RING_COPY_BYTES 32768
#endif

namespace anode_b200 {
namespace ANODE_RING_NS {

constexpr uint32_t kConsumers = ANODE_RING_CONSUMERS;   // consumer threads (a power of two, 256..1024)
constexpr uint32_t kRingThreads = kConsumers + 96;   // + producer, delivery and coefficient warps
constexpr uint32_t kCopyBytes = ANODE_RING_COPY_BYTES;   // size of one bulk copy (a multiple of 16)
constexpr long long kWaitCycles = 3000000000ll;      // about 1.5 s at 2 GHz

struct RingCtl {
  unsigned long long full[kMaxSlots], empty[kMaxSlots];
  unsigned long long res_full[kResQ], res_empty[kResQ];
  unsigned long long coef_full[kCoefQ], coef_empty[kCoefQ];
  float mom[3 * (kConsumers / 32)];
  volatile uint32_t abort;
  uint32_t last_block;
  uint32_t parity;       // which of the two tagged-partial buffers this launch uses
};
static_assert(sizeof(RingCtl) <= kRingCtlBytes, "RingCtl outgrew the room reserved for it");

// ---- mbarrier / bulk-copy primitives --------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned long long *bar, uint32_t parity)
{
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try(unsigned long long *bar, uint32_t parity)
{
  uint32_t ok;
  // the last operand lets the hardware keep the thread suspended (up to that many nanoseconds)
  // until the phase completes, instead of returning early to a polling loop
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(100000u) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after raising the abort flag) when the barrier did not flip in time
// or when another role already gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, uint32_t parity, RingCtl *ctl, uint32_t *status, uint32_t bit)
{
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    // back off: a spinning waiter takes issue slots from the warps that do the work
    __nanosleep(ANODE_RING_BACKOFF_NS);
    if ((++it & 15u) == 0u) {
      if (ctl->abort) return false;
      if (clock64() - t0 > kWaitCycles) {
        atomicOr(status, bit);
        ctl->abort = 1;
        return false;
      }
    }
  }
}
// Every lane gets the same answer.  The common case, a phase that is already complete (or completes while the
// hardware holds the warp), is one instruction for the whole warp; only a wait that outlasts that is handed to
// one lane, which polls with the time limit.
__device__ __forceinline__ bool warp_wait(unsigned long long *bar, uint32_t parity, RingCtl *ctl, uint32_t *status, uint32_t bit)
{
  if (__all_sync(0xffffffffu, mbar_try(bar, parity))) return true;
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, ctl, status, bit) ? 1u : 0u;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// global -> shared bulk copy, completion counted on `bar`; bytes and both addresses are multiples of 16
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, unsigned long long *bar, uint64_t policy)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
// ---- the block's schedule --------------------------------------------------------------------
// Operation k of a block: steps s = 0, 1, ...; at step s first REDUCE tile s (if any is left), then
// APPLY tile s - look (if s >= look).  Every role walks this same sequence with its own cursor.
struct Sched {
  uint32_t my_tiles, look, b, G;
  bool do_reduce, do_apply;
  uint32_t s, phase;     // phase 0: reduce of step s pending; 1: apply of step s pending
  TileIter it_reduce, it_apply;     // the reduce visits and the apply visits both walk b, b+G, ...
  __device__ __forceinline__ void init(const FusedArgs &a)
  {
    b = blockIdx.x; G = gridDim.x;
    my_tiles = (b < a.plan.total_tiles) ? (a.plan.total_tiles - b + G - 1) / G : 0;
    look = (a.mode == MODE_FUSED) ? a.plan.lookahead_steps : 0;
    do_reduce = a.mode != MODE_APPLY; do_apply = a.mode != MODE_STATS;
    s = 0; phase = 0;
    it_reduce.init(a.plan, b, G); it_apply.init(a.plan, b, G);
  }
  // Same walk, but hands out the tile's range without any per-tile division.
  __device__ __forceinline__ bool next_range(const Plan &P, uint32_t &kind, TileRange &tr)
  {
    for (;;) {
      if (s >= my_tiles + look) return false;
      if (phase == 0) {
        phase = 1;
        if (do_reduce && s < my_tiles) { kind = 0; tr = it_reduce.range(P); it_reduce.advance(P); return true; }
      } else {
        phase = 0;
        const uint32_t ss = s++;
        if (do_apply && ss >= look) { kind = 1; tr = it_apply.range(P); it_apply.advance(P); return true; }
      }
    }
  }
  // Advances to the next operation; returns false at the end.  kind: 0 reduce, 1 apply.
  __device__ __forceinline__ bool next(uint32_t &kind, uint32_t &tile)
  {
    for (;;) {
      if (s >= my_tiles + look) return false;
      if (phase == 0) {
        phase = 1;
        if (do_reduce && s < my_tiles) { kind = 0; tile = b + s * G; return true; }
      } else {
        phase = 0;
        const uint32_t ss = s++;
        if (do_apply && ss >= look) { kind = 1; tile = b + (ss - look) * G; return true; }
      }
    }
  }
};


// dynamic shared memory accessors
__device__ __forceinline__ float *slot_x(unsigned char *sm, const RingGeom &g, uint32_t slot) { return reinterpret_cast<float *>(sm + g.off_slots + (size_t)slot * g.slot_stride); }
template <int DIR> __device__ __forceinline__ float *slot_dy(unsigned char *sm, const RingGeom &g, uint32_t slot) { return slot_x(sm, g, slot) + g.slot_floats; }
template <int DIR> __device__ __forceinline__ float4 *slot_side(unsigned char *sm, const RingGeom &g, uint32_t slot)
{
  return reinterpret_cast<float4 *>(slot_x(sm, g, slot) + (DIR == 1 ? 2 : 1) * g.slot_floats);
}
__device__ __forceinline__ float4 *res_box(unsigned char *sm, const RingGeom &g, uint32_t q) { return reinterpret_cast<float4 *>(sm + g.off_res) + (size_t)q * g.res_stride; }
__device__ __forceinline__ float4 *coef_box(unsigned char *sm, const RingGeom &g, uint32_t cb, uint32_t q) { return reinterpret_cast<float4 *>(sm + g.off_coef) + (size_t)q * cb * 2; }

// ======================================================================================
// consumer side
// ======================================================================================
// ---- each consumer warp handles vectors warp*32 + lane + i*256 of the tile ----------
constexpr uint32_t kCWarps = kConsumers / 32;
constexpr uint32_t kPerTurn = 32 / kCWarps;      // mailbox entries the delivery warp merges per turn

// 128-bit shared load by 32-bit shared address (keeps the address arithmetic in 32 bits)
__device__ __forceinline__ Pack<4> lds128(uint32_t saddr)
{
  Pack<4> r;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]) : "r"(saddr) : "memory");
  return r;
}
constexpr uint32_t kVecStride = kConsumers * 16;     // bytes between consecutive vectors of one thread

template <int DIR>
__device__ __forceinline__ void warp_reduce_R(const FusedArgs &a, const RingGeom &g, unsigned char *sm, RingCtl *ctl,
                                              const TileRange &tr, uint32_t slot, float4 *res)
{
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t nvec = (tr.len / 4) * tr.rows;        // the slot holds the tile's rows back to back
  const uint32_t cnt = tid < nvec ? (nvec - tid + kConsumers - 1) / kConsumers : 0;   // this thread's vectors
  uint32_t ax = smem_u32(slot_x(sm, g, slot)) + tid * 16;
  if constexpr (DIR == 0) {
    // shifted sums (see bn_fused.cuh), two accumulator pairs
    // K: the first element of the warp's share (lane 0 has the lowest vector index, so it has a
    // vector whenever any lane has one).  One shift per warp makes s and q plain sums over lanes.
    float K = cnt ? lds128(ax).v[0] : 0.f;
    K = __shfl_sync(0xffffffffu, K, 0);
    float s0 = 0.f, q0 = 0.f, s1 = 0.f, q1 = 0.f;
    uint32_t i = 0;
    for (; i + 4 <= cnt; i += 4, ax += 4 * kVecStride) {
      const Pack<4> v0 = lds128(ax), v1 = lds128(ax + kVecStride), v2 = lds128(ax + 2 * kVecStride), v3 = lds128(ax + 3 * kVecStride);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float d0 = v0.v[e] - K, d1 = v1.v[e] - K, d2 = v2.v[e] - K, d3 = v3.v[e] - K;
        s0 += d0; q0 = fmaf(d0, d0, q0); s1 += d1; q1 = fmaf(d1, d1, q1);
        s0 += d2; q0 = fmaf(d2, d2, q0); s1 += d3; q1 = fmaf(d3, d3, q1);
      }
    }
    for (; i + 2 <= cnt; i += 2, ax += 2 * kVecStride) {
      const Pack<4> v0 = lds128(ax), v1 = lds128(ax + kVecStride);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float d0 = v0.v[e] - K, d1 = v1.v[e] - K;
        s0 += d0; q0 = fmaf(d0, d0, q0); s1 += d1; q1 = fmaf(d1, d1, q1);
      }
    }
    if (i < cnt) {
      const Pack<4> v0 = lds128(ax);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float d0 = v0.v[e] - K; s0 += d0; q0 = fmaf(d0, d0, q0); }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ctl->empty[slot]);
    const float s = warp_sum(s0 + s1), q = warp_sum(q0 + q1);
    const uint32_t nw = __reduce_add_sync(0xffffffffu, cnt * 4);
    if (lane == 0) {
      Moments m{0.f, 0.f, 0.f};
      if (nw) {
        m.n = (float)nw;
        const float inv = __fdividef(1.0f, m.n);
        m.mean = fmaf(s, inv, K);
        m.m2 = fmaxf(q - s * s * inv, 0.f);
      }
      res[warp] = make_float4(m.n, m.mean, m.m2, 0.f);
    }
  } else {
    uint32_t ad = ax + g.slot_floats * 4;
    const float4 cf = slot_side<1>(sm, g, slot)[0];
    const float mean = cf.x, scale = cf.y, beta = cf.z;
    const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
    float s1 = 0.f, s2 = 0.f;
    // (one vector per tensor at a time: with two in flight the sixteen warps of this pass were measured slower)
    for (uint32_t i = 0; i < cnt; ++i, ax += kVecStride, ad += kVecStride) {
      const Pack<4> x0 = lds128(ax), g0 = lds128(ad);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float d0 = x0.v[e] - mean;
        const float y0 = fmaf(d0, scale, beta);
        // dz = dy * (float)(y > 0)  (routines_gpu/flat_map.cu:191-192)
        const float z0 = g0.v[e] * (y0 > 0.0f ? 1.0f : slope);
        s1 += z0; s2 = fmaf(z0, d0, s2);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ctl->empty[slot]);
    s1 = warp_sum(s1); s2 = warp_sum(s2);
    if (lane == 0) res[warp] = make_float4(s1, s2, 0.f, 0.f);
  }
}

template <int DIR>
__device__ __forceinline__ void warp_apply_R(const FusedArgs &a, const RingGeom &g, unsigned char *sm, RingCtl *ctl,
                                             const TileRange &tr, uint32_t slot, const float4 *coef, uint32_t coef_q)
{
  const uint32_t tid = threadIdx.x, lane = tid & 31;
  const float slope = a.neg_slope;      // activation: t * (t > 0 ? 1 : slope)
  const bool acc = a.accumulate != 0;
  const uint64_t drop = policy_drop();
  const uint64_t rs = (uint64_t)a.plan.C * a.plan.dim0;
  float *out = a.out + tr.base;
  const float4 c0 = coef[0], c1 = coef[1];
  const float mean = c0.x, scale = c0.y, beta = c0.z, cB = c1.x, cC = c1.y;
  const uint32_t per_row = tr.len / 4, nvec = per_row * tr.rows;
  const uint32_t cnt = tid < nvec ? (nvec - tid + kConsumers - 1) / kConsumers : 0;
  uint32_t ax = smem_u32(slot_x(sm, g, slot)) + tid * 16;
  uint32_t ad = ax + g.slot_floats * 4;
  // The thread's vectors are tid, tid + kConsumers, ... of the tile's rows laid back to back; their places in
  // global memory are found by walking (column, row) along, without a division or a 64-bit product per vector.
  uint32_t col = tid, row = 0;
  if (tr.rows > 1) { row = fast_div(tid, a.plan.div_mul); col = tid - row * per_row; }   // rows > 1 only occurs with whole rows, where per_row matches div_mul
  float *dst = out + (size_t)row * rs + 4 * (size_t)col;
  const uint32_t step_rows = tr.rows > 1 ? fast_div(kConsumers, a.plan.div_mul) : 0;     // kConsumers = step_rows * per_row + step_cols
  const uint32_t step_cols = kConsumers - step_rows * per_row;
  const size_t step_ptr = (size_t)step_rows * rs + 4 * (size_t)step_cols;               // floats from one vector of the thread to the next
  const size_t wrap_ptr = rs - 4 * (size_t)per_row;                                      // on top of that when the column wraps into the next row
  auto advance = [&]() {
    dst += step_ptr; col += step_cols;
    if (col >= per_row) { col -= per_row; dst += wrap_ptr; }
  };
  // one vector: o = activation(bn(x)) or the input gradient
  auto one = [&](const Pack<4> &vx, const Pack<4> &vd, float *p) {
    Pack<4> o;
    if constexpr (DIR == 0) {
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float yb = fmaf(vx.v[e] - mean, scale, beta); o.v[e] = yb * (yb > 0.0f ? 1.0f : slope); }
    } else {
      if (acc) o = Pack<4>::load(p);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float d = vx.v[e] - mean;
        const float yb = fmaf(d, scale, beta);
        const float dz = vd.v[e] * (yb > 0.0f ? 1.0f : slope);
        const float dx = fmaf(scale, dz, fmaf(cB, d, cC));
        o.v[e] = acc ? o.v[e] + dx : dx;
      }
    }
#if ANODE_RING_STORE == 1
    o.store_stream(p);
#elif ANODE_RING_STORE == 2
    *reinterpret_cast<float4 *>(p) = make_float4(o.v[0], o.v[1], o.v[2], o.v[3]);
#else
    o.store(p, drop);
#endif
  };
  for (uint32_t i = 0; i < cnt; ++i, ax += kVecStride, ad += kVecStride) {
    const Pack<4> x0 = lds128(ax);
    Pack<4> d0 = x0;
    if constexpr (DIR == 1) d0 = lds128(ad);
    one(x0, d0, dst);
    advance();
  }
  __syncwarp();
  if (lane == 0) { mbar_arrive(&ctl->empty[slot]); mbar_arrive(&ctl->coef_empty[coef_q]); }
}

// ======================================================================================
// delivery warp: unit completion
// ======================================================================================
// (count, mean, M2) in double precision and Chan's pairwise update; used to merge a unit's
// partials in ONE pass over them, so that every partial is loaded exactly once and all loads
// of a batch are in flight together (the merge sits on the critical path of the pipeline).
struct Moments64 { double n, mean, m2; };
__device__ __forceinline__ Moments64 merge64(Moments64 a, Moments64 b)
{
  const double n = a.n + b.n;
  if (n <= 0.0) return Moments64{0.0, 0.0, 0.0};
  const double f = b.n / n, d = b.mean - a.mean;
  return Moments64{n, a.mean + d * f, a.m2 + b.m2 + d * d * a.n * f};
}
__device__ __forceinline__ Moments64 warp_merge64(Moments64 a)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Moments64 b;
    b.n = __shfl_down_sync(0xffffffffu, a.n, o);
    b.mean = __shfl_down_sync(0xffffffffu, a.mean, o);
    b.m2 = __shfl_down_sync(0xffffffffu, a.m2, o);
    a = merge64(a, b);
  }
  return a;
}
constexpr int kFinBatch = 8;     // partial loads a lane keeps in flight (regime S)
constexpr int kFinRegs = 16;     // partials a lane holds in registers (regime R: 512 tiles per unit)

// Regime R: one channel, up to thousands of partials.  The merge sits on the critical path of the
// pipeline, so all of a lane's loads are issued together (one round trip) and both passes of the
// two-pass merge (weighted mean, then M2 about it) run from registers.  Units with more than
// 32*kFinRegs tiles take further rounds and fold each round in with Chan's update.
template <int DIR>
__device__ __forceinline__ void warp_finish_unit_R(const FusedArgs &a, uint32_t u)
{
  const Plan &P = a.plan;
  const uint32_t lane = threadIdx.x & 31, T = P.tiles_per_unit;
  const float4 *part = ws_f4(a, P.off_part) + (size_t)u * T;
  Moments64 tot{0.0, 0.0, 0.0};
  double s1 = 0.0, s2 = 0.0;
  for (uint32_t k0 = 0; k0 < T; k0 += 32u * kFinRegs) {
    float rx[kFinRegs], ry[kFinRegs], rz[kFinRegs];
#pragma unroll
    for (int i = 0; i < kFinRegs; ++i) {
      const uint32_t k = k0 + lane + 32u * i;
      const float4 p = (k < T) ? __ldcg(part + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      rx[i] = p.x; ry[i] = p.y; rz[i] = p.z;
    }
    if constexpr (DIR == 0) {
      double sn = 0.0, sm = 0.0;
#pragma unroll
      for (int i = 0; i < kFinRegs; ++i) { sn += (double)rx[i]; sm = fma((double)rx[i], (double)ry[i], sm); }
      sn = warp_sum_all(sn); sm = warp_sum_all(sm);
      const double mean = sn > 0.0 ? sm / sn : 0.0;
      double sq = 0.0;
#pragma unroll
      for (int i = 0; i < kFinRegs; ++i) { const double d = (double)ry[i] - mean; sq += (double)rz[i] + (double)rx[i] * d * d; }
      sq = warp_sum_all(sq);
      tot = merge64(tot, Moments64{sn, mean, sq});
    } else {
#pragma unroll
      for (int i = 0; i < kFinRegs; ++i) { s1 += (double)rx[i]; s2 += (double)ry[i]; }
    }
  }
  if constexpr (DIR == 0) {
    if (lane == 0) finish_channel_fwd(a, u, tot.n, tot.mean, tot.m2);
  } else {
    s1 = warp_sum_all(s1); s2 = warp_sum_all(s2);
    if (lane == 0) finish_channel_bwd(a, u, s1, s2);
  }
}

// ======================================================================================
// fused mode, regime R: every block merges the partials of the units it applies itself
// ======================================================================================
// Instead of counting deliveries and electing a finisher, a delivery is a single 8-byte store of a
// tagged partial -- forward (mean, M2), backward (sum dz, sum dz*(x-mean)), lowest mantissa bit of
// the second value forced to one so the word is never all zero -- and whoever needs a unit polls
// the unit's partial words until none is zero, then merges them in a fixed order in double
// precision.  All blocks compute bit-identical coefficients; no atomics, fences or extra round
// trips sit between the last delivery and the first apply.  The element count of a partial
// follows from the tile geometry.  Two buffers are used alternately, launch by launch (parity
// word in the workspace header): a delivery also zeroes its word in the other buffer.
__device__ __forceinline__ unsigned long long *tag_buf(const FusedArgs &a, uint32_t parity)
{
  return reinterpret_cast<unsigned long long *>(a.ws + a.plan.off_tag) + (size_t)parity * a.plan.total_tiles * a.plan.cb;
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long *p)
{
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long *p, unsigned long long v)
{
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long *p)
{
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long *p, unsigned long long v)
{
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// partial words per lane per round of pull_merge_unit: the backward pass has four times the tiles per unit of the
// forward pass (smaller tiles), and a round costs a trip to L2; the forward merge does more arithmetic per word
constexpr int kPullRegsFwd = 8, kPullRegsBwd = 16;

// Whole warp.  Returns false when the wait ran out (abort raised).  On success c0 / c1 hold the
// unit's coefficients in every lane; `owner` makes lane 0 write the per-channel outputs.
template <int DIR>
__device__ __forceinline__ bool pull_merge_unit(const FusedArgs &a, RingCtl *ctl, uint32_t *status, uint32_t u, bool owner,
                                                float4 &c0, float4 &c1)
{
  constexpr int kPullRegs = DIR == 0 ? kPullRegsFwd : kPullRegsBwd;
  const Plan &P = a.plan;
  const uint32_t lane = threadIdx.x & 31, T = P.tiles_per_unit;
  const unsigned long long *buf = tag_buf(a, ctl->parity) + (size_t)u * T;
  // inputs that do not depend on the partials: fetch them while waiting
  const float gm = a.gamma ? a.gamma[u] : 1.0f;
  const float bt = (a.gamma && a.beta) ? a.beta[u] : 0.0f;
  float mean_in = 0.f, var_in = 1.f;
  if constexpr (DIR == 1) { mean_in = a.mean_in[u]; var_in = a.var_in[u]; }
  Moments64 tot{0.0, 0.0, 0.0};
  double s1 = 0.0, s2 = 0.0;
  const long long t0 = clock64();
  // With several GPUs only the unit's owner block needs the local merge (it ships the result to
  // every rank); all other blocks go straight to the exchanged records.
  const bool local = (a.world <= 1) || owner;
  for (uint32_t k0 = 0; local && k0 < T; k0 += 32u * kPullRegs) {
    unsigned long long r[kPullRegs];
    for (;;) {
      bool all = true;
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        const uint32_t k = k0 + lane + 32u * i;
        r[i] = (k < T) ? ld_relaxed_gpu_u64(buf + k) : 1ull;
        all = all && (r[i] != 0ull);
      }
      if (__all_sync(0xffffffffu, all)) break;
      __nanosleep(100);
      uint32_t stop = 0;
      if (lane == 0) {
        if (ctl->abort) stop = 1;
        else if (clock64() - t0 > kWaitCycles) { atomicOr(status, ANODE_ST_WAIT_STATS); ctl->abort = 1; stop = 1; }
      }
      if (__shfl_sync(0xffffffffu, stop, 0)) return false;
    }
    if constexpr (DIR == 0) {
      // element count of partial k, from the tile geometry (no division when rows are not split)
      auto count_of = [&](uint32_t k) -> float {
        if (k >= T) return 0.f;
        uint32_t sb = k, piece = 0;
        if (P.pieces != 1) { sb = k / P.pieces; piece = k - sb * P.pieces; }
        const uint32_t n0 = sb * P.rows_per_tile, col0 = piece * P.piece_len;
        const uint32_t rows = (P.N - n0 < P.rows_per_tile) ? (P.N - n0) : P.rows_per_tile;
        const uint32_t len = (P.dim0 - col0 < P.piece_len) ? (P.dim0 - col0) : P.piece_len;
        return (float)(rows * len);
      };
      float nk[kPullRegs];
      double sn = 0.0, sm = 0.0;
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        nk[i] = count_of(k0 + lane + 32u * i);
        const double mk = (double)__uint_as_float((uint32_t)(r[i] & 0xffffffffull));
        sn += (double)nk[i]; sm = fma((double)nk[i], mk, sm);
      }
      sn = warp_sum_all(sn); sm = warp_sum_all(sm);
      const double mean = sm / sn;
      double sq = 0.0;
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        const double mk = (double)__uint_as_float((uint32_t)(r[i] & 0xffffffffull));
        const double m2 = (double)__uint_as_float((uint32_t)(r[i] >> 32));
        const double d = mk - mean;
        if (nk[i] > 0.f) sq += m2 + (double)nk[i] * d * d;
      }
      sq = warp_sum_all(sq);
      tot = merge64(tot, Moments64{sn, mean, sq});
    } else {
#pragma unroll
      for (int i = 0; i < kPullRegs; ++i) {
        const uint32_t k = k0 + lane + 32u * i;
        if (k < T) {
          s1 += (double)__uint_as_float((uint32_t)(r[i] & 0xffffffffull));
          s2 += (double)__uint_as_float((uint32_t)(r[i] >> 32));
        }
      }
    }
  }
  if constexpr (DIR == 1) { if (local) { s1 = warp_sum_all(s1); s2 = warp_sum_all(s2); } }
  if (a.world > 1) {
    // ---- exchange between GPUs.  A record is three 8-byte words (value in the low half, the
    // call's epoch in the high half): every word validates itself, so plain peer stores suffice
    // and nothing is ever zeroed; consecutive calls alternate between two buffers.
    const uint32_t par = a.epoch & 1u;
    const size_t slot = (((size_t)par * a.world) * a.xchg_channels + u) * 4;      // + src * xchg_channels * 4
    const size_t src_stride = (size_t)a.xchg_channels * 4;
    if (owner && lane < a.world) {
      // word 0 of a forward record is the element count as an exact integer (a float would round counts above 2^24)
      const uint32_t w0 = DIR == 0 ? (uint32_t)tot.n : __float_as_uint((float)s1);
      const uint32_t w1 = __float_as_uint(DIR == 0 ? (float)tot.mean : (float)s2);
      const uint32_t w2 = __float_as_uint(DIR == 0 ? (float)tot.m2 : 0.f);
      unsigned long long *dst = a.xchg[lane] + slot + a.rank * src_stride;       // this rank's slot in peer `lane`
      const unsigned long long e = (unsigned long long)a.epoch << 32;
      st_relaxed_sys_u64(dst + 0, e | w0);
      st_relaxed_sys_u64(dst + 1, e | w1);
      st_relaxed_sys_u64(dst + 2, e | w2);
    }
    // lane r collects rank r's record from this GPU's own buffer
    const unsigned long long *mine = a.xchg[a.rank] + slot + (lane < a.world ? lane : 0) * src_stride;
    unsigned long long v0 = 0, v1 = 0, v2 = 0;
    for (;;) {
      bool ok = true;
      if (lane < a.world) {
        v0 = ld_relaxed_sys_u64(mine + 0); v1 = ld_relaxed_sys_u64(mine + 1); v2 = ld_relaxed_sys_u64(mine + 2);
        ok = (uint32_t)(v0 >> 32) == a.epoch && (uint32_t)(v1 >> 32) == a.epoch && (uint32_t)(v2 >> 32) == a.epoch;
      }
      if (__all_sync(0xffffffffu, ok)) break;
      __nanosleep(200);
      uint32_t stop = 0;
      if (lane == 0) {
        if (ctl->abort) stop = 1;
        else if (clock64() - t0 > a.wait_cycles) { atomicOr(status, ANODE_ST_WAIT_PEER); ctl->abort = 1; stop = 1; }
      }
      if (__shfl_sync(0xffffffffu, stop, 0)) return false;
    }
    // merge in rank order (lane = rank; the shuffle tree is the same on every GPU, so all ranks
    // obtain bit-identical statistics)
    const bool live = lane < a.world;
    const double f0 = live ? (DIR == 0 ? (double)(uint32_t)v0 : (double)__uint_as_float((uint32_t)v0)) : 0.0;
    const double f1 = live ? (double)__uint_as_float((uint32_t)v1) : 0.0;
    const double f2 = live ? (double)__uint_as_float((uint32_t)v2) : 0.0;
    if constexpr (DIR == 0) {
      const double sn = warp_sum_all(f0), sm = warp_sum_all(f0 * f1);
      const double mean = sm / sn;
      const double d = f1 - mean;
      const double sq = warp_sum_all(live ? f2 + f0 * d * d : 0.0);
      tot = Moments64{sn, mean, sq};
    } else {
      s1 = warp_sum_all(f0); s2 = warp_sum_all(f1);
    }
  }
  if constexpr (DIR == 0) {
    const float mf = (float)tot.mean;
    const float vf = (float)(tot.m2 / tot.n + (double)a.epsilon);     // biased, epsilon folded in (batch_norm.cu:160)
    c0 = make_float4(mf, gm * inv_std(vf), bt, 0.f);
    c1 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (owner && lane == 0) {
      a.mean[u] = mf; a.var[u] = vf;
      if (a.run_mean) { const float o = a.run_mean[u]; a.run_mean[u] = o + a.avg_rate * (mf - o); }
      if (a.run_var) { const float o = a.run_var[u]; a.run_var[u] = o + a.avg_rate * (vf - o); }
    }
  } else {
    const float r = inv_std(var_in);
    const double rs2 = (double)r * s2;                       // sum(dz * xhat)
    const double A = (double)gm * (double)r;
    const double invM = 1.0 / a.count_total;
    c0 = make_float4(mean_in, gm * r, bt, 0.f);
    c1 = make_float4((float)(-A * (double)r * rs2 * invM), (float)(-A * s1 * invM), 0.f, 0.f);
    if (owner && lane == 0) {
      if (a.dbeta) a.dbeta[u] = (float)s1;
      if (a.dgamma) a.dgamma[u] = (float)rs2;
    }
  }
  return true;
}

// ======================================================================================
// the kernel
// ======================================================================================
// Whole-row tiles only (one channel per unit): short-row shapes are served by the cluster kernel
// (bn_segres.cu) and the plain kernel.
template <int DIR>
__global__ void __launch_bounds__(kRingThreads, 1) bn_ring_kernel(const FusedArgs a, const RingGeom g)
{
  extern __shared__ __align__(128) unsigned char sm[];
  RingCtl *ctl = reinterpret_cast<RingCtl *>(sm);
  const Plan &P = a.plan;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t *status = a.status;
  uint32_t *exit_ctr = ws_u32(a, 4);
  uint32_t *done = ws_u32(a, P.off_done);

  if (tid == 0) {
    for (uint32_t i = 0; i < g.slots; ++i) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->empty[i], kCWarps); }
    for (uint32_t i = 0; i < kResQ; ++i) { mbar_init(&ctl->res_full[i], kCWarps); mbar_init(&ctl->res_empty[i], 1); }
    for (uint32_t i = 0; i < kCoefQ; ++i) { mbar_init(&ctl->coef_full[i], 1); mbar_init(&ctl->coef_empty[i], kCWarps); }
    ctl->abort = 0; ctl->last_block = 0;
    ctl->parity = *ws_u32(a, 8) & 1u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  Sched sc; sc.init(a);
  uint32_t kind;

  if (warp < kConsumers / 32) {
    // ------------------------------------------------------------------ consumers
    uint32_t nres = 0, ncoef = 0;             // reduce count, apply count
    uint32_t slot = g.slots - 1, par = 1;     // ring position, stepped without divisions
    TileRange tr;
    while (sc.next_range(P, kind, tr)) {
      if (++slot == g.slots) { slot = 0; par ^= 1u; }
      if (kind == 0) {
        const uint32_t q = nres % kResQ, qpar = (nres / kResQ) & 1u; ++nres;
        // the partial mailbox entry must have been emptied by the delivery warp (first pass: free)
        bool ok = warp_wait(&ctl->res_empty[q], qpar ^ 1u, ctl, status, ANODE_ST_WAIT_STATS);
        ok = ok && warp_wait(&ctl->full[slot], par, ctl, status, ANODE_ST_WAIT_STATS);
        if (!ok) break;                                 // warps are independent: no barrier to honour
        warp_reduce_R<DIR>(a, g, sm, ctl, tr, slot, res_box(sm, g, q));
        if (lane == 0) mbar_arrive(&ctl->res_full[q]);
      } else {
        const uint32_t q = ncoef % kCoefQ, qpar = (ncoef / kCoefQ) & 1u; ++ncoef;
        bool ok = warp_wait(&ctl->coef_full[q], qpar, ctl, status, ANODE_ST_WAIT_STATS);
        ok = ok && warp_wait(&ctl->full[slot], par, ctl, status, ANODE_ST_WAIT_STATS);
        if (!ok) break;
        warp_apply_R<DIR>(a, g, sm, ctl, tr, slot, coef_box(sm, g, P.cb, q), q);
      }
    }
  } else if (warp == kConsumers / 32) {
    // ------------------------------------------------------------------ producer
    // where the window between the two visits exceeds what L2 keeps, only the fraction that fits is marked "keep"
    const uint64_t keep = g.keep_frac < 1.0f ? policy_keep_fraction(g.keep_frac) : policy_keep(), drop = policy_drop();
    const uint64_t rs = (uint64_t)P.C * P.dim0;
    uint32_t k = 0;
    uint32_t slot = g.slots - 1, par = 1;
    bool ok = true;
    TileRange tr;
    // backward pass: (mean, gamma / std, beta) of the current channel and, fetched ahead, of the next one
    uint32_t side_c = 0xffffffffu, next_c = 0xffffffffu, next_age = 0;
    float4 side_v = make_float4(0.f, 0.f, 0.f, 0.f), next_v = side_v, next_raw = side_v;
    bool next_pending = false;
    auto load_side_raw = [&](uint32_t c) {      // the loads only; the arithmetic waits until the values are used
      float4 r = make_float4(0.f, 1.f, 1.f, 0.f);
      if constexpr (DIR == 1) {
        r.x = a.mean_in[c]; r.y = a.var_in[c];
        r.z = a.gamma ? a.gamma[c] : 1.0f;
        r.w = (a.gamma && a.beta) ? a.beta[c] : 0.0f;
      }
      return r;
    };
    auto finish_side = [&](const float4 &r) { return make_float4(r.x, r.z * inv_std(r.y), r.w, 0.f); };
    while (ok && sc.next_range(P, kind, tr)) {
      ++k;
      if (++slot == g.slots) { slot = 0; par ^= 1u; }
      // (one lane polls here: a producer that reacts sooner was measured slower where the window between the two
      // visits exceeds what L2 keeps, and hardly faster elsewhere)
      uint32_t okw = 1;
      if (lane == 0) okw = mbar_wait(&ctl->empty[slot], par ^ 1u, ctl, status, ANODE_ST_WAIT_STATS) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, okw, 0) != 0;     // one lane decides for the warp
      if (!ok) { --k; break; }
      float *xs = slot_x(sm, g, slot);
      if (DIR == 1 && kind == 0) {
        // coefficients of the reduce visit's ReLU mask (one channel per unit here).  They change only when the
        // block moves on to another channel, and the next channel's are fetched ahead of time: a visit's issue
        // must not wait for global memory, or the slot stays empty for that long.
        if (tr.c0 != side_c) {
          if (tr.c0 == next_c) side_v = next_pending ? finish_side(next_raw) : next_v;
          else side_v = finish_side(load_side_raw(tr.c0));
          side_c = tr.c0;
          next_c = tr.c0 + 1 < P.C ? tr.c0 + 1 : tr.c0;
          next_raw = load_side_raw(next_c); next_pending = true; next_age = 0;
        }
        if (lane == 0) slot_side<1>(sm, g, slot)[0] = side_v;
      }
      __syncwarp();
      const uint32_t row_bytes = tr.len * 4u;
      if (lane == 0) mbar_arrive_expect_tx(&ctl->full[slot], row_bytes * tr.rows * (DIR == 1 ? 2u : 1u));
      __syncwarp();
      const uint64_t pol = (kind == 0 && a.mode == MODE_FUSED) ? keep : drop;
      // every row is fetched as several bulk copies (one per lane at a time), so that a tile made of
      // one long row still has many copies in flight
      const uint32_t per_row = (row_bytes + kCopyBytes - 1) / kCopyBytes, ncopies = per_row * tr.rows;
      for (uint32_t c = lane; c < ncopies; c += 32) {
        const uint32_t r = c / per_row, o = (c - r * per_row) * kCopyBytes;
        const uint32_t nb = row_bytes - o < kCopyBytes ? row_bytes - o : kCopyBytes;
        const size_t goff = (size_t)tr.base + (size_t)r * rs + o / 4;
        float *dst = xs + (size_t)r * tr.len + o / 4;
        bulk_g2s(dst, a.x + goff, nb, &ctl->full[slot], pol);
        if (DIR == 1) bulk_g2s(dst + g.slot_floats, a.dy + goff, nb, &ctl->full[slot], pol);
      }
      // the values fetched ahead are turned into coefficients one visit later, when they have arrived
      if (DIR == 1 && next_pending && next_age++ >= 1) { next_v = finish_side(next_raw); next_pending = false; }
    }
    // after an abort: wait (bounded) for copies that were issued but will not be consumed
    if (!ok && lane == 0) {
      const uint32_t first = k > g.slots ? k - g.slots : 0;
      for (uint32_t kk = first; kk < k; ++kk) {
        const long long t0 = clock64();
        while (!mbar_test(&ctl->full[kk % g.slots], (kk / g.slots) & 1u) && clock64() - t0 < kWaitCycles / 8) {}
      }
    }
  } else if (warp == kConsumers / 32 + 1) {
    // ------------------------------------------------------------------ delivery warp
    // Reduce visit j of this block is tile b + j*G.  Each turn serves every partial that waits,
    // one lane per partial, so the fences and atomics of several tiles overlap.
    const uint32_t n_red = sc.do_reduce ? sc.my_tiles : 0;
    uint32_t nres = 0;
    while (nres < n_red) {
      // sleep on the next entry's barrier (no polling loop competing with the consumers for issue
      // slots), then take along whatever else has arrived in the meantime
      if (!warp_wait(&ctl->res_full[nres % kResQ], (nres / kResQ) & 1u, ctl, status, ANODE_ST_WAIT_STATS)) break;
      const uint32_t jd = nres + lane;
      const bool d_ok = lane < kResQ && jd < n_red && mbar_test(&ctl->res_full[jd % kResQ], (jd / kResQ) & 1u);
      const uint32_t d_mask = __ballot_sync(0xffffffffu, d_ok);
      uint32_t nd = __ffs(~d_mask) - 1;                               // in order: leading run of ones
      if (nd > kPerTurn) nd = kPerTurn;
      if (nd) {
        {
          // entry e is served by lanes 8e .. 8e+7: one warp partial each, merged in a fixed order
          const uint32_t e = lane / kCWarps, w = lane % kCWarps;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (e < nd) v = res_box(sm, g, (nres + e) % kResQ)[w];
          if constexpr (DIR == 0) {
            Moments m{v.x, v.y, v.z};
#pragma unroll
            for (int o = (int)kCWarps / 2; o > 0; o >>= 1) {
              Moments c;
              c.n = __shfl_down_sync(0xffffffffu, m.n, o, kCWarps);
              c.mean = __shfl_down_sync(0xffffffffu, m.mean, o, kCWarps);
              c.m2 = __shfl_down_sync(0xffffffffu, m.m2, o, kCWarps);
              m = merge(m, c);
            }
            v = make_float4(m.n, m.mean, m.m2, 0.f);
          } else {
#pragma unroll
            for (int o = (int)kCWarps / 2; o > 0; o >>= 1) {
              v.x += __shfl_down_sync(0xffffffffu, v.x, o, kCWarps);
              v.y += __shfl_down_sync(0xffffffffu, v.y, o, kCWarps);
            }
          }
          if (a.mode == MODE_FUSED) {
            // one tagged 8-byte word per tile; nothing else to do for a delivery
            if (e < nd && w == 0) {
              const size_t t = (size_t)(sc.b + (nres + e) * sc.G);
              const float lo = DIR == 0 ? v.y : v.x, hi = DIR == 0 ? v.z : v.y;
              st_relaxed_gpu_u64(tag_buf(a, ctl->parity) + t, pack_rec(lo, __uint_as_float(__float_as_uint(hi) | 1u)));
              tag_buf(a, ctl->parity ^ 1u)[t] = 0ull;
            }
            __syncwarp();
            if (lane < nd) mbar_arrive(&ctl->res_empty[(nres + lane) % kResQ]);
            nres += nd;
            continue;
          }
          if (e < nd && w == 0) __stcg(ws_f4(a, P.off_part) + (size_t)(sc.b + (nres + e) * sc.G), v);
        }
        __syncwarp();
        uint32_t last = 0, unit = 0;
        if (lane < nd) {
          const uint32_t j = nres + lane;
          unit = (sc.b + j * sc.G) / P.tiles_per_unit;
          mbar_arrive(&ctl->res_empty[j % kResQ]);
          // release: the partial stored above is visible before the count; acquire: whoever sees the
          // full count also sees every partial counted before
          uint32_t old;
          asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(done + unit) : "memory");
          last = (old + 1 == P.tiles_per_unit) ? 1u : 0u;
        }
        uint32_t lmask = __ballot_sync(0xffffffffu, last != 0);
        while (lmask) {
          const uint32_t src = __ffs(lmask) - 1; lmask &= lmask - 1;
          const uint32_t u = __shfl_sync(0xffffffffu, unit, src);
          warp_finish_unit_R<DIR>(a, u);
          if (lane == 0) done[u] = 0;
        }
        nres += nd;
      }
    }
  } else {
    // ------------------------------------------------------------------ coefficient warp
    // Apply visit j of this block is tile b + j*G (one channel per unit).
    const uint32_t n_app = sc.do_apply ? sc.my_tiles : 0;
    uint32_t ncoef = 0;
    if (a.mode == MODE_FUSED) {
      // merge each unit's partials here (see pull_merge_unit); consecutive visits of the same unit reuse
      // the result
      uint32_t have = 0xffffffffu;
      float4 c0 = make_float4(0.f, 0.f, 0.f, 0.f), c1 = c0;
      while (ncoef < n_app) {
        if (!warp_wait(&ctl->coef_empty[ncoef % kCoefQ], ((ncoef / kCoefQ) & 1u) ^ 1u, ctl, status, ANODE_ST_WAIT_STATS)) break;
        const uint32_t t = sc.b + ncoef * sc.G, u = t / P.tiles_per_unit;
        if (u != have) {
          // the block that owns the unit's first tile also writes the per-channel outputs
          if (!pull_merge_unit<DIR>(a, ctl, status, u, t == u * P.tiles_per_unit, c0, c1)) break;
          have = u;
        }
        if (lane == 0) {
          float4 *box = coef_box(sm, g, P.cb, ncoef % kCoefQ);
          box[0] = c0; box[1] = c1;
          mbar_arrive(&ctl->coef_full[ncoef % kCoefQ]);
        }
        ++ncoef;
      }
    } else {
      // apply pass of the three-launch form: the coefficients were prepared by the exchange / merge kernel
      while (ncoef < n_app) {
        if (!warp_wait(&ctl->coef_empty[ncoef % kCoefQ], ((ncoef / kCoefQ) & 1u) ^ 1u, ctl, status, ANODE_ST_WAIT_STATS)) break;
        const uint32_t c = (sc.b + ncoef * sc.G) / P.tiles_per_unit;
        if (lane == 0) {
          const float4 *coef = ws_f4(a, P.off_coef) + 2 * (size_t)c;
          float4 *box = coef_box(sm, g, P.cb, ncoef % kCoefQ);
          box[0] = __ldcg(coef); box[1] = __ldcg(coef + 1);
          mbar_arrive(&ctl->coef_full[ncoef % kCoefQ]);
        }
        ++ncoef;
      }
    }
  }

  // ---- leave: the last block out lowers the ready flags so that the workspace is clean again
  __syncthreads();
  if (ctl->abort) {
    if (tid == 0) atomicOr(status, ANODE_ST_ABORTED);
    return;
  }
  if (a.mode == MODE_FUSED) {
    if (tid == 0) {
      __threadfence();
      ctl->last_block = (atomicAdd(exit_ctr, 1u) + 1 == gridDim.x) ? 1u : 0u;
    }
    __syncthreads();
    if (ctl->last_block && tid == 0) {
      *ws_u32(a, 8) = ctl->parity ^ 1u;       // the next launch uses the other partial buffer
      *exit_ctr = 0;
    }
  }
}

}  // namespace ANODE_RING_NS
}  // namespace anode_b200
