// Plan and schedule of the slice-resident batch-norm kernel (bn_resident.cu).  Plain C++ (no CUDA
// types): the same code runs in the host-side planner, inside the kernel, and in CPU-only tests of
// the schedule.
//
// Vocabulary
//   piece   what one shared-memory slot holds: `rows` whole rows of one channel (short rows) or
//           one part [col0, col0+len) of a single row (long rows).  A channel has U pieces,
//           numbered sample-block major: u = sample_block*P + part.
//   team    Gt thread blocks (one per SM) that share a channel: block b of the team owns the
//           pieces [b*U/Gt, (b+1)*U/Gt) of every channel the team handles.  Team t handles the
//           channels t, t + teams, t + 2*teams, ... in that order.
//   slice   a block's pieces of one channel.  The first Rz of them are RESIDENT: loaded once,
//           reduced, kept in their slot until the channel's statistics are known, normalised in
//           place and stored from there.  The remaining Ts are STREAMED: loaded, reduced and
//           released, then loaded again (from L2, where they were asked to stay) for the apply.
//   lag     resident pieces of all channels form one sequence i = k*Rz + j; piece i - lag is
//           applied right after piece i has been reduced, so between the end of a channel's
//           reduction and the first use of its statistics the block reduces `lag - Rz` more
//           resident pieces (and the next channel's streamed pieces): that work hides the time the
//           team needs to combine its partials.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "bn_plan.h"

namespace anode_b200 {

constexpr uint32_t kResMaxSlots = 64;          // slots per block (the roles keep one parity bit per slot in a 64-bit word)
constexpr uint32_t kResMaxRows = 32;           // rows per piece (one bulk copy per row, one lane each)
constexpr uint32_t kResCtlBytes = 6144;        // barriers, mailboxes, flags and the piece table in front of the slots
constexpr uint32_t kResMaxPieces = 256;        // pieces per slice (entries of the piece table)
constexpr uint32_t kResSmemBudget = 227u * 1024u;
constexpr uint32_t kResPartWords = 4;          // 8-byte words per (channel, block) partial in the workspace

struct ResPlan {
  uint32_t dim0, C, N;
  uint32_t planes;          // tensors per slot: x [, dy] [, residual or saved output]
  uint32_t rpp;             // rows per piece (1 when rows are split)
  uint32_t P;               // parts per row (1 when pieces hold whole rows)
  uint32_t piece_len;       // floats of a row in one piece (a multiple of 4)
  uint32_t SB;              // sample blocks per channel = ceil(N / rpp)
  uint32_t U;               // pieces per channel = SB * P
  uint32_t Gt, teams, grid; // blocks per team, teams, blocks launched = Gt * teams
  uint32_t T;               // most pieces any block has per channel = ceil(U / Gt)
  uint32_t plane_bytes;     // bytes of one tensor in a slot (largest piece, padded to 128)
  uint32_t slot_bytes;      // planes * plane_bytes
  uint32_t Q, Qr, Qs;       // slots: total, resident ring, streaming ring
  uint32_t Rz_max;          // resident pieces per channel and block (blocks with fewer pieces keep all)
  uint32_t pf;              // slots by which loads run ahead of the reduce visits in the resident ring
  uint32_t smem_bytes;
  uint64_t ws_bytes;        // workspace bytes of this kernel's region: C * Gt partial records
  double score;             // estimated share of the SM-slot-time that does useful work (planner's ranking)
};

// What one block does, derived from the plan and the block's position in its team.
struct ResBlock {
  uint32_t team, b;         // team index, block index inside the team
  uint32_t u0, Tb;          // first piece and number of pieces per channel
  uint32_t Rz, Ts, lag;     // resident pieces, streamed pieces, apply lag (in resident pieces)
  uint32_t K;               // channels this block's team handles
};

ANODE_HD ResBlock res_block(const ResPlan &p, uint32_t block)
{
  ResBlock r;
  r.team = block / p.Gt; r.b = block - r.team * p.Gt;
  r.u0 = (uint32_t)(((uint64_t)r.b * p.U) / p.Gt);
  const uint32_t u1 = (uint32_t)(((uint64_t)(r.b + 1) * p.U) / p.Gt);
  r.Tb = u1 - r.u0;
  r.Rz = r.Tb < p.Rz_max ? r.Tb : p.Rz_max;
  r.Ts = r.Tb - r.Rz;
  // fully resident plans let the applies trail as far as the ring allows; otherwise a channel's
  // resident pieces are applied as soon as the next channel starts to need their slots
  r.lag = p.Qs == 0 ? p.Qr - p.pf : r.Rz;
  if (r.lag < r.Rz) r.lag = r.Rz;
  r.K = r.team < p.C ? (p.C - r.team + p.teams - 1) / p.teams : 0;
  return r;
}

// Geometry of piece u of a channel: first sample, samples, first column, floats per row.
struct ResPiece { uint32_t n0, rows, col0, len; };
ANODE_HD ResPiece res_piece(const ResPlan &p, uint32_t u)
{
  ResPiece r;
  uint32_t sb = u, part = 0;
  if (p.P != 1) { sb = u / p.P; part = u - sb * p.P; }
  r.n0 = sb * p.rpp;
  r.rows = (p.N - r.n0 < p.rpp) ? (p.N - r.n0) : p.rpp;
  r.col0 = part * p.piece_len;
  r.len = (p.dim0 - r.col0 < p.piece_len) ? (p.dim0 - r.col0) : p.piece_len;
  return r;
}

// ---- the schedule ------------------------------------------------------------------------------
// Every role of a block (loader, consumers, storer, delivery, coefficients) walks the same event
// sequence and acts on the events that concern it.
enum : uint32_t {
  EV_RED_STR = 0,    // load a streamed piece (asked to stay in L2), reduce it, release the slot
  EV_RED_RES = 1,    // load a resident piece, reduce it, keep the slot
  EV_PUBLISH = 2,    // the block's partial of channel k is complete
  EV_NEED_COEF = 3,  // the applies of channel k follow: its statistics are needed now
  EV_APP_STR = 4,    // load a streamed piece again, normalise in place, store, release the slot
  EV_APP_RES = 5,    // normalise a resident piece in place, store, release the slot
};
struct ResEvent {
  uint32_t kind;
  uint32_t k;        // index into the team's channel list (channel = team + k*teams)
  uint32_t piece;    // piece index inside the block's slice (0 .. Tb-1); resident pieces come first
  uint32_t slot;     // shared-memory slot (resident ring: 0 .. Qr-1, streaming ring: Qr .. Qr+Qs-1)
};

// Calls v(event) for every event in order; v returns false to stop the walk (abort).  Slot numbers
// advance by counting (no division per event: every role of a block walks the whole sequence).
template <class V>
ANODE_HD void res_walk(const ResPlan &p, const ResBlock &r, V &&v)
{
  if (r.K == 0 || r.Tb == 0) return;
  const uint32_t Qr = p.Qr, Qs = p.Qs ? p.Qs : 1;
  uint32_t ss = 0, sr = 0, sa = 0;        // next slot of the streaming ring, of the resident reduces, of the resident applies
  uint32_t ka = 0, ja = 0, ia = 0;        // next resident piece to apply
  bool go = true;
  auto apply_next = [&]() {
    if (ja == 0) {
      go = v(ResEvent{EV_NEED_COEF, ka, 0, 0});
      // most recently reduced first: the streamed pieces were reduced in increasing order
      for (uint32_t s = r.Ts; go && s-- > 0;) { go = v(ResEvent{EV_APP_STR, ka, r.Rz + s, Qr + ss}); if (++ss == Qs) ss = 0; }
    }
    if (go) go = v(ResEvent{EV_APP_RES, ka, ja, sa});
    if (++sa == Qr) sa = 0;
    ++ia;
    if (++ja == r.Rz) { ja = 0; ++ka; }
  };
  uint32_t i = 0;
  for (uint32_t k = 0; go && k < r.K; ++k) {
    for (uint32_t s = 0; go && s < r.Ts; ++s) { go = v(ResEvent{EV_RED_STR, k, r.Rz + s, Qr + ss}); if (++ss == Qs) ss = 0; }
    for (uint32_t j = 0; go && j < r.Rz; ++j, ++i) {
      go = v(ResEvent{EV_RED_RES, k, j, sr});
      if (++sr == Qr) sr = 0;
      if (go && i >= r.lag) apply_next();
    }
    if (go) go = v(ResEvent{EV_PUBLISH, k, 0, 0});
  }
  while (go && ia < r.K * r.Rz) apply_next();
}

// ---- the planner ---------------------------------------------------------------------------------
// Fills in everything that follows from (rpp, P, piece_len, Gt, teams); false when the candidate is
// not usable.  `cover_bytes`: how much reduce work should separate the end of a channel's reduction
// from the first use of its statistics.
inline bool res_finish_plan(ResPlan &p, uint32_t sms, uint32_t cover_bytes, uint32_t stream_bytes, uint32_t ahead_bytes)
{
  p.SB = ceil_div_u32(p.N, p.rpp);
  p.U = p.SB * p.P;
  if (p.Gt == 0 || p.teams == 0 || p.Gt > p.U || p.teams > p.C) return false;
  p.grid = p.Gt * p.teams;
  p.T = ceil_div_u32(p.U, p.Gt);
  if (p.T > kResMaxPieces) return false;
  p.plane_bytes = (uint32_t)align_up_u64((uint64_t)p.rpp * p.piece_len * 4, 128);
  p.slot_bytes = p.planes * p.plane_bytes;
  if (p.slot_bytes > kResSmemBudget - kResCtlBytes) return false;
  p.Q = (kResSmemBudget - kResCtlBytes) / p.slot_bytes;
  if (p.Q > kResMaxSlots) p.Q = kResMaxSlots;
  // bytes of loads that must be in flight to cover the memory latency, in slots
  p.pf = ceil_div_u32(ahead_bytes, p.slot_bytes);
  if (p.pf < 2) p.pf = 2;
  const uint32_t stream_slots = ceil_div_u32(stream_bytes, p.slot_bytes);
  uint32_t cover = ceil_div_u32(cover_bytes, p.slot_bytes);
  if (cover < 1) cover = 1;
  if (p.T + cover + p.pf <= p.Q) {
    // every piece stays in shared memory; the applies trail by lag = Q - pf >= T + cover pieces
    p.Qs = 0; p.Qr = p.Q; p.Rz_max = p.T;
    // no use holding more channels than the lag can hide: trim the ring to about three slices
    const uint32_t want = 3 * p.T + p.pf > p.T + cover + p.pf ? 3 * p.T + p.pf : p.T + cover + p.pf;
    if (p.Qr > want) p.Qr = want;
    p.Q = p.Qr;
  } else {
    p.Qs = stream_slots < 2 ? 2 : stream_slots;
    if (p.Q < p.Qs + p.pf + 1) return false;
    p.Qr = p.Q - p.Qs;
    uint32_t rz = p.Qr - p.pf;                             // lag = Rz: the ring holds Rz + pf pieces
    const uint32_t all_min = p.U / p.Gt;                   // pieces of the smallest slice
    // leave at least `cover` pieces of every slice to the streaming ring: they are what the block
    // works on while the previous channel's statistics are being combined
    if (all_min > cover && rz > all_min - cover) rz = all_min - cover;
    if (all_min <= cover) rz = 1;
    if (rz < 1) rz = 1;
    p.Rz_max = rz;
    p.Qr = rz + p.pf;
    p.Q = p.Qr + p.Qs;
  }
  p.smem_bytes = kResCtlBytes + p.Q * p.slot_bytes;
  p.ws_bytes = align_up_u64((uint64_t)p.C * p.Gt * kResPartWords * 8, 256);
  // ranking: share of (SM, piece visit) slots that carry a real piece, discounted for streamed
  // pieces (a second trip through L2), small copies and idle SMs
  const uint32_t chan_rounds = ceil_div_u32(p.C, p.teams);
  double eff = ((double)p.C * p.U) / ((double)chan_rounds * p.T * p.teams * p.Gt);
  eff *= p.grid >= sms ? 1.0 : (double)p.grid / (double)sms;
  const double streamed = p.T > p.Rz_max ? (double)(p.T - p.Rz_max) / p.T : 0.0;
  eff *= 1.0 - 0.25 * streamed;
  // every piece costs a fixed amount of barrier traffic and copy issue, about what 384 bytes cost to move
  const double piece_bytes = (double)p.rpp * p.piece_len * 4.0;
  eff *= piece_bytes / (piece_bytes + 384.0);
  if (p.piece_len * 4 < 2048) eff *= 0.9;                  // short bulk copies use the memory pipes poorly
  if (p.T < 2) eff *= 0.9;                                 // one piece per channel: no overlap inside a slice
  p.score = eff;
  return true;
}

// Chooses piece shape and team size for a [dim0, C, N] problem with `planes` tensors per slot, on a
// device with `sms` SMs.  Returns false when the kernel does not apply (rows that cannot be moved
// with 16-byte bulk copies, or pieces that do not fit).
inline bool make_res_plan(uint32_t dim0, uint32_t C, uint32_t N, uint32_t planes, uint32_t sms,
                          uint32_t cover_bytes, uint32_t stream_bytes, uint32_t ahead_bytes, ResPlan &best)
{
  if (dim0 % 4 != 0 || dim0 < 64 || planes < 1 || planes > 3 || sms == 0) return false;
  if (sms > 160) sms = 160;         // the merge of a team's records keeps five per lane in registers
  bool have = false;
  const uint32_t targets[] = {4096, 3072, 2048, 1536, 1024, 512};
  for (uint32_t ti = 0; ti < sizeof(targets) / sizeof(targets[0]); ++ti) {
    const uint32_t tf = targets[ti];
    ResPlan c{};
    c.dim0 = dim0; c.C = C; c.N = N; c.planes = planes;
    if (dim0 > tf) {
      c.rpp = 1;
      c.P = ceil_div_u32(dim0, tf);
      c.piece_len = ceil_div_u32(ceil_div_u32(dim0, c.P), 4) * 4;
      c.P = ceil_div_u32(dim0, c.piece_len);
    } else {
      c.P = 1; c.piece_len = dim0;
      c.rpp = tf / dim0; if (c.rpp < 1) c.rpp = 1;
      if (c.rpp > kResMaxRows) c.rpp = kResMaxRows;
      if (c.rpp > N) c.rpp = N;
    }
    for (uint32_t gt = 1; gt <= sms; ++gt) {
      ResPlan d = c;
      d.Gt = gt;
      d.teams = sms / gt; if (d.teams > C) d.teams = C;
      if (!res_finish_plan(d, sms, cover_bytes, stream_bytes, ahead_bytes)) continue;
      // prefer, at equal score, larger pieces and then larger teams (fewer channels in flight)
      if (!have || d.score > best.score + 1e-9) { best = d; have = true; }
    }
  }
  return have;
}

}  // namespace anode_b200
