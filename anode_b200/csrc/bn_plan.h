// Work decomposition of one [dim0, C, N] batch-norm problem into tiles, and the layout of
// the scratch workspace.  Plain C++ (no CUDA types) so the same code runs in the host-side
// planner, inside the kernels, and in CPU-only tests of the index arithmetic.
//
// Vocabulary
//   row    the dim0 contiguous floats of one (sample n, channel c) pair; row (n, c) starts
//          at (n*C + c)*dim0  (reference routines_gpu/common.cuh:88-94, Index3::Pack).
//   unit   the set of channels whose statistics are completed together.  Regime R ("rows"):
//          one channel.  Regime S ("segments", small dim0): a block of `cb` adjacent
//          channels, so that one sample contributes a contiguous segment of cb*dim0 floats.
//   tile   what one thread block processes at a time: `rows_per_tile` samples of one unit,
//          restricted (regime R, long rows) to one piece [col0, col0+piece_len) of each row.
//          Tiles are numbered unit-major: t = unit*tiles_per_unit + sample_block*pieces + piece.
//   step   thread block b visits tiles b, b+grid, b+2*grid, ...; at step s it reduces tile
//          number s and then applies tile number s - lookahead_steps, so that the re-read of a
//          tile follows its first read by a bounded number of bytes (kept in L2).
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define ANODE_HD __host__ __device__ __forceinline__
#else
#define ANODE_HD inline
#endif

namespace anode_b200 {

constexpr uint32_t kThreads = 256;        // threads per block of every fused kernel
constexpr uint32_t kSegSlots = 2;         // regime S: float4 slots per thread per sample
constexpr uint32_t kMaxTileElems = 65532; // fast division below is exact up to here

struct Plan {
  uint32_t dim0, C, N;
  uint32_t regime;          // 0 = R, 1 = S
  uint32_t vec;             // elements per load: 4 (128-bit) or 1
  uint32_t cb;              // channels per unit
  uint32_t units;           // ceil(C / cb)
  uint32_t rows_per_tile;   // samples per tile
  uint32_t piece_len;       // floats of a row covered by one tile (R); cb*dim0 (S)
  uint32_t pieces;          // pieces per row (R); 1 (S)
  uint32_t sample_blocks;   // ceil(N / rows_per_tile)
  uint32_t tiles_per_unit;  // sample_blocks * pieces
  uint32_t total_tiles;     // units * tiles_per_unit
  uint32_t grid;            // thread blocks launched
  uint32_t lookahead_steps; // distance, in steps, between reducing and applying a tile
  uint32_t div_mul;         // floor(2^32 / (piece_len/vec)) + 1, see fast_div; 0 when piece_len/vec == 1
  // workspace offsets, in bytes from the workspace base
  uint32_t off_done, off_ready, off_applied, off_coef, off_rec, off_local, off_tag, off_part;
  uint64_t ws_bytes;
};

struct TileRange {
  uint32_t unit, c0, cw;     // unit index, first channel, channels in this unit
  uint32_t n0, rows;         // first sample, samples
  uint32_t col0, len;        // first column and floats per row (R); 0 and cw*dim0 (S)
  uint64_t base;             // float offset of (n0, c0, col0)
};

// n / d with mul = floor(2^32/d) + 1 (d >= 2; mul == 0 stands for d == 1).  Exact whenever
// n <= 65535 and (n/d + 1)*d <= 65536, which holds for a vector index n inside a tile of at
// most kMaxTileElems elements.
ANODE_HD uint32_t fast_div(uint32_t n, uint32_t mul)
{
  if (mul == 0) return n;
#if defined(__CUDA_ARCH__)
  return __umulhi(n, mul);
#else
  return (uint32_t)(((uint64_t)n * mul) >> 32);
#endif
}

ANODE_HD TileRange tile_range(const Plan &p, uint32_t t)
{
  TileRange r;
  r.unit = t / p.tiles_per_unit;
  const uint32_t k = t - r.unit * p.tiles_per_unit;
  const uint32_t sb = k / p.pieces;
  const uint32_t piece = k - sb * p.pieces;
  r.c0 = r.unit * p.cb;
  r.cw = (p.C - r.c0 < p.cb) ? (p.C - r.c0) : p.cb;
  r.n0 = sb * p.rows_per_tile;
  r.rows = (p.N - r.n0 < p.rows_per_tile) ? (p.N - r.n0) : p.rows_per_tile;
  if (p.regime == 0) {
    r.col0 = piece * p.piece_len;
    r.len = (p.dim0 - r.col0 < p.piece_len) ? (p.dim0 - r.col0) : p.piece_len;
  } else {
    r.col0 = 0;
    r.len = r.cw * p.dim0;
  }
  r.base = ((uint64_t)r.n0 * p.C + r.c0) * p.dim0 + r.col0;
  return r;
}

// Walks the tiles b, b+G, b+2G, ... of one thread block without a division per tile (a block
// visits hundreds of tiles and every thread needs each tile's range).  range() equals
// tile_range(p, tile()).
struct TileIter {
  uint32_t t, unit, k, G;
  ANODE_HD void init(const Plan &p, uint32_t first, uint32_t stride)
  {
    t = first; G = stride;
    unit = t / p.tiles_per_unit;
    k = t - unit * p.tiles_per_unit;
  }
  ANODE_HD uint32_t tile() const { return t; }
  ANODE_HD void advance(const Plan &p)
  {
    t += G; k += G;
    if (k >= p.tiles_per_unit) {
      if (k - p.tiles_per_unit < p.tiles_per_unit) { k -= p.tiles_per_unit; ++unit; }
      else { const uint32_t q = k / p.tiles_per_unit; unit += q; k -= q * p.tiles_per_unit; }
    }
  }
  ANODE_HD TileRange range(const Plan &p) const
  {
    TileRange r;
    r.unit = unit;
    uint32_t sb = k, piece = 0;
    if (p.pieces != 1) { sb = k / p.pieces; piece = k - sb * p.pieces; }
    r.c0 = unit * p.cb;
    r.cw = (p.C - r.c0 < p.cb) ? (p.C - r.c0) : p.cb;
    r.n0 = sb * p.rows_per_tile;
    r.rows = (p.N - r.n0 < p.rows_per_tile) ? (p.N - r.n0) : p.rows_per_tile;
    if (p.regime == 0) {
      r.col0 = piece * p.piece_len;
      r.len = (p.dim0 - r.col0 < p.piece_len) ? (p.dim0 - r.col0) : p.piece_len;
    } else {
      r.col0 = 0;
      r.len = r.cw * p.dim0;
    }
    r.base = ((uint64_t)r.n0 * p.C + r.c0) * p.dim0 + r.col0;
    return r;
  }
};

inline uint32_t ceil_div_u32(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
inline uint64_t align_up_u64(uint64_t a, uint64_t b) { return (a + b - 1) / b * b; }

// Chooses the decomposition.  `aligned16` says whether every tensor pointer of the call is
// 16-byte aligned; `resident_blocks` is how many blocks the device can hold at once
// (SM count x occupancy); `tile_floats` is the tile-size target and `slack_steps` the extra
// lookahead that hides the latency of completing a unit's statistics (both tunable).
inline Plan make_plan(uint32_t dim0, uint32_t C, uint32_t N, bool aligned16,
                      uint32_t resident_blocks, uint32_t tile_floats, uint32_t slack_steps)
{
  Plan p{};
  p.dim0 = dim0; p.C = C; p.N = N;
  const uint64_t row_stride = (uint64_t)C * dim0;
  const bool seg_ok = aligned16 && (row_stride % 4 == 0) && dim0 < 512;
  const bool row_vec = aligned16 && (dim0 % 4 == 0);
  if (tile_floats > kMaxTileElems) tile_floats = kMaxTileElems;
  if (tile_floats < 256) tile_floats = 256;

  if (seg_ok && (dim0 < 256 || !row_vec)) {
    // Regime S: rows are short and not 16-byte aligned one by one, but a block of cb channels
    // of one sample is a contiguous, aligned segment when cb*dim0 is a multiple of 4.
    p.regime = 1; p.vec = 4;
    uint32_t q = 4; if (dim0 % 2 == 0) q = 2; if (dim0 % 4 == 0) q = 1;   // cb must be a multiple of q
    const uint32_t cap4 = kThreads * kSegSlots;                          // float4 slots per sample
    uint32_t best_cb = q; double best_fill = -1.0;
    for (uint32_t cb = q; cb <= C + q - 1 && cb <= 256 && (uint64_t)cb * dim0 <= 4ull * cap4; cb += q) {
      const uint32_t seg4 = cb * dim0 / 4;
      const uint32_t slots = ceil_div_u32(seg4, kThreads) * kThreads;
      const double fill = (double)seg4 / slots;
      if (fill > best_fill + 1e-9 || (fill > best_fill - 1e-9 && cb > best_cb)) { best_fill = fill; best_cb = cb; }
    }
    p.cb = best_cb < C ? best_cb : C;   // cb == C is fine: C*dim0 is a multiple of 4 here
    p.units = ceil_div_u32(C, p.cb);
    p.piece_len = p.cb * dim0;
    p.pieces = 1;
    uint32_t rpt = tile_floats / p.piece_len; if (rpt < 1) rpt = 1; if (rpt > N) rpt = N;
    // keep at least ~2 tiles per resident block when the problem allows it
    while (rpt > 4 && (uint64_t)p.units * ceil_div_u32(N, rpt) < 2ull * resident_blocks) rpt /= 2;
    p.rows_per_tile = rpt;
  } else {
    p.regime = 0; p.vec = row_vec ? 4 : 1; p.cb = 1; p.units = C;
    uint32_t tf = tile_floats;
    for (;;) {
      if (dim0 >= tf) {
        p.pieces = ceil_div_u32(dim0, tf);
        uint32_t pl = ceil_div_u32(dim0, p.pieces);
        pl = ceil_div_u32(pl, 4) * 4;                       // keep piece starts 16-byte aligned
        p.piece_len = pl; p.pieces = ceil_div_u32(dim0, pl);
        p.rows_per_tile = 1;
      } else {
        p.pieces = 1; p.piece_len = dim0;
        uint32_t rpt = tf / dim0; if (rpt < 1) rpt = 1; if (rpt > N) rpt = N;
        p.rows_per_tile = rpt;
      }
      const uint64_t tiles = (uint64_t)C * ceil_div_u32(N, p.rows_per_tile) * p.pieces;
      if (tiles >= 2ull * resident_blocks || tf <= 1024) break;
      tf /= 2;
    }
  }
  p.sample_blocks = ceil_div_u32(N, p.rows_per_tile);
  p.tiles_per_unit = p.sample_blocks * p.pieces;
  p.total_tiles = p.units * p.tiles_per_unit;
  p.grid = p.total_tiles < resident_blocks ? p.total_tiles : resident_blocks;
  if (p.grid == 0) p.grid = 1;
  // A tile may be applied once every tile of its unit has been reduced.  Block b reduces tile
  // i + lookahead*grid before it applies tile i, so lookahead*grid >= tiles_per_unit makes the
  // wait for the unit free of cycles; the slack steps give its completion time to land.
  p.lookahead_steps = ceil_div_u32(p.tiles_per_unit, p.grid) + slack_steps;
  const uint32_t per_row = p.piece_len / p.vec ? p.piece_len / p.vec : 1;
  p.div_mul = per_row > 1 ? (uint32_t)((1ull << 32) / per_row) + 1 : 0;   // 0: divide by one

  uint64_t off = 256;                                     // header: status word and padding
  p.off_done = (uint32_t)off;    off = align_up_u64(off + 4ull * p.units, 256);
  p.off_ready = (uint32_t)off;   off = align_up_u64(off + 4ull * p.units, 256);
  p.off_applied = (uint32_t)off; off = align_up_u64(off + 4ull * p.units, 256);
  p.off_coef = (uint32_t)off;    off = align_up_u64(off + 32ull * C, 256);   // 8 floats / channel
  p.off_rec = (uint32_t)off;     off = align_up_u64(off + 8ull * C, 256);    // one tagged 64-bit record / channel
  p.off_local = (uint32_t)off;   off = align_up_u64(off + 16ull * C, 256);   // 4 floats / channel
  // two buffers of one tagged 64-bit partial per tile (used alternately, launch by launch)
  p.off_tag = (uint32_t)off;     off = align_up_u64(off + 16ull * p.total_tiles * p.cb, 256);
  p.off_part = (uint32_t)off;    off = align_up_u64(off + 16ull * p.total_tiles * p.cb, 256);
  p.ws_bytes = off;
  return p;
}

}  // namespace anode_b200
