/* Diagnostic exports of libanode_routines_gpu: the planners behind the fused batch-norm kernels, as
 * plain index arithmetic that runs without a GPU.  They exist for the tests of the tile plans and
 * schedules and for measurements (which kernel serves a shape); no counterpart in the reference,
 * whose kernels take their launch shape from KernelConfig (routines_gpu/common.cuh:51-67). */
#ifndef ANODE_ROUTINES_GPU_DIAG_H
#define ANODE_ROUTINES_GPU_DIAG_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Kernel that serves direction `dir` (0 forward, 1 backward) of a plain fused call on 16-byte
 * aligned tensors on one GPU: an ANODE_KERNEL_* value of anode_routines_gpu.h. */
int anode_gpu_batch_norm_fused_kernel_kind(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir);

/* The same for the residual-epilogue calls (anode_gpu_batch_norm_add_act_fused_*). */
int anode_gpu_batch_norm_add_act_fused_kernel_kind(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir);

/* Tile plan of the tiled and plain kernels.  out (15 values): regime, vec, cb, units, rows_per_tile,
 * piece_len, pieces, sample_blocks, tiles_per_unit, total_tiles, grid, lookahead_steps, div_mul,
 * workspace bytes (low, high).  Zero for resident_blocks / tile_floats / slack_steps = the library's
 * own values. */
int anode_gpu_batch_norm_fused_plan(uint32_t dim0, uint32_t dim1, uint32_t dim2, int aligned,
                                    uint32_t resident_blocks, uint32_t tile_floats, uint32_t slack_steps,
                                    uint32_t *out, uint32_t out_len);
/* One tile of that plan.  out (8 values): unit, c0, cw, n0, rows, col0, len, base. */
int anode_gpu_batch_norm_fused_plan_tile(uint32_t dim0, uint32_t dim1, uint32_t dim2, int aligned,
                                         uint32_t resident_blocks, uint32_t tile_floats, uint32_t tile, uint64_t *out);
/* `count` tiles first, first + stride, ... as the kernels' division-free iterator walks them (8 values each). */
int anode_gpu_batch_norm_fused_plan_walk(uint32_t dim0, uint32_t dim1, uint32_t dim2, int aligned,
                                         uint32_t resident_blocks, uint32_t tile_floats,
                                         uint32_t first, uint32_t stride, uint32_t count, uint64_t *out);

/* Geometry of the cluster kernel.  out (6 values): applies, channels per unit, blocks per cluster, samples
 * per block, units, shared-memory bytes. */
int anode_gpu_batch_norm_segres_geometry(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir, uint32_t *out);

/* Geometry of the tiled kernel (bn_ring.cuh) for direction `dir` of a fused call on 16-byte aligned tensors.
 * out (12 values): applies, rows per tile, floats per row piece, tiles per unit, slots, bytes per slot, dynamic
 * shared memory bytes, KiB between a tile's two visits (what L2 has to hold), the fraction (in 1/1000) of
 * that window loaded with the "keep" priority, thread blocks, steps between a tile's two visits, tiles. */
int anode_gpu_batch_norm_tiled_geometry(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir, uint32_t *out);

/* Plan of the slice-resident kernel for `planes` tensors per shared-memory slot.  out (16 values): applies,
 * rows per piece, parts per row, floats per part, pieces per channel, blocks per team, teams, grid, pieces
 * per block and channel, slot bytes, slots, resident-ring slots, streaming-ring slots, resident pieces per
 * channel, load-ahead slots, shared-memory bytes. */
int anode_gpu_batch_norm_resident_plan(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t planes, uint32_t *out);
/* Event sequence of thread block `block` of that plan, 4 values per event (kind, channel index in the
 * team's list, piece, slot); returns the number of events (at most max_events are written) or a negative
 * ANODE_E_* code. */
long long anode_gpu_batch_norm_resident_schedule(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t planes,
                                                 uint32_t block, uint32_t *out, uint64_t max_events);

#ifdef __cplusplus
}
#endif
#endif
