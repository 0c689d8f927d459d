/*
 * C ABI of libanode_routines_gpu (sm_100a build): the batch-norm / ReLU slice of anode's
 * GPU routine library, plus fused and multi-GPU entry points in the same style.
 *
 * Drop-in contract.  The first block below re-declares, name for name and argument for
 * argument, the symbols anode's Rust side binds through bindgen (reference
 * routines_gpu/lib.h, whitelist in build.rs:65-82 and :91-106, used from src/ops_gpu.rs via
 * src/ffi.rs:35).  An existing anode build that links this library instead of its own
 * routines for these symbols keeps working unchanged.
 *
 * Conventions shared by every entry point (reference src/ops_gpu.rs:3763-3771):
 *   - arrays are packed f32; element (i0, c, n) of a [dim0, dim1, dim2] array is at
 *     i0 + dim0*(c + dim1*n): dim0 = product of the spatial sizes, dim1 = channels,
 *     dim2 = batch.  That is a contiguous NCHW / NCDHW tensor.
 *   - every pointer is a device pointer owned by the caller; the callee allocates nothing,
 *     frees nothing and keeps no state between calls;
 *   - work is enqueued on `stream` and the call returns at once (no device synchronisation);
 *   - `cfg` is the caller's launch-shape hint {block_sz, max_block_ct}
 *     (routines_gpu/common.cuh:51-67).  It may be NULL.  The kernels here choose their own
 *     launch shapes and only read it to honour the power-of-two contract of the reduce
 *     kernels (routines_gpu/batch_norm.cu:68);
 *   - `_accumulate_` twins add into the destination (WriteCap::Accumulate,
 *     routines_gpu/common.cuh:188-193); the others overwrite it;
 *   - dim0*dim1*dim2 must be below 2^32 (the callers' sz2uint, src/ops_gpu.rs:57-61).
 */
#ifndef ANODE_ROUTINES_GPU_B200_H
#define ANODE_ROUTINES_GPU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

struct CUstream_st;

/* routines_gpu/common.cuh:51-67 (data members); Rust mirror src/ffi.rs:28-33. */
struct KernelConfig {
  uint32_t block_sz;
  uint32_t max_block_ct;
};

/* ===================================================================================
 * 1. The reference's own entry points (same names, same signatures, same semantics).
 * =================================================================================== */

/* routines_gpu/lib.h:32-39 / batch_norm.cu:59-71.  mean[c] = sum(x) / (dim0*dim2). */
void anode_gpu_batch_mean_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *x, float *mean,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:40-55 / batch_norm.cu:97-123.  dx (+)= dmean[c] / (dim0*dim2). */
void anode_gpu_batch_mean_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dmean, float *dx,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
void anode_gpu_batch_mean_bwd_3d1_packed_accumulate_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dmean, float *dx,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:56-65 / batch_norm.cu:165-179.  var[c] = sum((x-mean[c])^2)/(dim0*dim2) + epsilon
 * (biased; epsilon is folded into the stored value). */
void anode_gpu_batch_var_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon,
    const float *x, const float *mean, float *var,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:66-85 / batch_norm.cu:208-238.  dx (+)= dvar[c]*(x-mean[c])*2/(dim0*dim2). */
void anode_gpu_batch_var_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dvar, const float *x, const float *mean, float *dx,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
void anode_gpu_batch_var_bwd_3d1_packed_accumulate_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dvar, const float *x, const float *mean, float *dx,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:86-105 / batch_norm.cu:282-312.  dmean[c] (+)= sum((x-mean[c])*(-2*dvar[c]))/(dim0*dim2). */
void anode_gpu_batch_var_bwd_mean_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dvar, const float *x, const float *mean, float *dmean,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
void anode_gpu_batch_var_bwd_mean_3d1_packed_accumulate_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dvar, const float *x, const float *mean, float *dmean,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:106-115 / batch_norm.cu:338-352.  y = (x-mean[c]) * rsqrt(var[c]). */
void anode_gpu_batch_norm_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *x, const float *mean, const float *var, float *y,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:116-133 / batch_norm.cu:378-406.  dx (+)= dy * rsqrt(var[c]). */
void anode_gpu_batch_norm_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *var, float *dx,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
void anode_gpu_batch_norm_bwd_3d1_packed_accumulate_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *var, float *dx,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:134-151 / batch_norm.cu:446-474.  dmean[c] (+)= sum(dy) * (-rsqrt(var[c])). */
void anode_gpu_batch_norm_bwd_mean_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *var, float *dmean,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
void anode_gpu_batch_norm_bwd_mean_3d1_packed_accumulate_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *var, float *dmean,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:152-173 / batch_norm.cu:517-549.
 * dvar[c] (+)= sum(dy*(x-mean[c])) * (-0.5*rsqrt(var[c])/var[c]). */
void anode_gpu_batch_norm_bwd_var_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *x, const float *mean, const float *var, float *dvar,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
void anode_gpu_batch_norm_bwd_var_3d1_packed_accumulate_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *x, const float *mean, const float *var, float *dvar,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:174-193 / batch_norm.cu:589-619.  dvar[c] (+)= sum(-dy*y*0.5/var[c]), y the
 * normalized output saved from the forward pass. */
void anode_gpu_batch_norm_bwd_var_v2_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *y, const float *var, float *dvar,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
void anode_gpu_batch_norm_bwd_var_v2_3d1_packed_accumulate_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    const float *dy, const float *y, const float *var, float *dvar,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:296-302 / flat_join.cu:50-60.  y = x1 * (float)(x2 > 0). */
void anode_gpu_M1_copy_map_M2_unit_step_map_R_product_reduce_flat_join_f32(
    uint32_t len, const float *x1, const float *x2, float *y,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:344-349 / flat_map.cu:392-401.  y = x * (float)(x > 0); y may alias x
 * (src/ops_gpu.rs:7912-7918). */
void anode_gpu_positive_clip_flat_map_f32(
    uint32_t len, const float *x, float *y,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* lib.h:350-356 / flat_map.cu:403-413.  dx = dy * (float)(y > 0); dx may alias dy
 * (src/ops_gpu.rs:7929-7939). */
void anode_gpu_positive_clip_flat_map_bwd_f32(
    uint32_t len, const float *dy, const float *y, float *dx,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* ===================================================================================
 * 2. Fused batch-norm + ReLU (new; backs BatchNormalize{2,3}dFusedOp and
 *    BatchNormalize{2,3}dBwdFusedOp, which src/ops.rs:105-106 declares but never builds).
 *
 * One launch per direction replaces the reference's eleven (src/ops.rs:999-1014 forward,
 * src/ops_gpu.rs:4344-4352, 3997-4003, 3787-3791 backward, flat_map.cu:392-413 ReLU).
 *
 * Return value: 0 on success, a negative ANODE_E_* code when the arguments are rejected
 * before anything is enqueued.  Run-time trouble inside the kernel (a bounded wait that
 * ran out) is reported through the status word read by anode_gpu_batch_norm_fused_status.
 * =================================================================================== */

#define ANODE_OK            0
#define ANODE_E_NULL       -1   /* a required pointer is NULL */
#define ANODE_E_DIMS       -2   /* a dimension is 0 or dim0*dim1*dim2 >= 2^32 */
#define ANODE_E_WORKSPACE  -3   /* workspace missing, misaligned or too small */
#define ANODE_E_LAUNCH     -4   /* the CUDA runtime refused the launch */
#define ANODE_E_COMM       -5   /* communicator missing / inconsistent / NCCL failure */
#define ANODE_E_ALIGN      -6   /* tensor pointers must be 4-byte aligned */
#define ANODE_E_TOO_LARGE  -7   /* the problem needs more scratch than the library's built-in array holds */

/* Bits of the device status word. */
#define ANODE_ST_WAIT_STATS   1u  /* a wait for a channel's statistics ran out */
#define ANODE_ST_WAIT_PEER    2u  /* a wait for another GPU's partials ran out */
#define ANODE_ST_ABORTED      4u  /* some block saw the bits above and skipped work */

/* Kernels behind the fused calls.  ANODE_KERNEL_AUTO (the default) picks by shape:
 *   TILED     persistent kernel streaming tiles through a shared-memory ring, re-reading them from L2
 *             (long 16-byte aligned rows);
 *   CLUSTER   thread-block clusters keeping a unit's slice in shared memory (short rows, small channels);
 *   RESIDENT  slices resident in shared memory, all global traffic by bulk copies; takes the residual
 *             epilogue on long rows, also in synchronized calls;
 *   PLAIN     plain loads and stores (any shape, any alignment; one GPU).
 * anode_gpu_batch_norm_fused_set_kernel makes another choice process-wide: that kernel is used wherever
 * it applies, the automatic choice elsewhere.  Meant for tests and measurements. */
#define ANODE_KERNEL_AUTO      0
#define ANODE_KERNEL_TILED     1
#define ANODE_KERNEL_CLUSTER   2
#define ANODE_KERNEL_RESIDENT  3
#define ANODE_KERNEL_PLAIN     4
int anode_gpu_batch_norm_fused_set_kernel(int kernel);

/* Bound of every wait inside the kernels (for a channel's statistics, for another GPU's records), in
 * milliseconds of SM clock at 2 GHz; default 1500.  A wait that runs out sets ANODE_ST_WAIT_* and
 * ANODE_ST_ABORTED in the status word, the kernel drains and returns, and the workspace has to be
 * re-initialised before its next use.  Process-wide; applies to calls made afterwards. */
int anode_gpu_batch_norm_fused_set_wait_limit_ms(uint32_t ms);

/* Scratch the fused kernels need for a [dim0, dim1, dim2] problem: per-tile partial
 * statistics, per-channel coefficients, progress counters; one part per direction (each
 * direction keeps state in its part from launch to launch).  A few hundred KB to a few MB. */
size_t anode_gpu_batch_norm_fused_workspace_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2);

/* Zeroes a workspace (cudaMemsetAsync on `stream`).  Needed once after allocation, after any call
 * whose status word came back non-zero, and whenever the workspace is to serve ANOTHER problem: a
 * workspace belongs to one (dim0, dim1, dim2) and one alignment class of the tensor pointers (all
 * 16-byte aligned or not), because the kernels keep state in it from launch to launch that is laid
 * out by the problem's tile plan.  Otherwise the kernels leave it ready for the next launch, so
 * back-to-back launches of the same problem on one stream share it. */
int anode_gpu_batch_norm_fused_workspace_init(void *workspace, size_t bytes, struct CUstream_st *stream);

/* Copies the status word of a workspace to the host (synchronises `stream`). 0 = clean. */
int anode_gpu_batch_norm_fused_status(const void *workspace, struct CUstream_st *stream, uint32_t *status);

/* Forward, training mode:
 *   mean[c] = sum(x)/M                              M = dim0*dim2
 *   var[c]  = sum((x-mean)^2)/M + epsilon           (biased, epsilon folded in, as anode stores it)
 *   run_mean += avg_rate*(mean - run_mean); run_var += avg_rate*(var - run_var)
 *                                                   (skipped when the pointer is NULL)
 *   y = relu(gamma[c]*(x-mean[c])*var[c]^-1/2 + beta[c])
 * gamma == NULL means no affine (the reference's behaviour); beta may be NULL with gamma set.
 * relu == 0 leaves out the ReLU.  x and y may alias. */
int anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    float epsilon, float avg_rate, int relu,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* Backward of the above.  The ReLU mask is recomputed from x (y is not read):
 *   dz = dy * (gamma*xhat + beta > 0)         xhat = (x-mean)*var^-1/2
 *   dbeta = sum(dz), dgamma = sum(dz*xhat)    (written when the pointers are non-NULL)
 *   dx = gamma*var^-1/2 * (dz - dbeta/M - xhat*dgamma/M)
 * which is the closed form of the reference's dvar/dmean/dx kernel chain.
 * accumulate != 0 adds into dx instead of overwriting it.  dx may alias dy. */
int anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, int relu, int accumulate,
    const float *dy, const float *x, const float *mean, const float *var,
    const float *gamma, const float *beta,
    float *dx, float *dgamma, float *dbeta,
    void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* The two calls above with a general activation after the affine step,
 *   act(t) = t * (t > 0 ? 1 : neg_slope):   0 = ReLU (the calls above with relu = 1), 1 = none
 *   (relu = 0), c = leaky ReLU with constant c, the reference's LeakyReluFlatMap
 *   y = (mask + (1-mask)*c)*x and its adjoint dx = (mask + (1-mask)*c)*dy (flat_map.cu:44-69). */
int anode_gpu_batch_norm_act_fused_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    float epsilon, float avg_rate, float neg_slope,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
int anode_gpu_batch_norm_act_fused_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float neg_slope, int accumulate,
    const float *dy, const float *x, const float *mean, const float *var,
    const float *gamma, const float *beta,
    float *dx, float *dgamma, float *dbeta,
    void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* Residual-block epilogue: y = act(bn(x) + residual), act as above -- the step that follows
 * batch-norm in every residual block (examples/run_imagenet_mpi.rs:191-195, 224-226: shortcut plus
 * normalized branch, then positive_clip).  Backward: the mask is taken from the saved output y (as
 * the reference's positive_clip adjoint does, flat_map.cu:187-194); dresidual = dy*mask is the
 * gradient of the shortcut (may be NULL, may alias dy); dx, dgamma, dbeta as in the calls above.
 * Served by the cluster kernel for short rows, by the slice-resident kernel for long 16-byte aligned
 * rows and by the plain kernel otherwise (12 / 20 algorithmic bytes per element forward / backward). */
int anode_gpu_batch_norm_add_act_fused_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    float epsilon, float avg_rate, float neg_slope,
    const float *x, const float *residual, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
int anode_gpu_batch_norm_add_act_fused_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float neg_slope, int accumulate,
    const float *dy, const float *x, const float *y, const float *mean, const float *var,
    const float *gamma, const float *beta,
    float *dx, float *dresidual, float *dgamma, float *dbeta,
    void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* Forward pass for callers that have no scratch memory to give.  No counterpart in the
 * reference.  Same arguments and results as anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32
 * minus the workspace: anode's op closures pass only dimensions, inputs, pre-made outputs, a
 * launch hint and a stream (src/ops_gpu.rs:3763-3771), and code inside a memory-pool transaction
 * must not call cudaMalloc (it synchronises the device), so neither can provide a workspace.
 * The scratch is a fixed array of ANODE_STATIC_SCRATCH_BYTES inside the library, held on every GPU
 * that loads it until the process exits; this call allocates and frees nothing.
 *   - Problems whose forward kernel needs more scratch than the array holds return ANODE_E_TOO_LARGE
 *     and enqueue nothing (half of anode_gpu_batch_norm_fused_workspace_bytes is an upper bound of the
 *     need; shapes served by the cluster kernel need none).
 *   - All calls on a device share the array, which keeps the previous call's contents; every call
 *     first clears, on `stream`, the part that has to start at zero.  Calls that may overlap on
 *     the GPU (different streams without an ordering between them) race on it: serialise them.
 *   - The first call on each device looks up the array's device address; make that first call
 *     with the device current and outside of any stream capture. */
#define ANODE_STATIC_SCRATCH_BYTES (4u << 20)
int anode_gpu_batch_norm_relu_fused_fwd_static_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    float epsilon, float avg_rate, int relu,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
/* Status word of the built-in array (as anode_gpu_batch_norm_fused_status for a workspace; synchronises
 * `stream`).  It describes the last call of the entry point above on the current device and is cleared
 * by the next one, so read it before making another call.  No counterpart in the reference. */
int anode_gpu_batch_norm_fused_static_status(struct CUstream_st *stream, uint32_t *status);

/* Forward + backward of one layer whose tensors are in HOST memory (no counterpart in the
 * reference, which moves whole arrays with separate copies: MemArray4d -> device array,
 * tests/test_gpu.rs:138-160).  host_x, host_dy, host_y, host_dx are packed [dim0, dim1, dim2]
 * host tensors, page-locked for the copies to overlap; every other pointer is a device pointer as
 * in the two calls above (mean, var, dgamma, dbeta ... are [dim1]).  The layer is processed in
 * blocks of `chunk_channels` channels (0 = let the library choose): block k+1 is copied to the
 * device while block k is computed and block k-1 is copied back, so both directions of the link
 * are busy at once.  `staging` is device memory of anode_gpu_batch_norm_host_step_staging_bytes
 * bytes, 256-byte aligned, contents irrelevant (it also holds the workspace; its first word is the
 * status word anode_gpu_batch_norm_fused_status reads).  Kernels run on `stream`, copies on two
 * streams the library creates once per device; when the call returns everything is enqueued and
 * `stream` ends after the last copy.  Make the first call on a device outside of stream capture.
 * host_y may be host_x and host_dx may be host_dy. */
size_t anode_gpu_batch_norm_host_step_staging_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                                    uint32_t chunk_channels);
/* Number of channel blocks the call below cuts the layer into (two kernel launches each). */
uint32_t anode_gpu_batch_norm_host_step_blocks(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                               uint32_t chunk_channels);
int anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    float epsilon, float avg_rate, int relu,
    const float *host_x, const float *host_dy, const float *gamma, const float *beta,
    float *host_y, float *host_dx,
    float *mean, float *var, float *run_mean, float *run_var, float *dgamma, float *dbeta,
    void *staging, size_t staging_bytes, uint32_t chunk_channels,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* Batch-norm with given statistics fused with the activation that follows it (one pass, 8 bytes
 * per element): the inference branch of batch_normalize_2d/3d (src/ops.rs:1010-1011, the switch on
 * `online` selects the running averages; anode_gpu_batch_norm_3d1_packed_f32 computes it without
 * activation) followed by positive_clip (flat_map.cu:172-179) or leaky ReLU (flat_map.cu:44-52):
 *   y = act(gamma[c]*(x-mean[c])*var[c]^-1/2 + beta[c]),  act(t) = t*(t > 0 ? 1 : neg_slope)
 * neg_slope = 0: ReLU, 1: no activation, c: leaky ReLU with constant c.  var is biased variance +
 * epsilon, as anode stores it.  gamma/beta may be NULL.  y may be x. */
int anode_gpu_batch_norm_act_infer_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float neg_slope,
    const float *x, const float *mean, const float *var, const float *gamma, const float *beta,
    float *y, const struct KernelConfig *cfg, struct CUstream_st *stream);

/* Running-statistic update on its own (OnlineAverageOp, src/ops_gpu.rs:6034-6077; rule
 * pinned by tests/test_gpu.rs:561-593):  y[i] += rate*(x[i] - y[i]). */
int anode_gpu_online_average_f32(
    uint32_t len, float rate, const float *x, float *y,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* ===================================================================================
 * 3. Synchronized batch-norm over the GPUs of one node (new).
 *
 * Every rank holds a shard of the batch (or a spatial slab) with all dim1 channels; statistics
 * and the backward sums are taken over all shards.  The reference has no counterpart: its
 * batch-norm is per process, and its one collective is the host-staged MPI allreduce of
 * gradients (src/proc_mpi.rs:138-148 called from SumSpmdOp, src/ops_gpu.rs:538-545), whose
 * role for this path the exchange below takes over, on the device, over NVLink.
 *
 * One process per GPU.  Rank 0 obtains a unique id, distributes it by any means (128 bytes),
 * and every rank creates its communicator with the CUDA device it will use made current.
 * Calls on a communicator are collective: every rank makes the same sequence of calls.
 * =================================================================================== */
struct AnodeSyncComm;

size_t anode_gpu_sync_unique_id_bytes(void);
int anode_gpu_sync_get_unique_id(void *out);
int anode_gpu_sync_comm_create(const void *unique_id, int rank, int world, struct AnodeSyncComm **out);
int anode_gpu_sync_comm_destroy(struct AnodeSyncComm *comm);
/* The same handle without NCCL behind it, for callers that bring their own peer-mapped memory: the
 * synchronized calls work once an exchange buffer is attached (below) and return ANODE_E_COMM before;
 * anode_gpu_sync_allreduce_sum_f32 is not available on it.  Nothing blocks on the host. */
int anode_gpu_sync_comm_create_exchange_only(int rank, int world, struct AnodeSyncComm **out);

/* In-place sum of buf[0..len) over the ranks (ncclAllReduce on `stream`): the device-side form of
 * SumSpmdOp's host-staged MPI_Allreduce of gradients (src/ops_gpu.rs:538-545,
 * src/proc_mpi.rs:138-148), reusing the communicator of the synchronized batch-norm. */
int anode_gpu_sync_allreduce_sum_f32(struct AnodeSyncComm *comm, float *buf, size_t len, struct CUstream_st *stream);

/* Optional: exchange inside the kernels instead of an NCCL all-gather between them.
 * Every rank allocates a buffer of anode_gpu_sync_exchange_bytes(max_channels, world) bytes that
 * all ranks of the node can address (peer-mapped / symmetric memory), zeroes it once, and passes
 * the world's buffers, as mapped into its own address space and indexed by rank, to
 * anode_gpu_sync_comm_attach_exchange (peer_ptrs[rank] is the local buffer).  From then on the
 * synchronized calls with dim1 <= max_channels run as ONE kernel per direction: the block that
 * completes a channel on a GPU stores that GPU's 24-byte record into every rank's buffer with
 * plain stores over NVLink and all blocks read the records from their own GPU's memory (no
 * multicast, no loads from peer memory).  Records carry the call's sequence number, so nothing
 * has to be cleared between calls; all ranks must make the same sequence of synchronized calls.
 * Waits on peers are bounded (ANODE_ST_WAIT_PEER in the status word). */
size_t anode_gpu_sync_exchange_bytes(uint32_t max_channels, int world);
int anode_gpu_sync_comm_attach_exchange(struct AnodeSyncComm *comm, void *const *peer_ptrs, uint32_t max_channels);

/* Scratch for a LOCAL [dim0, dim1, dim2] shard when `world` ranks take part. */
size_t anode_gpu_sync_batch_norm_workspace_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2, int world);

/* Forward: as anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32, with mean / var / running
 * statistics over the global batch (every rank receives the same values). */
int anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    float epsilon, float avg_rate, int relu,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* Backward: as anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32; dgamma / dbeta are the
 * global sums (identical on every rank) and `global_count` is the number of elements per
 * channel over all ranks (the M of the formulas). */
int anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count, int relu, int accumulate,
    const float *dy, const float *x, const float *mean, const float *var,
    const float *gamma, const float *beta,
    float *dx, float *dgamma, float *dbeta,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32 for one rank's shard of a batch sharded over
 * the ranks of `comm`: host tensors in, host tensors out, channel blocks travelling in both directions
 * while the synchronized kernels of the block in between run.  Every rank cuts the layer into the same
 * blocks (the default block size follows from global_count and the number of ranks; pass the same
 * chunk_channels everywhere otherwise) and so makes the same sequence of synchronized launches.
 * `staging` as in the one-GPU call, sized by anode_gpu_sync_batch_norm_host_step_staging_bytes. */
size_t anode_gpu_sync_batch_norm_host_step_staging_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count,
                                                         struct AnodeSyncComm *comm, uint32_t chunk_channels);
uint32_t anode_gpu_sync_batch_norm_host_step_blocks(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count,
                                                    struct AnodeSyncComm *comm, uint32_t chunk_channels);
int anode_gpu_sync_batch_norm_relu_step_host_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count,
    float epsilon, float avg_rate, int relu,
    const float *host_x, const float *host_dy, const float *gamma, const float *beta,
    float *host_y, float *host_dx,
    float *mean, float *var, float *run_mean, float *run_var, float *dgamma, float *dbeta,
    struct AnodeSyncComm *comm, void *staging, size_t staging_bytes, uint32_t chunk_channels,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

/* The residual-block epilogue of anode_gpu_batch_norm_add_act_fused_{fwd,bwd}_3d1_packed_f32 with
 * statistics and backward sums over all ranks: y = act(bn(x) + residual) per shard (shortcut plus
 * normalized branch, then positive_clip: examples/run_imagenet_mpi.rs:191-195, 224-226, which the
 * reference trains data-parallel).  On long 16-byte aligned rows one kernel per direction (the
 * slice-resident kernel with the exchange inside), on short rows the cluster kernel, otherwise reduce
 * kernel, exchange kernel, apply kernel. */
int anode_gpu_sync_batch_norm_add_act_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2,
    float epsilon, float avg_rate, float neg_slope,
    const float *x, const float *residual, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);
int anode_gpu_sync_batch_norm_add_act_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count, float neg_slope, int accumulate,
    const float *dy, const float *x, const float *y, const float *mean, const float *var,
    const float *gamma, const float *beta,
    float *dx, float *dresidual, float *dgamma, float *dbeta,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream);

#ifdef __cplusplus
}
#endif
#endif
