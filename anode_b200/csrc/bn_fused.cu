// Host side of the fused batch-norm (+ReLU) entry points: argument checks, the tile plan,
// and the cooperative launch of the persistent kernels of bn_fused.cuh.
#include "bn_host.h"
// the warp-specialised kernel, instantiated with 8 and with 16 consumer warps
#define ANODE_RING_NS ring8
#define ANODE_RING_CONSUMERS 256
#include "bn_ring.cuh"
#undef ANODE_RING_NS
#undef ANODE_RING_CONSUMERS
#define ANODE_RING_NS ring16
#define ANODE_RING_CONSUMERS 512
#include "bn_ring.cuh"
#undef ANODE_RING_NS
#undef ANODE_RING_CONSUMERS

namespace anode_b200 {

// ---- planner constants, from sweeps on B200 -------------------------------------------------------
#ifndef ANODE_SLACK_STEPS
#define ANODE_SLACK_STEPS 2
#endif
#ifndef ANODE_RING_SLOTS_FWD
#define ANODE_RING_SLOTS_FWD 3
#endif
#ifndef ANODE_RING_SLOTS_BWD
#define ANODE_RING_SLOTS_BWD 4
#endif
#ifndef ANODE_RING_FLOATS_FWD
#define ANODE_RING_FLOATS_FWD 16384
#endif
#ifndef ANODE_RING_FLOATS_BWD
#define ANODE_RING_FLOATS_BWD 8192
#endif
const Tunables &tunables()
{
  static const Tunables t = {
      32768,    // tile_floats
      ANODE_SLACK_STEPS,        // slack_steps
      4,        // blocks_per_sm
      ANODE_RING_SLOTS_FWD,     // ring_slots
      ANODE_RING_SLOTS_BWD,     // ring_slots_bwd
      ANODE_RING_FLOATS_FWD,    // ring_floats_fwd
      ANODE_RING_FLOATS_BWD,    // ring_floats_bwd
      1,        // ring_blocks_per_sm
      8,        // ring_warps_fwd
      16,       // ring_warps_bwd
  };
  return t;
}

// Which kernel serves the fused calls: ANODE_KERNEL_AUTO picks by shape; any other value is tried first
// where that kernel applies (set by tests and measurements, process-wide).
static std::atomic<int> g_kernel_choice{ANODE_KERNEL_AUTO};
int kernel_choice() { return g_kernel_choice.load(std::memory_order_relaxed); }

uint32_t sm_count()
{
  // one entry per device ordinal; 148 (B200) when no device can be queried, so that the
  // planning helpers stay callable on a machine without a GPU
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return 148; }
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
      (void)cudaGetLastError();
      v = 148;
    }
    cache[dev].store(v, std::memory_order_relaxed);
  }
  return (uint32_t)v;
}

Plan plan_for(uint32_t dim0, uint32_t C, uint32_t N, bool aligned16)
{
  const Tunables &t = tunables();
  return make_plan(dim0, C, N, aligned16, sm_count() * t.blocks_per_sm, t.tile_floats, 1);
}

// Shared-memory layout of the warp-specialised kernel for plan `p` (see bn_ring.cuh).
// consumer warps of direction `dir`: 8 or 16 (the two instantiations of bn_ring.cuh)
static uint32_t ring_warps(int dir)
{
  const Tunables &t = tunables();
  return (dir == 0 ? t.ring_warps_fwd : t.ring_warps_bwd) >= 16 ? 16u : 8u;
}

static RingGeom ring_geom(const Plan &p, int dir, uint32_t slots, uint32_t slot_floats)
{
  RingGeom g{};
  g.slots = slots; g.slot_floats = slot_floats;
  uint32_t off = kRingCtlBytes;
  const uint32_t cwarps = ring_warps(dir);
  g.res_stride = p.cb > cwarps ? p.cb : cwarps;   // regime R: one partial per consumer warp
  g.off_res = off;  off += (uint32_t)align_up_u64((uint64_t)kResQ * g.res_stride * 16, 128);
  g.off_coef = off; off += (uint32_t)align_up_u64((uint64_t)kCoefQ * p.cb * 32, 128);
  g.off_slots = off;
  g.slot_stride = (uint32_t)align_up_u64((uint64_t)slot_floats * 4 * (dir == 1 ? 2 : 1) + (dir == 1 ? (uint64_t)p.cb * 16 : 0), 128);
  g.smem_bytes = off + slots * g.slot_stride;
  return g;
}

// Plan for the warp-specialised kernel, or false when it does not apply (scalar paths, tiles that
// do not fit a slot, too little shared memory): the caller then uses the plain kernel.
// Plan and geometry for `slots` slots of `slot_floats` floats (per tensor); false when they do not fit.
static bool ring_plan_with(uint32_t dim0, uint32_t C, uint32_t N, int dir, uint32_t slots, uint32_t slot_floats, Plan &p, RingGeom &g)
{
  const Tunables &t = tunables();
  slot_floats = (slot_floats / 4) * 4;
  if (slot_floats < 1024) slot_floats = 1024;
  slots = slots < 2 ? 2 : (slots > kMaxSlots ? kMaxSlots : slots);
  uint32_t bps = t.ring_blocks_per_sm ? t.ring_blocks_per_sm : 1;
  p = make_plan(dim0, C, N, true, sm_count() * bps, slot_floats, t.slack_steps);
  // short rows (regime S) belong to the cluster kernel or the plain kernel
  if (p.vec != 4 || p.regime != 0) return false;
  // a tile must fit one slot: rows * len <= slot_floats
  const uint64_t tile_max = (uint64_t)p.rows_per_tile * p.piece_len;
  if (tile_max > slot_floats) return false;
  slot_floats = (uint32_t)((tile_max + 31) / 32 * 32);     // slots no larger than the largest tile
  g = ring_geom(p, dir, slots, slot_floats);
  const uint32_t budget = 227u * 1024u;
  while (g.smem_bytes > budget && slots > 2) { --slots; g = ring_geom(p, dir, slots, slot_floats); }
  return g.smem_bytes <= budget;
}

// Bytes between the two visits of a tile: what L2 has to hold for the apply visit to find its tile there.
static uint64_t ring_window_bytes(const Plan &p, int dir)
{
  return (uint64_t)p.lookahead_steps * p.grid * p.rows_per_tile * p.piece_len * 4 * (dir == 1 ? 2 : 1);
}

// Backward pass: three slots of larger tiles are faster than four of the standard ones as long as the larger
// window they make still fits what L2 keeps ([256,256,56,56]: 0.50 -> 0.44 ms; with a 56 MB window 10 % slower).
constexpr uint32_t kRingLargeSlotsBwd = 3, kRingLargeFloatsBwd = 9408;
constexpr uint64_t kRingLargeWindowMax = 48ull << 20;     // also the part of a larger window that is marked "keep" (launch_ring)

bool ring_plan_for(uint32_t dim0, uint32_t C, uint32_t N, bool aligned, int dir, Plan &p, RingGeom &g)
{
  const Tunables &t = tunables();
  if (!aligned) return false;
  if (!ring_plan_with(dim0, C, N, dir, dir == 0 ? t.ring_slots : t.ring_slots_bwd,
                      dir == 0 ? t.ring_floats_fwd : t.ring_floats_bwd, p, g)) return false;
  if (dir == 1) {
    Plan pl; RingGeom gl;
    if (ring_plan_with(dim0, C, N, dir, kRingLargeSlotsBwd, kRingLargeFloatsBwd, pl, gl) && gl.slots == kRingLargeSlotsBwd &&
        (uint64_t)pl.rows_per_tile * pl.piece_len > (uint64_t)p.rows_per_tile * p.piece_len &&
        ring_window_bytes(pl, dir) <= kRingLargeWindowMax) {
      p = pl; g = gl;
    }
  }
  return true;
}

typedef void (*RingKernel)(const FusedArgs, const RingGeom);

static RingKernel pick_ring_kernel(const Plan &p, int dir, uint32_t &threads)
{
  // only regime R reaches this point (ring_plan_for)
  (void)p;
  if (ring_warps(dir) == 16) {
    threads = ring16::kRingThreads;
    return dir == 0 ? ring16::bn_ring_kernel<0> : ring16::bn_ring_kernel<1>;
  }
  threads = ring8::kRingThreads;
  return dir == 0 ? ring8::bn_ring_kernel<0> : ring8::bn_ring_kernel<1>;
}

int launch_ring(FusedArgs &a, const RingGeom &g_in, int dir, cudaStream_t stream)
{
  RingGeom g = g_in;
  uint32_t threads = 0;
  RingKernel k = pick_ring_kernel(a.plan, dir, threads);
  static std::mutex mu;
  static std::map<std::pair<const void *, uint32_t>, int> occ;     // (kernel, smem) -> blocks per SM
  int per_sm = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_pair((const void *)k, g.smem_bytes);
    auto it = occ.find(key);
    if (it == occ.end()) {
      if (cudaFuncSetAttribute((const void *)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024)) != cudaSuccess ||
          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, (int)threads, g.smem_bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        per_sm = 0;
      }
      occ[key] = per_sm;
    } else {
      per_sm = it->second;
    }
  }
  const uint32_t fit = (uint32_t)per_sm * sm_count();
  if (fit == 0) return ANODE_E_LAUNCH;
  if (a.plan.grid > fit) {
    a.plan.grid = fit;
    a.plan.lookahead_steps = ceil_div_u32(a.plan.tiles_per_unit, a.plan.grid) + tunables().slack_steps;
  }
  a.use_rec = a.mode == MODE_FUSED ? 1u : 0u;
  // A window larger than what L2 keeps would cycle through it whole (config 3, backward: 67 MB); marking only
  // the part that fits lets that part stay (backward 4.42 -> 4.27 ms).  Smaller windows keep everything.
  const uint64_t window = ring_window_bytes(a.plan, dir);
  g.keep_frac = window > kRingLargeWindowMax ? (float)((double)kRingLargeWindowMax / (double)window) : 1.0f;
  void *params[] = {(void *)&a, (void *)&g};
  cudaError_t e;
  if (a.mode == MODE_FUSED)
    e = cudaLaunchCooperativeKernel((const void *)k, dim3(a.plan.grid), dim3(threads), params, g.smem_bytes, stream);
  else
    e = cudaLaunchKernel((const void *)k, dim3(a.plan.grid), dim3(threads), params, g.smem_bytes, stream);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return ANODE_E_LAUNCH; }
  return ANODE_OK;
}

// The caller's workspace holds two independent parts, one per direction (forward first): a
// direction's kernels keep state in their part from launch to launch (which partial buffer is
// current, words waiting to be cleared), laid out by that direction's own tile plan, so forward
// and backward launches must not share one.  The status word is the first word of the whole.
// Bytes of a part taken by the tile-plan kernels (plain, warp-specialised, cluster); the records of the
// slice-resident kernel follow behind them.
static uint64_t tiled_part_bytes(uint32_t dim0, uint32_t C, uint32_t N)
{
  // the plan depends on pointer alignment, which is not known yet: cover both cases
  const Plan a = plan_for(dim0, C, N, true), b = plan_for(dim0, C, N, false);
  uint64_t need = a.ws_bytes > b.ws_bytes ? a.ws_bytes : b.ws_bytes;
  for (int dir = 0; dir < 2; ++dir) {
    Plan rp; RingGeom g;
    if (ring_plan_for(dim0, C, N, true, dir, rp, g) && rp.ws_bytes > need) need = rp.ws_bytes;
  }
  return align_up_u64(need, 256);
}

uint64_t workspace_part_bytes(uint32_t dim0, uint32_t C, uint32_t N)
{
  return align_up_u64(tiled_part_bytes(dim0, C, N) + resident_ws_bytes(dim0, C, N), 256);
}

// Bytes at the start of a workspace that hold progress counters, flags and records, i.e. what has
// to be zero when a launch begins (the per-tile partials behind them are written before they are read).
uint64_t control_region_bytes(uint32_t dim0, uint32_t C, uint32_t N, bool aligned)
{
  uint64_t n = plan_for(dim0, C, N, aligned).off_part;
  for (int dir = 0; dir < 2; ++dir) {
    Plan rp; RingGeom g;
    if (ring_plan_for(dim0, C, N, aligned, dir, rp, g) && rp.off_part > n) n = rp.off_part;
  }
  // the slice-resident kernel's records validate themselves against the launch counter in the header,
  // which the clearing resets: they have to go too
  if (aligned && resident_ws_bytes(dim0, C, N)) n = workspace_part_bytes(dim0, C, N);
  return n;
}

// True when the warp-specialised kernel will serve this call (the in-kernel exchange needs it).
bool ring_applies(const FusedArgs &a, int dir, bool aligned)
{
  Plan rp; RingGeom g;
  return ring_plan_for(a.plan.dim0, a.plan.C, a.plan.N, aligned, dir, rp, g) && rp.ws_bytes <= a.ws_capacity;
}

// Which kernel launch_best takes for a prepared call: ANODE_KERNEL_* (never AUTO), or -1 when none can
// (a synchronized call in fused mode on a shape only the plain kernel takes: it has no exchange).
int pick_kernel_kind(const FusedArgs &a, int dir, bool aligned)
{
  const bool extra = a.res || a.ymask || a.dres;        // residual epilogue
  const bool plain_ok = !(a.mode == MODE_FUSED && a.world > 1);
  Plan rp; RingGeom g;
  const bool tiled_ok = !extra && ring_plan_for(a.plan.dim0, a.plan.C, a.plan.N, aligned, dir, rp, g) && rp.ws_bytes <= a.ws_capacity;
  switch (kernel_choice()) {
    case ANODE_KERNEL_TILED: if (tiled_ok) return ANODE_KERNEL_TILED; break;
    case ANODE_KERNEL_CLUSTER: if (segres_applies(a, dir, aligned)) return ANODE_KERNEL_CLUSTER; break;
    case ANODE_KERNEL_RESIDENT: if (resident_applies(a, dir, aligned)) return ANODE_KERNEL_RESIDENT; break;
    case ANODE_KERNEL_PLAIN: if (plain_ok) return ANODE_KERNEL_PLAIN; break;
    default: break;
  }
  if (extra) {
    // short rows: the cluster kernel; otherwise the plain kernel on one GPU (measured faster there) and
    // the slice-resident kernel, which has the exchange inside, in synchronized calls
    if (segres_applies(a, dir, aligned)) return ANODE_KERNEL_CLUSTER;
    if (plain_ok) return ANODE_KERNEL_PLAIN;
    return resident_applies(a, dir, aligned) ? ANODE_KERNEL_RESIDENT : -1;
  }
  // short rows, and channels small enough to sit in a few blocks' shared memory: the cluster kernel
  if (segres_preferred(a, dir, aligned)) return ANODE_KERNEL_CLUSTER;
  if (tiled_ok) return ANODE_KERNEL_TILED;
  if (segres_applies(a, dir, aligned)) return ANODE_KERNEL_CLUSTER;
  if (plain_ok) return ANODE_KERNEL_PLAIN;
  return resident_applies(a, dir, aligned) ? ANODE_KERNEL_RESIDENT : -1;
}

// Launches direction `dir` of a prepared call with the kernel pick_kernel_kind names.  A cluster launch
// the device refuses falls back to the next kernel that applies.
int launch_best(FusedArgs &a, int dir, bool aligned, cudaStream_t stream)
{
  int kind = pick_kernel_kind(a, dir, aligned);
  if (kind == ANODE_KERNEL_CLUSTER) {
    if (launch_segres(a, dir, stream) == ANODE_OK) return ANODE_OK;
    const bool extra = a.res || a.ymask || a.dres;
    Plan rp; RingGeom g;
    if (!extra && ring_plan_for(a.plan.dim0, a.plan.C, a.plan.N, aligned, dir, rp, g) && rp.ws_bytes <= a.ws_capacity) kind = ANODE_KERNEL_TILED;
    else if (resident_applies(a, dir, aligned)) kind = ANODE_KERNEL_RESIDENT;
    else kind = (a.mode == MODE_FUSED && a.world > 1) ? -1 : ANODE_KERNEL_PLAIN;
  }
  if (kind == ANODE_KERNEL_TILED) {
    Plan rp; RingGeom g;
    if (!ring_plan_for(a.plan.dim0, a.plan.C, a.plan.N, aligned, dir, rp, g)) return ANODE_E_LAUNCH;
    a.plan = rp;
    return launch_ring(a, g, dir, stream);
  }
  if (kind == ANODE_KERNEL_RESIDENT) return launch_resident(a, dir, tiled_part_bytes(a.plan.dim0, a.plan.C, a.plan.N), stream);
  if (kind == ANODE_KERNEL_PLAIN) return launch_pipeline(a, dir, stream);
  return ANODE_E_LAUNCH;
}

int check_dims(uint32_t dim0, uint32_t dim1, uint32_t dim2)
{
  if (dim0 == 0 || dim1 == 0 || dim2 == 0) return ANODE_E_DIMS;
  const unsigned __int128 len = (unsigned __int128)dim0 * dim1 * dim2;
  if (len >= ((unsigned __int128)1 << 32)) return ANODE_E_DIMS;
  return ANODE_OK;
}

typedef void (*PipelineKernel)(const FusedArgs);

static PipelineKernel pick_kernel(const Plan &p, int dir)
{
  if (p.regime == 1) return dir == 0 ? bn_pipeline_kernel<4, 0, 1> : bn_pipeline_kernel<4, 1, 1>;
  if (p.vec == 4) return dir == 0 ? bn_pipeline_kernel<4, 0, 0> : bn_pipeline_kernel<4, 1, 0>;
  return dir == 0 ? bn_pipeline_kernel<1, 0, 0> : bn_pipeline_kernel<1, 1, 0>;
}

// Blocks of `k` that fit on one SM (cached per kernel; same answer on every B200).
static uint32_t blocks_per_sm(PipelineKernel k)
{
  static std::mutex mu;
  static std::map<const void *, int> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find((const void *)k);
  if (it != cache.end()) return (uint32_t)it->second;
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k, (int)kThreads, 0) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
  cache[(const void *)k] = n;
  return (uint32_t)n;
}

int launch_pipeline(FusedArgs &a, int dir, cudaStream_t stream)
{
  PipelineKernel k = pick_kernel(a.plan, dir);
  const uint32_t fit = blocks_per_sm(k) * sm_count();
  if (fit == 0) return ANODE_E_LAUNCH;
  if (a.plan.grid > fit) {
    // fewer blocks are resident than planned: shrink the grid and re-derive the lookahead
    a.plan.grid = fit;
    a.plan.lookahead_steps = ceil_div_u32(a.plan.tiles_per_unit, a.plan.grid) + 1;
  }
  void *params[] = {(void *)&a};
  cudaError_t e;
  if (a.mode == MODE_FUSED) {
    // Blocks wait on one another's results, so all of them must be resident: a cooperative
    // launch fails instead of deadlocking when they would not be.
    e = cudaLaunchCooperativeKernel((const void *)k, dim3(a.plan.grid), dim3(kThreads), params, 0, stream);
  } else {
    e = cudaLaunchKernel((const void *)k, dim3(a.plan.grid), dim3(kThreads), params, 0, stream);
  }
  if (e != cudaSuccess) { (void)cudaGetLastError(); return ANODE_E_LAUNCH; }
  return ANODE_OK;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool aligned4(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

int prepare_fwd(FusedArgs &a, uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate,
                int relu, const float *x, const float *gamma, const float *beta, float *y, float *mean,
                float *var, float *run_mean, float *run_var, void *ws, size_t ws_bytes)
{
  const int rc = check_dims(dim0, dim1, dim2);
  if (rc) return rc;
  if (!x || !y || !mean || !var) return ANODE_E_NULL;
  if (!aligned4(x) || !aligned4(y)) return ANODE_E_ALIGN;
  if (!ws || !aligned16(ws)) return ANODE_E_WORKSPACE;
  a = FusedArgs{};
  a.plan = plan_for(dim0, dim1, dim2, aligned16(x) && aligned16(y));
  const uint64_t part = workspace_part_bytes(dim0, dim1, dim2);
  if (ws_bytes < part) return ANODE_E_WORKSPACE;              // forward uses the first part only
  a.ws_capacity = part;
  a.status = static_cast<uint32_t *>(ws);
  a.x = x; a.gamma = gamma; a.beta = beta; a.out = y;
  a.mean = mean; a.var = var; a.run_mean = run_mean; a.run_var = run_var;
  a.ws = static_cast<unsigned char *>(ws);
  a.epsilon = epsilon; a.avg_rate = avg_rate; a.relu = relu ? 1u : 0u; a.neg_slope = relu ? 0.0f : 1.0f;
  a.mode = MODE_FUSED;
  a.count_total = (double)dim0 * (double)dim2;
  a.wait_cycles = wait_limit_cycles();
  return ANODE_OK;
}

int prepare_bwd(FusedArgs &a, uint32_t dim0, uint32_t dim1, uint32_t dim2, int relu, int accumulate,
                const float *dy, const float *x, const float *mean, const float *var, const float *gamma,
                const float *beta, float *dx, float *dgamma, float *dbeta, void *ws, size_t ws_bytes)
{
  const int rc = check_dims(dim0, dim1, dim2);
  if (rc) return rc;
  if (!x || !dy || !dx || !mean || !var) return ANODE_E_NULL;
  if (!aligned4(x) || !aligned4(dy) || !aligned4(dx)) return ANODE_E_ALIGN;
  if (!ws || !aligned16(ws)) return ANODE_E_WORKSPACE;
  a = FusedArgs{};
  a.plan = plan_for(dim0, dim1, dim2, aligned16(x) && aligned16(dy) && aligned16(dx));
  const uint64_t part = workspace_part_bytes(dim0, dim1, dim2);
  if (ws_bytes < 2 * part) return ANODE_E_WORKSPACE;
  a.ws_capacity = part;
  a.status = static_cast<uint32_t *>(ws);
  a.x = x; a.dy = dy; a.gamma = gamma; a.beta = beta; a.mean_in = mean; a.var_in = var;
  a.out = dx; a.dgamma = dgamma; a.dbeta = dbeta;
  a.ws = static_cast<unsigned char *>(ws) + part;              // the backward part
  a.relu = relu ? 1u : 0u; a.neg_slope = relu ? 0.0f : 1.0f; a.accumulate = accumulate ? 1u : 0u;
  a.mode = MODE_FUSED;
  a.count_total = (double)dim0 * (double)dim2;
  a.wait_cycles = wait_limit_cycles();
  return ANODE_OK;
}

__global__ void online_average_kernel(uint32_t len, float rate, const float *x, float *y)
{
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < len; i += gridDim.x * blockDim.x) {
    const float o = y[i];
    y[i] = o + rate * (x[i] - o);
  }
}

}  // namespace anode_b200

using namespace anode_b200;

extern "C" size_t anode_gpu_batch_norm_fused_workspace_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2)
{
  if (check_dims(dim0, dim1, dim2)) return 0;
  return (size_t)(2 * workspace_part_bytes(dim0, dim1, dim2));
}

extern "C" int anode_gpu_batch_norm_fused_workspace_init(void *workspace, size_t bytes, struct CUstream_st *stream)
{
  if (!workspace) return ANODE_E_NULL;
  if (cudaMemsetAsync(workspace, 0, bytes, stream) != cudaSuccess) { (void)cudaGetLastError(); return ANODE_E_LAUNCH; }
  return ANODE_OK;
}

extern "C" int anode_gpu_batch_norm_fused_status(const void *workspace, struct CUstream_st *stream, uint32_t *status)
{
  if (!workspace || !status) return ANODE_E_NULL;
  if (cudaMemcpyAsync(status, workspace, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess) {
    (void)cudaGetLastError();
    return ANODE_E_LAUNCH;
  }
  return ANODE_OK;
}

extern "C" int anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, int relu,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    void *workspace, size_t workspace_bytes, const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  FusedArgs a;
  const int rc = prepare_fwd(a, dim0, dim1, dim2, epsilon, avg_rate, relu, x, gamma, beta, y, mean, var,
                             run_mean, run_var, workspace, workspace_bytes);
  if (rc) return rc;
  if (workspace_bytes < anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2)) return ANODE_E_WORKSPACE;
  return launch_best(a, 0, aligned16(x) && aligned16(y), stream);
}

extern "C" int anode_gpu_batch_norm_relu_fused_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, int relu, int accumulate,
    const float *dy, const float *x, const float *mean, const float *var,
    const float *gamma, const float *beta, float *dx, float *dgamma, float *dbeta,
    void *workspace, size_t workspace_bytes, const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  FusedArgs a;
  const int rc = prepare_bwd(a, dim0, dim1, dim2, relu, accumulate, dy, x, mean, var, gamma, beta, dx,
                             dgamma, dbeta, workspace, workspace_bytes);
  if (rc) return rc;
  return launch_best(a, 1, aligned16(x) && aligned16(dy) && aligned16(dx), stream);
}

// The two calls above with a general activation t*(t > 0 ? 1 : neg_slope) instead of the ReLU switch.
extern "C" int anode_gpu_batch_norm_act_fused_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, float neg_slope,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    void *workspace, size_t workspace_bytes, const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  FusedArgs a;
  const int rc = prepare_fwd(a, dim0, dim1, dim2, epsilon, avg_rate, 1, x, gamma, beta, y, mean, var,
                             run_mean, run_var, workspace, workspace_bytes);
  if (rc) return rc;
  if (workspace_bytes < anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2)) return ANODE_E_WORKSPACE;
  a.neg_slope = neg_slope;
  return launch_best(a, 0, aligned16(x) && aligned16(y), stream);
}

extern "C" int anode_gpu_batch_norm_act_fused_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float neg_slope, int accumulate,
    const float *dy, const float *x, const float *mean, const float *var,
    const float *gamma, const float *beta, float *dx, float *dgamma, float *dbeta,
    void *workspace, size_t workspace_bytes, const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  FusedArgs a;
  const int rc = prepare_bwd(a, dim0, dim1, dim2, 1, accumulate, dy, x, mean, var, gamma, beta, dx,
                             dgamma, dbeta, workspace, workspace_bytes);
  if (rc) return rc;
  a.neg_slope = neg_slope;
  return launch_best(a, 1, aligned16(x) && aligned16(dy) && aligned16(dx), stream);
}

// Residual block epilogue: y = act(bn(x) + residual), the step after batch-norm in every residual
// block (examples/run_imagenet_mpi.rs:191-195, 224-226: sum of the shortcut and the normalized
// branch, then positive_clip).  Backward: the mask comes from the saved output y (as the reference's
// positive_clip adjoint takes it, flat_map.cu:187-194), dresidual = dy*mask is the gradient of the
// shortcut (the sum's adjoint fans dz out to both inputs), dx / dgamma / dbeta as before.
extern "C" int anode_gpu_batch_norm_add_act_fused_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, float neg_slope,
    const float *x, const float *residual, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    void *workspace, size_t workspace_bytes, const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!residual) return ANODE_E_NULL;
  if (!aligned4(residual)) return ANODE_E_ALIGN;
  FusedArgs a;
  const int rc = prepare_fwd(a, dim0, dim1, dim2, epsilon, avg_rate, 1, x, gamma, beta, y, mean, var,
                             run_mean, run_var, workspace, workspace_bytes);
  if (rc) return rc;
  if (workspace_bytes < anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2)) return ANODE_E_WORKSPACE;
  a.neg_slope = neg_slope;
  a.res = residual;
  if (!aligned16(residual)) a.plan = plan_for(dim0, dim1, dim2, false);      // scalar path
  return launch_best(a, 0, aligned16(x) && aligned16(y) && aligned16(residual), stream);
}

extern "C" int anode_gpu_batch_norm_add_act_fused_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float neg_slope, int accumulate,
    const float *dy, const float *x, const float *y, const float *mean, const float *var,
    const float *gamma, const float *beta, float *dx, float *dresidual, float *dgamma, float *dbeta,
    void *workspace, size_t workspace_bytes, const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!y) return ANODE_E_NULL;
  if (!aligned4(y) || (dresidual && !aligned4(dresidual))) return ANODE_E_ALIGN;
  FusedArgs a;
  const int rc = prepare_bwd(a, dim0, dim1, dim2, 1, accumulate, dy, x, mean, var, gamma, beta, dx,
                             dgamma, dbeta, workspace, workspace_bytes);
  if (rc) return rc;
  a.neg_slope = neg_slope;
  a.ymask = y; a.dres = dresidual;
  const bool al = aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(y) && (!dresidual || aligned16(dresidual));
  if (!al) a.plan = plan_for(dim0, dim1, dim2, false);
  return launch_best(a, 1, al, stream);
}

extern "C" int anode_gpu_online_average_f32(uint32_t len, float rate, const float *x, float *y,
                                            const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!x || !y) return ANODE_E_NULL;
  if (len == 0) return ANODE_OK;
  const uint32_t blocks = (len + 255) / 256 < 1184 ? (len + 255) / 256 : 1184;
  online_average_kernel<<<blocks, 256, 0, stream>>>(len, rate, x, y);
  if (cudaGetLastError() != cudaSuccess) return ANODE_E_LAUNCH;
  return ANODE_OK;
}

// Which kernel serves direction `dir` of a plain [dim0, dim1, dim2] call with 16-byte aligned tensors on
// one GPU: an ANODE_KERNEL_* value.
extern "C" int anode_gpu_batch_norm_fused_kernel_kind(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir)
{
  if (check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  FusedArgs a{};
  a.plan = plan_for(dim0, dim1, dim2, true);
  a.mode = MODE_FUSED;
  a.ws_capacity = workspace_part_bytes(dim0, dim1, dim2);
  return pick_kernel_kind(a, dir, true);
}

// The same for the residual-epilogue calls (anode_gpu_batch_norm_add_act_fused_*).
extern "C" int anode_gpu_batch_norm_add_act_fused_kernel_kind(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir)
{
  if (check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  static const float dummy = 0.f;
  FusedArgs a{};
  a.plan = plan_for(dim0, dim1, dim2, true);
  a.mode = MODE_FUSED;
  a.ws_capacity = workspace_part_bytes(dim0, dim1, dim2);
  if (dir == 0) a.res = &dummy; else a.ymask = &dummy;       // only their presence matters here
  return pick_kernel_kind(a, dir, true);
}

extern "C" int anode_gpu_batch_norm_fused_set_kernel(int kernel)
{
  if (kernel < ANODE_KERNEL_AUTO || kernel > ANODE_KERNEL_PLAIN) return ANODE_E_DIMS;
  g_kernel_choice.store(kernel, std::memory_order_relaxed);
  return ANODE_OK;
}

// ---- diagnostics: geometry of the tiled kernel for a shape (no GPU needed) ----------------------
// out (12 values): applies, rows per tile, floats per row piece, tiles per unit, slots, bytes per slot, dynamic
// shared memory bytes, KiB between a tile's two visits, the fraction (in 1/1000) of that window loaded with the
// "keep" priority, blocks, steps between a tile's two visits, tiles
extern "C" int anode_gpu_batch_norm_tiled_geometry(uint32_t dim0, uint32_t dim1, uint32_t dim2, int dir, uint32_t *out)
{
  using namespace anode_b200;
  if (!out || (dir != 0 && dir != 1) || check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  Plan p; RingGeom g;
  for (int i = 0; i < 12; ++i) out[i] = 0;
  if (!ring_plan_for(dim0, dim1, dim2, true, dir, p, g)) return ANODE_OK;
  const uint64_t window = ring_window_bytes(p, dir);
  out[0] = 1; out[1] = p.rows_per_tile; out[2] = p.piece_len; out[3] = p.tiles_per_unit; out[4] = g.slots;
  out[5] = g.slot_stride; out[6] = g.smem_bytes; out[7] = (uint32_t)(window >> 10);
  out[8] = window > kRingLargeWindowMax ? (uint32_t)(1000.0 * (double)kRingLargeWindowMax / (double)window) : 1000u;
  out[9] = p.grid; out[10] = p.lookahead_steps; out[11] = p.total_tiles;
  return ANODE_OK;
}

// ---- diagnostics: the tile plan, for tests of the index arithmetic (no GPU needed) ----------
extern "C" int anode_gpu_batch_norm_fused_plan(uint32_t dim0, uint32_t dim1, uint32_t dim2, int aligned,
                                               uint32_t resident_blocks, uint32_t tile_floats,
                                               uint32_t slack_steps, uint32_t *out, uint32_t out_len)
{
  if (!out || check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  const Tunables &t = tunables();
  const Plan p = make_plan(dim0, dim1, dim2, aligned != 0,
                           resident_blocks ? resident_blocks : sm_count() * t.blocks_per_sm,
                           tile_floats ? tile_floats : t.tile_floats, slack_steps ? slack_steps : t.slack_steps);
  const uint32_t v[] = {p.regime, p.vec, p.cb, p.units, p.rows_per_tile, p.piece_len, p.pieces,
                        p.sample_blocks, p.tiles_per_unit, p.total_tiles, p.grid, p.lookahead_steps,
                        p.div_mul, (uint32_t)(p.ws_bytes & 0xffffffffu), (uint32_t)(p.ws_bytes >> 32)};
  for (uint32_t i = 0; i < out_len && i < sizeof(v) / sizeof(v[0]); ++i) out[i] = v[i];
  return ANODE_OK;
}

extern "C" int anode_gpu_batch_norm_fused_plan_tile(uint32_t dim0, uint32_t dim1, uint32_t dim2, int aligned,
                                                    uint32_t resident_blocks, uint32_t tile_floats,
                                                    uint32_t tile, uint64_t *out)
{
  if (!out || check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  const Tunables &t = tunables();
  const Plan p = make_plan(dim0, dim1, dim2, aligned != 0,
                           resident_blocks ? resident_blocks : sm_count() * t.blocks_per_sm,
                           tile_floats ? tile_floats : t.tile_floats, t.slack_steps);
  if (tile >= p.total_tiles) return ANODE_E_DIMS;
  const TileRange r = tile_range(p, tile);
  out[0] = r.unit; out[1] = r.c0; out[2] = r.cw; out[3] = r.n0; out[4] = r.rows; out[5] = r.col0;
  out[6] = r.len; out[7] = r.base;
  return ANODE_OK;
}

// Walks `count` tiles first, first+stride, ... with the division-free iterator the kernels use.
// out: 8 values per tile as in anode_gpu_batch_norm_fused_plan_tile.
extern "C" int anode_gpu_batch_norm_fused_plan_walk(uint32_t dim0, uint32_t dim1, uint32_t dim2, int aligned,
                                                    uint32_t resident_blocks, uint32_t tile_floats,
                                                    uint32_t first, uint32_t stride, uint32_t count, uint64_t *out)
{
  if (!out || check_dims(dim0, dim1, dim2) || stride == 0) return ANODE_E_DIMS;
  const Tunables &t = tunables();
  const Plan p = make_plan(dim0, dim1, dim2, aligned != 0,
                           resident_blocks ? resident_blocks : sm_count() * t.blocks_per_sm,
                           tile_floats ? tile_floats : t.tile_floats, t.slack_steps);
  TileIter it; it.init(p, first, stride);
  for (uint32_t i = 0; i < count; ++i) {
    if (it.tile() >= p.total_tiles) return ANODE_E_DIMS;
    const TileRange r = it.range(p);
    uint64_t *o = out + 8 * (size_t)i;
    o[0] = r.unit; o[1] = r.c0; o[2] = r.cw; o[3] = r.n0; o[4] = r.rows; o[5] = r.col0; o[6] = r.len; o[7] = r.base;
    it.advance(p);
  }
  return ANODE_OK;
}
