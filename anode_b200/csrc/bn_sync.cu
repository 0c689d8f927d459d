// Synchronized batch-norm across the GPUs of one node: every rank holds a shard of the batch
// (or a spatial slab) with all C channels, runs the local reduce pass, exchanges 16 bytes per
// channel, and applies with the global statistics.
//
// The reference has no such path: its batch-norm is per process and its only collective is a
// host-staged MPI allreduce of gradients (src/proc_mpi.rs:138-148, src/ops_gpu.rs:538-545).
// Parity definition: G-way result == the single-device kernels run on the concatenated batch.
//
// Exchange through NCCL: all-gather of the local (count, mean, M2) resp. (sum dz, sum dz*(x-mean))
// records, then every rank merges the G records of a channel in rank order in double precision,
// so all ranks obtain bit-identical statistics.  NCCL is resolved at run time (dlopen of the
// copy already loaded in the process, e.g. the one PyTorch ships), never linked.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "bn_host.h"
#include "bn_sync.h"

namespace anode_b200 {

// ---- NCCL entry points, looked up once ----------------------------------------------------
struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId *);
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  const char *(*GetErrorString)(ncclResult_t);
  bool ok;
};

static const NcclApi &nccl()
{
  static NcclApi api = [] {
    NcclApi a{};
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);     // the copy already in the process
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW);
    if (!h) return a;
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(h, "ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(h, "ncclCommDestroy");
    a.AllGather = (decltype(a.AllGather))dlsym(h, "ncclAllGather");
    a.AllReduce = (decltype(a.AllReduce))dlsym(h, "ncclAllReduce");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(h, "ncclGetErrorString");
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllGather && a.AllReduce;
    return a;
  }();
  return api;
}

// ---- merge kernels: G records per channel -> global statistics and coefficients ---------------
// gathered: [world][C] float4; the first word of a forward record is the element count as an integer.
// One thread per channel; every rank computes the same thing.
__global__ void sync_merge_fwd_kernel(FusedArgs a, const float4 *gathered, uint32_t world)
{
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.plan.C) return;
  double sn = 0.0, sm = 0.0;
  for (uint32_t r = 0; r < world; ++r) {
    const float4 p = gathered[(size_t)r * a.plan.C + c];
    const double n = (double)__float_as_uint(p.x);
    sn += n; sm += n * (double)p.y;
  }
  const double mean = sm / sn;
  double sq = 0.0;
  for (uint32_t r = 0; r < world; ++r) {
    const float4 p = gathered[(size_t)r * a.plan.C + c];
    const double d = (double)p.y - mean;
    sq += (double)p.z + (double)__float_as_uint(p.x) * d * d;
  }
  a.mode = MODE_APPLY;          // makes finish_channel_fwd write outputs and coefficients
  a.use_rec = 0;
  finish_channel_fwd(a, c, sn, mean, sq);
}

__global__ void sync_merge_bwd_kernel(FusedArgs a, const float4 *gathered, uint32_t world)
{
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.plan.C) return;
  double s1 = 0.0, s2 = 0.0;
  for (uint32_t r = 0; r < world; ++r) {
    const float4 p = gathered[(size_t)r * a.plan.C + c];
    s1 += (double)p.x; s2 += (double)p.y;
  }
  a.mode = MODE_APPLY;
  a.use_rec = 0;
  finish_channel_bwd(a, c, s1, s2);
}

// The exchange of the one-kernel form as a kernel of its own, for shapes none of the kernels with a
// built-in exchange takes (scalar paths): same records, same buffers, same sequence numbers, so ranks
// may mix the two forms freely.  One thread per channel: ship this GPU's record to every rank, collect
// the ranks' records from this GPU's own buffer (bounded wait), merge in rank order.
template <int DIR>
__global__ void sync_exchange_kernel(FusedArgs a, const float4 *local)
{
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.plan.C) return;
  const float4 mine = __ldcg(local + c);
  const size_t slot = ((((size_t)(a.epoch & 1u)) * a.world) * a.xchg_channels + c) * 4;
  const size_t src_stride = (size_t)a.xchg_channels * 4;
  const unsigned long long e = (unsigned long long)a.epoch << 32;
  for (uint32_t r = 0; r < a.world; ++r) {
    unsigned long long *dst = a.xchg[r] + slot + a.rank * src_stride;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + 0), "l"(e | __float_as_uint(mine.x)) : "memory");
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + 1), "l"(e | __float_as_uint(mine.y)) : "memory");
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + 2), "l"(e | __float_as_uint(mine.z)) : "memory");
  }
  double n[8], m[8], q[8];
  const long long t0 = clock64();
  for (uint32_t r = 0; r < a.world; ++r) {
    const unsigned long long *src = a.xchg[a.rank] + slot + r * src_stride;
    unsigned long long v0, v1, v2;
    for (;;) {
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v0) : "l"(src + 0) : "memory");
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v1) : "l"(src + 1) : "memory");
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v2) : "l"(src + 2) : "memory");
      if ((uint32_t)(v0 >> 32) == a.epoch && (uint32_t)(v1 >> 32) == a.epoch && (uint32_t)(v2 >> 32) == a.epoch) break;
      if (clock64() - t0 > a.wait_cycles) { atomicOr(a.status, ANODE_ST_WAIT_PEER | ANODE_ST_ABORTED); return; }   // leave a mark, publish nothing
      __nanosleep(200);
    }
    n[r] = DIR == 0 ? (double)(uint32_t)v0 : (double)__uint_as_float((uint32_t)v0);
    m[r] = (double)__uint_as_float((uint32_t)v1);
    q[r] = (double)__uint_as_float((uint32_t)v2);
  }
  a.mode = MODE_APPLY;
  a.use_rec = 0;
  if (DIR == 0) {
    double sn = 0.0, sm = 0.0, sq = 0.0;
    for (uint32_t r = 0; r < a.world; ++r) { sn += n[r]; sm += n[r] * m[r]; }
    const double mean = sm / sn;
    for (uint32_t r = 0; r < a.world; ++r) { const double d = m[r] - mean; sq += q[r] + n[r] * d * d; }
    finish_channel_fwd(a, c, sn, mean, sq);
  } else {
    double s1 = 0.0, s2 = 0.0;
    for (uint32_t r = 0; r < a.world; ++r) { s1 += n[r]; s2 += m[r]; }
    finish_channel_bwd(a, c, s1, s2);
  }
}

static size_t gather_bytes(uint32_t C, uint32_t world) { return (size_t)align_up_u64((uint64_t)16 * C * world, 256); }

// True when a kernel with the exchange built in serves this call.
static bool fused_exchange_applies(const FusedArgs &a, int dir, bool aligned)
{
  FusedArgs probe = a;
  probe.mode = MODE_FUSED;
  const int kind = pick_kernel_kind(probe, dir, aligned);
  return kind == ANODE_KERNEL_TILED || kind == ANODE_KERNEL_CLUSTER || kind == ANODE_KERNEL_RESIDENT;
}

static int run_sync(FusedArgs &a, int dir, bool aligned, AnodeSyncComm *comm, size_t fused_ws_bytes, cudaStream_t stream)
{
  const NcclApi &api = nccl();
  if (!comm) return ANODE_E_COMM;
  if (comm->world == 1) {
    // nothing to exchange: the one-GPU launch
    a.mode = MODE_FUSED;
    return launch_best(a, dir, aligned, stream);
  }
  const bool exchange = comm->xchg_channels != 0;
  // Which protocol carries the records is a property of the communicator, never of this rank's shard:
  // once an exchange buffer is attached every rank uses it (a rank that fell back to NCCL on its own
  // would enqueue a collective nobody else joins).
  if (exchange && comm->xchg_channels < a.plan.C) return ANODE_E_COMM;
  if (exchange) {
    a.rank = (uint32_t)comm->rank; a.world = (uint32_t)comm->world;
    a.xchg_channels = comm->xchg_channels;
    a.epoch = comm->epoch + 1;
    for (int r = 0; r < comm->world; ++r) a.xchg[r] = comm->xchg[r];
    int rc;
    if (fused_exchange_applies(a, dir, aligned)) {
      // One kernel per direction: the block that owns a channel stores this GPU's record into every
      // rank's exchange buffer (plain peer stores over NVLink), every block reads the records of all
      // ranks from its own GPU's buffer.  No collective call, no extra launches.
      a.mode = MODE_FUSED;
      rc = launch_best(a, dir, aligned, stream);
    } else {
      // reduce kernel, exchange kernel, apply kernel
      const Plan base = a.plan;
      const uint32_t world = a.world;
      a.mode = MODE_STATS; a.world = 1;
      rc = launch_best(a, dir, aligned, stream);
      if (rc == ANODE_OK) {
        const float4 *local = reinterpret_cast<const float4 *>(a.ws + a.plan.off_local);
        FusedArgs m = a;
        m.world = world;
        const uint32_t threads = 128, blocks = (a.plan.C + threads - 1) / threads;
        if (dir == 0) sync_exchange_kernel<0><<<blocks, threads, 0, stream>>>(m, local);
        else sync_exchange_kernel<1><<<blocks, threads, 0, stream>>>(m, local);
        if (cudaGetLastError() != cudaSuccess) rc = ANODE_E_LAUNCH;
      }
      if (rc == ANODE_OK) {
        a.plan = base;
        a.mode = MODE_APPLY;
        rc = launch_best(a, dir, aligned, stream);
      }
    }
    // the sequence number advances only when this rank really took part
    if (rc == ANODE_OK) comm->epoch = a.epoch;
    return rc;
  }
  if (!api.ok || !comm->nccl) return ANODE_E_COMM;
  // the gather buffer sits behind the single-GPU workspace
  float4 *gathered = reinterpret_cast<float4 *>(reinterpret_cast<unsigned char *>(a.status) + fused_ws_bytes);
  const Plan base = a.plan;
  a.mode = MODE_STATS;
  int rc = launch_best(a, dir, aligned, stream);
  if (rc) return rc;
  const float4 *local = reinterpret_cast<const float4 *>(a.ws + a.plan.off_local);
  if (api.AllGather(local, gathered, (size_t)4 * a.plan.C, ncclFloat, comm->nccl, stream) != ncclSuccess) return ANODE_E_COMM;
  FusedArgs m = a;
  const uint32_t threads = 128, blocks = (a.plan.C + threads - 1) / threads;
  if (dir == 0) sync_merge_fwd_kernel<<<blocks, threads, 0, stream>>>(m, gathered, (uint32_t)comm->world);
  else sync_merge_bwd_kernel<<<blocks, threads, 0, stream>>>(m, gathered, (uint32_t)comm->world);
  if (cudaGetLastError() != cudaSuccess) return ANODE_E_LAUNCH;
  a.plan = base;
  a.mode = MODE_APPLY;
  return launch_best(a, dir, aligned, stream);
}

// What the host-buffer step (bn_hoststep.cu) needs of this file.
int sync_launch(FusedArgs &a, int dir, bool aligned, AnodeSyncComm *comm, size_t fused_ws_bytes, cudaStream_t stream)
{
  return run_sync(a, dir, aligned, comm, fused_ws_bytes, stream);
}
size_t sync_gather_bytes(uint32_t C, const AnodeSyncComm *comm) { return comm ? gather_bytes(C, (uint32_t)comm->world) : 0; }
int sync_world(const AnodeSyncComm *comm) { return comm ? comm->world : 1; }

}  // namespace anode_b200

using namespace anode_b200;

extern "C" size_t anode_gpu_sync_unique_id_bytes(void) { return sizeof(ncclUniqueId); }

extern "C" int anode_gpu_sync_get_unique_id(void *out)
{
  const NcclApi &api = nccl();
  if (!out) return ANODE_E_NULL;
  if (!api.ok) return ANODE_E_COMM;
  ncclUniqueId id;
  if (api.GetUniqueId(&id) != ncclSuccess) return ANODE_E_COMM;
  memcpy(out, &id, sizeof(id));
  return ANODE_OK;
}

extern "C" int anode_gpu_sync_comm_create(const void *unique_id, int rank, int world, struct AnodeSyncComm **out)
{
  const NcclApi &api = nccl();
  if (!unique_id || !out) return ANODE_E_NULL;
  if (!api.ok || world < 1 || rank < 0 || rank >= world) return ANODE_E_COMM;
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  AnodeSyncComm *c = new AnodeSyncComm{};
  c->rank = rank; c->world = world;
  if (api.CommInitRank(&c->nccl, world, id, rank) != ncclSuccess) { delete c; return ANODE_E_COMM; }
  *out = c;
  return ANODE_OK;
}

// A communicator without NCCL: the records travel through an attached exchange buffer only (callers
// that set up peer-mapped memory themselves and want no second communication library in the process).
// Synchronized calls on it fail with ANODE_E_COMM until an exchange buffer is attached.
extern "C" int anode_gpu_sync_comm_create_exchange_only(int rank, int world, struct AnodeSyncComm **out)
{
  if (!out) return ANODE_E_NULL;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return ANODE_E_COMM;
  AnodeSyncComm *c = new AnodeSyncComm{};
  c->rank = rank; c->world = world;
  *out = c;
  return ANODE_OK;
}

extern "C" size_t anode_gpu_sync_exchange_bytes(uint32_t max_channels, int world)
{
  if (max_channels == 0 || world < 1 || world > 8) return 0;
  return (size_t)2 * (size_t)world * max_channels * 4 * sizeof(unsigned long long);    // [buffer][source rank][channel][word]
}

extern "C" int anode_gpu_sync_comm_attach_exchange(struct AnodeSyncComm *comm, void *const *peer_ptrs, uint32_t max_channels)
{
  if (!comm || !peer_ptrs) return ANODE_E_NULL;
  if (comm->world > 8 || max_channels == 0) return ANODE_E_COMM;
  for (int r = 0; r < comm->world; ++r) {
    if (!peer_ptrs[r] || (reinterpret_cast<uintptr_t>(peer_ptrs[r]) & 7u)) return ANODE_E_COMM;
    comm->xchg[r] = static_cast<unsigned long long *>(peer_ptrs[r]);
  }
  comm->xchg_channels = max_channels;
  comm->epoch = 0;
  return ANODE_OK;
}

// Sum of a device buffer over the ranks of `comm`, in place, on `stream`: what SumSpmdOp does for
// gradients through a host-staged MPI_Allreduce (src/ops_gpu.rs:538-545, src/proc_mpi.rs:138-148),
// here over NVLink without leaving the device.
extern "C" int anode_gpu_sync_allreduce_sum_f32(struct AnodeSyncComm *comm, float *buf, size_t len, struct CUstream_st *stream)
{
  if (!comm) return ANODE_E_COMM;
  if (!buf && len) return ANODE_E_NULL;
  if (len == 0 || comm->world == 1) return ANODE_OK;
  const NcclApi &api = nccl();
  if (!api.ok || !comm->nccl) return ANODE_E_COMM;
  if (api.AllReduce(buf, buf, len, ncclFloat, ncclSum, comm->nccl, stream) != ncclSuccess) return ANODE_E_COMM;
  return ANODE_OK;
}

extern "C" int anode_gpu_sync_comm_destroy(struct AnodeSyncComm *comm)
{
  if (!comm) return ANODE_E_NULL;
  const NcclApi &api = nccl();
  if (api.ok && comm->nccl) api.CommDestroy(comm->nccl);
  delete comm;
  return ANODE_OK;
}

extern "C" size_t anode_gpu_sync_batch_norm_workspace_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2, int world)
{
  const size_t base = anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2);
  if (base == 0 || world < 1) return 0;
  return base + gather_bytes(dim1, (uint32_t)world);
}

extern "C" int anode_gpu_sync_batch_norm_relu_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, int relu,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!comm) return ANODE_E_COMM;
  const size_t fused = anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2);
  if (fused == 0) return ANODE_E_DIMS;
  if (workspace_bytes < fused + gather_bytes(dim1, (uint32_t)comm->world)) return ANODE_E_WORKSPACE;
  FusedArgs a;
  const int rc = prepare_fwd(a, dim0, dim1, dim2, epsilon, avg_rate, relu, x, gamma, beta, y, mean, var,
                             run_mean, run_var, workspace, fused);
  if (rc) return rc;
  return run_sync(a, 0, aligned16(x) && aligned16(y), comm, fused, stream);
}

extern "C" int anode_gpu_sync_batch_norm_relu_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count, int relu, int accumulate,
    const float *dy, const float *x, const float *mean, const float *var,
    const float *gamma, const float *beta, float *dx, float *dgamma, float *dbeta,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!comm) return ANODE_E_COMM;
  const size_t fused = anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2);
  if (fused == 0 || global_count < (uint64_t)dim0 * dim2) return ANODE_E_DIMS;
  if (workspace_bytes < fused + gather_bytes(dim1, (uint32_t)comm->world)) return ANODE_E_WORKSPACE;
  FusedArgs a;
  const int rc = prepare_bwd(a, dim0, dim1, dim2, relu, accumulate, dy, x, mean, var, gamma, beta, dx,
                             dgamma, dbeta, workspace, fused);
  if (rc) return rc;
  a.count_total = (double)global_count;
  return run_sync(a, 1, aligned16(x) && aligned16(dy) && aligned16(dx), comm, fused, stream);
}

// Residual-block epilogue across GPUs: anode_gpu_batch_norm_add_act_fused_{fwd,bwd}_3d1_packed_f32 with the
// statistics and the backward sums taken over all ranks' shards.
extern "C" int anode_gpu_sync_batch_norm_add_act_fwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, float neg_slope,
    const float *x, const float *residual, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!comm) return ANODE_E_COMM;
  if (!residual) return ANODE_E_NULL;
  if (!aligned4(residual)) return ANODE_E_ALIGN;
  const size_t fused = anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2);
  if (fused == 0) return ANODE_E_DIMS;
  if (workspace_bytes < fused + gather_bytes(dim1, (uint32_t)comm->world)) return ANODE_E_WORKSPACE;
  FusedArgs a;
  const int rc = prepare_fwd(a, dim0, dim1, dim2, epsilon, avg_rate, 1, x, gamma, beta, y, mean, var,
                             run_mean, run_var, workspace, fused);
  if (rc) return rc;
  a.neg_slope = neg_slope;
  a.res = residual;
  const bool al = aligned16(x) && aligned16(y) && aligned16(residual);
  if (!al) a.plan = plan_for(dim0, dim1, dim2, false);
  return run_sync(a, 0, al, comm, fused, stream);
}

extern "C" int anode_gpu_sync_batch_norm_add_act_bwd_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count, float neg_slope, int accumulate,
    const float *dy, const float *x, const float *y, const float *mean, const float *var,
    const float *gamma, const float *beta, float *dx, float *dresidual, float *dgamma, float *dbeta,
    struct AnodeSyncComm *comm, void *workspace, size_t workspace_bytes,
    const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!comm) return ANODE_E_COMM;
  if (!y) return ANODE_E_NULL;
  if (!aligned4(y) || (dresidual && !aligned4(dresidual))) return ANODE_E_ALIGN;
  const size_t fused = anode_gpu_batch_norm_fused_workspace_bytes(dim0, dim1, dim2);
  if (fused == 0 || global_count < (uint64_t)dim0 * dim2) return ANODE_E_DIMS;
  if (workspace_bytes < fused + gather_bytes(dim1, (uint32_t)comm->world)) return ANODE_E_WORKSPACE;
  FusedArgs a;
  const int rc = prepare_bwd(a, dim0, dim1, dim2, 1, accumulate, dy, x, mean, var, gamma, beta, dx,
                             dgamma, dbeta, workspace, fused);
  if (rc) return rc;
  a.neg_slope = neg_slope;
  a.ymask = y; a.dres = dresidual;
  a.count_total = (double)global_count;
  const bool al = aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(y) && (!dresidual || aligned16(dresidual));
  if (!al) a.plan = plan_for(dim0, dim1, dim2, false);
  return run_sync(a, 1, al, comm, fused, stream);
}
