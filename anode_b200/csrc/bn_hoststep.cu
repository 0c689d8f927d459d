// Fused forward + backward of one layer whose tensors live in host memory.
//
// anode keeps activations in device arrays, but what a training script hands to a layer starts in
// host memory (MemArray4d, e.g. tests/test_gpu.rs:138-139, the data loader of
// examples/run_imagenet_mpi.rs:310-417).  For callers on that side of the boundary the cost of a
// layer is the PCIe transfer, not the kernels, so this entry point overlaps the two directions of
// the link: channels are independent in batch-norm, so the layer is cut into blocks of channels and
// block k+1 travels to the device while block k is computed and block k-1 travels back.
//
// Streams: the kernels run on the caller's stream; host->device and device->host copies run on two
// streams owned by the library (created on first use, one pair per device), ordered against the
// caller's stream with events.  When the call returns everything is enqueued and the caller's
// stream waits for the last copy, so "synchronise the stream" means "the results are in host
// memory".  Host buffers should be page-locked; with pageable memory the copies still give the
// right result but do not overlap.
#include "bn_host.h"

namespace anode_b200 {

constexpr int kStageBufs = 3;

struct HostPipe {
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, in_done[kStageBufs] = {}, k_done[kStageBufs] = {}, out_done[kStageBufs] = {};
  bool ok = false;
};

static std::mutex g_pipe_mu;

// The pipe of the current device (created once), or nullptr.  Call with g_pipe_mu held.
static HostPipe *host_pipe()
{
  static HostPipe pipes[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return nullptr; }
  HostPipe &p = pipes[dev];
  if (p.ok) return &p;
  bool good = cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; good && i < kStageBufs; ++i)
    good = cudaEventCreateWithFlags(&p.in_done[i], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&p.k_done[i], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&p.out_done[i], cudaEventDisableTiming) == cudaSuccess;
  if (!good) { (void)cudaGetLastError(); return nullptr; }
  p.ok = true;
  return &p;
}

// Channels per block: about 256 MB per tensor, a multiple of 4 channels (keeps every block's first
// element 16-byte aligned in the host tensor whatever dim0 is), at least 4 blocks when C allows.
static uint32_t default_chunk(uint32_t dim0, uint32_t C, uint32_t N)
{
  const uint64_t per_channel = (uint64_t)dim0 * N * 4;
  uint64_t cc = (256ull << 20) / (per_channel ? per_channel : 1);
  if (cc > C / 4) cc = C / 4;
  cc = cc / 4 * 4;
  if (cc < 4) cc = 4;
  if (cc > C) cc = C;
  return (uint32_t)cc;
}

struct StageLayout {
  uint32_t chunk;            // channels per block
  uint64_t ws_bytes;         // one workspace, large enough for a full block and for the last one
  uint64_t tensor_bytes;     // one staged tensor of a full block
  uint64_t total;
};

// `samples_for_chunk`: the sample count the default block size is derived from (with several GPUs the
// same number on every rank, so that all ranks cut the layer into the same blocks); `gather`: bytes
// behind the workspace that a synchronized launch may need for its records.
static bool stage_layout(uint32_t dim0, uint32_t C, uint32_t N, uint32_t chunk, StageLayout &L,
                         uint32_t samples_for_chunk = 0, const AnodeSyncComm *comm = nullptr)
{
  if (chunk == 0) chunk = default_chunk(dim0, C, samples_for_chunk ? samples_for_chunk : N);
  if (chunk > C) chunk = C;
  L.chunk = chunk;
  const uint32_t tail = C % chunk;
  uint64_t ws = 2 * workspace_part_bytes(dim0, chunk, N) + sync_gather_bytes(chunk, comm);
  if (tail) { const uint64_t w = 2 * workspace_part_bytes(dim0, tail, N) + sync_gather_bytes(tail, comm); if (w > ws) ws = w; }
  L.ws_bytes = align_up_u64(ws, 256);
  L.tensor_bytes = align_up_u64((uint64_t)dim0 * chunk * N * 4, 256);
  L.total = L.ws_bytes + (uint64_t)kStageBufs * 3 * L.tensor_bytes;      // per buffer: x, dy (dx in place), y
  return true;
}

// One tensor block [N][cc][dim0] between the packed host tensor [N][C][dim0] and a dense device block.
static cudaError_t copy_block(float *dev, float *host, uint32_t dim0, uint32_t C, uint32_t N, uint32_t c0, uint32_t cc,
                              bool to_device, cudaStream_t s)
{
  const size_t width = (size_t)cc * dim0 * 4, hpitch = (size_t)C * dim0 * 4;
  float *h = host + (size_t)c0 * dim0;
  const cudaMemcpyKind kind = to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
  if (cc == C) return to_device ? cudaMemcpyAsync(dev, h, width * N, kind, s) : cudaMemcpyAsync(h, dev, width * N, kind, s);
  if (hpitch < ((size_t)1 << 31))
    return to_device ? cudaMemcpy2DAsync(dev, width, h, hpitch, width, N, kind, s)
                     : cudaMemcpy2DAsync(h, hpitch, dev, width, width, N, kind, s);
  for (uint32_t n = 0; n < N; ++n) {        // pitch beyond what a 2-D copy takes: one copy per sample
    float *hn = h + (size_t)n * C * dim0, *dn = dev + (size_t)n * cc * dim0;
    const cudaError_t e = to_device ? cudaMemcpyAsync(dn, hn, width, kind, s) : cudaMemcpyAsync(hn, dn, width, kind, s);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace anode_b200

using namespace anode_b200;

extern "C" size_t anode_gpu_batch_norm_host_step_staging_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                                               uint32_t chunk_channels)
{
  if (check_dims(dim0, dim1, dim2)) return 0;
  StageLayout L;
  stage_layout(dim0, dim1, dim2, chunk_channels, L);
  return (size_t)L.total;
}

extern "C" uint32_t anode_gpu_batch_norm_host_step_blocks(uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                                          uint32_t chunk_channels)
{
  if (check_dims(dim0, dim1, dim2)) return 0;
  StageLayout L;
  stage_layout(dim0, dim1, dim2, chunk_channels, L);
  return ceil_div_u32(dim1, L.chunk);
}

// Number of samples per rank the block size of a synchronized step is derived from.
static uint32_t sync_chunk_samples(uint32_t dim0, uint64_t global_count, const AnodeSyncComm *comm)
{
  const uint64_t per_rank = global_count / ((uint64_t)dim0 * (uint64_t)sync_world(comm));
  return per_rank ? (uint32_t)per_rank : 1u;
}

// The step, on one GPU (comm == nullptr) or synchronized over the ranks of `comm`: every rank then makes
// the same sequence of synchronized launches, one pair per channel block.
static int host_step(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count, float epsilon, float avg_rate, int relu,
                     const float *host_x, const float *host_dy, const float *gamma, const float *beta,
                     float *host_y, float *host_dx,
                     float *mean, float *var, float *run_mean, float *run_var, float *dgamma, float *dbeta,
                     AnodeSyncComm *comm, void *staging, size_t staging_bytes, uint32_t chunk_channels, cudaStream_t stream)
{
  const int drc = check_dims(dim0, dim1, dim2);
  if (drc) return drc;
  if (!host_x || !host_dy || !host_y || !host_dx || !mean || !var) return ANODE_E_NULL;
  if (!aligned4(host_x) || !aligned4(host_dy) || !aligned4(host_y) || !aligned4(host_dx)) return ANODE_E_ALIGN;
  if (!staging || (reinterpret_cast<uintptr_t>(staging) & 255u)) return ANODE_E_WORKSPACE;
  if (comm && global_count < (uint64_t)dim0 * dim2) return ANODE_E_DIMS;
  StageLayout L;
  stage_layout(dim0, dim1, dim2, chunk_channels, L, comm ? sync_chunk_samples(dim0, global_count, comm) : 0, comm);
  if (staging_bytes < L.total) return ANODE_E_WORKSPACE;

  std::lock_guard<std::mutex> lock(g_pipe_mu);
  HostPipe *P = host_pipe();
  if (!P) return ANODE_E_LAUNCH;
  unsigned char *base = static_cast<unsigned char *>(staging);
  unsigned char *ws = base;
  auto tensor = [&](int buf, int which) {
    return reinterpret_cast<float *>(base + L.ws_bytes + ((uint64_t)buf * 3 + which) * L.tensor_bytes);
  };
#define ANODE_TRY(call) do { if ((call) != cudaSuccess) { (void)cudaGetLastError(); return ANODE_E_LAUNCH; } } while (0)
  // the copy streams start after whatever the caller's stream holds so far
  ANODE_TRY(cudaMemsetAsync(ws, 0, L.ws_bytes, stream));
  ANODE_TRY(cudaEventRecord(P->start, stream));
  ANODE_TRY(cudaStreamWaitEvent(P->in, P->start, 0));
  ANODE_TRY(cudaStreamWaitEvent(P->out, P->start, 0));

  const uint32_t nchunks = ceil_div_u32(dim1, L.chunk);
  uint32_t prev_cc = 0;
  for (uint32_t k = 0; k < nchunks; ++k) {
    const int b = (int)(k % kStageBufs);
    const uint32_t c0 = k * L.chunk, cc = (dim1 - c0 < L.chunk) ? (dim1 - c0) : L.chunk;
    float *dx_ = tensor(b, 1);        // dy arrives here, dx replaces it
    // host -> device, once the buffer's previous contents have left
    if (k >= (uint32_t)kStageBufs) ANODE_TRY(cudaStreamWaitEvent(P->in, P->out_done[b], 0));
    ANODE_TRY(copy_block(tensor(b, 0), const_cast<float *>(host_x), dim0, dim1, dim2, c0, cc, true, P->in));
    ANODE_TRY(copy_block(dx_, const_cast<float *>(host_dy), dim0, dim1, dim2, c0, cc, true, P->in));
    ANODE_TRY(cudaEventRecord(P->in_done[b], P->in));
    // both kernels on the caller's stream
    ANODE_TRY(cudaStreamWaitEvent(stream, P->in_done[b], 0));
    if (prev_cc != 0 && cc != prev_cc)   // the last block is tiled differently: start from a clean workspace
      ANODE_TRY(cudaMemsetAsync(ws + 256, 0, L.ws_bytes - 256, stream));
    prev_cc = cc;
    FusedArgs a;
    const size_t fused = (size_t)(2 * workspace_part_bytes(dim0, cc, dim2));      // the records of a synchronized launch sit behind it
    int rc = prepare_fwd(a, dim0, cc, dim2, epsilon, avg_rate, relu, tensor(b, 0), gamma ? gamma + c0 : nullptr,
                         (gamma && beta) ? beta + c0 : nullptr, tensor(b, 2), mean + c0, var + c0,
                         run_mean ? run_mean + c0 : nullptr, run_var ? run_var + c0 : nullptr, ws, fused);
    if (rc) return rc;
    rc = comm ? sync_launch(a, 0, true, comm, fused, stream) : launch_best(a, 0, true, stream);
    if (rc) return rc;
    rc = prepare_bwd(a, dim0, cc, dim2, relu, 0, dx_, tensor(b, 0), mean + c0, var + c0, gamma ? gamma + c0 : nullptr,
                     (gamma && beta) ? beta + c0 : nullptr, dx_, dgamma ? dgamma + c0 : nullptr,
                     dbeta ? dbeta + c0 : nullptr, ws, fused);
    if (rc) return rc;
    if (comm) a.count_total = (double)global_count;
    rc = comm ? sync_launch(a, 1, true, comm, fused, stream) : launch_best(a, 1, true, stream);
    if (rc) return rc;
    ANODE_TRY(cudaEventRecord(P->k_done[b], stream));
    // device -> host
    ANODE_TRY(cudaStreamWaitEvent(P->out, P->k_done[b], 0));
    ANODE_TRY(copy_block(tensor(b, 2), host_y, dim0, dim1, dim2, c0, cc, false, P->out));
    ANODE_TRY(copy_block(dx_, host_dx, dim0, dim1, dim2, c0, cc, false, P->out));
    ANODE_TRY(cudaEventRecord(P->out_done[b], P->out));
  }
  // the caller's stream ends after the last copies
  for (int b = 0; b < kStageBufs && (uint32_t)b < nchunks; ++b) ANODE_TRY(cudaStreamWaitEvent(stream, P->out_done[b], 0));
#undef ANODE_TRY
  return ANODE_OK;
}

extern "C" int anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, int relu,
    const float *host_x, const float *host_dy, const float *gamma, const float *beta,
    float *host_y, float *host_dx,
    float *mean, float *var, float *run_mean, float *run_var, float *dgamma, float *dbeta,
    void *staging, size_t staging_bytes, uint32_t chunk_channels,
    const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  return host_step(dim0, dim1, dim2, 0, epsilon, avg_rate, relu, host_x, host_dy, gamma, beta, host_y, host_dx, mean, var,
                   run_mean, run_var, dgamma, dbeta, nullptr, staging, staging_bytes, chunk_channels, stream);
}

// The same step for one rank's shard of a batch sharded over the ranks of `comm`: the kernels of every
// channel block are the synchronized ones, so statistics and backward sums are those of the global
// batch while each rank's copies overlap with its kernels as above.
extern "C" size_t anode_gpu_sync_batch_norm_host_step_staging_bytes(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count,
                                                                    struct AnodeSyncComm *comm, uint32_t chunk_channels)
{
  if (!comm || check_dims(dim0, dim1, dim2) || global_count < (uint64_t)dim0 * dim2) return 0;
  StageLayout L;
  stage_layout(dim0, dim1, dim2, chunk_channels, L, sync_chunk_samples(dim0, global_count, comm), comm);
  return (size_t)L.total;
}

extern "C" uint32_t anode_gpu_sync_batch_norm_host_step_blocks(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count,
                                                               struct AnodeSyncComm *comm, uint32_t chunk_channels)
{
  if (!comm || check_dims(dim0, dim1, dim2) || global_count < (uint64_t)dim0 * dim2) return 0;
  StageLayout L;
  stage_layout(dim0, dim1, dim2, chunk_channels, L, sync_chunk_samples(dim0, global_count, comm), comm);
  return ceil_div_u32(dim1, L.chunk);
}

extern "C" int anode_gpu_sync_batch_norm_relu_step_host_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, uint64_t global_count, float epsilon, float avg_rate, int relu,
    const float *host_x, const float *host_dy, const float *gamma, const float *beta,
    float *host_y, float *host_dx,
    float *mean, float *var, float *run_mean, float *run_var, float *dgamma, float *dbeta,
    struct AnodeSyncComm *comm, void *staging, size_t staging_bytes, uint32_t chunk_channels,
    const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  if (!comm) return ANODE_E_COMM;
  return host_step(dim0, dim1, dim2, global_count, epsilon, avg_rate, relu, host_x, host_dy, gamma, beta, host_y, host_dx, mean, var,
                   run_mean, run_var, dgamma, dbeta, comm, staging, staging_bytes, chunk_channels, stream);
}
