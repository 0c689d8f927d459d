// Fused batch-norm + ReLU forward for callers that cannot hand over scratch memory.
//
// Who that is: anode's op closures reach a kernel through a fixed argument list of dimensions,
// inputs, pre-made outputs, a launch hint and a stream (src/ops_gpu.rs:3763-3771).  A caller that
// keeps that shape has no workspace pointer to pass, and code that runs inside a memory-pool
// transaction or on a stream whose ordering it does not own must not call cudaMalloc, which
// synchronises the device.  For them the scratch lives in this library: one fixed array in
// device memory, reserved on every GPU that loads the library until the process exits.
//
// Consequences the caller has to know:
//   - the array is shared by every call on a device and keeps the last call's contents; each call
//     clears the part that must start at zero, on the caller's stream;
//   - two calls that overlap on the GPU (different streams, no ordering between them) race on it;
//   - problems whose scratch need exceeds ANODE_STATIC_SCRATCH_BYTES are rejected;
//   - the first call on a device looks up the array's device address (cudaGetSymbolAddress);
//     make that first call outside of any stream capture.
#include "bn_host.h"

namespace anode_b200 {

// In host code this name is only a stand-in for the symbol; kernels must be given the address
// that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_static_scratch[ANODE_STATIC_SCRATCH_BYTES];

// Device address of the array on the current device (looked up once per device), or nullptr.
static unsigned char *static_scratch_ptr()
{
  static std::mutex mu;
  static unsigned char *cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return nullptr; }
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) { (void)cudaGetLastError(); return nullptr; }
    cache[dev] = static_cast<unsigned char *>(p);
  }
  return cache[dev];
}

}  // namespace anode_b200

using namespace anode_b200;

// Scratch bytes the forward kernel that will serve this call needs, and how many of them have to be
// zero when it starts (progress counters, flags, records).  `a` is a prepared call whose workspace is
// the built-in array.
static void static_need(const FusedArgs &a, bool aligned, uint64_t &need, uint64_t &clear)
{
  const uint32_t dim0 = a.plan.dim0, C = a.plan.C, N = a.plan.N;
  switch (pick_kernel_kind(a, 0, aligned)) {
    case ANODE_KERNEL_CLUSTER:        // keeps everything on chip: only the status word lives in the array
      need = clear = 256;
      break;
    case ANODE_KERNEL_PLAIN: {
      const Plan p = plan_for(dim0, C, N, aligned);
      need = p.ws_bytes; clear = p.off_part;
      break;
    }
    default:                          // tiled and slice-resident kernels: their share of a workspace part
      need = workspace_part_bytes(dim0, C, N);
      clear = control_region_bytes(dim0, C, N, aligned);
      break;
  }
}

extern "C" int anode_gpu_batch_norm_relu_fused_fwd_static_3d1_packed_f32(
    uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, int relu,
    const float *x, const float *gamma, const float *beta,
    float *y, float *mean, float *var, float *run_mean, float *run_var,
    const struct KernelConfig *cfg, struct CUstream_st *stream)
{
  (void)cfg;
  const int drc = check_dims(dim0, dim1, dim2);
  if (drc) return drc;
  if (!x || !y || !mean || !var) return ANODE_E_NULL;
  unsigned char *scratch = static_scratch_ptr();
  if (!scratch) return ANODE_E_LAUNCH;
  FusedArgs a;
  // (the size handed to prepare_fwd is the size a caller-owned workspace would have; what this call
  // really needs is checked against the built-in array below)
  const int rc = prepare_fwd(a, dim0, dim1, dim2, epsilon, avg_rate, relu, x, gamma, beta, y, mean, var,
                             run_mean, run_var, scratch, (size_t)workspace_part_bytes(dim0, dim1, dim2));
  if (rc) return rc;
  const bool aligned = aligned16(x) && aligned16(y);
  if (a.ws_capacity > ANODE_STATIC_SCRATCH_BYTES) a.ws_capacity = ANODE_STATIC_SCRATCH_BYTES;
  uint64_t need = 0, clear = 0;
  static_need(a, aligned, need, clear);
  if (need > ANODE_STATIC_SCRATCH_BYTES) return ANODE_E_TOO_LARGE;     // the built-in array is too small for this problem
  // counters, flags and records must start at zero whatever the previous call left behind
  if (clear > need) clear = need;
  if (cudaMemsetAsync(scratch, 0, (size_t)clear, stream) != cudaSuccess) { (void)cudaGetLastError(); return ANODE_E_LAUNCH; }
  return launch_best(a, 0, aligned, stream);
}

extern "C" int anode_gpu_batch_norm_fused_static_status(struct CUstream_st *stream, uint32_t *status)
{
  if (!status) return ANODE_E_NULL;
  unsigned char *scratch = static_scratch_ptr();
  if (!scratch) return ANODE_E_LAUNCH;
  return anode_gpu_batch_norm_fused_status(scratch, stream, status);
}
