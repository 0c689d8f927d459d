// Host-side declarations shared by the translation units of libanode_routines_gpu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

#include "../../include/anode_routines_gpu.h"
#include "bn_fused.cuh"

namespace anode_b200 {

struct Tunables {
  uint32_t tile_floats;     // target floats per tile
  uint32_t slack_steps;     // extra lookahead steps beyond the minimum
  uint32_t blocks_per_sm;   // persistent blocks planned per SM
  uint32_t ring_slots;      // shared-memory slots per block (forward)
  uint32_t ring_slots_bwd;  // shared-memory slots per block (backward; a slot holds x and dy)
  uint32_t ring_floats_fwd; // floats per slot (forward: x)
  uint32_t ring_floats_bwd; // floats per tensor per slot (backward: x and dy)
  uint32_t ring_blocks_per_sm;
  uint32_t ring_warps_fwd;  // consumer warps of the forward kernel (8 or 16)
  uint32_t ring_warps_bwd;  // consumer warps of the backward kernel (8 or 16)
};
const Tunables &tunables();

uint32_t sm_count();
Plan plan_for(uint32_t dim0, uint32_t C, uint32_t N, bool aligned16);
int check_dims(uint32_t dim0, uint32_t dim1, uint32_t dim2);
bool aligned16(const void *p);
bool aligned4(const void *p);

int prepare_fwd(FusedArgs &a, uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate,
                int relu, const float *x, const float *gamma, const float *beta, float *y, float *mean,
                float *var, float *run_mean, float *run_var, void *ws, size_t ws_bytes);
int prepare_bwd(FusedArgs &a, uint32_t dim0, uint32_t dim1, uint32_t dim2, int relu, int accumulate,
                const float *dy, const float *x, const float *mean, const float *var, const float *gamma,
                const float *beta, float *dx, float *dgamma, float *dbeta, void *ws, size_t ws_bytes);
int launch_pipeline(FusedArgs &a, int dir, cudaStream_t stream);
// the kernel that serves a prepared call (ANODE_KERNEL_*, -1 for none), and its launch
int pick_kernel_kind(const FusedArgs &a, int dir, bool aligned);
int launch_best(FusedArgs &a, int dir, bool aligned, cudaStream_t stream);
int kernel_choice();
bool ring_applies(const FusedArgs &a, int dir, bool aligned);
// the cluster kernel for short rows (bn_segres.cu)
bool segres_applies(const FusedArgs &a, int dir, bool aligned);
bool segres_preferred(const FusedArgs &a, int dir, bool aligned);      // take it even where the tiled kernel applies
int launch_segres(FusedArgs &a, int dir, cudaStream_t stream);
uint64_t workspace_part_bytes(uint32_t dim0, uint32_t C, uint32_t N);
// the slice-resident kernel (bn_resident.cu)
bool resident_applies(const FusedArgs &a, int dir, bool aligned);
uint64_t resident_ws_bytes(uint32_t dim0, uint32_t C, uint32_t N);
int launch_resident(FusedArgs &a, int dir, uint64_t ws_off, cudaStream_t stream);
long long wait_limit_cycles();
uint64_t control_region_bytes(uint32_t dim0, uint32_t C, uint32_t N, bool aligned);

// synchronized launches (bn_sync.cu), for the host-buffer step
int sync_launch(FusedArgs &a, int dir, bool aligned, struct ::AnodeSyncComm *comm, size_t fused_ws_bytes, cudaStream_t stream);
size_t sync_gather_bytes(uint32_t C, const struct ::AnodeSyncComm *comm);
int sync_world(const struct ::AnodeSyncComm *comm);

}  // namespace anode_b200
