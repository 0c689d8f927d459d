// Diagnostics of the slice-resident kernel's planner: the plan and the event sequence of a thread
// block, for CPU tests of the schedule (host code only; no GPU needed).
#include <stdint.h>

#include "../../include/anode_routines_gpu.h"
#include "bn_resident_plan.h"

namespace anode_b200 {
bool resident_plan_for(uint32_t dim0, uint32_t C, uint32_t N, uint32_t planes, ResPlan &p);
int check_dims(uint32_t dim0, uint32_t dim1, uint32_t dim2);
}  // namespace anode_b200

using namespace anode_b200;

// out (16 values): applies, rpp, P, piece_len, U, Gt, teams, grid, T, slot_bytes, Q, Qr, Qs, Rz_max, pf, smem_bytes
extern "C" int anode_gpu_batch_norm_resident_plan(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t planes, uint32_t *out)
{
  if (!out || check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  ResPlan p{};
  const bool ok = resident_plan_for(dim0, dim1, dim2, planes, p);
  const uint32_t v[16] = {ok ? 1u : 0u, p.rpp, p.P, p.piece_len, p.U, p.Gt, p.teams, p.grid, p.T, p.slot_bytes, p.Q, p.Qr, p.Qs, p.Rz_max, p.pf, p.smem_bytes};
  for (int i = 0; i < 16; ++i) out[i] = v[i];
  return ANODE_OK;
}

// Writes the event sequence of thread block `block` (4 values per event: kind, k, piece, slot) and
// returns the number of events, or a negative error; at most `max_events` are written.
extern "C" long long anode_gpu_batch_norm_resident_schedule(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t planes,
                                                            uint32_t block, uint32_t *out, uint64_t max_events)
{
  if (check_dims(dim0, dim1, dim2)) return ANODE_E_DIMS;
  ResPlan p{};
  if (!resident_plan_for(dim0, dim1, dim2, planes, p) || block >= p.grid) return ANODE_E_DIMS;
  const ResBlock rb = res_block(p, block);
  uint64_t n = 0;
  res_walk(p, rb, [&](const ResEvent &e) -> bool {
    if (out && n < max_events) { out[4 * n] = e.kind; out[4 * n + 1] = e.k; out[4 * n + 2] = e.piece; out[4 * n + 3] = e.slot; }
    ++n;
    return true;
  });
  return (long long)n;
}
