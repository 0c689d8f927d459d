// Device-side building blocks shared by the batch-norm kernels: 128-bit packs, acquire /
// release accesses, warp and block reductions, and the merge of (count, mean, M2) partials.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "bn_plan.h"

namespace anode_b200 {

// ---- memory-ordering helpers ----------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p)
{
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t *p)
{
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t *p, uint32_t v)
{
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---- L2 eviction policies ----------------------------------------------------------------
// keep: data that will be read a second time (the reduce pass of a tile);
// drop: data that is dead after this access (the apply pass's re-read, and every output).
__device__ __forceinline__ uint64_t policy_keep()
{
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// keep for a fraction of the lines (chosen by address), drop for the rest: for a working set larger than what
// L2 can hold, so that the kept part stays instead of all of it cycling through
__device__ __forceinline__ uint64_t policy_keep_fraction(float f)
{
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.L2::evict_first.b64 %0, %1;" : "=l"(p) : "f"(f));
  return p;
}
__device__ __forceinline__ uint64_t policy_drop()
{
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---- packs of VEC floats ----------------------------------------------------------------
template <int VEC> struct Pack;
template <> struct Pack<4> {
  float v[4];
  __device__ __forceinline__ static Pack load(const float *p)
  {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    Pack r; r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; return r;
  }
  __device__ __forceinline__ static Pack load(const float *p, uint64_t pol)
  {
    Pack r;
    asm volatile("ld.global.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]) : "l"(p), "l"(pol));
    return r;
  }
  // streaming store: the written tensor is not read again by this kernel
  __device__ __forceinline__ void store_stream(float *p) const
  {
    __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
  __device__ __forceinline__ void store(float *p, uint64_t pol) const
  {
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;"
                 ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "l"(pol) : "memory");
  }
};
template <> struct Pack<1> {
  float v[1];
  __device__ __forceinline__ static Pack load(const float *p) { Pack r; r.v[0] = *p; return r; }
  __device__ __forceinline__ static Pack load(const float *p, uint64_t pol)
  {
    Pack r;
    asm volatile("ld.global.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(r.v[0]) : "l"(p), "l"(pol));
    return r;
  }
  __device__ __forceinline__ void store_stream(float *p) const { __stcs(p, v[0]); }
  __device__ __forceinline__ void store(float *p, uint64_t pol) const
  {
    asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(p), "f"(v[0]), "l"(pol) : "memory");
  }
};
template <int VEC> __device__ __forceinline__ Pack<VEC> pack_fill(float f)
{
  Pack<VEC> r;
#pragma unroll
  for (int i = 0; i < VEC; ++i) r.v[i] = f;
  return r;
}

// ReLU exactly as the reference writes it (routines_gpu/flat_map.cu:176-177): x * (float)(x > 0).
// Negative inputs give -0, NaN stays NaN, -inf gives NaN.
__device__ __forceinline__ float positive_clip(float x) { return x * (x > 0.0f ? 1.0f : 0.0f); }

// ---- reductions ------------------------------------------------------------------------
struct Moments { float n, mean, m2; };

// Chan et al. pairwise update of (count, mean, sum of squared deviations).
__device__ __forceinline__ Moments merge(Moments a, Moments b)
{
  const float n = a.n + b.n;
  if (n <= 0.0f) return Moments{0.f, 0.f, 0.f};
  const float f = __fdividef(b.n, n);
  const float d = b.mean - a.mean;
  Moments r;
  r.n = n;
  r.mean = fmaf(d, f, a.mean);
  r.m2 = a.m2 + b.m2 + d * d * a.n * f;
  return r;
}

__device__ __forceinline__ Moments warp_merge(Moments a)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Moments b;
    b.n = __shfl_down_sync(0xffffffffu, a.n, o);
    b.mean = __shfl_down_sync(0xffffffffu, a.mean, o);
    b.m2 = __shfl_down_sync(0xffffffffu, a.m2, o);
    a = merge(a, b);
  }
  return a;
}

// Block-wide merge in a fixed order; the result is valid in thread 0.  `buf` holds
// 3 * (kThreads/32) floats of shared memory.  Contains two block barriers.
__device__ __forceinline__ Moments block_merge(Moments a, float *buf)
{
  constexpr int kWarps = kThreads / 32;
  a = warp_merge(a);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();   // buf may still be read from a previous use
  if (lane == 0) { buf[warp] = a.n; buf[kWarps + warp] = a.mean; buf[2 * kWarps + warp] = a.m2; }
  __syncthreads();
  if (warp == 0) {
    Moments b{0.f, 0.f, 0.f};
    if (lane < kWarps) { b.n = buf[lane]; b.mean = buf[kWarps + lane]; b.m2 = buf[2 * kWarps + lane]; }
#pragma unroll
    for (int o = kWarps / 2; o > 0; o >>= 1) {
      Moments c;
      c.n = __shfl_down_sync(0xffffffffu, b.n, o);
      c.mean = __shfl_down_sync(0xffffffffu, b.mean, o);
      c.m2 = __shfl_down_sync(0xffffffffu, b.m2, o);
      b = merge(b, c);
    }
    a = b;
  }
  return a;
}

template <typename T> __device__ __forceinline__ T warp_sum(T v)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  return v;
}
template <typename T> __device__ __forceinline__ T warp_sum_all(T v)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum of two values in a fixed order; result broadcast to every thread.
// `buf` holds 2 * (kThreads/32) elements of T.  Contains three block barriers.
template <typename T> __device__ __forceinline__ void block_sum2(T &a, T &b, T *buf)
{
  constexpr int kWarps = kThreads / 32;
  a = warp_sum(a); b = warp_sum(b);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { buf[warp] = a; buf[kWarps + warp] = b; }
  __syncthreads();
  T ta = 0, tb = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) { ta += buf[w]; tb += buf[kWarps + w]; }
  a = ta; b = tb;
  __syncthreads();
}

}  // namespace anode_b200
