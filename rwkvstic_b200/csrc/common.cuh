// Shared device helpers for the sm_100a kernels: mbarrier / bulk-copy (TMA) PTX wrappers,
// bounded waits, programmatic-dependent-launch controls, small reductions.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200rwkv.h"

namespace b200 {

// A device-side wait never spins for ever: after this many nanoseconds it gives up, raises an
// abort flag in shared memory and a status bit in global memory, and the kernel runs to its end.
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- programmatic dependent launch -------------------------------------------------------------
// launch_dependents: lets the next kernel in the stream start its weight prefetch while this one
// still runs.  wait: blocks until every kernel this launch depends on has finished and its
// writes are visible; a no-op when the kernel was launched without the attribute.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- mbarrier -----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.shared::cta.b64 t, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait for `parity` of `bar`, at most limit_ns.  Returns false (and raises *abort_flag) when
// the limit is hit or another thread already raised the flag.
__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > limit_ns) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_wait_limited(bar, parity, abort_flag, kWaitLimitNs);
}

// ---- TMA bulk copy (1-D, global -> shared), completion counted in bytes on an mbarrier ----------
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// ---- named barrier over a subset of warps --------------------------------------------------------
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- integer dot products ------------------------------------------------------------------------
// Four unsigned bytes of `q` times four SIGNED bytes of `x`, added to acc.
__device__ __forceinline__ int dp4a_us(uint32_t q, uint32_t x, int acc) {
  int r;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(q), "r"(x), "r"(acc));
  return r;
}
// Four unsigned bytes times four unsigned bytes.
__device__ __forceinline__ uint32_t dp4a_uu(uint32_t q, uint32_t x, uint32_t acc) {
  uint32_t r;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(q), "r"(x), "r"(acc));
  return r;
}

// Loads whose ISSUE POINT matters (they are placed early so that their latency hides behind other
// work).  volatile asm keeps them where they are written relative to the barrier / dependency
// instructions; a plain or __ldg load may legally be sunk to its first use.
// ld_param_v4: read-only data no kernel writes.  ld_act_v4: data an earlier kernel produced (L2 only).
__device__ __forceinline__ float4 ld_param_v4(const float4* p) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float4 ld_act_v4(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float ld_param_f32(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_act_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// One WKV-4 step in the max-trick form (state aa, bb scaled by exp(-pp); decay applied when the
// state is advanced).  Same arithmetic as the reference's agnosticRwkv.py:68-103.
__device__ __forceinline__ float wkv_step(float k, float v, float w, float u, float& aa, float& bb, float& pp) {
  const float ww = u + k;
  const float p = fmaxf(pp, ww);
  const float e1 = expf(pp - p), e2 = expf(ww - p);
  const float y = (e1 * aa + e2 * v) / (e1 * bb + e2);
  const float ww2 = pp + w;
  const float p2 = fmaxf(ww2, k);
  const float f1 = expf(ww2 - p2), f2 = expf(k - p2);
  aa = f1 * aa + f2 * v;
  bb = f1 * bb + f2;
  pp = p2;
  return y;
}

}  // namespace b200
