// Flags, counters and bounded waits shared by the kernels that exchange data between the GPUs
// of a tensor-parallel group (and between the CTAs of one kernel).
//
// All remote traffic is plain stores, plain loads and reductions on peer-mapped global memory;
// nothing here issues a bulk or tensor copy. Every wait carries a clock limit: when it runs
// out the caller records an error word and carries on with whatever has arrived, so a lost
// peer ends in an error the host can read, never in a kernel that spins forever.
#pragma once
#include "common.cuh"

namespace lq {

constexpr long long kDefaultWaitCycles = 4000000000LL;  // ~2 s of SM clock

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_f4(float* p, float a, float b, float c, float d) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ float4 ld_peer_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Waits until the counter at `p` has reached `target` (counters only grow; the comparison is
// on the wrapped difference). False if `limit` clocks pass first.
template <bool SYS>
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target, long long limit) {
  uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
  if ((int32_t)(v - target) >= 0) return true;
  const long long t0 = clock64();
  for (;;) {
    v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int32_t)(v - target) >= 0) return true;
    if (clock64() - t0 > limit) return false;
  }
}

}  // namespace lq
