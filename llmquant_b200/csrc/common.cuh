// Shared helpers for the sm_100a kernels behind the C ABI in include/llmquant_b200.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/llmquant_b200.h"

namespace lq {

constexpr float kScaleEps = 1e-8f;  // floor of every abs-max scale
constexpr int kSmCount = 148;       // B200; grids are sized from the queried value at run time

// Thread-local message returned by lq_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
int sm_count();
// Raises a kernel's dynamic shared-memory limit once per (kernel, device); the attribute is a
// property of the device the kernel is loaded on, so the bookkeeping is keyed by both.
int ensure_smem_limit(const void* kernel, int bytes, const char* what);

#define LQ_REQUIRE(cond, code, ...)            \
  do {                                         \
    if (!(cond)) return lq::fail(code, __VA_ARGS__); \
  } while (0)

template <typename T>
struct Conv;
template <>
struct Conv<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <>
struct Conv<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <>
struct Conv<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The one quantization rule of the path: IEEE division, round-half-even, clamp.
__device__ __forceinline__ float scale_of(float amax, float qmax) {
  return fmaxf(__fdiv_rn(amax, qmax), kScaleEps);
}
__device__ __forceinline__ float code_of(float v, float scale, float qmin, float qmax) {
  return fminf(fmaxf(rintf(__fdiv_rn(v, scale)), qmin), qmax);
}

// ---- mbarrier / bulk-copy primitives (shared::cta addresses as 32-bit values)
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// The same test, but the thread may be suspended for up to `ns` nanoseconds while the phase
// is incomplete: it is woken when the phase completes and issues nothing until then.
__device__ __forceinline__ bool mbar_try_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return done != 0;
}
// Bounded wait: false if the phase did not complete within ~1 s of SM clock. The clock is only
// read once the first try has failed, so a wait on data that has already landed costs three
// instructions; after that the thread sleeps in the barrier between looks at the clock, so a
// waiting warp leaves the issue slots to the warps that work.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_suspend(bar, parity, 20000u)) return true;
    if (clock64() - t0 > 2000000000LL) return false;
  }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}


#define LQ_DISPATCH_DTYPE(dtype, T, ...)                   \
  switch (dtype) {                                         \
    case LQ_F32: { using T = float; __VA_ARGS__; break; }  \
    case LQ_F16: { using T = __half; __VA_ARGS__; break; } \
    case LQ_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    default: return lq::fail(LQ_ERR_DTYPE, "x must be float32, float16 or bfloat16, got dtype id %d", (int)(dtype)); \
  }

}  // namespace lq
