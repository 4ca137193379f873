// Decode GEMV on the reference's canonical layout: qweight [N, G, gs] int8 (one byte per
// weight, int4 included), wscale [scale_rows, G] fp32, x [M, G*gs] in fp32 / fp16 / bf16.
//
// This is the operator-level drop-in: it accepts exactly the tensors the reference's
// KernelQuantLinear holds, so that module runs unchanged on top of it. The faster path that
// streams true nibbles lives in gemv_stream.cu.
//
// One warp owns one output row and walks it in 16-byte chunks (4-byte chunks when the group
// size is not a multiple of 16), so a warp's load is one contiguous 512-byte piece of the
// row. A chunk never straddles a group; its fp32 partial sum is scaled once and the warp
// reduces with shuffles at the end of the row. Up to eight activation rows share one pass
// over the weight.
//
// The stacked-expert form (Mixture-of-Experts decode, reference wq_gemv_batched.cu:45-130)
// is the same kernel with the weight chosen per grid row: the host lists blocks of
// (expert, first activation row, row count <= 8); block b multiplies its rows with
// qweight[expert] ([E, N, G, gs]) and wscale[expert] ([E, scale_rows, G]).
#include "common.cuh"

namespace lq {
namespace {

constexpr int kRows = 8;    // activation rows per pass (grid.y covers more)
constexpr int kWarps = 4;

template <typename T, int VEC>
__global__ void __launch_bounds__(kWarps * 32)
gemv_canonical_kernel(const T* __restrict__ x, const int8_t* __restrict__ qweight,
                      const float* __restrict__ wscale, T* __restrict__ out, int M, int N,
                      int groups, int gs, int out_group, const int* __restrict__ block_expert,
                      const int* __restrict__ block_row0, const int* __restrict__ block_rows,
                      int scale_rows) {
  const int lane = threadIdx.x & 31;
  const int kp = groups * gs;
  int m0 = blockIdx.y * kRows;
  int rows = min(kRows, M - m0);
  if (block_expert != nullptr) {  // stacked experts: this grid row's weight and activation rows
    const int e = block_expert[blockIdx.y];
    m0 = block_row0[blockIdx.y];
    rows = min(min(kRows, block_rows[blockIdx.y]), M - m0);
    if (rows <= 0) return;
    qweight += (int64_t)e * N * kp;
    wscale += (int64_t)e * scale_rows * groups;
  }
  const int chunks = kp / VEC;
  for (int n = blockIdx.x * kWarps + (threadIdx.x >> 5); n < N; n += gridDim.x * kWarps) {
    const int8_t* wrow = qweight + (int64_t)n * kp;
    const float* srow = wscale + (int64_t)(out_group > 0 ? n / out_group : n) * groups;
    float acc[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r] = 0.f;
    for (int c = lane; c < chunks; c += 32) {
      const int k0 = c * VEC;
      int8_t wv[VEC];
      if (VEC == 16)
        *reinterpret_cast<int4*>(wv) = __ldg(reinterpret_cast<const int4*>(wrow + k0));
      else
        *reinterpret_cast<int*>(wv) = __ldg(reinterpret_cast<const int*>(wrow + k0));
      const float s = __ldg(srow + k0 / gs);
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (r < rows) {
          const T* xr = x + (int64_t)(m0 + r) * kp + k0;
          T xv[VEC];
          if (VEC == 16) {
#pragma unroll
            for (int j = 0; j < (int)(VEC * sizeof(T) / 16); ++j)
              reinterpret_cast<int4*>(xv)[j] = __ldg(reinterpret_cast<const int4*>(xr) + j);
          } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) xv[i] = xr[i];
          }
          float p = 0.f;
#pragma unroll
          for (int i = 0; i < VEC; ++i) p = fmaf(Conv<T>::to_f32(xv[i]), (float)wv[i], p);
          acc[r] = fmaf(p, s, acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      if (r < rows) {
        const float t = warp_sum(acc[r]);
        if (lane == 0) out[(int64_t)(m0 + r) * N + n] = Conv<T>::from_f32(t);
      }
    }
  }
}

}  // namespace
}  // namespace lq

extern "C" int lq_wq_gemv(const void* x, const int8_t* qweight, const float* wscale, void* out,
                          int M, int N, int groups, int group_size, int out_group, int dtype,
                          void* stream) {
  using namespace lq;
  LQ_REQUIRE(group_size > 0 && group_size % 4 == 0, LQ_ERR_ARG,
             "group_size must be a multiple of 4, got %d", group_size);
  LQ_REQUIRE(M >= 0 && N >= 0 && groups >= 0 && out_group >= 0, LQ_ERR_ARG, "negative dimension");
  if (M == 0 || N == 0) return LQ_OK;
  LQ_REQUIRE(x && qweight && wscale && out, LQ_ERR_ARG, "null tensor pointer");
  const bool vec16 = group_size % 16 == 0 && ((uintptr_t)qweight % 16) == 0 && ((uintptr_t)x % 16) == 0;
  LQ_REQUIRE(((uintptr_t)qweight % 4) == 0, LQ_ERR_ARG, "qweight must be 4-byte aligned");
  const int want = (N + kWarps - 1) / kWarps;
  const int cap = sm_count() * 16;
  dim3 grid((unsigned)(want < cap ? want : cap), (unsigned)((M + kRows - 1) / kRows));
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    if (vec16)
      gemv_canonical_kernel<T, 16><<<grid, kWarps * 32, 0, s>>>(
          (const T*)x, qweight, wscale, (T*)out, M, N, groups, group_size, out_group, nullptr, nullptr, nullptr, 0);
    else
      gemv_canonical_kernel<T, 4><<<grid, kWarps * 32, 0, s>>>(
          (const T*)x, qweight, wscale, (T*)out, M, N, groups, group_size, out_group, nullptr, nullptr, nullptr, 0);
  });
  return check_launch("lq_wq_gemv");
}

extern "C" int lq_wq_gemv_batched_max_rows(void) { return lq::kRows; }

extern "C" int lq_wq_gemv_batched(const void* x, const int8_t* qweight, const float* wscale,
                                  const int* block_expert, const int* block_row0, const int* block_rows,
                                  void* out, int R, int N, int groups, int group_size, int scale_rows,
                                  int out_group, int blocks, int dtype, void* stream) {
  using namespace lq;
  LQ_REQUIRE(group_size > 0 && group_size % 4 == 0, LQ_ERR_ARG,
             "group_size must be a multiple of 4, got %d", group_size);
  LQ_REQUIRE(R >= 0 && N >= 0 && groups >= 0 && out_group >= 0 && blocks >= 0 && scale_rows >= 0, LQ_ERR_ARG,
             "negative dimension");
  if (blocks == 0 || R == 0 || N == 0) return LQ_OK;
  LQ_REQUIRE(x && qweight && wscale && out && block_expert && block_row0 && block_rows, LQ_ERR_ARG,
             "null tensor pointer");
  LQ_REQUIRE(blocks <= 65535, LQ_ERR_ARG, "at most 65535 blocks per call, got %d", blocks);
  // every expert's [N, G, gs] slab starts on a 16-byte boundary only if N*G*gs does
  const bool vec16 = group_size % 16 == 0 && ((uintptr_t)qweight % 16) == 0 && ((uintptr_t)x % 16) == 0 &&
                     ((int64_t)N * groups * group_size) % 16 == 0;
  LQ_REQUIRE(((uintptr_t)qweight % 4) == 0, LQ_ERR_ARG, "qweight must be 4-byte aligned");
  const int want = (N + kWarps - 1) / kWarps;
  const int cap = sm_count() * 16;
  dim3 grid((unsigned)(want < cap ? want : cap), (unsigned)blocks);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    if (vec16)
      gemv_canonical_kernel<T, 16><<<grid, kWarps * 32, 0, s>>>(
          (const T*)x, qweight, wscale, (T*)out, R, N, groups, group_size, out_group, block_expert, block_row0,
          block_rows, scale_rows);
    else
      gemv_canonical_kernel<T, 4><<<grid, kWarps * 32, 0, s>>>(
          (const T*)x, qweight, wscale, (T*)out, R, N, groups, group_size, out_group, block_expert, block_row0,
          block_rows, scale_rows);
  });
  return check_launch("lq_wq_gemv_batched");
}
