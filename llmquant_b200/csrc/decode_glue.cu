// The bookkeeping around one decoded token, as two small kernels that take part in the
// programmatic-dependent-launch chain of the decode step (the reference's graphed decoder does
// this with host-driven torch ops: copy_, fill_, argmax per token -- runtime/graph_decode.py:40-157):
//
//   lq_embed_gather   hidden[b, :] = embedding[tokens[b], :]                 (start of a step)
//   lq_next_token     tokens[b] = argmax(logits[b, :]) (lowest index among equal maxima, as
//                     torch.argmax), history[b, pos + 1] = tokens[b], pos += 1   (end of a step)
//
// The cursor is advanced by the CTA that finishes last (a ticket in a caller-provided int32,
// which it puts back to zero), so every row reads the same cursor value.
#include "common.cuh"

namespace lq {
namespace {

constexpr int kGlueThreads = 1024;

__global__ void __launch_bounds__(256)
embed_gather_kernel(const __nv_bfloat16* __restrict__ table, const int64_t* __restrict__ tokens,
                    __nv_bfloat16* __restrict__ hidden, int H, int64_t vocab) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int b = blockIdx.x;
  int64_t tok = tokens[b];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const __nv_bfloat16* src = table + tok * H;
  __nv_bfloat16* dst = hidden + (int64_t)b * H;
  if (H % 8 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
  }
}

__global__ void __launch_bounds__(kGlueThreads)
next_token_kernel(const __nv_bfloat16* __restrict__ logits, int64_t V, int64_t* __restrict__ tokens,
                  int64_t* pos, int64_t* __restrict__ history, int64_t hist_len, int* ticket) {
  __shared__ float best_s[kGlueThreads / 32];
  __shared__ int64_t idx_s[kGlueThreads / 32];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int b = blockIdx.x;
  const int64_t p = *pos;  // read before any CTA can advance it (see the ticket below)
  const __nv_bfloat16* row = logits + (int64_t)b * V;
  float best = -INFINITY;
  int64_t idx = 0;
  // strided scan: a thread's indices ascend, so "strictly greater" keeps its lowest maximum
  for (int64_t i = threadIdx.x; i < V; i += kGlueThreads) {
    const float v = __bfloat162float(row[i]);
    if (v > best || (i == threadIdx.x && !(v < best))) { best = v; idx = i; }
  }
  auto better = [](float v, int64_t i, float bv, int64_t bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { best_s[threadIdx.x >> 5] = best; idx_s[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < kGlueThreads / 32 ? best_s[threadIdx.x] : -INFINITY;
    idx = threadIdx.x < kGlueThreads / 32 ? idx_s[threadIdx.x] : (int64_t)1 << 62;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if (threadIdx.x == 0) {
      tokens[b] = idx;
      if (history != nullptr && p + 1 >= 0 && p + 1 < hist_len) history[(int64_t)b * hist_len + p + 1] = idx;
      __threadfence();
      if (atomicAdd(ticket, 1) == (int)gridDim.x - 1) {  // every row has read the cursor
        *pos = p + 1;
        *ticket = 0;
      }
    }
  }
}

template <typename Kern, typename... Args>
int launch_glue(Kern kern, dim3 grid, dim3 block, cudaStream_t s, int pdl, const char* what, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  return LQ_OK;
}

}  // namespace
}  // namespace lq

extern "C" int lq_embed_gather(const void* table, const int64_t* tokens, void* hidden, int B, int H,
                               int64_t vocab, int pdl, void* stream) {
  using namespace lq;
  LQ_REQUIRE(B >= 0 && H > 0 && vocab > 0, LQ_ERR_ARG, "bad shape B=%d H=%d", B, H);
  if (B == 0) return LQ_OK;
  LQ_REQUIRE(table && tokens && hidden, LQ_ERR_ARG, "null tensor pointer");
  return launch_glue(embed_gather_kernel, dim3((unsigned)B), dim3(256), (cudaStream_t)stream, pdl, "lq_embed_gather",
                     (const __nv_bfloat16*)table, tokens, (__nv_bfloat16*)hidden, H, vocab);
}

extern "C" int lq_next_token(const void* logits, int64_t V, int64_t* tokens, int64_t* pos, int64_t* history,
                             int64_t hist_len, int* ticket, int B, int pdl, void* stream) {
  using namespace lq;
  LQ_REQUIRE(B >= 0 && V > 0, LQ_ERR_ARG, "bad shape B=%d V=%lld", B, (long long)V);
  if (B == 0) return LQ_OK;
  LQ_REQUIRE(logits && tokens && pos && ticket, LQ_ERR_ARG, "null tensor pointer");
  return launch_glue(next_token_kernel, dim3((unsigned)B), dim3(kGlueThreads), (cudaStream_t)stream, pdl,
                     "lq_next_token", (const __nv_bfloat16*)logits, V, tokens, pos, history, hist_len, ticket);
}
