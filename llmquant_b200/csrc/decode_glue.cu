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
#include "peer_sync.cuh"

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

// The same step under tensor parallelism, where every rank holds the logits of its slice of the
// vocabulary: each rank finds its local maximum and sends one 8-byte record per sequence --
// (global index, bf16 value, sequence tag) -- to every rank's exchange buffer with a single
// store, then waits (bounded) until the records of all ranks carry this step's tag and picks
// the largest value, the lowest index among equals; all ranks see the same records, so they
// pick the same token. Records alternate between two banks by step parity, so a rank that is
// already one step ahead never overwrites a record a slower rank still has to read. The step
// counter advances with the cursor.
__global__ void __launch_bounds__(kGlueThreads)
next_token_tp_kernel(const __nv_bfloat16* __restrict__ logits, int64_t V, int rank, int world,
                     const uint64_t* __restrict__ peers, int64_t record_off, int max_b,
                     int64_t* __restrict__ tokens, int64_t* pos, int64_t* __restrict__ history,
                     int64_t hist_len, int* ticket, uint32_t* step_ptr, long long wait_cycles,
                     int* error_word) {
  __shared__ float best_s[kGlueThreads / 32];
  __shared__ int64_t idx_s[kGlueThreads / 32];
  __shared__ uint64_t mine_s;
  __shared__ uint64_t rec_s[16];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int b = blockIdx.x;
  const int64_t p = *pos;
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(step_ptr);
  const __nv_bfloat16* row = logits + (int64_t)b * V;
  float best = -INFINITY;
  int64_t idx = 0;
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
  const uint32_t tag = step % 65535u + 1u;  // never zero, the state of a fresh buffer
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
      const uint64_t gidx = (uint64_t)((int64_t)rank * V + idx);
      const uint32_t bits = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(best));
      mine_s = (gidx << 32) | ((uint64_t)bits << 16) | tag;
    }
  }
  __syncthreads();
  // record (bank, source rank, sequence) of every rank's buffer
  const int64_t slot = ((int64_t)(step & 1u) * 16 + rank) * max_b + b;
  if ((int)threadIdx.x < world) {
    uint64_t* theirs = reinterpret_cast<uint64_t*>(peers[threadIdx.x] + record_off) + slot;
    st_relaxed_sys_u64(theirs, mine_s);
    const uint64_t* from = reinterpret_cast<const uint64_t*>(peers[rank] + record_off) +
                           ((int64_t)(step & 1u) * 16 + threadIdx.x) * max_b + b;
    uint64_t rec = ld_relaxed_sys_u64(from);
    if ((uint32_t)(rec & 0xFFFFu) != tag) {
      const long long t0 = clock64();
      for (;;) {
        rec = ld_relaxed_sys_u64(from);
        if ((uint32_t)(rec & 0xFFFFu) == tag) break;
        if (clock64() - t0 > wait_cycles) { atomicExch(error_word, 5); break; }
      }
    }
    rec_s[threadIdx.x] = rec;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bv = -INFINITY;
    int64_t bi = (int64_t)1 << 62;
    for (int r = 0; r < world; ++r) {
      const uint64_t rec = rec_s[r];
      const float v = __uint_as_float((uint32_t)((rec >> 16) & 0xFFFFu) << 16);
      const int64_t i = (int64_t)(rec >> 32);
      if (r == 0 || better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    tokens[b] = bi;
    if (history != nullptr && p + 1 >= 0 && p + 1 < hist_len) history[(int64_t)b * hist_len + p + 1] = bi;
    __threadfence();
    if (atomicAdd(ticket, 1) == (int)gridDim.x - 1) {  // every row has read the cursor and the step
      *pos = p + 1;
      *step_ptr = step + 1;
      *ticket = 0;
    }
  }
}

__device__ int g_glue_error = 0;

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

extern "C" int lq_glue_device_error(void) {
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_glue_error) != cudaSuccess) { cudaGetLastError(); return -1; }
  int value = 0;
  if (cudaMemcpy(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(ptr, 0, sizeof(int));
  return value;
}

extern "C" int lq_next_token_tp(const void* local_logits, int64_t V_local, int rank, int world,
                                const uint64_t* peer_bases_dev, int64_t record_offset_bytes, int max_batch,
                                int64_t* tokens, int64_t* pos, int64_t* history, int64_t hist_len,
                                int* ticket, uint32_t* step, int B, int64_t wait_cycles, int pdl,
                                void* stream) {
  using namespace lq;
  LQ_REQUIRE(B >= 0 && V_local > 0 && B <= max_batch, LQ_ERR_ARG, "bad shape B=%d V=%lld max_batch=%d", B,
             (long long)V_local, max_batch);
  LQ_REQUIRE(world >= 1 && world <= 16 && rank >= 0 && rank < world, LQ_ERR_ARG, "bad rank %d / world %d", rank, world);
  LQ_REQUIRE((int64_t)world * V_local < ((int64_t)1 << 32), LQ_ERR_ARG, "vocabulary too large for a 32-bit index");
  LQ_REQUIRE(record_offset_bytes % 8 == 0, LQ_ERR_ARG, "record offset must be 8-byte aligned");
  if (B == 0) return LQ_OK;
  LQ_REQUIRE(local_logits && peer_bases_dev && tokens && pos && ticket && step, LQ_ERR_ARG, "null tensor pointer");
  void* err_ptr = nullptr;
  if (cudaGetSymbolAddress(&err_ptr, g_glue_error) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "cannot resolve the device error word");
  }
  return launch_glue(next_token_tp_kernel, dim3((unsigned)B), dim3(kGlueThreads), (cudaStream_t)stream, pdl,
                     "lq_next_token_tp", (const __nv_bfloat16*)local_logits, V_local, rank, world,
                     peer_bases_dev, record_offset_bytes, max_batch, tokens, pos, history, hist_len, ticket,
                     step, (long long)(wait_cycles > 0 ? wait_cycles : kDefaultWaitCycles), (int*)err_ptr);
}
