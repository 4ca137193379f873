// One-shot all-reduce of the row-parallel partial outputs, fused with the residual add.
//
// Tensor-parallel decode sums a [batch, hidden] fp32 partial per rank after o_proj and after
// down_proj: 16 KB at batch 1, 64 times per token. At that size a collective is pure
// latency, so instead of a library call every rank runs one small kernel: the GEMV before it
// has written the rank's partial into a buffer that all peers have mapped (NVLink peer
// memory); the kernel publishes a sequence number to every peer's flag array, waits until
// every peer's number has arrived (bounded), then reads all partials with ordinary loads,
// adds them in rank order -- the same order on every rank, so all ranks get identical bits --
// and applies the residual with the roundings of the single-GPU epilogue. Two buffer slots
// alternate so that a fast rank can already write its next partial while a slow one is still
// reading the previous one. No bulk / TMA copies touch peer memory, only plain loads and
// stores. The reference is single-GPU and has no counterpart.
#include "common.cuh"
#include "peer_sync.cuh"

namespace lq {
namespace {

constexpr int kArThreads = 1024;
constexpr int kMaxWorld = 16;

// peers[r]: base of rank r's shared buffer: float data[2][slot_floats], then uint32
// flags[2][kMaxWorld] at byte offset flag_off. n is a multiple of 4.
__global__ void __launch_bounds__(kArThreads)
allreduce_residual_kernel(const uint64_t* __restrict__ peers, int rank, int world, int slot,
                          int64_t slot_floats, int64_t flag_off, uint32_t* seq_counter,
                          const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                          int n, long long wait_cycles, int* error_word) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ uint64_t base_s[kMaxWorld];
  __shared__ int timed_out;
  const int tid = threadIdx.x;
  const uint32_t seq = *seq_counter + 1;
  if (tid < world) base_s[tid] = peers[tid];
  if (tid == 0) timed_out = 0;
  __syncthreads();
  __threadfence_system();
  if (tid < world) {
    uint32_t* theirs = reinterpret_cast<uint32_t*>(base_s[tid] + flag_off) + slot * kMaxWorld + rank;
    st_release_sys(theirs, seq);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(base_s[rank] + flag_off) + slot * kMaxWorld + tid;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) != seq) {
      if (clock64() - t0 > wait_cycles) {  // a peer never arrived
        timed_out = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (timed_out) {
    if (tid == 0) atomicExch(error_word, 1);
  }
  for (int i = tid * 4; i < n; i += kArThreads * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < world; r0 += 4) {  // four peer loads in flight, added in rank order
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (r0 + j < world)
          v[j] = ld_peer_f4(reinterpret_cast<const float4*>(
              reinterpret_cast<const float*>(base_s[r0 + j]) + slot * slot_floats + i));
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (r0 + j < world) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
    }
    const float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float y = __bfloat162float(__float2bfloat16_rn(a[j]));
      if (residual != nullptr) y += __bfloat162float(residual[i + j]);
      out[i + j] = __float2bfloat16_rn(y);
    }
  }
  __syncthreads();
  if (tid == 0) *seq_counter = seq;
}

__device__ int g_allreduce_error = 0;

}  // namespace
}  // namespace lq

extern "C" int lq_allreduce_max_world(void) { return lq::kMaxWorld; }

extern "C" int lq_allreduce_device_error(void) {
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_allreduce_error) != cudaSuccess) { cudaGetLastError(); return -1; }
  int value = 0;
  if (cudaMemcpy(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(ptr, 0, sizeof(int));
  return value;
}

extern "C" int lq_allreduce_residual(const uint64_t* peer_bases_dev, int rank, int world, int slot,
                                     int64_t slot_floats, int64_t flag_offset_bytes,
                                     uint32_t* seq_counter_dev, const void* residual, void* out, int n,
                                     int64_t wait_cycles, int pdl, void* stream) {
  using namespace lq;
  LQ_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, LQ_ERR_ARG,
             "bad rank %d / world %d", rank, world);
  LQ_REQUIRE(slot == 0 || slot == 1, LQ_ERR_ARG, "slot must be 0 or 1");
  LQ_REQUIRE(n > 0 && n % 4 == 0 && n <= slot_floats, LQ_ERR_ARG,
             "n=%d must be a positive multiple of 4 within the slot", n);
  LQ_REQUIRE(flag_offset_bytes % 16 == 0 && flag_offset_bytes >= 2 * slot_floats * 4, LQ_ERR_ARG,
             "flag array must follow the two data slots");
  LQ_REQUIRE(peer_bases_dev && seq_counter_dev && out, LQ_ERR_ARG, "null pointer");
  void* err_ptr = nullptr;
  if (cudaGetSymbolAddress(&err_ptr, g_allreduce_error) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "cannot resolve the device error word");
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, allreduce_residual_kernel, peer_bases_dev, rank, world, slot,
                                     slot_floats, flag_offset_bytes, seq_counter_dev,
                                     (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, n,
                                     (long long)(wait_cycles > 0 ? wait_cycles : kDefaultWaitCycles),
                                     (int*)err_ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "lq_allreduce_residual: %s", cudaGetErrorString(e));
  }
  return LQ_OK;
}
