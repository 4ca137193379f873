// Entry points of the streaming decode GEMV and the layout (repack / un-repack / dequant)
// kernels. The GEMV kernel template lives in gemv_stream.cuh and is instantiated per
// (code width, arithmetic variant) in gemv_stream_b*v*.cu.
#include "gemv_stream.cuh"

#include <cstdlib>

namespace lq {
namespace gemv {
int run_b4v1(GemvParams, const lq_gemv_args&, int, int, cudaStream_t);
int run_b4v2(GemvParams, const lq_gemv_args&, int, int, cudaStream_t);
int run_b4v3(GemvParams, const lq_gemv_args&, int, int, cudaStream_t);
int run_b8v1(GemvParams, const lq_gemv_args&, int, int, cudaStream_t);
int run_b8v2(GemvParams, const lq_gemv_args&, int, int, cudaStream_t);
bool mma_eligible(const lq_gemv_args& a);
int run_mma(const lq_gemv_args& a, int* error_word, unsigned long long* debug, cudaStream_t s);
int run_decode_gemm(const lq_gemv_args& a, cudaStream_t s);  // decode_gemm.cu
int run_b8v3(GemvParams, const lq_gemv_args&, int, int, cudaStream_t);
}  // namespace gemv

namespace {

// ------------------------------------------------------------------ layout kernels
// canonical [N, G, gs] -> codes [N, Kd] (strip = keep the first `span` codes of each group)
__global__ void repack_codes_kernel(const int8_t* __restrict__ canonical, uint8_t* __restrict__ codes,
                                    int64_t total_out, int groups, int gs, int span, int bits,
                                    int inverse) {
  // one thread per output byte of the forward direction
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int Kd = groups * span;
  const int per_byte = bits == 8 ? 1 : 2;
  for (int64_t i = i0; i < total_out; i += stride) {
    const int64_t e0 = i * per_byte;  // first stored element of this byte
    const int64_t n = e0 / Kd;
    const int kd = (int)(e0 % Kd);
    const int g = kd / span, j = kd % span;
    int8_t* src = const_cast<int8_t*>(canonical) + (n * groups + g) * gs + j;
    if (!inverse) {
      if (bits == 8) codes[i] = (uint8_t)src[0];
      else codes[i] = (uint8_t)(((src[0] + 8) & 0xF) | (((src[1] + 8) & 0xF) << 4));
    } else {
      if (bits == 8) src[0] = (int8_t)codes[i];
      else {
        src[0] = (int8_t)((int)(codes[i] & 0xF) - 8);
        src[1] = (int8_t)((int)(codes[i] >> 4) - 8);
      }
    }
  }
}

// wscale [scale_rows, G] <-> scale tiles [ceil(N/4), G, 4] (one entry per output row; rows that
// share a scale under out_group get copies of it)
__global__ void scale_tiles_kernel(const float* __restrict__ wscale, float* __restrict__ tiles,
                                   int N, int groups, int out_group, int NP, int inverse) {
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t total = (int64_t)NP * groups;
  for (int64_t i = i0; i < total; i += stride) {
    const int u = (int)(i % 4);
    const int g = (int)((i / 4) % groups);
    const int n = (int)(i / (4 * (int64_t)groups)) * 4 + u;
    const int64_t sr = out_group > 0 ? n / out_group : n;
    if (!inverse) tiles[i] = n < N ? wscale[sr * groups + g] : 0.f;
    else if (n < N && (out_group == 0 || n % out_group == 0))
      const_cast<float*>(wscale)[sr * groups + g] = tiles[i];
  }
}

// streaming layout -> dense [N, K] matrix of T (the real, unpadded reduction width)
template <typename T>
__global__ void dequant_stream_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales_t,
                                      T* __restrict__ out, int N, int K, int rowbytes, int span,
                                      int groups, int bits) {
  const int64_t total = (int64_t)N * K;
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = i0; i < total; i += stride) {
    const int n = (int)(i / K), k = (int)(i % K);
    int code;
    if (bits == 8) code = (int)(int8_t)codes[(int64_t)n * rowbytes + k];
    else {
      const uint8_t b = codes[(int64_t)n * rowbytes + (k >> 1)];
      code = (int)((k & 1) ? (b >> 4) : (b & 0xF)) - 8;
    }
    const float s = scales_t[((int64_t)(n / 4) * groups + k / span) * 4 + (n & 3)];
    out[i] = Conv<T>::from_f32(__fmul_rn((float)code, s));
  }
}

int layout_sizes(int N, int groups, int gs, int head_dim, int bits, int* Kd, int* span, int* NP) {
  LQ_REQUIRE(bits == 4 || bits == 8, LQ_ERR_ARG, "unsupported num_bits %d, expected 4 or 8", bits);
  LQ_REQUIRE(N >= 0 && groups >= 0 && gs > 0 && head_dim >= 0, LQ_ERR_ARG, "bad layout arguments");
  const int sp = (head_dim > 0 && head_dim < gs) ? head_dim : gs;
  const int epl = bits == 8 ? 16 : 32;
  LQ_REQUIRE(sp % epl == 0, LQ_ERR_UNSUPPORTED,
             "group span %d is not a multiple of %d codes; use the canonical-layout GEMV", sp, epl);
  *span = sp;
  *Kd = groups * sp;
  *NP = (N + 3) / 4 * 4;
  return LQ_OK;
}

int repack_common(const int8_t* canonical, const float* wscale, void* codes, float* tiles, int N,
                  int groups, int gs, int head_dim, int bits, int out_group, void* stream,
                  int inverse) {
  int Kd, span, NP;
  const int rc = layout_sizes(N, groups, gs, head_dim, bits, &Kd, &span, &NP);
  if (rc) return rc;
  LQ_REQUIRE(out_group >= 0, LQ_ERR_ARG, "out_group must be >= 0");
  if (N == 0 || groups == 0) return LQ_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = (int64_t)N * Kd * bits / 8;
  if (inverse && span < gs)
    cudaMemsetAsync(const_cast<int8_t*>(canonical), 0, (size_t)N * groups * gs, s);
  int64_t want = (total + 255) / 256;
  repack_codes_kernel<<<(unsigned)(want < 148 * 32 ? want : 148 * 32), 256, 0, s>>>(
      canonical, (uint8_t*)codes, total, groups, gs, span, bits, inverse);
  want = ((int64_t)groups * NP + 255) / 256;
  scale_tiles_kernel<<<(unsigned)(want < 148 * 8 ? want : 148 * 8), 256, 0, s>>>(
      wscale, tiles, N, groups, out_group, NP, inverse);
  return check_launch(inverse ? "lq_unrepack_stream" : "lq_repack_stream");
}

__device__ int g_gemv_error = 0;
#ifdef LQ_DIAGNOSTICS
unsigned long long* g_debug_timeline = nullptr;  // diagnostic builds: where kernels write their stamps
#else
constexpr unsigned long long* g_debug_timeline = nullptr;
#endif

int* error_word() {
  static thread_local int cached_dev = -1;
  static thread_local int* cached = nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev != cached_dev) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_gemv_error) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cached = (int*)ptr;
    cached_dev = dev;
  }
  return cached;
}

}  // namespace
}  // namespace lq

extern "C" int lq_stream_layout_sizes(int N, int groups, int group_size, int head_dim, int bits,
                                      int* Kd, int* span, int* NP) {
  return lq::layout_sizes(N, groups, group_size, head_dim, bits, Kd, span, NP);
}

extern "C" int lq_repack_stream(const int8_t* canonical, const float* wscale, void* codes,
                                float* scale_tiles, int N, int groups, int group_size, int head_dim,
                                int bits, int out_group, void* stream) {
  return lq::repack_common(canonical, wscale, codes, scale_tiles, N, groups, group_size, head_dim,
                           bits, out_group, stream, 0);
}

extern "C" int lq_unrepack_stream(const void* codes, const float* scale_tiles, int8_t* canonical,
                                  float* wscale, int N, int groups, int group_size, int head_dim,
                                  int bits, int out_group, void* stream) {
  return lq::repack_common(canonical, wscale, const_cast<void*>(codes), const_cast<float*>(scale_tiles),
                           N, groups, group_size, head_dim, bits, out_group, stream, 1);
}

extern "C" int lq_dequant_stream(const void* codes, const float* scale_tiles, void* out, int dtype,
                                 int N, int K, int Kd, int span, int bits, void* stream) {
  using namespace lq;
  LQ_REQUIRE(bits == 4 || bits == 8, LQ_ERR_ARG, "unsupported num_bits %d, expected 4 or 8", bits);
  LQ_REQUIRE(N >= 0 && K >= 0 && Kd >= K && span > 0 && Kd % span == 0, LQ_ERR_ARG,
             "bad shape N=%d K=%d Kd=%d", N, K, Kd);
  if (N == 0 || K == 0) return LQ_OK;
  const int64_t want = ((int64_t)N * K + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 64 ? want : 148 * 64);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    dequant_stream_kernel<T><<<grid, 256, 0, s>>>((const uint8_t*)codes, scale_tiles, (T*)out, N, K,
                                                  Kd * bits / 8, span, Kd / span, bits);
  });
  return check_launch("lq_dequant_stream");
}

#ifdef LQ_DIAGNOSTICS
// Diagnostic builds only: every GEMV CTA writes eight %globaltimer stamps of its phases to
// `device_buffer` (8 * grid uint64); NULL switches it off. Not part of the shipped ABI.
extern "C" void lq_gemv_set_timeline(void* device_buffer) {
  lq::g_debug_timeline = (unsigned long long*)device_buffer;
}
#endif

extern "C" int lq_gemv_device_error(void) {
  int* word = lq::error_word();
  if (word == nullptr) return -1;
  int value = 0;
  if (cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(word, 0, sizeof(int));
  return value;
}

extern "C" int lq_wq_gemv_fused(const lq_gemv_args* a, void* stream) {
  using namespace lq;
  using namespace lq::gemv;
  LQ_REQUIRE(a != nullptr, LQ_ERR_ARG, "null argument block");
  const int bits = a->bits, M = a->M, N = a->N, K = a->K, Kd = a->Kd;
  LQ_REQUIRE(bits == 4 || bits == 8, LQ_ERR_ARG, "unsupported num_bits %d, expected 4 or 8", bits);
  LQ_REQUIRE(M >= 0 && M <= (a->variant == 5 ? 64 : 8), LQ_ERR_ARG,
             "the decode GEMV takes at most 8 activation rows (variant 5: 64), got %d", M);
  LQ_REQUIRE(N >= 0 && K >= 0 && Kd >= K, LQ_ERR_ARG, "bad shape N=%d K=%d Kd=%d", N, K, Kd);
  LQ_REQUIRE(a->out_dtype == LQ_BF16 || a->out_dtype == LQ_F32, LQ_ERR_DTYPE, "out must be bfloat16 or float32");
  if (M == 0 || N == 0) return LQ_OK;
  const int epl = bits == 8 ? 16 : 32;
  LQ_REQUIRE(a->span > 0 && a->span % epl == 0 && Kd % a->span == 0, LQ_ERR_ARG,
             "group span %d must be a positive multiple of %d dividing Kd=%d", a->span, epl, Kd);
  const bool pushing = a->tp != nullptr && a->tp->mode == LQ_TP_PUSH;
  LQ_REQUIRE(a->x && a->codes && a->scale_tiles && (a->out || pushing), LQ_ERR_ARG, "null tensor pointer");
  LQ_REQUIRE(((uintptr_t)a->codes % 16) == 0 && ((uintptr_t)a->scale_tiles % 16) == 0, LQ_ERR_ARG,
             "codes and scales must be 16-byte aligned");
  LQ_REQUIRE(a->ldx >= K, LQ_ERR_ARG, "x row stride %d is shorter than K=%d", a->ldx, K);
  LQ_REQUIRE(a->epilogue == 0 || a->epilogue == 1, LQ_ERR_ARG, "unknown epilogue %d", a->epilogue);
  if (a->epilogue == 1)
    LQ_REQUIRE(N % 4 == 0 && a->bias == nullptr && a->residual == nullptr, LQ_ERR_ARG,
               "the silu-mul epilogue needs N %% 4 == 0 and no bias / residual");
  const lq_gemv_tp* tp = a->tp;
  if (tp != nullptr && tp->mode != 0) {
    LQ_REQUIRE(tp->mode == LQ_TP_PUSH || tp->mode == LQ_TP_SUM, LQ_ERR_ARG, "unknown tensor-parallel mode %d", tp->mode);
    LQ_REQUIRE(tp->world >= 1 && tp->world <= 16 && tp->rank >= 0 && tp->rank < tp->world, LQ_ERR_ARG,
               "bad rank %d / world %d", tp->rank, tp->world);
    LQ_REQUIRE(a->variant == 0 || a->variant == 2, LQ_ERR_UNSUPPORTED,
               "the tensor-parallel coupling is built into the streaming kernel's default arithmetic (variant 2)");
    LQ_REQUIRE(M <= (bits == 4 ? 2 : 4), LQ_ERR_UNSUPPORTED,
               "the tensor-parallel coupling takes the rows of one pass (%d given)", M);
    if (tp->mode == LQ_TP_PUSH) {
      LQ_REQUIRE(a->epilogue == 0 && a->residual == nullptr && N % 4 == 0 && M * tp->world <= 32, LQ_ERR_ARG,
                 "a pushing GEMV needs epilogue 0, no residual, N %% 4 == 0 and M * world <= 32");
      LQ_REQUIRE(tp->peers != nullptr && tp->data_offset % 16 == 0, LQ_ERR_ARG,
                 "peer table missing or exchange offset misaligned");
    } else {
      LQ_REQUIRE(K % (bits == 8 ? 16 : 32) == 0 && a->ldx == K, LQ_ERR_ARG,
                 "a summing GEMV needs dense rows of a whole number of 16-byte code pieces");
      LQ_REQUIRE(tp->parts && tp->residual, LQ_ERR_ARG, "null tensor-parallel pointer");
      LQ_REQUIRE(((uintptr_t)tp->parts % 16) == 0 && ((uintptr_t)tp->residual % 16) == 0 && ((uintptr_t)a->x % 16) == 0,
                 LQ_ERR_ARG, "partials, residual and x must be 16-byte aligned");
    }
  } else {
    tp = nullptr;
  }
  int variant = a->variant == 0 ? 2 : a->variant;
  // Default choice by measurement: the SIMT kernel keeps 2 (int4) or 4 (int8) activation rows in
  // registers per pass over the weight; from the row count where it would need a second pass the
  // tensor-core kernel, which takes 8 rows in one pass, is the faster one (B200, Llama-3-8B
  // shapes, 8 rows: gate|up 44 vs 96 us, lm_head 185 vs 303 us).
  if (a->variant == 0 && tp == nullptr && ((bits == 4 && M >= 3) || M >= 5) && mma_eligible(*a)) variant = 4;
  LQ_REQUIRE(variant >= 1 && variant <= 5, LQ_ERR_ARG, "unknown arithmetic variant %d", variant);
  LQ_REQUIRE(a->ldo == 0 || a->ldo >= (a->epilogue == 1 ? N / 2 : N), LQ_ERR_ARG, "ldo=%d is shorter than a row", a->ldo);
  LQ_REQUIRE(a->ldo == 0 || tp == nullptr, LQ_ERR_ARG, "an output row stride and the tensor-parallel coupling exclude each other");
  if (variant == 5) {
    LQ_REQUIRE(tp == nullptr, LQ_ERR_UNSUPPORTED, "the decode GEMM has no tensor-parallel coupling");
    return run_decode_gemm(*a, (cudaStream_t)stream);
  }
  if (variant == 4) {
    LQ_REQUIRE(mma_eligible(*a), LQ_ERR_UNSUPPORTED,
               "the tensor-core GEMV needs scale groups of 128 stored codes, activation planes within 64 KB and "
               "five row stages within 200 KB (span=%d, M=%d, Kd=%d, bits=%d)", a->span, M, Kd, bits);
    int* word = error_word();
    LQ_REQUIRE(word != nullptr, LQ_ERR_LAUNCH, "cannot resolve the device error word");
    return run_mma(*a, word, g_debug_timeline, (cudaStream_t)stream);
  }

  GemvParams p;
  p.ldx = a->ldx; p.codes = (const uint8_t*)a->codes; p.scales = a->scale_tiles;
  p.bias = (const __nv_bfloat16*)a->bias;
  p.out_f32 = a->out_dtype == LQ_F32;
  p.ldo = a->ldo > 0 ? a->ldo : (a->epilogue == 1 ? N / 2 : N);
  p.N = N; p.K = K; p.Kd = Kd; p.rowbytes = Kd * bits / 8; p.span = a->span;
  p.groups = Kd / a->span;
  p.norm_weight = a->norm_weight; p.norm_eps = a->norm_eps; p.pdl = a->pdl;
  p.error_word = error_word();
  p.debug = g_debug_timeline;
  p.tp_mode = 0; p.tp_world = 0; p.tp_rank = 0; p.tp_peers = nullptr; p.tp_data_off = 0;
  p.tp_parts = nullptr; p.tp_residual = nullptr;
  p.tp_wait = kDefaultWaitCycles;
  if (tp != nullptr) {
    p.tp_mode = tp->mode; p.tp_world = tp->world; p.tp_rank = tp->rank; p.tp_peers = tp->peers;
    p.tp_data_off = tp->data_offset; p.tp_parts = tp->parts;
    p.tp_residual = (__nv_bfloat16*)tp->residual;
    if (tp->wait_cycles > 0) p.tp_wait = tp->wait_cycles;
  }
  LQ_REQUIRE(p.error_word != nullptr, LQ_ERR_LAUNCH, "cannot resolve the device error word");
  p.S = (p.rowbytes + 511) / 512;
  int spw = 1;
  while (spw <= 4 && (p.S + spw - 1) / spw > kMaxWarps) spw *= 2;
#ifdef LQ_DIAGNOSTICS
  if (const char* e = getenv("LQ_X_SPW")) {  // diagnostic builds: column chunks per lane
    const int want = atoi(e);
    if ((want == 2 || want == 4) && want > spw && M <= (bits == 8 && want == 2 ? 2 : 1) && !(want == 4 && a->epilogue == 1))
      spw = want;
  }
#endif
  LQ_REQUIRE(spw <= 4, LQ_ERR_UNSUPPORTED, "reduction axis too long for the streaming GEMV (Kd=%d)", Kd);
  LQ_REQUIRE(!(spw == 4 && a->epilogue == 1), LQ_ERR_UNSUPPORTED, "reduction axis too long for the fused epilogue");
  p.KW = (p.S + spw - 1) / spw;
  p.nbatch = (N + kU - 1) / kU;
  p.tile_bytes = kU * p.rowbytes;
  p.scale_bytes = p.groups * kU * (int)sizeof(float);
  p.stage_bytes = (p.tile_bytes + p.scale_bytes + 127) / 128 * 128;
  // Ring depth: enough CTAs per SM for ~20 consumer warps (the dot products are dependent
  // chains and need warps to hide their latency), all rings together within ~112 KB per SM so
  // that the next kernel's CTAs can become resident early (see launch_one).
  const int want_ctas = (kRingWarps + p.KW - 1) / p.KW;
  int stages = (kRingKb * 1024) / (want_ctas * p.stage_bytes);
#ifdef LQ_DIAGNOSTICS
  if (const char* e = getenv("LQ_X_STAGES")) stages = atoi(e);
#endif
  stages = stages < 2 ? 2 : (stages > kMaxStages ? kMaxStages : stages);
  LQ_REQUIRE((size_t)stages * p.stage_bytes <= 200 * 1024, LQ_ERR_UNSUPPORTED,
             "row tile of %d bytes does not fit the shared-memory ring", p.stage_bytes);
  p.stages = stages;
  // consumers + producer, and with more than one consumer warp the finisher
  const int threads = (p.KW + (p.KW > 1 ? 2 : 1)) * 32;
  cudaStream_t s = (cudaStream_t)stream;
  if (bits == 8) {
    if (variant == 1) return run_b8v1(p, *a, spw, threads, s);
    if (variant == 2) return run_b8v2(p, *a, spw, threads, s);
    return run_b8v3(p, *a, spw, threads, s);
  }
  if (variant == 1) return run_b4v1(p, *a, spw, threads, s);
  if (variant == 2) return run_b4v2(p, *a, spw, threads, s);
  return run_b4v3(p, *a, spw, threads, s);
}

extern "C" int lq_wq_gemv_stream(const void* x, int ldx, const void* codes, const float* scale_tiles,
                                 const void* bias, const void* residual, void* out, int out_dtype,
                                 int M, int N, int K, int Kd, int span, int bits, int variant,
                                 void* stream) {
  lq_gemv_args a = {};
  a.x = x; a.ldx = ldx; a.codes = codes; a.scale_tiles = scale_tiles; a.bias = bias;
  a.residual = residual; a.out = out; a.out_dtype = out_dtype; a.M = M; a.N = N; a.K = K;
  a.Kd = Kd; a.span = span; a.bits = bits; a.variant = variant;
  return lq_wq_gemv_fused(&a, stream);
}
