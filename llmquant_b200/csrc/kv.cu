// Quantized KV cache: quantize-on-write, dequantize, fused RoPE + write, and a decode
// attention that reads the int8 codes directly.
//
// Storage (per layer): codes [B, Hkv, Tmax, D] int8 and scales [B, Hkv, Tmax, NG] fp32 with
// NG = ceil(D / 128): one symmetric abs-max scale per token, per KV head, per 128-wide
// group of head_dim -- the grouping of the reference's FakeQuantCache
// (llmquant/quantizers/fake.py:46-55), which keeps the dequantized values in bf16; here the
// integer codes are what lives in HBM (half the bytes of bf16). code * scale rounded to the
// model dtype equals the value the reference stores, except that an integer cannot carry
// the sign of a zero.
//
// Positions and lengths can come from device memory (an int64 counter), so every kernel is
// CUDA-graph capturable with a moving write cursor.
#include <type_traits>

#include "common.cuh"

#include <map>
#include <mutex>

namespace lq {
namespace {

constexpr int kGroup = 128;

__device__ __forceinline__ int64_t read_pos(const int64_t* dev, int64_t host) {
  return dev != nullptr ? *dev : host;
}

// ---------------------------------------------------------------- quantize-on-write
// One warp per (b, h, t) row of new K and of new V. Source rows are strided (transformers
// hands over a transposed view); head_dim is contiguous.
template <typename T>
__global__ void __launch_bounds__(256)
kv_write_kernel(const T* __restrict__ k, const T* __restrict__ v, int64_t ksb, int64_t ksh,
                int64_t kst, int64_t vsb, int64_t vsh, int64_t vst, int8_t* __restrict__ kc,
                int8_t* __restrict__ vc, float* __restrict__ ks, float* __restrict__ vs, int B, int H,
                int Tn, int D, int Tmax, const int64_t* pos_dev, int64_t pos_host, float qmin,
                float qmax) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t rows = (int64_t)B * H * Tn * 2;
  if (row >= rows) return;
  const bool is_v = row >= rows / 2;
  const int64_t r = is_v ? row - rows / 2 : row;
  const int t = (int)(r % Tn);
  const int h = (int)((r / Tn) % H);
  const int b = (int)(r / ((int64_t)Tn * H));
  const int64_t pos = read_pos(pos_dev, pos_host) + t;
  if (pos < 0 || pos >= Tmax) return;  // never write outside the cache
  const T* src = is_v ? v + b * vsb + h * vsh + t * vst : k + b * ksb + h * ksh + t * kst;
  int8_t* dst = (is_v ? vc : kc) + (((int64_t)b * H + h) * Tmax + pos) * D;
  const int ng = (D + kGroup - 1) / kGroup;
  float* sdst = (is_v ? vs : ks) + (((int64_t)b * H + h) * Tmax + pos) * ng;
  for (int g = 0; g < ng; ++g) {
    const int lo = g * kGroup, hi = min(D, lo + kGroup);
    float amax = 0.f;
    for (int i = lo + lane; i < hi; i += 32) amax = fmaxf(amax, fabsf(Conv<T>::to_f32(src[i])));
    amax = warp_max(amax);
    const float scale = scale_of(amax, qmax);
    if (lane == 0) sdst[g] = scale;
    for (int i = lo + lane; i < hi; i += 32)
      dst[i] = (int8_t)code_of(Conv<T>::to_f32(src[i]), scale, qmin, qmax);
  }
}

// ---------------------------------------------------------------- dequantize
template <typename T>
__global__ void kv_dequant_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales,
                                  T* __restrict__ out, int64_t BH, int T_len, int D, int Tmax) {
  const int ng = (D + kGroup - 1) / kGroup;
  const int64_t total = BH * T_len * D;
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = i0; i < total; i += stride) {
    const int d = (int)(i % D);
    const int64_t t = (i / D) % T_len;
    const int64_t bh = i / ((int64_t)D * T_len);
    const int64_t row = bh * Tmax + t;
    out[i] = Conv<T>::from_f32(__fmul_rn((float)codes[row * D + d], scales[row * ng + d / kGroup]));
  }
}

// ---------------------------------------------------------------- fused RoPE + write
// Input: one decode token per sequence, the fused q|k|v projection output [B, (Hq+2Hkv)*D]
// bf16. A warp owns one head: lanes hold (i, i + D/2) pairs, so rotate_half needs no
// exchange. RoPE follows the bf16 arithmetic of transformers' apply_rotary_pos_emb
// (q*cos and rotate_half(q)*sin each rounded to bf16, then their sum). q heads go to q_out
// [B, Hq, D] bf16; k (rotated) and v heads are quantized into the cache at the cursor.
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ cos_t,
                     const __nv_bfloat16* __restrict__ sin_t, __nv_bfloat16* __restrict__ q_out,
                     int8_t* __restrict__ kc, int8_t* __restrict__ vc, float* __restrict__ ks,
                     float* __restrict__ vs, int B, int Hq, int Hkv, int D, int Tmax, int table_len,
                     const int64_t* pos_dev, int64_t pos_host, float qmin, float qmax) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (int64_t)B * heads) return;
  const int b = (int)(w / heads), head = (int)(w % heads);
  const int64_t pos = read_pos(pos_dev, pos_host);
  if (pos < 0 || pos >= Tmax || pos >= table_len) return;
  const __nv_bfloat16* src = qkv + ((int64_t)b * heads + head) * D;
  const int half = D / 2;
  const bool is_v = head >= Hq + Hkv;
  constexpr int kMaxPairs = 4;  // D <= 256
  float lo[kMaxPairs], hi[kMaxPairs];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxPairs; ++j) {
    const int i = lane + 32 * j;
    lo[j] = hi[j] = 0.f;
    if (i < half) {
      float a = __bfloat162float(src[i]), c = __bfloat162float(src[i + half]);
      if (!is_v) {
        const float c0 = __bfloat162float(cos_t[pos * D + i]), s0 = __bfloat162float(sin_t[pos * D + i]);
        const float c1 = __bfloat162float(cos_t[pos * D + i + half]);
        const float s1 = __bfloat162float(sin_t[pos * D + i + half]);
        auto r = [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); };
        const float na = r(r(a * c0) + r(-c * s0));
        const float nc = r(r(c * c1) + r(a * s1));
        a = na; c = nc;
      }
      lo[j] = a; hi[j] = c;
      amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(c)));
    }
  }
  if (head < Hq) {
    __nv_bfloat16* dst = q_out + ((int64_t)b * Hq + head) * D;
#pragma unroll
    for (int j = 0; j < kMaxPairs; ++j) {
      const int i = lane + 32 * j;
      if (i < half) { dst[i] = __float2bfloat16_rn(lo[j]); dst[i + half] = __float2bfloat16_rn(hi[j]); }
    }
    return;
  }
  const int kvh = is_v ? head - Hq - Hkv : head - Hq;
  const int64_t row = ((int64_t)b * Hkv + kvh) * Tmax + pos;
  int8_t* dst = (is_v ? vc : kc) + row * D;
  const int ng = (D + kGroup - 1) / kGroup;
  if (ng == 1) {
    amax = warp_max(amax);
    const float scale = scale_of(amax, qmax);
    if (lane == 0) (is_v ? vs : ks)[row] = scale;
#pragma unroll
    for (int j = 0; j < kMaxPairs; ++j) {
      const int i = lane + 32 * j;
      if (i < half) {
        dst[i] = (int8_t)code_of(lo[j], scale, qmin, qmax);
        dst[i + half] = (int8_t)code_of(hi[j], scale, qmin, qmax);
      }
    }
  } else {
    // head_dim 256: the low halves form group 0 and the high halves group 1
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPairs; ++j) { a0 = fmaxf(a0, fabsf(lo[j])); a1 = fmaxf(a1, fabsf(hi[j])); }
    a0 = warp_max(a0); a1 = warp_max(a1);
    const float s0 = scale_of(a0, qmax), s1 = scale_of(a1, qmax);
    if (lane == 0) { (is_v ? vs : ks)[row * 2] = s0; (is_v ? vs : ks)[row * 2 + 1] = s1; }
#pragma unroll
    for (int j = 0; j < kMaxPairs; ++j) {
      const int i = lane + 32 * j;
      if (i < half) {
        dst[i] = (int8_t)code_of(lo[j], s0, qmin, qmax);
        dst[i + half] = (int8_t)code_of(hi[j], s1, qmin, qmax);
      }
    }
  }
}

// ---------------------------------------------------------------- decode attention
// One query token per sequence. grid (NS, Hkv, B): a CTA owns one KV head of one sequence
// and one of NS slices of the cached tokens, and serves the G query heads that share the KV
// head from a single pass over the codes. Inside a warp, 8 lanes split head_dim and 4 such
// lane groups take 4 consecutive tokens, so a warp instruction reads 4 whole rows. Each lane
// group keeps an online-softmax state per query head; groups and warps merge through shared
// memory, slices through the scratch arrays and the combine kernel below.
template <int D, int G>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const int8_t* __restrict__ kc,
                   const int8_t* __restrict__ vc, const float* __restrict__ ks,
                   const float* __restrict__ vs, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int Hq, int Hkv, int Tmax, const int64_t* len_dev,
                   int64_t len_host, int len_add, float scaling) {
  constexpr int DPL = D / 8;        // dims per lane
  constexpr int NGRP = 16;          // lane groups per CTA (4 warps x 4)
  __shared__ float q_s[G][D];
  __shared__ float m_s[NGRP][G], l_s[NGRP][G];
  __shared__ float o_s[NGRP / 2][G][D];  // merged in two halves to stay under 48 KB

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int ns = gridDim.x, split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, grp = warp * 4 + (lane >> 3);
  int64_t len = read_pos(len_dev, len_host) + len_add;
  if (len > Tmax) len = Tmax;
  if (len < 0) len = 0;
  const int per = (int)((len + ns - 1) / ns);
  const int t_lo = split * per;
  const int t_hi = (int)min((int64_t)(t_lo + per), len);

  for (int i = threadIdx.x; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    q_s[g][d] = __bfloat162float(q[((int64_t)b * Hq + kvh * G + g) * D + d]) * scaling;
  }
  __syncthreads();

  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }
  const int64_t head_row = ((int64_t)b * Hkv + kvh) * Tmax;
  // The trip count is the same for every lane of the warp (the shuffles below name all 32
  // lanes); a lane group whose token falls past the slice computes on zeros and is masked.
  for (int t0 = t_lo; t0 < t_hi; t0 += NGRP) {
    const int t = t0 + grp;
    const bool valid = t < t_hi;
    const int64_t row = head_row + (valid ? t : t_lo);
    int8_t kb[DPL], vb[DPL];
    if (DPL == 16) {
      *reinterpret_cast<uint4*>(kb) = *reinterpret_cast<const uint4*>(kc + row * D + sub * DPL);
      *reinterpret_cast<uint4*>(vb) = *reinterpret_cast<const uint4*>(vc + row * D + sub * DPL);
    } else {
      *reinterpret_cast<uint2*>(kb) = *reinterpret_cast<const uint2*>(kc + row * D + sub * DPL);
      *reinterpret_cast<uint2*>(vb) = *reinterpret_cast<const uint2*>(vc + row * D + sub * DPL);
    }
    const float sk = ks[row], sv = vs[row];
    float kf[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) kf[i] = (float)kb[i];
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) d = fmaf(q_s[g][sub * DPL + i], kf[i], d);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      s[g] = d * sk;
    }
    if (valid) {
      float vf[DPL];
#pragma unroll
      for (int i = 0; i < DPL; ++i) vf[i] = (float)vb[i] * sv;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (s[g] > m[g]) {  // rare after the first tokens: rescale only when the maximum moves
          const float corr = __expf(m[g] - s[g]);
          l[g] *= corr;
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[g][i] *= corr;
          m[g] = s[g];
        }
        const float p = __expf(s[g] - m[g]);
        l[g] += p;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i]);
      }
    }
  }

  // ---- merge the 16 lane groups of the CTA
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) { m_s[grp][g] = m[g]; l_s[grp][g] = l[g]; }
  }
  __syncthreads();
  float mt[G], w[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mm = -INFINITY;
    for (int r = 0; r < NGRP; ++r) mm = fmaxf(mm, m_s[r][g]);
    mt[g] = mm;
    w[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mm);
  }
  float* po = part_o + (((int64_t)b * Hq + kvh * G) * ns + split) * D;   // [g][ns][D] strides below
  for (int halfsel = 0; halfsel < 2; ++halfsel) {
    const bool mine = (grp / (NGRP / 2)) == halfsel;
    if (mine) {
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < DPL; ++i) o_s[grp % (NGRP / 2)][g][sub * DPL + i] = acc[g][i] * w[g];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += 128) {
      const int g = i / D, d = i % D;
      float t = 0.f;
      for (int r = 0; r < NGRP / 2; ++r) t += o_s[r][g][d];
      float* dst = po + (int64_t)g * ns * D + d;
      if (halfsel == 0) *dst = t; else *dst += t;
    }
    __syncthreads();
  }
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    float mm = -INFINITY;
    for (int r = 0; r < NGRP; ++r) mm = fmaxf(mm, m_s[r][g]);
    float lt = 0.f;
    for (int r = 0; r < NGRP; ++r)
      lt += (m_s[r][g] == -INFINITY) ? 0.f : l_s[r][g] * __expf(m_s[r][g] - mm);
    float* ml = part_ml + (((int64_t)b * Hq + kvh * G + g) * ns + split) * 2;
    ml[0] = mm; ml[1] = lt;
  }
}

// grid (Hq, B), D threads: merge the NS slices of one query head and write bf16.
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int Hq, int D, int ns) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int64_t base = ((int64_t)b * Hq + h) * ns;
  float mm = -INFINITY;
  for (int s = 0; s < ns; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float lt = 0.f, o = 0.f;
  for (int s = 0; s < ns; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    lt += part_ml[(base + s) * 2 + 1] * w;
    if (d < D) o += part_o[(base + s) * D + d] * w;
  }
  if (d < D) out[((int64_t)b * Hq + h) * D + d] = __float2bfloat16_rn(lt > 0.f ? o / lt : 0.f);
}

template <typename Kern, typename... Args>
int launch_pdl(Kern kern, dim3 grid, dim3 block, cudaStream_t s, int pdl, const char* what, Args... args) {
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

template <typename Kern, typename... Args>
int launch_pdl_smem(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t s, int pdl,
                    const char* what, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
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

// Whether clusters of `cluster_x` CTAs of this kernel can become resident on the current device
// (sizes above 8 need the non-portable opt-in first). Asked once per (kernel, device, size).
template <typename Kern>
bool cluster_fits(Kern kern, int cluster_x, dim3 grid, dim3 block, size_t smem) {
  struct Key { const void* k; int dev, cx; bool operator<(const Key& o) const {
    return k != o.k ? k < o.k : (dev != o.dev ? dev < o.dev : cx < o.cx); } };
  static std::mutex mu;
  static std::map<Key, bool> known;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return false; }
  std::lock_guard<std::mutex> lock(mu);
  const Key key{reinterpret_cast<const void*>(kern), dev, cluster_x};
  auto it = known.find(key);
  if (it != known.end()) return it->second;
  bool ok = true;
  if (cluster_x > 8 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    ok = false;
  }
  if (ok) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    ok = n >= 1;
  }
  known[key] = ok;
  return ok;
}

template <typename Kern, typename... Args>
int launch_cluster(Kern kern, dim3 grid, dim3 block, size_t smem, int cluster_x, cudaStream_t s, int pdl,
                   const char* what, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  return LQ_OK;
}

}  // namespace
}  // namespace lq

extern "C" int lq_kv_write(const void* k, const void* v, const int64_t* k_strides,
                           const int64_t* v_strides, int dtype, int8_t* k_codes, int8_t* v_codes,
                           float* k_scales, float* v_scales, int B, int H, int T_new, int D, int Tmax,
                           const int64_t* pos_dev, int64_t pos, int num_bits, void* stream) {
  using namespace lq;
  LQ_REQUIRE(num_bits >= 2 && num_bits <= 8, LQ_ERR_ARG, "num_bits must be in [2, 8], got %d", num_bits);
  LQ_REQUIRE(B >= 0 && H >= 0 && T_new >= 0 && D > 0 && Tmax > 0, LQ_ERR_ARG, "bad cache shape");
  if (B == 0 || H == 0 || T_new == 0) return LQ_OK;
  LQ_REQUIRE(k && v && k_strides && v_strides && k_codes && v_codes && k_scales && v_scales,
             LQ_ERR_ARG, "null tensor pointer");
  LQ_REQUIRE(pos_dev != nullptr || (pos >= 0 && pos + T_new <= Tmax), LQ_ERR_ARG,
             "write of %d tokens at %lld does not fit a cache of %d", T_new, (long long)pos, Tmax);
  const float qmax = (float)((1 << (num_bits - 1)) - 1);
  const int64_t rows = (int64_t)B * H * T_new * 2;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    kv_write_kernel<T><<<grid, 256, 0, s>>>((const T*)k, (const T*)v, k_strides[0], k_strides[1],
                                            k_strides[2], v_strides[0], v_strides[1], v_strides[2],
                                            k_codes, v_codes, k_scales, v_scales, B, H, T_new, D, Tmax,
                                            pos_dev, pos, -qmax - 1.f, qmax);
  });
  return check_launch("lq_kv_write");
}

extern "C" int lq_kv_dequant(const int8_t* codes, const float* scales, void* out, int dtype, int B,
                             int H, int T_len, int D, int Tmax, void* stream) {
  using namespace lq;
  LQ_REQUIRE(B >= 0 && H >= 0 && T_len >= 0 && T_len <= Tmax && D > 0, LQ_ERR_ARG, "bad cache shape");
  const int64_t total = (int64_t)B * H * T_len * D;
  if (total == 0) return LQ_OK;
  const int64_t want = (total + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 32 ? want : 148 * 32);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    kv_dequant_kernel<T><<<grid, 256, 0, s>>>(codes, scales, (T*)out, (int64_t)B * H, T_len, D, Tmax);
  });
  return check_launch("lq_kv_dequant");
}

extern "C" int lq_rope_kv_write(const void* qkv, const void* cos_table, const void* sin_table,
                                void* q_out, int8_t* k_codes, int8_t* v_codes, float* k_scales,
                                float* v_scales, int B, int Hq, int Hkv, int D, int Tmax,
                                int table_len, const int64_t* pos_dev, int64_t pos, int num_bits,
                                int pdl, void* stream) {
  using namespace lq;
  LQ_REQUIRE(num_bits >= 2 && num_bits <= 8, LQ_ERR_ARG, "num_bits must be in [2, 8], got %d", num_bits);
  LQ_REQUIRE(D % 64 == 0 && D <= 256, LQ_ERR_UNSUPPORTED, "head_dim %d: the fused RoPE/KV write needs a multiple of 64 up to 256", D);
  LQ_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Tmax > 0, LQ_ERR_ARG, "bad shape");
  LQ_REQUIRE(qkv && cos_table && sin_table && q_out && k_codes && v_codes && k_scales && v_scales,
             LQ_ERR_ARG, "null tensor pointer");
  const float qmax = (float)((1 << (num_bits - 1)) - 1);
  const int64_t warps = (int64_t)B * (Hq + 2 * Hkv);
  return launch_pdl(rope_kv_write_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256),
                    (cudaStream_t)stream, pdl, "lq_rope_kv_write",
                    (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)cos_table,
                    (const __nv_bfloat16*)sin_table, (__nv_bfloat16*)q_out, k_codes, v_codes,
                    k_scales, v_scales, B, Hq, Hkv, D, Tmax, table_len, pos_dev, pos, -qmax - 1.f, qmax);
}

extern "C" int64_t lq_attn_decode_scratch_bytes(int B, int Hq, int D, int splits) {
  return (int64_t)B * Hq * splits * (D + 2) * (int64_t)sizeof(float);
}

extern "C" int lq_attn_decode_kv_i8(const void* q, const int8_t* k_codes, const int8_t* v_codes,
                                    const float* k_scales, const float* v_scales, void* out,
                                    void* scratch, int B, int Hq, int Hkv, int D, int Tmax,
                                    const int64_t* len_dev, int64_t len, int len_add, float scaling,
                                    int splits, int pdl, void* stream) {
  using namespace lq;
  LQ_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, LQ_ERR_ARG, "bad head counts %d / %d", Hq, Hkv);
  LQ_REQUIRE(splits >= 1 && splits <= 1024, LQ_ERR_ARG, "splits must be in [1, 1024]");
  LQ_REQUIRE(q && k_codes && v_codes && k_scales && v_scales && out && scratch, LQ_ERR_ARG, "null tensor pointer");
  const int G = Hq / Hkv;
  float* part_o = (float*)scratch;
  float* part_ml = part_o + (int64_t)B * Hq * splits * D;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
  int rc = LQ_ERR_UNSUPPORTED;
#define LQ_ATTN_CASE(DD, GG)                                                                   \
  if (D == DD && G == GG)                                                                      \
    rc = launch_pdl(attn_decode_kernel<DD, GG>, grid, dim3(128), s, pdl, "lq_attn_decode_kv_i8", \
                    (const __nv_bfloat16*)q, k_codes, v_codes, k_scales, v_scales, part_o, part_ml, \
                    Hq, Hkv, Tmax, len_dev, len, len_add, scaling);
  LQ_ATTN_CASE(64, 1) LQ_ATTN_CASE(64, 2) LQ_ATTN_CASE(64, 4) LQ_ATTN_CASE(64, 8)
  LQ_ATTN_CASE(128, 1) LQ_ATTN_CASE(128, 2) LQ_ATTN_CASE(128, 4) LQ_ATTN_CASE(128, 8)
#undef LQ_ATTN_CASE
  if (rc == LQ_ERR_UNSUPPORTED)
    return fail(LQ_ERR_UNSUPPORTED, "decode attention is built for head_dim 64/128 and 1/2/4/8 query heads per KV head, got %d / %d", D, G);
  if (rc) return rc;
  return launch_pdl(attn_combine_kernel, dim3((unsigned)Hq, (unsigned)B), dim3((unsigned)((D + 31) / 32 * 32)),
                    s, pdl, "lq_attn_decode_kv_i8(combine)", (const float*)part_o, (const float*)part_ml,
                    (__nv_bfloat16*)out, Hq, D, splits);
}

// ---------------------------------------------------------------- decode attention without a caller-provided scratch
// Some hosts of this library cannot hand it a scratch buffer: a plugin loaded into a
// process whose device memory is owned by another allocator (an inference server that
// pre-allocates the whole GPU, a sandboxed extension that is forbidden to call cudaMalloc),
// or a caller that only ever sees the tensors of the model itself. For them the slices'
// partial results live in a fixed array inside the library image. Every GPU that loads the
// library carries this array until the process exits.
namespace lq {
namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB: e.g. B=8, Hq=32, D=128, 31 slices
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;

// Device address of the array on the current device, resolved once per device. The symbol
// name is only a host-side handle; the address a kernel can use comes from the runtime.
int static_scratch_address(void** out) {
  static void* cached[kMaxDevices] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(LQ_ERR_UNSUPPORTED, "device index %d out of range", dev);
  void* ptr = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    e = cudaGetSymbolAddress(&ptr, g_static_attn_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return fail(LQ_ERR_LAUNCH, "cannot resolve the built-in scratch array: %s", cudaGetErrorString(e));
    }
    __atomic_store_n(&cached[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return LQ_OK;
}

}  // namespace
}  // namespace lq

extern "C" int64_t lq_attn_decode_static_scratch_bytes(void) {
  return (int64_t)lq::kStaticScratchBytes;
}

extern "C" int lq_attn_decode_kv_i8_static(const void* q, const int8_t* k_codes, const int8_t* v_codes,
                                           const float* k_scales, const float* v_scales, void* out,
                                           int B, int Hq, int Hkv, int D, int Tmax,
                                           const int64_t* len_dev, int64_t len, int len_add,
                                           float scaling, int splits, int pdl, void* stream) {
  using namespace lq;
  LQ_REQUIRE(B > 0 && Hq > 0 && D > 0 && splits >= 1, LQ_ERR_ARG, "bad shape");
  const int64_t need = lq_attn_decode_scratch_bytes(B, Hq, D, splits);
  LQ_REQUIRE(need <= (int64_t)kStaticScratchBytes, LQ_ERR_UNSUPPORTED,
             "this call needs %lld bytes of scratch but the built-in array holds %lld; use fewer "
             "slices or lq_attn_decode_kv_i8 with your own buffer",
             (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  return lq_attn_decode_kv_i8(q, k_codes, v_codes, k_scales, v_scales, out, scratch, B, Hq, Hkv, D,
                              Tmax, len_dev, len, len_add, scaling, splits, pdl, stream);
}

// ---------------------------------------------------------------- one kernel per layer: RoPE + KV write + attention + merge
// The decode step's attention block as a single launch. grid (NS, Hkv, B), 128 threads.
// Every CTA rotates the G query heads of its KV head itself (a few hundred multiply-adds)
// instead of reading them back from a separate kernel's output. The CTA of the last slice
// also rotates and quantizes the new token's K and V rows, appends them to the cache at the
// cursor and folds them into its softmax from registers, so the cached tokens [0, pos) are
// the only thing read from HBM. Slices meet through the scratch arrays; the CTA that
// finishes last (an atomic ticket per KV head) merges them and writes the bf16 output, then
// puts the ticket back to zero for the next launch.
namespace lq {
namespace {

constexpr int kFusedThreads = 256;            // 8 warps: 16 lanes per token, 2 tokens per warp
constexpr int kFusedChunkBytes = 28 * 1024;  // K (and as much V) staged per chunk of a slice

template <int D, int G>
__global__ void __launch_bounds__(kFusedThreads)
attn_fused_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ cos_t,
                  const __nv_bfloat16* __restrict__ sin_t, int8_t* kc, int8_t* vc, float* ks, float* vs,
                  __nv_bfloat16* __restrict__ out, float* part_o, float* part_ml, int* tickets,
                  int Hq, int Hkv, int Tmax, int table_len, const int64_t* pos_dev, int64_t pos_host,
                  float scaling, float qmin, float qmax, int* error_word, unsigned long long* debug) {
#ifdef LQ_DIAGNOSTICS
#define ATT_STAMP(slot) do { if (debug != nullptr && threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); debug[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (slot)] = t_; } } while (0)
#else
#define ATT_STAMP(slot) do { } while (0)
#endif
  constexpr int DPL = D / 16;  // dims per lane
  constexpr int NGRP = 16;     // lane groups per CTA (8 warps x 2)
  constexpr int NT = kFusedThreads;
  constexpr int HALF = D / 2;
  constexpr int CAP = kFusedChunkBytes / D;  // tokens per staged chunk
  extern __shared__ __align__(128) uint8_t stage[];  // K codes [CAP, D], V codes [CAP, D], scores [CAP, G]
  __shared__ __align__(8) uint64_t bar;
  __shared__ float sk_s[CAP], sv_s[CAP];
  __shared__ float q_s[G][D];
  __shared__ float knew_s[D], vnew_s[D];
  __shared__ float m_s[NGRP][G], l_s[NGRP][G];
  __shared__ float newscale_s[2];
  __shared__ int last_s;
  float (*o_s)[G][D] = reinterpret_cast<float (*)[G][D]>(stage);  // reused after the loop

  const int ns = gridDim.x, split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 15, grp = warp * 2 + (lane >> 4);
  ATT_STAMP(0);
  // The cursor was advanced by the previous step, long before the kernel ahead of this one
  // started, and the cached rows [0, pos) are older still: both may be read before the
  // dependency wait, so the slice's first chunk is already on its way while q is computed.
  int64_t pos = read_pos(pos_dev, pos_host);   // index of the new token = number of cached ones
  if (pos < 0) pos = 0;
  if (pos > Tmax - 1) pos = Tmax - 1;
  const int64_t len = pos;
  const int per = (int)((len + ns - 1) / ns);
  const int t_lo = split * per;
  const int t_hi = (int)min((int64_t)(t_lo + per), len);
  const int64_t head_row = ((int64_t)b * Hkv + kvh) * Tmax;
  const uint32_t bar_a = smem_u32(&bar);
  const uint32_t k_a = smem_u32(stage), v_a = k_a + CAP * D;

  auto issue = [&](int c_lo) {  // one thread: request K and V codes of a chunk
    const int n = min(CAP, t_hi - c_lo);
    const uint32_t bytes = (uint32_t)n * D;
    mbar_expect_tx(bar_a, 2 * bytes);
    bulk_g2s(k_a, kc + (head_row + c_lo) * D, bytes, bar_a);
    bulk_g2s(v_a, vc + (head_row + c_lo) * D, bytes, bar_a);
  };
  if (threadIdx.x == 0) {
    mbar_init(bar_a, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (t_lo < t_hi) issue(t_lo);
  }

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  ATT_STAMP(1);
  const int64_t tpos = pos < table_len ? pos : table_len - 1;
  const int heads = Hq + 2 * Hkv;
  const __nv_bfloat16* row = qkv + (int64_t)b * heads * D;
  auto r16 = [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); };

  // ---- rotate the G query heads (bf16 arithmetic of apply_rotary_pos_emb), pre-scaled
  for (int i = threadIdx.x; i < G * HALF; i += NT) {
    const int g = i / HALF, d = i % HALF;
    const __nv_bfloat16* src = row + (int64_t)(kvh * G + g) * D;
    const float a = __bfloat162float(src[d]), c = __bfloat162float(src[d + HALF]);
    const float c0 = __bfloat162float(cos_t[tpos * D + d]), s0 = __bfloat162float(sin_t[tpos * D + d]);
    const float c1 = __bfloat162float(cos_t[tpos * D + d + HALF]), s1 = __bfloat162float(sin_t[tpos * D + d + HALF]);
    q_s[g][d] = r16(r16(a * c0) + r16(-c * s0)) * scaling;
    q_s[g][d + HALF] = r16(r16(c * c1) + r16(a * s1)) * scaling;
  }
  ATT_STAMP(2);
  // ---- the last slice owns the new token: rotate K, quantize K and V, append to the cache
  const bool owner = split == ns - 1;
  if (owner && warp < 2) {
    const bool is_v = warp == 1;
    const __nv_bfloat16* src = row + (int64_t)(Hq + (is_v ? Hkv : 0) + kvh) * D;
    float val[D / 32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int d = lane + 32 * j;
      float x = __bfloat162float(src[d]);
      if (!is_v) {
        const int partner = d < HALF ? d + HALF : d - HALF;
        const float y = __bfloat162float(src[partner]);
        const float cc = __bfloat162float(cos_t[tpos * D + d]), ss = __bfloat162float(sin_t[tpos * D + d]);
        x = d < HALF ? r16(r16(x * cc) + r16(-y * ss)) : r16(r16(x * cc) + r16(y * ss));
      }
      val[j] = x;
      amax = fmaxf(amax, fabsf(x));
    }
    amax = warp_max(amax);
    const float scale = scale_of(amax, qmax);
    const int64_t crow = head_row + pos;
    if (lane == 0) { (is_v ? vs : ks)[crow] = scale; newscale_s[is_v] = scale; }
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int d = lane + 32 * j;
      const float code = code_of(val[j], scale, qmin, qmax);
      (is_v ? vc : kc)[crow * D + d] = (int8_t)code;
      (is_v ? vnew_s : knew_s)[d] = code;
    }
  }

  // Online softmax per chunk, in two passes over the staged codes: scores first (their
  // maximum is then known for the whole CTA), probabilities and the V sum second. No value
  // depends on the previous token inside a pass, so the loops pipeline freely.
  float M[G], l[G], acc[G][DPL];   // M is the same in every thread of the CTA
#pragma unroll
  for (int g = 0; g < G; ++g) {
    M[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }
  float* sc_s = reinterpret_cast<float*>(stage + 2 * (size_t)CAP * D);  // [CAP][G] scores
  using Vec = typename std::conditional<DPL == 8, uint2, uint32_t>::type;
  auto raise_max = [&](const float (&cmax)[G]) {  // CTA-wide maximum, then rescale what we hold
    if (sub == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) m_s[grp][g] = cmax[g];
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mm = M[g];
      for (int r = 0; r < NGRP; ++r) mm = fmaxf(mm, m_s[r][g]);
      if (mm > M[g]) {
        const float corr = (M[g] == -INFINITY) ? 0.f : __expf(M[g] - mm);
        l[g] *= corr;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] *= corr;
        M[g] = mm;
      }
    }
    __syncthreads();  // m_s is free again
  };

  ATT_STAMP(3);
  // ---- cached tokens of this slice, chunk by chunk out of shared memory
  bool dead = false;
  int phase = 0;
  for (int c_lo = t_lo; c_lo < t_hi; c_lo += CAP) {
    const int n = min(CAP, t_hi - c_lo);
    for (int i = threadIdx.x; i < n; i += NT) {
      sk_s[i] = ks[head_row + c_lo + i];
      sv_s[i] = vs[head_row + c_lo + i];
    }
    __syncthreads();  // also orders q_s before its first use
    if (!mbar_wait(bar_a, phase)) { dead = true; break; }  // every thread waits on the same phase
    phase ^= 1;
    float cmax[G];
#pragma unroll
    for (int g = 0; g < G; ++g) cmax[g] = -INFINITY;
    // pass 1 (warp-uniform trip count: the shuffles name all 32 lanes)
#pragma unroll 2
    for (int i0 = 0; i0 < n; i0 += NGRP) {
      const int i = i0 + grp;
      const bool valid = i < n;
      const int r = valid ? i : 0;
      int8_t kb[DPL];
      *reinterpret_cast<Vec*>(kb) = *reinterpret_cast<const Vec*>(stage + (size_t)r * D + sub * DPL);
      const float sk = sk_s[r];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) d = fmaf(q_s[g][sub * DPL + j], (float)kb[j], d);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        d += __shfl_xor_sync(0xffffffffu, d, 8);
        d *= sk;
        if (valid) {
          cmax[g] = fmaxf(cmax[g], d);
          if (sub == 0) sc_s[r * G + g] = d;
        }
      }
    }
    raise_max(cmax);  // (its barriers also publish sc_s)
    // pass 2
#pragma unroll 2
    for (int i0 = 0; i0 < n; i0 += NGRP) {
      const int i = i0 + grp;
      if (i < n) {
        int8_t vb[DPL];
        *reinterpret_cast<Vec*>(vb) = *reinterpret_cast<const Vec*>(stage + (size_t)(CAP + i) * D + sub * DPL);
        const float sv = sv_s[i];
        float vf[DPL];
#pragma unroll
        for (int j = 0; j < DPL; ++j) vf[j] = (float)vb[j] * sv;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pgt = __expf(sc_s[i * G + g] - M[g]);
          l[g] += pgt;
#pragma unroll
          for (int j = 0; j < DPL; ++j) acc[g][j] = fmaf(pgt, vf[j], acc[g][j]);
        }
      }
    }
    __syncthreads();  // everyone is done with the stage before it is refilled
    if (threadIdx.x == 0 && c_lo + CAP < t_hi) issue(c_lo + CAP);
  }
  if (dead) {
    if (threadIdx.x == 0) atomicExch(error_word, 3);
    return;
  }
  __syncthreads();
  if (owner) {  // the new token, from shared memory: every lane joins the shuffles
    float snew[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < DPL; ++j) d = fmaf(q_s[g][sub * DPL + j], knew_s[sub * DPL + j], d);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      d += __shfl_xor_sync(0xffffffffu, d, 8);
      snew[g] = d * newscale_s[0];
    }
    raise_max(snew);
    if (grp == 0) {  // one lane group adds it
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pgt = __expf(snew[g] - M[g]);
        l[g] += pgt;
#pragma unroll
        for (int j = 0; j < DPL; ++j)
          acc[g][j] = fmaf(pgt, vnew_s[sub * DPL + j] * newscale_s[1], acc[g][j]);
      }
    }
  }

  ATT_STAMP(4);
  // ---- sum the 16 lane groups of the CTA (same M everywhere; the staging area is free now)
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) l_s[grp][g] = l[g];
  }
  constexpr int OUT_PER_THREAD = (G * D + NT - 1) / NT;
  float osum[OUT_PER_THREAD];
#pragma unroll
  for (int k = 0; k < OUT_PER_THREAD; ++k) osum[k] = 0.f;
  for (int halfsel = 0; halfsel < 2; ++halfsel) {
    __syncthreads();
    if ((grp / (NGRP / 2)) == halfsel) {
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < DPL; ++i) o_s[grp % (NGRP / 2)][g][sub * DPL + i] = acc[g][i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < OUT_PER_THREAD; ++k) {
      const int i = threadIdx.x + NT * k;
      if (i < G * D) {
        const int g = i / D, d = i % D;
#pragma unroll
        for (int r = 0; r < NGRP / 2; ++r) osum[k] += o_s[r][g][d];
      }
    }
  }
  float* po = part_o + (((int64_t)b * Hq + kvh * G) * ns + split) * D;
#pragma unroll
  for (int k = 0; k < OUT_PER_THREAD; ++k) {
    const int i = threadIdx.x + NT * k;
    if (i < G * D) po[(int64_t)(i / D) * ns * D + (i % D)] = osum[k];
  }
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    float lt = 0.f;
    for (int r = 0; r < NGRP; ++r) lt += l_s[r][g];
    float* ml = part_ml + (((int64_t)b * Hq + kvh * G + g) * ns + split) * 2;
    ml[0] = M[g]; ml[1] = lt;
  }

  // ---- the CTA that finishes last merges the slices
  ATT_STAMP(5);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&tickets[b * Hkv + kvh], 1);
    last_s = ticket == ns - 1;
  }
  __syncthreads();
  ATT_STAMP(6);
  if (!last_s) return;
  __threadfence();
  // weights of the slices: w_s[s][g] = exp(m_s - max) (shared memory reused again). Then the
  // warps split the slices between them, every lane keeps all its loads in flight at once,
  // and the per-warp sums meet in shared memory.
  float* wsl = reinterpret_cast<float*>(stage);          // [ns][G]
  float* lsum = wsl + (size_t)ns * G;                    // [G]
  float* psum = lsum + G;                                // [8 warps][G * D]
  for (int g = warp; g < G; g += NT / 32) {
    const int64_t base = ((int64_t)b * Hq + kvh * G + g) * ns;
    float mm = -INFINITY;
    for (int s = lane; s < ns; s += 32) mm = fmaxf(mm, __ldcg(part_ml + (base + s) * 2));
    mm = warp_max(mm);
    float lt = 0.f;
    for (int s = lane; s < ns; s += 32) {
      const float ms = __ldcg(part_ml + (base + s) * 2);
      const float ws = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
      wsl[s * G + g] = ws;
      lt = fmaf(__ldcg(part_ml + (base + s) * 2 + 1), ws, lt);
    }
    lt = warp_sum(lt);
    if (lane == 0) lsum[g] = lt;
  }
  __syncthreads();
  constexpr int PER_LANE = (G * D + 31) / 32;  // outputs a lane covers for its warp's slices
  float part[PER_LANE];
#pragma unroll
  for (int k = 0; k < PER_LANE; ++k) part[k] = 0.f;
  for (int s0 = warp; s0 < ns; s0 += 4 * (NT / 32)) {  // four slices of this warp per round
    float v[4][PER_LANE];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int s = s0 + j * (NT / 32);
#pragma unroll
      for (int k = 0; k < PER_LANE; ++k) {
        const int i = lane + 32 * k;
        const int g = i / D, d = i % D;
        v[j][k] = (s < ns && i < G * D)
                      ? __ldcg(part_o + (((int64_t)b * Hq + kvh * G + g) * ns + s) * D + d) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int s = s0 + j * (NT / 32);
      if (s < ns) {
#pragma unroll
        for (int k = 0; k < PER_LANE; ++k) {
          const int i = lane + 32 * k;
          if (i < G * D) part[k] = fmaf(v[j][k], wsl[s * G + i / D], part[k]);
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < PER_LANE; ++k) {
    const int i = lane + 32 * k;
    if (i < G * D) psum[warp * (G * D) + i] = part[k];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += NT) {
    const int g = i / D, d = i % D;
    float o = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < NT / 32; ++w8) o += psum[w8 * (G * D) + i];
    const float lt = lsum[g];
    out[((int64_t)b * Hq + kvh * G + g) * D + d] = __float2bfloat16_rn(lt > 0.f ? o / lt : 0.f);
  }
  if (threadIdx.x == 0) tickets[b * Hkv + kvh] = 0;
  ATT_STAMP(7);
#undef ATT_STAMP
}

// ---------------------------------------------------------------- the same block on mma.sync
// The SIMT kernel above spends ~20 instructions per cached byte, four times what an HBM-bound
// stream allows when four query heads share a KV head. This version keeps the same data flow
// (bulk-copy staging, chunked online softmax, slice merge by the last CTA) but does the two
// contractions on the tensor cores, shaped so that the int8 codes are consumed as they are:
//   scores  m16n8k32 s8 x s8 -> s32: A rows 0..7 hold the high byte and rows 8..15 the low byte
//           of the query heads re-expressed as 15-bit block-floating-point integers (exact for
//           a bf16 query up to 2^-14 of the head's maximum), B is the K codes read straight
//           from the staged rows, so one thread ends up with both halves of a score;
//   values  m16n8k16 bf16: A is p * v_scale in bf16 taken from the score accumulators, B the V
//           codes of four token rows widened to bf16 in registers.
// Staged rows are padded by 16 bytes so that both fragment access patterns are free of
// shared-memory bank conflicts (one bulk copy per row).
//
// Two ways to merge the slices of one KV head (template flag CL):
//   CL = false  every CTA writes its partial (max, sum, output) to global scratch and the CTA
//               that takes the last ticket merges them: any number of slices.
//   CL = true   the slices of a KV head form ONE thread-block cluster (2, 4, 8 or 16 CTAs): every
//               CTA sends each piece of its partial output straight into the shared memory of
//               the CTA that owns those output elements (st.shared::cluster), one cluster
//               barrier follows, and every CTA finishes its own G * D / slices outputs -- no
//               global scratch, no ticket, no second trip through L2. Every path reaches the
//               cluster barrier (the waits before it are bounded), so it always completes.
constexpr int kMmaThreads = 256;
constexpr int kMmaCap = 128;      // tokens staged per chunk: one 16-token block per warp (192 left half the
                                  // warps waiting at the chunk's barrier for the others' second block)
constexpr int kClusterCap = 288;  // the same for the cluster variant: 16 slices of a 4.6k context in one chunk
constexpr int kMaxCluster = 16;

__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t zero = 0;  // rows 8..15 of A (no query head there)
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void mma_h16(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t zero = 0;  // rows 8..15 of A (no query head there)
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h16(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// Bytes i and i + 1 of two words of (signed code + 128) -> two half2 (code_a, code_b), exact:
// a byte u under the high byte 0x64 is the half 1024 + u, and 1024 + 128 is subtracted.
__device__ __forceinline__ void codes_to_h2(uint32_t wa, uint32_t wb, int i, uint32_t& h_i, uint32_t& h_i1) {
  const uint32_t sel = i == 0 ? 0x5140u : 0x7362u;  // (a_i, b_i, a_i+1, b_i+1)
  const uint32_t t = __byte_perm(wa, wb, sel);
  const uint32_t x0 = __byte_perm(t, 0x64646464u, 0x5140u);  // [a_i, 0x64, b_i, 0x64]
  const uint32_t x1 = __byte_perm(t, 0x64646464u, 0x5342u);  // [a_i+1, 0x64, b_i+1, 0x64]
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
  const __half2 r0 = __hsub2(*reinterpret_cast<const __half2*>(&x0), bias);
  const __half2 r1 = __hsub2(*reinterpret_cast<const __half2*>(&x1), bias);
  h_i = *reinterpret_cast<const uint32_t*>(&r0);
  h_i1 = *reinterpret_cast<const uint32_t*>(&r1);
}

template <int D, int G, bool CL>
__global__ void __launch_bounds__(kMmaThreads)
attn_mma_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ cos_t,
                const __nv_bfloat16* __restrict__ sin_t, int8_t* kc, int8_t* vc, float* ks, float* vs,
                __nv_bfloat16* __restrict__ out, float* part_o, float* part_ml, int* tickets,
                int Hq, int Hkv, int Tmax, int table_len, const int64_t* pos_dev, int64_t pos_host,
                float scaling, float qmin, float qmax, int* error_word, unsigned long long* debug) {
#ifdef LQ_DIAGNOSTICS
#define ATT_STAMP(slot) do { if (debug != nullptr && threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); debug[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (slot)] = t_; } } while (0)
#else
#define ATT_STAMP(slot) do { } while (0)
#endif
  constexpr int NT = kMmaThreads, NW = NT / 32;
  constexpr int HALF = D / 2, CAP = CL ? kClusterCap : kMmaCap, PK = D;  // unpadded rows: one bulk copy per chunk
  constexpr int KS = D / 32;   // k-steps of the score MMA
  constexpr int DT = D / 8;    // n-tiles of the value MMA
  extern __shared__ __align__(128) uint8_t stage[];  // per staging area: K rows [CAP][PK], then V rows [CAP][PK]
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ float sk_s[CAP], sv_s[CAP];
  __shared__ float q_s[G][D];                       // rotated query heads (bf16 values)
  __shared__ __align__(16) int8_t qhi_s[G][D], qlo_s[G][D];
  __shared__ float qunit_s[G];
  __shared__ float knew_s[D], vnew_s[D];
  __shared__ float newscale_s[2], snew_s[G];
  __shared__ float mw_s[NW][8], lw_s[NW][8];
  __shared__ int last_s;
  // cluster variant: what the other slices send here -- their pieces of this CTA's outputs and
  // their (max, sum) per head
  __shared__ float recv_o[CL ? G * D : 1];
  __shared__ float recv_ml[CL ? kMaxCluster * G * 2 : 1];

  const int ns = gridDim.x, split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, q4 = lane & 3;  // fragment coordinates
  // A CTA's shared memory may be written by its cluster peers only once it has started: every
  // CTA announces itself here and waits for the others right before its first remote store.
  if (CL) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  ATT_STAMP(0);
  int64_t pos = read_pos(pos_dev, pos_host);
  if (pos < 0) pos = 0;
  if (pos > Tmax - 1) pos = Tmax - 1;
  const int64_t len = pos;
  const int per = (int)((len + ns - 1) / ns);
  const int t_lo = split * per;
  const int t_hi = (int)min((int64_t)(t_lo + per), len);
  const int64_t head_row = ((int64_t)b * Hkv + kvh) * Tmax;
  // Two staging areas (one in the cluster variant, whose chunks are larger): the copies of the
  // next chunk travel while this one is multiplied, which is what a CTA that walks several
  // chunks -- a batch of sequences, a long context -- spends most of its time on otherwise.
  constexpr int NST = CL ? 1 : 2;
  constexpr size_t STAGE_BYTES = 2 * (size_t)CAP * PK;
  const uint32_t bar_a = smem_u32(&bar[0]);

  auto issue = [&](int c_lo, int st) {  // warp 0: the chunk's K rows and V rows, one bulk copy each
    const int n = min(CAP, t_hi - c_lo);
    if (lane == 0) {
      const uint32_t bytes = (uint32_t)n * D;
      const uint32_t dst = smem_u32(stage + st * STAGE_BYTES);
      mbar_expect_tx(bar_a + 8 * st, 2u * bytes);
      bulk_g2s(dst, kc + (head_row + c_lo) * D, bytes, bar_a + 8 * st);
      bulk_g2s(dst + CAP * PK, vc + (head_row + c_lo) * D, bytes, bar_a + 8 * st);
    }
    __syncwarp();
  };
  if (threadIdx.x == 0) {
    mbar_init(bar_a, 1);
    mbar_init(bar_a + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // cached rows and the cursor are older than the kernel ahead of this one: prefetch first
  if (warp == 0 && t_lo < t_hi) issue(t_lo, 0);
  // so are the rotary tables and the cached rows' scales: the pieces this thread needs first
  // are requested before the wait for the producer of q|k|v, off the dependent chain
  const int64_t tpos = pos < table_len ? pos : table_len - 1;
  float pre_cs[4] = {0.f, 0.f, 0.f, 0.f};
  if ((int)threadIdx.x < G * HALF) {
    const int d = threadIdx.x % HALF;
    pre_cs[0] = __bfloat162float(cos_t[tpos * D + d]);
    pre_cs[1] = __bfloat162float(sin_t[tpos * D + d]);
    pre_cs[2] = __bfloat162float(cos_t[tpos * D + d + HALF]);
    pre_cs[3] = __bfloat162float(sin_t[tpos * D + d + HALF]);
  }
  float pre_sk = 0.f, pre_sv = 0.f;
  if ((int)threadIdx.x < min(CAP, t_hi - t_lo)) {
    pre_sk = ks[head_row + t_lo + threadIdx.x];
    pre_sv = vs[head_row + t_lo + threadIdx.x];
  }

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  ATT_STAMP(1);
  const int heads = Hq + 2 * Hkv;
  const __nv_bfloat16* row = qkv + (int64_t)b * heads * D;
  auto r16 = [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); };

  for (int i = threadIdx.x; i < G * HALF; i += NT) {
    const int g = i / HALF, d = i % HALF;
    const __nv_bfloat16* src = row + (int64_t)(kvh * G + g) * D;
    const float a = __bfloat162float(src[d]), c = __bfloat162float(src[d + HALF]);
    const bool first = i == (int)threadIdx.x;  // the prefetched table entries are this d's
    const float c0 = first ? pre_cs[0] : __bfloat162float(cos_t[tpos * D + d]);
    const float s0 = first ? pre_cs[1] : __bfloat162float(sin_t[tpos * D + d]);
    const float c1 = first ? pre_cs[2] : __bfloat162float(cos_t[tpos * D + d + HALF]);
    const float s1 = first ? pre_cs[3] : __bfloat162float(sin_t[tpos * D + d + HALF]);
    q_s[g][d] = r16(r16(a * c0) + r16(-c * s0));
    q_s[g][d + HALF] = r16(r16(c * c1) + r16(a * s1));
  }
  const bool owner = split == ns - 1;
  if (owner && warp >= NW - 2) {  // the last two warps (warp 0 is busy issuing copies)
    const bool is_v = warp == NW - 1;
    const __nv_bfloat16* src = row + (int64_t)(Hq + (is_v ? Hkv : 0) + kvh) * D;
    float val[D / 32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int d = lane + 32 * j;
      float x = __bfloat162float(src[d]);
      if (!is_v) {
        const int partner = d < HALF ? d + HALF : d - HALF;
        const float y = __bfloat162float(src[partner]);
        const float cc = __bfloat162float(cos_t[tpos * D + d]), ss = __bfloat162float(sin_t[tpos * D + d]);
        x = d < HALF ? r16(r16(x * cc) + r16(-y * ss)) : r16(r16(x * cc) + r16(y * ss));
      }
      val[j] = x;
      amax = fmaxf(amax, fabsf(x));
    }
    amax = warp_max(amax);
    const float scale = scale_of(amax, qmax);
    const int64_t crow = head_row + pos;
    if (lane == 0) { (is_v ? vs : ks)[crow] = scale; newscale_s[is_v] = scale; }
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int d = lane + 32 * j;
      const float code = code_of(val[j], scale, qmin, qmax);
      (is_v ? vc : kc)[crow * D + d] = (int8_t)code;
      (is_v ? vnew_s : knew_s)[d] = code;
    }
  }
  __syncthreads();

  // ---- query heads as 15-bit block-floating-point integers, split into two signed bytes
  if (warp < G) {
    const int g = warp;
    float v[D / 32], amax = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) { v[j] = q_s[g][lane + 32 * j]; amax = fmaxf(amax, fabsf(v[j])); }
    amax = warp_max(amax);
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;
    e = max(e, -100);
    const float up = __uint_as_float((unsigned)(127 + 13 - e) << 23);  // |m| < 2^14
    if (lane == 0) qunit_s[g] = __uint_as_float((unsigned)(127 - 13 + e) << 23);
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int m = __float2int_rn(v[j] * up);
      const int hi = (m + 128) >> 8, lo = m - hi * 256;
      qhi_s[g][lane + 32 * j] = (int8_t)hi;
      qlo_s[g][lane + 32 * j] = (int8_t)lo;
    }
  }
  // the new token's scores on the CUDA cores (one warp per head, plain dot product)
  if (owner && warp < G) {
    const int g = warp;
    float d = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) d = fmaf(q_s[g][lane + 32 * j], knew_s[lane + 32 * j], d);
    d = warp_sum(d);
    if (lane == 0) snew_s[g] = d * newscale_s[0] * scaling;
  }
  __syncthreads();
  uint32_t qa[KS][4];
#pragma unroll
  for (int ksx = 0; ksx < KS; ++ksx) {
    // The MMA's k index is mapped onto the head's dims so that the 8 K bytes a thread feeds per
    // k-step are contiguous in a cached row and its D/4 bytes for all k-steps one vector load:
    // thread q4 owns dims [q4 * D/4, (q4 + 1) * D/4), k-step ksx the eight from ksx * 8 on.
    const int c = q4 * (D / 4) + ksx * 8;
    const bool have = gid < G;
    qa[ksx][0] = have ? *reinterpret_cast<const uint32_t*>(&qhi_s[have ? gid : 0][c]) : 0u;
    qa[ksx][1] = have ? *reinterpret_cast<const uint32_t*>(&qlo_s[have ? gid : 0][c]) : 0u;
    qa[ksx][2] = have ? *reinterpret_cast<const uint32_t*>(&qhi_s[have ? gid : 0][c + 4]) : 0u;
    qa[ksx][3] = have ? *reinterpret_cast<const uint32_t*>(&qlo_s[have ? gid : 0][c + 4]) : 0u;
  }
  const float qscale = (gid < G ? qunit_s[gid < G ? gid : 0] : 0.f) * scaling;

  ATT_STAMP(2);
  // ---- per-warp online softmax over blocks of 16 tokens
  float m_run = -INFINITY, l_run = 0.f;  // row gid of this thread's quad
  float o[DT][4];
#pragma unroll
  for (int dt = 0; dt < DT; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }

  bool dead = false;
  int st = 0, phases = 0;  // staging area of the chunk at hand; one phase bit per area
  for (int c_lo = t_lo; c_lo < t_hi; c_lo += CAP) {
    const int n = min(CAP, t_hi - c_lo);
    // the other area was released by the barrier that ended the round before: refill it now
    if (NST == 2 && warp == 0 && c_lo + CAP < t_hi) issue(c_lo + CAP, st ^ 1);
    for (int i = threadIdx.x; i < n; i += NT) {
      const bool pre = i == (int)threadIdx.x;  // each thread's first scale of a chunk was requested a round ahead
      sk_s[i] = pre ? pre_sk : ks[head_row + c_lo + i];
      sv_s[i] = pre ? pre_sv : vs[head_row + c_lo + i];
    }
    if (c_lo + CAP + (int)threadIdx.x < t_hi) {  // next chunk's: in flight during this chunk's products
      pre_sk = ks[head_row + c_lo + CAP + threadIdx.x];
      pre_sv = vs[head_row + c_lo + CAP + threadIdx.x];
    }
    __syncthreads();
    if (!mbar_wait(bar_a + 8 * st, (phases >> st) & 1)) { dead = true; break; }
    phases ^= 1 << st;
    const uint8_t* k_st = stage + st * STAGE_BYTES;
    const uint8_t* v_st = k_st + (size_t)CAP * PK;
    if (c_lo == t_lo) ATT_STAMP(3);
    const int blocks = (n + 15) / 16;
    for (int blk = warp; blk < blocks; blk += NW) {
      const int r0 = blk * 16;
      float sc[2][2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        int c[4] = {0, 0, 0, 0};
        const uint8_t* krow = k_st + (size_t)min(r0 + j * 8 + gid, CAP - 1) * PK + q4 * (D / 4);
        uint32_t kw[2 * KS];  // this thread's D/4 dims of the token: 16-byte loads
#pragma unroll
        for (int v = 0; v < KS / 2; ++v) {
          const uint4 t4 = *reinterpret_cast<const uint4*>(krow + v * 16);
          kw[4 * v] = t4.x; kw[4 * v + 1] = t4.y; kw[4 * v + 2] = t4.z; kw[4 * v + 3] = t4.w;
        }
#pragma unroll
        for (int ksx = 0; ksx < KS; ++ksx) mma_s8(c, qa[ksx], kw[2 * ksx], kw[2 * ksx + 1]);
        const int t0 = r0 + j * 8 + q4 * 2;
        sc[j][0] = t0 < n ? (float)(c[0] * 256 + c[2]) * qscale * sk_s[t0] : -INFINITY;
        sc[j][1] = t0 + 1 < n ? (float)(c[1] * 256 + c[3]) * qscale * sk_s[min(t0 + 1, CAP - 1)] : -INFINITY;
      }
      float mx = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float corr = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
      float pr[2][2];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          pr[j][e] = (sc[j][e] == -INFINITY || m_new == -INFINITY) ? 0.f : __expf(sc[j][e] - m_new);
      l_run = l_run * corr + (pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1]);
      m_run = m_new;
#pragma unroll
      for (int dt = 0; dt < DT; ++dt) { o[dt][0] *= corr; o[dt][1] *= corr; }
      const int ta = r0 + q4 * 2, tb = ta + 8;  // this thread's token rows in the block
      const int ra0 = min(ta, CAP - 1), ra1 = min(ta + 1, CAP - 1), rb0 = min(tb, CAP - 1), rb1 = min(tb + 1, CAP - 1);
      // (rows past the end of the chunk hold stale bytes and no scale: their weight is a plain 0)
      // probabilities x value scales and the value codes as fp16 (codes exactly; the weights with
      // 11 significant bits), fp32 accumulate
      const uint32_t a0 = pack_h16(ta < n ? pr[0][0] * sv_s[ra0] : 0.f, ta + 1 < n ? pr[0][1] * sv_s[ra1] : 0.f);
      const uint32_t a2 = pack_h16(tb < n ? pr[1][0] * sv_s[rb0] : 0.f, tb + 1 < n ? pr[1][1] * sv_s[rb1] : 0.f);
      // Output tile dt, column j of the MMA is dim j * DT + dt, so the DT codes a thread feeds for
      // one token (its column j = gid) are contiguous: one vector load per token row.
      uint32_t vw[4][DT / 4];
      {
        const uint8_t* rows[4] = {v_st + (size_t)ra0 * PK, v_st + (size_t)ra1 * PK, v_st + (size_t)rb0 * PK,
                                  v_st + (size_t)rb1 * PK};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          if (DT == 16) {
            const uint4 t4 = *reinterpret_cast<const uint4*>(rows[r] + gid * DT);
            vw[r][0] = t4.x ^ 0x80808080u; vw[r][1] = t4.y ^ 0x80808080u;
            vw[r][DT / 4 - 2] = t4.z ^ 0x80808080u; vw[r][DT / 4 - 1] = t4.w ^ 0x80808080u;
          } else {
            const uint2 t2 = *reinterpret_cast<const uint2*>(rows[r] + gid * DT);
            vw[r][0] = t2.x ^ 0x80808080u; vw[r][1] = t2.y ^ 0x80808080u;
          }
        }
      }
#pragma unroll
      for (int w = 0; w < DT / 4; ++w) {
#pragma unroll
        for (int i = 0; i < 4; i += 2) {
          uint32_t b0a, b0b, b1a, b1b;
          codes_to_h2(vw[0][w], vw[1][w], i, b0a, b0b);  // tokens ta, ta + 1
          codes_to_h2(vw[2][w], vw[3][w], i, b1a, b1b);  // tokens tb, tb + 1
          mma_h16(o[4 * w + i], a0, a2, b0a, b1a);
          mma_h16(o[4 * w + i + 1], a0, a2, b0b, b1b);
        }
      }
    }
    __syncthreads();  // everyone is done with the area before it is refilled
    if (NST == 1 && warp == 0 && c_lo + CAP < t_hi) issue(c_lo + CAP, 0);
    if (NST == 2) st ^= 1;
  }
  if (dead) {
    if (threadIdx.x == 0) atomicExch(error_word, 4);
    if (!CL) return;  // (a cluster's CTAs all go on to the cluster barrier)
  }
  ATT_STAMP(4);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

  // ---- merge the warps (and the new token) of the CTA; the staging area is free now
  float (*ow_s)[G][D] = reinterpret_cast<float (*)[G][D]>(stage);  // [NW][G][D]
  if (CL) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // every peer has started
  if (q4 == 0 && gid < 8) { mw_s[warp][gid] = m_run; lw_s[warp][gid] = l_run; }
  if (gid < G) {
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      ow_s[warp][gid][(q4 * 2) * DT + dt] = o[dt][0];  // column j of tile dt is dim j * DT + dt
      ow_s[warp][gid][(q4 * 2 + 1) * DT + dt] = o[dt][1];
    }
  }
  __syncthreads();
  // one thread merges the two outputs (g, d) and (g, d + D/2): the warps' weights exp(m_w - m)
  // are computed once for both
  for (int i = threadIdx.x; i < G * (D / 2); i += NT) {
    const int g = i / (D / 2), d = i % (D / 2);
    float mm = owner ? snew_s[g] : -INFINITY;
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, mw_s[w][g]);
    float acc0 = 0.f, acc1 = 0.f, lt = 0.f;
    for (int w = 0; w < NW; ++w) {
      const float mw = mw_s[w][g];
      if (mw != -INFINITY) {
        const float e = __expf(mw - mm);
        acc0 = fmaf(ow_s[w][g][d], e, acc0);
        acc1 = fmaf(ow_s[w][g][d + D / 2], e, acc1);
        lt = fmaf(lw_s[w][g], e, lt);
      }
    }
    if (owner) {
      const float e = __expf(snew_s[g] - mm);
      acc0 = fmaf(vnew_s[d] * newscale_s[1], e, acc0);
      acc1 = fmaf(vnew_s[d + D / 2] * newscale_s[1], e, acc1);
      lt += e;
    }
    if (CL) {
      // output j = g * D + d belongs to CTA j / OPC of the cluster; this slice's piece lands at
      // [split][j % OPC] of that CTA's receive area, its (max, sum) in everyone's table
      const int OPC = G * D / ns;
      const int j0 = g * D + d, j1 = j0 + D / 2;
      st_cluster_f32(cluster_map(smem_u32(&recv_o[split * OPC + j0 % OPC]), j0 / OPC), acc0);
      st_cluster_f32(cluster_map(smem_u32(&recv_o[split * OPC + j1 % OPC]), j1 / OPC), acc1);
      if (d == 0) {
        for (int c = 0; c < ns; ++c) {
          st_cluster_f32(cluster_map(smem_u32(&recv_ml[(split * G + g) * 2]), c), mm);
          st_cluster_f32(cluster_map(smem_u32(&recv_ml[(split * G + g) * 2 + 1]), c), lt);
        }
      }
    } else {
      float* po = part_o + (((int64_t)b * Hq + kvh * G + g) * ns + split) * D;
      po[d] = acc0;
      po[d + D / 2] = acc1;
      if (d == 0) {
        float* ml = part_ml + (((int64_t)b * Hq + kvh * G + g) * ns + split) * 2;
        ml[0] = mm; ml[1] = lt;
      }
    }
  }
  if (CL) {
    // ---- every slice has delivered: finish this CTA's share of the head's outputs
    cluster_barrier();
    const int OPC = G * D / ns;
    for (int i = threadIdx.x; i < OPC; i += NT) {
      const int j = split * OPC + i, g = j / D, d = j % D;
      float mm = -INFINITY;
      for (int c = 0; c < ns; ++c) mm = fmaxf(mm, recv_ml[(c * G + g) * 2]);
      float ov = 0.f, lt = 0.f;
      for (int c = 0; c < ns; ++c) {
        const float mc = recv_ml[(c * G + g) * 2];
        if (mc != -INFINITY) {
          const float e = __expf(mc - mm);
          ov = fmaf(recv_o[c * OPC + i], e, ov);
          lt = fmaf(recv_ml[(c * G + g) * 2 + 1], e, lt);
        }
      }
      out[((int64_t)b * Hq + kvh * G + g) * D + d] = __float2bfloat16_rn(lt > 0.f ? ov / lt : 0.f);
    }
    ATT_STAMP(7);
    return;
  }

  // ---- the CTA that finishes last merges the slices
  ATT_STAMP(5);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&tickets[b * Hkv + kvh], 1);
    last_s = ticket == ns - 1;
  }
  __syncthreads();
  ATT_STAMP(6);
  if (!last_s) return;
  __threadfence();
  float* wsl = reinterpret_cast<float*>(stage);          // [ns][G]
  float* lsum = wsl + (size_t)ns * G;                    // [G]
  float* psum = lsum + G;                                // [NW][G * D]
  // The first batch of partial outputs is requested before the slice weights are known, so
  // that the two trips to L2 overlap.
  constexpr int PER_LANE = (G * D + 31) / 32;
  constexpr int VB = PER_LANE <= 16 ? 5 : 4;  // slices per warp fetched at once (register budget)
  float v[VB][PER_LANE];
  auto load_batch = [&](int s0) {
#pragma unroll
    for (int j = 0; j < VB; ++j) {
      const int s = s0 + j * NW;
#pragma unroll
      for (int k = 0; k < PER_LANE; ++k) {
        const int i = lane + 32 * k;
        v[j][k] = (s < ns && i < G * D)
                      ? __ldcg(part_o + (((int64_t)b * Hq + kvh * G + i / D) * ns + s) * D + i % D) : 0.f;
      }
    }
  };
  load_batch(warp);
  for (int g = warp; g < G; g += NW) {
    // (max, sum) of every slice of this head: one 8-byte load per slice, kept in registers for
    // up to 64 slices, so the maximum and the weights cost one trip to L2, not three
    const float2* mlp = reinterpret_cast<const float2*>(part_ml) + ((int64_t)b * Hq + kvh * G + g) * ns;
    float2 held[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int s = lane + 32 * j;
      held[j] = s < ns ? __ldcg(mlp + s) : make_float2(-INFINITY, 0.f);
    }
    float mm = fmaxf(held[0].x, held[1].x);
    for (int s = lane + 64; s < ns; s += 32) mm = fmaxf(mm, __ldcg(mlp + s).x);
    mm = warp_max(mm);
    float lt = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int s = lane + 32 * j;
      if (s < ns) {
        const float ws = (held[j].x == -INFINITY) ? 0.f : __expf(held[j].x - mm);
        wsl[s * G + g] = ws;
        lt = fmaf(held[j].y, ws, lt);
      }
    }
    for (int s = lane + 64; s < ns; s += 32) {
      const float2 e = __ldcg(mlp + s);
      const float ws = (e.x == -INFINITY) ? 0.f : __expf(e.x - mm);
      wsl[s * G + g] = ws;
      lt = fmaf(e.y, ws, lt);
    }
    lt = warp_sum(lt);
    if (lane == 0) lsum[g] = lt;
  }
  __syncthreads();
  float part[PER_LANE];
#pragma unroll
  for (int k = 0; k < PER_LANE; ++k) part[k] = 0.f;
  for (int s0 = warp; s0 < ns; s0 += VB * NW) {
    if (s0 != warp) load_batch(s0);
#pragma unroll
    for (int j = 0; j < VB; ++j) {
      const int s = s0 + j * NW;
      if (s < ns) {
#pragma unroll
        for (int k = 0; k < PER_LANE; ++k) {
          const int i = lane + 32 * k;
          if (i < G * D) part[k] = fmaf(v[j][k], wsl[s * G + i / D], part[k]);
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < PER_LANE; ++k) {
    const int i = lane + 32 * k;
    if (i < G * D) psum[warp * (G * D) + i] = part[k];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += NT) {
    const int g = i / D, d = i % D;
    float ov = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < NW; ++w8) ov += psum[w8 * (G * D) + i];
    const float lt = lsum[g];
    out[((int64_t)b * Hq + kvh * G + g) * D + d] = __float2bfloat16_rn(lt > 0.f ? ov / lt : 0.f);
  }
  if (threadIdx.x == 0) tickets[b * Hkv + kvh] = 0;
  ATT_STAMP(7);
#undef ATT_STAMP
}

__device__ int g_attn_error = 0;
#ifdef LQ_DIAGNOSTICS
unsigned long long* g_attn_timeline = nullptr;
#else
constexpr unsigned long long* g_attn_timeline = nullptr;
#endif

}  // namespace
}  // namespace lq

#ifdef LQ_DIAGNOSTICS
// Diagnostic builds only: eight %globaltimer stamps per CTA of lq_attn_decode_fused.
extern "C" void lq_attn_set_timeline(void* device_buffer) {
  lq::g_attn_timeline = (unsigned long long*)device_buffer;
}
#endif

extern "C" int lq_attn_device_error(void) {
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_attn_error) != cudaSuccess) { cudaGetLastError(); return -1; }
  int value = 0;
  if (cudaMemcpy(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(ptr, 0, sizeof(int));
  return value;
}

extern "C" int64_t lq_attn_fused_scratch_bytes(int B, int Hq, int Hkv, int D, int splits) {
  return (int64_t)B * Hq * splits * (D + 2) * (int64_t)sizeof(float) + (int64_t)B * Hkv * (int64_t)sizeof(int);
}

extern "C" int lq_attn_decode_fused(const void* qkv, const void* cos_table, const void* sin_table,
                                    int8_t* k_codes, int8_t* v_codes, float* k_scales, float* v_scales,
                                    void* out, void* scratch, int B, int Hq, int Hkv, int D, int Tmax,
                                    int table_len, const int64_t* pos_dev, int64_t pos, int num_bits,
                                    float scaling, int splits, int impl, int pdl, void* stream) {
  using namespace lq;
  LQ_REQUIRE(num_bits >= 2 && num_bits <= 8, LQ_ERR_ARG, "num_bits must be in [2, 8], got %d", num_bits);
  LQ_REQUIRE(impl >= 0 && impl <= 3, LQ_ERR_ARG, "unknown attention implementation %d", impl);
  LQ_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Tmax > 0 && table_len > 0, LQ_ERR_ARG, "bad shape");
  LQ_REQUIRE(splits >= 1 && splits <= 1024, LQ_ERR_ARG, "splits must be in [1, 1024]");
  LQ_REQUIRE(qkv && cos_table && sin_table && k_codes && v_codes && k_scales && v_scales && out && scratch,
             LQ_ERR_ARG, "null tensor pointer");
  const int G = Hq / Hkv;
  float* part_o = (float*)scratch;
  float* part_ml = part_o + (int64_t)B * Hq * splits * D;
  int* tickets = (int*)(part_ml + (int64_t)B * Hq * splits * 2);
  const float qmax = (float)((1 << (num_bits - 1)) - 1);
  dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
  int rc = LQ_ERR_UNSUPPORTED;
  void* err_ptr = nullptr;
  if (cudaGetSymbolAddress(&err_ptr, g_attn_error) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "cannot resolve the device error word");
  }
  // one thread-block cluster per KV head when the slices can form one (2, 4, 8 or 16 of them,
  // dividing the head's outputs evenly) and such clusters fit the device
  const bool cluster_shape = splits >= 2 && splits <= kMaxCluster && (splits & (splits - 1)) == 0 &&
                             (G * D) % splits == 0 && (G * D) / splits >= 1 && (D == 64 || D == 128);
  // (on request only: measured on B200 at a 4k context the cluster variant is no faster than the
  // merge by the last CTA -- 13.4 us with 16 slices against 10.9 us with 37 -- because a CTA of
  // a 16-slice cluster walks 2.3 times the tokens and the cluster launch itself is slower)
  if (impl == LQ_ATTN_CLUSTER && cluster_shape) {
    const size_t csmem = 2 * (size_t)kClusterCap * D;
    bool tried = false;
#define LQ_CL_CASE(DD, GG)                                                                         \
  if (D == DD && G == GG) {                                                                        \
    auto kern = attn_mma_kernel<DD, GG, true>;                                                     \
    if (const int rs = ensure_smem_limit(reinterpret_cast<const void*>(kern), (int)csmem, "lq_attn_decode_fused")) return rs; \
    if (cluster_fits(kern, splits, grid, dim3(kMmaThreads), csmem)) {                              \
      tried = true;                                                                                \
      rc = launch_cluster(kern, grid, dim3(kMmaThreads), csmem, splits, (cudaStream_t)stream, pdl, \
                    "lq_attn_decode_fused", (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)cos_table, \
                    (const __nv_bfloat16*)sin_table, k_codes, v_codes, k_scales, v_scales,         \
                    (__nv_bfloat16*)out, part_o, part_ml, tickets, Hq, Hkv, Tmax, table_len, pos_dev, \
                    pos, scaling, -qmax - 1.f, qmax, (int*)err_ptr, g_attn_timeline);              \
    }                                                                                              \
  }
    LQ_CL_CASE(64, 1) LQ_CL_CASE(64, 2) LQ_CL_CASE(64, 4) LQ_CL_CASE(64, 8)
    LQ_CL_CASE(128, 1) LQ_CL_CASE(128, 2) LQ_CL_CASE(128, 4) LQ_CL_CASE(128, 8)
#undef LQ_CL_CASE
    if (tried) return rc;
  }
  if (impl == LQ_ATTN_CLUSTER)
    return fail(LQ_ERR_UNSUPPORTED, "clusters of %d CTAs are not available for this shape on this device (head_dim %d, %d "
                "query heads per KV head; the slice count must be 2, 4, 8 or 16)", splits, D, G);
  if (impl != LQ_ATTN_SIMT) {
    // K and V rows of a chunk; a second staging area only if a slice can span several chunks
    const size_t msmem = ((Tmax + splits - 1) / splits > kMmaCap ? 2 : 1) * 2 * (size_t)kMmaCap * D;
    LQ_REQUIRE((size_t)splits * G * 4 + (size_t)(kMmaThreads / 32 + 1) * G * D * 4 + 64 <= msmem, LQ_ERR_ARG,
               "too many slices (%d) for the merge area of the attention kernel", splits);
#define LQ_MMA_CASE(DD, GG)                                                                        \
  if (D == DD && G == GG) {                                                                        \
    if (const int rs = ensure_smem_limit(reinterpret_cast<const void*>(attn_mma_kernel<DD, GG, false>), (int)msmem, "lq_attn_decode_fused")) return rs; \
    rc = launch_pdl_smem(attn_mma_kernel<DD, GG, false>, grid, dim3(kMmaThreads), msmem, (cudaStream_t)stream, pdl, \
                    "lq_attn_decode_fused", (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)cos_table, \
                    (const __nv_bfloat16*)sin_table, k_codes, v_codes, k_scales, v_scales,         \
                    (__nv_bfloat16*)out, part_o, part_ml, tickets, Hq, Hkv, Tmax, table_len, pos_dev, \
                    pos, scaling, -qmax - 1.f, qmax, (int*)err_ptr, g_attn_timeline);              \
  }
    LQ_MMA_CASE(64, 1) LQ_MMA_CASE(64, 2) LQ_MMA_CASE(64, 4) LQ_MMA_CASE(64, 8)
    LQ_MMA_CASE(128, 1) LQ_MMA_CASE(128, 2) LQ_MMA_CASE(128, 4) LQ_MMA_CASE(128, 8)
#undef LQ_MMA_CASE
    if (rc != LQ_ERR_UNSUPPORTED) return rc;
  }
  const size_t smem = 2 * (size_t)kFusedChunkBytes + (size_t)(kFusedChunkBytes / 64) * 8 * sizeof(float);
#define LQ_FUSED_CASE(DD, GG)                                                                      \
  if (D == DD && G == GG) {                                                                        \
    if (const int rs = ensure_smem_limit(reinterpret_cast<const void*>(attn_fused_kernel<DD, GG>), (int)smem, "lq_attn_decode_fused")) return rs; \
    rc = launch_pdl_smem(attn_fused_kernel<DD, GG>, grid, dim3(kFusedThreads), smem, (cudaStream_t)stream, pdl, \
                    "lq_attn_decode_fused", (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)cos_table, \
                    (const __nv_bfloat16*)sin_table, k_codes, v_codes, k_scales, v_scales,         \
                    (__nv_bfloat16*)out, part_o, part_ml, tickets, Hq, Hkv, Tmax, table_len, pos_dev, \
                    pos, scaling, -qmax - 1.f, qmax, (int*)err_ptr, g_attn_timeline);                               \
  }
  LQ_FUSED_CASE(64, 1) LQ_FUSED_CASE(64, 2) LQ_FUSED_CASE(64, 4) LQ_FUSED_CASE(64, 8)
  LQ_FUSED_CASE(128, 1) LQ_FUSED_CASE(128, 2) LQ_FUSED_CASE(128, 4) LQ_FUSED_CASE(128, 8)
#undef LQ_FUSED_CASE
  if (rc == LQ_ERR_UNSUPPORTED)
    return fail(LQ_ERR_UNSUPPORTED, "fused decode attention is built for head_dim 64/128 and 1/2/4/8 query heads per KV head, got %d / %d", D, G);
  return rc;
}
