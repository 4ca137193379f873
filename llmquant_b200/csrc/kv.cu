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
#include "common.cuh"

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
