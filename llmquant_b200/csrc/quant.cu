// Symmetric round-to-nearest quantization: fused quant-dequant, code emission, the one-shot
// weight quantizer, the nibble codec and the dense dequantizer.
//
// The arithmetic rule (fp32 abs-max, IEEE division by qmax, 1e-8 floor, round-half-even,
// clamp to [-qmax-1, qmax], product rounded once to the output dtype) is the one the
// reference fixes in core/observers.py:74-98 and core/quant_ops.py:13-37; results are
// bit-identical to it.
//
// Memory behaviour: one warp owns one group and reads it ONCE with 8-byte loads, keeping up
// to four packets per lane in registers between the abs-max pass and the rounding pass
// (groups up to 512 bf16 / 256 fp32 elements; longer groups re-read through L1/L2).
#include "common.cuh"

namespace lq {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kHeld = 4;  // 8-byte packets a lane keeps in registers

template <typename T>
struct Packet {
  static constexpr int kElems = 8 / sizeof(T);
  uint2 raw;
  __device__ __forceinline__ float get(int i) const {
    const T* p = reinterpret_cast<const T*>(&raw);
    return Conv<T>::to_f32(p[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    T* p = reinterpret_cast<T*>(&raw);
    p[i] = Conv<T>::from_f32(v);
  }
};

// MODE 0: write dequantized values (dtype T); MODE 1: write int8 codes.
template <typename T, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
group_quant_vec_kernel(const T* __restrict__ x, void* __restrict__ out_v,
                       float* __restrict__ scale_out, int64_t groups, int group_size,
                       float qmin, float qmax) {
  constexpr int E = Packet<T>::kElems;
  const int lane = threadIdx.x & 31;
  const int packets = group_size / E;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  for (int64_t g = warp0; g < groups; g += stride) {
    const uint2* src = reinterpret_cast<const uint2*>(x + g * group_size);
    Packet<T> held[kHeld];
    float amax = 0.f;
#pragma unroll
    for (int h = 0; h < kHeld; ++h) {
      const int p = lane + h * 32;
      if (p < packets) {
        held[h].raw = __ldg(src + p);
#pragma unroll
        for (int i = 0; i < E; ++i) amax = fmaxf(amax, fabsf(held[h].get(i)));
      }
    }
    for (int p = lane + kHeld * 32; p < packets; p += 32) {
      Packet<T> t;
      t.raw = __ldg(src + p);
#pragma unroll
      for (int i = 0; i < E; ++i) amax = fmaxf(amax, fabsf(t.get(i)));
    }
    amax = warp_max(amax);
    const float scale = scale_of(amax, qmax);
    if (scale_out != nullptr && lane == 0) scale_out[g] = scale;

    auto emit = [&](const Packet<T>& in, int p) {
      if (MODE == 0) {
        Packet<T> o;
#pragma unroll
        for (int i = 0; i < E; ++i)
          o.set(i, __fmul_rn(code_of(in.get(i), scale, qmin, qmax), scale));
        reinterpret_cast<uint2*>(reinterpret_cast<T*>(out_v) + g * group_size)[p] = o.raw;
      } else {
        int8_t* dst = reinterpret_cast<int8_t*>(out_v) + g * group_size + (int64_t)p * E;
        if (E == 4) {
          char4 c;
          c.x = (signed char)code_of(in.get(0), scale, qmin, qmax);
          c.y = (signed char)code_of(in.get(1), scale, qmin, qmax);
          c.z = (signed char)code_of(in.get(E > 2 ? 2 : 0), scale, qmin, qmax);
          c.w = (signed char)code_of(in.get(E > 2 ? 3 : 0), scale, qmin, qmax);
          *reinterpret_cast<char4*>(dst) = c;
        } else {
          char2 c;
          c.x = (signed char)code_of(in.get(0), scale, qmin, qmax);
          c.y = (signed char)code_of(in.get(1), scale, qmin, qmax);
          *reinterpret_cast<char2*>(dst) = c;
        }
      }
    };
#pragma unroll
    for (int h = 0; h < kHeld; ++h) {
      const int p = lane + h * 32;
      if (p < packets) emit(held[h], p);
    }
    for (int p = lane + kHeld * 32; p < packets; p += 32) {
      Packet<T> t;
      t.raw = __ldg(src + p);
      emit(t, p);
    }
  }
}

// Any group size (including ones whose byte length is not a multiple of 8): scalar loads.
template <typename T, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
group_quant_scalar_kernel(const T* __restrict__ x, void* __restrict__ out_v,
                          float* __restrict__ scale_out, int64_t groups, int group_size,
                          float qmin, float qmax) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  for (int64_t g = warp0; g < groups; g += stride) {
    const T* src = x + g * group_size;
    float amax = 0.f;
    for (int i = lane; i < group_size; i += 32) amax = fmaxf(amax, fabsf(Conv<T>::to_f32(src[i])));
    amax = warp_max(amax);
    const float scale = scale_of(amax, qmax);
    if (scale_out != nullptr && lane == 0) scale_out[g] = scale;
    for (int i = lane; i < group_size; i += 32) {
      const float q = code_of(Conv<T>::to_f32(src[i]), scale, qmin, qmax);
      if (MODE == 0)
        reinterpret_cast<T*>(out_v)[g * group_size + i] = Conv<T>::from_f32(__fmul_rn(q, scale));
      else
        reinterpret_cast<int8_t*>(out_v)[g * group_size + i] = (int8_t)q;
    }
  }
}

template <int MODE>
int launch_group_quant(const void* x, void* out, float* scale_out, int64_t groups, int group_size,
                       int num_bits, int dtype, void* stream) {
  LQ_REQUIRE(num_bits >= 2 && num_bits <= 8, LQ_ERR_ARG, "num_bits must be in [2, 8], got %d", num_bits);
  LQ_REQUIRE(group_size > 0, LQ_ERR_ARG, "group_size must be positive, got %d", group_size);
  LQ_REQUIRE(groups >= 0, LQ_ERR_ARG, "negative group count");
  if (groups == 0) return LQ_OK;
  LQ_REQUIRE(x != nullptr && out != nullptr, LQ_ERR_ARG, "null tensor pointer");
  const float qmax = (float)((1 << (num_bits - 1)) - 1);
  const float qmin = -qmax - 1.f;
  const int64_t want = (groups + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int64_t cap = (int64_t)sm_count() * 64;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    const bool vec = ((size_t)group_size * sizeof(T)) % 8 == 0 && ((uintptr_t)x % 8) == 0 &&
                     ((uintptr_t)out % (MODE == 0 ? 8 : 4)) == 0;
    if (vec)
      group_quant_vec_kernel<T, MODE><<<grid, kWarpsPerBlock * 32, 0, s>>>(
          (const T*)x, out, scale_out, groups, group_size, qmin, qmax);
    else
      group_quant_scalar_kernel<T, MODE><<<grid, kWarpsPerBlock * 32, 0, s>>>(
          (const T*)x, out, scale_out, groups, group_size, qmin, qmax);
  });
  return check_launch(MODE == 0 ? "lq_fake_quant_group" : "lq_quantize_group_i8");
}

// ---------------------------------------------------------------------------- weights
// One warp per (scale row, group). Source column of canonical slot (g, j):
//   head_dim == 0:  c = g*gs + j                          (valid while c < K)
//   head_dim  > 0:  h = g / gph, gi = g % gph, o = gi*gs + j, c = h*head_dim + o (o < head_dim)
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quantize_weight_kernel(const T* __restrict__ w, int8_t* __restrict__ canonical,
                       float* __restrict__ wscale, int N, int K, int gs, int head_dim, int gph,
                       int groups, int out_group, int scale_rows, float qmin, float qmax) {
  const int lane = threadIdx.x & 31;
  const int64_t cell = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (cell >= (int64_t)scale_rows * groups) return;
  const int sr = (int)(cell / groups), g = (int)(cell % groups);
  const int rows_per = out_group > 0 ? out_group : 1;
  const int r0 = sr * rows_per;
  const int r1 = min(N, r0 + rows_per);
  int col0, valid;
  if (head_dim > 0) {
    const int h = g / gph, gi = g % gph;
    col0 = h * head_dim + gi * gs;
    valid = min(gs, head_dim - gi * gs);
  } else {
    col0 = g * gs;
    valid = min(gs, K - col0);
  }
  if (valid < 0) valid = 0;
  float amax = 0.f;
  for (int r = r0; r < r1; ++r)
    for (int j = lane; j < valid; j += 32)
      amax = fmaxf(amax, fabsf(Conv<T>::to_f32(w[(int64_t)r * K + col0 + j])));
  amax = warp_max(amax);
  const float scale = scale_of(amax, qmax);
  if (lane == 0) wscale[(int64_t)sr * groups + g] = scale;
  for (int r = r0; r < r1; ++r) {
    int8_t* dst = canonical + ((int64_t)r * groups + g) * gs;
    for (int j = lane; j < gs; j += 32) {
      int8_t c = 0;
      if (j < valid) c = (int8_t)code_of(Conv<T>::to_f32(w[(int64_t)r * K + col0 + j]), scale, qmin, qmax);
      dst[j] = c;
    }
  }
}

__global__ void pack_int4_kernel(const int8_t* __restrict__ codes, uint8_t* __restrict__ packed,
                                 int64_t n_bytes) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t b = i; b < n_bytes; b += stride) {
    const uint8_t lo = (uint8_t)(codes[2 * b] + 8) & 0xF;
    const uint8_t hi = (uint8_t)(codes[2 * b + 1] + 8) & 0xF;
    packed[b] = lo | (hi << 4);
  }
}

__global__ void unpack_int4_kernel(const uint8_t* __restrict__ packed, int8_t* __restrict__ codes,
                                   int64_t n_bytes) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t b = i; b < n_bytes; b += stride) {
    const uint8_t v = packed[b];
    codes[2 * b] = (int8_t)((int)(v & 0xF) - 8);
    codes[2 * b + 1] = (int8_t)((int)(v >> 4) - 8);
  }
}

template <typename T>
__global__ void dequant_weight_kernel(const int8_t* __restrict__ canonical,
                                      const float* __restrict__ wscale, T* __restrict__ out,
                                      int64_t total, int groups, int gs, int out_group) {
  const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t i = i0; i < total; i += stride) {  // gs % 4 == 0, so 4 codes share a scale
    const int64_t cell = i / gs;
    const int g = (int)(cell % groups);
    const int64_t n = cell / groups;
    const int64_t sr = out_group > 0 ? n / out_group : n;
    const float s = wscale[sr * groups + g];
    const char4 c = *reinterpret_cast<const char4*>(canonical + i);
    out[i] = Conv<T>::from_f32(__fmul_rn((float)c.x, s));
    out[i + 1] = Conv<T>::from_f32(__fmul_rn((float)c.y, s));
    out[i + 2] = Conv<T>::from_f32(__fmul_rn((float)c.z, s));
    out[i + 3] = Conv<T>::from_f32(__fmul_rn((float)c.w, s));
  }
}

// out = bf16(bf16(sum) + residual): the residual add that follows a row-parallel linear whose
// partial sums were all-reduced in fp32 (same roundings as the single-GPU GEMV epilogue).
__global__ void residual_add_kernel(const float* __restrict__ sum, const __nv_bfloat16* __restrict__ residual,
                                    __nv_bfloat16* __restrict__ out, int64_t n) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float y = __bfloat162float(__float2bfloat16_rn(sum[i]));
    out[i] = __float2bfloat16_rn(residual != nullptr ? y + __bfloat162float(residual[i]) : y);
  }
}

}  // namespace
}  // namespace lq

extern "C" int lq_residual_add(const float* sum, const void* residual, void* out, int64_t n, int pdl,
                               void* stream) {
  using namespace lq;
  LQ_REQUIRE(n >= 0, LQ_ERR_ARG, "negative length");
  if (n == 0) return LQ_OK;
  LQ_REQUIRE(sum && out, LQ_ERR_ARG, "null tensor pointer");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((n + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, residual_add_kernel, sum, (const __nv_bfloat16*)residual,
                                     (__nv_bfloat16*)out, n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "lq_residual_add: %s", cudaGetErrorString(e));
  }
  return LQ_OK;
}

extern "C" int lq_fake_quant_group(const void* x, void* out, float* scale_out, int64_t groups,
                                   int group_size, int num_bits, int dtype, void* stream) {
  return lq::launch_group_quant<0>(x, out, scale_out, groups, group_size, num_bits, dtype, stream);
}

extern "C" int lq_quantize_group_i8(const void* x, int8_t* codes, float* scale_out, int64_t groups,
                                    int group_size, int num_bits, int dtype, void* stream) {
  return lq::launch_group_quant<1>(x, codes, scale_out, groups, group_size, num_bits, dtype, stream);
}

extern "C" int lq_quantize_weight(const void* w, int dtype, int N, int K, int group_size,
                                  int head_dim, int out_group, int num_bits, int8_t* canonical,
                                  float* wscale, void* stream) {
  using namespace lq;
  LQ_REQUIRE(num_bits >= 2 && num_bits <= 8, LQ_ERR_ARG, "num_bits must be in [2, 8], got %d", num_bits);
  LQ_REQUIRE(N >= 0 && K >= 0 && group_size > 0, LQ_ERR_ARG, "bad weight shape [%d, %d] / group %d", N, K, group_size);
  LQ_REQUIRE(head_dim >= 0 && out_group >= 0, LQ_ERR_ARG, "head_dim and out_group must be >= 0");
  if (N == 0 || K == 0) return LQ_OK;
  LQ_REQUIRE(head_dim == 0 || K % head_dim == 0, LQ_ERR_ARG,
             "last dim %d is not a multiple of head_dim %d", K, head_dim);
  const int gph = head_dim > 0 ? (head_dim + group_size - 1) / group_size : 0;
  const int groups = head_dim > 0 ? (K / head_dim) * gph : (K + group_size - 1) / group_size;
  const int scale_rows = out_group > 0 ? (N + out_group - 1) / out_group : N;
  const float qmax = (float)((1 << (num_bits - 1)) - 1);
  const int64_t cells = (int64_t)scale_rows * groups;
  const unsigned grid = (unsigned)((cells + kWarpsPerBlock - 1) / kWarpsPerBlock);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    quantize_weight_kernel<T><<<grid, kWarpsPerBlock * 32, 0, s>>>(
        (const T*)w, canonical, wscale, N, K, group_size, head_dim, gph, groups, out_group,
        scale_rows, -qmax - 1.f, qmax);
  });
  return check_launch("lq_quantize_weight");
}

extern "C" int lq_pack_int4(const int8_t* codes, uint8_t* packed, int64_t n_codes, void* stream) {
  using namespace lq;
  LQ_REQUIRE(n_codes >= 0 && n_codes % 2 == 0, LQ_ERR_ARG, "last dim %lld must be even to pack into nibbles", (long long)n_codes);
  if (n_codes == 0) return LQ_OK;
  const int64_t nb = n_codes / 2;
  const int64_t want = (nb + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 32 ? want : 148 * 32);
  pack_int4_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(codes, packed, nb);
  return check_launch("lq_pack_int4");
}

extern "C" int lq_unpack_int4(const uint8_t* packed, int8_t* codes, int64_t n_codes, void* stream) {
  using namespace lq;
  LQ_REQUIRE(n_codes >= 0 && n_codes % 2 == 0, LQ_ERR_ARG, "n_codes %lld must be even", (long long)n_codes);
  if (n_codes == 0) return LQ_OK;
  const int64_t nb = n_codes / 2;
  const int64_t want = (nb + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 32 ? want : 148 * 32);
  unpack_int4_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(packed, codes, nb);
  return check_launch("lq_unpack_int4");
}

extern "C" int lq_dequant_weight(const int8_t* canonical, const float* wscale, void* out, int dtype,
                                 int N, int groups, int group_size, int out_group, void* stream) {
  using namespace lq;
  LQ_REQUIRE(group_size > 0 && group_size % 4 == 0, LQ_ERR_ARG, "group_size must be a multiple of 4, got %d", group_size);
  const int64_t total = (int64_t)N * groups * group_size;
  if (total == 0) return LQ_OK;
  const int64_t want = (total / 4 + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 64 ? want : 148 * 64);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    dequant_weight_kernel<T><<<grid, 256, 0, s>>>(canonical, wscale, (T*)out, total, groups,
                                                  group_size, out_group);
  });
  return check_launch("lq_dequant_weight");
}
