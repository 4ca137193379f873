// Decode GEMV (M <= 8 activation rows) over the streaming layout, plus the layout's
// repack / un-repack kernels.
//
// Layout (see include/llmquant_b200.h): codes [N, Kd] int8 or [N, Kd/2] nibble bytes, rows
// contiguous and 16-byte aligned; scales transposed to [G, SRp]. A warp reads one
// contiguous 512-byte "slab" of a row per instruction (32 lanes x one 128-bit load), so HBM
// sees whole 128-byte lines and nothing is fetched twice.
//
// Work split: a lane owns a fixed 16-byte column position (its "chunk": 16 int8 or 32 int4
// codes, always inside one scale group) and walks DOWN the rows. Everything that depends
// only on the column -- the activation values, their block exponent, the nibble-bias
// correction -- is prepared once per lane and stays in registers; the row loop is: 128-bit
// weight load, dot product, one multiply by the (group, row) scale. Warps of a CTA split the
// K axis (KW of them cover a row) and the rows (RW row-warps); the KW partial sums meet in
// shared memory behind a named barrier that only those KW warps join. No tensor cores: the
// kernel is HBM-bound and the arithmetic is sized to stay under the instruction-issue
// budget of a 6.5 TB/s stream.
//
// Arithmetic variants (argument `variant`):
//   1  fp32: codes turned into floats with a mantissa-injection trick (no I2F), fp32 FMA
//      with the bf16 activations widened exactly. Same operations as the reference kernel
//      (llmquant/cuda/csrc/wq_gemv.cu:78-112), different summation order.
//   2/3  integer dot products (dp4a). The lane's activation chunk is re-expressed exactly as
//      a block-floating-point integer vector (shared power-of-two exponent, 16-bit (2) or
//      24-bit (3) mantissas split into byte planes); chunk sums are exact integer
//      arithmetic, converted once to fp32 and scaled. bf16 inputs within 2^-7 (2) / 2^-15
//      (3) of the chunk maximum are represented exactly; smaller ones are rounded at
//      2^-15 / 2^-23 of the chunk maximum.
#include "common.cuh"

namespace lq {
namespace {

constexpr int kU = 4;           // output rows per batch (one float4 of scales)
constexpr int kMaxWarps = 16;   // warps per CTA

struct GemvParams {
  const __nv_bfloat16* x;
  int ldx;
  const uint8_t* codes;
  const float* scales;
  const __nv_bfloat16* bias;
  const void* residual;
  void* out;
  int out_f32;
  int M, N, K, Kd, rowbytes, span, SRp, out_group;
  int KW, RW, S;
  int nbatch;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ int dp4a_ss(unsigned a, unsigned b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_su(unsigned a, unsigned b, int c) {  // a signed, b unsigned
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_uu(unsigned a, unsigned b, int c) {
  int d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(unsigned a, unsigned b, int c) {  // a unsigned, b signed
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// ------------------------------------------------------------------ per-lane activation state
// VAR 1: the chunk as fp32. VAR 2/3: byte planes of the block-floating-point mantissas,
// ordered like the weight bytes they meet (int4: even-k plane words then odd-k plane words).
template <int BITS, int VAR>
struct XChunk;

template <int BITS>
struct XChunk<BITS, 1> {
  static constexpr int EPL = BITS == 8 ? 16 : 32;
  float v[EPL];
  __device__ __forceinline__ void build(const float* xf) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = xf[i];
  }
  // one row's chunk (four 32-bit words) against this activation chunk
  __device__ __forceinline__ float dot(const uint4& w) const {
    const unsigned ww[4] = {w.x, w.y, w.z, w.w};
    float acc = 0.f;
    if (BITS == 8) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const unsigned u = ww[q] ^ 0x80808080u;  // signed byte -> byte + 128
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          // bytes [b, 0, 0, 0x4B] = float 2^23 + (code + 128)
          const float f = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440u | b));
          acc = fmaf(v[q * 4 + b], f - 8388736.f, acc);
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const unsigned nib = (ww[q] >> (4 * b)) & 0xFu;
          const float f = __uint_as_float(nib | 0x4B000000u);  // 2^23 + (code + 8)
          acc = fmaf(v[q * 8 + b], f - 8388616.f, acc);
        }
      }
    }
    return acc;
  }
};

template <int BITS, int PLANES>
struct XPlanes {
  static constexpr int EPL = BITS == 8 ? 16 : 32;
  static constexpr int WORDS = EPL / 4;  // plane words
  unsigned hi[WORDS];
  unsigned mid[PLANES == 3 ? WORDS : 1];
  unsigned lo[WORDS];
  int bias_hi, bias_mid, bias_lo;  // -8 * sum(plane bytes): the nibble bias, int4 only
  float unit;                      // value of one mantissa unit (a power of two)

  __device__ __forceinline__ void build(const float* xf) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) amax = fmaxf(amax, fabsf(xf[i]));
    // e = floor(log2(amax)), clamped so both powers of two below stay normal floats
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;
    e = max(e, -100);
    constexpr int MBITS = PLANES == 3 ? 22 : 14;  // |mantissa| < 2^(MBITS+1)
    const float up = __uint_as_float((unsigned)(127 + MBITS - e) << 23);
    unit = __uint_as_float((unsigned)(127 - MBITS + e) << 23);
    int m[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) m[i] = __float2int_rn(xf[i] * up);
    int sh = 0, sm = 0, sl = 0;
#pragma unroll
    for (int w = 0; w < WORDS; ++w) {
      unsigned ph = 0, pm = 0, pl = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        // int8: word w byte b meets k = 4w+b. int4: words 0..3 are the even k of weight
        // word w (k = 8w + 2b), words 4..7 the odd k of weight word w-4.
        int k;
        if (BITS == 8) k = 4 * w + b;
        else k = w < 4 ? 8 * w + 2 * b : 8 * (w - 4) + 2 * b + 1;
        const int mv = m[k];
        const int h = PLANES == 3 ? (mv >> 16) : (mv >> 8);
        const int mdl = (mv >> 8) & 0xFF;
        const int l = mv & 0xFF;
        ph |= (unsigned)(h & 0xFF) << (8 * b);
        pm |= (unsigned)mdl << (8 * b);
        pl |= (unsigned)l << (8 * b);
        sh += h; sm += mdl; sl += l;
      }
      hi[w] = ph;
      if (PLANES == 3) mid[w] = pm;
      lo[w] = pl;
    }
    bias_hi = BITS == 4 ? -8 * sh : 0;
    bias_mid = BITS == 4 ? -8 * sm : 0;
    bias_lo = BITS == 4 ? -8 * sl : 0;
  }

  __device__ __forceinline__ float dot(const uint4& w) const {
    const unsigned ww[4] = {w.x, w.y, w.z, w.w};
    int ah = bias_hi, am = bias_mid, al = bias_lo;
    if (BITS == 8) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        ah = dp4a_ss(ww[q], hi[q], ah);
        if (PLANES == 3) am = dp4a_su(ww[q], mid[q], am);
        al = dp4a_su(ww[q], lo[q], al);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const unsigned ev = ww[q] & 0x0F0F0F0Fu;
        const unsigned od = (ww[q] >> 4) & 0x0F0F0F0Fu;
        ah = dp4a_us(ev, hi[q], ah);
        ah = dp4a_us(od, hi[q + 4], ah);
        if (PLANES == 3) {
          am = dp4a_uu(ev, mid[q], am);
          am = dp4a_uu(od, mid[q + 4], am);
        }
        al = dp4a_uu(ev, lo[q], al);
        al = dp4a_uu(od, lo[q + 4], al);
      }
    }
    if (PLANES == 3) return fmaf((float)ah, 65536.f, (float)(am * 256 + al)) * unit;
    return (float)(ah * 256 + al) * unit;
  }
};

template <int BITS>
struct XChunk<BITS, 2> : XPlanes<BITS, 2> {};
template <int BITS>
struct XChunk<BITS, 3> : XPlanes<BITS, 3> {};

// ------------------------------------------------------------------ the kernel
template <int BITS, int VAR, int M, int SPW>
__global__ void __launch_bounds__(kMaxWarps * 32)
gemv_stream_kernel(const GemvParams p) {
  constexpr int EPL = BITS == 8 ? 16 : 32;
  __shared__ float red[2][kMaxWarps][M * kU];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int kw = warp % p.KW;
  const int rw = warp / p.KW;

  // ---- per-lane column state
  XChunk<BITS, VAR> xc[M][SPW];
  int cb[SPW];      // byte offset of the chunk inside a row, -1 if outside the row
  int grp[SPW];     // scale group of the chunk
#pragma unroll
  for (int j = 0; j < SPW; ++j) {
    const int s = kw + j * p.KW;
    const int off = s * 512 + lane * 16;
    const bool live = s < p.S && off < p.rowbytes;
    cb[j] = live ? off : -1;
    const int k0 = live ? off * (8 / BITS) : 0;
    grp[j] = k0 / p.span;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float xf[EPL];
      const __nv_bfloat16* xr = p.x + (int64_t)m * p.ldx + k0;
      const bool full = live && m < p.M && k0 + EPL <= p.K &&
                        ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
      if (full) {
#pragma unroll
        for (int v = 0; v < EPL / 8; ++v) {
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xr) + v);
          const unsigned r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            xf[v * 8 + 2 * t] = __uint_as_float(r[t] << 16);
            xf[v * 8 + 2 * t + 1] = __uint_as_float(r[t] & 0xFFFF0000u);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < EPL; ++i)
          xf[i] = (live && m < p.M && k0 + i < p.K) ? __bfloat162float(xr[i]) : 0.f;
      }
      xc[m][j].build(xf);
    }
  }

  // ---- rows: batches of kU, a contiguous balanced range per row-warp slot
  const int slots = gridDim.x * p.RW;
  const int slot = blockIdx.x * p.RW + rw;
  const int b_begin = (int)(((int64_t)p.nbatch * slot) / slots);
  const int b_end = (int)(((int64_t)p.nbatch * (slot + 1)) / slots);
  // every CTA's row-warps must run the same number of barrier rounds
  const int rounds = (p.nbatch + slots - 1) / slots;
  const int barrier_id = 1 + rw;
  const int barrier_threads = p.KW * 32;

  for (int it = 0; it < rounds; ++it) {
    const int b = b_begin + it;
    const bool active = b < b_end;
    const int n0 = b * kU;
    float acc[M][kU];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int u = 0; u < kU; ++u) acc[m][u] = 0.f;

    if (active) {
      uint4 wv[SPW][kU];
#pragma unroll
      for (int j = 0; j < SPW; ++j)
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int n = min(n0 + u, p.N - 1);
          if (cb[j] >= 0) wv[j][u] = ldg_stream(p.codes + (int64_t)n * p.rowbytes + cb[j]);
          else wv[j][u] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int j = 0; j < SPW; ++j) {
        float sc[kU];
        if (p.out_group == 0) {
          const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.scales + (int64_t)grp[j] * p.SRp + n0));
          sc[0] = s4.x; sc[1] = s4.y; sc[2] = s4.z; sc[3] = s4.w;
        } else {
#pragma unroll
          for (int u = 0; u < kU; ++u)
            sc[u] = __ldg(p.scales + (int64_t)grp[j] * p.SRp + min(n0 + u, p.N - 1) / p.out_group);
        }
        if (cb[j] >= 0) {
#pragma unroll
          for (int u = 0; u < kU; ++u)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[m][u] = fmaf(xc[m][j].dot(wv[j][u]), sc[u], acc[m][u]);
        }
      }
    }

    // ---- reduce over the warp's lanes, then over the KW warps of this row-warp group
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int u = 0; u < kU; ++u) acc[m][u] = warp_sum(acc[m][u]);

    if (p.KW > 1) {
      float* slotp = red[it & 1][warp];
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int u = 0; u < kU; ++u) slotp[m * kU + u] = acc[m][u];
      }
      asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "r"(barrier_threads) : "memory");
    }
    if (kw == 0 && active && lane < M * kU) {
      const int m = lane / kU, u = lane % kU;
      float total;
      if (p.KW > 1) {
        total = 0.f;
        for (int w = 0; w < p.KW; ++w) total += red[it & 1][rw * p.KW + w][lane];
      } else {
        total = 0.f;
#pragma unroll
        for (int mm = 0; mm < M; ++mm)
#pragma unroll
          for (int uu = 0; uu < kU; ++uu)
            if (mm * kU + uu == lane) total = acc[mm][uu];
      }
      const int n = n0 + u;
      if (n < p.N && m < p.M) {
        if (p.bias != nullptr) total += __bfloat162float(p.bias[n]);
        const int64_t o = (int64_t)m * p.N + n;
        if (p.out_f32) {
          if (p.residual != nullptr) total += reinterpret_cast<const float*>(p.residual)[o];
          reinterpret_cast<float*>(p.out)[o] = total;
        } else {
          if (p.residual != nullptr)
            total += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[o]);
          reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(total);
        }
      }
    }
  }
}

template <int BITS, int VAR, int M, int SPW>
int launch_one(const GemvParams& p, int threads, cudaStream_t s) {
  static thread_local int occ_threads = 0, occ = 0;
  if (occ_threads != threads) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_stream_kernel<BITS, VAR, M, SPW>,
                                                      threads, 0) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 1;
    }
    occ = n;
    occ_threads = threads;
  }
  // At least two row batches per row-warp slot, at most one full wave of resident CTAs.
  const int want = (p.nbatch + 2 * p.RW - 1) / (2 * p.RW);
  const int cap = sm_count() * occ;
  int grid = want < cap ? want : cap;
  if (grid < 1) grid = 1;
  gemv_stream_kernel<BITS, VAR, M, SPW><<<grid, threads, 0, s>>>(p);
  return check_launch("lq_wq_gemv_stream");
}

// Activation rows one pass can keep in registers next to SPW column chunks per lane; wider
// requests run as several passes over the weight.
template <int BITS, int VAR>
constexpr int max_rows(int spw) {
  if (spw == 1) return (BITS == 4 && VAR == 1) ? 2 : 4;
  if (spw == 2) return BITS == 8 ? (VAR == 1 ? 1 : 2) : 1;
  return 1;
}

template <int BITS, int VAR>
int launch_m(const GemvParams& p, int spw, int threads, cudaStream_t s) {
  if (spw == 1) {
    if (p.M == 1) return launch_one<BITS, VAR, 1, 1>(p, threads, s);
    if (p.M == 2) return launch_one<BITS, VAR, 2, 1>(p, threads, s);
    if constexpr (max_rows<BITS, VAR>(1) >= 4) return launch_one<BITS, VAR, 4, 1>(p, threads, s);
  } else if (spw == 2) {
    if (p.M == 1) return launch_one<BITS, VAR, 1, 2>(p, threads, s);
    if constexpr (max_rows<BITS, VAR>(2) >= 2) return launch_one<BITS, VAR, 2, 2>(p, threads, s);
  } else if (spw == 4) {
    if (p.M == 1) return launch_one<BITS, VAR, 1, 4>(p, threads, s);
  }
  return fail(LQ_ERR_UNSUPPORTED, "internal: no GEMV instance for M=%d spw=%d", p.M, spw);
}

template <int BITS, int VAR>
int launch_passes(GemvParams p, const void* x, const void* residual, void* out, int M, int spw,
                  int threads, cudaStream_t s) {
  const int step = max_rows<BITS, VAR>(spw);
  const size_t out_es = p.out_f32 ? 4 : 2;
  for (int m0 = 0; m0 < M; m0 += step) {
    p.M = M - m0 < step ? M - m0 : step;
    p.x = (const __nv_bfloat16*)x + (int64_t)m0 * p.ldx;
    p.out = (char*)out + (size_t)m0 * p.N * out_es;
    p.residual = residual ? (const char*)residual + (size_t)m0 * p.N * out_es : nullptr;
    const int rc = launch_m<BITS, VAR>(p, spw, threads, s);
    if (rc) return rc;
  }
  return LQ_OK;
}

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

__global__ void transpose_scales_kernel(const float* __restrict__ wscale, float* __restrict__ scales_t,
                                        int scale_rows, int groups, int SRp, int inverse) {
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t total = (int64_t)groups * SRp;
  for (int64_t i = i0; i < total; i += stride) {
    const int g = (int)(i / SRp), r = (int)(i % SRp);
    if (!inverse) scales_t[i] = r < scale_rows ? wscale[(int64_t)r * groups + g] : 0.f;
    else if (r < scale_rows) const_cast<float*>(wscale)[(int64_t)r * groups + g] = scales_t[i];
  }
}

// streaming layout -> dense [N, K] matrix of T (the real, unpadded reduction width)
template <typename T>
__global__ void dequant_stream_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales_t,
                                      T* __restrict__ out, int N, int K, int rowbytes, int span,
                                      int SRp, int out_group, int bits) {
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
    const float s = scales_t[(int64_t)(k / span) * SRp + (out_group > 0 ? n / out_group : n)];
    out[i] = Conv<T>::from_f32(__fmul_rn((float)code, s));
  }
}

int layout_sizes(int groups, int gs, int head_dim, int bits, int scale_rows, int* Kd, int* span,
                 int* SRp) {
  LQ_REQUIRE(bits == 4 || bits == 8, LQ_ERR_ARG, "unsupported num_bits %d, expected 4 or 8", bits);
  LQ_REQUIRE(groups >= 0 && gs > 0 && head_dim >= 0 && scale_rows >= 0, LQ_ERR_ARG, "bad layout arguments");
  const int sp = (head_dim > 0 && head_dim < gs) ? head_dim : gs;
  const int epl = bits == 8 ? 16 : 32;
  LQ_REQUIRE(sp % epl == 0, LQ_ERR_UNSUPPORTED,
             "group span %d is not a multiple of %d codes; use the canonical-layout GEMV", sp, epl);
  *span = sp;
  *Kd = groups * sp;
  *SRp = (scale_rows + 3) / 4 * 4;
  return LQ_OK;
}

int repack_common(const int8_t* canonical, const float* wscale, void* codes, float* scales_t, int N,
                  int groups, int gs, int head_dim, int bits, int scale_rows, void* stream,
                  int inverse) {
  int Kd, span, SRp;
  const int rc = layout_sizes(groups, gs, head_dim, bits, scale_rows, &Kd, &span, &SRp);
  if (rc) return rc;
  if (N == 0 || groups == 0) return LQ_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = (int64_t)N * Kd * bits / 8;
  if (inverse && span < gs)
    cudaMemsetAsync(const_cast<int8_t*>(canonical), 0, (size_t)N * groups * gs, s);
  int64_t want = (total + 255) / 256;
  repack_codes_kernel<<<(unsigned)(want < 148 * 32 ? want : 148 * 32), 256, 0, s>>>(
      canonical, (uint8_t*)codes, total, groups, gs, span, bits, inverse);
  want = ((int64_t)groups * SRp + 255) / 256;
  transpose_scales_kernel<<<(unsigned)(want < 148 * 8 ? want : 148 * 8), 256, 0, s>>>(
      wscale, scales_t, scale_rows, groups, SRp, inverse);
  return check_launch(inverse ? "lq_unrepack_stream" : "lq_repack_stream");
}

}  // namespace
}  // namespace lq

extern "C" int lq_stream_layout_sizes(int groups, int group_size, int head_dim, int bits,
                                      int scale_rows, int* Kd, int* span, int* SRp) {
  return lq::layout_sizes(groups, group_size, head_dim, bits, scale_rows, Kd, span, SRp);
}

extern "C" int lq_repack_stream(const int8_t* canonical, const float* wscale, void* codes,
                                float* scales_t, int N, int groups, int group_size, int head_dim,
                                int bits, int scale_rows, void* stream) {
  return lq::repack_common(canonical, wscale, codes, scales_t, N, groups, group_size, head_dim,
                           bits, scale_rows, stream, 0);
}

extern "C" int lq_unrepack_stream(const void* codes, const float* scales_t, int8_t* canonical,
                                  float* wscale, int N, int groups, int group_size, int head_dim,
                                  int bits, int scale_rows, void* stream) {
  return lq::repack_common(canonical, wscale, const_cast<void*>(codes), const_cast<float*>(scales_t),
                           N, groups, group_size, head_dim, bits, scale_rows, stream, 1);
}

extern "C" int lq_dequant_stream(const void* codes, const float* scales_t, void* out, int dtype,
                                 int N, int K, int Kd, int span, int SRp, int out_group, int bits,
                                 void* stream) {
  using namespace lq;
  LQ_REQUIRE(bits == 4 || bits == 8, LQ_ERR_ARG, "unsupported num_bits %d, expected 4 or 8", bits);
  LQ_REQUIRE(N >= 0 && K >= 0 && Kd >= K && span > 0, LQ_ERR_ARG, "bad shape N=%d K=%d Kd=%d", N, K, Kd);
  if (N == 0 || K == 0) return LQ_OK;
  const int64_t want = ((int64_t)N * K + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 64 ? want : 148 * 64);
  cudaStream_t s = (cudaStream_t)stream;
  LQ_DISPATCH_DTYPE(dtype, T, {
    dequant_stream_kernel<T><<<grid, 256, 0, s>>>((const uint8_t*)codes, scales_t, (T*)out, N, K,
                                                  Kd * bits / 8, span, SRp, out_group, bits);
  });
  return check_launch("lq_dequant_stream");
}

extern "C" int lq_wq_gemv_stream(const void* x, int ldx, const void* codes, const float* scales_t,
                                 const void* bias, const void* residual, void* out, int out_dtype,
                                 int M, int N, int K, int Kd, int span, int SRp, int out_group,
                                 int bits, int variant, void* stream) {
  using namespace lq;
  LQ_REQUIRE(bits == 4 || bits == 8, LQ_ERR_ARG, "unsupported num_bits %d, expected 4 or 8", bits);
  LQ_REQUIRE(M >= 0 && M <= 8, LQ_ERR_ARG, "the decode GEMV takes at most 8 activation rows, got %d", M);
  LQ_REQUIRE(N >= 0 && K >= 0 && Kd >= K, LQ_ERR_ARG, "bad shape N=%d K=%d Kd=%d", N, K, Kd);
  LQ_REQUIRE(out_dtype == LQ_BF16 || out_dtype == LQ_F32, LQ_ERR_DTYPE, "out must be bfloat16 or float32");
  if (M == 0 || N == 0) return LQ_OK;
  const int epl = bits == 8 ? 16 : 32;
  LQ_REQUIRE(span > 0 && span % epl == 0 && Kd % span == 0, LQ_ERR_ARG,
             "group span %d must be a positive multiple of %d dividing Kd=%d", span, epl, Kd);
  LQ_REQUIRE(SRp % 4 == 0 && out_group >= 0, LQ_ERR_ARG, "scale row pitch must be a multiple of 4");
  LQ_REQUIRE(x && codes && scales_t && out, LQ_ERR_ARG, "null tensor pointer");
  LQ_REQUIRE(((uintptr_t)codes % 16) == 0 && ((uintptr_t)scales_t % 16) == 0, LQ_ERR_ARG,
             "codes and scales must be 16-byte aligned");
  LQ_REQUIRE(ldx >= K, LQ_ERR_ARG, "x row stride %d is shorter than K=%d", ldx, K);
  if (variant == 0) variant = 2;
  LQ_REQUIRE(variant >= 1 && variant <= 3, LQ_ERR_ARG, "unknown arithmetic variant %d", variant);

  GemvParams p;
  p.ldx = ldx; p.codes = (const uint8_t*)codes; p.scales = scales_t;
  p.bias = (const __nv_bfloat16*)bias;
  p.out_f32 = out_dtype == LQ_F32;
  p.N = N; p.K = K; p.Kd = Kd; p.rowbytes = Kd * bits / 8; p.span = span; p.SRp = SRp;
  p.out_group = out_group;
  p.S = (p.rowbytes + 511) / 512;
  int spw = 1;
  while (spw <= 4 && (p.S + spw - 1) / spw > kMaxWarps) spw *= 2;
  LQ_REQUIRE(spw <= 4, LQ_ERR_UNSUPPORTED, "reduction axis too long for the streaming GEMV (Kd=%d)", Kd);
  // keep the per-lane activation state within the register file: M * SPW chunks
  p.KW = (p.S + spw - 1) / spw;
  p.RW = p.KW >= 8 ? 1 : 8 / p.KW;
  p.nbatch = (N + kU - 1) / kU;
  const int threads = p.KW * p.RW * 32;
  cudaStream_t s = (cudaStream_t)stream;

  if (bits == 8) {
    if (variant == 1) return launch_passes<8, 1>(p, x, residual, out, M, spw, threads, s);
    if (variant == 2) return launch_passes<8, 2>(p, x, residual, out, M, spw, threads, s);
    return launch_passes<8, 3>(p, x, residual, out, M, spw, threads, s);
  }
  if (variant == 1) return launch_passes<4, 1>(p, x, residual, out, M, spw, threads, s);
  if (variant == 2) return launch_passes<4, 2>(p, x, residual, out, M, spw, threads, s);
  return launch_passes<4, 3>(p, x, residual, out, M, spw, threads, s);
}
