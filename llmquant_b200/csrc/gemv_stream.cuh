// Decode GEMV (M <= 8 activation rows) over the streaming layout, plus the layout's
// repack / un-repack kernels.
//
// Layout (see include/llmquant_b200.h): codes [N, Kd] int8 or [N, Kd/2] nibble bytes, rows
// contiguous and 16-byte aligned, so four consecutive rows are ONE contiguous piece of
// memory; scales in tiles [ceil(N/4), G, 4] so the scales of those four rows are one
// contiguous piece too.
//
// Data movement: a producer warp streams row tiles (4 rows x the whole K axis, plus their
// scale tile) from HBM into a ring of shared-memory stages with bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier per stage); tens of KB per SM are in
// flight at any time without occupying registers. The first stages are requested BEFORE the
// kernel waits for its producer kernel (programmatic dependent launch), because weights do
// not depend on it.
//
// Work split: KW consumer warps cover the K axis. A lane owns a fixed 16-byte column
// position (its "chunk": 16 int8 or 32 int4 codes, always inside one scale group) and
// walks DOWN the rows. Everything that depends only on the column -- the activation values,
// their block exponent, the nibble-bias correction -- is prepared once per lane and stays in
// registers; per row: one 128-bit shared-memory load, a dot product, one multiply by the
// (group, row) scale. The KW partial sums meet in shared memory behind a named barrier, where a
// further warp (the finisher) picks them up: it adds them, applies bias / residual / SiLU*mul
// and stores, while the consumers are already on the next rows -- the serial tail of a row
// batch is off the path the stream depends on. No tensor cores: the kernel is HBM-bound and
// the arithmetic is sized to stay under the instruction-issue budget of a 6.5 TB/s stream.
//
// Every wait on an mbarrier is bounded by a clock limit; on expiry the kernel records an
// error word (lq_gemv_device_error) and returns instead of spinning.
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
#pragma once
#include "common.cuh"
#include "peer_sync.cuh"

#include <cstdlib>

namespace lq {
namespace gemv {

constexpr int kU = 4;           // output rows per batch (one float4 of scales)
constexpr int kMaxWarps = 16;   // consumer warps per CTA (one more warp produces)
constexpr int kMaxStages = 8;
constexpr int kRingWarps = 20;  // consumer warps per SM the ring depth aims at
constexpr int kRingKb = 112;    // shared memory per SM the rings of one kernel may take (KB)

struct GemvParams {
  const __nv_bfloat16* x;
  int ldx;
  const uint8_t* codes;
  const float* scales;
  const __nv_bfloat16* bias;
  const void* residual;
  void* out;
  int out_f32;
  int ldo;  // elements between two activation rows of out / residual
  int M, N, K, Kd, rowbytes, span, groups;
  int KW, S;
  int nbatch;
  int stages, stage_bytes, tile_bytes, scale_bytes;
  const void* norm_weight;
  float norm_eps;
  int pdl;
  int* error_word;
  unsigned long long* debug;  // optional per-CTA timeline (8 stamps per CTA), normally null
  // tensor-parallel coupling (see lq_gemv_tp): 0 none, LQ_TP_PUSH, LQ_TP_SUM
  int tp_mode, tp_world, tp_rank;
  const uint64_t* tp_peers;
  int64_t tp_data_off;
  float* tp_parts;
  __nv_bfloat16* tp_residual;
  long long tp_wait;
};

// Row-parallel epilogue of a tensor-parallel linear: lane (m, u) of the warp holds output
// (m, n0 + u) of a 4-row batch; lane (m, peer) sends the four values of row m as one 16-byte
// store into part[rank][m][n0 ..] of that peer's exchange buffer.
__device__ __forceinline__ void tp_push_batch(const GemvParams& p, uint64_t peer_base, float total,
                                              int lane, int n0) {
  const int m = lane / p.tp_world;
  const int src = (m < 8 ? m : 0) * kU;
  const float v0 = __shfl_sync(0xffffffffu, total, src);
  const float v1 = __shfl_sync(0xffffffffu, total, src + 1);
  const float v2 = __shfl_sync(0xffffffffu, total, src + 2);
  const float v3 = __shfl_sync(0xffffffffu, total, src + 3);
  if (m < p.M && n0 < p.N) {
    float* dst = reinterpret_cast<float*>(peer_base + p.tp_data_off) +
                 ((int64_t)p.tp_rank * p.M + m) * p.N + n0;
    st_peer_f4(dst, v0, v1, v2, v3);
  }
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Per-CTA phase stamps exist only in diagnostic builds (-DLQ_DIAGNOSTICS).
#ifdef LQ_DIAGNOSTICS
#define LQ_STAMP(slot)                                                             \
  do {                                                                             \
    if (p.debug != nullptr && threadIdx.x == 0) p.debug[(size_t)blockIdx.x * 8 + (slot)] = global_ns(); \
  } while (0)
#else
#define LQ_STAMP(slot) do { } while (0)
#endif

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
    // Mantissas as integers. Two planes: |m| < 2^15, so adding 1.5 * 2^23 in the same FMA
    // leaves round-to-nearest-even(m) in the low mantissa bits (the low 16 bits of the float's
    // pattern are m's two's complement), on the FMA pipe instead of the conversion unit, which
    // the set-up of a whole wave of CTAs would otherwise saturate. Three planes (|m| < 2^23) do
    // not fit that trick and convert.
    int m[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      m[i] = PLANES == 3 ? __float2int_rn(xf[i] * up) : __float_as_int(fmaf(xf[i], up, 12582912.f));
    int sh = 0, sm = 0, sl = 0;
#pragma unroll
    for (int w = 0; w < WORDS; ++w) {
      // int8: word w byte b meets k = 4w+b. int4: words 0..3 are the even k of weight
      // word w (k = 8w + 2b), words 4..7 the odd k of weight word w-4.
      int k[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        if (BITS == 8) k[b] = 4 * w + b;
        else k[b] = w < 4 ? 8 * w + 2 * b : 8 * (w - 4) + 2 * b + 1;
      }
      // byte planes of the four mantissas by byte permutes: byte 0 = low plane, byte 1 = the
      // high (2 planes) or middle (3 planes) one, byte 2 = the high plane of 3
      const unsigned m0 = (unsigned)m[k[0]], m1 = (unsigned)m[k[1]], m2 = (unsigned)m[k[2]], m3 = (unsigned)m[k[3]];
      const unsigned pl = __byte_perm(__byte_perm(m0, m1, 0x0040), __byte_perm(m2, m3, 0x0040), 0x5410);
      const unsigned p1 = __byte_perm(__byte_perm(m0, m1, 0x0051), __byte_perm(m2, m3, 0x0051), 0x5410);
      unsigned ph = p1, pm = 0;
      if (PLANES == 3) {
        pm = p1;
        ph = __byte_perm(__byte_perm(m0, m1, 0x0062), __byte_perm(m2, m3, 0x0062), 0x5410);
      }
      hi[w] = ph;
      if (PLANES == 3) mid[w] = pm;
      lo[w] = pl;
      if (BITS == 4) {  // byte sums for the nibble bias: the high plane is signed, the others unsigned
        sh = dp4a_ss(ph, 0x01010101u, sh);
        if (PLANES == 3) sm = dp4a_uu(pm, 0x01010101u, sm);
        sl = dp4a_uu(pl, 0x01010101u, sl);
      }
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

// Tensor-parallel input of a GEMV: x = bf16(bf16(sum over ranks of the partials) + residual),
// built once by the first CTAs of the grid (each a slice of the row) and read by all of them.
//
// Both hand-overs -- partials from the other GPUs to the CTAs that sum, summed rows from those
// CTAs to every CTA of the grid -- carry their own arrival signal: a 32-bit word of the exchange
// buffer (an fp32 partial) or of a hidden-state row (a pair of bf16) holds the bit pattern
// kTpEmpty (NaNs no computation here produces) until a value is stored there, and a reader
// re-reads a 16-byte piece until none of its words is empty. No flag, no fence, no counter,
// and no second trip over NVLink behind the data. Whoever consumes a buffer for the last time
// before its next use puts kTpEmpty back: the summing thread into the partial words it has
// read and into the residual row it has read (the hidden-state buffers alternate, so that row
// is the next one to be rebuilt). The next write to either is at least one kernel of every
// rank away.
constexpr uint32_t kTpEmpty = 0xFFFFFFFFu;
__device__ __forceinline__ bool tp_piece_missing(const float4& v) {
  return __float_as_uint(v.x) == kTpEmpty || __float_as_uint(v.y) == kTpEmpty ||
         __float_as_uint(v.z) == kTpEmpty || __float_as_uint(v.w) == kTpEmpty;
}
__device__ __forceinline__ bool tp_piece_missing(const uint4& v) {
  return v.x == kTpEmpty || v.y == kTpEmpty || v.z == kTpEmpty || v.w == kTpEmpty;
}
__device__ __forceinline__ uint4 ld_volatile_u4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// 16 bytes of a hidden-state row that other CTAs of this kernel are still writing.
__device__ __forceinline__ uint4 tp_wait_row_piece(const GemvParams& p, const void* src) {
  uint4 v = ld_volatile_u4(src);
  if (tp_piece_missing(v)) {
    const long long t0 = clock64();
    do {
      v = ld_volatile_u4(src);
      if (clock64() - t0 > 2 * p.tp_wait) {  // (twice the partials' limit: their error is the one recorded)
        atomicCAS(p.error_word, 0, 4);
        break;
      }
    } while (tp_piece_missing(v));
  }
  return v;
}
__device__ __forceinline__ void tp_sum_prologue(const GemvParams& p, int KW, int warp, int lane) {
  const int T = KW * 32, tid = warp * 32 + lane;
  const int total4 = p.M * p.K / 4;
  const int R = min((int)gridDim.x, (total4 + T - 1) / T);
  if ((int)blockIdx.x >= R) return;
  __nv_bfloat16* hx = const_cast<__nv_bfloat16*>(p.x);
  const int64_t stride = (int64_t)p.M * p.K;  // floats between two ranks' partials
  const float empty = __uint_as_float(kTpEmpty);
  bool late = false;
  for (int i = blockIdx.x * T + tid; i < total4; i += R * T) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < p.tp_world; r0 += 4) {  // four loads in flight, summed in rank order
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (r0 + j < p.tp_world)
          v[j] = ld_peer_f4(reinterpret_cast<const float4*>(p.tp_parts + (r0 + j) * stride) + i);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (r0 + j < p.tp_world) {
          float4* src = reinterpret_cast<float4*>(p.tp_parts + (r0 + j) * stride) + i;
          if (tp_piece_missing(v[j])) {  // not there yet: wait for it (bounded)
            const long long t0 = clock64();
            do {
              v[j] = ld_peer_f4(src);
              if (clock64() - t0 > p.tp_wait) { late = true; break; }
            } while (tp_piece_missing(v[j]));
          }
          acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w;
          st_peer_f4(reinterpret_cast<float*>(src), empty, empty, empty, empty);
        }
      }
    }
    uint2* res = reinterpret_cast<uint2*>(p.tp_residual) + i;
    const uint2 rr = __ldcg(res);
    const float r4[4] = {__uint_as_float(rr.x << 16), __uint_as_float(rr.x & 0xFFFF0000u),
                         __uint_as_float(rr.y << 16), __uint_as_float(rr.y & 0xFFFF0000u)};
    const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
    unsigned short o4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)  // round the layer output, add the residual stream, round
      o4[j] = __bfloat16_as_ushort(__float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(a4[j])) + r4[j]));
    uint2 packed;
    packed.x = (unsigned)o4[0] | ((unsigned)o4[1] << 16);
    packed.y = (unsigned)o4[2] | ((unsigned)o4[3] << 16);
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(reinterpret_cast<uint2*>(hx) + i), "r"(packed.x),
                 "r"(packed.y) : "memory");
    *res = make_uint2(kTpEmpty, kTpEmpty);  // this row is the next one to be rebuilt
  }
  if (late) atomicCAS(p.error_word, 0, 3);
}

// ------------------------------------------------------------------ the kernel
// Sums four per-lane values over the warp with 6 shuffles: afterwards lane l holds the total
// of value (l & 3).
__device__ __forceinline__ float reduce4(const float (&v)[kU], int lane) {
  const bool o1 = lane & 1, o2 = lane & 2;
  float a = o1 ? v[1] : v[0];
  a += __shfl_xor_sync(0xffffffffu, o1 ? v[0] : v[1], 1);
  float b = o1 ? v[3] : v[2];
  b += __shfl_xor_sync(0xffffffffu, o1 ? v[2] : v[3], 1);
  float c = o2 ? b : a;
  c += __shfl_xor_sync(0xffffffffu, o2 ? a : b, 2);
  c += __shfl_xor_sync(0xffffffffu, c, 4);
  c += __shfl_xor_sync(0xffffffffu, c, 8);
  c += __shfl_xor_sync(0xffffffffu, c, 16);
  return c;
}

// EPI 0: out[m, n] = acc (+ bias) (+ residual).  EPI 1: rows come in (gate, up) pairs and
// out[m, n/2] = silu(gate) * up with the roundings of a bf16 MLP (gate, up, silu(gate) and
// the product are each rounded to bf16).
// TP: 0 = no tensor-parallel coupling (the kernel every single-GPU launch uses, with none of
// the coupling's code in it), LQ_TP_PUSH, LQ_TP_SUM.
template <int BITS, int VAR, int M, int SPW, int EPI, int TP>
__global__ void __launch_bounds__((kMaxWarps + 2) * 32)
gemv_stream_kernel(const GemvParams p) {
  constexpr int EPL = BITS == 8 ? 16 : 32;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages];
  __shared__ float red[2][kMaxWarps][M * kU];
  __shared__ float nrm[kMaxWarps][M];
  __shared__ volatile int dead_s;  // a pipeline wait expired: everyone winds down

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int KW = p.KW;
  const int barrier_threads = KW * 32;
  LQ_STAMP(0);

  // contiguous balanced range of row batches for this CTA
  const int b_begin = (int)(((int64_t)p.nbatch * blockIdx.x) / gridDim.x);
  const int b_end = (int)(((int64_t)p.nbatch * (blockIdx.x + 1)) / gridDim.x);
  const int nb = b_end - b_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), KW);
    }
    dead_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // With more than one consumer warp a further warp (index KW + 1) finishes the rows: it sums
  // the consumers' partials of a batch and runs the epilogue while they are already on the
  // next batch. One named barrier per batch, which it shares, hands a batch over; the
  // partials are double-buffered, and because the finisher arrives at a barrier only after
  // it is done with the batch before, a buffer is never overwritten while it is read.
  const int round_threads = (KW + 1) * 32;

  // ------------------------------------------------------------ producer warp
  if (warp == KW) {
    if (lane == 0) {
      int s = 0, wrap = 0;  // ring slot and how often the ring has wrapped, kept without divisions
      for (int it = 0; it < nb; ++it) {
        if (it >= p.stages) {
          if (!mbar_wait(smem_u32(&empty_bar[s]), (wrap - 1) & 1)) {
            atomicExch(p.error_word, 1);
            break;
          }
        }
        const int b = b_begin + it;
        const int rows = min(kU, p.N - b * kU);
        const uint32_t bytes = (uint32_t)rows * p.rowbytes;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t dst = smem_u32(ring + (size_t)s * p.stage_bytes);
        mbar_expect_tx(bar, bytes + p.scale_bytes);
        bulk_g2s(dst, p.codes + (int64_t)b * kU * p.rowbytes, bytes, bar);
        bulk_g2s(dst + p.tile_bytes, p.scales + (int64_t)b * p.groups * kU, p.scale_bytes, bar);
        if (++s == p.stages) { s = 0; ++wrap; }
      }
    }
    return;
  }

  // ------------------------------------------------------------ finisher warp
  if (warp == KW + 1) {
    constexpr bool push = EPI == 0 && TP == LQ_TP_PUSH;
    uint64_t peer_base = 0;
    if constexpr (push) peer_base = p.tp_peers[lane % p.tp_world];
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the residual comes from earlier kernels
    for (int it = 0; it < nb; ++it) {
      const int parity = it & 1;
      const int n0 = (b_begin + it) * kU;
      const int m = lane / kU, u = lane % kU;
      const int n = n0 + u;
      const bool mine = lane < M * kU && n < p.N && m < p.M;
      // bias and residual do not depend on the products: fetch them before the hand-over
      float bias_pre = 0.f, res_pre = 0.f;
      if (EPI == 0 && mine) {
        if (p.bias != nullptr) bias_pre = __bfloat162float(p.bias[n]);
        if (p.residual != nullptr) {
          const int64_t po = (int64_t)m * p.ldo + n;
          res_pre = p.out_f32 ? reinterpret_cast<const float*>(p.residual)[po]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[po]);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"r"(round_threads) : "memory");
      if (dead_s) return;
      float total = 0.f;
      if (lane < M * kU) {
        float t0 = 0.f, t1 = 0.f;  // two chains, so the loads of a pair are in flight together
        int w = 0;
        for (; w + 1 < KW; w += 2) {
          t0 += red[parity][w][lane];
          t1 += red[parity][w + 1][lane];
        }
        if (w < KW) t0 += red[parity][w][lane];
        total = t0 + t1;
      }
      if (EPI == 1) {
        const float up = __shfl_down_sync(0xffffffffu, total, 1);
        if (lane < M * kU && (u & 1) == 0 && n + 1 < p.N && m < p.M) {
          const float g = __bfloat162float(__float2bfloat16_rn(total));
          const float uq = __bfloat162float(__float2bfloat16_rn(up));
          const float sg = __bfloat162float(__float2bfloat16_rn(g / (1.f + expf(-g))));
          const float y = sg * uq;
          const int64_t o = (int64_t)m * p.ldo + n / 2;
          if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = __bfloat162float(__float2bfloat16_rn(y));
          else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(y);
        }
      } else if constexpr (push) {
        tp_push_batch(p, peer_base, total + bias_pre, lane, n0);
      } else if (mine) {
        total += bias_pre;
        const int64_t o = (int64_t)m * p.ldo + n;
        if (p.out_f32) {
          reinterpret_cast<float*>(p.out)[o] = total + res_pre;
        } else {
          // a bf16 layer output added to a bf16 residual stream: round, add, round
          if (p.residual != nullptr) total = __bfloat162float(__float2bfloat16_rn(total)) + res_pre;
          reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(total);
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------ consumer warps
  const int kw = warp;
  int cb[SPW];   // byte offset of the chunk inside a row, -1 if outside the row
  int grp[SPW];  // scale group of the chunk
#pragma unroll
  for (int j = 0; j < SPW; ++j) {
    const int s = kw + j * KW;
    const int off = s * 512 + lane * 16;
    const bool live = s < p.S && off < p.rowbytes;
    cb[j] = live ? off : -1;
    grp[j] = live ? (off * (8 / BITS)) / p.span : 0;
  }

  // Column chunks that can be fetched with 128-bit loads keep their raw bf16 pairs in
  // registers, so x is read from memory exactly once (for the norm's sum of squares and for
  // the conversion); ragged or unaligned chunks fall back to scalar loads.
  constexpr int PW = EPL / 2;  // packed bf16 pairs per chunk
  bool fast[SPW];
  int k0s[SPW];
#pragma unroll
  for (int j = 0; j < SPW; ++j) {
    k0s[j] = cb[j] >= 0 ? cb[j] * (8 / BITS) : 0;
    fast[j] = cb[j] >= 0 && k0s[j] + EPL <= p.K && (p.ldx % 8) == 0 &&
              ((reinterpret_cast<uintptr_t>(p.x + k0s[j]) & 15) == 0);
  }
  // the norm weight is a constant of the model: fetch it before waiting for the producer
  uint32_t graw[SPW][PW];
  const bool has_norm = p.norm_weight != nullptr;
  if (has_norm) {
#pragma unroll
    for (int j = 0; j < SPW; ++j) {
      const __nv_bfloat16* gw = reinterpret_cast<const __nv_bfloat16*>(p.norm_weight) + k0s[j];
      if (fast[j] && ((reinterpret_cast<uintptr_t>(gw) & 15) == 0)) {
#pragma unroll
        for (int v = 0; v < PW / 4; ++v) {
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(gw) + v);
          graw[j][4 * v] = raw.x; graw[j][4 * v + 1] = raw.y; graw[j][4 * v + 2] = raw.z; graw[j][4 * v + 3] = raw.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < PW; ++i) {
          const int k = k0s[j] + 2 * i;
          const unsigned lo = (cb[j] >= 0 && k < p.K) ? __bfloat16_as_ushort(gw[2 * i]) : 0u;
          const unsigned hi = (cb[j] >= 0 && k + 1 < p.K) ? __bfloat16_as_ushort(gw[2 * i + 1]) : 0u;
          graw[j][i] = lo | (hi << 16);
        }
      }
    }
  }

  // x is produced by the kernel before this one: wait for it (a no-op without programmatic
  // dependent launch), then let the kernel after this one start its own weight stream.
  LQ_STAMP(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  LQ_STAMP(2);

  // ---- tensor-parallel input: the hidden rows are first built from the ranks' partial sums
  constexpr bool tp_sum = TP == LQ_TP_SUM;
  if constexpr (tp_sum) tp_sum_prologue(p, KW, warp, lane);

  uint32_t xraw[M][SPW][PW];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int j = 0; j < SPW; ++j) {
      const __nv_bfloat16* xr = p.x + (int64_t)m * p.ldx + k0s[j];
      if (fast[j] && m < p.M) {
#pragma unroll
        for (int v = 0; v < PW / 4; ++v) {
          // rows other CTAs of this kernel are writing: wait for each piece to be there
          uint4 raw;
          if constexpr (tp_sum) raw = tp_wait_row_piece(p, reinterpret_cast<const uint4*>(xr) + v);
          else raw = __ldg(reinterpret_cast<const uint4*>(xr) + v);
          xraw[m][j][4 * v] = raw.x; xraw[m][j][4 * v + 1] = raw.y;
          xraw[m][j][4 * v + 2] = raw.z; xraw[m][j][4 * v + 3] = raw.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < PW; ++i) {
          const int k = k0s[j] + 2 * i;
          const bool ok = cb[j] >= 0 && m < p.M;
          unsigned lo, hi;
          if constexpr (tp_sum) {  // rows written by another CTA of this kernel: no cached path
            const volatile unsigned short* xv = reinterpret_cast<const volatile unsigned short*>(xr);
            lo = (ok && k < p.K) ? xv[2 * i] : 0u;
            hi = (ok && k + 1 < p.K) ? xv[2 * i + 1] : 0u;
          } else {
            lo = (ok && k < p.K) ? __bfloat16_as_ushort(xr[2 * i]) : 0u;
            hi = (ok && k + 1 < p.K) ? __bfloat16_as_ushort(xr[2 * i + 1]) : 0u;
          }
          xraw[m][j][i] = lo | (hi << 16);
        }
      }
    }

  // ---- optional fused RMSNorm: rstd[m] = 1 / sqrt(mean(x^2) + eps) over the whole row
  float rstd[M];
  if (has_norm) {
    float ss[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      ss[m] = 0.f;
#pragma unroll
      for (int j = 0; j < SPW; ++j)
#pragma unroll
        for (int i = 0; i < PW; ++i) {
          const float lo = __uint_as_float(xraw[m][j][i] << 16);
          const float hi = __uint_as_float(xraw[m][j][i] & 0xFFFF0000u);
          ss[m] = fmaf(lo, lo, ss[m]);
          ss[m] = fmaf(hi, hi, ss[m]);
        }
      ss[m] = warp_sum(ss[m]);
    }
    LQ_STAMP(6);
    if (KW > 1) {
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) nrm[warp][m] = ss[m];
      }
      asm volatile("bar.sync 2, %0;" ::"r"(barrier_threads) : "memory");
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float t = 0.f;
        for (int w = 0; w < KW; ++w) t += nrm[w][m];
        ss[m] = t;
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) rstd[m] = __frsqrt_rn(ss[m] / (float)p.K + p.norm_eps);
    LQ_STAMP(7);
  }

  // ---- per-lane activation state
  XChunk<BITS, VAR> xc[M][SPW];
#pragma unroll
  for (int j = 0; j < SPW; ++j) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float xf[EPL];
#pragma unroll
      for (int i = 0; i < PW; ++i) {
        xf[2 * i] = __uint_as_float(xraw[m][j][i] << 16);
        xf[2 * i + 1] = __uint_as_float(xraw[m][j][i] & 0xFFFF0000u);
      }
      if (has_norm) {
        // weight * bf16(x * rstd), the product rounded to bf16 again: the two roundings of
        // a bf16 RMSNorm module
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const uint32_t gp = graw[j][i >> 1];
          const float g = __uint_as_float((i & 1) ? (gp & 0xFFFF0000u) : (gp << 16));
          const float nx = __bfloat162float(__float2bfloat16_rn(xf[i] * rstd[m]));
          xf[i] = __bfloat162float(__float2bfloat16_rn(g * nx));
        }
      }
      xc[m][j].build(xf);
    }
  }

  LQ_STAMP(3);
  // ---- the row loop over the ring
  const uint32_t ring_base = smem_u32(ring);
  int s = 0, phase = 0;  // ring slot and its phase bit, kept without divisions
  for (int it = 0; it < nb; ++it) {
    const int parity = it & 1;
    const int n0 = (b_begin + it) * kU;
    // bias and residual of this batch's outputs do not depend on the tile: fetch them now,
    // so their latency hides behind the wait for the tile and the dot products
    float bias_pre = 0.f, res_pre = 0.f;
    if (EPI == 0 && KW == 1 && lane < M * kU) {  // with a finisher warp, that warp fetches them
      const int pm = lane / kU, pn = n0 + lane % kU;
      if (pn < p.N && pm < p.M) {
        if (p.bias != nullptr) bias_pre = __bfloat162float(p.bias[pn]);
        if (p.residual != nullptr) {
          const int64_t po = (int64_t)pm * p.ldo + pn;
          res_pre = p.out_f32 ? reinterpret_cast<const float*>(p.residual)[po]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[po]);
        }
      }
    }
    if (!mbar_wait(smem_u32(&full_bar[s]), phase)) {
      // the KW warps wait for the same stage, so they all give up here together; the finisher
      // is released from its barrier and sees the flag
      if (lane == 0) atomicExch(p.error_word, 2);
      if (KW > 1) {
        dead_s = 1;
        asm volatile("bar.arrive 1, %0;" ::"r"(round_threads) : "memory");
      }
      return;
    }
    if (it == 0) LQ_STAMP(4);
    const uint32_t stage = ring_base + (uint32_t)s * p.stage_bytes;
    uint4 wv[SPW][kU];
    float sc[SPW][kU];
#pragma unroll
    for (int j = 0; j < SPW; ++j) {
      if (cb[j] >= 0) {
#pragma unroll
        for (int u = 0; u < kU; ++u) wv[j][u] = lds128(stage + u * p.rowbytes + cb[j]);
        const uint4 s4 = lds128(stage + p.tile_bytes + grp[j] * 16);
        sc[j][0] = __uint_as_float(s4.x); sc[j][1] = __uint_as_float(s4.y);
        sc[j][2] = __uint_as_float(s4.z); sc[j][3] = __uint_as_float(s4.w);
      }
    }
    // the loads above must have returned before the arrival that lets the next bulk copy
    // overwrite the stage: an arrival is not held back by an earlier shared-memory load of its
    // warp whose data is still on its way (seen in decode_gemm.cu under a busy load path)
    __threadfence_block();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));  // the stage can be refilled
    if (++s == p.stages) { s = 0; phase ^= 1; }

    float acc[M][kU];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int u = 0; u < kU; ++u) acc[m][u] = 0.f;
#pragma unroll
    for (int j = 0; j < SPW; ++j) {
      if (cb[j] >= 0) {
#pragma unroll
        for (int u = 0; u < kU; ++u)
#pragma unroll
          for (int m = 0; m < M; ++m)
            acc[m][u] = fmaf(xc[m][j].dot(wv[j][u]), sc[j][u], acc[m][u]);
      }
    }
    float tot[M];
#pragma unroll
    for (int m = 0; m < M; ++m) tot[m] = reduce4(acc[m], lane);  // lane l: row (l & 3)

    if (KW > 1) {
      if (lane < kU) {
#pragma unroll
        for (int m = 0; m < M; ++m) red[parity][warp][m * kU + lane] = tot[m];
      }
      // hand the batch to the finisher warp (which arrives once it is done with the one before)
      asm volatile("bar.sync 1, %0;" ::"r"(round_threads) : "memory");
    } else {
      constexpr bool push = EPI == 0 && TP == LQ_TP_PUSH;
      float total = 0.f;
      // lane u (< 4) holds row u for every m: lane (m, u) fetches it (all lanes shuffle)
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float v = __shfl_sync(0xffffffffu, tot[m], lane % kU);
        if (lane / kU == m) total = v;
      }
      const int m = lane / kU, u = lane % kU;
      const int n = n0 + u;
      if (EPI == 1) {
        const float up = __shfl_down_sync(0xffffffffu, total, 1);
        if (lane < M * kU && (u & 1) == 0 && n + 1 < p.N && m < p.M) {
          const float g = __bfloat162float(__float2bfloat16_rn(total));
          const float uq = __bfloat162float(__float2bfloat16_rn(up));
          const float sg = __bfloat162float(__float2bfloat16_rn(g / (1.f + expf(-g))));
          const float y = sg * uq;
          const int64_t o = (int64_t)m * p.ldo + n / 2;
          if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = __bfloat162float(__float2bfloat16_rn(y));
          else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(y);
        }
      } else if constexpr (push) {
        tp_push_batch(p, p.tp_peers[lane % p.tp_world], total + bias_pre, lane, n0);
      } else if (lane < M * kU && n < p.N && m < p.M) {
        total += bias_pre;
        const int64_t o = (int64_t)m * p.ldo + n;
        if (p.out_f32) {
          reinterpret_cast<float*>(p.out)[o] = total + res_pre;
        } else {
          // a bf16 layer output added to a bf16 residual stream: round, add, round
          if (p.residual != nullptr) total = __bfloat162float(__float2bfloat16_rn(total)) + res_pre;
          reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(total);
        }
      }
    }
  }
  LQ_STAMP(5);
}

template <int BITS, int VAR, int M, int SPW, int EPI, int TP = 0>
int launch_tp(const GemvParams& p, int threads, cudaStream_t s) {
  auto kern = gemv_stream_kernel<BITS, VAR, M, SPW, EPI, TP>;
  const size_t smem = (size_t)p.stages * p.stage_bytes;
  if (const int rc = ensure_smem_limit(reinterpret_cast<const void*>(kern), 200 * 1024, "lq_wq_gemv")) return rc;
  static thread_local int occ_threads = 0, occ = 0, occ_dev = -1;
  static thread_local size_t occ_smem = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (occ_threads != threads || occ_smem != smem || occ_dev != dev) {
    occ_dev = dev;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 1;
    }
    occ = n;
    occ_threads = threads;
    occ_smem = smem;
  }
  // A single resident wave: one row batch per CTA until every SM holds its complement. The
  // rings of one kernel are kept to about half an SM's shared memory, so that the CTAs of the
  // NEXT kernel on the stream (programmatic dependent launch) find room to become resident
  // and fill their own rings while this kernel is still computing.
  int per_sm = occ;
  const int by_smem = (int)(((size_t)kRingKb * 1024) / (smem > 0 ? smem : 1));
  if (by_smem >= 1 && per_sm > by_smem) per_sm = by_smem;
#ifdef LQ_DIAGNOSTICS
  if (const char* e = getenv("LQ_X_PERSM")) {  // diagnostic builds: resident CTAs per SM
    const int want = atoi(e);
    if (want >= 1 && want <= occ) per_sm = want;
  }
#endif
  const int cap = sm_count() * per_sm;
  int grid = p.nbatch < cap ? p.nbatch : cap;
  if (grid < 1) grid = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "lq_wq_gemv: %s", cudaGetErrorString(e));
  }
  return LQ_OK;
}

// The tensor-parallel instances exist for the default arithmetic (variant 2) only.
template <int BITS, int VAR, int M, int SPW, int EPI>
int launch_one(const GemvParams& p, int threads, cudaStream_t s) {
  if (p.tp_mode == 0) return launch_tp<BITS, VAR, M, SPW, EPI, 0>(p, threads, s);
  if constexpr (VAR == 2 && SPW <= 2) {
    if (p.tp_mode == LQ_TP_SUM) return launch_tp<BITS, VAR, M, SPW, EPI, LQ_TP_SUM>(p, threads, s);
    if constexpr (EPI == 0) {
      if (p.tp_mode == LQ_TP_PUSH) return launch_tp<BITS, VAR, M, SPW, EPI, LQ_TP_PUSH>(p, threads, s);
    }
  }
  return fail(LQ_ERR_UNSUPPORTED, "no tensor-parallel GEMV instance for this variant / shape (variant %d, %d column "
              "chunks per lane, epilogue %d)", VAR, SPW, EPI);
}

// Activation rows one pass can keep in registers next to SPW column chunks per lane; wider
// requests run as several passes over the weight.
template <int BITS, int VAR>
constexpr int max_rows(int spw) {
  if (spw == 1) return BITS == 4 ? 2 : 4;  // keep the instances free of register spills
  if (spw == 2) return BITS == 8 ? (VAR == 1 ? 1 : 2) : 1;
  return 1;
}

template <int BITS, int VAR, int EPI>
int launch_m(const GemvParams& p, int spw, int threads, cudaStream_t s) {
  if (spw == 1) {
    if (p.M == 1) return launch_one<BITS, VAR, 1, 1, EPI>(p, threads, s);
    if (p.M == 2) return launch_one<BITS, VAR, 2, 1, EPI>(p, threads, s);
    if constexpr (max_rows<BITS, VAR>(1) >= 4) return launch_one<BITS, VAR, 4, 1, EPI>(p, threads, s);
  } else if (spw == 2) {
    if (p.M == 1) return launch_one<BITS, VAR, 1, 2, EPI>(p, threads, s);
    if constexpr (max_rows<BITS, VAR>(2) >= 2) return launch_one<BITS, VAR, 2, 2, EPI>(p, threads, s);
  } else if (spw == 4) {
    if constexpr (EPI == 0) {
      if (p.M == 1) return launch_one<BITS, VAR, 1, 4, 0>(p, threads, s);
    }
  }
  return fail(LQ_ERR_UNSUPPORTED, "internal: no GEMV instance for M=%d spw=%d", p.M, spw);
}

template <int BITS, int VAR>
int launch_passes(GemvParams p, const lq_gemv_args& a, int spw, int threads, cudaStream_t s) {
  const int step = max_rows<BITS, VAR>(spw);
  if (p.tp_mode != 0 && a.M > step)
    return fail(LQ_ERR_UNSUPPORTED, "the tensor-parallel coupling takes the rows of one pass (%d > %d)", a.M, step);
  const size_t out_es = p.out_f32 ? 4 : 2;
  const int n_out = a.epilogue == 1 ? a.N / 2 : a.N;
  for (int m0 = 0; m0 < a.M; m0 += step) {
    p.M = a.M - m0 < step ? a.M - m0 : step;
    p.x = (const __nv_bfloat16*)a.x + (int64_t)m0 * p.ldx;
    p.out = (char*)a.out + (size_t)m0 * p.ldo * out_es;
    p.residual = a.residual ? (const char*)a.residual + (size_t)m0 * p.ldo * out_es : nullptr;
    const int rc = a.epilogue == 1 ? launch_m<BITS, VAR, 1>(p, spw, threads, s)
                                   : launch_m<BITS, VAR, 0>(p, spw, threads, s);
    if (rc) return rc;
  }
  return LQ_OK;
}

}  // namespace gemv
}  // namespace lq
