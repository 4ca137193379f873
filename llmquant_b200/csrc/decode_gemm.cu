// Decode GEMM: the quantized linear for a small batch of activation rows (up to 64 tokens of
// a decode step) on the 5th-generation tensor cores, with the WEIGHTS on the 128-row side of
// the MMA and the tokens on its narrow side.
//
// Why another kernel: the GEMVs (gemv_stream.cuh, gemv_mma.cu) take at most 8 rows per pass over
// the weights, so 32 sequences stream every weight four times, and their per-weight instruction
// count makes even one pass issue-bound. Here the tensor core does all multiplications, the
// weights are streamed once for all tokens, and the CUDA cores only move bytes, widen int4
// nibbles and apply scales.
//
// Three launches per linear:
//   act_planes_kernel   x [T, K] bf16 (optionally through RMSNorm) -> per scale group of 128
//                       columns a power-of-two unit and 15-bit signed mantissas split into a
//                       signed high byte plane and a signed low byte plane (the block
//                       floating point of gemv_mma.cu), laid out as the B operand tiles:
//                       planes[g][2 * TP][128] int8 (rows 0..TP-1 high planes, TP..2TP-1 low
//                       planes), units[g][TP] fp32.
//   decode_gemm_kernel  one CTA per (128 weight rows, slice of the scale groups). Per group:
//                       A = 128 rows x 128 codes as signed bytes (int8 codes as they are; int4
//                       nibbles as 16 * code, the 1/16 folded into the scale), B = the group's
//                       2 * TP plane rows, four tcgen05.mma kind::i8 (K = 32 each) into one of
//                       two TMEM accumulators [128 lanes = weight rows][2 * TP columns]. Warp
//                       roles as in the prefill kernel: 4 fill warps (cp.async into 128-byte
//                       swizzled tiles, three groups ahead), one MMA-issuing thread, 8 drain
//                       warps (tcgen05.ld; hi * 256 + lo; times weight scale x unit; fp32
//                       registers). This is the reference's order of operations: one exact
//                       product sum per group, scaled, accumulated in fp32 over the groups
//                       (quantizers/real.py:93-99). The CTA's sums go to partial[split][T][N].
//   decode_finish_kernel  adds the splits in order, then bias / residual / silu(gate) * up and
//                       the roundings of the bf16 modules, and stores the output rows.
//
// Every wait is bounded (mbar_wait); on expiry the CTA records the error word, all roles leave
// their loops, TMEM is freed.
#include "common.cuh"
#include "tcgen05.cuh"

namespace lq {
namespace {

constexpr int kDgThreads = 416;  // 8 drain warps, 4 fill warps, 1 MMA warp
constexpr int kDgStages = 5;     // shared-memory stages (operand tiles of one group each)
constexpr int kDgAhead = 3;      // groups whose copies are in flight ahead of the one handed over
constexpr int kDgRows = 128;     // weight rows per CTA = TMEM lanes
constexpr int KT = 128;          // codes per scale group = bytes per operand row

__device__ int g_decode_gemm_error = 0;

struct DgParams {
  const uint8_t* codes;      // streaming layout [N, rowbytes]
  const float* scale_tiles;  // [N/4, G, 4]
  const int8_t* planes;      // [G][2 * TP][128]
  const float* units;        // [G][TP]
  float* partial;            // [splits][T][N]
  int T, N, groups, rowbytes, gper;
  int* error_word;
};

constexpr uint32_t dg_idesc(int ncol) {
  // D = s32, A = B = s8, both K-major, N = ncol, M = 128
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ncol >> 3) << 17) | ((uint32_t)(kDgRows >> 4) << 24);
}

template <int BITS, int TP>
__global__ void __launch_bounds__(kDgThreads)
decode_gemm_kernel(const DgParams p) {
  constexpr int NCOL = 2 * TP;                      // accumulator columns: high planes, low planes
  constexpr int TMEM_COLS = 2 * NCOL < 32 ? 32 : 2 * NCOL;
  constexpr int A_TILE = kDgRows * KT;              // 16 KB
  constexpr int B_TILE = NCOL * KT;
  constexpr int STAGE = A_TILE + B_TILE;
  constexpr int RAW = kDgRows * (KT / 2);           // int4: a group's nibble bytes as they come
  constexpr int DW = TP >= 16 ? 8 : 4;              // drain warps in use
  constexpr int TPH = TP / (DW / 4);                // tokens per drain thread
  constexpr int CH = TPH < 16 ? 8 : 16;             // tokens per tensor-memory load
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar[kDgStages], sfree_bar[kDgStages], tfull_bar[2], tfree_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ float ws_s[8][kDgRows];
  __shared__ __align__(16) float us_s[8][TP];
  __shared__ volatile int dead_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kDgRows;
  const int g_lo = blockIdx.y * p.gper;
  const int GL = min(p.gper, p.groups - g_lo);  // groups of this CTA
  uint8_t* const tiles = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
  constexpr uint32_t kIdesc = dg_idesc(NCOL);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int i = 0; i < kDgStages; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 128);
      mbar_init(smem_u32(&sfree_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tfree_bar[i]), DW * 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    dead_s = 0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  // the planes come from the kernel before this one
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp >= 8 && warp < 12) {
    // ------------------------------------------------------------------ fill
    const int ft = tid - 256;  // 0..127 among the fill threads; also the row whose scale it stages
    const int n = n0 + ft;
    uint8_t* const raw_base = tiles + kDgStages * STAGE;
    auto cp16 = [](uint32_t dst, const void* src, bool valid) {
      const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    };
    auto issue = [&](const int j) -> bool {  // j: group index within this CTA's slice
      const int st = j % kDgStages, g = g_lo + j;
      if (j >= kDgStages && !mbar_wait(smem_u32(&sfree_bar[st]), ((j / kDgStages) - 1) & 1)) return false;
      const uint32_t a_tile = smem_u32(tiles + st * STAGE), b_tile = a_tile + A_TILE;
      if (BITS == 8) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {  // piece (row, kc) = item / 8, item % 8
          const int item = it * 128 + ft, row = item >> 3, kc = item & 7;
          const int nn = n0 + row;
          cp16(a_tile + (uint32_t)row * 128 + ((kc ^ (row & 7)) << 4),
               p.codes + (int64_t)(nn < p.N ? nn : 0) * p.rowbytes + g * KT + kc * 16, nn < p.N);
        }
      } else {
#pragma unroll
        for (int it = 0; it < 4; ++it) {  // staging piece (row, q) = item / 4, item % 4
          const int item = it * 128 + ft, row = item >> 2, q = item & 3;
          const int nn = n0 + row;
          cp16(smem_u32(raw_base + st * RAW + item * 16),
               p.codes + (int64_t)(nn < p.N ? nn : 0) * p.rowbytes + g * (KT / 2) + q * 16, nn < p.N);
        }
      }
      // the group's plane rows: contiguous in global memory, piece (row, kc) = item / 8, item % 8
      const int8_t* psrc = p.planes + (int64_t)g * B_TILE;
#pragma unroll
      for (int it = 0; it < (NCOL * 8 + 127) / 128; ++it) {
        const int item = it * 128 + ft, row = item >> 3, kc = item & 7;
        if (NCOL * 8 >= 128 || item < NCOL * 8)
          cp16(b_tile + (uint32_t)row * 128 + ((kc ^ (row & 7)) << 4), psrc + item * 16, true);
      }
      {
        const float* ssrc = p.scale_tiles + ((int64_t)((n < p.N ? n : 0) >> 2) * p.groups + g) * 4 + (n & 3);
        const int bytes = n < p.N ? 4 : 0;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
                     ::"r"(smem_u32(&ws_s[j & 7][ft])), "l"(ssrc), "r"(bytes) : "memory");
      }
      if (ft < TP / 4) cp16(smem_u32(&us_s[j & 7][ft * 4]), p.units + (int64_t)g * TP + ft * 4, true);
      asm volatile("cp.async.commit_group;" ::: "memory");
      return true;
    };
    bool ok = true;
    for (int j = 0; j < kDgAhead && j < GL && ok; ++j) ok = issue(j);
    for (int j = 0; j < GL && ok; ++j) {
      const int st = j % kDgStages;
      if (dead_s) break;
      // the copies of group j are complete once at most (groups issued after j) are pending
      const int after = min(kDgAhead - 1, GL - 1 - j);
      if (after >= 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
      else if (after == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      if (BITS == 4) {
        uint8_t* a_tile = tiles + st * STAGE;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int item = it * 128 + ft, row = item >> 2, q = item & 3;
          const uint4 v = *reinterpret_cast<const uint4*>(raw_base + st * RAW + item * 16);
          const unsigned w4[4] = {v.x, v.y, v.z, v.w};
          unsigned o[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // word of 8 nibbles (code + 8): even positions and odd positions as bytes 16 * code,
            // interleaved back into K order. A zero-filled row (beyond N) becomes bytes -128:
            // its outputs are never stored.
            const unsigned ev = ((w4[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
            const unsigned od = (w4[i] & 0xF0F0F0F0u) ^ 0x80808080u;
            o[2 * i] = __byte_perm(ev, od, 0x5140);      // codes 0..3 of the word
            o[2 * i + 1] = __byte_perm(ev, od, 0x7362);  // codes 4..7
          }
          uint8_t* rowp = a_tile + row * 128;
          *reinterpret_cast<uint4*>(rowp + (((2 * q) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(rowp + (((2 * q + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic / cp.async writes -> MMA reads
      mbar_arrive(smem_u32(&full_bar[st]));
      if (j + kDgAhead < GL) ok = issue(j + kDgAhead);
    }
    if (!ok) dead_s = 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == 12) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      for (int j = 0; j < GL; ++j) {
        const int st = j % kDgStages, tb = j & 1;
        if (dead_s) break;
        if (!mbar_wait(smem_u32(&full_bar[st]), (j / kDgStages) & 1)) { dead_s = 1; break; }
        if (j >= 2 && !mbar_wait(smem_u32(&tfree_bar[tb]), ((j >> 1) - 1) & 1)) { dead_s = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(tiles + st * STAGE), b_addr = a_addr + A_TILE;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          // 32 bytes of K per MMA: the start address moves along the 128-byte row
          mma_i8(tmem_base + tb * NCOL, smem_desc_sw128(a_addr + s * 32), smem_desc_sw128(b_addr + s * 32),
                 kIdesc, s > 0);
        }
        mma_commit(smem_u32(&sfree_bar[st]));
        mma_commit(smem_u32(&tfull_bar[tb]));
      }
    }
  } else if (warp < DW) {
    // ------------------------------------------------------------------ drain
    float acc[TPH];
#pragma unroll
    for (int c = 0; c < TPH; ++c) acc[c] = 0.f;
    const int quarter = warp & 3, t0 = (warp >> 2) * TPH;  // TMEM lanes and tokens of this warp
    const int row = quarter * 32 + lane, nrow = n0 + row;
    bool dead = false;
    for (int j = 0; j < GL; ++j) {
      const int tb = j & 1;
      if (dead_s) { dead = true; break; }
      if (!mbar_wait(smem_u32(&tfull_bar[tb]), (j >> 1) & 1)) { dead_s = 1; dead = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // (the scales of group j were complete before its tiles were handed to the MMA thread)
      const float wsx = ws_s[j & 7][row] * (BITS == 4 ? 0.0625f : 1.f);  // 1/16: nibbles ride as 16 * code
      const uint32_t taddr = tmem_base + tb * NCOL + ((uint32_t)(quarter * 32) << 16) + t0;
#pragma unroll
      for (int c0 = 0; c0 < TPH; c0 += CH) {
        uint32_t hi[CH], lo[CH];
        tmem_ld(taddr + c0, hi);
        tmem_ld(taddr + TP + c0, lo);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < CH; q += 4) {
          const float4 u = *reinterpret_cast<const float4*>(&us_s[j & 7][t0 + c0 + q]);
          const float uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            acc[c0 + q + e] = fmaf((float)((int)hi[q + e] * 256 + (int)lo[q + e]), uu[e] * wsx, acc[c0 + q + e]);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(smem_u32(&tfree_bar[tb]));
    }
    if (!dead && nrow < p.N) {
      float* dst = p.partial + ((int64_t)blockIdx.y * p.T + t0) * p.N + nrow;
#pragma unroll
      for (int c = 0; c < TPH; ++c)
        if (t0 + c < p.T) dst[(int64_t)c * p.N] = acc[c];
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && dead_s) atomicExch(p.error_word, 1);
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// x [T, K] bf16 -> B operand tiles. One CTA per token row (rows T .. TP-1 are written as zeros);
// a thread owns 16-column chunks, the eight lanes of a scale group agree on its exponent.
constexpr int kApThreads = 256;

__device__ __forceinline__ void ap_load16(const __nv_bfloat16* base, int k0, int K, bool vec, float (&f)[16]) {
  if (vec && k0 + 16 <= K) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(base + k0));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(base + k0) + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = k0 + i < K ? __bfloat162float(base[k0 + i]) : 0.f;
  }
}

__global__ void __launch_bounds__(kApThreads)
act_planes_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ norm_weight,
                  float norm_eps, int8_t* __restrict__ planes, float* __restrict__ units, int T, int TP, int K,
                  int groups) {
  __shared__ float red_s[kApThreads / 32];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunk = groups * 8;  // 16-column chunks of the padded row
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const bool live = t < T;
  const __nv_bfloat16* xr = x + (int64_t)(live ? t : 0) * ldx;
  const bool vec_x = (ldx % 8) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const bool vec_g = norm_weight != nullptr && (reinterpret_cast<uintptr_t>(norm_weight) & 15) == 0;
  float rstd = 0.f;
  if (norm_weight != nullptr && live) {
    float ss = 0.f;
    for (int ch = tid; ch < nchunk; ch += kApThreads) {
      float f[16];
      ap_load16(xr, ch * 16, K, vec_x, f);
#pragma unroll
      for (int i = 0; i < 16; ++i) ss = fmaf(f[i], f[i], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) red_s[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < kApThreads / 32; ++w) tot += red_s[w];
    rstd = __frsqrt_rn(tot / (float)K + norm_eps);
  }
  // all threads of a warp run the same number of rounds (the exponent is agreed by shuffles)
  for (int base = 0; base < nchunk; base += kApThreads) {
    const int ch = base + tid;
    const bool valid = ch < nchunk;
    float f[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = 0.f;
    if (valid && live) {
      ap_load16(xr, ch * 16, K, vec_x, f);
      if (norm_weight != nullptr) {
        float gf[16];
        ap_load16(norm_weight, ch * 16, K, vec_g, gf);
        // weight * bf16(x * rstd), the product rounded to bf16 again: the two roundings of a
        // bf16 RMSNorm module
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float nx = __bfloat162float(__float2bfloat16_rn(f[i] * rstd));
          f[i] = __bfloat162float(__float2bfloat16_rn(gf[i] * nx));
        }
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;
    e = max(e, -100);
    // |mantissa| + 128 must stay below 2^15 so that the rounded high byte fits a signed byte
    if (__float2int_rn(amax * __uint_as_float((unsigned)(127 + 14 - e) << 23)) >= 32640) ++e;
    const float up = __uint_as_float((unsigned)(127 + 14 - e) << 23);
    unsigned hw[4] = {0, 0, 0, 0}, lw[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      // round-to-nearest-even by adding 1.5 * 2^23 in the FMA (|m| < 2^15), not a conversion
      const int m = __float_as_int(fmaf(f[i], up, 12582912.f)) - 0x4B400000;
      const int h = (m + 128) >> 8;
      const int l = m - h * 256;
      hw[i >> 2] |= (unsigned)(h & 0xFF) << (8 * (i & 3));
      lw[i >> 2] |= (unsigned)(l & 0xFF) << (8 * (i & 3));
    }
    if (valid) {
      const int g = ch >> 3, sub = ch & 7;
      int8_t* hp = planes + ((int64_t)g * 2 * TP + t) * KT + sub * 16;
      *reinterpret_cast<uint4*>(hp) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
      *reinterpret_cast<uint4*>(hp + (int64_t)TP * KT) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
      if (sub == 0) units[(int64_t)g * TP + t] = live && amax > 0.f ? __uint_as_float((unsigned)(127 + e - 14) << 23) : 0.f;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// out = epilogue(sum over the splits): EPI 0 bias / residual, EPI 1 silu(gate) * up over
// interleaved (gate, up) rows, with the roundings of gemv_stream_kernel's epilogues.
template <int EPI>
__global__ void __launch_bounds__(256)
decode_finish_kernel(const float* __restrict__ partial, int splits, int T, int N, const __nv_bfloat16* __restrict__ bias,
                     const void* __restrict__ residual, void* __restrict__ out, int out_f32, int ldo) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int NO = EPI == 1 ? N / 2 : N;
  const int64_t total = (int64_t)T * NO;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / NO), j = (int)(i % NO);
    const int64_t o = (int64_t)t * ldo + j;
    if (EPI == 1) {
      float2 gu = make_float2(0.f, 0.f);
      for (int s = 0; s < splits; ++s) {
        const float2 v = *reinterpret_cast<const float2*>(partial + ((int64_t)s * T + t) * N + 2 * j);
        gu.x += v.x;
        gu.y += v.y;
      }
      const float g = __bfloat162float(__float2bfloat16_rn(gu.x));
      const float uq = __bfloat162float(__float2bfloat16_rn(gu.y));
      const float sg = __bfloat162float(__float2bfloat16_rn(g / (1.f + expf(-g))));
      const float y = sg * uq;
      if (out_f32) reinterpret_cast<float*>(out)[o] = __bfloat162float(__float2bfloat16_rn(y));
      else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(y);
    } else {
      float total_v = 0.f;
      for (int s = 0; s < splits; ++s) total_v += partial[((int64_t)s * T + t) * N + j];
      if (bias != nullptr) total_v += __bfloat162float(bias[j]);
      if (out_f32) {
        float r = 0.f;
        if (residual != nullptr) r = reinterpret_cast<const float*>(residual)[o];
        reinterpret_cast<float*>(out)[o] = total_v + r;
      } else {
        // a bf16 layer output added to a bf16 residual stream: round, add, round
        if (residual != nullptr)
          total_v = __bfloat162float(__float2bfloat16_rn(total_v)) +
                    __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(residual)[o]);
        reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(total_v);
      }
    }
  }
}

template <typename Kern, typename... Args>
int launch_dep(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t s, int pdl, const char* what, Args... args) {
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
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  return LQ_OK;
}

int tokens_padded(int M) { return M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64)); }

// Slices of the scale groups per row tile: enough CTAs to fill the GPU's SMs, in as few
// waves as possible (a CTA occupies an SM by itself).
int choose_splits(int tiles, int groups) {
  const int sms = sm_count();
  int best = 1;
  long best_cost = -1;
  for (int ks = 1; ks <= 8 && ks <= groups; ++ks) {
    const int gper = (groups + ks - 1) / ks;
    if ((ks - 1) * gper >= groups) continue;  // the last slice would be empty
    const long waves = ((long)tiles * ks + sms - 1) / sms;
    const long cost = waves * (gper + 4);  // 4: set-up and drain of a CTA, in group times
    if (best_cost < 0 || cost < best_cost) { best = ks; best_cost = cost; }
  }
  return best;
}

struct Workspace {
  int8_t* planes;
  float* units;
  float* partial;
  int64_t bytes;
};
Workspace carve(void* base, int TP, int M, int N, int groups, int splits) {
  Workspace w;
  int64_t off = 0;
  w.planes = reinterpret_cast<int8_t*>(reinterpret_cast<uint8_t*>(base) + off);
  off += (int64_t)groups * 2 * TP * KT;
  w.units = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(base) + off);
  off += ((int64_t)groups * TP * 4 + 255) / 256 * 256;
  w.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(base) + off);
  off += (int64_t)splits * M * N * 4;
  w.bytes = off;
  return w;
}

}  // namespace

namespace gemv {

// The decode GEMM behind lq_wq_gemv_fused (variant 5). The caller has validated the common fields.
int run_decode_gemm(const lq_gemv_args& a, cudaStream_t s) {
  LQ_REQUIRE(a.span == 128 && a.Kd % 128 == 0, LQ_ERR_UNSUPPORTED,
             "the decode GEMM needs scale groups of 128 stored codes (span=%d, Kd=%d)", a.span, a.Kd);
  LQ_REQUIRE(a.M >= 1 && a.M <= 64, LQ_ERR_ARG, "the decode GEMM takes 1..64 rows, got %d", a.M);
  LQ_REQUIRE(a.tp == nullptr, LQ_ERR_ARG, "the decode GEMM has no tensor-parallel coupling");
  LQ_REQUIRE(a.workspace != nullptr && (reinterpret_cast<uintptr_t>(a.workspace) & 255) == 0, LQ_ERR_ARG,
             "the decode GEMM needs a 256-byte aligned workspace");
  LQ_REQUIRE(a.epilogue == 0 || a.N % 2 == 0, LQ_ERR_ARG, "the gate|up epilogue needs an even number of rows");
  const int groups = a.Kd / 128, TP = tokens_padded(a.M), tiles = (a.N + kDgRows - 1) / kDgRows;
  const int splits = choose_splits(tiles, groups);
  const Workspace w = carve(a.workspace, TP, a.M, a.N, groups, splits);
  LQ_REQUIRE(w.bytes <= a.workspace_bytes, LQ_ERR_ARG, "the decode GEMM needs %lld bytes of workspace, got %lld",
             (long long)w.bytes, (long long)a.workspace_bytes);
  void* err_ptr = nullptr;
  if (cudaGetSymbolAddress(&err_ptr, g_decode_gemm_error) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "cannot resolve the device error word");
  }
  if (const int rc = launch_dep(act_planes_kernel, dim3((unsigned)TP), dim3(kApThreads), 0, s, a.pdl, "lq_wq_gemv_fused",
                                (const __nv_bfloat16*)a.x, a.ldx, (const __nv_bfloat16*)a.norm_weight, a.norm_eps,
                                w.planes, w.units, a.M, TP, a.K, groups))
    return rc;
  DgParams p;
  p.codes = (const uint8_t*)a.codes; p.scale_tiles = a.scale_tiles; p.planes = w.planes; p.units = w.units;
  p.partial = w.partial; p.T = a.M; p.N = a.N; p.groups = groups; p.rowbytes = a.Kd * a.bits / 8;
  p.gper = (groups + splits - 1) / splits; p.error_word = (int*)err_ptr;
  const dim3 grid((unsigned)tiles, (unsigned)splits);
  int rc = LQ_ERR_UNSUPPORTED;
#define LQ_DG_CASE(B, TPV)                                                                              \
  if (a.bits == B && TP == TPV) {                                                                       \
    auto kern = decode_gemm_kernel<B, TPV>;                                                             \
    const size_t smem = (size_t)kDgStages * (kDgRows * KT + 2 * TPV * KT) + (B == 4 ? (size_t)kDgStages * kDgRows * (KT / 2) : 0) + 1024; \
    if (const int rs = ensure_smem_limit(reinterpret_cast<const void*>(kern), (int)smem, "lq_wq_gemv_fused")) return rs; \
    rc = launch_dep(kern, grid, dim3(kDgThreads), smem, s, a.pdl, "lq_wq_gemv_fused", p);               \
  }
  LQ_DG_CASE(4, 8) LQ_DG_CASE(4, 16) LQ_DG_CASE(4, 32) LQ_DG_CASE(4, 64)
  LQ_DG_CASE(8, 8) LQ_DG_CASE(8, 16) LQ_DG_CASE(8, 32) LQ_DG_CASE(8, 64)
#undef LQ_DG_CASE
  if (rc == LQ_ERR_UNSUPPORTED) return fail(LQ_ERR_UNSUPPORTED, "no decode GEMM instance for bits=%d", a.bits);
  if (rc) return rc;
  const int NO = a.epilogue == 1 ? a.N / 2 : a.N;
  const int ldo = a.ldo > 0 ? a.ldo : NO;
  const int64_t total = (int64_t)a.M * NO;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
  if (a.epilogue == 1)
    return launch_dep(decode_finish_kernel<1>, dim3(blocks), dim3(256), 0, s, a.pdl, "lq_wq_gemv_fused",
                      (const float*)w.partial, splits, a.M, a.N, (const __nv_bfloat16*)a.bias, a.residual, a.out,
                      a.out_dtype == LQ_F32 ? 1 : 0, ldo);
  return launch_dep(decode_finish_kernel<0>, dim3(blocks), dim3(256), 0, s, a.pdl, "lq_wq_gemv_fused",
                    (const float*)w.partial, splits, a.M, a.N, (const __nv_bfloat16*)a.bias, a.residual, a.out,
                    a.out_dtype == LQ_F32 ? 1 : 0, ldo);
}

}  // namespace gemv
}  // namespace lq

extern "C" int64_t lq_decode_gemm_workspace_bytes(int M, int N, int Kd) {
  if (M < 1 || M > 64 || N < 1 || Kd < 128) return 0;
  const int groups = Kd / 128;
  const int TP = lq::tokens_padded(M);
  const int splits = lq::choose_splits((N + lq::kDgRows - 1) / lq::kDgRows, groups);
  return lq::carve(nullptr, TP, M, N, groups, splits).bytes;
}

extern "C" int lq_decode_gemm_device_error(void) {
  int value = 0;
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_decode_gemm_error) != cudaSuccess) return -1;
  if (cudaMemcpy(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(ptr, 0, sizeof(int));
  return value;
}
