// Prefill GEMM (more than 8 activation rows) on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory (TMEM), operands staged in shared memory
// in the canonical K-major core-matrix layout, dequantization of the weight codes done by the
// CTA's threads on the way into shared memory (the integer codes are exactly representable in
// bf16 / int8, so the tensor core multiplies exact integers), and the per-group scale applied
// in the epilogue that drains TMEM:
//
//     out[m, n] = sum_g s_w[n, g] * (s_x[m, g]) * sum_{k in g} a[m, k] * q[n, k]
//
// which is the order of operations of the reference's real mode (quantizers/real.py:93-99):
// one exact product sum per 128-wide group, scaled, accumulated in fp32 across groups. Two
// operand modes: A16 (bf16 activations x codes widened to bf16, kind::f16, fp32 accumulate)
// and A8 (activations quantized per token per group to int8 codes, kind::i8, int32
// accumulate, both scales in the epilogue).
//
// Tile: 128 tokens x 128 output features per CTA, one scale group (span = 64 or 128 K
// elements) per round: fill A and B tiles, one thread issues span/16 (bf16) or span/32 (int8)
// MMAs and commits them to an mbarrier, all four warps drain the 128x128 accumulator
// (tcgen05.ld, one TMEM lane = one token row per thread), scale, and add into registers.
// Every wait is bounded; on expiry the kernel records an error word, frees its TMEM and
// returns. This first version does not overlap the fill of the next group with the MMAs of the
// current one.
//
// The reference dequantizes the whole weight to bf16 and calls cuBLAS above its row threshold
// (quantizers/kernel.py:68-79,90-91); its own fused tensor-core prototype was rejected at
// 0.34x cuBLAS.
#include "common.cuh"
#include "tcgen05.cuh"

namespace lq {
namespace {

constexpr int BM = 128, BN = 128, kThreads = 128;
constexpr int kTmemCols = 128;

// instruction descriptor: D format, A/B formats, K-major both, N/8 and M/16
constexpr uint32_t idesc(uint32_t c_fmt, uint32_t ab_fmt) {
  return (c_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((uint32_t)(BN >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

struct GemmParams {
  const __nv_bfloat16* x;   // [M, K] (A16) -- unused for A8
  int ldx;
  const int8_t* x_codes;    // [M, Kd] int8 (A8) or null
  const float* x_scales;    // [M, G] (A8)
  const uint8_t* codes;     // streaming layout
  const float* scale_tiles; // [NP/4, G, 4]
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;       // [M, N]
  int M, N, K, Kd, span, groups, rowbytes;
  int* error_word;
};

// ES = bytes per operand element (2: bf16 operands, 1: int8 operands)
template <int BITS, int ES>
__global__ void __launch_bounds__(kThreads)
prefill_gemm_kernel(const GemmParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t mma_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ float ws_s[BN];
  __shared__ int dead_s;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const int KT = p.span;                        // K elements per round (one scale group)
  constexpr int CORE_K = 16 / ES;               // K elements per core-matrix row
  const int cores_k = KT / CORE_K;              // core matrices along K
  const uint32_t lbo = 128, sbo = (uint32_t)cores_k * 128;
  const int tile_bytes = BM * KT * ES;          // A tile; the B tile has the same size
  uint8_t* a_tile = smem;
  uint8_t* b_tile = smem + tile_bytes;
  const uint32_t a_addr = smem_u32(a_tile), b_addr = smem_u32(b_tile);
  const uint32_t bar = smem_u32(&mma_bar);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    dead_s = 0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  float acc[BN];
#pragma unroll
  for (int c = 0; c < BN; ++c) acc[c] = 0.f;
  const int my_m = m0 + tid;  // this thread's token row (TMEM lane tid)

  constexpr uint32_t kIdesc = ES == 2 ? idesc(1, 1) : idesc(2, 1);  // f32 <- bf16 x bf16 ; s32 <- s8 x s8
  const int pieces = BM * cores_k;  // 16-byte core-matrix rows per tile
  uint32_t phase = 0;

  for (int g = 0; g < p.groups; ++g) {
    const int kbase = g * KT;
    // ---- A tile: activations of this group, row r / K chunk kc -> core matrix (r/8, kc)
    for (int idx = tid; idx < pieces; idx += kThreads) {
      const int r = idx / cores_k, kc = idx % cores_k;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int m = m0 + r;
      if (m < p.M) {
        if (ES == 2) {
          const int k = kbase + kc * CORE_K;
          const __nv_bfloat16* src = p.x + (int64_t)m * p.ldx + k;
          if (k + CORE_K <= p.K && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
            v = __ldg(reinterpret_cast<const uint4*>(src));
          } else {
            __nv_bfloat16 t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = k + j < p.K ? src[j] : __float2bfloat16_rn(0.f);
            v = *reinterpret_cast<uint4*>(t);
          }
        } else {
          v = __ldg(reinterpret_cast<const uint4*>(p.x_codes + (int64_t)m * p.Kd + kbase + kc * CORE_K));
        }
      }
      *reinterpret_cast<uint4*>(a_tile + (r >> 3) * sbo + kc * lbo + (r & 7) * 16) = v;
    }
    // ---- B tile: weight codes of rows n0.. widened to the operand type (exact)
    for (int idx = tid; idx < pieces; idx += kThreads) {
      const int r = idx / cores_k, kc = idx % cores_k;
      const int n = n0 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (n < p.N) {
        const int k = kbase + kc * CORE_K;  // stored-K index
        int8_t c[16];
        if (BITS == 8) {
          const uint8_t* src = p.codes + (int64_t)n * p.rowbytes + k;
          if (CORE_K == 8) *reinterpret_cast<uint2*>(c) = __ldg(reinterpret_cast<const uint2*>(src));
          else *reinterpret_cast<uint4*>(c) = __ldg(reinterpret_cast<const uint4*>(src));
        } else {
          const uint8_t* src = p.codes + (int64_t)n * p.rowbytes + (k >> 1);
          uint8_t b[8];
          if (CORE_K == 8) *reinterpret_cast<uint32_t*>(b) = __ldg(reinterpret_cast<const uint32_t*>(src));
          else *reinterpret_cast<uint2*>(b) = __ldg(reinterpret_cast<const uint2*>(src));
#pragma unroll
          for (int j = 0; j < CORE_K / 2; ++j) {
            c[2 * j] = (int8_t)((int)(b[j] & 0xF) - 8);
            c[2 * j + 1] = (int8_t)((int)(b[j] >> 4) - 8);
          }
        }
        if (ES == 2) {
          __nv_bfloat16 t[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] = __float2bfloat16_rn((float)c[j]);
          v = *reinterpret_cast<uint4*>(t);
        } else {
          v = *reinterpret_cast<uint4*>(c);
        }
      }
      *reinterpret_cast<uint4*>(b_tile + (r >> 3) * sbo + kc * lbo + (r & 7) * 16) = v;
    }
    // ---- the weight scales of this group for the tile's 128 columns
    {
      const int n = n0 + tid;
      ws_s[tid] = n < p.N ? p.scale_tiles[((int64_t)(n >> 2) * p.groups + g) * 4 + (n & 3)] : 0.f;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic stores -> async reads
    __syncthreads();

    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int steps = KT / (32 / ES);  // 32 bytes of K per MMA: 16 bf16 or 32 int8
      for (int s = 0; s < steps; ++s) {
        const uint64_t da = smem_desc(a_addr + s * 2 * lbo, lbo, sbo);
        const uint64_t db = smem_desc(b_addr + s * 2 * lbo, lbo, sbo);
        if (ES == 2) mma_f16(tmem_base, da, db, kIdesc, s > 0);
        else mma_i8(tmem_base, da, db, kIdesc, s > 0);
      }
      mma_commit(bar);
    }
    if (!mbar_wait(bar, phase)) dead_s = 1;  // bounded; every thread waits on the same phase
    phase ^= 1;
    __syncthreads();
    if (dead_s) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- drain: TMEM lane = token row of this thread, 4 x 32 columns
    const float xs = (ES == 1 && my_m < p.M) ? p.x_scales[(int64_t)my_m * p.groups + g] : 1.f;
#pragma unroll
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t v[32];
      tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + c0, v);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float d = ES == 2 ? __uint_as_float(v[j]) : (float)(int)v[j];
        acc[c0 + j] = fmaf(d, ws_s[c0 + j] * xs, acc[c0 + j]);
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // TMEM and the tiles are free for the next group
  }

  if (dead_s) {
    if (tid == 0) atomicExch(p.error_word, 1);
  } else if (my_m < p.M) {
    __nv_bfloat16* dst = p.out + (int64_t)my_m * p.N + n0;
#pragma unroll
    for (int c = 0; c < BN; ++c) {
      if (n0 + c < p.N) {
        float y = acc[c];
        if (p.bias != nullptr) y += __bfloat162float(p.bias[n0 + c]);
        dst[c] = __float2bfloat16_rn(y);
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}


// ---------------------------------------------------------------------------------------------
// Pipelined variant for int8 activations (kind::i8) and scale groups of 128 codes: three roles
// in one CTA, so that the tensor pipe, the dequantizing fill and the scaling drain overlap.
//
//   warps 0-7  drain: wait for a group's accumulator in TMEM, tcgen05.ld their part (warp w
//              reads TMEM lanes 32 (w % 4) .. + 31 = token rows, columns 64 (w / 4) .. + 63),
//              multiply by (activation scale x weight scale) and add into registers; hand the
//              accumulator back.
//   warps 8-11 fill: token codes and weight codes of the next group into one of two
//              shared-memory stages in the K-major core-matrix layout; int4 nibbles become the
//              signed byte 16 * code ((n ^ 8) << 4, exact; the 1/16 goes into the scale) and
//              are interleaved back into K order with byte permutes.
//   warp 12    one thread issues the group's four MMAs into one of two TMEM accumulators and
//              commits them to two mbarriers: "stage free" for the fill warps, "accumulator
//              ready" for the drain warps.
//
// Handshakes are mbarriers with bounded waits; a wait that expires marks the CTA dead, every
// role leaves its loop, the error word is set and TMEM is freed.
constexpr int kWsThreads = 416;  // 8 drain warps, 4 fill warps, 1 MMA warp
constexpr int kWsStages = 5;   // shared-memory stages (operand tiles of one group each)
constexpr int kWsAcc = 4;      // accumulators in tensor memory (128 columns each): the MMA -> drain -> hand-back
                               // loop is several hundred clocks of latency, which two accumulators do not cover
constexpr int kWsAhead = 3;    // groups whose copies are in flight ahead of the one being handed over; two
                               // fewer than the stages, so a refill waits for an MMA issued two groups ago

template <int BITS>
__global__ void __launch_bounds__(kWsThreads)
prefill_gemm_ws_kernel(const GemmParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar[kWsStages], sfree_bar[kWsStages], tfull_bar[kWsAcc], tfree_bar[kWsAcc];
  __shared__ uint32_t tmem_base_s;
  __shared__ float ws_s[16][BN];  // a slot is rewritten 16 groups later: by then its drain is done (4 accumulators, 5 stages)
  __shared__ volatile int dead_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  constexpr int KT = 128;                        // one group: 128 codes = one 128-byte row per tile row
  constexpr int TILE = BM * KT;                  // bytes of an A or B tile (int8 operands)
  // Operand tiles: row r at r * 128, its 16-byte piece kc at ((kc ^ (r & 7)) * 16) -- the
  // 128-byte swizzle of the MMA descriptor. Eight lanes that copy the eight pieces of one row
  // read one 128-byte line of global memory and write all 32 banks once.
  uint8_t* const tiles = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
  constexpr uint32_t kIdesc = idesc(2, 1);       // s32 <- s8 x s8

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kWsAcc * kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int i = 0; i < kWsStages; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 4);  // one arrival per fill warp (an arrival is an atomic on the barrier word)
      mbar_init(smem_u32(&sfree_bar[i]), 1);
    }
    for (int i = 0; i < kWsAcc; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tfree_bar[i]), 8);  // one arrival per drain warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    dead_s = 0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  const int G = p.groups;

  if (warp >= 8 && warp < 12) {
    // ------------------------------------------------------------------ fill
    const int ft = tid - 256;  // 0..127 among the fill threads
    const int r = ft;          // the column whose weight scale this thread stages
    const int n = n0 + r;
    uint8_t* raw_base = tiles + kWsStages * 2 * TILE;  // int4: the rows' nibble bytes as they come
    // Operands travel with cp.async (16 bytes per copy, no registers), kWsAhead groups ahead
    // of the group being handed to the MMA thread, so the trip to L2 / HBM is off the critical
    // path. Token codes and int8 weight codes land directly in the swizzled tile; int4 weight
    // rows land in staging rows and are widened from there by the thread that copied them.
    auto cp16 = [](uint32_t dst, const void* src, bool valid) {
      const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    };
    auto issue = [&](const int g) -> bool {
      const int st = g % kWsStages;
      if (g >= kWsStages && !mbar_wait(smem_u32(&sfree_bar[st]), ((g / kWsStages) - 1) & 1)) return false;
      const uint32_t a_tile = smem_u32(tiles + st * 2 * TILE), b_tile = a_tile + TILE;
#pragma unroll
      for (int it = 0; it < 8; ++it) {  // piece (row, kc) = item / 8, item % 8
        const int item = it * 128 + ft, row = item >> 3, kc = item & 7;
        const uint32_t dst = (uint32_t)row * 128 + ((kc ^ (row & 7)) << 4);
        const int m = m0 + row;
        cp16(a_tile + dst, reinterpret_cast<const uint8_t*>(p.x_codes) + (int64_t)(m < p.M ? m : 0) * p.Kd + g * KT + kc * 16,
             m < p.M);
        if (BITS == 8) {
          const int nn = n0 + row;
          cp16(b_tile + dst, p.codes + (int64_t)(nn < p.N ? nn : 0) * p.rowbytes + g * KT + kc * 16, nn < p.N);
        }
      }
      if (BITS == 4) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {  // staging piece (row, q) = item / 4, item % 4
          const int item = it * 128 + ft, row = item >> 2, q = item & 3;
          const int nn = n0 + row;
          cp16(smem_u32(raw_base + st * (BN * 64) + item * 16),
               p.codes + (int64_t)(nn < p.N ? nn : 0) * p.rowbytes + g * (KT / 2) + q * 16, nn < p.N);
        }
      }
      {
        const float* ssrc = p.scale_tiles + ((int64_t)((n < p.N ? n : 0) >> 2) * G + g) * 4 + (n & 3);
        const int bytes = n < p.N ? 4 : 0;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
                     ::"r"(smem_u32(&ws_s[g & 15][r])), "l"(ssrc), "r"(bytes) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      return true;
    };
    bool ok = true;
    for (int g = 0; g < kWsAhead && g < G && ok; ++g) ok = issue(g);
    for (int g = 0; g < G && ok; ++g) {
      const int st = g % kWsStages;
      if (dead_s) break;
      // the copies of group g are complete once at most (groups issued after g) are pending
      const int after = min(kWsAhead - 1, G - 1 - g);
      if (after >= 3) asm volatile("cp.async.wait_group 3;" ::: "memory");
      else if (after == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
      else if (after == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      if (BITS == 4) {
        uint8_t* b_tile = tiles + st * 2 * TILE + TILE;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int item = it * 128 + ft, row = item >> 2, q = item & 3;
          const uint4 v = *reinterpret_cast<const uint4*>(raw_base + st * (BN * 64) + item * 16);
          const unsigned w4[4] = {v.x, v.y, v.z, v.w};
          unsigned o[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // word of 8 nibbles (code + 8): even positions and odd positions as bytes 16 * code.
            // A zero-filled row (beyond N) becomes bytes -128: its columns are never stored.
            const unsigned ev = ((w4[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
            const unsigned od = (w4[i] & 0xF0F0F0F0u) ^ 0x80808080u;
            o[2 * i] = __byte_perm(ev, od, 0x5140);      // codes 0..3 of the word
            o[2 * i + 1] = __byte_perm(ev, od, 0x7362);  // codes 4..7
          }
          uint8_t* rowp = b_tile + row * 128;
          *reinterpret_cast<uint4*>(rowp + (((2 * q) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(rowp + (((2 * q + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic / cp.async writes -> MMA reads
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&full_bar[st]));
      if (g + kWsAhead < G) ok = issue(g + kWsAhead);
    }
    if (!ok) dead_s = 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == 12) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      for (int g = 0; g < G; ++g) {
        const int st = g % kWsStages, tb = g % kWsAcc;
        if (dead_s) break;
        if (!mbar_wait(smem_u32(&full_bar[st]), (g / kWsStages) & 1)) { dead_s = 1; break; }
        if (g >= kWsAcc && !mbar_wait(smem_u32(&tfree_bar[tb]), ((g / kWsAcc) - 1) & 1)) { dead_s = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(tiles + st * 2 * TILE), b_addr = a_addr + TILE;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          // 32 bytes of K per MMA: the start address moves along the 128-byte row
          const uint64_t da = smem_desc_sw128(a_addr + s * 32);
          const uint64_t db = smem_desc_sw128(b_addr + s * 32);
          mma_i8(tmem_base + tb * kTmemCols, da, db, kIdesc, s > 0);
        }
        mma_commit(smem_u32(&sfree_bar[st]));
        mma_commit(smem_u32(&tfull_bar[tb]));
      }
    }
  } else {
    // ------------------------------------------------------------------ drain
    constexpr int HALF = BN / 2;
    float acc[HALF];
#pragma unroll
    for (int c = 0; c < HALF; ++c) acc[c] = 0.f;
    const int quarter = warp & 3, cbase = (warp >> 2) * HALF;  // TMEM lanes and columns of this warp
    const int my_m = m0 + quarter * 32 + lane;
    bool dead = false;
    for (int g = 0; g < G; ++g) {
      const int st = g % kWsAcc;
      if (dead_s) { dead = true; break; }
      // 1/16 undoes the shift that turned int4 codes into signed bytes
      const float xs = my_m < p.M ? p.x_scales[(int64_t)my_m * G + g] * (BITS == 4 ? 0.0625f : 1.f) : 0.f;
      if (!mbar_wait(smem_u32(&tfull_bar[st]), (g / kWsAcc) & 1)) { dead_s = 1; dead = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float* wsg = ws_s[g & 15] + cbase;
#pragma unroll
      for (int c0 = 0; c0 < HALF; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + st * kTmemCols + ((uint32_t)(quarter * 32) << 16) + cbase + c0, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c0 + j] = fmaf((float)(int)v[j] * xs, wsg[c0 + j], acc[c0 + j]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __threadfence_block();  // the scale loads have returned before their ring slot is handed back
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tfree_bar[st]));
    }
    if (!dead && my_m < p.M) {
      __nv_bfloat16* dst = p.out + (int64_t)my_m * p.N + n0 + cbase;
#pragma unroll
      for (int c = 0; c < HALF; ++c) {
        if (n0 + cbase + c < p.N) {
          float y = acc[c];
          if (p.bias != nullptr) y += __bfloat162float(p.bias[n0 + cbase + c]);
          dst[c] = __float2bfloat16_rn(y);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && dead_s) atomicExch(p.error_word, 2);
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kWsAcc * kTmemCols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// Pipelined variant for bf16 activations (kind::f16). The weight scale is folded into the B
// operand: a code becomes bf16(float(code) * scale) -- bit for bit the tensor the reference's
// kernel mode builds before its library GEMM (quantizers/kernel.py:68-79,
// `(qweight * scale).to(dtype)`) -- so the whole K axis accumulates in ONE TMEM accumulator
// and is drained once, at the end.
//
//   warps 0-7  fill: bf16 token rows by cp.async into a 128-byte-swizzled tile (two 64-column
//              halves per 128-column stage), weight codes through registers (fetched two
//              stages ahead) -> float by mantissa injection (exact) -> times the group scale
//              -> bf16 pairs -> the swizzled B tile. After the last stage the same warps drain
//              the accumulator (warp w: TMEM lanes 32 (w % 4).., columns 64 (w / 4)..).
//   warp 8     one thread issues eight MMAs (K = 16 each) per stage and commits them to the
//              stage's "free" barrier; after the last stage to the "done" barrier.
constexpr int kF16Threads = 288;
constexpr int kF16Stages = 3;

template <int BITS>
__global__ void __launch_bounds__(kF16Threads)
prefill_gemm_f16_kernel(const GemmParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar[kF16Stages], sfree_bar[kF16Stages], done_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int dead_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  constexpr int KT = 128;                 // K columns per stage
  constexpr int ATOM = BM * 128;          // bytes of one 64-column half of a tile
  constexpr int TILE = 2 * ATOM;          // bytes of an A or B tile (bf16 operands)
  constexpr uint32_t kIdesc = idesc(1, 1);  // f32 <- bf16 x bf16
  uint8_t* const tiles = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
  const int S = p.Kd / KT;                // stages of work (Kd is a multiple of 128 here)

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int i = 0; i < kF16Stages; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 8);  // one arrival per fill warp
      mbar_init(smem_u32(&sfree_bar[i]), 1);
    }
    mbar_init(smem_u32(&done_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    dead_s = 0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp < 8) {
    // ------------------------------------------------------------------ fill
    const int ft = tid;                       // 0..255
    const int brow = ft & 127, half = ft >> 7;  // the weight row and 64-column half this thread widens
    const int n = n0 + brow;
    constexpr int NRAW = BITS == 8 ? 4 : 2;   // 16-byte pieces of 64 codes
    uint4 raw[2][NRAW];
    float sc[2];
    auto fetch_b = [&](const int set, const int g) {
#pragma unroll
      for (int q = 0; q < NRAW; ++q) raw[set][q] = make_uint4(0, 0, 0, 0);
      sc[set] = 0.f;  // rows beyond N: every product is zero
      if (n < p.N && g < S) {
        const int k0 = g * KT + half * 64;
        const uint4* src = reinterpret_cast<const uint4*>(p.codes + (int64_t)n * p.rowbytes + k0 * BITS / 8);
#pragma unroll
        for (int q = 0; q < NRAW; ++q) raw[set][q] = __ldg(src + q);
        sc[set] = p.scale_tiles[((int64_t)(n >> 2) * p.groups + k0 / p.span) * 4 + (n & 3)];
      }
    };
    auto cp16 = [](uint32_t dst, const void* src, bool valid) {
      const int bytes = valid ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    };
    auto issue_a = [&](const int g) -> bool {
      const int st = g % kF16Stages;
      if (g >= kF16Stages && !mbar_wait(smem_u32(&sfree_bar[st]), ((g / kF16Stages) - 1) & 1)) return false;
      const uint32_t a_tile = smem_u32(tiles + st * 2 * TILE);
#pragma unroll
      for (int it = 0; it < 8; ++it) {  // piece (row, pc) = item / 16, item % 16; 8 columns each
        const int item = it * 256 + ft, row = item >> 4, pc = item & 15;
        const int m = m0 + row, k = g * KT + pc * 8;
        const bool valid = m < p.M && k < p.K;
        const uint32_t dst = (uint32_t)(pc >> 3) * ATOM + (uint32_t)row * 128 + (((pc & 7) ^ (row & 7)) << 4);
        cp16(a_tile + dst, p.x + (int64_t)(valid ? m : 0) * p.ldx + (valid ? k : 0), valid);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      return true;
    };
    auto widen_store = [&](const int set, const int g) {
      uint8_t* rowp = tiles + (g % kF16Stages) * 2 * TILE + TILE + half * ATOM + brow * 128;
      const float s = sc[set];
#pragma unroll
      for (int kc = 0; kc < 8; ++kc) {  // eight columns -> one 16-byte piece
        float f[8];
        if (BITS == 4) {
          const uint4 v = raw[set][kc >> 2];
          const unsigned w = (kc & 3) == 0 ? v.x : (kc & 3) == 1 ? v.y : (kc & 3) == 2 ? v.z : v.w;
#pragma unroll
          for (int j = 0; j < 8; ++j)  // nibble (code + 8) into the mantissa of 2^23: exact
            f[j] = (__uint_as_float(((w >> (4 * j)) & 0xFu) | 0x4B000000u) - 8388616.f) * s;
        } else {
          const uint4 v = raw[set][kc >> 1];
          const unsigned w0 = ((kc & 1) == 0 ? v.x : v.z) ^ 0x80808080u, w1 = ((kc & 1) == 0 ? v.y : v.w) ^ 0x80808080u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // byte (code + 128) into the mantissa of 2^23: exact
            f[j] = (__uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7440u | j)) - 8388736.f) * s;
            f[4 + j] = (__uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7440u | j)) - 8388736.f) * s;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
        o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
        *reinterpret_cast<uint4*>(rowp + ((kc ^ (brow & 7)) << 4)) = o;
      }
    };
    bool ok = true;
    fetch_b(0, 0);
    fetch_b(1, 1);
    for (int g = 0; g < 2 && g < S && ok; ++g) ok = issue_a(g);
    for (int g = 0; g < S && ok; ++g) {
      const int st = g % kF16Stages;
      if (dead_s) break;
      if (g + 1 < S) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      // the B half of stage st was last read by the MMAs of stage g - 3, which the A copies of
      // this stage already waited for
      if ((g & 1) == 0) { widen_store(0, g); fetch_b(0, g + 2); }
      else { widen_store(1, g); fetch_b(1, g + 2); }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&full_bar[st]));
      if (g + 2 < S) ok = issue_a(g + 2);
    }
    if (!ok) dead_s = 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // ------------------------------------------------------------------ drain (once)
    if (ok && !dead_s) {
      if (!mbar_wait(smem_u32(&done_bar), 0)) {
        dead_s = 1;
      } else {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quarter = warp & 3, cbase = (warp >> 2) * 64;
        const int my_m = m0 + quarter * 32 + lane;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + cbase + c0, v);
          if (my_m < p.M) {
            __nv_bfloat16* dst = p.out + (int64_t)my_m * p.N + n0 + cbase + c0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (n0 + cbase + c0 + j < p.N) {
                float y = __uint_as_float(v[j]);
                if (p.bias != nullptr) y += __bfloat162float(p.bias[n0 + cbase + c0 + j]);
                dst[j] = __float2bfloat16_rn(y);
              }
            }
          }
        }
      }
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------------ MMA issue
    bool ok = true;
    for (int g = 0; g < S; ++g) {
      const int st = g % kF16Stages;
      if (dead_s) { ok = false; break; }
      if (!mbar_wait(smem_u32(&full_bar[st]), (g / kF16Stages) & 1)) { dead_s = 1; ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = smem_u32(tiles + st * 2 * TILE), b_addr = a_addr + TILE;
#pragma unroll
      for (int s = 0; s < 8; ++s) {  // 16 columns (32 bytes) per MMA, four per 64-column half
        const uint32_t off = (uint32_t)(s >> 2) * ATOM + (s & 3) * 32;
        mma_f16(tmem_base, smem_desc_sw128(a_addr + off), smem_desc_sw128(b_addr + off), kIdesc, (g > 0 || s > 0) ? 1u : 0u);
      }
      mma_commit(smem_u32(&sfree_bar[st]));
    }
    if (ok) mma_commit(smem_u32(&done_bar));
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && dead_s) atomicExch(p.error_word, 3);
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <int BITS>
int launch_gemm_f16(const GemmParams& p, cudaStream_t s) {
  auto kern = prefill_gemm_f16_kernel<BITS>;
  const size_t smem = 1024 + (size_t)kF16Stages * 4 * BM * 128;  // A and B tiles of 32 KB per stage
  if (const int rc = ensure_smem_limit(reinterpret_cast<const void*>(kern), 210 * 1024, "lq_wq_gemm_prefill")) return rc;
  dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + BM - 1) / BM));
  kern<<<grid, kF16Threads, smem, s>>>(p);
  return check_launch("lq_wq_gemm_prefill");
}

template <int BITS>
int launch_gemm_ws(const GemmParams& p, cudaStream_t s) {
  auto kern = prefill_gemm_ws_kernel<BITS>;
  // operand tiles of kWsStages groups, plus (int4) the staging rows of nibble bytes
  const size_t smem = 1024 + (size_t)kWsStages * 2 * BM * 128 + (BITS == 4 ? (size_t)kWsStages * BN * 64 : 0);
  if (const int rc = ensure_smem_limit(reinterpret_cast<const void*>(kern), 210 * 1024, "lq_wq_gemm_prefill")) return rc;
  dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + BM - 1) / BM));
  kern<<<grid, kWsThreads, smem, s>>>(p);
  return check_launch("lq_wq_gemm_prefill");
}

__device__ int g_gemm_error = 0;

template <int BITS, int ES>
int launch_gemm(const GemmParams& p, cudaStream_t s) {
  auto kern = prefill_gemm_kernel<BITS, ES>;
  const size_t smem = 2 * (size_t)BM * p.span * ES;
  if (const int rc = ensure_smem_limit(reinterpret_cast<const void*>(kern), 64 * 1024, "lq_wq_gemm_prefill")) return rc;
  dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + BM - 1) / BM));
  kern<<<grid, kThreads, smem, s>>>(p);
  return check_launch("lq_wq_gemm_prefill");
}

}  // namespace
}  // namespace lq

extern "C" int lq_gemm_device_error(void) {
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_gemm_error) != cudaSuccess) { cudaGetLastError(); return -1; }
  int value = 0;
  if (cudaMemcpy(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(ptr, 0, sizeof(int));
  return value;
}

extern "C" int lq_wq_gemm_prefill(const void* x, int ldx, const int8_t* x_codes, const float* x_scales,
                                  const void* codes, const float* scale_tiles, const void* bias,
                                  void* out, int M, int N, int K, int Kd, int span, int bits,
                                  int flags, void* stream) {
  using namespace lq;
  LQ_REQUIRE(bits == 4 || bits == 8, LQ_ERR_ARG, "unsupported num_bits %d, expected 4 or 8", bits);
  LQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && Kd >= K, LQ_ERR_ARG, "bad shape M=%d N=%d K=%d Kd=%d", M, N, K, Kd);
  if (M == 0 || N == 0) return LQ_OK;
  LQ_REQUIRE(span == 64 || span == 128, LQ_ERR_UNSUPPORTED,
             "the prefill GEMM is built for scale groups of 64 or 128 stored codes, got %d", span);
  LQ_REQUIRE(Kd % span == 0, LQ_ERR_ARG, "Kd=%d is not a whole number of groups of %d", Kd, span);
  LQ_REQUIRE(codes && scale_tiles && out, LQ_ERR_ARG, "null tensor pointer");
  const bool a8 = x_codes != nullptr;
  LQ_REQUIRE(a8 ? x_scales != nullptr : x != nullptr, LQ_ERR_ARG, "null activation pointer");
  LQ_REQUIRE(a8 || ldx >= K, LQ_ERR_ARG, "x row stride %d is shorter than K=%d", ldx, K);
  LQ_REQUIRE(!a8 || ((uintptr_t)x_codes % 16 == 0 && Kd % 16 == 0), LQ_ERR_ARG, "activation codes must be 16-byte aligned");
  LQ_REQUIRE((uintptr_t)codes % 16 == 0, LQ_ERR_ARG, "codes must be 16-byte aligned");
  GemmParams p;
  p.x = (const __nv_bfloat16*)x; p.ldx = ldx; p.x_codes = x_codes; p.x_scales = x_scales;
  p.codes = (const uint8_t*)codes; p.scale_tiles = scale_tiles; p.bias = (const __nv_bfloat16*)bias;
  p.out = (__nv_bfloat16*)out; p.M = M; p.N = N; p.K = K; p.Kd = Kd; p.span = span;
  p.groups = Kd / span; p.rowbytes = Kd * bits / 8;
  void* err = nullptr;
  if (cudaGetSymbolAddress(&err, g_gemm_error) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "cannot resolve the device error word");
  }
  p.error_word = (int*)err;
  cudaStream_t s = (cudaStream_t)stream;
  const bool serial = (flags & LQ_GEMM_SERIAL) != 0;
  if (a8 && span == 128 && !serial) return bits == 8 ? launch_gemm_ws<8>(p, s) : launch_gemm_ws<4>(p, s);
  // bf16 activations: the pipelined kernel needs 16-byte pieces of x (8 columns) to be whole
  if (!a8 && (flags & LQ_GEMM_FOLD_SCALES) && !serial && Kd % 128 == 0 && K % 8 == 0 && ldx % 8 == 0 &&
      (uintptr_t)x % 16 == 0)
    return bits == 8 ? launch_gemm_f16<8>(p, s) : launch_gemm_f16<4>(p, s);
  if (bits == 8) return a8 ? launch_gemm<8, 1>(p, s) : launch_gemm<8, 2>(p, s);
  return a8 ? launch_gemm<4, 1>(p, s) : launch_gemm<4, 2>(p, s);
}
