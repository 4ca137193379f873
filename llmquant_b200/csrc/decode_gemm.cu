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
//                       floating point of gemv_mma.cu), laid out as the B operand tiles the MMA
//                       reads from shared memory: per group one block of 2 * TP plane rows
//                       (rows 0..TP-1 high planes, TP..2TP-1 low planes, 128-byte swizzled)
//                       followed by the TP units.
//   decode_gemm_kernel  one CTA per SM; the weight's (128-row tile, scale group) steps are cut
//                       into equal contiguous runs, one per CTA. The weight
//                       is read in a TILE-MAJOR layout (lq_tile_weight): per tile and group one
//                       contiguous block of codes and scales, so a group arrives with one
//                       linear bulk copy. Per group: A = 128 rows x 128 codes as signed bytes
//                       (int8 codes as they are; int4 nibbles as 16 * code, the 1/16 folded
//                       into the scale), B = the group's 2 * TP plane rows, four tcgen05.mma
//                       kind::i8 (K = 32 each) into one of up to eight TMEM accumulators
//                       [128 lanes = weight rows][2 * TP columns]. Warp roles: int8 codes
//                       arrive in the A tiles by bulk copies, issued by two threads, and one
//                       thread issues the plane copies (issuing a bulk copy occupies a thread
//                       for ~500 clocks); int4 nibbles are loaded from global memory and
//                       widened into the A tiles by eight warps, each a whole group by
//                       itself; two threads issue the MMAs (even / odd groups); eight drain
//                       warps read the accumulators (tcgen05.ld), form hi * 256 + lo, multiply
//                       by weight scale x unit and add into fp32 registers. This is the
//                       reference's order of operations: one exact product sum per group,
//                       scaled, accumulated in fp32 over the groups (quantizers/real.py:93-99).
//                       A tile's sums go to partial[part][T][N], one part per CTA that touched it.
//   decode_finish_kernel  adds the parts in CTA order, then bias / residual / silu(gate) * up and
//                       the roundings of the bf16 modules, and stores the output rows.
//
// What sets the pace (measured with per-role clock stamps, a diagnostic build): not HBM and
// not the tensor core, but per-group latencies -- a bulk copy's issue, a barrier operation
// (~100 clocks each), the proxy fence after widening, the MMA -> commit -> drain -> hand-back
// loop. Hence: few copies per group, one arrival per warp, deep rings with a barrier ring of
// their own each, eight accumulators, eight groups being widened at once.
//
// Every wait is bounded (mbar_wait); on expiry the CTA records the error word, all roles leave
// their loops, TMEM is freed.
#include "common.cuh"
#include "tcgen05.cuh"

namespace lq {
namespace {

constexpr int kDgWidenWarps = 8;  // each widens every eighth group by itself
constexpr int kDgRows = 128;     // weight rows per CTA = TMEM lanes
constexpr int KT = 128;          // codes per scale group = bytes per operand row
constexpr int kDgSmem = 216 * 1024;  // dynamic shared memory the rings are sized for
constexpr int kDgRing = 16;      // slots of the small per-group rings (weight scales, units)

// Shared-memory plan of an instance. A CTA streams its rows at the rate its bytes in flight allow
// (HBM answers after about a microsecond). int8 codes land directly in a ring of A operand tiles
// by bulk copies (their scales behind them). int4 nibbles are loaded from global memory into
// registers by the widening warps -- a whole group per warp, eight groups in flight -- and
// stored as signed bytes into the A tiles (a ring of raw bytes in shared memory in between --
// bulk copy in, vector load out -- was no faster and cost 70 KB). The activation planes (B
// tiles, their units behind them) have a ring of their own. Issuing a bulk copy occupies the
// issuing thread for some hundred clocks, which is why a group costs at most two of them and
// every ring has its own issuing threads.
constexpr int kScaleBytes = kDgRows * 4;  // the 128 weight scales of a group
template <int BITS, int TP>
struct DgPlan {
  static constexpr int NCOL = 2 * TP;
  static constexpr int A_TILE = kDgRows * KT;  // 16 KB
  static constexpr int B_TILE = NCOL * KT;
  static constexpr int UNIT_BYTES = (TP * 4 + 127) / 128 * 128;
  static constexpr int B_BLOCK = B_TILE + UNIT_BYTES;   // what one copy brings: planes + units
  static constexpr int RAW = kDgRows * (KT / 2);        // int4: a group's nibble bytes
  static constexpr int W_BLOCK = (BITS == 8 ? A_TILE : RAW) + kScaleBytes;  // codes + scales
  // slots keep the operand tiles on 1024-byte boundaries (the 128-byte swizzle)
  static constexpr int A_SLOT = A_TILE + (BITS == 8 ? 1024 : 0);
  static constexpr int B_SLOT = B_TILE + 1024;
  static constexpr int SA8_ = kDgSmem / (A_SLOT + B_SLOT) > 8 ? 8 : kDgSmem / (A_SLOT + B_SLOT);
  // int4: one A tile per widening warp (a warp always widens into the same tile)
  static constexpr int SA = BITS == 8 ? (SA8_ & ~1) : kDgWidenWarps;
  static constexpr int BN_ = (kDgSmem - SA * A_SLOT) / B_SLOT > 8 ? 8 : (kDgSmem - SA * A_SLOT) / B_SLOT;
  static constexpr int BN = BITS == 8 ? SA : (BN_ & ~1);
  static constexpr size_t SMEM = (size_t)SA * A_SLOT + (size_t)BN * B_SLOT + 1024;
  // warps: 0-7 drain, then (int4) 8 widening warps, 2 MMA-issuing, 1 for the plane copies,
  // (int8) 2 for the weight copies
  static constexpr int W_MMA = BITS == 8 ? 8 : 8 + kDgWidenWarps;
  static constexpr int W_PLANES = W_MMA + 2;
  static constexpr int W_WEIGHTS = W_PLANES + 1;  // int8 only
  static constexpr int THREADS = 32 * (BITS == 8 ? W_WEIGHTS + 2 : W_PLANES + 1);
  // Accumulators in tensor memory: as many as its 512 columns hold, up to 8. An MMA, the
  // commit that follows it, the drain's tensor-memory load and the hand-back are each a few
  // hundred clocks of latency: the ring has to cover that loop.
  static constexpr int NACC = 512 / NCOL < 8 ? 512 / NCOL : 8;
  // Whoever tests a barrier for its n-th completion must know the (n-1)-th has happened (a
  // test that comes a whole phase early reads as "complete"). So the rings are laid out such
  // that all uses of one slot fall to one thread, which takes them in order: even depths for
  // the rings walked by the even / odd thread pairs, one A tile per widening warp, and 16-deep
  // barrier rings ("group multiplied", "group drained") behind rings of at
  // most 8.
  static_assert(SA % 2 == 0 && BN % 2 == 0 && BN >= 4 && NACC % 2 == 0, "ring depths must be even");
  static_assert(SA <= 8 && BN <= 8 && NACC <= 8 && SA + NACC <= kDgRing, "rings deeper than the barrier rings allow");
  static_assert(kDgRing % kDgWidenWarps == 0, "a widening warp must meet a barrier slot again after 16 groups");
};

__device__ int g_decode_gemm_error = 0;

#ifdef LQ_DIAGNOSTICS
// Diagnostic builds: SM clocks the role leaders of CTA 0..255 spent in each part of a round,
// summed over the rounds. [cta][slot]: widen 0 wait-copies 1 widen | mma 4 wait-operands
// 5 wait-accumulator 6 issue | drain 8 wait 9 load+scale | 12 whole kernel
__device__ unsigned long long g_dg_diag[256 * 16];
// and for CTA (0, 0) the SM clock of eight events per group: 0 nibble loads issued by the widen
// warp, 1 group widened, 2 planes requested, 3 MMA thread has its operands, 4 MMAs issued,
// 5 drain sees the group multiplied, 6 drain done, 7 int8 codes requested
__device__ long long g_dg_trace[128 * 8];
#define DG_EV(j, e) do { if (blockIdx.x == 0 && (j) < 128) g_dg_trace[(j) * 8 + (e)] = clock64(); } while (0)
#define DG_T0() const long long dg_t0_ = clock64()
#define DG_ADD(slot) do { (void)dg_t0_; } while (0)  // (sums off: they cost a round trip to memory each, which distorts the trace)
#else
#define DG_T0() do { } while (0)
#define DG_ADD(slot) do { } while (0)
#define DG_EV(j, e) do { } while (0)
#endif

struct DgParams {
  const uint8_t* codes;      // tile-major [tiles][G] blocks: codes of 128 rows, then their 128 scales
  const uint8_t* planes;     // [G] blocks: plane rows [2 * TP][128] swizzled as the MMA reads them, then TP units
  float* partial;            // [splits][T][N]
  int T, N, groups, rowbytes;
  int steps, ncta;           // (row tile, scale group) steps of the whole weight; CTAs that share them evenly
  int parts;                 // > 0: every row tile is finished in exactly this many parts (runs do not cross tiles)
  int* error_word;
};

// The weight's (row tile, scale group) steps, in tile-major order -- the order of the blocks in
// memory -- are cut into `ncta` contiguous runs of equal length (to within one): CTA c takes steps
// [c * steps / ncta, (c + 1) * steps / ncta). A run may end inside a row tile: the tile's sums
// are then finished by the next CTA, and the parts are added by the finish kernel.
__host__ __device__ inline int dg_first_step(int c, int steps, int ncta) { return (int)((long long)c * steps / ncta); }
__host__ __device__ inline int dg_cta_of(int step, int steps, int ncta) {
  return (int)((((long long)step + 1) * ncta + steps - 1) / steps) - 1;
}

constexpr uint32_t dg_idesc(int ncol) {
  // D = s32, A = B = s8, both K-major, N = ncol, M = 128
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ncol >> 3) << 17) | ((uint32_t)(kDgRows >> 4) << 24);
}

template <int BITS, int TP>
__global__ void __launch_bounds__(DgPlan<BITS, TP>::THREADS)
decode_gemm_kernel(const DgParams p) {
  using Plan = DgPlan<BITS, TP>;
  constexpr int NCOL = Plan::NCOL;                  // accumulator columns: high planes, low planes
  constexpr int NACC = Plan::NACC;
  constexpr int TMEM_COLS = NACC * NCOL < 32 ? 32 : NACC * NCOL;
  constexpr int A_TILE = Plan::A_TILE, B_TILE = Plan::B_TILE, RAW = Plan::RAW;
  constexpr int A_SLOT = Plan::A_SLOT, B_SLOT = Plan::B_SLOT;
  constexpr int SA = Plan::SA, BN = Plan::BN;
  constexpr int W_MMA = Plan::W_MMA, W_PLANES = Plan::W_PLANES, W_WEIGHTS = Plan::W_WEIGHTS;
  constexpr int DW = TP >= 16 ? 8 : 4;              // drain warps in use
  constexpr int TPH = TP / (DW / 4);                // tokens per drain thread
  constexpr int CH = TPH < 16 ? 8 : 16;             // tokens per tensor-memory load
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t a_full[SA], b_full[BN];
  __shared__ __align__(8) uint64_t mma_done[kDgRing], drained[kDgRing];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float ws_s[BITS == 4 ? kDgRing : 1][kDgRows];  // int4: scales, kept by the widening warps
  __shared__ volatile int dead_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s0 = dg_first_step(blockIdx.x, p.steps, p.ncta);
  const int GL = dg_first_step(blockIdx.x + 1, p.steps, p.ncta) - s0;  // steps of this CTA
  uint8_t* const a_ring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
  uint8_t* const b_ring = a_ring + SA * A_SLOT;
  constexpr uint32_t kIdesc = dg_idesc(NCOL);
  // "group k has been multiplied" / "... drained": slot k % 16 of the ring, its (k / 16)-th completion
  auto wait_done = [&](int k) { return mbar_wait(smem_u32(&mma_done[k & (kDgRing - 1)]), (k / kDgRing) & 1); };
  auto wait_drained = [&](int k) { return mbar_wait(smem_u32(&drained[k & (kDgRing - 1)]), (k / kDgRing) & 1); };

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    // (arrivals are one per warp, after the warp has synchronized: an arrival is an atomic
    // operation on the barrier word, and hundreds of them per group are what a round would cost)
    for (int i = 0; i < SA; ++i) mbar_init(smem_u32(&a_full[i]), 1);
    for (int i = 0; i < BN; ++i) mbar_init(smem_u32(&b_full[i]), 1);
    for (int i = 0; i < kDgRing; ++i) {
      mbar_init(smem_u32(&mma_done[i]), 1);
      mbar_init(smem_u32(&drained[i]), DW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    dead_s = 0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  DG_T0();

  if (BITS == 8 && (warp == W_WEIGHTS || warp == W_WEIGHTS + 1)) {
    // ------------------------------------------------------------------ weight copies (int8; two threads)
    // Weights do not depend on the kernel before this one: their copies start at once. One
    // contiguous block per step: the codes of the 128 rows, then their scales. Issuing a bulk
    // copy occupies a thread for about 500 clocks, more than a step's bytes take to arrive:
    // one thread takes the even steps, another the odd ones.
    if (lane == 0) {
      const uint8_t* my_codes = p.codes + (int64_t)s0 * Plan::W_BLOCK;  // the run's blocks are contiguous
      for (int j = warp - W_WEIGHTS; j < GL && !dead_s; j += 2) {
        // the slot's scales are read by the drain of the step that used it last
        if (j >= SA && !wait_drained(j - SA)) { dead_s = 1; break; }
        mbar_expect_tx(smem_u32(&a_full[j % SA]), Plan::W_BLOCK);
        bulk_g2s(smem_u32(a_ring + (j % SA) * A_SLOT), my_codes + (int64_t)j * Plan::W_BLOCK, Plan::W_BLOCK,
                 smem_u32(&a_full[j % SA]));
        DG_EV(j, 7);
      }
    }
  } else if (warp == W_PLANES) {
    // ------------------------------------------------------------------ plane copies (one thread)
    // The activation planes and units are the output of the kernel before this one.
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      int g = s0 % p.groups;  // scale group of step j
      for (int j = 0; j < GL && !dead_s; ++j) {
        // the slot's units are read by the drain of the group that used it last
        if (j >= BN && !wait_drained(j - BN)) { dead_s = 1; break; }
        mbar_expect_tx(smem_u32(&b_full[j % BN]), Plan::B_BLOCK);
        bulk_g2s(smem_u32(b_ring + (j % BN) * B_SLOT), p.planes + (int64_t)g * Plan::B_BLOCK, Plan::B_BLOCK,
                 smem_u32(&b_full[j % BN]));
        if (++g == p.groups) g = 0;
        DG_EV(j, 2);
      }
    }
  } else if (BITS == 4 && warp >= 8 && warp < 8 + kDgWidenWarps) {
    // ------------------------------------------------------------------ widen (int4)
    // Each warp takes every eighth step by itself and always widens into the same A tile: the
    // step's 8 KB of nibble bytes and its scales come straight from global memory (contiguous:
    // 512 bytes per load instruction), requested before the wait for the tile, so that with
    // eight warps eight steps' bytes are in flight.
    {
      const int w = warp - 8;
      uint8_t* const a_tile = a_ring + w * A_SLOT;
      const uint8_t* my_codes = p.codes + (int64_t)s0 * Plan::W_BLOCK;
      for (int j = w; j < GL; j += kDgWidenWarps) {
        if (dead_s) break;
        const uint8_t* src = my_codes + (int64_t)j * Plan::W_BLOCK;  // [128 rows][64 bytes], then 128 scales
        uint4 raw[16];
#pragma unroll
        for (int it = 0; it < 16; ++it) raw[it] = __ldg(reinterpret_cast<const uint4*>(src) + it * 32 + lane);
        const float4 sc = __ldg(reinterpret_cast<const float4*>(src + RAW) + lane);
        if (lane == 0) DG_EV(j, 0);
        if (j >= SA && !wait_done(j - SA)) { dead_s = 1; break; }
        DG_T0();
        // the scales go where the drain finds them after the MMAs
        *reinterpret_cast<float4*>(&ws_s[j & (kDgRing - 1)][lane * 4]) = sc;
#pragma unroll
        for (int it = 0; it < 16; ++it) {
          const int item = it * 32 + lane, row = item >> 2, q = item & 3;
          const unsigned w4[4] = {raw[it].x, raw[it].y, raw[it].z, raw[it].w};
          unsigned o[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // word of 8 nibbles (code + 8): even positions and odd positions as bytes 16 * code,
            // interleaved back into K order. A row beyond N is stored as zeros and becomes
            // bytes -128: its outputs are never stored.
            const unsigned ev = ((w4[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
            const unsigned od = (w4[i] & 0xF0F0F0F0u) ^ 0x80808080u;
            o[2 * i] = __byte_perm(ev, od, 0x5140);      // codes 0..3 of the word
            o[2 * i + 1] = __byte_perm(ev, od, 0x7362);  // codes 4..7
          }
          uint8_t* rowp = a_tile + row * 128;
          *reinterpret_cast<uint4*>(rowp + (((2 * q) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(rowp + (((2 * q + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> MMA reads
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&a_full[w]));
        if (lane == 0) { DG_ADD(1); DG_EV(j, 1); }
      }
    }
  } else if (warp == W_MMA || warp == W_MMA + 1) {
    // ------------------------------------------------------------------ MMA issue
    // Two issuing threads, one for the even groups and one for the odd ones (a group has an
    // accumulator of its own): issuing a group's four MMAs and its commit takes one thread
    // longer than the group's bytes take to arrive.
    if (lane == 0) {
      for (int j = warp - W_MMA; j < GL; j += 2) {
        const int tb = j % NACC;
        if (dead_s) break;
        { DG_T0(); if (!mbar_wait(smem_u32(&a_full[j % SA]), (j / SA) & 1) || !mbar_wait(smem_u32(&b_full[j % BN]), (j / BN) & 1)) { dead_s = 1; break; } if (warp == W_MMA) DG_ADD(4); }
        { DG_T0(); if (j >= NACC && !wait_drained(j - NACC)) { dead_s = 1; break; } if (warp == W_MMA) DG_ADD(5); }
        DG_T0();
        DG_EV(j, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc_sw128(smem_u32(a_ring + (j % SA) * A_SLOT));
        const uint64_t db = smem_desc_sw128(smem_u32(b_ring + (j % BN) * B_SLOT));
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          // 32 bytes of K per MMA: the start address (in 16-byte units) moves along the 128-byte row
          mma_i8(tmem_base + tb * NCOL, da + 2 * s, db + 2 * s, kIdesc, s > 0);
        }
        mma_commit(smem_u32(&mma_done[j & (kDgRing - 1)]));
        DG_EV(j, 4);
        if (warp == W_MMA) DG_ADD(6);
      }
    }
  } else if (warp < DW) {
    // ------------------------------------------------------------------ drain
    float acc[TPH];
#pragma unroll
    for (int c = 0; c < TPH; ++c) acc[c] = 0.f;
    const int quarter = warp & 3, t0 = (warp >> 2) * TPH;  // TMEM lanes and tokens of this warp
    const int row = quarter * 32 + lane;
    bool dead = false, may_store = false;
    int g = s0 % p.groups, tile = s0 / p.groups;  // scale group and row tile of step j
    for (int j = 0; j < GL; ++j) {
      const int tb = j % NACC, ring = j & (kDgRing - 1);
      if (dead_s) { dead = true; break; }
      { DG_T0(); if (!wait_done(j)) { dead_s = 1; dead = true; break; } if (tid == 0) DG_ADD(8); }
      DG_T0();
      if (tid == 0) DG_EV(j, 5);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // the group's scales (behind its codes, or saved by the widening warps) and units (behind its planes)
      const float* ws = BITS == 8 ? reinterpret_cast<const float*>(a_ring + (j % SA) * A_SLOT + A_TILE) : ws_s[BITS == 4 ? ring : 0];
      const float* us = reinterpret_cast<const float*>(b_ring + (j % BN) * B_SLOT + B_TILE);
      const float wsx = ws[row] * (BITS == 4 ? 0.0625f : 1.f);  // 1/16: nibbles ride as 16 * code
      const uint32_t taddr = tmem_base + tb * NCOL + ((uint32_t)(quarter * 32) << 16) + t0;
#pragma unroll
      for (int c0 = 0; c0 < TPH; c0 += CH) {
        uint32_t hi[CH], lo[CH];
        tmem_ld(taddr + c0, hi);
        tmem_ld(taddr + TP + c0, lo);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < CH; q += 4) {
          const float4 u = *reinterpret_cast<const float4*>(us + t0 + c0 + q);
          const float uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            acc[c0 + q + e] = fmaf((float)((int)hi[q + e] * 256 + (int)lo[q + e]), uu[e] * wsx, acc[c0 + q + e]);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      // The loads above (units, scales) must have returned before the arrival that lets a bulk
      // copy overwrite their slot: an arrival is not held back by an earlier shared-memory load
      // of its warp whose data is still on its way, and with the widening warps' global loads
      // queued in the same load path that took long enough for a warp to read the units of the
      // step eight later. The fence waits for this thread's loads.
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&drained[ring]));
      if (tid == 0) { DG_ADD(9); DG_EV(j, 6); }
      // end of a row tile, or of this CTA's run inside one: its sums go out as one part of the tile
      if (g == p.groups - 1 || j == GL - 1) {
        if (!may_store) {
          // the buffer the sums go to may still be read by a kernel before this one: nothing of
          // this kernel is stored before its predecessors are complete
          asm volatile("griddepcontrol.wait;" ::: "memory");
          may_store = true;
        }
        const int nrow = tile * kDgRows + row;
        const int part = p.parts > 0 ? (int)blockIdx.x % p.parts
                                     : (int)blockIdx.x - dg_cta_of(tile * p.groups, p.steps, p.ncta);
        if (nrow < p.N) {
          float* dst = p.partial + ((int64_t)part * p.T + t0) * p.N + nrow;
#pragma unroll
          for (int c = 0; c < TPH; ++c)
            if (t0 + c < p.T) dst[(int64_t)c * p.N] = acc[c];
        }
#pragma unroll
        for (int c = 0; c < TPH; ++c) acc[c] = 0.f;
      }
      if (++g == p.groups) { g = 0; ++tile; }
    }
    (void)dead;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == 0) DG_ADD(12);
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
                  float norm_eps, uint8_t* __restrict__ planes, int block_bytes, int T, int TP, int K, int groups) {
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
      // a group's block: the plane rows as the MMA reads them from shared memory -- 16-byte piece
      // `sub` of row r sits at piece (sub ^ (r & 7)), the 128-byte swizzle -- then the TP units;
      // one linear bulk copy stages it
      uint8_t* blk = planes + (int64_t)g * block_bytes;
      uint8_t* hp = blk + (int64_t)t * KT + ((sub ^ (t & 7)) << 4);
      *reinterpret_cast<uint4*>(hp) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
      *reinterpret_cast<uint4*>(hp + (int64_t)TP * KT) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
      if (sub == 0)
        reinterpret_cast<float*>(blk + (int64_t)2 * TP * KT)[t] =
            live && amax > 0.f ? __uint_as_float((unsigned)(127 + e - 14) << 23) : 0.f;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// out = epilogue(sum over the parts of the row tile, in CTA order): EPI 0 bias / residual, EPI 1 silu(gate) * up over
// interleaved (gate, up) rows, with the roundings of gemv_stream_kernel's epilogues.
template <int EPI>
__global__ void __launch_bounds__(256)
decode_finish_kernel(const float* __restrict__ partial, int groups, int steps, int ncta, int uniform_parts, int T, int N,
                     const __nv_bfloat16* __restrict__ bias, const void* __restrict__ residual, void* __restrict__ out,
                     int out_f32, int ldo) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int NO = EPI == 1 ? N / 2 : N;
  const int64_t total = (int64_t)T * NO;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / NO), j = (int)(i % NO);
    const int64_t o = (int64_t)t * ldo + j;
    // the parts of this output's row tile: one per CTA whose run of steps touches the tile
    const int tile = (EPI == 1 ? 2 * j : j) / kDgRows;
    const int splits = uniform_parts > 0 ? uniform_parts
                                         : dg_cta_of(tile * groups + groups - 1, steps, ncta) - dg_cta_of(tile * groups, steps, ncta) + 1;
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

// ---------------------------------------------------------------------------------------------
// Streaming layout -> the layout the decode GEMM reads: per tile of 128 weight rows and per
// scale group one contiguous block, so that a CTA fetches a group with ONE linear bulk copy
// (fetching 128 pieces of 64 or 128 bytes a whole weight row apart limits an SM to a fraction
// of its share of the HBM bandwidth). int8 blocks are the shared-memory image the MMA reads
// (16-byte piece kc of row r at piece kc ^ (r & 7)); int4 blocks are the nibble bytes, 64 per
// row; rows beyond N are zeros. Scales: [tile][G][128] fp32.
__global__ void tile_weight_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scale_tiles,
                                   uint8_t* __restrict__ out, int N, int groups, int rowbytes, int bits) {
  const int tile = blockIdx.x, g = blockIdx.y;
  const int gb = KT * bits / 8, pieces = gb / 16;  // bytes and 16-byte pieces of a group in a row
  uint8_t* dst = out + ((int64_t)tile * groups + g) * (kDgRows * gb + kScaleBytes);
  for (int i = threadIdx.x; i < kDgRows * pieces; i += blockDim.x) {
    const int r = i / pieces, kc = i % pieces, n = tile * kDgRows + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n < N) v = *reinterpret_cast<const uint4*>(codes + (int64_t)n * rowbytes + g * gb + kc * 16);
    const int pos = bits == 8 ? (kc ^ (r & 7)) : kc;
    *reinterpret_cast<uint4*>(dst + r * gb + pos * 16) = v;
  }
  float* sdst = reinterpret_cast<float*>(dst + kDgRows * gb);
  for (int r = threadIdx.x; r < kDgRows; r += blockDim.x) {
    const int n = tile * kDgRows + r;
    sdst[r] = n < N ? scale_tiles[((int64_t)(n >> 2) * groups + g) * 4 + (n & 3)] : 0.f;
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

// How the weight's steps are shared out, and the most parts any row tile is finished in (the
// depth of the partial buffer). Two kinds of plan, both "equal contiguous runs": tiles x k CTAs,
// whose runs never cross a row tile (k slices of the scale groups per tile), or one CTA per SM
// with runs that may. A run that crosses tiles costs a few steps' time (a flush in mid-stream,
// more parts to add), more than one wave of CTAs costs the set-up again and leaves SMs idle in
// the last wave; the estimate below, in step times, picks (measured on the Llama-3-8B shapes:
// q|k|v 48 tiles x 3, o and down 32 x 4, gate|up and lm_head one CTA per SM).
struct StepPlan {
  int steps, ncta, max_parts;
  int uniform_parts;  // tiles x k CTAs: k; one CTA per SM: 0
};
StepPlan plan_steps(int tiles, int groups) {
  StepPlan q;
  q.steps = tiles * groups;
  const int sms = sm_count();
  const int by_work = (q.steps + 3) / 4;  // at least ~4 steps per CTA
  const int per_sm = by_work < 1 ? 1 : (by_work < sms ? by_work : sms);
  long best = ((long)q.steps + per_sm - 1) / per_sm + 4 + 3;  // one CTA per SM: runs cross tiles
  q.ncta = per_sm;
  q.uniform_parts = 0;
  for (int k = 1; k <= 8 && k <= groups; ++k) {
    const long waves = ((long)tiles * k + sms - 1) / sms;
    const long cost = waves * ((groups + k - 1) / k + 4);
    if (cost <= best) { best = cost; q.ncta = tiles * k; q.uniform_parts = k; }
  }
  q.max_parts = 1;
  for (int t = 0; t < tiles; ++t) {
    const int parts = dg_cta_of(t * groups + groups - 1, q.steps, q.ncta) - dg_cta_of(t * groups, q.steps, q.ncta) + 1;
    if (parts > q.max_parts) q.max_parts = parts;
  }
  return q;
}

int plane_block_bytes(int TP) { return 2 * TP * KT + (TP * 4 + 127) / 128 * 128; }

struct Workspace {
  uint8_t* planes;
  float* partial;
  int64_t bytes;
};
Workspace carve(void* base, int TP, int M, int N, int groups, int splits) {
  Workspace w;
  int64_t off = 0;
  w.planes = reinterpret_cast<uint8_t*>(base) + off;
  off += ((int64_t)groups * plane_block_bytes(TP) + 255) / 256 * 256;
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
  const StepPlan sp = plan_steps(tiles, groups);
  const Workspace w = carve(a.workspace, TP, a.M, a.N, groups, sp.max_parts);
  LQ_REQUIRE(w.bytes <= a.workspace_bytes, LQ_ERR_ARG, "the decode GEMM needs %lld bytes of workspace, got %lld",
             (long long)w.bytes, (long long)a.workspace_bytes);
  void* err_ptr = nullptr;
  if (cudaGetSymbolAddress(&err_ptr, g_decode_gemm_error) != cudaSuccess) {
    cudaGetLastError();
    return fail(LQ_ERR_LAUNCH, "cannot resolve the device error word");
  }
  if (const int rc = launch_dep(act_planes_kernel, dim3((unsigned)TP), dim3(kApThreads), 0, s, a.pdl, "lq_wq_gemv_fused",
                                (const __nv_bfloat16*)a.x, a.ldx, (const __nv_bfloat16*)a.norm_weight, a.norm_eps,
                                w.planes, plane_block_bytes(TP), a.M, TP, a.K, groups))
    return rc;
  DgParams p;
  p.codes = (const uint8_t*)a.codes; p.planes = w.planes;
  p.partial = w.partial; p.T = a.M; p.N = a.N; p.groups = groups; p.rowbytes = a.Kd * a.bits / 8;
  p.steps = sp.steps; p.ncta = sp.ncta; p.parts = sp.uniform_parts; p.error_word = (int*)err_ptr;
  const dim3 grid((unsigned)sp.ncta);
  int rc = LQ_ERR_UNSUPPORTED;
#define LQ_DG_CASE(B, TPV)                                                                              \
  if (a.bits == B && TP == TPV) {                                                                       \
    auto kern = decode_gemm_kernel<B, TPV>;                                                             \
    const size_t smem = DgPlan<B, TPV>::SMEM;                                                           \
    if (const int rs = ensure_smem_limit(reinterpret_cast<const void*>(kern), (int)smem, "lq_wq_gemv_fused")) return rs; \
    rc = launch_dep(kern, grid, dim3(DgPlan<B, TPV>::THREADS), smem, s, a.pdl, "lq_wq_gemv_fused", p); \
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
                      (const float*)w.partial, groups, sp.steps, sp.ncta, sp.uniform_parts, a.M, a.N, (const __nv_bfloat16*)a.bias,
                      a.residual, a.out, a.out_dtype == LQ_F32 ? 1 : 0, ldo);
  return launch_dep(decode_finish_kernel<0>, dim3(blocks), dim3(256), 0, s, a.pdl, "lq_wq_gemv_fused",
                    (const float*)w.partial, groups, sp.steps, sp.ncta, sp.uniform_parts, a.M, a.N, (const __nv_bfloat16*)a.bias,
                    a.residual, a.out, a.out_dtype == LQ_F32 ? 1 : 0, ldo);
}

}  // namespace gemv
}  // namespace lq

extern "C" int64_t lq_decode_gemm_workspace_bytes(int M, int N, int Kd) {
  if (M < 1 || M > 64 || N < 1 || Kd < 128) return 0;
  const int groups = Kd / 128;
  const int TP = lq::tokens_padded(M);
  const lq::StepPlan sp = lq::plan_steps((N + lq::kDgRows - 1) / lq::kDgRows, groups);
  return lq::carve(nullptr, TP, M, N, groups, sp.max_parts).bytes;
}

extern "C" int lq_decode_gemm_device_error(void) {
  int value = 0;
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_decode_gemm_error) != cudaSuccess) return -1;
  if (cudaMemcpy(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(ptr, 0, sizeof(int));
  return value;
}

#ifdef LQ_DIAGNOSTICS
// Diagnostic builds only: copies the per-role clock sums out (256 CTAs x 16 slots) and clears them.
extern "C" int lq_decode_gemm_trace(long long* out_host) {
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_dg_trace) != cudaSuccess) return -1;
  if (cudaMemcpy(out_host, ptr, sizeof(long long) * 128 * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  cudaMemset(ptr, 0, sizeof(long long) * 128 * 8);
  return 0;
}
extern "C" int lq_decode_gemm_diag(unsigned long long* out_host) {
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, lq::g_dg_diag) != cudaSuccess) return -1;
  if (cudaMemcpy(out_host, ptr, sizeof(unsigned long long) * 256 * 16, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  cudaMemset(ptr, 0, sizeof(unsigned long long) * 256 * 16);
  return 0;
}
#endif

extern "C" int64_t lq_tile_weight_bytes(int N, int Kd, int bits) {
  if (N <= 0 || Kd <= 0 || Kd % 128 != 0 || (bits != 4 && bits != 8)) return 0;
  const int64_t tiles = (N + lq::kDgRows - 1) / lq::kDgRows, groups = Kd / 128;
  return tiles * groups * (lq::kDgRows * (lq::KT * bits / 8) + lq::kScaleBytes);
}

extern "C" int lq_tile_weight(const void* codes, const float* scale_tiles, void* out, int N, int Kd, int bits,
                              void* stream) {
  using namespace lq;
  LQ_REQUIRE(codes && scale_tiles && out, LQ_ERR_ARG, "null tensor pointer");
  LQ_REQUIRE(N > 0 && Kd > 0 && Kd % 128 == 0 && (bits == 4 || bits == 8), LQ_ERR_ARG,
             "tile layout: N > 0, Kd a positive multiple of 128, 4 or 8 bits");
  LQ_REQUIRE(((uintptr_t)codes % 16) == 0 && ((uintptr_t)out % 16) == 0, LQ_ERR_ARG, "codes must be 16-byte aligned");
  const dim3 grid((unsigned)((N + kDgRows - 1) / kDgRows), (unsigned)(Kd / 128));
  tile_weight_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)codes, scale_tiles, (uint8_t*)out, N,
                                                             Kd / 128, Kd * bits / 8, bits);
  return check_launch("lq_tile_weight");
}
