// Decode GEMV (M <= 8 activation rows) over the streaming layout on the warp-level tensor
// core path (mma.sync m16n8k32, int8 x int8 -> int32), for scale groups of 128 stored codes.
//
// Why tensor cores for a memory-bound product: the SIMT kernel (gemv_stream.cuh) spends about
// three issue slots per weight on mid-size int4 matrices and is limited by instruction issue,
// not by HBM. Here one MMA covers 16 weight rows x 32 codes against 8 activation columns, so
// the arithmetic is a few percent of the issue budget and a batch of four activation rows
// costs the same as one.
//
//   A operand (16 x 32, row-major)  = weight codes. MMA row r < 8 is tile row 2r, MMA row
//       r + 8 is tile row 2r + 1, so a lane ends up holding two adjacent outputs (a gate / up
//       pair of the fused MLP epilogue). int8 codes are used as they are; int4 nibbles (value
//       + 8) become the signed byte 16 * value with one shift and one logic op per four codes
//       ((n ^ 8) << 4); the factor 16 is folded into the activations' power-of-two unit.
//   B operand (32 x 8, column-major) = the activations as block-floating-point integers: per
//       (activation row, scale group) one shared power-of-two exponent and 15-bit signed
//       mantissas split into a signed high byte and a signed low byte; column 2b is the high
//       plane of activation row b, column 2b + 1 its low plane. The planes live in shared
//       memory in fragment order (a lane fetches the B registers of two MMAs with one 128-bit
//       load) and are built ONCE per CTA, fused with the optional RMSNorm.
//   D (16 x 8, int32): exact integer sums over one scale group; lane (g, t) holds rows 2g and
//       2g + 1 against the two planes of activation row t, recombines hi * 256 + lo, converts
//       once and multiplies by (weight scale x activation unit), accumulating groups in fp32.
//       This is the reference's order of operations (one product sum per 128-wide group,
//       scaled, summed in fp32 -- quantizers/real.py:93-99, cuda/csrc/wq_gemv.cu:78-112) with
//       the activations rounded at 2^-15 of their group maximum.
//
// Data movement: stages of R whole rows (R = 4, 8 or 16, about 32 KB; rows are contiguous in
// the streaming layout, so a stage is ONE bulk asynchronous copy plus one for its scale tiles
// -- bulk copies cost about 80 ns each to issue, so they have to be large) stream into a
// shared-memory ring, an mbarrier per stage counting the bytes. A 16-row MMA tile spans
// 16 / R consecutive stages. The W warps take the scale groups of the rows in turn; their
// partial sums meet in shared memory behind one named barrier per tile, and that barrier is
// also the proof that every warp has read the tile's stages: right after it one thread refills
// them, so there is no producer warp and no second set of barriers. The first stages are
// requested before the kernel waits for its predecessor on the stream (programmatic dependent
// launch). 8 warps at <= 128 registers and <= ~112 KB of shared memory are half an SM, so the
// next kernel's CTA fits beside this one.
//
// Every mbarrier wait is bounded; on expiry the CTA records an error word, stops computing and
// still walks through its named barriers, so no warp is left waiting.
#include "common.cuh"

namespace lq {
namespace gemv {

namespace {

constexpr int kMaxW = 8;        // warps per CTA
constexpr int kMaxStagesMma = 16;
constexpr int kTileRows = 16;

struct MmaParams {
  const __nv_bfloat16* x;
  int ldx;
  const uint8_t* codes;
  const float* scales;
  const __nv_bfloat16* bias;
  const void* residual;
  void* out;
  int out_f32;
  const void* norm_weight;
  float norm_eps;
  int M, N, K, Kd, rowbytes, groups;
  int ldo;  // elements between two activation rows of out / residual
  int W, ntiles, R, H, stages, stage_bytes, scale_off;  // R rows per stage, H = 16 / R stages per tile
  int plane_stride, ncols0, ncols1, unit_off, ring_off;
  int pdl;
  int* error_word;
  unsigned long long* debug;
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#ifdef LQ_DIAGNOSTICS
#define LQ_MMA_STAMP(slot)                                                                     \
  do {                                                                                         \
    if (p.debug != nullptr && threadIdx.x == 0) p.debug[(size_t)blockIdx.x * 8 + (slot)] = global_ns(); \
  } while (0)
#else
#define LQ_MMA_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ void mma_s8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds32f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void named_barrier(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// 16 activations starting at column k0 of one row, widened to fp32; zero beyond K.
__device__ __forceinline__ void load_chunk16(const __nv_bfloat16* row, int k0, int K, bool vec, uint4 (&raw)[2]) {
  if (vec && k0 + 16 <= K) {
    raw[0] = __ldg(reinterpret_cast<const uint4*>(row + k0));
    raw[1] = __ldg(reinterpret_cast<const uint4*>(row + k0) + 1);
  } else {
    unsigned w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = k0 + 2 * i;
      const unsigned lo = k < K ? __bfloat16_as_ushort(row[k]) : 0u;
      const unsigned hi = k + 1 < K ? __bfloat16_as_ushort(row[k + 1]) : 0u;
      w[i] = lo | (hi << 16);
    }
    raw[0] = make_uint4(w[0], w[1], w[2], w[3]);
    raw[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}
__device__ __forceinline__ void widen16(const uint4 (&raw)[2], float (&f)[16]) {
  const unsigned w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// NB = number of B column sets (4 activation rows each); EPI as in the SIMT kernel: 0 = bias /
// residual, 1 = silu(gate) * up over interleaved (gate, up) rows.
// NSEG > 0: a warp owns at most NSEG scale groups of a row and keeps their B fragments and
// units in registers for the whole kernel (they are the same for every tile); NSEG == 0: any
// number of groups, B fragments fetched from shared memory per tile.
template <int BITS, int NB, int EPI, int NSEG>
__global__ void __launch_bounds__(kMaxW * 32, 2)
gemv_mma_kernel(const MmaParams p) {
  constexpr int SEGB = 128 * BITS / 8;  // bytes of one scale group (128 codes) in a weight row
  constexpr int NA = BITS == 8 ? 2 : 1;  // 128-bit loads per row and group
  constexpr int PASSMAX = BITS == 8 ? 2 : 4;  // groups whose A fragments are in registers at once
  constexpr int PASS = (NSEG > 0 && NSEG < PASSMAX) ? NSEG : PASSMAX;
  constexpr int NPASS = NSEG > 0 ? NSEG / PASS : 0;
  extern __shared__ __align__(128) uint8_t dyn[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStagesMma];
  __shared__ float red[2][kMaxW][NB * 2][33];  // 33: the sixteen warps' partials of a slot fall into distinct banks
  __shared__ float nrm[kMaxW][8];
  __shared__ volatile int dead_s;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int W = p.W;
  const int consumers = W * 32;
  LQ_MMA_STAMP(0);

  const int t_begin = (int)(((int64_t)p.ntiles * blockIdx.x) / gridDim.x);
  const int t_end = (int)(((int64_t)p.ntiles * (blockIdx.x + 1)) / gridDim.x);
  const int ntile_cta = t_end - t_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
    }
    dead_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const uint32_t ring_base = smem_u32(dyn + p.ring_off);

  // ------------------------------------------------------------------ stage requests
  // Stage number `it` of this CTA (tile it / H, rows (it % H) * R .. + R of it) goes to ring
  // slot `slot`; called by one thread.
  const int nit = ntile_cta * p.H;
  const int scale_tiles_total = (p.N + 3) / 4;
  auto request = [&](const int it, const int slot, const int row0) {
    const int rows = max(0, min(p.R, p.N - row0));
    const int nt = max(0, min(p.R / 4, scale_tiles_total - row0 / 4));
    const uint32_t bar = smem_u32(&full_bar[slot]);
    const uint32_t dst = ring_base + (uint32_t)slot * p.stage_bytes;
    if (rows == 0) {
      mbar_arrive(bar);  // a stage past the last row: nothing to copy
    } else {
      const uint32_t code_bytes = (uint32_t)rows * p.rowbytes, sc_bytes = (uint32_t)nt * p.groups * 16;
      mbar_expect_tx(bar, code_bytes + sc_bytes);
      bulk_g2s(dst, p.codes + (int64_t)row0 * p.rowbytes, code_bytes, bar);
      bulk_g2s(dst + p.scale_off, p.scales + (int64_t)(row0 / 4) * p.groups * 4, sc_bytes, bar);
    }
    (void)it;
  };
  int next_it = 0;                        // thread 0: the next stage number to request
  int next_row = t_begin * kTileRows;     // and its first row
  if (threadIdx.x == 0) {
    for (; next_it < nit && next_it < p.stages; ++next_it, next_row += p.R) request(next_it, next_it, next_row);
  }

  // ------------------------------------------------------------------ consumer warps
  const int tid = threadIdx.x;  // 0 .. consumers-1
  const int g = lane >> 2, t = lane & 3;
  uint8_t* planes = dyn;
  float* unit_s = reinterpret_cast<float*>(dyn + p.unit_off);  // [4 * NB][groups], 0 beyond M

  // ---- activation set-up, shared by the CTA: items are (row b, 16-column chunk)
  const int nchunk = p.Kd / 16;
  const int items = p.M * nchunk;
  const bool has_norm = p.norm_weight != nullptr;
  const bool vec_x = (p.ldx % 8) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0;
  const bool vec_g = has_norm && (reinterpret_cast<uintptr_t>(p.norm_weight) & 15) == 0;
  const __nv_bfloat16* gw = reinterpret_cast<const __nv_bfloat16*>(p.norm_weight);
  constexpr int kCache = 2;   // items whose norm weights are fetched ahead
  constexpr int kCacheX = 4;  // items whose raw activations stay in registers between the passes
  uint4 gcache[kCache][2];
  if (has_norm) {
    // the norm weight is a constant of the model: fetch it before waiting for the producer
#pragma unroll
    for (int c = 0; c < kCache; ++c) {
      const int it = tid + c * consumers;
      if (it < items) load_chunk16(gw, (it % nchunk) * 16, p.K, vec_g, gcache[c]);
    }
  }
  // activation rows beyond M meet a zero unit, so the lanes that own them accumulate zeros
  for (int i = p.M * p.groups + tid; i < 4 * NB * p.groups; i += consumers) unit_s[i] = 0.f;

  LQ_MMA_STAMP(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  LQ_MMA_STAMP(2);

  uint4 xcache[kCacheX][2];
#pragma unroll
  for (int c = 0; c < kCacheX; ++c) {
    const int it = tid + c * consumers;
    if (it < items) load_chunk16(p.x + (int64_t)(it / nchunk) * p.ldx, (it % nchunk) * 16, p.K, vec_x, xcache[c]);
  }
  if (has_norm) {
    float ss[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) ss[b] = 0.f;
    int c = 0;
    for (int it = tid; it < items; it += consumers, ++c) {
      uint4 raw[2];
      if (c == 0) { raw[0] = xcache[0][0]; raw[1] = xcache[0][1]; }
      else if (c == 1) { raw[0] = xcache[1][0]; raw[1] = xcache[1][1]; }
      else if (c == 2) { raw[0] = xcache[2][0]; raw[1] = xcache[2][1]; }
      else if (c == 3) { raw[0] = xcache[3][0]; raw[1] = xcache[3][1]; }
      else load_chunk16(p.x + (int64_t)(it / nchunk) * p.ldx, (it % nchunk) * 16, p.K, vec_x, raw);
      float f[16];
      widen16(raw, f);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) s = fmaf(f[i], f[i], s);
      const int b = it / nchunk;
#pragma unroll
      for (int bb = 0; bb < 8; ++bb) ss[bb] += (bb == b) ? s : 0.f;
    }
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b < p.M) {
        const float v = warp_sum(ss[b]);
        if (lane == 0) nrm[warp][b] = v;
      }
    }
    named_barrier(consumers);
  }
  LQ_MMA_STAMP(6);

  {
    int c = 0;
    for (int base = 0; base < items; base += consumers, ++c) {
      const int it = base + tid;
      const bool valid = it < items;
      const int b = valid ? it / nchunk : 0, ch = valid ? it % nchunk : 0;
      uint4 raw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
      if (valid) {
        if (c == 0) { raw[0] = xcache[0][0]; raw[1] = xcache[0][1]; }
        else if (c == 1) { raw[0] = xcache[1][0]; raw[1] = xcache[1][1]; }
        else if (c == 2) { raw[0] = xcache[2][0]; raw[1] = xcache[2][1]; }
        else if (c == 3) { raw[0] = xcache[3][0]; raw[1] = xcache[3][1]; }
        else load_chunk16(p.x + (int64_t)b * p.ldx, ch * 16, p.K, vec_x, raw);
      }
      float f[16];
      widen16(raw, f);
      if (has_norm && valid) {
        float tot = 0.f;
        for (int w = 0; w < W; ++w) tot += nrm[w][b];
        const float rstd = __frsqrt_rn(tot / (float)p.K + p.norm_eps);
        uint4 graw[2];
        if (c == 0) { graw[0] = gcache[0][0]; graw[1] = gcache[0][1]; }
        else if (c == 1) { graw[0] = gcache[1][0]; graw[1] = gcache[1][1]; }
        else load_chunk16(gw, ch * 16, p.K, vec_g, graw);
        float gf[16];
        widen16(graw, gf);
        // weight * bf16(x * rstd), the product rounded to bf16 again: the two roundings of a
        // bf16 RMSNorm module
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float nx = __bfloat162float(__float2bfloat16_rn(f[i] * rstd));
          f[i] = __bfloat162float(__float2bfloat16_rn(gf[i] * nx));
        }
      }
      // block exponent of the scale group: eight neighbouring lanes hold its 128 values
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
      unsigned hw[4], lw[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) { hw[q] = 0; lw[q] = 0; }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        // round-to-nearest-even by adding 1.5 * 2^23 in the FMA (|m| < 2^15), not a conversion
        const int m = __float_as_int(fmaf(f[i], up, 12582912.f)) - 0x4B400000;
        const int h = (m + 128) >> 8;
        const int l = m - h * 256;
        // int8: word q = columns 4q .. 4q+3. int4: word 2j = even columns of the j-th eight,
        // word 2j + 1 its odd columns (the order the nibbles unpack in).
        int word, byte;
        if (BITS == 8) { word = i >> 2; byte = i & 3; }
        else { word = 2 * (i >> 3) + (i & 1); byte = (i & 7) >> 1; }
        hw[word] |= (unsigned)(h & 0xFF) << (8 * byte);
        lw[word] |= (unsigned)(l & 0xFF) << (8 * byte);
      }
      if (valid) {
        const int seg = ch >> 3, sub = ch & 7;
        const int col = 2 * (b & 3), set = b >> 2;
        // plane set 0 holds columns of rows 0..3, set 1 those of rows 4..7
        uint8_t* hp = planes + (size_t)(set * p.ncols0 + col) * p.plane_stride + seg * 128;
        uint8_t* lp = hp + p.plane_stride;
        if (BITS == 8) {
          // chunk sub = half * 4 + quad: bytes quad*32 + i*8 + half*4
          const int off = (sub & 3) * 32 + (sub >> 2) * 4;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            *reinterpret_cast<unsigned*>(hp + off + q * 8) = hw[q];
            *reinterpret_cast<unsigned*>(lp + off + q * 8) = lw[q];
          }
        } else {
          // chunk sub = quad * 2 + half16: 16 contiguous bytes
          *reinterpret_cast<uint4*>(hp + sub * 16) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
          *reinterpret_cast<uint4*>(lp + sub * 16) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
        }
        if ((lane & 7) == 0) {
          // value of one mantissa unit; the int4 operand bytes carry 16 * code
          const int ue = e - 14 - (BITS == 4 ? 4 : 0);
          unit_s[b * p.groups + seg] = __uint_as_float((unsigned)(127 + ue) << 23);
        }
      }
    }
  }
  named_barrier(consumers);
  LQ_MMA_STAMP(3);

  // ---- the tile loop over the ring
  // columns a lane feeds as B operand: its group id, folded onto the columns that exist
  const uint32_t planes_u = smem_u32(planes);
  uint32_t bcol[NB];
  bcol[0] = planes_u + (uint32_t)(g % p.ncols0) * p.plane_stride + t * 32;
  if (NB == 2) bcol[NB - 1] = planes_u + (uint32_t)(p.ncols0 + g % p.ncols1) * p.plane_stride + t * 32;
  const uint32_t unit_u = smem_u32(unit_s);
  // rows 2g and 2g + 1 of the tile: which of the tile's H stages, and where inside it
  const int my_h = (2 * g) / p.R;
  const uint32_t a_off = (uint32_t)((2 * g) % p.R) * p.rowbytes + t * 16;
  const uint32_t sc_off = p.scale_off + (uint32_t)(((2 * g) % p.R) >> 2) * p.groups * 16 + (g & 1) * 8;

  constexpr int NREG = NSEG > 0 ? NSEG : 1;
  unsigned breg[NREG][NB][8];
  float ureg[NREG][NB];
  if (NSEG > 0) {
#pragma unroll
    for (int j = 0; j < NREG; ++j) {
      const int grp = warp + j * W;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        uint4 b01 = make_uint4(0, 0, 0, 0), b23 = b01;
        ureg[j][nb] = 0.f;
        if (grp < p.groups) {
          b01 = lds128(bcol[nb] + grp * 128);
          b23 = lds128(bcol[nb] + grp * 128 + 16);
          ureg[j][nb] = lds32f(unit_u + (uint32_t)((t + 4 * nb) * p.groups + grp) * 4);
        }
        breg[j][nb][0] = b01.x; breg[j][nb][1] = b01.y; breg[j][nb][2] = b01.z; breg[j][nb][3] = b01.w;
        breg[j][nb][4] = b23.x; breg[j][nb][5] = b23.y; breg[j][nb][6] = b23.z; breg[j][nb][7] = b23.w;
      }
    }
  }

  float facc[NB][2];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) facc[nb][0] = facc[nb][1] = 0.f;
  float bias_pre[2] = {0.f, 0.f}, res_pre[NB][2];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) res_pre[nb][0] = res_pre[nb][1] = 0.f;

  long long waited = 0, ph[3] = {0, 0, 0};  // diagnostics: SM clocks of thread 0 per phase, summed over tiles
  int cur_stage = 0, cur_phase = 0;  // ring position of the next tile's first stage, kept without divisions
  int n0 = t_begin * kTileRows - kTileRows;
  for (int tile_local = 0; tile_local < ntile_cta; ++tile_local) {
    n0 += kTileRows;
    int sidx[4];  // the tile's stages (H <= 4 of them)
    uint32_t my_stage = 0;
    // Each warp finishes the outputs of two lane positions ("slots", one per half warp) of the
    // tile: their bias and residual do not depend on the products, so fetch them early.
    const int my_slot = 2 * warp + (lane >> 4);  // slot = (g, t) of the lane that owns the pair
    if (EPI == 0 && (lane & 15) == 0 && my_slot < 32) {
      const int n = n0 + 2 * (my_slot >> 2);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (n + r < p.N) {
          if (p.bias != nullptr) bias_pre[r] = __bfloat162float(p.bias[n + r]);
          if (p.residual != nullptr) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              const int b = (my_slot & 3) + 4 * nb;
              if (b < p.M) {
                const int64_t o = (int64_t)b * p.ldo + n + r;
                res_pre[nb][r] = p.out_f32 ? reinterpret_cast<const float*>(p.residual)[o]
                                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[o]);
              }
            }
          }
        }
      }
    }
    bool alive = dead_s == 0;
    const long long w0 = p.debug != nullptr ? clock64() : 0;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      if (h < p.H) {
        sidx[h] = cur_stage;
        if (h == my_h) my_stage = ring_base + (uint32_t)cur_stage * p.stage_bytes;
        if (alive && !mbar_wait(smem_u32(&full_bar[cur_stage]), cur_phase)) {
          dead_s = 1;
          alive = false;
          if (lane == 0) atomicExch(p.error_word, 2);
        }
        if (++cur_stage == p.stages) { cur_stage = 0; cur_phase ^= 1; }
      }
    }
    if (p.debug != nullptr) waited += clock64() - w0;
    if (tile_local == 0) LQ_MMA_STAMP(4);
    if (alive) {
      const uint32_t stage = my_stage;
      // The A fragments of up to PASS scale groups go to registers first, then their products.
      auto do_pass = [&](const int sg0, const int jbase) {
        uint4 ra[PASS][NA], rb[PASS][NA];
        uint2 sc2[PASS];
#pragma unroll
        for (int j = 0; j < PASS; ++j) {
          const int sg = sg0 + j * W;
          if (sg < p.groups) {
            const uint32_t a_addr = stage + a_off + sg * SEGB;
            ra[j][0] = lds128(a_addr);
            rb[j][0] = lds128(a_addr + p.rowbytes);
            if (BITS == 8) {
              ra[j][NA - 1] = lds128(a_addr + 64);
              rb[j][NA - 1] = lds128(a_addr + p.rowbytes + 64);
            }
            sc2[j] = lds64(stage + sc_off + sg * 16);
          }
        }
#pragma unroll
        for (int j = 0; j < PASS; ++j) {
          const int grp = sg0 + j * W;
          if (grp < p.groups) {
            int acc[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0;
              unsigned bw[8];
              if (NSEG > 0) {
                // with NSEG > 0 the pass loop runs once per PASS groups and jj is a constant
#pragma unroll
                for (int q = 0; q < 8; ++q) bw[q] = breg[(jbase + j) % NREG][nb][q];
              } else {
                const uint4 b01 = lds128(bcol[nb] + grp * 128);
                const uint4 b23 = lds128(bcol[nb] + grp * 128 + 16);
                bw[0] = b01.x; bw[1] = b01.y; bw[2] = b01.z; bw[3] = b01.w;
                bw[4] = b23.x; bw[5] = b23.y; bw[6] = b23.z; bw[7] = b23.w;
              }
              const unsigned wa[4] = {ra[j][0].x, ra[j][0].y, ra[j][0].z, ra[j][0].w};
              const unsigned wb[4] = {rb[j][0].x, rb[j][0].y, rb[j][0].z, rb[j][0].w};
              const unsigned wa2[4] = {ra[j][NA - 1].x, ra[j][NA - 1].y, ra[j][NA - 1].z, ra[j][NA - 1].w};
              const unsigned wb2[4] = {rb[j][NA - 1].x, rb[j][NA - 1].y, rb[j][NA - 1].z, rb[j][NA - 1].w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                unsigned a0, a1, a2, a3;
                if (BITS == 8) {
                  a0 = wa[i]; a1 = wb[i]; a2 = wa2[i]; a3 = wb2[i];
                } else {
                  a0 = ((wa[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                  a1 = ((wb[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                  a2 = (wa[i] & 0xF0F0F0F0u) ^ 0x80808080u;
                  a3 = (wb[i] & 0xF0F0F0F0u) ^ 0x80808080u;
                }
                mma_s8(acc[nb], a0, a1, a2, a3, bw[2 * i], bw[2 * i + 1]);
              }
            }
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              const float unit = NSEG > 0 ? ureg[(jbase + j) % NREG][nb]
                                          : lds32f(unit_u + (uint32_t)((t + 4 * nb) * p.groups + grp) * 4);
              facc[nb][0] = fmaf((float)(acc[nb][0] * 256 + acc[nb][1]), __uint_as_float(sc2[j].x) * unit, facc[nb][0]);
              facc[nb][1] = fmaf((float)(acc[nb][2] * 256 + acc[nb][3]), __uint_as_float(sc2[j].y) * unit, facc[nb][1]);
            }
          }
        }
      };
      if (NSEG > 0) {
#pragma unroll
        for (int pass = 0; pass < NPASS; ++pass) do_pass(warp + pass * PASS * W, pass * PASS);
      } else {
        for (int sg0 = warp; sg0 < p.groups; sg0 += W * PASS) do_pass(sg0, 0);
      }
    }

    {
      const int parity = tile_local & 1;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        red[parity][warp][nb * 2][lane] = facc[nb][0];
        red[parity][warp][nb * 2 + 1][lane] = facc[nb][1];
        facc[nb][0] = facc[nb][1] = 0.f;
      }
      if (p.debug != nullptr && threadIdx.x == 0) ph[0] += clock64() - w0;
      named_barrier(consumers);
      if (p.debug != nullptr && threadIdx.x == 0) ph[1] += clock64() - w0;
      // every warp is past its loads of this tile: its stages take the next rows of the stream
      if (threadIdx.x == 0) {
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          if (h < p.H && next_it < nit) {
            request(next_it, sidx[h], next_row);
            ++next_it;
            next_row += p.R;
          }
        }
      }
      // Every warp sums the W (<= 8) partials of two slots per round: lane (half h, index i) reads
      // warp i's partial of slot s + h, a four-step shuffle tree adds the sixteen lanes of the
      // half (fixed order, so results are reproducible), lanes 0 and 16 write the outputs.
      if (dead_s == 0) {
        const int pw = lane & 15;
        for (int s0 = 2 * warp; s0 < 32; s0 += 2 * W) {
          const int slot = s0 + (lane >> 4);
          float tot[NB][2];
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              float v = pw < W ? red[parity][pw][nb * 2 + r][slot] : 0.f;
              v += __shfl_xor_sync(0xffffffffu, v, 8);
              v += __shfl_xor_sync(0xffffffffu, v, 4);
              v += __shfl_xor_sync(0xffffffffu, v, 2);
              v += __shfl_xor_sync(0xffffffffu, v, 1);
              tot[nb][r] = v;
            }
          }
          if (pw != 0) continue;
          const int n = n0 + 2 * (slot >> 2);
          const bool pre = s0 == 2 * warp;  // the prefetched bias / residual belong to this slot
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            const int b = (slot & 3) + 4 * nb;
            if (b >= p.M) continue;
            if (EPI == 1) {
              if (n + 1 < p.N) {
                const float gt = __bfloat162float(__float2bfloat16_rn(tot[nb][0]));
                const float uq = __bfloat162float(__float2bfloat16_rn(tot[nb][1]));
                const float sg = __bfloat162float(__float2bfloat16_rn(gt / (1.f + expf(-gt))));
                const float y = sg * uq;
                const int64_t o = (int64_t)b * p.ldo + n / 2;
                if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = __bfloat162float(__float2bfloat16_rn(y));
                else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(y);
              }
            } else {
#pragma unroll
              for (int r = 0; r < 2; ++r) {
                if (n + r < p.N) {
                  const int64_t o = (int64_t)b * p.ldo + n + r;
                  float bias_v = bias_pre[r], res_v = res_pre[nb][r];
                  if (!pre) {
                    bias_v = p.bias != nullptr ? __bfloat162float(p.bias[n + r]) : 0.f;
                    res_v = 0.f;
                    if (p.residual != nullptr)
                      res_v = p.out_f32 ? reinterpret_cast<const float*>(p.residual)[o]
                                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[o]);
                  }
                  float total = tot[nb][r] + bias_v;
                  if (p.out_f32) {
                    reinterpret_cast<float*>(p.out)[o] = total + res_v;
                  } else {
                    // a bf16 layer output added to a bf16 residual stream: round, add, round
                    if (p.residual != nullptr) total = __bfloat162float(__float2bfloat16_rn(total)) + res_v;
                    reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(total);
                  }
                }
              }
            }
          }
        }
      }
      if (p.debug != nullptr && threadIdx.x == 0) ph[2] += clock64() - w0;
    }
  }
  LQ_MMA_STAMP(5);
  if (p.debug != nullptr && threadIdx.x == 0) {
    p.debug[(size_t)blockIdx.x * 8 + 7] = (unsigned long long)waited;
    if (blockIdx.x == 0) {
      unsigned long long* extra = p.debug + (size_t)gridDim.x * 8;
      extra[0] = (unsigned long long)ph[0]; extra[1] = (unsigned long long)ph[1]; extra[2] = (unsigned long long)ph[2];
      extra[3] = (unsigned long long)ntile_cta;
    }
  }
}

template <int BITS, int NB, int EPI, int NSEG>
int launch_mma(const MmaParams& p, size_t smem, cudaStream_t s) {
  auto kern = gemv_mma_kernel<BITS, NB, EPI, NSEG>;
  if (const int rc = ensure_smem_limit(reinterpret_cast<const void*>(kern), 200 * 1024, "lq_wq_gemv")) return rc;
  const int cap = sm_count();
  int grid = p.ntiles < cap ? p.ntiles : cap;
  if (grid < 1) grid = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)(p.W * 32));
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

}  // namespace

// Shared-memory plan of one launch; false when the shape is outside what the kernel is built for.
struct Plan {
  int nb, ncols0, ncols1, plane_stride, unit_off, ring_off, R, H, scale_off, stage_bytes, W, stages;
  size_t smem;
};
bool make_plan(int M, int Kd, int span, int bits, Plan* out) {
  if (span != 128 || M < 1 || M > 8 || Kd % 128 != 0 || (bits != 4 && bits != 8)) return false;
  Plan q;
  const int rowbytes = Kd * bits / 8, groups = Kd / 128;
  q.nb = M > 4 ? 2 : 1;
  q.ncols0 = 2 * (M > 4 ? 4 : M);
  q.ncols1 = M > 4 ? 2 * (M - 4) : 2;
  q.plane_stride = Kd + 16;
  const int ncols = q.ncols0 + (q.nb == 2 ? q.ncols1 : 0);
  q.unit_off = (ncols * q.plane_stride + 127) / 128 * 128;
  q.ring_off = (q.unit_off + 4 * q.nb * groups * 4 + 127) / 128 * 128;
  if (q.ring_off > 96 * 1024) return false;
  // rows per stage: the largest of 16 / 8 / 4 whose codes stay within 32 KB
  int R = 16;
  while (R > 4 && R * rowbytes > 32 * 1024) R /= 2;
  q.R = R;
  q.H = kTileRows / R;
  q.scale_off = R * rowbytes;
  q.stage_bytes = (q.scale_off + (R / 4) * groups * 16 + 127) / 128 * 128;
  // consumer warps: as many as 8, evened out so that every warp owns the same number of groups
  const int per = (groups + kMaxW - 1) / kMaxW;
  int W = (groups + per - 1) / per;
  if (W > groups) W = groups;
  if (W > kMaxW) W = kMaxW;
  if (W < 1) W = 1;
  q.W = W;
  // ring depth: whatever of ~112 KB per SM the activation planes leave, so that the next
  // kernel's CTA can become resident while this one still computes; a tile and the first
  // stage of the next one have to fit in any case
  int stages = (112 * 1024 - q.ring_off) / q.stage_bytes;
  stages = stages < q.H + 1 ? q.H + 1 : (stages > kMaxStagesMma ? kMaxStagesMma : stages);
  q.stages = stages;
  q.smem = (size_t)q.ring_off + (size_t)stages * q.stage_bytes;
  if (q.smem > 200 * 1024) return false;
  *out = q;
  return true;
}

bool mma_eligible(const lq_gemv_args& a) {
  Plan q;
  return make_plan(a.M, a.Kd, a.span, a.bits, &q);
}

// Runs the tensor-core GEMV. The caller has validated the argument block.
int run_mma(const lq_gemv_args& a, int* error_word, unsigned long long* debug, cudaStream_t s) {
  MmaParams p = {};
  p.x = (const __nv_bfloat16*)a.x; p.ldx = a.ldx; p.codes = (const uint8_t*)a.codes;
  p.scales = a.scale_tiles; p.bias = (const __nv_bfloat16*)a.bias; p.residual = a.residual;
  p.out = a.out; p.out_f32 = a.out_dtype == LQ_F32;
  p.norm_weight = a.norm_weight; p.norm_eps = a.norm_eps;
  p.M = a.M; p.N = a.N; p.K = a.K; p.Kd = a.Kd; p.rowbytes = a.Kd * a.bits / 8; p.groups = a.Kd / 128;
  p.ldo = a.ldo > 0 ? a.ldo : (a.epilogue == 1 ? a.N / 2 : a.N);
  p.pdl = a.pdl; p.error_word = error_word; p.debug = debug;
  Plan q;
  LQ_REQUIRE(make_plan(a.M, a.Kd, a.span, a.bits, &q), LQ_ERR_UNSUPPORTED, "shape outside the tensor-core GEMV");
  const int nb = q.nb;
  p.ncols0 = q.ncols0; p.ncols1 = q.ncols1; p.plane_stride = q.plane_stride; p.unit_off = q.unit_off;
  p.ring_off = q.ring_off; p.R = q.R; p.H = q.H; p.scale_off = q.scale_off; p.stage_bytes = q.stage_bytes;
  p.W = q.W; p.stages = q.stages;
  p.ntiles = (a.N + kTileRows - 1) / kTileRows;
  const size_t smem = q.smem;
  // groups a warp owns: up to 2 or 4 of them keep their B fragments in registers (one column
  // set only; two sets would need too many registers)
  const int per_warp = (p.groups + p.W - 1) / p.W;
  const int nseg = nb == 1 ? (per_warp <= 2 ? 2 : (per_warp <= 4 ? 4 : 0)) : 0;
#define LQ_MMA_CASE(B, NBV, E, S) \
  if (a.bits == B && nb == NBV && a.epilogue == E && nseg == S) return launch_mma<B, NBV, E, S>(p, smem, s);
  LQ_MMA_CASE(8, 1, 0, 2) LQ_MMA_CASE(8, 1, 0, 4) LQ_MMA_CASE(8, 1, 0, 0)
  LQ_MMA_CASE(8, 1, 1, 2) LQ_MMA_CASE(8, 1, 1, 4) LQ_MMA_CASE(8, 1, 1, 0)
  LQ_MMA_CASE(4, 1, 0, 2) LQ_MMA_CASE(4, 1, 0, 4) LQ_MMA_CASE(4, 1, 0, 0)
  LQ_MMA_CASE(4, 1, 1, 2) LQ_MMA_CASE(4, 1, 1, 4) LQ_MMA_CASE(4, 1, 1, 0)
  LQ_MMA_CASE(8, 2, 0, 0) LQ_MMA_CASE(8, 2, 1, 0) LQ_MMA_CASE(4, 2, 0, 0) LQ_MMA_CASE(4, 2, 1, 0)
#undef LQ_MMA_CASE
  return fail(LQ_ERR_ARG, "no tensor-core GEMV instance for bits=%d epilogue=%d", a.bits, a.epilogue);
}

}  // namespace gemv
}  // namespace lq

extern "C" int lq_gemv_tensor_core_ok(int M, int Kd, int span, int bits) {
  lq_gemv_args a = {};
  a.M = M; a.Kd = Kd; a.span = span; a.bits = bits;
  return lq::gemv::mma_eligible(a) ? 1 : 0;
}
