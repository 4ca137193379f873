/* C ABI of libllmquant_b200.so -- hand-written sm_100a kernels for the quantized-linear and
 * quantized-KV path of pjh5672/llm-quant.
 *
 * Conventions
 *   - every pointer named *_d / documented "device" is a CUDA device pointer on the current
 *     device; the library never allocates, frees or synchronizes;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *     every call only enqueues work, so all entry points are CUDA-graph capturable;
 *   - return value 0 = ok, otherwise one of LQ_ERR_*; lq_last_error() returns the message
 *     of the last failing call on the calling thread;
 *   - dtype ids: LQ_F32 / LQ_F16 / LQ_BF16.
 *
 * Each entry point cites the reference interface (path inside pjh5672/llm-quant) whose
 * role it takes.
 */
#ifndef LLMQUANT_B200_H_
#define LLMQUANT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { LQ_F32 = 0, LQ_F16 = 1, LQ_BF16 = 2 };

enum {
  LQ_OK = 0,
  LQ_ERR_ARG = 1,      /* bad shape / size / alignment */
  LQ_ERR_DTYPE = 2,    /* unsupported dtype id */
  LQ_ERR_LAUNCH = 3,   /* the CUDA runtime rejected the launch */
  LQ_ERR_UNSUPPORTED = 4
};

int lq_version(void);
const char* lq_last_error(void);

/* ---------------------------------------------------------------- quantize / dequantize */

/* Fused symmetric RTN quant-dequant over groups of `group_size` along the last axis.
 * Replaces fake_quant_group (llmquant/cuda/csrc/fake_quant.cu:88-139, bound at
 * csrc/fake_quant.cpp:22-29). x, out: [groups * group_size] of `dtype`; scale_out: fp32
 * [groups] or NULL. num_bits in [2, 8]. Bit-exact with core/quant_ops.py:26-37. */
int lq_fake_quant_group(const void* x, void* out, float* scale_out, int64_t groups,
                        int group_size, int num_bits, int dtype, void* stream);

/* Same arithmetic, but emits the integer codes (int8) and the fp32 scale per group instead
 * of the dequantized values: the dynamic activation quantizer of the A8 path
 * (quantizers/real.py:88-90) and the arithmetic of the KV cache's quantize-on-write
 * (quantizers/fake.py:52-54). */
int lq_quantize_group_i8(const void* x, int8_t* codes, float* scale_out, int64_t groups,
                         int group_size, int num_bits, int dtype, void* stream);

/* One-shot weight quantizer: w [N, K] -> canonical codes [N, G, group_size] int8 (K padded
 * with zeros, per head when head_dim > 0) and scales [scale_rows, G] fp32, where
 * scale_rows = ceil(N / out_group) if out_group > 0 else N. Replaces quantize_weight +
 * group_view as called by KernelQuantLinear.from_linear (quantizers/real.py:29-47,
 * quantizers/kernel.py:56-66; scale rule core/observers.py:74-98). */
int lq_quantize_weight(const void* w, int dtype, int N, int K, int group_size, int head_dim,
                       int out_group, int num_bits, int8_t* canonical, float* wscale,
                       void* stream);

/* Nibble codec of the model.bin payload: value + 8, even index -> low nibble
 * (packing/packing.py:20-40). n_codes must be even. */
int lq_pack_int4(const int8_t* codes, uint8_t* packed, int64_t n_codes, void* stream);
int lq_unpack_int4(const uint8_t* packed, int8_t* codes, int64_t n_codes, void* stream);

/* Dequantize canonical codes to a dense [N, G*group_size] matrix of `dtype`:
 * (qweight * broadcast_scale).to(dtype), KernelQuantLinear._dequantized_weight
 * (quantizers/kernel.py:68-79). */
int lq_dequant_weight(const int8_t* canonical, const float* wscale, void* out, int dtype,
                      int N, int groups, int group_size, int out_group, void* stream);

/* out[i] = bf16(bf16(sum[i]) + residual[i]) over n elements (residual bf16 or NULL): the
 * residual add after a row-parallel linear whose fp32 partial outputs were summed over the
 * ranks. Tensor parallelism is not in the reference; on one GPU the GEMV epilogue does this. */
int lq_residual_add(const float* sum, const void* residual, void* out, int64_t n, int pdl, void* stream);

/* ---------------------------------------------------------------- tensor-parallel all-reduce
 * out = bf16(bf16(sum over ranks of partial_r) + residual) for n elements, as one small
 * kernel per rank over peer-mapped memory (no collective library call). Every rank owns a
 * buffer that all ranks have mapped: float data[2][slot_floats] followed, at
 * flag_offset_bytes, by uint32 flags[2][lq_allreduce_max_world()]; it must be zero before the
 * first call. peer_bases_dev is a device array of the `world` base addresses (index = rank).
 * The caller's previous kernel wrote this rank's partial into data[slot] of its own buffer;
 * consecutive calls must alternate slot 0 / 1. seq_counter_dev is a device uint32 (start 0)
 * the kernel advances by one per call -- every rank must make the same sequence of calls.
 * Waiting for the peers is bounded by wait_cycles SM clocks (0 = about two seconds); when the
 * wait runs out lq_allreduce_device_error() becomes 1 and the kernel finishes with what it has.
 * The reference is single-GPU: no counterpart. */
int lq_allreduce_max_world(void);
int lq_allreduce_device_error(void);
int lq_allreduce_residual(const uint64_t* peer_bases_dev, int rank, int world, int slot,
                          int64_t slot_floats, int64_t flag_offset_bytes, uint32_t* seq_counter_dev,
                          const void* residual, void* out, int n, int64_t wait_cycles, int pdl,
                          void* stream);

/* ---------------------------------------------------------------- decode GEMV */

/* Drop-in for wq_gemv (llmquant/cuda/csrc/wq_gemv.cu:134-185, bound at fake_quant.cpp:30-37):
 * out[m, n] = sum_g wscale[row(n), g] * sum_k x[m, g, k] * q[n, g, k], fp32 accumulate,
 * on the reference's canonical layout. x [M, G*group_size], qweight [N, G, group_size] int8,
 * wscale [scale_rows, G] fp32, out [M, N] in x's dtype. group_size % 4 == 0. */
int lq_wq_gemv(const void* x, const int8_t* qweight, const float* wscale, void* out, int M,
               int N, int groups, int group_size, int out_group, int dtype, void* stream);

/* Stacked-expert decode GEMV (Mixture-of-Experts): x [R, groups*group_size] holds the routed
 * rows grouped by expert; block b multiplies rows block_row0[b] .. + block_rows[b] (at most
 * lq_wq_gemv_batched_max_rows() of them) with expert block_expert[b] of qweight
 * [E, N, groups, group_size] int8 and wscale [E, scale_rows, groups] fp32; out [R, N] in x's
 * dtype. Rows no block covers are left untouched. Device int32 arrays of length `blocks`.
 * Replaces wq_gemv_batched (cuda/csrc/wq_gemv_batched.cu:45-185, fake_quant.cpp:14-20,39-51). */
int lq_wq_gemv_batched_max_rows(void);
int lq_wq_gemv_batched(const void* x, const int8_t* qweight, const float* wscale,
                       const int* block_expert, const int* block_row0, const int* block_rows,
                       void* out, int R, int N, int groups, int group_size, int scale_rows,
                       int out_group, int blocks, int dtype, void* stream);

/* Device ("streaming") layout of one quantized linear, built once per layer:
 *   codes        [N, Kd] int8 (bits = 8) or [N, Kd/2] bytes of biased nibbles, low nibble
 *                first (bits = 4) -- byte-identical to the model.bin payload when no head
 *                padding is involved; rows are 16-byte aligned and contiguous, so four
 *                consecutive rows are one contiguous piece of memory; head padding of the
 *                canonical form is stripped when head_dim < group_size (span = head_dim),
 *                otherwise span = group_size and Kd = G * group_size;
 *   scale_tiles  [NP/4, G, 4] fp32, NP = N rounded up to 4: the scales of four consecutive
 *                output rows for every group, contiguous per row tile (rows that share a
 *                scale under out_group each get their copy).
 * lq_stream_layout_sizes returns Kd, span, NP for a canonical shape. There is no
 * counterpart in the reference, which feeds canonical int8 to its kernel. */
int lq_stream_layout_sizes(int N, int groups, int group_size, int head_dim, int bits, int* Kd,
                           int* span, int* NP);
int lq_repack_stream(const int8_t* canonical, const float* wscale, void* codes, float* scale_tiles,
                     int N, int groups, int group_size, int head_dim, int bits, int out_group,
                     void* stream);
/* Exact inverse of lq_repack_stream (used to rebuild `qweight` for save_packed_model). */
int lq_unrepack_stream(const void* codes, const float* scale_tiles, int8_t* canonical,
                       float* wscale, int N, int groups, int group_size, int head_dim, int bits,
                       int out_group, void* stream);

/* Streaming layout -> dense [N, K] matrix of `dtype` (code * scale, rounded once): the
 * operand KernelQuantLinear._dequantized_weight builds for the library GEMM
 * (quantizers/kernel.py:68-79), without the canonical padding columns. */
int lq_dequant_stream(const void* codes, const float* scale_tiles, void* out, int dtype, int N,
                      int K, int Kd, int span, int bits, void* stream);

/* Decode GEMV on the streaming layout, M <= 8 activation rows.
 * x [M, K] bf16 (row stride ldx elements), K real in_features (K <= Kd; columns beyond K
 * read as zero), out [M, N] of out_dtype (LQ_BF16 or LQ_F32), bias bf16 [N] or NULL,
 * residual (out_dtype, [M, N]) or NULL added after the bias.
 * variant: 0 = default (2, or 4 where a second pass over the weight would be needed: 3+ rows on
 * int4, 5+ rows on int8, shapes variant 4 accepts), 1 = fp32 FMA arithmetic, 2 / 3 = integer dot products on 16- / 24-bit
 * block-floating-point activations (32-column blocks), 4 = tensor-core integer products
 * (mma.sync) on 15-bit block-floating-point activations (128-column blocks; needs span == 128
 * and a shape lq_gemv_tensor_core_ok accepts, else LQ_ERR_UNSUPPORTED); 5 (lq_wq_gemv_fused
 * only) = the tcgen05 decode GEMM for up to 64 rows, described with lq_gemv_args.
 * Takes the role of wq_gemv.cu:45-130 inside KernelQuantLinear.forward
 * (quantizers/kernel.py:81-95). */
int lq_wq_gemv_stream(const void* x, int ldx, const void* codes, const float* scale_tiles,
                      const void* bias, const void* residual, void* out, int out_dtype, int M,
                      int N, int K, int Kd, int span, int bits, int variant, void* stream);

/* The GEMV's waits on its shared-memory pipeline are bounded; if one ever expires the kernel
 * records a non-zero word and returns. This reads (and clears) that word; it synchronizes
 * with the device, so it is for tests and diagnostics. -1 = the word could not be read. */
int lq_gemv_device_error(void);

/* 1 if variant 4 of the GEMV serves M activation rows against a weight of Kd stored columns in
 * groups of `span` at `bits` per code, else 0 (the other variants serve every shape). */
int lq_gemv_tensor_core_ok(int M, int Kd, int span, int bits);
/* ---------------------------------------------------------------- decode step bookkeeping
 * Two small kernels that keep the token loop on the device and inside the dependent-launch
 * chain; they take the place of the host-driven copy_ / fill_ / argmax per token of the
 * reference's graphed decoder (runtime/graph_decode.py:40-157).
 * lq_embed_gather: hidden[b, :] = table[tokens[b], :] (bf16 [vocab, H] -> [B, H]).
 * lq_next_token: tokens[b] = argmax over logits[b, :V] (bf16; the lowest index among equal
 * maxima), history[b, *pos + 1] = tokens[b] (history [B, hist_len] int64 or NULL), then *pos += 1
 * once every row has read it. `ticket` is one device int32 holding zero between calls. */
int lq_embed_gather(const void* table, const int64_t* tokens, void* hidden, int B, int H,
                    int64_t vocab, int pdl, void* stream);
int lq_next_token(const void* logits, int64_t V, int64_t* tokens, int64_t* pos, int64_t* history,
                  int64_t hist_len, int* ticket, int B, int pdl, void* stream);

/* lq_next_token under tensor parallelism, where every rank holds the logits of its slice of the
 * vocabulary (local_logits [B, V_local] bf16, global index = rank * V_local + local index):
 * each rank sends (index, value, step tag) of its local maximum as one 8-byte record to every
 * rank's exchange buffer -- uint64 records[2][16][max_batch] at record_offset_bytes of the
 * buffers in peer_bases_dev, zero before the first call -- waits (bounded by wait_cycles SM
 * clocks, 0 = about two seconds) for all ranks' records of this step and picks the largest
 * value, the lowest index among equals, so all ranks pick the same token without gathering
 * the logits. Advances *pos and the device step counter *step (start 0; every rank must make
 * the same sequence of calls). lq_glue_device_error reads and clears the word a wait that ran
 * out sets to 5 (it synchronizes with the device). The reference is single-GPU: no counterpart. */
int lq_glue_device_error(void);
int lq_next_token_tp(const void* local_logits, int64_t V_local, int rank, int world,
                     const uint64_t* peer_bases_dev, int64_t record_offset_bytes, int max_batch,
                     int64_t* tokens, int64_t* pos, int64_t* history, int64_t hist_len, int* ticket,
                     uint32_t* step, int B, int64_t wait_cycles, int pdl, void* stream);

/* ---------------------------------------------------------------- quantized KV cache
 * Storage per layer: codes [B, Hkv, Tmax, D] int8, scales [B, Hkv, Tmax, ceil(D/128)] fp32.
 * A position / length can be given on the host (`pos`, `len`) or through a device int64
 * (`pos_dev`, `len_dev`, which win when non-NULL), so a captured graph follows a moving
 * cursor. */

/* Quantize-on-write: T_new new tokens of K and V ([B, H, T_new, D], element strides for
 * (b, h, t) in k_strides / v_strides, D contiguous) into the cache at `pos`. Takes the role
 * of FakeQuantCache.update's two fake_quantize calls (llmquant/quantizers/fake.py:52-55). */
int lq_kv_write(const void* k, const void* v, const int64_t* k_strides, const int64_t* v_strides,
                int dtype, int8_t* k_codes, int8_t* v_codes, float* k_scales, float* v_scales,
                int B, int H, int T_new, int D, int Tmax, const int64_t* pos_dev, int64_t pos,
                int num_bits, void* stream);

/* codes * scale, rounded to `dtype`: out [B, H, T_len, D] contiguous -- the tensors
 * FakeQuantCache.update returns (llmquant/quantizers/fake.py:55). */
int lq_kv_dequant(const int8_t* codes, const float* scales, void* out, int dtype, int B, int H,
                  int T_len, int D, int Tmax, void* stream);

/* One decode token: rotary embedding of the q and k heads of a fused q|k|v row
 * ([B, (Hq + 2 Hkv) * D] bf16; cos/sin tables [table_len, D] bf16), q to q_out [B, Hq, D]
 * bf16, k and v quantized into the cache at the cursor. In the reference these are
 * transformers' apply_rotary_pos_emb followed by FakeQuantCache.update. */
int lq_rope_kv_write(const void* qkv, const void* cos_table, const void* sin_table, void* q_out,
                     int8_t* k_codes, int8_t* v_codes, float* k_scales, float* v_scales, int B,
                     int Hq, int Hkv, int D, int Tmax, int table_len, const int64_t* pos_dev,
                     int64_t pos, int num_bits, int pdl, void* stream);

/* Dequantize-on-read decode attention: q [B, Hq, D] bf16 against the first
 * (len or *len_dev) + len_add cached tokens, softmax(q k^T * scaling) v, out [B, Hq, D] bf16.
 * The cached tokens are cut into `splits` slices processed by different CTAs; `scratch`
 * (lq_attn_decode_scratch_bytes) holds their partial results. head_dim 64 or 128,
 * Hq / Hkv in {1, 2, 4, 8}. The reference has no such kernel: it attends over the bf16
 * tensors its cache returns through transformers' attention. */
int64_t lq_attn_decode_scratch_bytes(int B, int Hq, int D, int splits);
int lq_attn_decode_kv_i8(const void* q, const int8_t* k_codes, const int8_t* v_codes,
                         const float* k_scales, const float* v_scales, void* out, void* scratch,
                         int B, int Hq, int Hkv, int D, int Tmax, const int64_t* len_dev,
                         int64_t len, int len_add, float scaling, int splits, int pdl, void* stream);

/* The attention block of one decode step as a single launch: rotary embedding of q and k
 * from the fused q|k|v row, quantize-and-append of the new token's K and V at the cursor,
 * attention over the cache including the new token, and the merge of the slices (done by
 * the CTA that finishes last). out [B, Hq, D] bf16. `scratch` (lq_attn_fused_scratch_bytes)
 * must be zero before the FIRST call; every call leaves its tail (the tickets) at zero
 * again. Same arithmetic as lq_rope_kv_write followed by lq_attn_decode_kv_i8. */
int64_t lq_attn_fused_scratch_bytes(int B, int Hq, int Hkv, int D, int splits);
/* Non-zero if a bounded wait inside lq_attn_decode_fused ever expired (reads and clears the
 * word; synchronizes with the device: for tests and diagnostics). */
int lq_attn_device_error(void);
/* `impl` selects the kernel: LQ_ATTN_AUTO = the library's choice (LQ_ATTN_MMA for every shape
 * it is built for), LQ_ATTN_SIMT = all-SIMT arithmetic, LQ_ATTN_MMA = contractions on
 * mma.sync tensor-core instructions with the slices merged through `scratch` by the CTA that
 * finishes last, LQ_ATTN_CLUSTER = the same contractions with the slices of a KV head running as
 * one thread-block cluster that merges through distributed shared memory (`splits` must be 2,
 * 4, 8 or 16; LQ_ERR_UNSUPPORTED if such clusters do not fit the device). Same results within
 * the attention tolerance. */
enum { LQ_ATTN_AUTO = 0, LQ_ATTN_SIMT = 1, LQ_ATTN_MMA = 2, LQ_ATTN_CLUSTER = 3 };
int lq_attn_decode_fused(const void* qkv, const void* cos_table, const void* sin_table,
                         int8_t* k_codes, int8_t* v_codes, float* k_scales, float* v_scales,
                         void* out, void* scratch, int B, int Hq, int Hkv, int D, int Tmax,
                         int table_len, const int64_t* pos_dev, int64_t pos, int num_bits,
                         float scaling, int splits, int impl, int pdl, void* stream);

/* lq_attn_decode_kv_i8 for callers that cannot provide scratch memory -- a plugin inside a
 * process whose device memory belongs to someone else's allocator, or a host that is not
 * allowed to call cudaMalloc. The partial results of the slices go to a fixed 4 MiB array that
 * is part of the library image (lq_attn_decode_static_scratch_bytes; every GPU that loads
 * the library holds it until the process exits); a call whose B * Hq * splits * (D + 2) * 4
 * bytes exceed it is rejected with LQ_ERR_UNSUPPORTED. Nothing is allocated or freed. The
 * first call on each device resolves the array's device address; make that call outside
 * any stream capture. The array belongs to the CURRENT device at the time of the call, so that
 * device must be the one that owns `stream` and every tensor passed (set it before calling);
 * the address is remembered per device ordinal for the life of the process, so a process that
 * resets a device (cudaDeviceReset) must not use this entry point on it afterwards. Nothing in the array has to start at zero (every slot a call reads it
 * has written first), but all calls share it: two calls that overlap on the GPU (different
 * streams, or graph branches) race -- serialize them. This entry point has no counterpart
 * in the reference. */
int64_t lq_attn_decode_static_scratch_bytes(void);
int lq_attn_decode_kv_i8_static(const void* q, const int8_t* k_codes, const int8_t* v_codes,
                                const float* k_scales, const float* v_scales, void* out, int B,
                                int Hq, int Hkv, int D, int Tmax, const int64_t* len_dev, int64_t len,
                                int len_add, float scaling, int splits, int pdl, void* stream);

/* ---------------------------------------------------------------- prefill GEMM (tcgen05 / TMEM)
 * out[m, n] = sum_g s_w[n, g] * s_x[m, g] * sum_{k in g} a[m, k] * q[n, k] on the streaming
 * layout, any M (tiles of 128 tokens x 128 features), out [M, N] bf16, bias bf16 or NULL.
 *   A16: x [M, K] bf16 (x_codes = NULL, s_x = 1): kind::f16 MMA on bf16(code), fp32 accumulate,
 *        scales applied per group in fp32 (the arithmetic of the reference's real mode). With
 *        LQ_GEMM_FOLD_SCALES in `flags` the B operand is bf16(float(code) * scale) instead -- the
 *        weight tensor the reference's kernel mode feeds its library GEMM
 *        (quantizers/kernel.py:68-79) -- and one accumulator runs over all of K: several
 *        times faster, with that mode's bf16 rounding of the weights (needs K % 8 == 0 and a
 *        16-byte aligned x, else the flag is ignored).
 *   A8:  x_codes [M, Kd] int8 + x_scales [M, G] fp32 as lq_quantize_group_i8 produces them
 *        (dynamic, per token per group): kind::i8 MMA, int32 accumulate -- the arithmetic of
 *        RealQuantLinear.forward with an int8 activation scheme (quantizers/real.py:88-99).
 * span must be 64 or 128. Replaces the dequantize-then-cuBLAS branch of
 * KernelQuantLinear.forward (quantizers/kernel.py:68-79,90-91). lq_gemm_device_error is
 * non-zero if a bounded wait for the tensor core ever expired (reads and clears). */
int lq_gemm_device_error(void);
/* flags: LQ_GEMM_FOLD_SCALES as described above; LQ_GEMM_SERIAL runs the first, unpipelined
 * kernel (fill, MMA and drain in turn) instead of the warp-specialized ones -- same results. */
#define LQ_GEMM_FOLD_SCALES 1
#define LQ_GEMM_SERIAL 2
int lq_wq_gemm_prefill(const void* x, int ldx, const int8_t* x_codes, const float* x_scales,
                       const void* codes, const float* scale_tiles, const void* bias, void* out,
                       int M, int N, int K, int Kd, int span, int bits, int flags, void* stream);

/* The same GEMV with the work of the neighbouring decoder-layer ops folded in. All fields
 * of lq_wq_gemv_stream, plus:
 *   norm_weight / norm_eps  bf16 [K] or NULL: RMSNorm applied to x inside the kernel
 *                           (x * rsqrt(mean(x^2) + eps), rounded to bf16, times weight,
 *                           rounded to bf16 -- the arithmetic of a bf16 RMSNorm module);
 *   epilogue                0 = none; 1 = rows are (gate, up) pairs and the output is
 *                           silu(gate) * up, [M, N/2];
 *   pdl                     1 = launch with programmatic stream serialization: the kernel
 *                           streams its first weights while the previous kernel on the
 *                           stream drains, and waits for it before touching x.
 * These fusions have no counterpart in the reference, which runs them as separate PyTorch
 * ops between its wq_gemv calls (llmquant/quantizers/kernel.py:81-95 is the call site). */
/* Tensor-parallel coupling of a GEMV (NULL in lq_gemv_args.tp = none). The reference is
 * single-GPU, so this has no counterpart there. Every rank owns one exchange buffer that all
 * ranks of the group have mapped (NVLink peer memory); per slot it holds the fp32 partial
 * outputs of every rank, float part[world][M][N]. A 32-bit word of it -- and of the bf16
 * hidden-state rows named below -- holds the bit pattern 0xFFFFFFFF ("empty": NaNs nothing here
 * computes) while no value is there, so data that arrives is its own signal: a reader re-reads
 * a 16-byte piece until none of its words is empty. Plain stores and loads only; no flags,
 * fences, counters or copies.
 *   mode LQ_TP_PUSH  (row-parallel linear: o_proj, down_proj) -- the epilogue writes this
 *        rank's fp32 partial rows straight into part[rank] of EVERY rank's buffer
 *        (peers[r] + data_offset). `out` and `residual` must be NULL / unused; N % 4 == 0.
 *   mode LQ_TP_SUM   (the linear that consumes the sum: gate|up after o_proj, the next
 *        layer's q|k|v or lm_head after down_proj) -- the first CTAs of the grid read the
 *        `world` partials of `parts` (waiting, bounded, for words still empty), add them in
 *        rank order (identical bits on every rank), round to bf16, add `residual` (bf16 [M, K])
 *        and store the new hidden rows to `x`, which must be EMPTY when the kernel starts;
 *        every CTA then reads x as the GEMV input, waiting for the pieces it needs. The CTAs
 *        that sum put "empty" back into the partial words and into the `residual` rows they
 *        have read -- so the caller alternates two hidden-state buffers between consecutive
 *        summing GEMVs (this one's `residual` is the next one's `x`) and fills the first `x`
 *        and the whole exchange buffer with 0xFF bytes before the first step.
 *        K a multiple of 16 (int8) / 32 (int4) codes, ldx == K, 16-byte aligned pointers.
 * wait_cycles bounds each wait in SM clocks (0 = about two seconds; rows are given twice
 * that); when one runs out lq_gemv_device_error() reports 3 (partials) or 4 (rows) and the
 * kernel finishes with the data it has. */
enum { LQ_TP_PUSH = 1, LQ_TP_SUM = 2 };
typedef struct lq_gemv_tp {
  int mode;
  int world, rank;
  const uint64_t* peers;       /* PUSH: device array [world], base address of every rank's buffer */
  int64_t data_offset;         /* PUSH: byte offset of part[0] of the slot inside a buffer */
  float* parts;                /* SUM: this rank's part[0] of the slot (local address) */
  void* residual;              /* SUM: bf16 [M, K]; left empty */
  int64_t wait_cycles;
} lq_gemv_tp;

typedef struct lq_gemv_args {
  const void* x;
  int ldx;
  const void* norm_weight;
  float norm_eps;
  const void* codes;
  const float* scale_tiles;
  const void* bias;
  const void* residual;
  void* out;
  int out_dtype;
  int M, N, K, Kd, span, bits;
  int epilogue;
  int variant;
  int pdl;
  const lq_gemv_tp* tp;        /* NULL = no tensor-parallel coupling */
  int ldo;                     /* elements between two rows of out / residual; 0 = dense (N, or N/2
                                  with epilogue 1). Lets a launch cover a block of the output
                                  columns: a slice of the weight's rows against all activation rows. */
  void* workspace;             /* variant 5 only: lq_decode_gemm_workspace_bytes(M, N, Kd) bytes, 256-byte aligned */
  int64_t workspace_bytes;
} lq_gemv_args;
int lq_wq_gemv_fused(const lq_gemv_args* args, void* stream);

/* variant 5 of lq_wq_gemv_fused: the decode GEMM for 1..64 activation rows (the sequences of a
 * decode step) on tcgen05 tensor cores -- the weights are streamed ONCE for all rows, where
 * the GEMV variants take 8 rows per pass. `codes` is the weight in the TILE-MAJOR layout of
 * lq_tile_weight (not the streaming layout of the other variants).
 * Three launches: the activation rows (through the optional RMSNorm) become 15-bit
 * block-floating-point byte planes in `workspace`; CTAs that share the weight's (128-row tile,
 * scale group) steps in equal contiguous runs multiply them with kind::i8 MMAs into tensor memory and applies (weight
 * scale x activation unit) per group in fp32 -- the order of operations of
 * quantizers/real.py:93-99; a last kernel adds the parts of every row tile and applies bias, residual or
 * silu(gate) * up. Needs span == 128. Same fusions and roundings as the other variants; no
 * tensor-parallel coupling. The workspace may be shared by consecutive launches on one stream.
 * lq_decode_gemm_device_error is non-zero if a bounded wait inside the kernel ever expired
 * (reads and clears the word; synchronizes: for sync points). Replaces, for batched decode,
 * the dequantize + library GEMM branch of quantizers/kernel.py:68-79,90-91.
 *
 * lq_tile_weight: streaming layout -> tile-major: per tile of 128 weight rows and per scale
 * group of 128 codes one contiguous block -- the codes (int8: 16 KB, already in the swizzled
 * order the MMA reads from shared memory; int4: 8 KB of nibble bytes), then the 128 fp32 scales
 * of the block's rows; rows beyond N are zeros -- so that a CTA fetches a group with one linear
 * bulk copy. `out` takes lq_tile_weight_bytes(N, Kd, bits) bytes; variant 5 is given it as
 * `codes` (its `scale_tiles` is not read). */
int64_t lq_tile_weight_bytes(int N, int Kd, int bits);
int lq_tile_weight(const void* codes, const float* scale_tiles, void* out, int N, int Kd, int bits,
                   void* stream);
int64_t lq_decode_gemm_workspace_bytes(int M, int N, int Kd);
int lq_decode_gemm_device_error(void);

#ifdef __cplusplus
}
#endif
#endif /* LLMQUANT_B200_H_ */
