/*
 * b200int — C ABI of the B200 (sm_100a) kernels for the integer-only W8A8 forward path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the given
 * CUDA stream and returns immediately: 0 on success, a negative B200_E_* code when
 * an argument is rejected (nothing is launched in that case).  No entry point
 * allocates, frees or synchronises unless its comment says so.  All pointers are
 * borrowed for the duration of the call; the caller owns every buffer.
 * b200_last_error_string() returns the message of the calling thread's last failure.
 *
 * Citations name the reference interface each entry point stands in for, as
 * file:line inside the mini-sgl-integer source tree (python/minisgl/...).
 */
#ifndef B200INT_H_
#define B200INT_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b200_stream_t; /* a cudaStream_t; NULL is the legacy default stream */

enum {
  B200_OK = 0,
  B200_E_NULL = -1,        /* a required pointer is NULL */
  B200_E_SHAPE = -2,       /* a size is zero/negative or inconsistent */
  B200_E_ALIGN = -3,       /* a pointer or row pitch is not 16-byte aligned */
  B200_E_UNSUPPORTED = -4, /* a size outside what the kernels are built for */
  B200_E_CUDA = -5         /* the CUDA runtime reported an error at launch */
};

B200_API int b200_version(void);
B200_API const char* b200_last_error_string(void);

/* Copies one compiled-in 1024-entry table to host memory.
 * which: 0 = inverse-sqrt (kernel/fixed_point/rmsnorm_int_only_v2.py:31-43),
 *        1 = exp2 for SiLU (kernel/fixed_point/silu_and_mul_int_only.py:35-46),
 *        2 = exp2 for attention (kernel/triton/int8_attention_kernels.py:27-29). */
B200_API int b200_get_lut(int which, int32_t* out_host_1024);

/* ---- Q15.16 conversion: kernel/fixed_point/q15_tensor.py:17-28 (to_fixed / from_fixed).
 * bf16 values travel as raw 16-bit patterns. */
B200_API int b200_to_fixed_f32(const float* x, int32_t* out, int64_t n, b200_stream_t s);
B200_API int b200_to_fixed_bf16(const uint16_t* x, int32_t* out, int64_t n, b200_stream_t s);
B200_API int b200_from_fixed_f32(const int32_t* x, float* out, int64_t n, b200_stream_t s);
B200_API int b200_from_fixed_bf16(const int32_t* x, uint16_t* out, int64_t n, b200_stream_t s);

/* ---- Fixed-point RMSNorm, optional residual add, optional per-token int8 quant.
 * Replaces rmsnorm_int_only_v2 (kernel/fixed_point/rmsnorm_int_only_v2.py:319-390),
 * fused_add_rmsnorm_int_only_v2 (:393-475) and, when codes != NULL, the
 * per_token_quant_int8_from_q15 that follows them inside apply_weights_q15
 * (layers/quantization/w8a8_int8.py:104-131).
 *   x, residual (nullable), residual_out (required iff residual), norm_out (nullable):
 *       int32 [rows, hidden], dense rows; weight int32 [hidden].
 *   codes int8 [rows, hidden], scale fp32 [rows], absmax int32 [rows]: all three or none.
 * hidden must be a multiple of 4 and at most 32768. */
B200_API int b200_rmsnorm_q15(const int32_t* x, const int32_t* residual, const int32_t* weight,
                     int32_t* residual_out, int32_t* norm_out,
                     int8_t* codes, float* scale, int32_t* absmax,
                     int64_t rows, int hidden, b200_stream_t s);

/* ---- SiLU(gate) * up, optional blocked Walsh-Hadamard rotation, optional per-token quant.
 * Replaces silu_and_mul_int_only (kernel/fixed_point/silu_and_mul_int_only.py:233-275),
 * apply_blockwise_fwht_q15 (models/utils_integer.py:46-60) and the per-token quant of the
 * following down_proj (layers/quantization/w8a8_int8.py:104-131).
 *   gate_up int32 [rows, 2*inter] laid out gate || up; q15_out int32 [rows, inter] (nullable);
 *   codes/scale/absmax as above (all three or none).
 * fwht_block: 0 = no rotation, or 128.  inter must be a multiple of 128 (of 4 when
 * fwht_block == 0 and codes == NULL) and at most 49152. */
B200_API int b200_silu_mul_q15(const int32_t* gate_up, int32_t* q15_out,
                      int8_t* codes, float* scale, int32_t* absmax,
                      int64_t rows, int inter, int fwht_block, b200_stream_t s);

/* ---- Walsh-Hadamard transform of every n-wide row with per-stage int32 saturation.
 * Replaces fwht_int_q15 (kernel/fixed_point/fwht_int.py:99-147). n: power of two, 2..1024. */
B200_API int b200_fwht_q15(const int32_t* x, int32_t* out, int64_t rows, int n, int normalize,
                  b200_stream_t s);

/* ---- Integer RoPE (neox halves), optionally followed by the FWHT over every head.
 * Replaces rope_int_q15 (kernel/fixed_point/rope_int.py:128-247) and rope_fwht_int_q15
 * (kernel/fixed_point/rope_fwht_int.py:9-23).
 *   positions int32 [tokens]; q int32 [tokens, q_heads, 128]; k int32 [tokens, kv_heads, 128];
 *   cos_sin int32 [max_pos, 128] (cos || sin, Q1.15).  head_dim is fixed at 128.
 *   q_norm_w / k_norm_w (nullable, int32 [128]): when given, each head row first goes
 *   through the fixed-point RMSNorm (the q_norm / k_norm of models/utils_integer.py:214-218).
 * Row pitches are in int32 elements so that q and k may be views into one qkv buffer. */
B200_API int b200_qk_rope_q15(const int32_t* positions, const int32_t* q, int64_t q_pitch,
                     const int32_t* k, int64_t k_pitch, const int32_t* cos_sin, int max_pos,
                     const int32_t* q_norm_w, const int32_t* k_norm_w,
                     int32_t* q_out, int32_t* k_out, int64_t tokens, int q_heads, int kv_heads,
                     int with_fwht, b200_stream_t s);

/* ---- Per-row int8 quantisation of Q15.16 values.
 * Replaces per_token_quant_int8_from_q15 (layers/quantization/w8a8_int8.py:104-131).
 * x int32 [rows, k] -> codes int8 [rows, k], scale fp32 [rows], absmax int32 [rows]. */
B200_API int b200_per_token_quant_q15(const int32_t* x, int8_t* codes, float* scale, int32_t* absmax,
                             int64_t rows, int k, b200_stream_t s);

/* ---- Fixed-point form (multiplier in [2^30,2^31), shift) of the scale absmax/(127*65536).
 * No counterpart in the reference (its requant is a float library epilogue). */
B200_API int b200_absmax_to_mul_shift(const int32_t* absmax, int32_t* mul, int32_t* shift, int64_t n,
                             b200_stream_t s);

/* ---- int8 paged KV pool, one layer:
 *   k_codes int8 [pages, kv_heads, 16, 128] (token rows);
 *   v_codes int8 [pages, kv_heads, 2048]: the page's 16 x 128 bytes in tensor-core operand
 *   order, byte (d, tok) at ((w>>2)<<9) + (l<<4) + ((w&3)<<2) + (tok&3) with
 *   w = (d>>4)*2 + ((d>>3)&1), l = (d&7)*4 + (tok>>2);
 *   meta int32 [pages, kv_heads, 40]: words 0-15 k multipliers, 16-31 v multipliers,
 *   32-35 sixteen int8 k shifts, 36-39 sixteen int8 v shifts.
 * A token location is page*16 + offset.  Pools are written by the two store entry points.
 *
 * b200_kv_store_q15 quantises Q15.16 K and V rows per token and KV head (codes as
 * per_token_quant_int8_from_q15 on each 128-wide row; multiplier/shift as
 * b200_absmax_to_mul_shift) and scatters them to out_loc.  It stands in for
 * MHAKVCache.store_kv (kvcache/mha_pool.py:46-57) -> store_cache (kernel/store.py:30-42)
 * -> store_kv_cache (kernel/csrc/jit/store.cu:27-56).  k, v: int32 rows of
 * kv_heads*128 with the given pitch (elements); out_loc int32 [tokens]. */
B200_API int b200_kv_store_q15(const int32_t* k, int64_t k_pitch, const int32_t* v, int64_t v_pitch,
                      const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes, int32_t* meta,
                      int64_t tokens, int kv_heads, int64_t num_pages, b200_stream_t s);

/* Scatter already-quantised tokens (codes int8 [tokens, kv_heads, 128]; mul/shift int32
 * [tokens, kv_heads]) into the pool.  Used to preload pools with given codes. */
B200_API int b200_kv_store_codes(const int8_t* k8, const int8_t* v8, const int32_t* k_mul,
                        const int32_t* k_shift, const int32_t* v_mul, const int32_t* v_shift,
                        const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes, int32_t* meta,
                        int64_t tokens, int kv_heads, int64_t num_pages, b200_stream_t s);

/* ---- Everything between the qkv projection and attention in one launch: per (token, head) row,
 * q-norm / k-norm (nullable weights) + RoPE + Hadamard rotation of q and k as b200_qk_rope_q15, then
 *   q rows: per-row int8 codes (b200_per_token_quant_q15) -> q8 int8 [tokens, q_heads, 128] and their
 *           (multiplier, shift) (b200_absmax_to_mul_shift) -> q_mul, q_shift int32 [tokens, q_heads];
 *   k rows and the untouched v rows: quantised and scattered into the pool as b200_kv_store_q15.
 * Same bits as those four calls in sequence.  Stands in for the part of AttentionLayerInteger.forward_q15
 * between qkv_proj and the backend (models/utils_integer.py:209-227) plus the backend's store_kv
 * (attention/triton_int8.py:125). */
B200_API int b200_qkv_prepare_q15(const int32_t* positions, const int32_t* q, int64_t q_pitch, const int32_t* k,
                                  int64_t k_pitch, const int32_t* v, int64_t v_pitch, const int32_t* cos_sin,
                                  int max_pos, const int32_t* q_norm_w, const int32_t* k_norm_w,
                                  const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes, int32_t* meta,
                                  int8_t* q8, int32_t* q_mul, int32_t* q_shift, int64_t tokens, int q_heads,
                                  int kv_heads, int64_t num_pages, int with_fwht, b200_stream_t s);

/* ---- Decode attention over the int8 paged pool with an exact fixed-point softmax.
 * Stands in for Int8Backend._forward_decode (attention/triton_int8.py:155-176), which in the
 * reference runs a bf16 kernel; the integer arithmetic follows int8_context_attention_fwd
 * (kernel/triton/int8_attention_kernels.py:278-383) generalised to per-key scales.
 *   q int8 [batch, q_heads, 128]; q_mul, q_shift int32 [batch, q_heads];
 *   page_table int32 [batch, table_pitch] of page ids; kv_lens int32 [batch];
 *   out_q15 int32 [batch, q_heads, 128] (nullable); out_codes int8 same shape with
 *   out_absmax int32 [batch, q_heads] (both or none): per (token, head) row quant.
 * q_heads / kv_heads must be 1, 2, 4 or 8.  max_kv_len bounds every kv_lens[i] (it sizes
 * shared memory); lengths above it are clamped.  cluster: CTAs that share one
 * (sequence, KV head), 1, 2, 4 or 8; 0 lets the library choose.
 * row_order int32 [batch] (nullable): a permutation of the batch rows, longest sequence first; the
 * CTAs take the rows in this order, which shortens the tail of the launch (the result does not depend
 * on it).  Whoever schedules the batch knows the lengths; without it, batches of up to 64 rows are
 * ranked inside the kernel and larger ones run in the given order. */
B200_API int b200_attn_decode(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                     const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                     const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                     const int32_t* row_order,
                     int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax,
                     int batch, int q_heads, int kv_heads, int64_t num_pages, int max_kv_len,
                     int cluster, b200_stream_t s);

/* ---- Extend (prefill over a cached prefix) attention on the same pool and arithmetic.
 * Stands in for Int8Backend._forward_prefill (attention/triton_int8.py:178-212) ->
 * int8_context_attention_fwd (kernel/triton/int8_attention_kernels.py:229-383), and unlike the
 * reference it attends the cached prefix as well as the new tokens.  The new tokens must already be
 * in the pool.  One query row per new token: q int8 [rows, q_heads, 128]; row_seq int32 [rows] is the
 * row's sequence (index into page_table / kv_lens); row_limit int32 [rows] the number of keys the row
 * may see (for the i-th of n new tokens of a sequence with L keys: L - n + i + 1).  The reference V
 * scale of a row is taken over all kv_lens[seq] keys.  rows <= 65535.  Every row re-reads its keys:
 * meant for short extends (chunked prefill tails, speculative/verify steps), not for long prompts. */
B200_API int b200_attn_extend(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                              const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                              const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                              const int32_t* row_seq, const int32_t* row_limit,
                              int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax,
                              int rows, int q_heads, int kv_heads, int64_t num_pages, int max_kv_len,
                              int cluster, b200_stream_t s);

/* ---- Prefill / extend attention for many new tokens per sequence: one CTA per (sequence, KV head, tile of
 * 128 / (q_heads / kv_heads) consecutive new tokens) with the query rows on the M side of the integer MMA, the
 * pages of K and V streamed through shared memory once per pass over the keys (three passes for K: the exact
 * softmax cannot be rescaled, so row maxima, sums and probabilities each recompute the scores; one for V).
 * Same arithmetic and results as b200_attn_extend, which re-reads all keys for every single query row.
 * Stands in for Int8Backend._forward_prefill (attention/triton_int8.py:178-212) -> int8_context_attention_fwd
 * (kernel/triton/int8_attention_kernels.py:229-383); unlike the reference it attends the cached prefix too.
 *   q int8 [rows, q_heads, 128], the sequences' new tokens back to back; q_mul, q_shift int32 [rows, q_heads];
 *   kv_lens int32 [batch] (new tokens included, already in the pool); q_lens int32 [batch]; q_start int32
 *   [batch]: the row of each sequence's first new token; max_q_len bounds every q_lens[i] (it sizes the grid).
 *   The i-th of n new tokens of a sequence with L keys sees keys 0 .. L - n + i.  Outputs as b200_attn_decode. */
B200_API int b200_attn_prefill(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                               const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                               const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                               const int32_t* q_lens, const int32_t* q_start,
                               int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax,
                               int batch, int max_q_len, int q_heads, int kv_heads, int64_t num_pages,
                               int max_kv_len, b200_stream_t s);

/* ---- The same decode / extend attention as a chain of grid-wide passes that meet in a caller-provided
 * workspace (scores, row maxima and sums, reference V scales, int32 output accumulators) instead of
 * inside thread-block clusters: better balanced, any context length.  Same arguments and results as
 * b200_attn_decode (row_seq == row_limit == NULL, rows = batch) and b200_attn_extend.
 * workspace: device memory, 256-byte aligned, at least b200_attn_workspace_bytes(...) bytes; its
 * contents need not survive the call.  Calls that share a workspace must not overlap on the GPU. */
B200_API size_t b200_attn_workspace_bytes(int rows, int q_heads, int kv_heads, int max_kv_len);
B200_API int b200_attn_paged_ws(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                                const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                                const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                                const int32_t* row_seq, const int32_t* row_limit,
                                int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax,
                                int rows, int q_heads, int kv_heads, int64_t num_pages, int max_kv_len,
                                void* workspace, size_t workspace_bytes, b200_stream_t s);

/* ---- b200_attn_paged_ws without a workspace argument: the scratch is a fixed area of
 * B200_ATTN_STATIC_SCRATCH_BYTES that is part of the library's device image.  This entry point has no
 * counterpart in the reference; it is for callers that cannot allocate device memory: a binding that only
 * forwards the model's tensors (a plain C host, a tvm-ffi wrapper) and so has no allocator, or an engine that
 * has already handed all free device memory to the KV pool and cannot rely on a later allocation.  The call
 * allocates and frees nothing.
 *  - Limit: b200_attn_workspace_bytes(rows, q_heads, kv_heads, max_kv_len) must not exceed
 *    B200_ATTN_STATIC_SCRATCH_BYTES, otherwise B200_E_UNSUPPORTED with the two sizes in the message
 *    (16 MiB holds e.g. 16 rows x 32 query heads x 7680 keys); use b200_attn_paged_ws beyond that.
 *  - The first call on each device looks up the area's device address (the device must be current, as for
 *    every call here); make that first call during set-up, before any stream capture begins.  With the CUDA
 *    runtime's lazy module loading the area itself comes into being when this part of the library is first
 *    used on the device, i.e. at that first call (or an earlier b200_attn_paged_ws): an engine that hands all
 *    free memory to its KV pool must make the first call BEFORE it sizes the pool, or the look-up fails with
 *    B200_E_CUDA.  From the second call on nothing changes in device memory.
 *  - There is one area per device and every call uses it: calls on the same device must not overlap on the
 *    GPU (issue them on one stream, or order them with events), else they corrupt each other's results.
 *    Nothing in the area has to be cleared by the caller: the first kernel of each call resets what the
 *    later ones accumulate into.
 * Arguments and results are those of b200_attn_paged_ws. */
#define B200_ATTN_STATIC_SCRATCH_BYTES (16u << 20)
B200_API int b200_attn_paged_static(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                                    const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                                    const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                                    const int32_t* row_seq, const int32_t* row_limit,
                                    int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax,
                                    int rows, int q_heads, int kv_heads, int64_t num_pages, int max_kv_len,
                                    b200_stream_t s);

/* ---- The two ends of the model and the bookkeeping of a decode step.
 * b200_embedding_bf16_q15: out[t, :] = to_fixed(table[ids[t] - vocab_start, :]) for a bf16 table of
 *   vocab_rows rows; ids outside the shard give zero rows (a vocabulary-parallel shard, summed over ranks).
 *   Stands in for VocabParallelEmbedding.forward (layers/embedding.py:33-42, csrc/jit/index.cu) followed by
 *   to_fixed at the model entry (models/integer/qwen3_integer.py:115-124).  hidden % 8 == 0.
 * b200_argmax_i32: out_idx[r] = index_offset + argmax_j logits[r, j], the lowest index among equal maxima;
 *   out_val[r] (nullable) the maximum.  Stands in for the greedy branch of the sampler (engine/sample.py:74)
 *   on integer logits.  Rows 16-byte aligned (pitch % 4 == 0).
 * b200_decode_prepare: for a decode batch whose lengths live on the device: positions[b] = seq_lens[b],
 *   out_loc[b] = page_table[b][pos / 16] * 16 + pos % 16, kv_lens[b] = pos + 1, then seq_lens[b] = pos + 1
 *   (pos is held at max_len - 1 once a sequence is full).  Replaces the per-request host loops of
 *   Int8Backend.prepare_metadata (attention/triton_int8.py:214-253) for decode, so a step can be replayed
 *   from a CUDA graph. */
B200_API int b200_embedding_bf16_q15(const uint16_t* table, const int32_t* ids, int32_t* out, int64_t rows,
                                     int hidden, int64_t vocab_start, int64_t vocab_rows, b200_stream_t s);
B200_API int b200_argmax_i32(const int32_t* logits, int64_t rows, int64_t n, int64_t pitch, int32_t index_offset,
                             int32_t* out_idx, int32_t* out_val, b200_stream_t s);
B200_API int b200_decode_prepare(const int32_t* page_table, int64_t table_pitch, int32_t* seq_lens,
                                 int32_t* positions, int32_t* out_loc, int32_t* kv_lens, int batch, int max_len,
                                 b200_stream_t s);

/* ---- Per-tensor int8 quantisation of a bf16 tensor with a (multiplier, shift) scale:
 * quantize_per_tensor_int8_ms (kernel/triton/int8_attention_kernels.py:41-53), which the reference's prefill
 * applies to q, k and v (attention/triton_int8.py:139-140,190).  x_bf16: n raw bf16 patterns; codes int8 [n];
 * mul_shift int32 [2] = (multiplier, shift) with value ~ code * multiplier / 2^shift; scratch_word: one
 * caller-owned uint32 on the device (holds the running maximum).  Three stream operations, no host sync. */
B200_API int b200_quantize_per_tensor_int8_ms(const uint16_t* x_bf16, int64_t n, int8_t* codes, int32_t* mul_shift,
                                              uint32_t* scratch_word, b200_stream_t s);

/* ---- Static activation quantisation for checkpoints that carry an `input_scale`:
 * codes = clamp(rint((fp32(x) / 65536) / input_scale), -128, 127) in fp32 with IEEE division, i.e.
 * per_tensor_quant_int8_static (layers/quantization/w8a8_int8.py:75-92) applied to from_fixed(x) as in
 * apply_weights_q15 (:251-254).  x int32 [n] (Q15.16), n % 4 == 0. */
B200_API int b200_static_quant_q15(const int32_t* x, float input_scale, int8_t* codes, int64_t n, b200_stream_t s);

/* ---- W8A8 linear: int8 x int8 -> int32 on the tcgen05 tensor cores, fixed-point requant.
 * Stands in for the GEMM + epilogue inside W8A8Int8LinearMethod.apply_weights_q15
 * (layers/quantization/w8a8_int8.py:242-286), i.e. the sgl_kernel.int8_scaled_mm call at :272-279
 * and the conversions around it; the per-token quant that precedes it is b200_per_token_quant_q15
 * or one of the fused row kernels.
 *   x8 int8 [m, k] (token rows), w8 int8 [n, k] (the checkpoint's [out, in] layout, untransposed);
 *   x_mul, x_shift int32 [m]: fixed-point per-token scale (b200_absmax_to_mul_shift);
 *   w_mul int32 [n], w_shift int32 [n] (nullable = 31 everywhere): per-output-channel scale;
 *   out_q15 int32 [m, n] (nullable): sat32(mul_shift(acc, (x_mul*w_mul)>>32, x_shift+w_shift-48));
 *   acc_out int32 [m, n] (nullable): the exact int32 accumulators.
 * k must be a multiple of 16.  Builds two TMA descriptors on the host per call.  For m <= 256 the
 * weights are streamed once by CTAs that each take a part of K; the parts are added into acc_out (or
 * out_q15 itself) with integer reductions after a memset on the stream, and a second small kernel
 * applies the epilogue - still no allocation and no synchronisation. */
B200_API int b200_gemm_w8a8(const int8_t* x8, const int8_t* w8, const int32_t* x_mul,
                            const int32_t* x_shift, const int32_t* w_mul, const int32_t* w_shift,
                            int32_t* out_q15, int32_t* acc_out, int64_t m, int64_t n, int64_t k,
                            b200_stream_t s);
/* The same with the per-token scale given as the integer absmax that the row kernels emit
 * (x_absmax int32 [m]); (x_mul, x_shift) = b200_absmax_to_mul_shift(x_absmax) are derived inside. */
B200_API int b200_gemm_w8a8_absmax(const int8_t* x8, const int8_t* w8, const int32_t* x_absmax,
                                   const int32_t* w_mul, const int32_t* w_shift, int32_t* out_q15,
                                   int32_t* acc_out, int64_t m, int64_t n, int64_t k, b200_stream_t s);

/* ---- The linear with its requantisation left to the kernel that consumes it ("pending" linear), for decode steps
 * where a launch costs as much as the work in it.  `zero_ws` is an int32 [m, n] workspace that the caller keeps and
 * that is ALL ZERO whenever no call is using it (allocate it zeroed once):
 *   b200_gemm_w8a8_absmax_ws  the linear of b200_gemm_w8a8_absmax; split-K parts are added into zero_ws without a
 *                             clearing launch and the requantising kernel zeroes what it read.  out_q15 != zero_ws.
 *   b200_gemm_w8a8_acc_ws     leaves the exact accumulators in zero_ws; exactly one of the two calls below must then
 *                             consume them (they zero the buffer again) before zero_ws is reused.
 *   b200_rmsnorm_q15_pending  b200_rmsnorm_q15 with x = the Q15.16 result of that linear, computed on the fly from
 *                             (acc, x_absmax int32 [rows], w_mul, w_shift int32 [hidden]): the same bits as
 *                             b200_gemm_w8a8_absmax followed by b200_rmsnorm_q15, in two launches instead of four.
 *   b200_qkv_prepare_pending  b200_qkv_prepare_q15 on the pending qkv linear (acc int32 [tokens, (q_heads + 2 kv_heads)
 *                             * 128], q | k | v heads side by side).
 * No reference counterpart: the reference materialises every linear's output (layers/quantization/w8a8_int8.py:242-286)
 * before RMSNorm (models/integer/qwen3_integer.py:62-80) or q/k-norm + RoPE (models/utils_integer.py:209-227) read it. */
B200_API int b200_gemm_w8a8_absmax_ws(const int8_t* x8, const int8_t* w8, const int32_t* x_absmax, const int32_t* w_mul,
                                      const int32_t* w_shift, int32_t* out_q15, int32_t* zero_ws, int64_t m, int64_t n,
                                      int64_t k, b200_stream_t s);
B200_API int b200_gemm_w8a8_acc_ws(const int8_t* x8, const int8_t* w8, int32_t* zero_ws, int64_t m, int64_t n, int64_t k,
                                   b200_stream_t s);
B200_API int b200_rmsnorm_q15_pending(int32_t* acc, const int32_t* x_absmax, const int32_t* w_mul, const int32_t* w_shift,
                                      const int32_t* residual, const int32_t* weight, int32_t* residual_out,
                                      int32_t* norm_out, int8_t* codes, float* scale, int32_t* absmax, int64_t rows,
                                      int hidden, b200_stream_t s);
B200_API int b200_qkv_prepare_pending(const int32_t* positions, int32_t* acc, const int32_t* x_absmax, const int32_t* w_mul,
                                      const int32_t* w_shift, const int32_t* cos_sin, int max_pos, const int32_t* q_norm_w,
                                      const int32_t* k_norm_w, const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes,
                                      int32_t* meta, int8_t* q8, int32_t* q_mul, int32_t* q_shift, int64_t tokens,
                                      int q_heads, int kv_heads, int64_t num_pages, int with_fwht, b200_stream_t s);

/* ---- gate_up projection with SiLU(gate) * up applied in the GEMM's epilogue (decode batches, m <= 256), and the row
 * kernel that follows it.  Together they replace gate_up_proj + silu_and_mul_int_only + apply_blockwise_fwht_q15 + the
 * per-token quant in front of down_proj (GatedMLPInteger.forward_q15, models/utils_integer.py:99-121) with the same bits:
 *   b200_gemm_gate_up_silu  x8 int8 [m, k], w8 int8 [n2, k] in the checkpoint's merged layout (n2 / 2 gate rows, then
 *                           n2 / 2 up rows; models/weight.py:86-104), x_absmax int32 [m], w_mul / w_shift int32 [n2]
 *                           -> act_out int32 [m, n2 / 2] Q15.16.  zero_ws: an all-zero int32 [m, n2] workspace as for
 *                           b200_gemm_w8a8_absmax_ws (zero again on return).  n2 % 256 == 0, k % 16 == 0.
 *   b200_fwht_quant_q15     act int32 [rows, inter] -> blocked Walsh-Hadamard rotation (fwht_block 128, or 0 = none) ->
 *                           per-token int8 codes [rows, inter], scale fp32 [rows], absmax int32 [rows]: the part of
 *                           b200_silu_mul_q15 behind the activation. */
B200_API int b200_gemm_gate_up_silu(const int8_t* x8, const int8_t* w8, const int32_t* x_absmax, const int32_t* w_mul,
                                    const int32_t* w_shift, int32_t* act_out, int32_t* zero_ws, int64_t m, int64_t n2,
                                    int64_t k, b200_stream_t s);
B200_API int b200_fwht_quant_q15(const int32_t* act, int8_t* codes, float* scale, int32_t* absmax, int64_t rows, int inter,
                                 int fwht_block, b200_stream_t s);

/* ---- Pieces of the W8A8 linear for tensor-parallel row-split layers, where the int32 partial
 * sums of the ranks are added (all-reduce) between the GEMM and its epilogue.  They stand in for
 * the per-rank quant + GEMM + all-reduce of LinearOProj / LinearRowParallel
 * (layers/linear.py:108-160) in a way that gives the same bits as one GPU: quantise every shard
 * with the maximum of the ranks' absmax, add the exact int32 accumulators, requantise once.
 *   b200_quant_given_absmax_q15: x int32 [rows, k], absmax int32 [rows] -> codes int8 [rows, k]
 *   b200_requant_q15: acc int32 [m, n] -> out int32 [m, n] with the epilogue formula of b200_gemm_w8a8
 *                     (w_shift nullable = 31). */
B200_API int b200_quant_given_absmax_q15(const int32_t* x, const int32_t* absmax, int8_t* codes,
                                         int64_t rows, int k, b200_stream_t s);
B200_API int b200_requant_q15(const int32_t* acc, const int32_t* x_mul, const int32_t* x_shift,
                              const int32_t* w_mul, const int32_t* w_shift, int32_t* out,
                              int64_t m, int64_t n, b200_stream_t s);

/* ---- Row-parallel GEMM fused with the tensor-parallel sum over peer memory (decode sizes, m <= 256).
 * Every rank calls it with its K-slice (x8 int8 [m, k_local], w8 int8 [n, k_local]); each accumulator tile is
 * added, as it leaves tensor memory, into peer_acc[0 .. n_peers-1]: the int32 [m, n] accumulators of ALL ranks
 * (this rank's own included), device pointers valid in this process (NVLink peer / symmetric memory).  The
 * transfer overlaps the MMAs tile by tile; integer addition makes the sums identical on every rank.  The caller
 * zeroes the accumulators before any rank starts, separates this call from the reads of the result by a
 * cross-rank barrier on the stream, and applies b200_requant_q15.  peer_acc is a HOST array of n_peers device
 * pointers.  Replaces GEMM + all-reduce of LinearOProj / LinearRowParallel (layers/linear.py:108-160,
 * distributed/impl.py:63-70). */
B200_API int b200_gemm_w8a8_reduce_peers(const int8_t* x8, const int8_t* w8, int32_t* const* peer_acc, int n_peers,
                                         int64_t m, int64_t n, int64_t k, b200_stream_t s);

/* ---- Tensor-parallel exchange over NVLink peer memory without a collective library (decode sizes).
 * They replace, for row-split linears at up to 256 tokens, DistributedCommunicator.all_reduce
 * (distributed/impl.py:63-70) -> TorchDistributedImpl / PyNCCLDistributedImpl (:25-60) ->
 * NCCLWrapper::all_reduce (kernel/csrc/src/pynccl.cu:93-134) as used by LinearOProj / LinearRowParallel
 * (layers/linear.py:108-160), and the all-gather of ParallelLMHead (layers/embedding.py:100-110).
 *
 * Every rank owns one exchange block of b200_tp_block_bytes(m_max, n) bytes of device memory, 256-byte
 * aligned, that is mapped into every rank's process (symmetric / peer memory); base[r] is rank r's block as
 * seen from the calling process, base[rank] the caller's own.  Clear the own block once with
 * b200_tp_block_clear and make sure (host barrier) that every rank has done so before the first exchange.
 * All ranks must issue the same sequence of these calls.  A row-split linear is
 *     b200_tp_absmax_put      the token's absmax over this rank's K-slice, folded into every rank's block
 *     b200_tp_quant_wait      waits for all ranks, quantises the slice with the agreed absmax
 *     b200_gemm_w8a8_tp       this rank's int32 partial sums, accumulated in its own block
 *     b200_tp_requant_scatter waits for all ranks, fetches (16-byte loads over NVLink) and adds every rank's partial
 *                             sums of the rows it owns (rank = row / ceil(m / size)), applies the epilogue of
 *                             b200_gemm_w8a8 and stores the finished rows into every rank's block
 *     b200_tp_collect         waits for all ranks, copies the m finished rows to out_q15 int32 [m, n]
 * With one or two ranks the last three steps are two: b200_tp_requant_direct fetches all rows from every rank (the
 * same bytes at two ranks) and finishes all m rows into out_q15.
 * and gives the bits of b200_gemm_w8a8 on the whole K on one GPU.  b200_tp_all_gather exchanges up to
 * 2 * m_max words per rank (dst int32 [size][words], rank order).  Producer kernels end with a signal,
 * consumer kernels start with a wait that is bounded (default 2 s, b200_tp_set_timeout_us): on expiry the
 * kernel carries on with what the block holds and b200_tp_status reports 1 (absmax exchange), 2 (sums),
 * 3 (gather) or 4 (finished rows).  Kernels only: a step made of these calls can be captured in a CUDA graph.  x: int32 rows with
 * the given pitch (elements); k and n multiples of 4; rows, m <= m_max (and <= 256 for the GEMM). */
typedef struct {
  int rank;        /* this process's rank, 0 .. size-1 */
  int size;        /* ranks, 1 .. 8 */
  int m_max;       /* token rows the block is sized for */
  int64_t n;       /* output channels of the row-split linears (the hidden size) */
  void* base[8];   /* base[r]: rank r's block in this process's address space */
} b200_tp_block;
B200_API size_t b200_tp_block_bytes(int m_max, int64_t n);
B200_API int b200_tp_block_clear(const b200_tp_block* blk, b200_stream_t s);
B200_API int b200_tp_absmax_put(const b200_tp_block* blk, const int32_t* x, int64_t pitch, int rows, int k,
                                b200_stream_t s);
B200_API int b200_tp_quant_wait(const b200_tp_block* blk, const int32_t* x, int64_t pitch, int rows, int k,
                                int8_t* codes, int32_t* absmax_out, b200_stream_t s);
/* b200_tp_absmax_put + b200_tp_quant_wait in one launch (rows <= 512): a row's CTA delivers, waits for the
 * peers' words of the same row and quantises; one kernel less in the step, same words and counters. */
B200_API int b200_tp_absmax_quant(const b200_tp_block* blk, const int32_t* x, int64_t pitch, int rows, int k,
                                  int8_t* codes, int32_t* absmax_out, b200_stream_t s);
B200_API int b200_gemm_w8a8_tp(const b200_tp_block* blk, const int8_t* x8, const int8_t* w8, int64_t m, int64_t n,
                               int64_t k, b200_stream_t s);
B200_API int b200_tp_requant_scatter(const b200_tp_block* blk, const int32_t* absmax, const int32_t* w_mul,
                                     const int32_t* w_shift, int m, b200_stream_t s);
B200_API int b200_tp_collect(const b200_tp_block* blk, int32_t* out_q15, int m, b200_stream_t s);
B200_API int b200_tp_requant_direct(const b200_tp_block* blk, const int32_t* absmax, const int32_t* w_mul,
                                    const int32_t* w_shift, int32_t* out_q15, int m, b200_stream_t s);
/* The row-split linear fused with the (residual add +) RMSNorm + per-token quantisation that follows it in the decoder
 * layer (o_proj -> post_attention_layernorm, down_proj -> the next input_layernorm / the final norm;
 * models/integer/qwen3_integer.py:62-80): after b200_gemm_w8a8_tp the rank that owns a token row (row / ceil(m / size))
 * fetches the row's partial sums from every rank, requantises, adds `residual` (int32 [m, n], updated in place for the
 * OWN rows only; nullable = no add), normalises with norm_weight, quantises, and stores the int8 codes and the absmax
 * of the row into every rank's block.  b200_tp_collect_codes waits for all owners and copies codes int8 [m, n] and
 * absmax int32 [m] out.  Same bits as b200_tp_requant_scatter + b200_tp_collect + b200_rmsnorm_q15 on every rank, with a
 * quarter of the bytes exchanged and the norm computed once per row instead of once per rank.  n % 16 == 0. */
B200_API int b200_tp_owner_norm(const b200_tp_block* blk, const int32_t* x_absmax, const int32_t* w_mul,
                                const int32_t* w_shift, int32_t* residual, const int32_t* norm_weight, int m,
                                b200_stream_t s);
/* SiLU(gate) * up + blocked Walsh-Hadamard rotation of this rank's columns fused with the absmax agreement and the
 * quantisation of b200_tp_absmax_quant: what GatedMLPInteger does between gate_up_proj and down_proj
 * (models/utils_integer.py:99-121) when down_proj is row-split.  gate_up int32 [rows, 2 * inter] (this rank's gate |
 * up columns), codes int8 [rows, inter], absmax int32 [rows] (the agreed value).  rows <= 256, inter % 128 == 0. */
B200_API int b200_tp_silu_absmax_quant(const b200_tp_block* blk, const int32_t* gate_up, int8_t* codes, int32_t* absmax,
                                       int rows, int inter, int fwht_block, b200_stream_t s);
B200_API int b200_tp_collect_codes(const b200_tp_block* blk, int8_t* codes, int32_t* absmax, int m, b200_stream_t s);
B200_API int b200_tp_all_gather(const b200_tp_block* blk, const int32_t* src, int words, int32_t* dst,
                                b200_stream_t s);
B200_API int b200_tp_status(int* out_host, int reset);        /* synchronises with the device */
B200_API int b200_tp_set_timeout_us(int64_t microseconds);    /* synchronises with the device */

/* Reads (and optionally clears) the device-side status word of the GEMM kernels: 0 = fine,
 * non-zero = a bounded wait inside a kernel expired (1 producer, 2 MMA issuer, 3 epilogue).
 * Synchronises with the device.  No counterpart in the reference. */
B200_API int b200_gemm_status(int* out_host, int reset);

#ifdef __cplusplus
}
#endif
#endif /* B200INT_H_ */
