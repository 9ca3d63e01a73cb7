/*
 * cubert_kernels.h -- C ABI of the fused non-GEMM BERT layer kernels for NVIDIA B200 (sm_100a).
 *
 * This is the launch layer that sits below cuBERT's host code. Every entry point takes
 * plain device pointers and sizes plus a CUDA stream, enqueues its kernel(s) on that
 * stream and returns immediately with a status: 0 on success, a negative CUBK_ERR_* code
 * otherwise. Nothing here allocates, synchronises, exits the process or traps on the
 * device. There is no CPU fallback: without a CUDA device every call fails.
 *
 * Each function names the reference operator interface it replaces (path:line inside the
 * zhihu/cuBERT source tree). The reference's operators are `void`, unchecked and one
 * kernel per elementary step; the functions below fuse the steps the reference spreads
 * over several kernels, GEMM alpha/beta tricks and device-to-device copies.
 *
 * Conventions
 *   - `_f32` entry points work on float storage, `_f16` on IEEE binary16 storage
 *     (`__half`); arithmetic is float32 in both.
 *   - Row-major tensors; rows are contiguous. Element counts are 64-bit safe
 *     (rows * channels may exceed 2^31).
 *   - A fast path is taken when pointers are 16-byte aligned and the row length is a
 *     multiple of 16 bytes; any other shape or alignment runs a slower generic kernel
 *     with identical results.
 *   - `stream` is a `cudaStream_t` passed as `void *` (as the reference does).
 */
#ifndef CUBERT_KERNELS_H
#define CUBERT_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CUBK_OK                 0
#define CUBK_ERR_INVALID_ARG   -1   /* null pointer, non-positive size, bad enum */
#define CUBK_ERR_UNSUPPORTED   -2   /* shape outside what the kernel family handles */
#define CUBK_ERR_LAUNCH        -3   /* the CUDA runtime refused the launch (see cubk_last_cuda_error) */
#define CUBK_ERR_SCRATCH       -4   /* scratch buffer missing or too small */

/* Bits OR-ed into the device status word of cubk_embed_* when an index is out of range.
 * The offending index is clamped into range so that no out-of-bounds read happens. */
#define CUBK_STATUS_BAD_TOKEN_ID   1u
#define CUBK_STATUS_BAD_SEGMENT_ID 2u
/* A wait for an asynchronous shared-memory copy inside cubk_embed_ln_* ran out of polls; the rows of
 * the affected warp from that point on were not written. Not expected in normal operation. */
#define CUBK_STATUS_COPY_TIMEOUT   4u

/* Library version and the text of the last CUDA error seen by a failed launch (thread-local). */
int cubk_version(void);
const char *cubk_last_cuda_error(void);

/* Process-wide tuning switches. Each starts from an environment variable (read once, when the library
 * first needs any switch) and can be changed at run time; a change applies to launches made after it.
 * They select between kernels that compute the same result, so they matter to benchmarks and tests only.
 * No counterpart in the reference.
 *   CUBK_OPT_EMBED_STAGED_ROWS  (env CUBK_BULK_COPY)          -1 = by shape (default), 0 = never, 1 = whenever it
 *                               fits: cubk_embed_ln_* fetches the gathered word rows into shared memory with
 *                               asynchronous bulk copies instead of register loads
 *   CUBK_OPT_SOFTMAX_MASK_SMEM  (env CUBK_SOFTMAX_MASK_SMEM)  1 (default) = long rows of cubk_masked_softmax_* keep
 *                               their additive mask terms in shared memory, 0 = in registers
 *   CUBK_OPT_EXACT_WIDTH_ROWS   (env CUBK_EXACT_WIDTH_ROWS)   1 (default) = cubk_bias_residual_ln_* uses the kernel
 *                               specialised for rows of exactly 32, 64, 96, 128, 192 or 256 16-byte vectors when
 *                               the shape allows, 0 = always the general kernel
 *   CUBK_OPT_EXACT_WIDTH_EMBED  (env CUBK_EXACT_WIDTH_EMBED)  the same for cubk_embed_ln_*
 *   CUBK_OPT_ATTENTION_TENSOR_MEMORY (env CUBK_ATTENTION_TENSOR_MEMORY)  1 = cubk_attention_small_f16 of 65 to 128
 *                               positions runs on tcgen05 with accumulators in tensor memory, 0 = on warp-level
 *                               matrix instructions
 * Both return CUBK_ERR_INVALID_ARG for an unknown switch or a value outside its range. */
#define CUBK_OPT_EMBED_STAGED_ROWS 0
#define CUBK_OPT_SOFTMAX_MASK_SMEM 1
#define CUBK_OPT_EXACT_WIDTH_ROWS  2
#define CUBK_OPT_EXACT_WIDTH_EMBED 3
#define CUBK_OPT_ATTENTION_TENSOR_MEMORY 4
#define CUBK_OPT_COUNT             5
int cubk_set_option(int option, int value);
int cubk_get_option(int option, int *value);

/* Warps, on the current device and since the library was loaded, that gave up waiting for one of the
 * asynchronous global-to-shared copies the staged variant of cubk_embed_ln_* fetches its word rows
 * with. Every such wait is bounded; a warp that gives up stops writing rows. Expected to
 * stay 0. Synchronises with the device. No counterpart in the reference. */
int cubk_copy_timeouts(unsigned int *count);

/* Exercises the give-up path of those bounded waits without any copy: one warp polls, at most `polls` times
 * (1..100000), a barrier that nothing completes, then ORs CUBK_STATUS_COPY_TIMEOUT into *status (device word,
 * may be NULL) and counts in cubk_copy_timeouts. The kernel always returns; the context stays usable.
 * For tests. No counterpart in the reference. */
int cubk_selftest_copy_wait_timeout(unsigned int polls, uint32_t *status, void *stream);

/* ---- K1: embedding lookup + position/token-type add + LayerNorm --------------------------
 * out[b,s,:] = LayerNorm((word[ids[b,s]] + pos[s]) + type[segment_ids[b,s]]; gamma, beta)
 * Replaces BertEmbeddings<T>::compute (src/cuBERT/op_bert/BertEmbeddings.cpp:50-66), i.e.
 * two embedding<T,V> gathers (op/Embedding.h:10), a rank-1 GEMM and layer_norm_<T>.
 * ids int32 [batch*seq], segment_ids int8 [batch*seq], word [vocab,hidden],
 * pos [>=seq,hidden], type [type_vocab,hidden], gamma/beta [hidden], out [batch*seq,hidden].
 * status: optional device uint32 word (may be NULL) that receives CUBK_STATUS_* bits. */
int cubk_embed_ln_f32(const int32_t *ids, const int8_t *segment_ids,
                      const float *word, const float *pos, const float *type,
                      const float *gamma, const float *beta,
                      int batch, int seq, int hidden, int vocab, int type_vocab,
                      float *out, uint32_t *status, void *stream);
int cubk_embed_ln_f16(const int32_t *ids, const int8_t *segment_ids,
                      const void *word, const void *pos, const void *type,
                      const void *gamma, const void *beta,
                      int batch, int seq, int hidden, int vocab, int type_vocab,
                      void *out, uint32_t *status, void *stream);

/* Plain row gather out[i,:] = table[ids[i],:], bit-exact copy.
 * Replaces embedding<int,V> / embedding<int8_t,V> (src/cuBERT/op/Embedding.h:10-15,
 * op/Embedding.cu:8-41). elem_bytes is 4 (float) or 2 (half). */
int cubk_embed_gather_i32(const int32_t *ids, int64_t n, const void *table, int vocab, int width,
                          int elem_bytes, void *out, uint32_t *status, void *stream);
int cubk_embed_gather_i8(const int8_t *ids, int64_t n, const void *table, int vocab, int width,
                         int elem_bytes, void *out, uint32_t *status, void *stream);

/* Row scatter out[idx[i],:] = in[i,:], bit-exact; the inverse of cubk_embed_gather_i32 (which doubles as
 * the general row gather out[i,:] = in[idx[i],:]). No counterpart in the reference: the pair moves
 * activations between the [batch*seq, width] layout and a packed list of the non-padding tokens, so that
 * the token-wise GEMMs and kernels can skip padding. in [n, width], out [rows_out, width]; rows of out
 * that no index names keep their contents; out-of-range indices are skipped; duplicate indices must
 * carry identical rows. elem_bytes is 4 or 2. */
int cubk_scatter_rows(const int32_t *idx, int64_t n, const void *in, int width, int elem_bytes, void *out,
                      int rows_out, void *stream);

/* ---- K2: bias + residual + LayerNorm -------------------------------------------------------
 * t = x (+ bias) (+ residual);  out = beta + gamma * (t - mean(t)) / sqrt(var(t) + 1e-12)
 * Replaces layer_norm_<T> (src/cuBERT/op/LayerNorm.h:6-15, op/LayerNorm.cu:11-100) together
 * with the Dense bias prefill it depends on (op/Dense.cpp:41-45). x, residual, out
 * [rows, channels]; bias, gamma, beta [channels]. bias and residual may be NULL. out may
 * alias x (the reference's in-place form: x = inout, residual = in). */
int cubk_bias_residual_ln_f32(const float *x, const float *bias, const float *residual,
                              const float *gamma, const float *beta,
                              int64_t rows, int channels, float *out, void *stream);
int cubk_bias_residual_ln_f16(const void *x, const void *bias, const void *residual,
                              const void *gamma, const void *beta,
                              int64_t rows, int channels, void *out, void *stream);

/* ---- K3: bias + GELU ------------------------------------------------------------------------
 * y = x (+ bias);  out = y * 0.5 * (1 + erf(y / sqrt(2)))
 * Replaces gelu<T> (src/cuBERT/op/GELU.h:7, op/GELU.cu:14-26) plus the Dense bias prefill.
 * x, out [rows, channels] (out may alias x); bias [channels] or NULL. */
int cubk_bias_gelu_f32(const float *x, const float *bias, int64_t rows, int channels,
                       float *out, void *stream);
int cubk_bias_gelu_f16(const void *x, const void *bias, int64_t rows, int channels,
                       void *out, void *stream);

/* ---- K4: masked scaled softmax ----------------------------------------------------------------
 * For row r of a [rows, seq] score matrix, with b = r / rows_per_batch:
 *   v[j] = scale * scores[r,j] + (mask && mask[b*seq + j] == 0 ? -10000 : 0)
 *   out[r,:] = softmax(v)
 * Replaces softmax_<T> (src/cuBERT/op/Softmax.h:9-14, op/Softmax.cu:17-115), _not<T> and the
 * mask broadcast (op_att/AttentionMask.h:9, op_att/AttentionMask.cpp:41-54), the per-layer
 * device copy of the broadcast mask and the GEMM's beta = -10000 accumulate
 * (op_att/AttentionSelf.cpp:58-60,99-101). For cuBERT's attention scores [B, S, heads, S]
 * pass rows = B*S*heads and rows_per_batch = S*heads. mask is int8 [rows/rows_per_batch, seq]
 * over the key axis, or NULL. out may alias scores. */
int cubk_masked_softmax_f32(const float *scores, const int8_t *mask, int64_t rows, int64_t rows_per_batch,
                            int seq, float scale, float *out, void *stream);
int cubk_masked_softmax_f16(const void *scores, const int8_t *mask, int64_t rows, int64_t rows_per_batch,
                            int seq, float scale, void *out, void *stream);

/* K4 for callers that know, per batch entry, where the kept keys end. key_extents is a device array of
 * int32, one per batch entry: n = key_extents[b] (clamped to 1..seq) promises that mask[b*seq + j] == 0 for
 * every j >= n and that some key below n is kept. Columns at or beyond n (rounded up to a whole 16-byte
 * vector) are then not read; their probabilities are exactly 0, as in the full computation. Of those columns,
 * the ones below zero_to are written as zeros, the rest are left untouched, so a consumer that multiplies
 * only the first n columns of entry b (a batched product with k = n) can pass zero_to = 0, and one that reads
 * a common extent E >= n passes zero_to = E; zero_to = seq gives the output of cubk_masked_softmax_*.
 * mask must not be NULL. Moves n / seq of the bytes of the plain call. The reference has no counterpart: it
 * computes, masks, exponentiates and multiplies every padded key (src/cuBERT/op_att/AttentionSelf.cpp:96-111,
 * op_att/BatchMatMul.cpp:57-68,124-135).
 * Where the two calls differ: a masked key whose scaled score exceeds the largest kept score of its row by
 * about 9900 or more would get a non-zero probability from the plain call and gets 0 here. */
int cubk_masked_softmax_extents_f32(const float *scores, const int8_t *mask, const int32_t *key_extents,
                                    int zero_to, int64_t rows, int64_t rows_per_batch, int seq, float scale,
                                    float *out, void *stream);
int cubk_masked_softmax_extents_f16(const void *scores, const int8_t *mask, const int32_t *key_extents,
                                    int zero_to, int64_t rows, int64_t rows_per_batch, int seq, float scale,
                                    void *out, void *stream);

/* Whole attention of short sequences in one launch: for every (sequence, head)
 *   scores = scale * Q.K^T, rounded to the storage type;  P = masked softmax(scores) as cubk_masked_softmax_*,
 *   rounded to the storage type;  context = P.V
 * i.e. what the reference's Att_Q_K product, mask, softmax and Att_QK_V product compute
 * (src/cuBERT/op_att/AttentionSelf.cpp:96-111, op_att/BatchMatMul.cpp:57-68,124-135, op/Softmax.cpp:19-35), rounding
 * where those round: one launch in place of two batched library products and K4, and the [seq, seq] scores
 * never reach device memory.
 * qkv [batch * seq, 3 * hidden] holds per token Q | K | V (head h at columns 64 * h of each part); mask int8
 * [batch, seq] over the keys or NULL; context [batch * seq, hidden]. hidden must be 64 * heads.
 *   _f16, seq <= 128, qkv and context on 16-byte boundaries: warp-level matrix instructions
 *     (binary16 operands, float32 accumulators), a block per (sequence, head), a strip of 16 query rows per warp
 *     kept in registers from the scores to the context. Past 64 positions the kernel finds each sequence's last
 *     kept key and neither loads nor multiplies the keys behind it (their probabilities are exactly 0; where
 *     that differs from the full computation is stated at cubk_masked_softmax_extents_*). Moves Q | K | V once
 *     and the context once: 4 * batch * seq * hidden elements. With CUBK_OPT_ATTENTION_TENSOR_MEMORY set, 65 to
 *     128 positions run on tcgen05 instead: one 128-row tile per (sequence, head), accumulators in tensor
 *     memory, a score row per thread; every wait on its MMA barrier is bounded (0.2 s), after which the block
 *     writes NaN rows, frees its tensor memory and returns.
 *   _f32 (and _f16 at other addresses), seq <= 64: the float32 pipes; pays for requests of a few hundred
 *     tokens, where a forward pass is bound by its chain of launches rather than by work.
 * Anything else: CUBK_ERR_UNSUPPORTED. */
int cubk_attention_small_f32(const float *qkv, const int8_t *mask, int batch, int seq, int heads, int hidden,
                             float scale, float *context, void *stream);
int cubk_attention_small_f16(const void *qkv, const int8_t *mask, int batch, int seq, int heads, int hidden,
                             float scale, void *context, void *stream);

/* ---- K5a: bias + tanh (BERT pooler activation) ---------------------------------------------------
 * out = tanh(x (+ bias)). Replaces tanh_<T> (src/cuBERT/op_bert/BertPooler.h:9,
 * op_bert/BertPooler.cu:14-26) plus the bias prefill of BertPooler<T>::compute
 * (op_bert/BertPooler.cpp:62-77). x, out [rows, channels]; out may alias x. */
int cubk_bias_tanh_f32(const float *x, const float *bias, int64_t rows, int channels,
                       float *out, void *stream);
int cubk_bias_tanh_f16(const void *x, const void *bias, int64_t rows, int channels,
                       void *out, void *stream);

/* ---- K5b: mean pooling over the sequence axis ---------------------------------------------------
 * out[b,c] = (sum_s x[b,s,c]) / seq   (every position counts; the mask is ignored)
 * Replaces reduce_mean_1<T> (src/cuBERT/op_bert/BertPooler.h:14-16, op_bert/BertPooler.cu:35-66).
 * When batch is small the sequence axis is split over several thread blocks: their float32 partial sums and
 * one arrival counter per (sequence, block of 256 columns) go through `scratch` (device memory, 16-byte
 * aligned, at least cubk_mean_pool_scratch_bytes(batch, seq, hidden) bytes; may be NULL when that is 0).
 * The call clears the counters itself (an asynchronous memset on `stream`); the contents of scratch before
 * and after a call mean nothing. The block that arrives last adds the slices in slice order, so the result
 * is the same from run to run. */
size_t cubk_mean_pool_scratch_bytes(int batch, int seq, int hidden);
int cubk_mean_pool_f32(const float *x, int batch, int seq, int hidden, float *out,
                       void *scratch, size_t scratch_bytes, void *stream);
int cubk_mean_pool_f16(const void *x, int batch, int seq, int hidden, void *out,
                       void *scratch, size_t scratch_bytes, void *stream);

/* Mean pooling for callers that must not allocate device memory. No counterpart in the reference.
 * Same result as cubk_mean_pool_f32 / _f16 (elem_bytes 4 / 2), but the float32 partial sums of the
 * split-sequence path live in a 512 KiB array built into the library (reserved on every GPU that loads
 * it, until the process exits) instead of a caller-provided scratch buffer, and the call performs no
 * cudaMalloc, cudaFree or other allocating call. For hosts where allocation is off limits on the
 * calling path: latency-critical serving loops that ban calls which can take the driver's allocation
 * lock, plug-ins whose host process owns all device memory, sandboxes that filter allocator calls.
 *   - Shapes whose partial sums exceed the array (more than CUBK_STATIC_POOL_SCRATCH_BYTES; e.g.
 *     binary16 [9, 512, 4096] needs 720 KiB) are refused with CUBK_ERR_SCRATCH before anything runs.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call outside any stream capture.
 *   - All calls on a device share the one array. It keeps whatever the previous call left: every partial
 *     sum is written before it is read, and the arrival counters, the one part that must start at zero,
 *     are cleared by each call before its kernel runs (an asynchronous memset on `stream`).
 *     Two calls whose kernels can overlap on the GPU (different streams, no ordering between them)
 *     race on it: order them on one stream or with events. */
#define CUBK_STATIC_POOL_SCRATCH_BYTES (512u * 1024u)
int cubk_mean_pool_static_scratch(const void *x, int elem_bytes, int batch, int seq, int hidden, void *out,
                                  void *stream);

/* ---- K5c: classifier head ---------------------------------------------------------------------
 * logits[b,l] = sum_c pooled[b,c] * weights[l,c] (+ bias[l]);  probs[b,:] = softmax(logits[b,:])
 * Replaces ClassifierOutputLayer<T>::_pre_compute/_in_compute
 * (src/cuBERT/op_out/AdditionalOutputLayer.cpp:44-66): bias copy, an n = num_labels GEMM and
 * the five softmax launches. weights [labels, hidden]; bias [labels] or NULL; probs may be
 * NULL. labels <= 4096. */
int cubk_logits_probs_f32(const float *pooled, const float *weights, const float *bias,
                          int batch, int hidden, int labels, float *logits, float *probs, void *stream);
int cubk_logits_probs_f16(const void *pooled, const void *weights, const void *bias,
                          int batch, int hidden, int labels, void *logits, void *probs, void *stream);

/* ---- K5a + K5c in one launch ----------------------------------------------------------------------
 * pooled = tanh(x + pooler_bias);  logits = pooled * weights^T (+ bias);  probs = softmax(logits)
 * The same results as cubk_bias_tanh_* followed by cubk_logits_probs_* on its output (the classifier reads
 * the pooled row in storage precision, the softmax the stored logits), for classification heads of up to
 * 8 labels: replaces tanh_<T> and the pooler bias (src/cuBERT/op_bert/BertPooler.cpp:62-77) together with
 * ClassifierOutputLayer (src/cuBERT/op_out/AdditionalOutputLayer.cpp:44-66). x [batch, hidden] is the pooler's
 * dense product; pooled may alias x; bias and probs may be NULL. Returns CUBK_ERR_UNSUPPORTED, having done
 * nothing, for more than 8 labels, rows that are not whole aligned 16-byte vectors or hidden above 4096
 * (binary16) / 2048 (float32): callers then use the two separate calls. */
int cubk_pooler_head_f32(const float *x, const float *pooler_bias, const float *weights, const float *bias,
                         int batch, int hidden, int labels, float *pooled, float *logits, float *probs,
                         void *stream);
int cubk_pooler_head_f16(const void *x, const void *pooler_bias, const void *weights, const void *bias,
                         int batch, int hidden, int labels, void *pooled, void *logits, void *probs,
                         void *stream);

/* ---- helpers ------------------------------------------------------------------------------------
 * out[i] = !in[i] as 0/1 in the storage type. Replaces _not<T> (src/cuBERT/op_att/AttentionMask.h:9). */
int cubk_not_f32(const int8_t *in, float *out, int64_t n, void *stream);
int cubk_not_f16(const int8_t *in, void *out, int64_t n, void *stream);

/* binary16 -> float32 on the device. Replaces the host loop half2float
 * (src/cuBERT/common.h:101-106) used by Bert<half>::output_to_float (src/cuBERT/Bert.cpp:218-259). */
int cubk_half_to_float(const void *in, float *out, int64_t n, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CUBERT_KERNELS_H */
