/*
 * CPU oracle for the cuBERT fused non-GEMM layer path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU ("mklBERT", HAVE_MKL) bodies, one
 * function per reference op, each citing the file:line it follows. Arithmetic is
 * float32 with the same operation order as the reference wherever the reference
 * fixes one (one-pass variance, (word+pos)+type, bias first then GEMM accumulate,
 * expf/erff/tanhf/sqrtf from libm). Matrix products use a straightforward loop
 * nest instead of MKL; the summation order inside a dot product therefore differs
 * from MKL's by ordinary float32 rounding.
 *
 * Parity status: PINNED against the reference's own known-answer tests and the
 * reference CPU sources compiled in place (see cubert_oracle.h).
 *
 * The product never calls this file.
 */
#include "cubert_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ gather */

/* src/cuBERT/op/Embedding.cpp:10-20 */
void orc_embedding_i32(const int32_t *ids, int n, const float *table, int width, float *out) {
    for (int i = 0; i < n; ++i) {
        memcpy(out + (size_t) i * width, table + (size_t) width * ids[i], sizeof(float) * width);
    }
}

/* src/cuBERT/op/Embedding.cpp:22-33 */
void orc_embedding_i8(const int8_t *ids, int n, const float *table, int width, float *out) {
    for (int i = 0; i < n; ++i) {
        memcpy(out + (size_t) i * width, table + (size_t) width * ids[i], sizeof(float) * width);
    }
}

/* -------------------------------------------------------------- layer norm */

/* src/cuBERT/op/LayerNorm.cpp:20-41: t = inout + in; one-pass mean / E[t^2];
 * var = 1/sqrtf(var + 1e-12f); out = beta + gamma * var * (t - mean). */
void orc_layer_norm_(const float *in, float *inout, int rows, int channels,
                     const float *beta, const float *gamma) {
#pragma omp parallel for
    for (int r = 0; r < rows; ++r) {
        const float *a = in + (size_t) r * channels;
        float *b = inout + (size_t) r * channels;
        float mean = 0.f;
        float var = 0.f;
        for (int i = 0; i < channels; ++i) {
            float t = b[i] + a[i];
            mean += t;
            var += t * t;
        }
        mean = mean / channels;
        var = var / channels - mean * mean;
        var = 1.f / sqrtf(var + 1e-12f);
        for (int i = 0; i < channels; ++i) {
            b[i] = beta[i] + gamma[i] * var * (b[i] + a[i] - mean);
        }
    }
}

/* -------------------------------------------------------------------- gelu */

/* src/cuBERT/op/GELU.cpp:11-14 */
void orc_gelu(size_t n, float *inout) {
#pragma omp parallel for
    for (long long i = 0; i < (long long) n; ++i) {
        inout[i] = inout[i] * 0.5f * (1.0f + erff(inout[i] * sqrtf(0.5f)));
    }
}

/* ----------------------------------------------------------------- softmax */

/* src/cuBERT/op/Softmax.cpp:18-35 */
void orc_softmax_(const float *in, float *out, int rows, int channel) {
#pragma omp parallel for
    for (int r = 0; r < rows; ++r) {
        const float *x = in + (size_t) r * channel;
        float *y = out + (size_t) r * channel;
        float max = -FLT_MAX;
        for (int i = 0; i < channel; ++i) {
            if (x[i] > max) {
                max = x[i];
            }
        }
        float sum = 0.f;
        for (int i = 0; i < channel; ++i) {
            y[i] = expf(x[i] - max);
            sum += y[i];
        }
        for (int i = 0; i < channel; ++i) {
            y[i] = y[i] / sum;
        }
    }
}

/* -------------------------------------------------------------------- mask */

/* src/cuBERT/op_att/AttentionMask.cpp:14-16 */
void orc_not(const int8_t *in, float *out, int n) {
    for (int i = 0; i < n; ++i) {
        out[i] = !in[i];
    }
}

/* src/cuBERT/op_att/AttentionMask.cpp:41-54: the k=1 strided-batched product
 * neg[b,:] (x) ones[H*S] written as out[b, q, j] = neg[b, j] for q in [0, S*H). */
void orc_attention_mask(const int8_t *mask, int batch, int seq, int heads, float *out) {
    for (int b = 0; b < batch; ++b) {
        for (int q = 0; q < seq * heads; ++q) {
            for (int j = 0; j < seq; ++j) {
                out[((size_t) b * seq * heads + q) * seq + j] = !mask[b * seq + j];
            }
        }
    }
}

/* src/cuBERT/op_att/AttentionSelf.cpp:58-60 (alpha = 1/sqrt(d), beta = -10000),
 * :99-101 (scores preloaded with the broadcast neg mask), op_att/BatchMatMul.cpp:57-68
 * (scores = alpha * K.Q^T + beta * scores), then op/Softmax.cpp:18-35 on every row.
 * Row r of the [B, S, H, S] tensor belongs to batch r / (S*H); the mask indexes the
 * key (last) axis. */
void orc_masked_softmax(const float *scores, const int8_t *mask, int batch, int heads, int seq,
                        float scale, float *out) {
    const long long rows = (long long) batch * seq * heads;
#pragma omp parallel for
    for (long long r = 0; r < rows; ++r) {
        const int b = (int) (r / ((long long) seq * heads));
        const float *x = scores + (size_t) r * seq;
        float *y = out + (size_t) r * seq;
        float max = -FLT_MAX;
        for (int j = 0; j < seq; ++j) {
            float neg = mask ? (float) (!mask[b * seq + j]) : 0.f;
            y[j] = scale * x[j] + -10000.0f * neg;
            if (y[j] > max) {
                max = y[j];
            }
        }
        float sum = 0.f;
        for (int j = 0; j < seq; ++j) {
            y[j] = expf(y[j] - max);
            sum += y[j];
        }
        for (int j = 0; j < seq; ++j) {
            y[j] = y[j] / sum;
        }
    }
}

/* ------------------------------------------------------------------ pooler */

/* src/cuBERT/op_bert/BertPooler.cpp:10-15 */
void orc_tanh_(float *inout, int n) {
    for (int i = 0; i < n; ++i) {
        inout[i] = tanhf(inout[i]);
    }
}

/* src/cuBERT/op_bert/BertPooler.cpp:21-31: sequential sum over seq, then / seq */
void orc_reduce_mean_1(const float *in, float *out, int batch, int seq, int hidden) {
#pragma omp parallel for
    for (int idx = 0; idx < batch * hidden; ++idx) {
        size_t b = idx / hidden;
        size_t c = idx % hidden;
        float sum = 0.f;
        for (int s = 0; s < seq; ++s) {
            sum += in[c + (size_t) s * hidden + b * seq * hidden];
        }
        out[idx] = sum / seq;
    }
}

/* ------------------------------------------------------------------- dense */

/* One row block of Y += X.W with W row-major [inputs, units]; vectorises over units. */
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
__attribute__((target_clones("avx512f", "avx2", "default")))
#endif
static void gemm_rows(const float *x, const float *w, float *y, int rows, int inputs, int units,
                      size_t ldx, size_t ldw, size_t ldy) {
    for (int r = 0; r < rows; ++r) {
        const float *xr = x + (size_t) r * ldx;
        float *yr = y + (size_t) r * ldy;
        for (int k = 0; k < inputs; ++k) {
            const float a = xr[k];
            const float *wk = w + (size_t) k * ldw;
            for (int j = 0; j < units; ++j) {
                yr[j] += a * wk[j];
            }
        }
    }
}

/* src/cuBERT/op/Dense.cpp:41-57: output preloaded with the broadcast bias
 * (_pre_compute), then the GEMM accumulates onto it with beta = 1 (_in_compute). */
void orc_dense(const float *x, const float *w, const float *bias, int rows, int inputs, int units,
               float *y) {
#pragma omp parallel for schedule(static)
    for (int r0 = 0; r0 < rows; r0 += 8) {
        int nr = rows - r0 < 8 ? rows - r0 : 8;
        for (int r = r0; r < r0 + nr; ++r) {
            for (int j = 0; j < units; ++j) {
                y[(size_t) r * units + j] = bias ? bias[j] : 0.f;
            }
        }
        gemm_rows(x + (size_t) r0 * inputs, w, y + (size_t) r0 * units, nr, inputs, units,
                  inputs, units, units);
    }
}

/* -------------------------------------------------------------- embeddings */

/* src/cuBERT/op_bert/BertEmbeddings.cpp:53-65: word rows gathered into out, type rows
 * gathered into a side buffer, positions added onto out by a rank-1 product with
 * beta = 1, then LayerNorm(in = type rows, inout = out) -- i.e. t = (word+pos)+type. */
void orc_bert_embeddings(const int32_t *ids, const int8_t *segment_ids, int batch, int seq, int hidden,
                         const float *word, const float *pos, const float *type,
                         const float *beta, const float *gamma, float *out) {
    const int n = batch * seq;
    float *type_rows = (float *) malloc(sizeof(float) * (size_t) n * hidden);
    orc_embedding_i32(ids, n, word, hidden, out);
    orc_embedding_i8(segment_ids, n, type, hidden, type_rows);
    for (int b = 0; b < batch; ++b) {
        for (int i = 0; i < seq * hidden; ++i) {
            out[(size_t) b * seq * hidden + i] += pos[i];
        }
    }
    orc_layer_norm_(type_rows, out, n, hidden, beta, gamma);
    free(type_rows);
}

/* src/cuBERT/op_bert/BertPooler.cpp:62-77: out = bias; out += first_token . kernel
 * (ldb = hidden*seq picks token 0 of each sequence); tanh in place. */
void orc_bert_pooler(const float *seq_out, int batch, int seq, int hidden,
                     const float *kernel, const float *bias, float *out) {
    for (int b = 0; b < batch; ++b) {
        float *y = out + (size_t) b * hidden;
        for (int j = 0; j < hidden; ++j) {
            y[j] = bias[j];
        }
        gemm_rows(seq_out + (size_t) b * seq * hidden, kernel, y, 1, hidden, hidden,
                  hidden, hidden, hidden);
    }
    orc_tanh_(out, batch * hidden);
}

/* src/cuBERT/op_out/AdditionalOutputLayer.cpp:44-66: logits preloaded with the bias
 * (or beta = 0 without one), logits += pooled . W^T with W [labels, hidden]; probs =
 * softmax over labels. */
void orc_classifier(const float *pooled, int batch, int hidden, int labels,
                    const float *w, const float *bias, float *logits, float *probs) {
    for (int b = 0; b < batch; ++b) {
        for (int l = 0; l < labels; ++l) {
            float acc = 0.f;
            for (int c = 0; c < hidden; ++c) {
                acc += w[(size_t) l * hidden + c] * pooled[(size_t) b * hidden + c];
            }
            logits[b * labels + l] = bias ? bias[l] + acc : acc;
        }
    }
    if (probs) {
        orc_softmax_(logits, probs, batch, labels);
    }
}

/* ------------------------------------------------------------- transformer */

/* Scores and context of one layer. Layouts follow op_att/BatchMatMul.h:10-14 and
 * op_att/BatchMatMul.cpp:33-37,57-68,100-104,124-135:
 *   q,k,v   [B, S, H, d]
 *   scores  [B, S_from, H, S_to]   (pointer for (b,h) = base + b*S*S*H + S*h, ld = S*H)
 *   context [B, S, H, d] */
void orc_att_q_k(const float *q, const float *k, int batch, int seq, int heads, int d,
                 float *scores) {
    const int hidden = heads * d;
#pragma omp parallel for collapse(2)
    for (int b = 0; b < batch; ++b) {
        for (int i = 0; i < seq; ++i) {
            for (int h = 0; h < heads; ++h) {
                const float *qi = q + ((size_t) (b * seq + i) * hidden) + h * d;
                float *row = scores + (((size_t) b * seq + i) * heads + h) * seq;
                for (int j = 0; j < seq; ++j) {
                    const float *kj = k + ((size_t) (b * seq + j) * hidden) + h * d;
                    float acc = 0.f;
                    for (int c = 0; c < d; ++c) {
                        acc += kj[c] * qi[c];
                    }
                    row[j] = acc;
                }
            }
        }
    }
}

void orc_att_qk_v(const float *probs, const float *v, int batch, int seq, int heads, int d,
                  float *ctx) {
    const int hidden = heads * d;
#pragma omp parallel for collapse(2)
    for (int b = 0; b < batch; ++b) {
        for (int i = 0; i < seq; ++i) {
            for (int h = 0; h < heads; ++h) {
                const float *row = probs + (((size_t) b * seq + i) * heads + h) * seq;
                float *out = ctx + ((size_t) (b * seq + i) * hidden) + h * d;
                for (int c = 0; c < d; ++c) {
                    out[c] = 0.f;
                }
                for (int j = 0; j < seq; ++j) {
                    const float *vj = v + ((size_t) (b * seq + j) * hidden) + h * d;
                    const float p = row[j];
                    for (int c = 0; c < d; ++c) {
                        out[c] += vj[c] * p;
                    }
                }
            }
        }
    }
}

/* src/cuBERT/op_att/AttentionSelf.cpp:96-111 with the reference's own operand: a
 * pre-broadcast float "neg mask" tensor [B, S*H, S] (1 = masked), as its unit test
 * passes it (test/cuBERT/op_att/AttentionSelfTest.cpp:55-57). */
void orc_attention_self(const float *x, const float *const *qkv /* q_k,q_b,k_k,k_b,v_k,v_b */,
                        int batch, int seq, int heads, int d, const float *neg_mask, float *ctx) {
    const int H = heads * d, rows = batch * seq;
    const float scale = (float) (1.0 / sqrt((double) d));
    float *q = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *k = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *v = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *scores = (float *) malloc(sizeof(float) * (size_t) batch * heads * seq * seq);
    orc_dense(x, qkv[0], qkv[1], rows, H, H, q);
    orc_dense(x, qkv[2], qkv[3], rows, H, H, k);
    orc_dense(x, qkv[4], qkv[5], rows, H, H, v);
    orc_att_q_k(q, k, batch, seq, heads, d, scores);
    for (size_t i = 0; i < (size_t) batch * heads * seq * seq; ++i) {
        scores[i] = scale * scores[i] + -10000.0f * neg_mask[i];
    }
    orc_softmax_(scores, scores, batch * heads * seq, seq);
    orc_att_qk_v(scores, v, batch, seq, heads, d, ctx);
    free(scores);
    free(v);
    free(k);
    free(q);
}

/* src/cuBERT/op_att/Transformer.cpp:145-175 with op_att/AttentionSelf.cpp:96-111 inlined. */
void orc_transformer(const orc_bert_weights *w, int batch, float *x, const int8_t *mask) {
    const int S = w->seq, H = w->hidden, I = w->intermediate, heads = w->heads;
    const int d = H / heads;
    const int rows = batch * S;
    const float scale = (float) (1.0 / sqrt((double) d)); /* op_att/AttentionSelf.cpp:58-60 */

    float *q = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *k = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *v = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *ctx = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *att = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *inter = (float *) malloc(sizeof(float) * (size_t) rows * I);
    float *out = (float *) malloc(sizeof(float) * (size_t) rows * H);
    float *scores = (float *) malloc(sizeof(float) * (size_t) batch * heads * S * S);

    for (int l = 0; l < w->layers; ++l) {
        const float *const *t = w->layer_tensors + (size_t) l * ORC_TENSORS_PER_LAYER;

        orc_dense(x, t[ORC_Q_KERNEL], t[ORC_Q_BIAS], rows, H, H, q);
        orc_dense(x, t[ORC_K_KERNEL], t[ORC_K_BIAS], rows, H, H, k);
        orc_dense(x, t[ORC_V_KERNEL], t[ORC_V_BIAS], rows, H, H, v);

        orc_att_q_k(q, k, batch, S, heads, d, scores);
        orc_masked_softmax(scores, mask, batch, heads, S, scale, scores);
        orc_att_qk_v(scores, v, batch, S, heads, d, ctx);

        /* attention/output: dense, then LayerNorm(in = layer input, inout = dense out) */
        orc_dense(ctx, t[ORC_ATT_OUT_KERNEL], t[ORC_ATT_OUT_BIAS], rows, H, H, att);
        orc_layer_norm_(x, att, rows, H, t[ORC_ATT_LN_BETA], t[ORC_ATT_LN_GAMMA]);

        /* intermediate: dense + gelu */
        orc_dense(att, t[ORC_INTER_KERNEL], t[ORC_INTER_BIAS], rows, H, I, inter);
        orc_gelu((size_t) rows * I, inter);

        /* output: dense, then LayerNorm(in = attention output, inout = dense out) */
        orc_dense(inter, t[ORC_OUT_KERNEL], t[ORC_OUT_BIAS], rows, I, H, out);
        orc_layer_norm_(att, out, rows, H, t[ORC_OUT_LN_BETA], t[ORC_OUT_LN_GAMMA]);

        memcpy(x, out, sizeof(float) * (size_t) rows * H);
    }

    free(scores);
    free(out);
    free(inter);
    free(att);
    free(ctx);
    free(v);
    free(k);
    free(q);
}

/* ------------------------------------------------------------- whole model */

/* src/cuBERT/Bert.cpp:99-136 */
void orc_bert_forward(const orc_bert_weights *w, int batch,
                      const int32_t *ids, const int8_t *mask, const int8_t *segment_ids,
                      float *embedding_output, float *sequence_output, float *pooled_output,
                      float *logits, float *probs) {
    if (batch == 0) { /* src/cuBERT/Bert.cpp:102-103 */
        return;
    }
    const int S = w->seq, H = w->hidden;
    const size_t n = (size_t) batch * S * H;
    float *x = (float *) malloc(sizeof(float) * n);
    float *pooled = (float *) malloc(sizeof(float) * (size_t) batch * H);

    orc_bert_embeddings(ids, segment_ids, batch, S, H, w->word_emb, w->pos_emb, w->type_emb,
                        w->emb_ln_beta, w->emb_ln_gamma, x);
    if (embedding_output) {
        memcpy(embedding_output, x, sizeof(float) * n);
    }

    orc_transformer(w, batch, x, mask);
    if (sequence_output) {
        memcpy(sequence_output, x, sizeof(float) * n);
    }

    if (w->pooler_kernel) {
        orc_bert_pooler(x, batch, S, H, w->pooler_kernel, w->pooler_bias, pooled);
    } else {
        orc_reduce_mean_1(x, pooled, batch, S, H);
    }
    if (pooled_output) {
        memcpy(pooled_output, pooled, sizeof(float) * (size_t) batch * H);
    }

    if (w->output_weights && (logits || probs)) {
        float *lg = logits ? logits : (float *) malloc(sizeof(float) * (size_t) batch * w->num_labels);
        orc_classifier(pooled, batch, H, w->num_labels, w->output_weights, w->output_bias, lg, probs);
        if (!logits) {
            free(lg);
        }
    }

    free(pooled);
    free(x);
}
