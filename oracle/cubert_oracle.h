/*
 * CPU oracle for the cuBERT fused non-GEMM layer path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * CPU ("mklBERT") algorithm for every op on the path; it exists to check the
 * CUDA kernels and to serve as a timed CPU baseline. Nothing in the product
 * (the kernel library, the host library) may link, load or call it.
 *
 * Parity status: PINNED. Every function below is checked (tests/test_oracle_*.py)
 * against the known-answer vectors held by the reference's own unit tests
 * (the op, op_att, op_bert and op_out folders under test/cuBERT) and against
 * the reference's CPU sources compiled in place (oracle/_ref, see oracle/Makefile).
 *
 * All tensors are float32, row-major, caller-owned.
 */
#ifndef CUBERT_ORACLE_H
#define CUBERT_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* out[i,:] = table[ids[i],:]  (src/cuBERT/op/Embedding.cpp:10-33) */
void orc_embedding_i32(const int32_t *ids, int n, const float *table, int width, float *out);
void orc_embedding_i8(const int8_t *ids, int n, const float *table, int width, float *out);

/* inout <- beta + gamma * (inout+in-mean) / sqrt(var+1e-12), var = E[t^2]-mean^2
 * (src/cuBERT/op/LayerNorm.cpp:11-42) */
void orc_layer_norm_(const float *in, float *inout, int rows, int channels,
                     const float *beta, const float *gamma);

/* inout <- x*0.5*(1+erff(x*sqrtf(0.5)))  (src/cuBERT/op/GELU.cpp:9-16) */
void orc_gelu(size_t n, float *inout);

/* row softmax with max subtraction  (src/cuBERT/op/Softmax.cpp:12-38) */
void orc_softmax_(const float *in, float *out, int rows, int channel);

/* out[i] = !in[i]  (src/cuBERT/op_att/AttentionMask.cpp:8-18) */
void orc_not(const int8_t *in, float *out, int n);

/* neg mask broadcast [B,S] -> [B, S*H, S]  (src/cuBERT/op_att/AttentionMask.cpp:41-54) */
void orc_attention_mask(const int8_t *mask, int batch, int seq, int heads, float *out);

/* inout <- tanhf(inout)  (src/cuBERT/op_bert/BertPooler.cpp:9-16) */
void orc_tanh_(float *inout, int n);

/* out[b,c] = (sum_s in[b,s,c]) / S  (src/cuBERT/op_bert/BertPooler.cpp:18-32) */
void orc_reduce_mean_1(const float *in, float *out, int batch, int seq, int hidden);

/* Y[rows,units] = bias + X[rows,inputs] . W[inputs,units]  (src/cuBERT/op/Dense.cpp:41-57) */
void orc_dense(const float *x, const float *w, const float *bias, int rows, int inputs, int units,
               float *y);

/* LN((word[id] + pos[s]) + type[seg])  (src/cuBERT/op_bert/BertEmbeddings.cpp:50-66) */
void orc_bert_embeddings(const int32_t *ids, const int8_t *segment_ids, int batch, int seq, int hidden,
                         const float *word, const float *pos, const float *type,
                         const float *beta, const float *gamma, float *out);

/* masked scaled softmax on a score tensor [B, S, H, S]:
 * p = softmax(scale*x + (-10000)*!mask[b, key])
 * (src/cuBERT/op_att/AttentionSelf.cpp:58-60,96-108; op_att/BatchMatMul.cpp:57-68) */
void orc_masked_softmax(const float *scores, const int8_t *mask, int batch, int heads, int seq,
                        float scale, float *out);

/* tanh(first_token . W + b)  (src/cuBERT/op_bert/BertPooler.cpp:62-77) */
void orc_bert_pooler(const float *seq_out, int batch, int seq, int hidden,
                     const float *kernel, const float *bias, float *out);

/* logits = pooled . W^T (+ b), probs = softmax(logits)
 * (src/cuBERT/op_out/AdditionalOutputLayer.cpp:44-66) */
void orc_classifier(const float *pooled, int batch, int hidden, int labels,
                    const float *w, const float *bias, float *logits, float *probs);

/* scores[b,i,h,j] = sum_c k[b,j,h,c]*q[b,i,h,c]; q,k [B,S,H,d], scores [B,S,H,S]
 * (src/cuBERT/op_att/BatchMatMul.cpp:33-37,57-68) */
void orc_att_q_k(const float *q, const float *k, int batch, int seq, int heads, int d, float *scores);

/* ctx[b,i,h,c] = sum_j v[b,j,h,c]*probs[b,i,h,j]  (src/cuBERT/op_att/BatchMatMul.cpp:100-104,124-135) */
void orc_att_qk_v(const float *probs, const float *v, int batch, int seq, int heads, int d, float *ctx);

/* Self-attention with the reference's pre-broadcast float neg mask [B, S*H, S]
 * (src/cuBERT/op_att/AttentionSelf.cpp:96-111). qkv = {q_kernel,q_bias,k_kernel,k_bias,v_kernel,v_bias}. */
void orc_attention_self(const float *x, const float *const *qkv,
                        int batch, int seq, int heads, int d, const float *neg_mask, float *ctx);

/* Tensors of one encoder layer, in this fixed order. */
enum {
    ORC_Q_KERNEL = 0, ORC_Q_BIAS, ORC_K_KERNEL, ORC_K_BIAS, ORC_V_KERNEL, ORC_V_BIAS,
    ORC_ATT_OUT_KERNEL, ORC_ATT_OUT_BIAS, ORC_ATT_LN_BETA, ORC_ATT_LN_GAMMA,
    ORC_INTER_KERNEL, ORC_INTER_BIAS, ORC_OUT_KERNEL, ORC_OUT_BIAS,
    ORC_OUT_LN_BETA, ORC_OUT_LN_GAMMA, ORC_TENSORS_PER_LAYER
};

typedef struct {
    int32_t vocab, type_vocab, hidden, layers, heads, intermediate, num_labels, seq;
    const float *word_emb, *type_emb, *pos_emb, *emb_ln_beta, *emb_ln_gamma;
    const float *const *layer_tensors; /* [layers * ORC_TENSORS_PER_LAYER] */
    const float *pooler_kernel, *pooler_bias;   /* NULL -> mean pooler (src/cuBERT/Bert.cpp:34-41) */
    const float *output_weights, *output_bias;  /* NULL -> no classifier (src/cuBERT/Bert.cpp:43-53) */
} orc_bert_weights;

/* One encoder stack over [B*S, hidden]  (src/cuBERT/op_att/Transformer.cpp:145-175,
 * op_att/AttentionSelf.cpp:96-111). `x` is overwritten with the final layer output. */
void orc_transformer(const orc_bert_weights *w, int batch, float *x, const int8_t *mask);

/* Whole forward pass (src/cuBERT/Bert.cpp:99-136). Any output may be NULL. */
void orc_bert_forward(const orc_bert_weights *w, int batch,
                      const int32_t *ids, const int8_t *mask, const int8_t *segment_ids,
                      float *embedding_output, float *sequence_output, float *pooled_output,
                      float *logits, float *probs);

#ifdef __cplusplus
}
#endif
#endif
