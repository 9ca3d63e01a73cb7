/*
 * C entry points over the UNMODIFIED reference CPU sources (HAVE_MKL build),
 * compiled in place from the reference tree by oracle/Makefile into
 * oracle/_ref/libcubert_ref_cpu.so. TEST INFRASTRUCTURE ONLY: used to validate
 * oracle/cubert_oracle.c, to generate tests/golden fixtures and as the timed CPU
 * baseline. Nothing in the product loads it.
 *
 * This file holds no reference code; it only calls the reference's public
 * templates and classes:
 *   op/LayerNorm.h:6, op/Softmax.h:9, op/GELU.h:7, op/Embedding.h:10,
 *   op_att/AttentionMask.h:9,19, op_bert/BertPooler.h:9,14,30,54,
 *   op_bert/BertEmbeddings.h:13, op_att/Transformer.h:15,
 *   op_out/AdditionalOutputLayer.h:28, Bert.h:15.
 */
#include <cstdint>
#include <cstring>
#include <string>
#include <unordered_map>

#include "cuBERT/common.h"
#include "cuBERT/Bert.h"
#include "cuBERT/op/Embedding.h"
#include "cuBERT/op/GELU.h"
#include "cuBERT/op/LayerNorm.h"
#include "cuBERT/op/Softmax.h"
#include "cuBERT/op_att/AttentionMask.h"
#include "cuBERT/op_att/Transformer.h"
#include "cuBERT/op_bert/BertEmbeddings.h"
#include "cuBERT/op_bert/BertPooler.h"
#include "cuBERT/op_out/AdditionalOutputLayer.h"

namespace {
typedef std::unordered_map<std::string, float *> VarMap;

VarMap make_map(int n, const char **names, float **ptrs) {
    VarMap var;
    for (int i = 0; i < n; ++i) {
        var[std::string(names[i])] = ptrs[i];
    }
    return var;
}
}

extern "C" {

void ref_layer_norm_(const float *in, float *inout, int rows, int channels,
                     const float *beta, const float *gamma) {
    cuBERT::layer_norm_<float>(in, inout, rows, channels, nullptr, nullptr, beta, gamma, nullptr);
}

void ref_softmax_(float *in, float *out, int rows, int channel) {
    cuBERT::softmax_<float>(in, out, rows, channel, nullptr, nullptr);
}

void ref_gelu(size_t n, float *inout) {
    cuBERT::gelu<float>(n, inout, nullptr);
}

void ref_embedding_i32(const int *ids, int n, const float *table, int width, float *out) {
    cuBERT::embedding<int, float>(ids, n, table, width, out, nullptr);
}

void ref_embedding_i8(const int8_t *ids, int n, const float *table, int width, float *out) {
    cuBERT::embedding<int8_t, float>(ids, n, table, width, out, nullptr);
}

void ref_not(const int8_t *in, float *out, int n) {
    cuBERT::_not<float>(in, out, n, nullptr);
}

void ref_tanh_(float *inout, int n) {
    cuBERT::tanh_<float>(inout, n, nullptr);
}

void ref_reduce_mean_1(const float *in, float *out, int batch, int seq, int hidden) {
    cuBERT::reduce_mean_1<float>(in, out, batch, seq, hidden, nullptr);
}

void ref_attention_mask(int8_t *mask, int batch, int seq, int heads, float *out) {
    cuBERT::AttentionMask<float> op(nullptr, seq, heads, batch);
    op.compute(batch, mask, out);
}

void ref_bert_embeddings(int n, const char **names, float **ptrs,
                         int batch, int seq, int vocab, int type_vocab, int hidden,
                         int *ids, int8_t *segment_ids, float *out) {
    VarMap var = make_map(n, names, ptrs);
    cuBERT::BertEmbeddings<float> op(nullptr, var, batch, vocab, type_vocab, hidden, seq);
    op.compute(batch, ids, segment_ids, out);
}

void ref_transformer(int n, const char **names, float **ptrs, const char *prefix,
                     int batch, int seq, int hidden, int layers, int heads, int intermediate,
                     float *input, int8_t *mask, float *out) {
    VarMap var = make_map(n, names, ptrs);
    cuBERT::Transformer<float> op(nullptr, prefix, var, batch, seq, hidden, layers, heads, intermediate);
    float *res = op.compute(batch, input, mask);
    std::memcpy(out, res, sizeof(float) * (size_t) batch * seq * hidden);
}

void ref_bert_pooler(float *kernel, float *bias, int batch, int seq, int hidden,
                     float *in, float *out) {
    cuBERT::BertPooler<float> op(nullptr, seq, hidden, kernel, bias, batch);
    op.compute(batch, in, out);
}

void ref_classifier(float *weights, float *bias, int batch, int hidden, int labels,
                    float *in, float *logits, float *probs) {
    cuBERT::ClassifierOutputLayer<float> op(nullptr, hidden, labels, weights, bias, batch);
    op.compute(batch, in, logits, probs);
}

void *ref_bert_open(int n, const char **names, float **ptrs,
                    int max_batch, int seq, int vocab, int type_vocab, int hidden,
                    int layers, int heads, int intermediate, int num_labels) {
    VarMap var = make_map(n, names, ptrs);
    return new cuBERT::Bert<float>(var, max_batch, seq, vocab, type_vocab, hidden,
                                   layers, heads, intermediate, num_labels);
}

void ref_bert_compute(void *model, int batch, int *ids, int8_t *mask, int8_t *segment_ids) {
    static_cast<cuBERT::Bert<float> *>(model)->compute(batch, ids, mask, segment_ids);
}

void ref_bert_output(void *model, int batch, float *logits, float *probs, float *pooled,
                     float *sequence, float *embedding) {
    cuBERT_Output out;
    out.logits = logits;
    out.probs = probs;
    out.pooled_output = pooled;
    out.sequence_output = sequence;
    out.embedding_output = embedding;
    static_cast<cuBERT::Bert<float> *>(model)->output(batch, &out);
}

void ref_bert_close(void *model) {
    delete static_cast<cuBERT::Bert<float> *>(model);
}

}
