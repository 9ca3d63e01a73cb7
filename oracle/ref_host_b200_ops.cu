/*
 * The reference's GPU operator bodies, served by this repository's kernels: every function template
 * that the reference defines in its six .cu files (op/Embedding.cu, op/GELU.cu, op/LayerNorm.cu,
 * op/Softmax.cu, op_att/AttentionMask.cu, op_bert/BertPooler.cu) is defined here instead, as a call
 * into the extern "C" launch layer of include/cubert_kernels.h. `make -C oracle ref_host_b200` links
 * this file with the reference's UNMODIFIED host sources (Bert.cpp, Transformer.cpp, Dense.cpp, ...,
 * compiled from the reference tree with HAVE_CUDA) into oracle/_ref/libcubert_ref_host_b200.so: the
 * reference's own C++ host code running on the B200 kernels. TEST INFRASTRUCTURE ONLY: it proves the
 * inner drop-in boundary; nothing in the product loads it. No reference code is in this file.
 *
 * Signatures: op/Embedding.h:10, op/GELU.h:7, op/LayerNorm.h:6, op/Softmax.h:9,
 * op_att/AttentionMask.h:9, op_bert/BertPooler.h:9,14. `half` is cuda_fp16's __half (common.h:9-13).
 */
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <climits>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "cuBERT/common.h"
#include "cuBERT/op/Embedding.h"
#include "cuBERT/op/GELU.h"
#include "cuBERT/op/LayerNorm.h"
#include "cuBERT/op/Softmax.h"
#include "cuBERT/op_att/AttentionMask.h"
#include "cuBERT/op_bert/BertPooler.h"
#include "cubert_kernels.h"

namespace {

void must(int rc, const char *what) {
    if (rc != CUBK_OK) {
        std::fprintf(stderr, "%s failed: %d (%s)\n", what, rc, cubk_last_cuda_error());
        std::abort();
    }
}

// A flat run of n elements as [rows, channels] with channels a multiple of 8 where n allows it.
void as_rows(size_t n, int64_t *rows, int *channels) {
    for (int c : {4096, 3072, 1024, 768, 512, 256, 64, 8}) {
        if (n % (size_t) c == 0) {
            *rows = (int64_t) (n / (size_t) c);
            *channels = c;
            return;
        }
    }
    *rows = 1;
    *channels = (int) n;
}

}  // namespace

namespace cuBERT {

template <>
void layer_norm_<float>(const float *in, float *inout, const int batch_size, const int channels, float *, float *,
                        const float *beta, const float *gamma, void *stream) {
    must(cubk_bias_residual_ln_f32(inout, nullptr, in, gamma, beta, batch_size, channels, inout, stream), "layer_norm_");
}

template <>
void layer_norm_<half>(const half *in, half *inout, const int batch_size, const int channels, half *, half *,
                       const half *beta, const half *gamma, void *stream) {
    must(cubk_bias_residual_ln_f16(inout, nullptr, in, gamma, beta, batch_size, channels, inout, stream), "layer_norm_");
}

template <>
void softmax_<float>(float *in, float *out, const int batch_size, const int channel, float *, void *stream) {
    must(cubk_masked_softmax_f32(in, nullptr, batch_size, batch_size, channel, 1.0f, out, stream), "softmax_");
}

template <>
void softmax_<half>(half *in, half *out, const int batch_size, const int channel, half *, void *stream) {
    must(cubk_masked_softmax_f16(in, nullptr, batch_size, batch_size, channel, 1.0f, out, stream), "softmax_");
}

template <>
void gelu<float>(size_t N, float *inout, void *stream) {
    int64_t rows;
    int channels;
    as_rows(N, &rows, &channels);
    must(cubk_bias_gelu_f32(inout, nullptr, rows, channels, inout, stream), "gelu");
}

template <>
void gelu<half>(size_t N, half *inout, void *stream) {
    int64_t rows;
    int channels;
    as_rows(N, &rows, &channels);
    must(cubk_bias_gelu_f16(inout, nullptr, rows, channels, inout, stream), "gelu");
}

template <>
void embedding<int, float>(const int *ids, const int n, const float *table, const int width, float *out, void *stream) {
    must(cubk_embed_gather_i32(ids, n, table, INT_MAX, width, 4, out, nullptr, stream), "embedding");
}

template <>
void embedding<int, half>(const int *ids, const int n, const half *table, const int width, half *out, void *stream) {
    must(cubk_embed_gather_i32(ids, n, table, INT_MAX, width, 2, out, nullptr, stream), "embedding");
}

template <>
void embedding<int8_t, float>(const int8_t *ids, const int n, const float *table, const int width, float *out,
                              void *stream) {
    must(cubk_embed_gather_i8(ids, n, table, INT_MAX, width, 4, out, nullptr, stream), "embedding");
}

template <>
void embedding<int8_t, half>(const int8_t *ids, const int n, const half *table, const int width, half *out,
                             void *stream) {
    must(cubk_embed_gather_i8(ids, n, table, INT_MAX, width, 2, out, nullptr, stream), "embedding");
}

template <>
void _not<float>(const int8_t *in, float *out, const int N, void *stream) {
    must(cubk_not_f32(in, out, N, stream), "_not");
}

template <>
void _not<half>(const int8_t *in, half *out, const int N, void *stream) {
    must(cubk_not_f16(in, out, N, stream), "_not");
}

template <>
void tanh_<float>(float *inout, const int N, void *stream) {
    int64_t rows;
    int channels;
    as_rows((size_t) N, &rows, &channels);
    must(cubk_bias_tanh_f32(inout, nullptr, rows, channels, inout, stream), "tanh_");
}

template <>
void tanh_<half>(half *inout, const int N, void *stream) {
    int64_t rows;
    int channels;
    as_rows((size_t) N, &rows, &channels);
    must(cubk_bias_tanh_f16(inout, nullptr, rows, channels, inout, stream), "tanh_");
}

template <>
void reduce_mean_1<float>(const float *in, float *out, const int batch_size, const int seq_length,
                          const int hidden_size, void *stream) {
    must(cubk_mean_pool_static_scratch(in, 4, batch_size, seq_length, hidden_size, out, stream), "reduce_mean_1");
}

template <>
void reduce_mean_1<half>(const half *in, half *out, const int batch_size, const int seq_length, const int hidden_size,
                         void *stream) {
    must(cubk_mean_pool_static_scratch(in, 2, batch_size, seq_length, hidden_size, out, stream), "reduce_mean_1");
}

}  // namespace cuBERT
