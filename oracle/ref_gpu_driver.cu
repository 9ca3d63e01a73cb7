/*
 * C entry points over the UNMODIFIED reference CUDA operator bodies (HAVE_CUDA build), compiled
 * for sm_100a from the reference tree by `make -C oracle ref_gpu` into
 * oracle/_ref/libcubert_ref_gpu.so. TEST AND MEASUREMENT INFRASTRUCTURE ONLY: these are the
 * reference's own GPU kernels, used as the binary16 parity reference (the reference's CPU path
 * has no half type) and timed as "the kernels to beat". Nothing in the product loads this.
 *
 * No reference code is in this file; it calls the reference's operator templates:
 *   op/LayerNorm.h:6, op/Softmax.h:9, op/GELU.h:7, op/Embedding.h:10,
 *   op_att/AttentionMask.h:9, op_bert/BertPooler.h:9,14.
 * All pointers are device pointers; `stream` is a cudaStream_t.
 */
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "cuBERT/op/Embedding.h"
#include "cuBERT/op/GELU.h"
#include "cuBERT/op/LayerNorm.h"
#include "cuBERT/op/Softmax.h"
#include "cuBERT/op_att/AttentionMask.h"
#include "cuBERT/op_bert/BertPooler.h"

extern "C" {

void refgpu_layer_norm_f32(const float *in, float *inout, int rows, int channels, float *mean, float *var,
                           const float *beta, const float *gamma, void *stream) {
    cuBERT::layer_norm_<float>(in, inout, rows, channels, mean, var, beta, gamma, stream);
}

void refgpu_layer_norm_f16(const void *in, void *inout, int rows, int channels, void *mean, void *var,
                           const void *beta, const void *gamma, void *stream) {
    cuBERT::layer_norm_<half>((const half *) in, (half *) inout, rows, channels, (half *) mean, (half *) var,
                              (const half *) beta, (const half *) gamma, stream);
}

void refgpu_softmax_f32(float *in, float *out, int rows, int channel, float *sum, void *stream) {
    cuBERT::softmax_<float>(in, out, rows, channel, sum, stream);
}

void refgpu_softmax_f16(void *in, void *out, int rows, int channel, void *sum, void *stream) {
    cuBERT::softmax_<half>((half *) in, (half *) out, rows, channel, (half *) sum, stream);
}

void refgpu_gelu_f32(size_t n, float *inout, void *stream) {
    cuBERT::gelu<float>(n, inout, stream);
}

void refgpu_gelu_f16(size_t n, void *inout, void *stream) {
    cuBERT::gelu<half>(n, (half *) inout, stream);
}

void refgpu_embedding_i32_f32(const int *ids, int n, const float *table, int width, float *out, void *stream) {
    cuBERT::embedding<int, float>(ids, n, table, width, out, stream);
}

void refgpu_embedding_i32_f16(const int *ids, int n, const void *table, int width, void *out, void *stream) {
    cuBERT::embedding<int, half>(ids, n, (const half *) table, width, (half *) out, stream);
}

void refgpu_embedding_i8_f32(const int8_t *ids, int n, const float *table, int width, float *out, void *stream) {
    cuBERT::embedding<int8_t, float>(ids, n, table, width, out, stream);
}

void refgpu_embedding_i8_f16(const int8_t *ids, int n, const void *table, int width, void *out, void *stream) {
    cuBERT::embedding<int8_t, half>(ids, n, (const half *) table, width, (half *) out, stream);
}

void refgpu_not_f32(const int8_t *in, float *out, int n, void *stream) {
    cuBERT::_not<float>(in, out, n, stream);
}

void refgpu_not_f16(const int8_t *in, void *out, int n, void *stream) {
    cuBERT::_not<half>(in, (half *) out, n, stream);
}

void refgpu_tanh_f32(float *inout, int n, void *stream) {
    cuBERT::tanh_<float>(inout, n, stream);
}

void refgpu_tanh_f16(void *inout, int n, void *stream) {
    cuBERT::tanh_<half>((half *) inout, n, stream);
}

void refgpu_reduce_mean_1_f32(const float *in, float *out, int batch, int seq, int hidden, void *stream) {
    cuBERT::reduce_mean_1<float>(in, out, batch, seq, hidden, stream);
}

void refgpu_reduce_mean_1_f16(const void *in, void *out, int batch, int seq, int hidden, void *stream) {
    cuBERT::reduce_mean_1<half>((const half *) in, (half *) out, batch, seq, hidden, stream);
}

}
