/*
 * C entry points over the reference's own Bert<T> host class (Bert.h:15) in its GPU build (HAVE_CUDA),
 * whose operator bodies come from ref_host_b200_ops.cu, i.e. from this repository's kernels.
 * Built by `make -C oracle ref_host_b200` into oracle/_ref/libcubert_ref_host_b200.so.
 * TEST INFRASTRUCTURE ONLY; holds no reference code.
 *
 * `ptrs` are HOST arrays in the storage type (float32, or binary16 when `half` is set), exactly what the
 * reference's model loader hands to the constructor. Inputs and outputs are host arrays, outputs in the
 * storage type (Bert.cpp:99-136,185-208).
 */
#include <cuda_fp16.h>

#include <cstdint>
#include <string>
#include <unordered_map>

#include "cuBERT/common.h"
#include "cuBERT/Bert.h"

namespace {

template <typename T>
void *open_model(int n, const char **names, void **ptrs, int max_batch, int seq, int vocab, int type_vocab, int hidden,
                 int layers, int heads, int intermediate, int num_labels) {
    std::unordered_map<std::string, T *> var;
    for (int i = 0; i < n; ++i) {
        var[std::string(names[i])] = static_cast<T *>(ptrs[i]);
    }
    return new cuBERT::Bert<T>(var, max_batch, seq, vocab, type_vocab, hidden, layers, heads, intermediate, num_labels);
}

template <typename T>
void output_of(void *model, int batch, void *logits, void *probs, void *pooled, void *sequence, void *embedding) {
    cuBERT_Output out;
    out.logits = logits;
    out.probs = probs;
    out.pooled_output = pooled;
    out.sequence_output = sequence;
    out.embedding_output = embedding;
    static_cast<cuBERT::Bert<T> *>(model)->output(batch, &out);
}

}  // namespace

extern "C" {

void *refhost_open(int n, const char **names, void **ptrs, int half_storage, int max_batch, int seq, int vocab,
                   int type_vocab, int hidden, int layers, int heads, int intermediate, int num_labels) {
    cuBERT::initialize();
    cuBERT::set_gpu(0);
    return half_storage ? open_model<half>(n, names, ptrs, max_batch, seq, vocab, type_vocab, hidden, layers, heads,
                                           intermediate, num_labels)
                        : open_model<float>(n, names, ptrs, max_batch, seq, vocab, type_vocab, hidden, layers, heads,
                                            intermediate, num_labels);
}

void refhost_compute(void *model, int half_storage, int batch, int *ids, int8_t *mask, int8_t *segment_ids) {
    if (half_storage) {
        static_cast<cuBERT::Bert<half> *>(model)->compute(batch, ids, mask, segment_ids);
    } else {
        static_cast<cuBERT::Bert<float> *>(model)->compute(batch, ids, mask, segment_ids);
    }
}

void refhost_output(void *model, int half_storage, int batch, void *logits, void *probs, void *pooled, void *sequence,
                    void *embedding) {
    if (half_storage) {
        output_of<half>(model, batch, logits, probs, pooled, sequence, embedding);
    } else {
        output_of<float>(model, batch, logits, probs, pooled, sequence, embedding);
    }
}

void refhost_close(void *model, int half_storage) {
    if (half_storage) {
        delete static_cast<cuBERT::Bert<half> *>(model);
    } else {
        delete static_cast<cuBERT::Bert<float> *>(model);
    }
}

}
