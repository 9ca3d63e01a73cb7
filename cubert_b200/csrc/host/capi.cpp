// extern "C" surface: the cuBERT API (include/cuBERT.h) and this library's additions
// (include/cubert_b200.h).
#include <algorithm>
#include <cstring>
#include <exception>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "bert_m.h"
#include "cuBERT.h"
#include "cubert_b200.h"
#include "tokenizer.h"

using cubert::BertM;

namespace {

thread_local std::string g_last_error;

// Runs `body` and maps exceptions to the status codes of cubert_b200.h.
template <typename F>
int guarded(F body) {
    try {
        body();
        return CUBERT_B200_OK;
    } catch (const std::invalid_argument &e) {
        g_last_error = e.what();
        return CUBERT_B200_ERR_INVALID_ARG;
    } catch (const std::out_of_range &e) {
        g_last_error = e.what();
        return CUBERT_B200_ERR_INVALID_ARG;
    } catch (const std::exception &e) {
        g_last_error = e.what();
        return CUBERT_B200_ERR_RUNTIME;
    }
}

// Calls `f(BertM<T>*)` with T chosen by compute_type (src/cuBERT.cpp:23-102 does the same cast).
template <typename F>
void with_model(void *model, int compute_type, F f) {
    if (model == nullptr) {
        throw std::invalid_argument("null model handle");
    }
    if (compute_type == cuBERT_COMPUTE_FLOAT) {
        f(static_cast<BertM<float> *>(model));
    } else if (compute_type == cuBERT_COMPUTE_HALF) {
        f(static_cast<BertM<__half> *>(model));
    } else {
        throw std::invalid_argument("invalid compute type");
    }
}

template <typename F>
void with_graph(void *graph, int compute_type, F f) {
    if (graph == nullptr) {
        throw std::invalid_argument("null graph handle");
    }
    if (compute_type == cuBERT_COMPUTE_FLOAT) {
        f(static_cast<cubert::FrozenGraph<float> *>(graph));
    } else if (compute_type == cuBERT_COMPUTE_HALF) {
        f(static_cast<cubert::FrozenGraph<__half> *>(graph));
    } else {
        throw std::invalid_argument("invalid compute type");
    }
}

// Rows of ids / mask / segment ids for a batch of texts (src/cuBERT.cpp:210-243; heap buffers instead
// of the reference's variable-length stack arrays).
void encode_batch(void *model, void *tokenizer, int batch_size, const char **text_a, const char **text_b,
                  int compute_type, std::vector<int> *ids, std::vector<int8_t> *mask, std::vector<int8_t> *seg) {
    if (tokenizer == nullptr || text_a == nullptr || batch_size < 0) {
        throw std::invalid_argument("invalid tokenizer arguments");
    }
    size_t seq = 0;
    with_model(model, compute_type, [&](auto *m) { seq = m->seq_length; });
    const auto *tok = static_cast<const cubert::FullTokenizer *>(tokenizer);
    ids->assign((size_t) batch_size * seq, 0);
    mask->assign((size_t) batch_size * seq, 0);
    seg->assign((size_t) batch_size * seq, 0);
    auto encode_range = [&](int begin, int end) {
        for (int b = begin; b < end; ++b) {
            tok->encode(seq, text_a[b], text_b == nullptr ? nullptr : text_b[b], ids->data() + b * seq,
                        mask->data() + b * seq, seg->data() + b * seq);
        }
    };
    // Texts are independent and the tokenizer is read-only: large batches are split over a few host
    // threads (a text of 100 words costs about 27 us, a 256-text batch 7 ms on one thread, as much as the
    // forward pass). CUBERT_TOKENIZER_THREADS caps the count (default 8; 1 = the calling thread only).
    int threads = cubert::env_int("CUBERT_TOKENIZER_THREADS", 8);
    const int hw = (int) std::thread::hardware_concurrency();
    threads = std::min(threads, hw > 0 ? hw : 1);
    threads = std::min(threads, batch_size / 8);
    if (threads <= 1) {
        encode_range(0, batch_size);
        return;
    }
    std::vector<std::thread> pool;
    std::vector<std::exception_ptr> errors((size_t) threads);
    for (int t = 0; t < threads; ++t) {
        const int begin = (int) ((int64_t) batch_size * t / threads);
        const int end = (int) ((int64_t) batch_size * (t + 1) / threads);
        pool.emplace_back([&, t, begin, end] {
            try {
                encode_range(begin, end);
            } catch (...) {
                errors[(size_t) t] = std::current_exception();
            }
        });
    }
    for (std::thread &th : pool) {
        th.join();
    }
    for (const std::exception_ptr &e : errors) {
        if (e) {
            std::rethrow_exception(e);
        }
    }
}

// Joins tokens with '\n' into a caller buffer; returns false if it does not fit.
bool join_tokens(const std::vector<std::string> &tokens, char *buffer, size_t buffer_size, int *count) {
    size_t need = 1;
    for (const std::string &t : tokens) {
        need += t.size() + 1;
    }
    if (buffer == nullptr || need > buffer_size) {
        return false;
    }
    char *p = buffer;
    for (size_t i = 0; i < tokens.size(); ++i) {
        std::memcpy(p, tokens[i].data(), tokens[i].size());
        p += tokens[i].size();
        *p++ = i + 1 < tokens.size() ? '\n' : '\0';
    }
    if (tokens.empty()) {
        *p = '\0';
    }
    if (count != nullptr) {
        *count = (int) tokens.size();
    }
    return true;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- reference API (src/cuBERT.h:10-97)

void cuBERT_initialize(void) {}

void cuBERT_finalize(void) {}

int cuBERT_get_gpu_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        (void) cudaGetLastError();
        return 0;
    }
    return count;
}

void *cuBERT_open(const char *model_file, int max_batch_size, int seq_length, int num_hidden_layers,
                  int num_attention_heads, cuBERT_ComputeType compute_type) {
    if (compute_type == cuBERT_COMPUTE_FLOAT) {
        return new BertM<float>(model_file, max_batch_size, seq_length, num_hidden_layers, num_attention_heads);
    }
    return new BertM<__half>(model_file, max_batch_size, seq_length, num_hidden_layers, num_attention_heads);
}

void cuBERT_compute(void *model, int batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                    void *output, cuBERT_OutputType output_type, cuBERT_ComputeType compute_type) {
    with_model(model, compute_type, [&](auto *m) {
        m->compute((size_t) batch_size, input_ids, input_mask, segment_ids, output, output_type);
    });
}

void cuBERT_compute_m(void *model, int batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                      cuBERT_Output *output, cuBERT_ComputeType compute_type, int output_to_float) {
    with_model(model, compute_type, [&](auto *m) {
        m->compute((size_t) batch_size, input_ids, input_mask, segment_ids, output, output_to_float != 0);
    });
}

void cuBERT_close(void *model, cuBERT_ComputeType compute_type) {
    if (model == nullptr) {
        return;
    }
    with_model(model, compute_type, [&](auto *m) { delete m; });
}

// Text API (src/cuBERT.cpp:104-280): tokenize on the calling thread, then the ordinary compute.
void *cuBERT_open_tokenizer(const char *vocab_file, int do_lower_case) {
    return new cubert::FullTokenizer(vocab_file, do_lower_case != 0);
}

void cuBERT_close_tokenizer(void *tokenizer) {
    delete static_cast<cubert::FullTokenizer *>(tokenizer);
}

void cuBERT_tokenize_compute(void *model, void *tokenizer, int batch_size, const char **text_a, const char **text_b,
                             void *output, cuBERT_OutputType output_type, cuBERT_ComputeType compute_type) {
    std::vector<int> ids;
    std::vector<int8_t> mask, seg;
    encode_batch(model, tokenizer, batch_size, text_a, text_b, compute_type, &ids, &mask, &seg);
    cuBERT_compute(model, batch_size, ids.data(), mask.data(), seg.data(), output, output_type, compute_type);
}

void cuBERT_tokenize_compute_m(void *model, void *tokenizer, int batch_size, const char **text_a,
                               const char **text_b, cuBERT_Output *output, cuBERT_ComputeType compute_type,
                               int output_to_float) {
    std::vector<int> ids;
    std::vector<int8_t> mask, seg;
    encode_batch(model, tokenizer, batch_size, text_a, text_b, compute_type, &ids, &mask, &seg);
    cuBERT_compute_m(model, batch_size, ids.data(), mask.data(), seg.data(), output, compute_type, output_to_float);
}

// ---------------------------------------------------------------- additions (include/cubert_b200.h)

const char *cubert_b200_last_error(void) {
    return g_last_error.c_str();
}

int cubert_b200_open(const char *model_file, int max_batch_size, int seq_length, int num_hidden_layers,
                     int num_attention_heads, int compute_type, void **model) {
    return guarded([&] {
        if (model == nullptr || model_file == nullptr) {
            throw std::invalid_argument("null argument");
        }
        if (compute_type != cuBERT_COMPUTE_FLOAT && compute_type != cuBERT_COMPUTE_HALF) {
            throw std::invalid_argument("invalid compute type");
        }
        if (max_batch_size <= 0 || seq_length <= 0 || num_hidden_layers < 0 || num_attention_heads <= 0) {
            throw std::invalid_argument("invalid model geometry");
        }
        *model = cuBERT_open(model_file, max_batch_size, seq_length, num_hidden_layers, num_attention_heads,
                             (cuBERT_ComputeType) compute_type);
    });
}

int cubert_b200_compute(void *model, int batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                        void *output, int output_type, int compute_type) {
    return guarded([&] {
        if (batch_size < 0) {
            throw std::invalid_argument("negative batch_size");
        }
        cuBERT_compute(model, batch_size, input_ids, input_mask, segment_ids, output,
                       (cuBERT_OutputType) output_type, (cuBERT_ComputeType) compute_type);
    });
}

int cubert_b200_compute_m(void *model, int batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                          cuBERT_Output *output, int compute_type, int output_to_float) {
    return guarded([&] {
        if (batch_size < 0 || output == nullptr) {
            throw std::invalid_argument("invalid argument");
        }
        cuBERT_compute_m(model, batch_size, input_ids, input_mask, segment_ids, output,
                         (cuBERT_ComputeType) compute_type, output_to_float);
    });
}

int cubert_b200_close(void *model, int compute_type) {
    return guarded([&] { cuBERT_close(model, (cuBERT_ComputeType) compute_type); });
}

int cubert_b200_model_info(void *model, int compute_type, cubert_b200_info *info) {
    return guarded([&] {
        if (info == nullptr) {
            throw std::invalid_argument("null info");
        }
        with_model(model, compute_type, [&](auto *m) {
            auto *b = m->replica(0);
            info->replicas = (int32_t) m->replicas();
            info->max_batch_size = (int32_t) b->max_batch_size;
            info->seq_length = (int32_t) b->seq_length;
            info->hidden_size = (int32_t) b->hidden_size;
            info->num_labels = b->has_classifier() ? (int32_t) b->num_labels : 0;
            info->vocab_size = (int32_t) b->vocab_size;
            info->type_vocab_size = (int32_t) b->type_vocab_size;
            info->intermediate_size = (int32_t) b->intermediate_size;
            info->num_hidden_layers = (int32_t) b->num_hidden_layers;
            info->num_attention_heads = (int32_t) b->num_attention_heads;
            info->has_pooler_dense = b->has_pooler_dense() ? 1 : 0;
            info->fp32_gemm_emulation = b->fp32_gemm_emulation() ? 1 : 0;
        });
    });
}

int cubert_b200_graph_open(const char *model_file, int compute_type, void **graph) {
    return guarded([&] {
        if (model_file == nullptr || graph == nullptr) {
            throw std::invalid_argument("null argument");
        }
        if (compute_type == cuBERT_COMPUTE_FLOAT) {
            *graph = new cubert::FrozenGraph<float>(model_file);
        } else if (compute_type == cuBERT_COMPUTE_HALF) {
            *graph = new cubert::FrozenGraph<__half>(model_file);
        } else {
            throw std::invalid_argument("invalid compute type");
        }
    });
}

int cubert_b200_graph_info(void *graph, int compute_type, cubert_b200_info *info) {
    return guarded([&] {
        if (info == nullptr) {
            throw std::invalid_argument("null info");
        }
        with_graph(graph, compute_type, [&](auto *g) {
            std::memset(info, 0, sizeof(*info));
            info->vocab_size = (int32_t) g->vocab_size;
            info->type_vocab_size = (int32_t) g->type_vocab_size;
            info->hidden_size = (int32_t) g->hidden_size;
            info->intermediate_size = (int32_t) g->intermediate_size;
            info->num_labels = g->has("output_weights") ? (int32_t) g->num_labels : 0;
            info->has_pooler_dense = g->has("bert/pooler/dense/kernel") ? 1 : 0;
        });
    });
}

int cubert_b200_graph_tensor(void *graph, int compute_type, const char *name, const void **data, int64_t *count) {
    return guarded([&] {
        if (name == nullptr || data == nullptr || count == nullptr) {
            throw std::invalid_argument("null argument");
        }
        with_graph(graph, compute_type, [&](auto *g) {
            *data = g->data(name);
            *count = (int64_t) g->var.at(name).size();
        });
    });
}

int cubert_b200_graph_close(void *graph, int compute_type) {
    return guarded([&] { with_graph(graph, compute_type, [&](auto *g) { delete g; }); });
}

int cubert_b200_open_tokenizer(const char *vocab_file, int do_lower_case, void **tokenizer) {
    return guarded([&] {
        if (vocab_file == nullptr || tokenizer == nullptr) {
            throw std::invalid_argument("null argument");
        }
        *tokenizer = cuBERT_open_tokenizer(vocab_file, do_lower_case);
    });
}

int cubert_b200_close_tokenizer(void *tokenizer) {
    return guarded([&] { cuBERT_close_tokenizer(tokenizer); });
}

int cubert_b200_encode(void *tokenizer, int max_seq_length, const char *text_a, const char *text_b,
                       int32_t *input_ids, int8_t *input_mask, int8_t *segment_ids) {
    return guarded([&] {
        if (tokenizer == nullptr || text_a == nullptr || input_ids == nullptr || input_mask == nullptr ||
            segment_ids == nullptr || max_seq_length <= 0) {
            throw std::invalid_argument("invalid argument");
        }
        static_cast<const cubert::FullTokenizer *>(tokenizer)->encode((size_t) max_seq_length, text_a, text_b,
                                                                     input_ids, input_mask, segment_ids);
    });
}

int cubert_b200_tokenize(void *tokenizer, const char *text, int do_lower_case, int max_tokens, char *buffer,
                         size_t buffer_size, int *count) {
    return guarded([&] {
        if (text == nullptr || max_tokens <= 0) {
            throw std::invalid_argument("invalid argument");
        }
        std::vector<std::string> tokens;
        if (tokenizer != nullptr) {
            static_cast<const cubert::FullTokenizer *>(tokenizer)->tokenize(text, &tokens, (size_t) max_tokens);
        } else {
            cubert::BasicTokenizer(do_lower_case != 0).tokenize(text, &tokens, (size_t) max_tokens);
        }
        if (!join_tokens(tokens, buffer, buffer_size, count)) {
            throw std::invalid_argument("token buffer too small");
        }
    });
}

int cubert_b200_tokenize_compute_m(void *model, void *tokenizer, int batch_size, const char **text_a,
                                   const char **text_b, cuBERT_Output *output, int compute_type,
                                   int output_to_float) {
    return guarded([&] {
        cuBERT_tokenize_compute_m(model, tokenizer, batch_size, text_a, text_b, output,
                                  (cuBERT_ComputeType) compute_type, output_to_float);
    });
}

int cubert_b200_replica_device(void *model, int compute_type, int replica, int *device) {
    return guarded([&] {
        with_model(model, compute_type, [&](auto *m) { *device = m->replica((size_t) replica)->device(); });
    });
}

int cubert_b200_replica_stream(void *model, int compute_type, int replica, void **stream) {
    return guarded([&] {
        with_model(model, compute_type, [&](auto *m) { *stream = m->replica((size_t) replica)->stream(); });
    });
}

int cubert_b200_forward_device(void *model, int compute_type, int replica, int batch_size,
                               const int32_t *input_ids, const int8_t *input_mask, const int8_t *segment_ids) {
    return guarded([&] {
        if (batch_size < 0) {
            throw std::invalid_argument("negative batch_size");
        }
        with_model(model, compute_type, [&](auto *m) {
            m->replica((size_t) replica)->compute_device((size_t) batch_size, input_ids, input_mask, segment_ids);
        });
    });
}

int cubert_b200_forward_device_masked(void *model, int compute_type, int replica, int batch_size,
                                      const int32_t *input_ids, const int8_t *input_mask, const int8_t *segment_ids,
                                      const int8_t *host_input_mask) {
    return guarded([&] {
        if (batch_size < 0) {
            throw std::invalid_argument("negative batch_size");
        }
        with_model(model, compute_type, [&](auto *m) {
            m->replica((size_t) replica)->compute_device((size_t) batch_size, input_ids, input_mask, segment_ids,
                                                         host_input_mask);
        });
    });
}

int cubert_b200_device_outputs(void *model, int compute_type, int replica, cuBERT_Output *outputs) {
    return guarded([&] {
        if (outputs == nullptr) {
            throw std::invalid_argument("null outputs");
        }
        with_model(model, compute_type,
                   [&](auto *m) { *outputs = m->replica((size_t) replica)->device_outputs(); });
    });
}

int cubert_b200_synchronize(void *model, int compute_type, int replica) {
    return guarded(
        [&] { with_model(model, compute_type, [&](auto *m) { m->replica((size_t) replica)->synchronize(); }); });
}

int cubert_b200_profile_enable(void *model, int compute_type, int replica, int enable) {
    return guarded([&] {
        with_model(model, compute_type,
                   [&](auto *m) { m->replica((size_t) replica)->profile_enable(enable != 0); });
    });
}

int cubert_b200_profile_read(void *model, int compute_type, int replica, cubert_b200_profile *out) {
    return guarded([&] {
        if (out == nullptr) {
            throw std::invalid_argument("null profile");
        }
        with_model(model, compute_type, [&](auto *m) { m->replica((size_t) replica)->profile_read(out); });
    });
}

}
