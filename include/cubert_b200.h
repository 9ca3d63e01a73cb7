/*
 * cubert_b200.h -- entry points this library adds to the cuBERT C API (include/cuBERT.h).
 *
 * None of these has a counterpart in the reference. They exist for callers that cannot use
 * C++ exceptions across a C boundary (ctypes, cgo, JNI), for measurements with inputs that
 * are already resident in device memory, and for per-kernel timing.
 *
 * Every function returns 0 on success or a negative CUBERT_B200_ERR_* code; the message of
 * the last failure on the calling thread is available from cubert_b200_last_error().
 * `model` is a handle returned by cuBERT_open / cubert_b200_open and `compute_type` must be
 * the one it was opened with, as for the reference API.
 */
#ifndef CUBERT_B200_H
#define CUBERT_B200_H

#include <stddef.h>
#include <stdint.h>

#include "cuBERT.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CUBERT_B200_OK                0
#define CUBERT_B200_ERR_INVALID_ARG  -1  /* what the reference reports as std::invalid_argument */
#define CUBERT_B200_ERR_RUNTIME      -2  /* CUDA, cuBLAS or kernel-launch failure */

const char *cubert_b200_last_error(void);

/* cuBERT_open / cuBERT_compute_m / cuBERT_compute with a status instead of an exception. */
int cubert_b200_open(const char *model_file, int max_batch_size, int seq_length, int num_hidden_layers,
                     int num_attention_heads, int compute_type, void **model);
int cubert_b200_compute(void *model, int batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                        void *output, int output_type, int compute_type);
int cubert_b200_compute_m(void *model, int batch_size, int *input_ids, int8_t *input_mask,
                          int8_t *segment_ids, struct cuBERT_Output *output, int compute_type,
                          int output_to_float);
int cubert_b200_close(void *model, int compute_type);

/* Geometry of an open model. */
struct cubert_b200_info {
    int32_t replicas;       /* model replicas (GPUs x CUBERT_NUM_MODELS_PER_GPU) */
    int32_t max_batch_size;
    int32_t seq_length;
    int32_t hidden_size;
    int32_t num_labels;     /* 0 when the model has no classifier head */
    int32_t vocab_size;
    int32_t type_vocab_size;
    int32_t intermediate_size;
    int32_t num_hidden_layers;
    int32_t num_attention_heads;
    int32_t has_pooler_dense; /* 1: first-token dense + tanh pooler, 0: mean pooler */
    int32_t fp32_gemm_emulation; /* 1: a float32 model whose cuBLAS products run as three-way bfloat16 splits on
                                    the tensor cores (cuBLAS 12.9 or newer; CUBERT_FP32_EMULATION=0 turns it off) */
};
int cubert_b200_model_info(void *model, int compute_type, struct cubert_b200_info *info);

/* The model-file reader on its own (no GPU needed): parse a frozen graph into storage type
 * `compute_type`, report the geometry sniffed from it (fields it cannot know are 0) and give
 * read access to a tensor by TensorFlow variable name (`*data` stays valid until graph_close). */
int cubert_b200_graph_open(const char *model_file, int compute_type, void **graph);
int cubert_b200_graph_info(void *graph, int compute_type, struct cubert_b200_info *info);
int cubert_b200_graph_tensor(void *graph, int compute_type, const char *name, const void **data, int64_t *count);
int cubert_b200_graph_close(void *graph, int compute_type);

/* The text front end on its own (CPU only). cubert_b200_open_tokenizer / _close_tokenizer /
 * _tokenize_compute_m are the status-returning twins of the cuBERT_* tokenizer calls.
 * cubert_b200_encode turns one text (or a pair, text_b may be NULL) into one row of
 * input_ids / input_mask / segment_ids of length max_seq_length ([CLS] a [SEP] b [SEP], zero padded).
 * cubert_b200_tokenize writes the tokens of `text`, separated by '\n' and NUL-terminated, into
 * `buffer`: WordPiece tokens when `tokenizer` is given, the basic tokenizer's words (with
 * `do_lower_case`) when it is NULL. */
int cubert_b200_open_tokenizer(const char *vocab_file, int do_lower_case, void **tokenizer);
int cubert_b200_close_tokenizer(void *tokenizer);
int cubert_b200_encode(void *tokenizer, int max_seq_length, const char *text_a, const char *text_b,
                       int32_t *input_ids, int8_t *input_mask, int8_t *segment_ids);
int cubert_b200_tokenize(void *tokenizer, const char *text, int do_lower_case, int max_tokens, char *buffer,
                         size_t buffer_size, int *count);
int cubert_b200_tokenize_compute_m(void *model, void *tokenizer, int batch_size, const char **text_a,
                                   const char **text_b, struct cuBERT_Output *output, int compute_type,
                                   int output_to_float);

/* Device of a replica and the CUDA stream (cudaStream_t) all of its work is enqueued on. */
int cubert_b200_replica_device(void *model, int compute_type, int replica, int *device);
int cubert_b200_replica_stream(void *model, int compute_type, int replica, void **stream);

/* Forward pass of one replica on inputs that already live in that replica's device memory.
 * Enqueues the work and returns; nothing is copied to the host. The results stay in the
 * replica's output buffers, whose DEVICE addresses cubert_b200_device_outputs reports (fields
 * are NULL for outputs the model does not have). Not serialised against cuBERT_compute on the
 * same replica: the caller owns the replica while it uses these two calls. */
int cubert_b200_forward_device(void *model, int compute_type, int replica, int batch_size,
                               const int32_t *input_ids, const int8_t *input_mask, const int8_t *segment_ids);
/* The same for a caller that also holds a HOST copy of the mask (batch_size * seq_length int8, equal to what
 * input_mask holds on the device). The host copy tells the replica where each sequence's kept keys end, which it
 * cannot learn from device memory without a round trip: the attention products and the softmax then leave the
 * masked key columns past that point out (their probabilities are exactly 0), as cuBERT_compute does for host
 * inputs. host_input_mask may be NULL (= cubert_b200_forward_device). */
int cubert_b200_forward_device_masked(void *model, int compute_type, int replica, int batch_size,
                                      const int32_t *input_ids, const int8_t *input_mask, const int8_t *segment_ids,
                                      const int8_t *host_input_mask);
int cubert_b200_device_outputs(void *model, int compute_type, int replica, struct cuBERT_Output *outputs);
int cubert_b200_synchronize(void *model, int compute_type, int replica);

/* Per-kernel device timing of one replica. While enabled, every kernel launch of the forward
 * pass is bracketed by CUDA events on the replica's stream; cubert_b200_profile_read waits for
 * the stream, adds up the elapsed times per kernel family since the last read and clears them.
 * Launch counters run whether timing is enabled or not. */
enum {
    CUBERT_B200_K_EMBED_LN = 0,
    CUBERT_B200_K_BIAS_RESIDUAL_LN,
    CUBERT_B200_K_BIAS_GELU,
    CUBERT_B200_K_MASKED_SOFTMAX,
    CUBERT_B200_K_BIAS_TANH,
    CUBERT_B200_K_MEAN_POOL,
    CUBERT_B200_K_LOGITS_PROBS,
    CUBERT_B200_K_HALF_TO_FLOAT,
    CUBERT_B200_K_GEMM,          /* cuBLAS / cuBLASLt calls: outside the product, timed for context */
    CUBERT_B200_K_EVENT_OVERHEAD, /* an EMPTY event bracket, once per timed forward pass: the least the event pair
                                     itself adds to every figure above (not a kernel; counted in `launches`) */
    CUBERT_B200_K_COUNT
};
struct cubert_b200_profile {
    double ms[CUBERT_B200_K_COUNT];        /* device time per family */
    int64_t launches[CUBERT_B200_K_COUNT]; /* launches per family */
    int64_t bytes[CUBERT_B200_K_COUNT];    /* algorithmic HBM bytes per family (0 for GEMM) */
};
int cubert_b200_profile_enable(void *model, int compute_type, int replica, int enable);
int cubert_b200_profile_read(void *model, int compute_type, int replica, struct cubert_b200_profile *out);

#ifdef __cplusplus
}
#endif
#endif /* CUBERT_B200_H */
