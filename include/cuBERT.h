/*
 * cuBERT.h -- the cuBERT C API, served by the B200 (sm_100a) implementation.
 *
 * Binary-compatible with zhihu/cuBERT's src/cuBERT.h:10-97: same symbol names, argument
 * order and types, enum values and cuBERT_Output field order, so that programs, the Cython
 * wrapper (python/_cuBERT.pxd) and the JNA wrapper (java/.../CLibrary.java) written against
 * the reference library bind to this one unchanged. Default arguments exist in C++ only, as
 * in the reference.
 *
 * Behaviour kept from the reference (file:line in its tree):
 *   - a model handle is a heap object owned by the caller until cuBERT_close with the SAME
 *     compute_type (src/cuBERT.cpp:23-44,92-102);
 *   - inputs and outputs are caller-owned, C-contiguous HOST arrays; output element type is the
 *     compute type (raw IEEE binary16 for cuBERT_COMPUTE_HALF) unless output_to_float is set
 *     (src/cuBERT.h:74-78); sizes: logits/probs batch*num_labels, pooled batch*hidden,
 *     sequence/embedding batch*seq_length*hidden (src/cuBERT/Bert.cpp:146-203);
 *   - std::invalid_argument is thrown for: no GPU, invalid output type, batch_size >
 *     max_batch_size, model file missing or without tensors (src/cuBERT/BertM.cpp:21,95;
 *     Bert.cpp:100-101; tensorflow/Graph.cpp:18,84); batch_size == 0 returns silently
 *     (Bert.cpp:102-103);
 *   - cuBERT_compute* may be called from several threads; calls are spread round-robin over the
 *     replicas and serialised per replica (src/cuBERT/BertM.cpp:65-76).
 *
 * Differences: replicas per GPU can be raised with the environment variable
 * CUBERT_NUM_MODELS_PER_GPU (default 1; the GPU twin of the reference's CUBERT_NUM_CPU_MODELS).
 * The tokenizer needs no utf8proc: its Unicode tables are built in.
 */
#ifndef CUBERT_LIBRARY_H
#define CUBERT_LIBRARY_H

#include <stdint.h>

#ifdef __cplusplus
#define CUBERT_DEFAULT(v) = v
extern "C" {
#else
#define CUBERT_DEFAULT(v)
#endif

enum cuBERT_ComputeType {
    cuBERT_COMPUTE_FLOAT = 0,
    cuBERT_COMPUTE_HALF = 1 /* binary16 storage, float32 arithmetic */
};

enum cuBERT_OutputType {
    cuBERT_LOGITS = 0,
    cuBERT_POOLED_OUTPUT = 1,
    cuBERT_SEQUENCE_OUTPUT = 2,
    cuBERT_EMBEDDING_OUTPUT = 3,
    cuBERT_PROBS = 4
};

#ifndef __cplusplus
typedef enum cuBERT_ComputeType cuBERT_ComputeType;
typedef enum cuBERT_OutputType cuBERT_OutputType;
#endif

void cuBERT_initialize(void);
void cuBERT_finalize(void);

int cuBERT_get_gpu_count(void);

/* Loads a TensorFlow frozen graph and builds one model replica per visible GPU. */
void *cuBERT_open(const char *model_file,
                  int max_batch_size,
                  int seq_length,
                  int num_hidden_layers,
                  int num_attention_heads,
                  cuBERT_ComputeType compute_type CUBERT_DEFAULT(cuBERT_COMPUTE_FLOAT));

/* One forward pass; writes the selected output to the host buffer `output`. */
void cuBERT_compute(void *model,
                    int batch_size,
                    int *input_ids,
                    int8_t *input_mask,
                    int8_t *segment_ids,
                    void *output,
                    cuBERT_OutputType output_type CUBERT_DEFAULT(cuBERT_LOGITS),
                    cuBERT_ComputeType compute_type CUBERT_DEFAULT(cuBERT_COMPUTE_FLOAT));

void cuBERT_close(void *model,
                  cuBERT_ComputeType compute_type CUBERT_DEFAULT(cuBERT_COMPUTE_FLOAT));

/* Several outputs from one forward pass: every non-NULL field is filled. */
struct cuBERT_Output {
    void *logits CUBERT_DEFAULT(nullptr);
    void *pooled_output CUBERT_DEFAULT(nullptr);
    void *sequence_output CUBERT_DEFAULT(nullptr);
    void *embedding_output CUBERT_DEFAULT(nullptr);
    void *probs CUBERT_DEFAULT(nullptr);
};

#ifndef __cplusplus
typedef struct cuBERT_Output cuBERT_Output;
#endif

/* output_to_float != 0: a binary16 model converts its outputs to float32 (on the device)
 * before copying them out; ignored by a float32 model. */
void cuBERT_compute_m(void *model,
                      int batch_size,
                      int *input_ids,
                      int8_t *input_mask,
                      int8_t *segment_ids,
                      cuBERT_Output *output,
                      cuBERT_ComputeType compute_type CUBERT_DEFAULT(cuBERT_COMPUTE_FLOAT),
                      int output_to_float CUBERT_DEFAULT(0));

/* Text API (src/cuBERT.h:46-60,80-94): BERT basic + WordPiece tokenization on the calling thread,
 * then the forward pass. text_b may be NULL (single sentences). */
void *cuBERT_open_tokenizer(const char *vocab_file, int do_lower_case CUBERT_DEFAULT(1));
void cuBERT_close_tokenizer(void *tokenizer);
void cuBERT_tokenize_compute(void *model, void *tokenizer, int batch_size, const char **text_a,
                             const char **text_b, void *output,
                             cuBERT_OutputType output_type CUBERT_DEFAULT(cuBERT_LOGITS),
                             cuBERT_ComputeType compute_type CUBERT_DEFAULT(cuBERT_COMPUTE_FLOAT));
void cuBERT_tokenize_compute_m(void *model, void *tokenizer, int batch_size, const char **text_a,
                               const char **text_b, cuBERT_Output *output,
                               cuBERT_ComputeType compute_type CUBERT_DEFAULT(cuBERT_COMPUTE_FLOAT),
                               int output_to_float CUBERT_DEFAULT(0));

#ifdef __cplusplus
}
#endif
#undef CUBERT_DEFAULT
#endif /* CUBERT_LIBRARY_H */
