// One BERT replica on one GPU: weights, activation buffers, a stream, and the forward pass.
//
// Mirrors the reference's Bert<T> (src/cuBERT/Bert.h:15-75, Bert.cpp) in interface and
// results; the execution plan underneath is different:
//   * every non-GEMM step is one of the fused kernels of include/cubert_kernels.h
//     (K1 embeddings, K2 bias+residual+LayerNorm, K3 bias+GELU, K4 masked softmax, K5 heads);
//   * GEMMs run with beta = 0: no replicated bias buffers, no bias refill after each request
//     (src/cuBERT/op/Dense.cpp:22-25,41-45, Bert.cpp:88-96), no broadcast mask tensor and no
//     per-layer device copy of it (op_att/AttentionSelf.cpp:99-101);
//   * Q, K and V come from one [hidden, 3*hidden] projection;
//   * activation buffers are shared by all layers instead of allocated per layer
//     (op_att/Transformer.cpp:38-43), so memory is O(batch) and not O(layers * batch).
#pragma once

#include <array>
#include <functional>
#include <map>
#include <tuple>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "blas.h"
#include "cuBERT.h"
#include "cubert_b200.h"
#include "frozen_graph.h"
#include "runtime.h"

namespace cubert {

template <typename T>
class Bert {
public:
    // `var`: TensorFlow variable name -> host array in storage type T, as the loader yields it.
    Bert(const std::unordered_map<std::string, const T *> &var, size_t max_batch_size, size_t seq_length,
         size_t vocab_size, size_t type_vocab_size, size_t hidden_size, size_t num_hidden_layers,
         size_t num_attention_heads, size_t intermediate_size, size_t num_labels, int device);
    ~Bert();
    Bert(const Bert &) = delete;
    Bert &operator=(const Bert &) = delete;

    // Host inputs -> device, then the forward pass; asynchronous on the replica's stream.
    // Throws std::invalid_argument when batch_size > max_batch_size; batch_size == 0 is a no-op.
    // all_positions = false promises that only pooled_output / logits / probs will be read
    // afterwards; with the first-token pooler the replica may then skip padding tokens (see
    // `forward`), which leaves sequence_output and embedding_output undefined for this call.
    void compute(size_t batch_size, const int *input_ids, const int8_t *input_mask, const int8_t *segment_ids,
                 bool all_positions = true);

    // Forward pass on inputs already in this replica's device memory. `host_mask`, when the caller has a
    // host copy of d_mask, lets the replica leave masked key columns out of the attention (see KeyPlan).
    void compute_device(size_t batch_size, const int32_t *d_ids, const int8_t *d_mask, const int8_t *d_segments,
                        const int8_t *host_mask = nullptr);

    // Copy the non-NULL outputs to the host and wait for them (src/cuBERT/Bert.cpp:185-208).
    // With to_float, a binary16 model converts on the device first (Bert.cpp:218-259 does it on the host).
    void output(size_t batch_size, cuBERT_Output *out, bool to_float);

    // compute() followed by output(), as one call. For a large request that wants sequence_output, the
    // last encoder layers run sub-batch by sub-batch and each sub-batch's rows start their device-to-host
    // copy on a second stream as soon as they are final, while the next sub-batch is computed;
    // embedding_output leaves right after the embedding kernel. Results are those of the plain pass.
    // CUBERT_TAIL_CHUNKS (sub-batches, default 4, 1 = off), CUBERT_TAIL_LAYERS (default 2) and
    // CUBERT_TAIL_LAST_PERCENT (size of the last sub-batch, default 6 % of the batch) tune it.
    void compute_output(size_t batch_size, const int *input_ids, const int8_t *input_mask,
                        const int8_t *segment_ids, cuBERT_Output *out, bool to_float);

    void synchronize();
    cuBERT_Output device_outputs() const;
    cudaStream_t stream() const { return stream_; }
    int device() const { return device_; }
    bool has_classifier() const { return has_classifier_; }
    bool has_pooler_dense() const { return has_pooler_dense_; }
    bool fp32_gemm_emulation() const { return blas_ && blas_->fp32_emulation(); }

    void profile_enable(bool on);
    void profile_read(cubert_b200_profile *out);

    size_t max_batch_size, seq_length, vocab_size, type_vocab_size, hidden_size, num_hidden_layers,
        num_attention_heads, intermediate_size, num_labels;

private:
    struct Layer {
        DeviceBuffer qkv_kernel, qkv_bias;           // [hidden, 3*hidden], [3*hidden]
        DeviceBuffer att_out_kernel, att_out_bias;   // [hidden, hidden], [hidden]
        DeviceBuffer att_ln_gamma, att_ln_beta;
        DeviceBuffer inter_kernel, inter_bias;       // [hidden, intermediate], [intermediate]
        DeviceBuffer out_kernel, out_bias;           // [intermediate, hidden], [hidden]
        DeviceBuffer out_ln_gamma, out_ln_beta;
    };

    // `packed` > 0: padding is skipped. The token-wise GEMMs, LayerNorms and GELU run on a packed list
    // of `packed` tokens (the positions whose mask is non-zero, plus position 0 of every sequence for
    // the pooler; rounded up to a sixteenth of the request, at least 64, by repeating the last one); only the attention
    // products and the softmax keep the [batch, seq] layout, with rows scattered in and gathered out.
    // A masked position never influences an unmasked one (its keys get probability exactly 0), so
    // pooled_output, logits and probs are the same as in the full computation.
    // `heads_only`: only pooled_output / logits / probs will be read and the pooler is the first-token
    // one, so the LAST encoder layer is evaluated for the first token of every sequence alone: its
    // attention has one query per sequence (keys and values still come from all positions) and its
    // attention-output, LayerNorm and feed-forward steps run on `batch` rows instead of batch * seq.
    void forward(size_t batch_size, const int32_t *d_ids, const int8_t *d_mask, const int8_t *d_segments,
                 size_t packed, bool heads_only = false);
    // its parts: embeddings, a range of encoder layers on a range of sequences, pooler + classifier
    void forward_embed(size_t batch_size, const int32_t *d_ids, const int8_t *d_segments, size_t packed);
    void forward_layers(size_t l_begin, size_t l_end, size_t b0, size_t nb, size_t batch_size, const int8_t *d_mask,
                        size_t packed);
    void forward_last_layer_first_tokens(size_t batch_size, const int8_t *d_mask, size_t packed);
    void forward_heads(size_t batch_size, const int8_t *d_mask, size_t packed, bool compact_first_rows = false);

    // The forward pass as a CUDA graph, captured on first use per (batch size, input addresses) and
    // replayed afterwards: about 125 kernel launches collapse into one graph launch, which removes
    // the per-launch gaps that dominate small batches. Off while per-kernel timing is on, or with
    // the environment variable CUBERT_CUDA_GRAPH=0.
    void run(size_t batch_size, const int32_t *d_ids, const int8_t *d_mask, const int8_t *d_segments,
             size_t packed, bool heads_only = false);
    enum Phase { kWholePass = 0, kWholePassHeadsOnly, kHeadLayers, kTailLayers, kHeads };
    struct GraphKey {
        size_t batch, packed;
        const void *ids, *mask, *segments;
        int phase;        // which part of the pass the graph holds
        size_t b0, nb;    // kTailLayers: the sequences it covers
        uint64_t keys;    // plan_key(): what the attention launches of the graph depend on
        bool operator<(const GraphKey &o) const {
            return std::tie(batch, packed, ids, mask, segments, phase, b0, nb, keys) <
                   std::tie(o.batch, o.packed, o.ids, o.mask, o.segments, o.phase, o.b0, o.nb, o.keys);
        }
    };
    struct GraphEntry {
        cudaGraphExec_t exec = nullptr;
        int seen = 0;  // calls with this key so far; the first runs eagerly, the second captures
        uint64_t last_use = 0;  // for eviction of the least recently used graph when the cache is full
        std::vector<int32_t> extents;  // the key extents the graph was captured with (guards against a hash collision)
        std::array<int64_t, CUBERT_B200_K_COUNT> launches{};  // launches per family inside the graph
    };
    void run_graph(const GraphKey &key, const std::function<void()> &body);
    std::map<GraphKey, GraphEntry> graphs_;
    uint64_t graph_clock_ = 0;
    bool use_graphs_ = true;

    // profiling: brackets one launch with events when enabled, always counts
    struct Scope;
    void begin(int family);
    void end(int family, int64_t bytes);

    int device_;
    cudaStream_t stream_ = nullptr;
    std::unique_ptr<Blas> blas_;
    bool has_pooler_dense_ = false;
    bool has_classifier_ = false;
    bool has_classifier_bias_ = false;
    bool fuse_heads_ = false;
    bool small_attention_ = false;
    int64_t small_attention_tokens_ = 512;

    // weights
    DeviceBuffer word_emb_, type_emb_, pos_emb_, emb_ln_gamma_, emb_ln_beta_;
    std::vector<Layer> layers_;
    DeviceBuffer pooler_kernel_, pooler_bias_, output_weights_, output_bias_;

    // inputs and activations (shared by all layers)
    // input_ids (int32), input_mask (int8) and segment_ids (int8) of a request live in ONE device buffer at
    // fixed offsets; small models' requests arrive through one pinned staging buffer and one copy
    DeviceBuffer inputs_, status_;
    int32_t *ids_ = nullptr;
    int8_t *mask_ = nullptr, *segments_ = nullptr;
    unsigned char *h_inputs_ = nullptr;  // pinned twin of inputs_, only when the whole span is small
    void upload_inputs(size_t tokens, const int *input_ids, const int8_t *input_mask, const int8_t *segment_ids);
    DeviceBuffer embedding_, hidden_[2], qkv_, scores_, context_, dense_out_, att_out_, inter_;
    DeviceBuffer pooled_, logits_, probs_, pool_scratch_, float_staging_;
    DeviceBuffer q_ptrs_, k_ptrs_, v_ptrs_, score_ptrs_, ctx_ptrs_;

    // padding skipping: packed-token index lists (host staging is pinned) and packed buffers
    bool skip_padding_ = true;
    int32_t *h_token_index_ = nullptr;   // [max_batch * seq + max_batch]: packed list, then first-token slots
    DeviceBuffer token_index_, first_index_, qkv_packed_, ctx_packed_, first_rows_;
    // last layer on first tokens only: row b * seq of every sequence, and one-query pointer arrays
    bool prune_last_layer_ = true;
    DeviceBuffer first_index_full_, score1_ptrs_, ctx1_ptrs_;
    size_t build_token_index(size_t batch_size, const int8_t *input_mask);
    T *sequence_output_ = nullptr;

    // Attention over kept keys only. When the host sees the mask, every sequence gets a key extent: the
    // position after its last kept key, rounded up (the whole sequence when no key is kept, the reference's
    // uniform attention). Key columns from the extent on are masked, so their probabilities are exactly 0:
    // K4 reads the per-sequence extents from device memory, does not load those scores and writes zeros.
    // Optionally (CUBERT_KEY_GEMM=1, see key_group_gemms_) the Q.K^T product does not compute them and the
    // P.V product does not multiply them either: sequences are grouped by extent (a counting sort, extents
    // in steps of key_granule_), each group runs the two batched products with its own extent over pointer
    // arrays in sorted order, and a range of sequences (the sub-batches of compute_output) uses the largest
    // extent of the range. Off with CUBERT_SKIP_MASKED_KEYS=0, for sequences under 64 positions, requests
    // under 2048 positions, and when less than a tenth of the key columns would be dropped.
    static constexpr int kMaxKeyGroups = 16;
    struct KeyPlan {
        bool active = false;
        int groups = 0;
        int start[kMaxKeyGroups + 1] = {};   // first sorted sequence of each group, and the end
        int extent[kMaxKeyGroups] = {};      // key columns of each group
        uint64_t signature = 0;              // hash of the per-sequence extents (2 or more when active)
        int64_t key_columns = 0;             // sum of the extents
    };
    KeyPlan plan_;
    bool skip_masked_keys_ = true;
    int key_granule_ = 32;
    std::vector<int32_t> seq_extent_;        // per sequence, batch order (host)
    int32_t *h_plan_ = nullptr;              // pinned: sorted order [max_batch], extents [max_batch]
    DeviceBuffer plan_dev_;                  // the same on the device
    DeviceBuffer q_sorted_, k_sorted_, v_sorted_, score_sorted_, ctx_sorted_;  // pointer arrays in sorted order
    void build_key_plan(size_t batch_size, const int8_t *input_mask);
    void sort_attention_pointers(size_t batch_size);   // device side of the plan; part of the forward pass
    int range_extent(size_t b0, size_t nb) const;
    // false (default): the two products keep every key column and only K4 uses the extents (it then reads
    // no score beyond them). true (CUBERT_KEY_GEMM=1): the products run per group of equal extent as well.
    // Measured on B200, BERT-base, 256 x 128 with lengths U[8,128] (four groups): the per-group products take
    // 47 us more per layer than the two whole ones (small pointer-array products have a floor of about
    // 15 us each), 7.43 against 7.07 ms per step; side by side on four streams 7.36 ms, as one
    // cublasGemmGroupedBatchedEx call 7.98 ms, with two groups of 64 and 128 keys 7.49 ms.
    bool key_group_gemms_ = false;
    // what the attention part of a captured graph depends on: 0 = no plan, 1 = extents read from device
    // memory by K4 only (the same graph serves every mask), otherwise the plan's signature
    uint64_t plan_key() const { return !plan_.active ? 0 : (key_group_gemms_ ? plan_.signature : 1); }
    // Q.K^T (scores_product) or P.V for every group of the plan
    void grouped_products(bool scores_product, int S, int d, int heads, int H, float alpha, int algo);
    cudaEvent_t staging_read_ = nullptr;     // after the last copy out of the pinned staging buffers
    bool staging_in_flight_ = false;
    void wait_for_staging();

    // overlapped output copies
    static constexpr size_t kMaxTailChunks = 8;
    int tail_chunks_ = 4, tail_layers_ = 2, tail_last_percent_ = 6;
    cudaStream_t copy_stream_ = nullptr;
    cudaEvent_t embed_ready_ = nullptr;
    cudaEvent_t chunk_ready_[kMaxTailChunks] = {};
    DeviceBuffer float_staging_embedding_, float_staging_small_;  // float32 conversions of the overlapped path

    int algo_attention_, algo_intermediate_, algo_output_, algo_pooler_, algo_qk_, algo_qkv_;

    // profiling state
    bool profiling_ = false;
    std::array<int64_t, CUBERT_B200_K_COUNT> launches_{};
    std::array<int64_t, CUBERT_B200_K_COUNT> bytes_{};
    std::array<double, CUBERT_B200_K_COUNT> ms_{};
    struct Timed {
        int family;
        cudaEvent_t start, stop;
    };
    std::vector<Timed> pending_;
    std::vector<cudaEvent_t> event_pool_;
    cudaEvent_t open_start_ = nullptr;
    cudaEvent_t take_event();
};

}  // namespace cubert
