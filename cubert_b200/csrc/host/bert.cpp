#include "bert.h"

#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <iostream>

#include "cubert_kernels.h"
#include "key_extents.h"

namespace cubert {

namespace {

// Kernel entry points by storage type.
template <typename T>
struct K;

template <>
struct K<float> {
    static constexpr auto embed_ln = cubk_embed_ln_f32;
    static constexpr auto bias_residual_ln = cubk_bias_residual_ln_f32;
    static constexpr auto bias_gelu = cubk_bias_gelu_f32;
    static constexpr auto masked_softmax = cubk_masked_softmax_f32;
    static constexpr auto masked_softmax_extents = cubk_masked_softmax_extents_f32;
    static constexpr auto attention_small = cubk_attention_small_f32;
    static constexpr auto bias_tanh = cubk_bias_tanh_f32;
    static constexpr auto mean_pool = cubk_mean_pool_f32;
    static constexpr auto logits_probs = cubk_logits_probs_f32;
    static constexpr auto pooler_head = cubk_pooler_head_f32;
};

template <>
struct K<__half> {
    static constexpr auto embed_ln = cubk_embed_ln_f16;
    static constexpr auto bias_residual_ln = cubk_bias_residual_ln_f16;
    static constexpr auto bias_gelu = cubk_bias_gelu_f16;
    static constexpr auto masked_softmax = cubk_masked_softmax_f16;
    static constexpr auto masked_softmax_extents = cubk_masked_softmax_extents_f16;
    static constexpr auto attention_small = cubk_attention_small_f16;
    static constexpr auto bias_tanh = cubk_bias_tanh_f16;
    static constexpr auto mean_pool = cubk_mean_pool_f16;
    static constexpr auto logits_probs = cubk_logits_probs_f16;
    static constexpr auto pooler_head = cubk_pooler_head_f16;
};

template <typename T>
const T *find(const std::unordered_map<std::string, const T *> &var, const std::string &name) {
    auto it = var.find(name);
    if (it == var.end()) {
        throw std::invalid_argument("model has no tensor named " + name);
    }
    return it->second;
}

constexpr size_t kMaxStagedInputBytes = 64 * 1024;  // one staged copy of the whole input span up to this size

// Up to here a layer's attention is one launch on short sequences (CUBERT_SMALL_ATTENTION_TOKENS overrides).
// Measured on the batch 1/8/32 serving mix (seq 32): requests of 32 and 256 tokens gain 40 us
// (0.43 -> 0.39 ms), requests of 1024 tokens lose 24-37 us (one or two query rows per warp alike).
constexpr size_t kSmallAttentionTokens = 512;

template <typename T>
void upload(DeviceBuffer &dst, const T *src, size_t count) {
    dst.allocate(count * sizeof(T));
    dst.upload(src, count * sizeof(T));
}

}  // namespace

template <typename T>
Bert<T>::Bert(const std::unordered_map<std::string, const T *> &var, size_t max_batch_size_, size_t seq_length_,
              size_t vocab_size_, size_t type_vocab_size_, size_t hidden_size_, size_t num_hidden_layers_,
              size_t num_attention_heads_, size_t intermediate_size_, size_t num_labels_, int device)
    : max_batch_size(max_batch_size_),
      seq_length(seq_length_),
      vocab_size(vocab_size_),
      type_vocab_size(type_vocab_size_),
      hidden_size(hidden_size_),
      num_hidden_layers(num_hidden_layers_),
      num_attention_heads(num_attention_heads_),
      intermediate_size(intermediate_size_),
      num_labels(num_labels_),
      device_(device) {
    if (max_batch_size == 0 || seq_length == 0 || hidden_size == 0 || num_attention_heads == 0 ||
        hidden_size % num_attention_heads != 0 || vocab_size == 0 || type_vocab_size == 0) {
        throw std::invalid_argument("invalid model geometry");
    }
    CUDA_CHECK(cudaSetDevice(device_));
    CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    {
        // float32 models: room for the largest product's operands split into three bfloat16 parts each
        // (weights [hidden x intermediate], activations [max tokens x intermediate]), capped at 4 GB
        size_t emulation_ws = 0;
        if (!Storage<T>::is_half) {
            const size_t widest = intermediate_size > 3 * hidden_size ? intermediate_size : 3 * hidden_size;
            emulation_ws = 8 * widest * (hidden_size + max_batch_size * seq_length) + (32u << 20);
            const size_t cap = (size_t) 4 << 30;
            emulation_ws = emulation_ws > cap ? cap : emulation_ws;
        }
        blas_.reset(new Blas(stream_, emulation_ws));
    }
    use_graphs_ = env_int("CUBERT_CUDA_GRAPH", 1) != 0;
    tail_chunks_ = env_int("CUBERT_TAIL_CHUNKS", 4);
    tail_chunks_ = tail_chunks_ < 1 ? 1 : (tail_chunks_ > (int) kMaxTailChunks ? (int) kMaxTailChunks : tail_chunks_);
    tail_layers_ = env_int("CUBERT_TAIL_LAYERS", 2);
    tail_layers_ = tail_layers_ < 0 ? 0 : tail_layers_;
    tail_last_percent_ = env_int("CUBERT_TAIL_LAST_PERCENT", 6);
    tail_last_percent_ = tail_last_percent_ < 0 ? 0 : (tail_last_percent_ > 50 ? 50 : tail_last_percent_);
    CUDA_CHECK(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
    CUDA_CHECK(cudaEventCreateWithFlags(&embed_ready_, cudaEventDisableTiming));
    CUDA_CHECK(cudaEventCreateWithFlags(&staging_read_, cudaEventDisableTiming));
    for (cudaEvent_t &ev : chunk_ready_) {
        CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    }

    const bool half = Storage<T>::is_half;
    algo_attention_ = gemm_algo_from_env("GEMM_ALGO_ATTENTION", half);
    algo_intermediate_ = gemm_algo_from_env("GEMM_ALGO_INTERMEDIATE", half);
    algo_output_ = gemm_algo_from_env("GEMM_ALGO_OUTPUT", half);
    algo_pooler_ = gemm_algo_from_env("GEMM_ALGO_POOLER", half);
    algo_qk_ = gemm_algo_from_env("GEMM_BATCH_ALGO_QK", half);
    algo_qkv_ = gemm_algo_from_env("GEMM_BATCH_ALGO_QKV", half);

    const size_t H = hidden_size, I = intermediate_size, S = seq_length, B = max_batch_size;
    const size_t heads = num_attention_heads, d = H / heads;
    const size_t R = B * S;

    // ---- embeddings (only the first seq_length position rows are needed,
    //      src/cuBERT/op_bert/BertEmbeddings.cpp:27-29)
    upload(word_emb_, find(var, "bert/embeddings/word_embeddings"), vocab_size * H);
    upload(type_emb_, find(var, "bert/embeddings/token_type_embeddings"), type_vocab_size * H);
    upload(pos_emb_, find(var, "bert/embeddings/position_embeddings"), S * H);
    upload(emb_ln_gamma_, find(var, "bert/embeddings/LayerNorm/gamma"), H);
    upload(emb_ln_beta_, find(var, "bert/embeddings/LayerNorm/beta"), H);

    // ---- encoder layers
    layers_.resize(num_hidden_layers);
    std::vector<T> fused(H * 3 * H), fused_bias(3 * H);
    for (size_t l = 0; l < num_hidden_layers; ++l) {
        const std::string p = "bert/encoder/layer_" + std::to_string(l);
        Layer &L = layers_[l];
        const T *w[3] = {find(var, p + "/attention/self/query/kernel"), find(var, p + "/attention/self/key/kernel"),
                         find(var, p + "/attention/self/value/kernel")};
        const T *b[3] = {find(var, p + "/attention/self/query/bias"), find(var, p + "/attention/self/key/bias"),
                         find(var, p + "/attention/self/value/bias")};
        for (size_t r = 0; r < H; ++r) {
            for (int j = 0; j < 3; ++j) {
                std::memcpy(static_cast<void *>(&fused[r * 3 * H + j * H]), w[j] + r * H, H * sizeof(T));
            }
        }
        for (int j = 0; j < 3; ++j) {
            std::memcpy(static_cast<void *>(&fused_bias[j * H]), b[j], H * sizeof(T));
        }
        upload(L.qkv_kernel, fused.data(), fused.size());
        upload(L.qkv_bias, fused_bias.data(), fused_bias.size());
        upload(L.att_out_kernel, find(var, p + "/attention/output/dense/kernel"), H * H);
        upload(L.att_out_bias, find(var, p + "/attention/output/dense/bias"), H);
        upload(L.att_ln_gamma, find(var, p + "/attention/output/LayerNorm/gamma"), H);
        upload(L.att_ln_beta, find(var, p + "/attention/output/LayerNorm/beta"), H);
        upload(L.inter_kernel, find(var, p + "/intermediate/dense/kernel"), H * I);
        upload(L.inter_bias, find(var, p + "/intermediate/dense/bias"), I);
        upload(L.out_kernel, find(var, p + "/output/dense/kernel"), I * H);
        upload(L.out_bias, find(var, p + "/output/dense/bias"), H);
        upload(L.out_ln_gamma, find(var, p + "/output/LayerNorm/gamma"), H);
        upload(L.out_ln_beta, find(var, p + "/output/LayerNorm/beta"), H);
    }

    // ---- pooler and classifier (src/cuBERT/Bert.cpp:34-53)
    has_pooler_dense_ = var.count("bert/pooler/dense/kernel") != 0;
    if (has_pooler_dense_) {
        upload(pooler_kernel_, find(var, "bert/pooler/dense/kernel"), H * H);
        upload(pooler_bias_, find(var, "bert/pooler/dense/bias"), H);
    }
    has_classifier_ = var.count("output_weights") != 0;
    if (has_classifier_) {
        if (num_labels == 0) {
            throw std::invalid_argument("classifier weights present but num_labels is 0");
        }
        upload(output_weights_, find(var, "output_weights"), num_labels * H);
        has_classifier_bias_ = var.count("output_bias") != 0;
        if (has_classifier_bias_) {
            upload(output_bias_, find(var, "output_bias"), num_labels);
        }
        logits_.allocate(sizeof(T) * B * num_labels);
        probs_.allocate(sizeof(T) * B * num_labels);
    }

    // heads of 64 and short sequences: the attention of a layer runs as one launch (cubk_attention_small_*)
    // instead of two batched products and K4. Binary16: up to 128 positions and any number of tokens (matrix
    // instructions; the scores never reach HBM). Float32: up to 64 positions, requests of up to
    // kSmallAttentionTokens tokens (float32 pipes: beyond that the library's products are ahead).
    small_attention_ = S <= (sizeof(T) == 2 ? 128 : 64) && H == heads * 64 && env_int("CUBERT_SMALL_ATTENTION", 1) != 0;
    small_attention_tokens_ = env_int("CUBERT_SMALL_ATTENTION_TOKENS", sizeof(T) == 2 ? 0x7fffffff : (int) kSmallAttentionTokens);

    // first-token pooler + a small classifier: K5a and K5c run as one launch (cubk_pooler_head_*)
    {
        const size_t epv = 16 / sizeof(T);
        fuse_heads_ = has_pooler_dense_ && has_classifier_ && num_labels <= 8 && H % epv == 0 && H / epv <= 512 &&
                      env_int("CUBERT_FUSE_HEADS", 1) != 0;
    }

    // ---- inputs, activations
    {
        const size_t mask_at = (sizeof(int32_t) * R + 15) / 16 * 16, seg_at = mask_at + (R + 15) / 16 * 16;
        inputs_.allocate(seg_at + R);
        ids_ = inputs_.template as<int32_t>();
        mask_ = inputs_.template as<int8_t>() + mask_at;
        segments_ = inputs_.template as<int8_t>() + seg_at;
        if (inputs_.bytes() <= kMaxStagedInputBytes) {
            CUDA_CHECK(cudaMallocHost(reinterpret_cast<void **>(&h_inputs_), inputs_.bytes()));
        }
    }
    status_.allocate(sizeof(uint32_t));
    CUDA_CHECK(cudaMemset(status_.get(), 0, sizeof(uint32_t)));
    embedding_.allocate(sizeof(T) * R * H);
    hidden_[0].allocate(sizeof(T) * R * H);
    hidden_[1].allocate(sizeof(T) * R * H);
    qkv_.allocate(sizeof(T) * R * 3 * H);
    scores_.allocate(sizeof(T) * B * heads * S * S);
    context_.allocate(sizeof(T) * R * H);
    dense_out_.allocate(sizeof(T) * R * H);
    att_out_.allocate(sizeof(T) * R * H);
    inter_.allocate(sizeof(T) * R * I);
    pooled_.allocate(sizeof(T) * B * H);
    if (!has_pooler_dense_) {
        // small batches split the sequence axis further, so size the scratch for the worst batch
        size_t need = 0;
        for (size_t b = 1; b <= B; ++b) {
            const size_t n = cubk_mean_pool_scratch_bytes((int) b, (int) S, (int) H);
            need = n > need ? n : need;
        }
        if (need > 0) {
            pool_scratch_.allocate(need);
        }
    }
    if (half) {
        float_staging_.allocate(sizeof(float) * R * H);
    }
    // Rows of the [batch, seq] buffers that a padding-skipping pass never writes must still hold
    // finite numbers (the attention products multiply them by an exact 0).
    CUDA_CHECK(cudaMemset(qkv_.get(), 0, qkv_.bytes()));
    CUDA_CHECK(cudaMemset(context_.get(), 0, context_.bytes()));
    prune_last_layer_ = has_pooler_dense_ && num_hidden_layers > 0 && env_int("CUBERT_PRUNE_LAST_LAYER", 1) != 0;
    if (has_pooler_dense_) {
        first_rows_.allocate(sizeof(T) * B * H);
    }
    skip_padding_ = has_pooler_dense_ && env_int("CUBERT_SKIP_PADDING", 1) != 0;
    if (skip_padding_) {
        CUDA_CHECK(cudaMallocHost(reinterpret_cast<void **>(&h_token_index_), sizeof(int32_t) * (R + B)));
        token_index_.allocate(sizeof(int32_t) * R);
        first_index_.allocate(sizeof(int32_t) * B);
        qkv_packed_.allocate(sizeof(T) * R * 3 * H);
        ctx_packed_.allocate(sizeof(T) * R * H);
    }

    // ---- pointer arrays of the batched attention products, one entry per (sequence, head).
    // Layouts follow src/cuBERT/op_att/BatchMatMul.h:10-14: Q/K/V [B, S, heads, d] (here the three
    // interleaved in one [B*S, 3*hidden] buffer), scores [B, S, heads, S], context [B, S, heads, d].
    std::vector<const T *> qp(B * heads), kp(B * heads), vp(B * heads);
    std::vector<T *> sp(B * heads), cp(B * heads);
    for (size_t b = 0; b < B; ++b) {
        for (size_t h = 0; h < heads; ++h) {
            const T *base = qkv_.template as<T>() + b * S * 3 * H + h * d;
            qp[b * heads + h] = base;
            kp[b * heads + h] = base + H;
            vp[b * heads + h] = base + 2 * H;
            sp[b * heads + h] = scores_.template as<T>() + b * S * S * heads + S * h;
            cp[b * heads + h] = context_.template as<T>() + b * S * H + h * d;
        }
    }
    skip_masked_keys_ = env_int("CUBERT_SKIP_MASKED_KEYS", 1) != 0 && S >= 64;
    if (skip_masked_keys_) {
        // extents in steps of 32 keys, or of an eighth of the sequence when that is more (at most 8 groups)
        key_granule_ = (int) ((S / 8 + 31) / 32 * 32);
        key_granule_ = key_granule_ < 32 ? 32 : key_granule_;
        const int forced_granule = env_int("CUBERT_KEY_GRANULE", 0);
        if (forced_granule >= 8 && forced_granule % 8 == 0) {
            key_granule_ = forced_granule;
        }
        key_group_gemms_ = env_int("CUBERT_KEY_GEMM", 0) != 0;
        seq_extent_.assign(B, (int32_t) S);
        CUDA_CHECK(cudaMallocHost(reinterpret_cast<void **>(&h_plan_), sizeof(int32_t) * 2 * B));
        plan_dev_.allocate(sizeof(int32_t) * 2 * B);
        if (key_group_gemms_) {
            for (DeviceBuffer *sorted : {&q_sorted_, &k_sorted_, &v_sorted_, &score_sorted_, &ctx_sorted_}) {
                sorted->allocate(sizeof(void *) * B * heads);
            }
        }
    }
    upload(q_ptrs_, qp.data(), qp.size());
    upload(k_ptrs_, kp.data(), kp.size());
    upload(v_ptrs_, vp.data(), vp.size());
    upload(score_ptrs_, sp.data(), sp.size());
    upload(ctx_ptrs_, cp.data(), cp.size());
    if (prune_last_layer_) {
        // one query per sequence: compact scores [B, heads, S] at the start of scores_, context [B, hidden]
        // at the start of context_
        std::vector<T *> s1(B * heads), c1(B * heads);
        std::vector<int32_t> first(B);
        for (size_t b = 0; b < B; ++b) {
            first[b] = (int32_t) (b * S);
            for (size_t h = 0; h < heads; ++h) {
                s1[b * heads + h] = scores_.template as<T>() + (b * heads + h) * S;
                c1[b * heads + h] = context_.template as<T>() + b * H + h * d;
            }
        }
        upload(score1_ptrs_, s1.data(), s1.size());
        upload(ctx1_ptrs_, c1.data(), c1.size());
        upload(first_index_full_, first.data(), first.size());
    }

    sequence_output_ = num_hidden_layers == 0 ? embedding_.template as<T>() : hidden_[(num_hidden_layers - 1) % 2].template as<T>();
    CUDA_CHECK(cudaDeviceSynchronize());
}

template <typename T>
Bert<T>::~Bert() {
    cudaSetDevice(device_);
    if (stream_ != nullptr) {
        cudaStreamSynchronize(stream_);
    }
    for (auto &kv : graphs_) {
        if (kv.second.exec != nullptr) {
            cudaGraphExecDestroy(kv.second.exec);
        }
    }
    for (cudaEvent_t e : event_pool_) {
        cudaEventDestroy(e);
    }
    for (Timed &t : pending_) {
        cudaEventDestroy(t.start);
        cudaEventDestroy(t.stop);
    }
    blas_.reset();
    if (copy_stream_ != nullptr) {
        cudaStreamSynchronize(copy_stream_);
        cudaStreamDestroy(copy_stream_);
    }
    if (embed_ready_ != nullptr) {
        cudaEventDestroy(embed_ready_);
    }
    for (cudaEvent_t ev : chunk_ready_) {
        if (ev != nullptr) {
            cudaEventDestroy(ev);
        }
    }
    if (staging_read_ != nullptr) {
        cudaEventDestroy(staging_read_);
    }
    if (h_plan_ != nullptr) {
        cudaFreeHost(h_plan_);
    }
    if (h_token_index_ != nullptr) {
        cudaFreeHost(h_token_index_);
    }
    if (h_inputs_ != nullptr) {
        cudaFreeHost(h_inputs_);
    }
    if (stream_ != nullptr) {
        cudaStreamDestroy(stream_);
    }
}

// ------------------------------------------------------------------ profiling
template <typename T>
cudaEvent_t Bert<T>::take_event() {
    if (!event_pool_.empty()) {
        cudaEvent_t e = event_pool_.back();
        event_pool_.pop_back();
        return e;
    }
    cudaEvent_t e;
    CUDA_CHECK(cudaEventCreate(&e));
    return e;
}

// NVTX range names per kernel family (visible to ncu --nvtx and other CUPTI tools; a no-op otherwise)
static const char *const kFamilyNames[CUBERT_B200_K_COUNT] = {
    "embed_ln", "bias_residual_ln", "bias_gelu", "masked_softmax", "bias_tanh", "mean_pool",
    "logits_probs", "half_to_float", "gemm", "event_overhead"};

template <typename T>
void Bert<T>::begin(int family) {
    nvtxRangePushA(kFamilyNames[family]);
    if (profiling_) {
        open_start_ = take_event();
        CUDA_CHECK(cudaEventRecord(open_start_, stream_));
    }
}

template <typename T>
void Bert<T>::end(int family, int64_t bytes) {
    nvtxRangePop();
    launches_[family] += 1;
    bytes_[family] += bytes;
    if (profiling_) {
        cudaEvent_t stop = take_event();
        CUDA_CHECK(cudaEventRecord(stop, stream_));
        pending_.push_back(Timed{family, open_start_, stop});
        open_start_ = nullptr;
    }
}

template <typename T>
void Bert<T>::profile_enable(bool on) {
    CUDA_CHECK(cudaSetDevice(device_));
    profiling_ = on;
}

template <typename T>
void Bert<T>::profile_read(cubert_b200_profile *out) {
    CUDA_CHECK(cudaSetDevice(device_));
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    for (Timed &t : pending_) {
        float ms = 0.f;
        CUDA_CHECK(cudaEventElapsedTime(&ms, t.start, t.stop));
        ms_[t.family] += ms;
        event_pool_.push_back(t.start);
        event_pool_.push_back(t.stop);
    }
    pending_.clear();
    for (int k = 0; k < CUBERT_B200_K_COUNT; ++k) {
        out->ms[k] = ms_[k];
        out->launches[k] = launches_[k];
        out->bytes[k] = bytes_[k];
        ms_[k] = 0.0;
        launches_[k] = 0;
        bytes_[k] = 0;
    }
}

// ------------------------------------------------------------------ forward pass
// Packed list of the tokens a padding-skipping pass works on; returns its (rounded) length, or 0
// when skipping would not pay: less than a fifth of the positions is padding, or the request is so
// small (under 2048 positions) that it is bound by launches rather than by work, where the extra
// gather and scatter launches cost more than the skipped rows save (measured on B200: 1.5x faster at
// 256 x 128 with half the positions padded, break-even near 4096 positions, 6 % slower at 1024).
constexpr size_t kMinPositionsForPacking = 2048;

template <typename T>
size_t Bert<T>::build_token_index(size_t batch_size, const int8_t *input_mask) {
    const size_t S = seq_length, R = batch_size * S;
    if (R < kMinPositionsForPacking) {
        return 0;
    }
    wait_for_staging();
    int32_t *list = h_token_index_;
    int32_t *first = h_token_index_ + max_batch_size * S;
    size_t n = 0;
    for (size_t b = 0; b < batch_size; ++b) {
        first[b] = (int32_t) n;  // position 0 is always kept: the pooler reads it
        list[n++] = (int32_t) (b * S);
        const int8_t *m = input_mask + b * S;
        bool any = m[0] != 0;
        for (size_t s = 1; s < S; ++s) {
            if (m[s] != 0) {
                list[n++] = (int32_t) (b * S + s);
                any = true;
            }
        }
        if (!any) {
            // No key of this sequence is kept: the reference then attends to ALL its positions uniformly
            // (every score gets the same -10000), so none of them may be dropped. Rare (the empty rows that
            // fill a fixed batch): the whole request takes the unpacked pass.
            return 0;
        }
    }
    // Rounded up to a sixteenth of the request (at least 64): the tail repeats the last token, which costs
    // up to 6 % more rows and keeps the number of distinct packed lengths, hence of captured graphs, small.
    size_t step = (R / 16 + 63) / 64 * 64;
    step = step < 64 ? 64 : step;
    size_t padded = (n + step - 1) / step * step;
    if (padded > R) {
        padded = R;
    }
    if (padded * 5 > R * 4) {
        return 0;
    }
    for (size_t i = n; i < padded; ++i) {
        list[i] = list[n - 1];
    }
    return padded;
}

// Before the host rewrites a pinned staging buffer: the copy that last read it has finished.
template <typename T>
void Bert<T>::wait_for_staging() {
    if (staging_in_flight_) {
        CUDA_CHECK(cudaEventSynchronize(staging_read_));
        staging_in_flight_ = false;
    }
}

// ------------------------------------------------------------------ attention over kept keys only
constexpr size_t kMinPositionsForKeyPlan = 2048;


template <typename T>
void Bert<T>::build_key_plan(size_t batch_size, const int8_t *input_mask) {
    plan_ = KeyPlan();
    const size_t S = seq_length;
    if (!skip_masked_keys_ || input_mask == nullptr || batch_size * S < kMinPositionsForKeyPlan) {
        return;
    }
    // per-group products want few distinct extents; K4 alone can use them vector by vector
    const int granule = key_group_gemms_ ? key_granule_ : 8;
    if (key_group_gemms_ && (int) ((S + granule - 1) / granule) > kMaxKeyGroups) {
        return;
    }
    int64_t columns = 0;
    uint64_t hash = 1469598103934665603ull;
    for (size_t b = 0; b < batch_size; ++b) {
        const int extent = key_extent(input_mask + b * S, (int) S, granule);
        seq_extent_[b] = extent;
        columns += extent;
        hash = (hash ^ (uint64_t) extent) * 1099511628211ull;
    }
    if (columns * 10 > (int64_t) batch_size * (int64_t) S * 9) {
        return;  // under a tenth of the key columns is padding: the extra launches would cost more
    }
    wait_for_staging();
    int32_t *order = h_plan_;
    int32_t *extents = h_plan_ + max_batch_size;
    int groups = 0;
    if (key_group_gemms_) {
        groups = group_by_extent(seq_extent_.data(), batch_size, (int) S, granule, kMaxKeyGroups, order, plan_.start,
                                 plan_.extent);
        if (groups == 0) {
            return;
        }
    }
    for (size_t b = 0; b < batch_size; ++b) {
        extents[b] = seq_extent_[b];
    }
    plan_.groups = groups;
    plan_.key_columns = columns;
    plan_.signature = hash < 2 ? 2 : hash;
    plan_.active = true;
    if (key_group_gemms_) {
        CUDA_CHECK(cudaMemcpyAsync(plan_dev_.get(), order, sizeof(int32_t) * batch_size, cudaMemcpyHostToDevice, stream_));
    }
    CUDA_CHECK(cudaMemcpyAsync(plan_dev_.template as<int32_t>() + max_batch_size, extents, sizeof(int32_t) * batch_size,
                               cudaMemcpyHostToDevice, stream_));
    CUDA_CHECK(cudaEventRecord(staging_read_, stream_));
    staging_in_flight_ = true;
}

// The five pointer arrays of the batched attention products, rows permuted into the plan's sorted order
// (a row = the `heads` pointers of one sequence, gathered as 2 * heads 32-bit words).
template <typename T>
void Bert<T>::sort_attention_pointers(size_t batch_size) {
    if (!plan_.active || !key_group_gemms_) {
        return;
    }
    const int heads = (int) num_attention_heads;
    const int32_t *order = plan_dev_.template as<int32_t>();
    const DeviceBuffer *from[5] = {&q_ptrs_, &k_ptrs_, &v_ptrs_, &score_ptrs_, &ctx_ptrs_};
    DeviceBuffer *to[5] = {&q_sorted_, &k_sorted_, &v_sorted_, &score_sorted_, &ctx_sorted_};
    for (int i = 0; i < 5; ++i) {
        KERNEL_CHECK(cubk_embed_gather_i32(order, (int64_t) batch_size, from[i]->get(), (int) max_batch_size, 2 * heads, 4,
                                           to[i]->get(), nullptr, stream_));
    }
}

// The two attention products of a whole batch, one per group of equal key extent, over the sorted pointer
// arrays: scores (keys x queries, k = d) or context (d x queries, k = keys).
template <typename T>
void Bert<T>::grouped_products(bool scores_product, int S, int d, int heads, int H, float alpha, int algo) {
    const T *const *a = scores_product ? k_sorted_.template as<const T *>() : v_sorted_.template as<const T *>();
    const T *const *b = scores_product ? q_sorted_.template as<const T *>() : score_sorted_.template as<const T *>();
    T *const *c = scores_product ? score_sorted_.template as<T *>() : ctx_sorted_.template as<T *>();
    const int lda = 3 * H, ldb = scores_product ? 3 * H : S * heads, ldc = scores_product ? S * heads : H;
    for (int g = 0; g < plan_.groups; ++g) {   // group g: the sequences start[g] .. start[g + 1] of the sorted order
        const size_t at = (size_t) plan_.start[g] * heads;
        const int count = (plan_.start[g + 1] - plan_.start[g]) * heads;
        if (scores_product) {
            blas_->gemm_batched<T>(true, false, plan_.extent[g], S, d, alpha, a + at, lda, b + at, ldb, 0.f, c + at, ldc, count,
                                   algo);
        } else {
            blas_->gemm_batched<T>(false, false, d, S, plan_.extent[g], alpha, a + at, lda, b + at, ldb, 0.f, c + at, ldc, count,
                                   algo);
        }
    }
}

template <typename T>
int Bert<T>::range_extent(size_t b0, size_t nb) const {
    int e = 0;
    for (size_t b = b0; b < b0 + nb; ++b) {
        e = seq_extent_[b] > e ? seq_extent_[b] : e;
    }
    return e;
}

// Host inputs to the device. When the model's whole input span is small (serving-size models), the three
// arrays are gathered in a pinned staging buffer laid out like the device buffer and go over in ONE copy;
// three copies from pageable caller memory each pay the driver's own staging. Otherwise three copies.
template <typename T>
void Bert<T>::upload_inputs(size_t tokens, const int *input_ids, const int8_t *input_mask, const int8_t *segment_ids) {
    if (h_inputs_ != nullptr) {
        wait_for_staging();
        const size_t mask_at = (size_t) (mask_ - inputs_.template as<int8_t>());
        const size_t seg_at = (size_t) (segments_ - inputs_.template as<int8_t>());
        std::memcpy(h_inputs_, input_ids, sizeof(int32_t) * tokens);
        std::memcpy(h_inputs_ + mask_at, input_mask, tokens);
        std::memcpy(h_inputs_ + seg_at, segment_ids, tokens);
        CUDA_CHECK(cudaMemcpyAsync(inputs_.get(), h_inputs_, seg_at + tokens, cudaMemcpyHostToDevice, stream_));
        CUDA_CHECK(cudaEventRecord(staging_read_, stream_));
        staging_in_flight_ = true;
        return;
    }
    CUDA_CHECK(cudaMemcpyAsync(ids_, input_ids, sizeof(int32_t) * tokens, cudaMemcpyHostToDevice, stream_));
    CUDA_CHECK(cudaMemcpyAsync(mask_, input_mask, sizeof(int8_t) * tokens, cudaMemcpyHostToDevice, stream_));
    CUDA_CHECK(cudaMemcpyAsync(segments_, segment_ids, sizeof(int8_t) * tokens, cudaMemcpyHostToDevice, stream_));
}

template <typename T>
void Bert<T>::compute(size_t batch_size, const int *input_ids, const int8_t *input_mask,
                      const int8_t *segment_ids, bool all_positions) {
    if (batch_size > max_batch_size) {
        throw std::invalid_argument("batch_size > max_batch_size");
    } else if (batch_size == 0) {
        return;
    }
    if (input_ids == nullptr || input_mask == nullptr || segment_ids == nullptr) {
        throw std::invalid_argument("null input");
    }
    CUDA_CHECK(cudaSetDevice(device_));
    const size_t n = batch_size * seq_length;
    upload_inputs(n, input_ids, input_mask, segment_ids);
    size_t packed = 0;
    if (!all_positions && skip_padding_) {
        packed = build_token_index(batch_size, input_mask);
        if (packed > 0) {
            CUDA_CHECK(cudaMemcpyAsync(token_index_.get(), h_token_index_, sizeof(int32_t) * packed,
                                       cudaMemcpyHostToDevice, stream_));
            CUDA_CHECK(cudaMemcpyAsync(first_index_.get(), h_token_index_ + max_batch_size * seq_length,
                                       sizeof(int32_t) * batch_size, cudaMemcpyHostToDevice, stream_));
            CUDA_CHECK(cudaEventRecord(staging_read_, stream_));
            staging_in_flight_ = true;
        }
    }
    build_key_plan(batch_size, input_mask);
    // the last layer for first tokens only: when nothing per-position is wanted and the request is large
    // enough for the saved rows to outweigh one extra gather launch
    const bool heads_only = !all_positions && prune_last_layer_ && (packed > 0 || n >= kMinPositionsForPacking);
    run(batch_size, ids_, mask_, segments_, packed, heads_only);
}

template <typename T>
void Bert<T>::compute_device(size_t batch_size, const int32_t *d_ids, const int8_t *d_mask,
                             const int8_t *d_segments, const int8_t *host_mask) {
    if (batch_size > max_batch_size) {
        throw std::invalid_argument("batch_size > max_batch_size");
    } else if (batch_size == 0) {
        return;
    }
    if (d_ids == nullptr || d_mask == nullptr || d_segments == nullptr) {
        throw std::invalid_argument("null input");
    }
    CUDA_CHECK(cudaSetDevice(device_));
    build_key_plan(batch_size, host_mask);
    run(batch_size, d_ids, d_mask, d_segments, 0);
}

constexpr size_t kMaxCachedGraphs = 256;

template <typename T>
void Bert<T>::run(size_t batch_size, const int32_t *d_ids, const int8_t *d_mask, const int8_t *d_segments,
                  size_t packed, bool heads_only) {
    const GraphKey key{batch_size, packed, d_ids, d_mask, d_segments, heads_only ? kWholePassHeadsOnly : kWholePass, 0, 0,
                       plan_key()};
    run_graph(key, [&] { forward(batch_size, d_ids, d_mask, d_segments, packed, heads_only); });
}

// Runs `body` (a sequence of launches on stream_) eagerly the first time a key is seen (cuBLASLt picks
// its algorithms, occupancy is queried), captures it into a CUDA graph the second time and replays that
// graph from then on.
template <typename T>
void Bert<T>::run_graph(const GraphKey &key, const std::function<void()> &body) {
    if (!use_graphs_ || profiling_) {
        body();
        return;
    }
    auto it = graphs_.find(key);
    if (it != graphs_.end() && key.keys > 1 &&
        (it->second.extents.size() != key.batch ||
         !std::equal(it->second.extents.begin(), it->second.extents.end(), seq_extent_.begin()))) {
        body();  // another set of key extents with the same hash: never replay a graph of other shapes
        return;
    }
    if (it == graphs_.end()) {
        if (graphs_.size() >= kMaxCachedGraphs) {
            // make room: the least recently used graph goes
            auto oldest = graphs_.begin();
            for (auto e = graphs_.begin(); e != graphs_.end(); ++e) {
                if (e->second.last_use < oldest->second.last_use) {
                    oldest = e;
                }
            }
            if (oldest->second.exec != nullptr) {
                cudaGraphExecDestroy(oldest->second.exec);
            }
            graphs_.erase(oldest);
        }
        it = graphs_.emplace(key, GraphEntry()).first;
        if (key.keys > 1) {
            it->second.extents.assign(seq_extent_.begin(), seq_extent_.begin() + (long) key.batch);
        }
    }
    it->second.last_use = ++graph_clock_;
    GraphEntry &g = it->second;
    if (g.exec != nullptr) {
        for (int k = 0; k < CUBERT_B200_K_COUNT; ++k) {
            launches_[k] += g.launches[k];  // the launch counters keep counting what the graph replays
        }
        CUDA_CHECK(cudaGraphLaunch(g.exec, stream_));
        return;
    }
    g.seen += 1;
    if (g.seen == 1) {
        body();
        return;
    }
    const auto saved_launches = launches_;
    const auto saved_bytes = bytes_;
    cudaGraph_t graph = nullptr;
    CUDA_CHECK(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
    try {
        body();
    } catch (...) {
        cudaStreamEndCapture(stream_, &graph);
        if (graph != nullptr) {
            cudaGraphDestroy(graph);
        }
        throw;
    }
    CUDA_CHECK(cudaStreamEndCapture(stream_, &graph));
    for (int k = 0; k < CUBERT_B200_K_COUNT; ++k) {
        g.launches[k] = launches_[k] - saved_launches[k];
    }
    launches_ = saved_launches;  // capturing launched nothing
    bytes_ = saved_bytes;
    cudaError_t err = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (err != cudaSuccess) {
        g.exec = nullptr;
        use_graphs_ = false;  // fall back to plain launches for good
        (void) cudaGetLastError();
        body();
        return;
    }
    run_graph(key, body);
}

template <typename T>
void Bert<T>::forward(size_t batch_size, const int32_t *d_ids, const int8_t *d_mask, const int8_t *d_segments,
                      size_t packed, bool heads_only) {
    forward_embed(batch_size, d_ids, d_segments, packed);
    sort_attention_pointers(batch_size);
    if (packed > 0) {
        // Rows of the [batch, seq] Q/K/V buffer that this pass never writes (dropped padding) are multiplied
        // by probabilities that are exactly 0: they must hold finite numbers, whatever earlier requests left.
        CUDA_CHECK(cudaMemsetAsync(qkv_.get(), 0, sizeof(T) * batch_size * seq_length * 3 * hidden_size, stream_));
    }
    if (heads_only && prune_last_layer_) {
        forward_layers(0, num_hidden_layers - 1, 0, batch_size, batch_size, d_mask, packed);
        forward_last_layer_first_tokens(batch_size, d_mask, packed);
        forward_heads(batch_size, d_mask, packed, true);
    } else {
        forward_layers(0, num_hidden_layers, 0, batch_size, batch_size, d_mask, packed);
        forward_heads(batch_size, d_mask, packed);
    }
}

// K1: embeddings (src/cuBERT/op_bert/BertEmbeddings.cpp:50-66); with `packed`, also the gather of the
// kept tokens' rows into the first layer's input.
template <typename T>
void Bert<T>::forward_embed(size_t batch_size, const int32_t *d_ids, const int8_t *d_segments, size_t packed) {
    const int B = (int) batch_size, S = (int) seq_length, H = (int) hidden_size;
    const int64_t R = (int64_t) B * S;
    const int64_t e = sizeof(T);
    void *st = stream_;
    begin(CUBERT_B200_K_EMBED_LN);
    KERNEL_CHECK(K<T>::embed_ln(d_ids, d_segments, word_emb_.template as<T>(), pos_emb_.template as<T>(), type_emb_.template as<T>(),
                                emb_ln_gamma_.template as<T>(), emb_ln_beta_.template as<T>(), B, S, H, (int) vocab_size,
                                (int) type_vocab_size, embedding_.template as<T>(), status_.template as<uint32_t>(), st));
    end(CUBERT_B200_K_EMBED_LN, 2 * R * H * e + 5 * R + (int64_t) S * H * e + (int64_t) type_vocab_size * H * e +
                                    2 * H * e);
    if (packed > 0) {
        // layer 0 writes hidden_[0], so the gathered rows go to hidden_[1]
        KERNEL_CHECK(cubk_embed_gather_i32(token_index_.template as<int32_t>(), (int64_t) packed, embedding_.get(), (int) R, H,
                                           (int) e, hidden_[1].get(), nullptr, st));
    }
}

// Encoder layers [l_begin, l_end) on the sequences [b0, b0 + nb) of a batch of `batch_size`
// (src/cuBERT/op_att/Transformer.cpp:145-175, op_att/AttentionSelf.cpp:96-111). Sequences are
// independent of one another, so a sub-range of them runs on the same rows of every buffer that the
// whole batch would use. `packed` > 0 (whole batch only): see the class comment.
template <typename T>
void Bert<T>::forward_layers(size_t l_begin, size_t l_end, size_t b0, size_t nb, size_t batch_size,
                             const int8_t *d_mask, size_t packed) {
    const int B = (int) nb, S = (int) seq_length, H = (int) hidden_size, I = (int) intermediate_size;
    const int heads = (int) num_attention_heads, d = H / heads;
    const int64_t R = (int64_t) B * S;      // rows of the [batch, seq] layout in this range
    const int64_t N = packed > 0 ? (int64_t) packed : R;  // rows the token-wise steps work on
    const int64_t e = sizeof(T);
    const int64_t row0 = (int64_t) b0 * S;  // first row of the range (0 when packed)
    void *st = stream_;
    const int32_t *tok = token_index_.template as<int32_t>();
    const int8_t *mask = d_mask + row0;

    const float att_scale = (float) (1.0 / std::sqrt((double) d));  // op_att/AttentionSelf.cpp:58-60
    T *qkv = qkv_.template as<T>() + row0 * 3 * H;
    T *scores = scores_.template as<T>() + (int64_t) b0 * heads * S * S;
    T *context = context_.template as<T>() + row0 * H;
    T *dense_out = dense_out_.template as<T>() + row0 * H;
    T *att_out = att_out_.template as<T>() + row0 * H;
    T *inter = inter_.template as<T>() + row0 * I;
    const size_t p0 = b0 * (size_t) heads;  // first entry of the range in the pointer arrays

    // key columns the attention works on (see KeyPlan)
    const bool grouped = plan_.active && key_group_gemms_ && b0 == 0 && nb == batch_size;
    const int keys = plan_.active && key_group_gemms_ && !grouped ? range_extent(b0, nb) : S;
    const int32_t *extents = plan_.active ? plan_dev_.template as<int32_t>() + max_batch_size + b0 : nullptr;
    for (size_t l = l_begin; l < l_end; ++l) {
        Layer &L = layers_[l];
        const T *x = l == 0 ? (packed > 0 ? hidden_[1].template as<T>() : embedding_.template as<T>() + row0 * H)
                            : hidden_[(l - 1) % 2].template as<T>() + row0 * H;
        T *y = hidden_[l % 2].template as<T>() + row0 * H;

        // Q, K, V in one projection with the bias in the GEMM epilogue
        T *qkv_out = packed > 0 ? qkv_packed_.template as<T>() : qkv;
        begin(CUBERT_B200_K_GEMM);
        blas_->gemm_bias<T>(3 * H, (int) N, H, L.qkv_kernel.template as<T>(), 3 * H, x, H, L.qkv_bias.template as<T>(), qkv_out,
                            3 * H);
        end(CUBERT_B200_K_GEMM, 0);
        if (packed > 0) {
            // back to [batch, seq] places for the attention products (padding rows keep old, finite values)
            KERNEL_CHECK(cubk_scatter_rows(tok, N, qkv_out, 3 * H, (int) e, qkv_.get(), (int) R, st));
        }

        if (small_attention_ && R <= small_attention_tokens_) {
            // the whole attention of the layer in one launch (timed in K4's slot; its bytes: Q | K | V read,
            // the context written, the mask)
            begin(CUBERT_B200_K_MASKED_SOFTMAX);
            KERNEL_CHECK(K<T>::attention_small(qkv, mask, B, S, heads, H, att_scale, context, st));
            end(CUBERT_B200_K_MASKED_SOFTMAX, 4 * R * H * e + R);
        } else {
            // scores[b, i, h, j] = (1/sqrt(d)) * sum_c K[b,j,h,c] * Q[b,i,h,c]   (op_att/BatchMatMul.cpp:57-68)
            // With a key plan only the key columns j below each sequence's extent exist: one product per group
            // of equal extent over the sorted pointer arrays, or (a range of sequences) the range's largest extent.
            begin(CUBERT_B200_K_GEMM);
            if (grouped) {
                grouped_products(true, S, d, heads, H, att_scale, algo_qk_);
            } else {
                blas_->gemm_batched<T>(true, false, keys, S, d, att_scale, k_ptrs_.template as<const T *>() + p0, 3 * H,
                                       q_ptrs_.template as<const T *>() + p0, 3 * H, 0.f, score_ptrs_.template as<T *>() + p0,
                                       S * heads, B * heads, algo_qk_);
            }
            end(CUBERT_B200_K_GEMM, 0);

            // K4: mask + softmax in place over rows [B*S*heads, S]
            begin(CUBERT_B200_K_MASKED_SOFTMAX);
            if (plan_.active) {
                KERNEL_CHECK(K<T>::masked_softmax_extents(scores, mask, extents, grouped ? 0 : keys, R * heads, (int64_t) S * heads,
                                                          S, 1.0f, scores, st));
            } else {
                KERNEL_CHECK(K<T>::masked_softmax(scores, mask, R * heads, (int64_t) S * heads, S, 1.0f, scores, st));
            }
            // charged with the bytes of the whole score matrix (the figure the roofline is quoted on), whatever
            // the key extents let it skip
            end(CUBERT_B200_K_MASKED_SOFTMAX, 2 * R * heads * S * e + R);

            // context[b, i, h, c] = sum_j V[b,j,h,c] * P[b,i,h,j]   (op_att/BatchMatMul.cpp:124-135)
            begin(CUBERT_B200_K_GEMM);
            if (grouped) {
                grouped_products(false, S, d, heads, H, 1.f, algo_qkv_);
            } else {
                blas_->gemm_batched<T>(false, false, d, S, keys, 1.f, v_ptrs_.template as<const T *>() + p0, 3 * H,
                                       score_ptrs_.template as<const T *>() + p0, S * heads, 0.f, ctx_ptrs_.template as<T *>() + p0,
                                       H, B * heads, algo_qkv_);
            }
            end(CUBERT_B200_K_GEMM, 0);
        }

        // attention output projection, then K2: LayerNorm(dense + bias + layer input)
        const T *ctx = context;
        if (packed > 0) {
            KERNEL_CHECK(cubk_embed_gather_i32(tok, N, context_.get(), (int) R, H, (int) e, ctx_packed_.get(), nullptr, st));
            ctx = ctx_packed_.template as<T>();
        }
        begin(CUBERT_B200_K_GEMM);
        blas_->gemm<T>(false, false, H, (int) N, H, 1.f, L.att_out_kernel.template as<T>(), H, ctx, H, 0.f, dense_out, H,
                       algo_attention_);
        end(CUBERT_B200_K_GEMM, 0);
        begin(CUBERT_B200_K_BIAS_RESIDUAL_LN);
        KERNEL_CHECK(K<T>::bias_residual_ln(dense_out, L.att_out_bias.template as<T>(), x, L.att_ln_gamma.template as<T>(),
                                            L.att_ln_beta.template as<T>(), N, H, att_out, st));
        end(CUBERT_B200_K_BIAS_RESIDUAL_LN, 3 * N * H * e + 3 * H * e);

        // intermediate projection, then K3: bias + GELU in place
        begin(CUBERT_B200_K_GEMM);
        blas_->gemm<T>(false, false, I, (int) N, H, 1.f, L.inter_kernel.template as<T>(), I, att_out, H, 0.f, inter, I,
                       algo_intermediate_);
        end(CUBERT_B200_K_GEMM, 0);
        begin(CUBERT_B200_K_BIAS_GELU);
        KERNEL_CHECK(K<T>::bias_gelu(inter, L.inter_bias.template as<T>(), N, I, inter, st));
        end(CUBERT_B200_K_BIAS_GELU, 2 * N * I * e + I * e);

        // output projection, then K2: LayerNorm(dense + bias + attention output)
        begin(CUBERT_B200_K_GEMM);
        blas_->gemm<T>(false, false, H, (int) N, I, 1.f, L.out_kernel.template as<T>(), H, inter, I, 0.f, dense_out, H,
                       algo_output_);
        end(CUBERT_B200_K_GEMM, 0);
        begin(CUBERT_B200_K_BIAS_RESIDUAL_LN);
        KERNEL_CHECK(K<T>::bias_residual_ln(dense_out, L.out_bias.template as<T>(), att_out, L.out_ln_gamma.template as<T>(),
                                            L.out_ln_beta.template as<T>(), N, H, y, st));
        end(CUBERT_B200_K_BIAS_RESIDUAL_LN, 3 * N * H * e + 3 * H * e);
    }
}

// The last encoder layer when only the first token of every sequence is read afterwards (the
// first-token pooler): Q, K and V are still projected for every position, since every key and value
// feeds the first token's attention, but there is ONE query per sequence, and everything after the
// attention runs on `batch` rows. Scores [batch, heads, seq] sit at the start of scores_, the context
// and later activations at the start of their buffers, the layer's output at the start of the
// hidden buffer the full layer would have written. Same operations on a subset of the rows, so the
// pooled output is the one the full layer gives.
template <typename T>
void Bert<T>::forward_last_layer_first_tokens(size_t batch_size, const int8_t *d_mask, size_t packed) {
    const int B = (int) batch_size, S = (int) seq_length, H = (int) hidden_size, I = (int) intermediate_size;
    const int heads = (int) num_attention_heads, d = H / heads;
    const int64_t R = (int64_t) B * S;
    const int64_t N = packed > 0 ? (int64_t) packed : R;
    const int64_t e = sizeof(T);
    void *st = stream_;
    const size_t l = num_hidden_layers - 1;
    Layer &L = layers_[l];
    const float att_scale = (float) (1.0 / std::sqrt((double) d));
    const T *x = l == 0 ? (packed > 0 ? hidden_[1].template as<T>() : embedding_.template as<T>())
                        : hidden_[(l - 1) % 2].template as<T>();
    T *y = hidden_[l % 2].template as<T>();  // [batch, hidden] here

    T *qkv_out = packed > 0 ? qkv_packed_.template as<T>() : qkv_.template as<T>();
    begin(CUBERT_B200_K_GEMM);
    blas_->gemm_bias<T>(3 * H, (int) N, H, L.qkv_kernel.template as<T>(), 3 * H, x, H, L.qkv_bias.template as<T>(), qkv_out,
                        3 * H);
    end(CUBERT_B200_K_GEMM, 0);
    if (packed > 0) {
        KERNEL_CHECK(cubk_scatter_rows(token_index_.template as<int32_t>(), N, qkv_out, 3 * H, (int) e, qkv_.get(), (int) R, st));
    }

    // scores[b, h, j] = (1/sqrt(d)) * sum_c K[b,j,h,c] * Q[b,0,h,c]: the batched product with one column
    begin(CUBERT_B200_K_GEMM);
    blas_->gemm_batched<T>(true, false, S, 1, d, att_scale, k_ptrs_.template as<const T *>(), 3 * H,
                           q_ptrs_.template as<const T *>(), 3 * H, 0.f, score1_ptrs_.template as<T *>(), S, B * heads, algo_qk_);
    end(CUBERT_B200_K_GEMM, 0);
    begin(CUBERT_B200_K_MASKED_SOFTMAX);
    KERNEL_CHECK(K<T>::masked_softmax(scores_.template as<T>(), d_mask, (int64_t) B * heads, heads, S, 1.0f,
                                      scores_.template as<T>(), st));
    end(CUBERT_B200_K_MASKED_SOFTMAX, 2 * (int64_t) B * heads * S * e + R);
    begin(CUBERT_B200_K_GEMM);
    blas_->gemm_batched<T>(false, false, d, 1, S, 1.f, v_ptrs_.template as<const T *>(), 3 * H,
                           score1_ptrs_.template as<const T *>(), S, 0.f, ctx1_ptrs_.template as<T *>(), H, B * heads, algo_qkv_);
    end(CUBERT_B200_K_GEMM, 0);

    // the layer input of the first tokens (the residual of the first LayerNorm)
    const int32_t *first = packed > 0 ? first_index_.template as<int32_t>() : first_index_full_.template as<int32_t>();
    KERNEL_CHECK(cubk_embed_gather_i32(first, B, x, (int) N, H, (int) e, first_rows_.get(), nullptr, st));

    begin(CUBERT_B200_K_GEMM);
    blas_->gemm<T>(false, false, H, B, H, 1.f, L.att_out_kernel.template as<T>(), H, context_.template as<T>(), H, 0.f,
                   dense_out_.template as<T>(), H, algo_attention_);
    end(CUBERT_B200_K_GEMM, 0);
    begin(CUBERT_B200_K_BIAS_RESIDUAL_LN);
    KERNEL_CHECK(K<T>::bias_residual_ln(dense_out_.template as<T>(), L.att_out_bias.template as<T>(), first_rows_.template as<T>(),
                                        L.att_ln_gamma.template as<T>(), L.att_ln_beta.template as<T>(), B, H,
                                        att_out_.template as<T>(), st));
    end(CUBERT_B200_K_BIAS_RESIDUAL_LN, 3 * (int64_t) B * H * e + 3 * H * e);

    begin(CUBERT_B200_K_GEMM);
    blas_->gemm<T>(false, false, I, B, H, 1.f, L.inter_kernel.template as<T>(), I, att_out_.template as<T>(), H, 0.f,
                   inter_.template as<T>(), I, algo_intermediate_);
    end(CUBERT_B200_K_GEMM, 0);
    begin(CUBERT_B200_K_BIAS_GELU);
    KERNEL_CHECK(K<T>::bias_gelu(inter_.template as<T>(), L.inter_bias.template as<T>(), B, I, inter_.template as<T>(), st));
    end(CUBERT_B200_K_BIAS_GELU, 2 * (int64_t) B * I * e + I * e);

    begin(CUBERT_B200_K_GEMM);
    blas_->gemm<T>(false, false, H, B, I, 1.f, L.out_kernel.template as<T>(), H, inter_.template as<T>(), I, 0.f,
                   dense_out_.template as<T>(), H, algo_output_);
    end(CUBERT_B200_K_GEMM, 0);
    begin(CUBERT_B200_K_BIAS_RESIDUAL_LN);
    KERNEL_CHECK(K<T>::bias_residual_ln(dense_out_.template as<T>(), L.out_bias.template as<T>(), att_out_.template as<T>(),
                                        L.out_ln_gamma.template as<T>(), L.out_ln_beta.template as<T>(), B, H, y, st));
    end(CUBERT_B200_K_BIAS_RESIDUAL_LN, 3 * (int64_t) B * H * e + 3 * H * e);
}

// Pooler and classifier over the whole batch (src/cuBERT/op_bert/BertPooler.cpp:62-77,93-96;
// src/cuBERT/op_out/AdditionalOutputLayer.cpp:44-66).
template <typename T>
void Bert<T>::forward_heads(size_t batch_size, const int8_t *d_mask, size_t packed, bool compact_first_rows) {
    const int B = (int) batch_size, S = (int) seq_length, H = (int) hidden_size;
    const int64_t R = (int64_t) B * S;
    const int64_t N = packed > 0 ? (int64_t) packed : R;
    const int64_t e = sizeof(T);
    void *st = stream_;
    // what the last layer wrote; with no layers, the embeddings (gathered into hidden_[1] when packed)
    const T *x = num_hidden_layers == 0 ? (packed > 0 ? hidden_[1].template as<T>() : embedding_.template as<T>())
                                        : hidden_[(num_hidden_layers - 1) % 2].template as<T>();

    if (has_pooler_dense_) {
        const T *first = x;       // first token of every sequence: rows S apart, or gathered when packed
        int first_ld = H * S;
        if (compact_first_rows) {
            first_ld = H;         // the last layer ran on the first tokens only: one row per sequence
        } else if (packed > 0) {
            KERNEL_CHECK(cubk_embed_gather_i32(first_index_.template as<int32_t>(), B, x, (int) N, H, (int) e,
                                               first_rows_.get(), nullptr, st));
            first = first_rows_.template as<T>();
            first_ld = H;
        }
        begin(CUBERT_B200_K_GEMM);
        blas_->gemm<T>(false, false, H, B, H, 1.f, pooler_kernel_.template as<T>(), H, first, first_ld, 0.f, pooled_.template as<T>(), H,
                       algo_pooler_);
        end(CUBERT_B200_K_GEMM, 0);
        begin(CUBERT_B200_K_BIAS_TANH);
        if (fuse_heads_) {
            // pooler activation and classifier in one launch (counted with the pooler activation)
            KERNEL_CHECK(K<T>::pooler_head(pooled_.template as<T>(), pooler_bias_.template as<T>(), output_weights_.template as<T>(),
                                           has_classifier_bias_ ? output_bias_.template as<T>() : nullptr, B, H, (int) num_labels,
                                           pooled_.template as<T>(), logits_.template as<T>(), probs_.template as<T>(), st));
            end(CUBERT_B200_K_BIAS_TANH, 2 * (int64_t) B * H * e + H * e + (int64_t) num_labels * H * e +
                                             2 * (int64_t) B * num_labels * e);
        } else {
            KERNEL_CHECK(K<T>::bias_tanh(pooled_.template as<T>(), pooler_bias_.template as<T>(), B, H, pooled_.template as<T>(), st));
            end(CUBERT_B200_K_BIAS_TANH, 2 * (int64_t) B * H * e + H * e);
        }
    } else {
        begin(CUBERT_B200_K_MEAN_POOL);
        KERNEL_CHECK(K<T>::mean_pool(x, B, S, H, pooled_.template as<T>(), pool_scratch_.get(), pool_scratch_.bytes(), st));
        end(CUBERT_B200_K_MEAN_POOL, R * H * e + (int64_t) B * H * e);
    }

    if (profiling_) {
        // calibration: the same event bracket around NOTHING. What it reads is the least an event pair adds to
        // a figure (the two timestamp commands back to back); a bracketed kernel also pays its own launch gap.
        begin(CUBERT_B200_K_EVENT_OVERHEAD);
        end(CUBERT_B200_K_EVENT_OVERHEAD, 0);
    }

    if (has_classifier_ && !(fuse_heads_ && has_pooler_dense_)) {
        begin(CUBERT_B200_K_LOGITS_PROBS);
        KERNEL_CHECK(K<T>::logits_probs(pooled_.template as<T>(), output_weights_.template as<T>(),
                                        has_classifier_bias_ ? output_bias_.template as<T>() : nullptr, B, H,
                                        (int) num_labels, logits_.template as<T>(), probs_.template as<T>(), st));
        end(CUBERT_B200_K_LOGITS_PROBS,
            (int64_t) B * H * e + (int64_t) num_labels * H * e + 2 * (int64_t) B * num_labels * e);
    }
}

// ------------------------------------------------------------------ outputs
template <typename T>
void Bert<T>::output(size_t batch_size, cuBERT_Output *out, bool to_float) {
    if (batch_size == 0) {
        return;
    }
    CUDA_CHECK(cudaSetDevice(device_));
    const size_t B = batch_size, S = seq_length, H = hidden_size;
    if ((out->logits != nullptr || out->probs != nullptr) && !has_classifier_) {
        // the reference warns and copies from unallocated buffers (src/cuBERT/Bert.cpp:140-142)
        std::cerr << "model does not have additional_output_layer, the output logits is wrong." << std::endl;
    }
    auto copy = [&](void *dst, const T *src, size_t count) {
        if (dst == nullptr || src == nullptr) {
            return;
        }
        if (to_float && Storage<T>::is_half) {
            begin(CUBERT_B200_K_HALF_TO_FLOAT);
            KERNEL_CHECK(cubk_half_to_float(src, float_staging_.template as<float>(), (int64_t) count, stream_));
            end(CUBERT_B200_K_HALF_TO_FLOAT, (int64_t) count * 6);
            CUDA_CHECK(cudaMemcpyAsync(dst, float_staging_.get(), sizeof(float) * count, cudaMemcpyDeviceToHost,
                                       stream_));
        } else {
            CUDA_CHECK(cudaMemcpyAsync(dst, src, sizeof(T) * count, cudaMemcpyDeviceToHost, stream_));
        }
    };
    copy(out->logits, has_classifier_ ? logits_.template as<T>() : nullptr, B * num_labels);
    copy(out->probs, has_classifier_ ? probs_.template as<T>() : nullptr, B * num_labels);
    copy(out->pooled_output, pooled_.template as<T>(), B * H);
    copy(out->sequence_output, sequence_output_, B * S * H);
    copy(out->embedding_output, embedding_.template as<T>(), B * S * H);
    CUDA_CHECK(cudaStreamSynchronize(stream_));
}

// ------------------------------------------------------------------ compute + output with overlapped copies
constexpr size_t kMinOverlapBytes = 8u << 20;   // per-position output below this: the plain path
constexpr size_t kMinChunkedTokens = 16384;      // the tail is split only when every sub-batch stays large

template <typename T>
void Bert<T>::compute_output(size_t batch_size, const int *input_ids, const int8_t *input_mask,
                             const int8_t *segment_ids, cuBERT_Output *out, bool to_float) {
    const bool per_position = out->sequence_output != nullptr || out->embedding_output != nullptr;
    const size_t S = seq_length, H = hidden_size, L = num_hidden_layers;
    const size_t tokens = batch_size * S;
    // worth it when the tail can be split (sequence_output of a large request) or when embedding_output,
    // which is final right after K1, can leave during the whole encoder
    const bool splittable = out->sequence_output != nullptr && tokens >= kMinChunkedTokens && L > 0 && tail_chunks_ > 1;
    if (!per_position || profiling_ || batch_size == 0 || batch_size > max_batch_size ||
        tokens * H * sizeof(T) < kMinOverlapBytes || !(splittable || out->embedding_output != nullptr)) {
        compute(batch_size, input_ids, input_mask, segment_ids, per_position);
        output(batch_size, out, to_float);
        return;
    }
    if (input_ids == nullptr || input_mask == nullptr || segment_ids == nullptr) {
        throw std::invalid_argument("null input");
    }
    CUDA_CHECK(cudaSetDevice(device_));
    if ((out->logits != nullptr || out->probs != nullptr) && !has_classifier_) {
        std::cerr << "model does not have additional_output_layer, the output logits is wrong." << std::endl;
    }
    const bool convert = to_float && Storage<T>::is_half;
    const size_t out_elem = convert ? sizeof(float) : sizeof(T);
    if (convert && out->embedding_output != nullptr && float_staging_embedding_.get() == nullptr) {
        float_staging_embedding_.allocate(sizeof(float) * max_batch_size * S * H);
    }
    if (convert && float_staging_small_.get() == nullptr) {
        float_staging_small_.allocate(sizeof(float) * max_batch_size * (H > num_labels ? H : num_labels));
    }

    upload_inputs(tokens, input_ids, input_mask, segment_ids);
    build_key_plan(batch_size, input_mask);
    const int32_t *d_ids = ids_;
    const int8_t *d_mask = mask_;
    const int8_t *d_seg = segments_;

    // ---- everything that computes goes to the compute stream first ...
    forward_embed(batch_size, d_ids, d_seg, 0);
    sort_attention_pointers(batch_size);
    const void *embedding_src = embedding_.get();
    if (out->embedding_output != nullptr) {
        if (convert) {
            KERNEL_CHECK(cubk_half_to_float(embedding_.get(), float_staging_embedding_.template as<float>(),
                                            (int64_t) (tokens * H), stream_));
            embedding_src = float_staging_embedding_.get();
        }
        CUDA_CHECK(cudaEventRecord(embed_ready_, stream_));
    }
    size_t chunks = 1;
    if (splittable) {
        chunks = (size_t) tail_chunks_ < batch_size ? (size_t) tail_chunks_ : batch_size;
    }
    const size_t tail = chunks > 1 ? ((size_t) tail_layers_ < L ? (size_t) tail_layers_ : L) : 0;
    // Sub-batch boundaries. Only the LAST sub-batch's copy cannot hide behind later work, so it is made
    // smaller than the others: tail_last_percent_ of the batch (CUBERT_TAIL_LAST_PERCENT, default 6; 0 = all
    // sub-batches equal). Measured at 256 x 128 binary16 through cuBERT_compute_m, 40 steps, twice each:
    // 7.40 / 7.40 ms with equal quarters, 7.28 / 7.34 ms with 6 %, 7.33 / 7.36 ms with 12 %.
    size_t chunk_begin[kMaxTailChunks + 1] = {};
    {
        size_t last = chunks > 1 && tail_last_percent_ > 0 ? batch_size * (size_t) tail_last_percent_ / 100 : 0;
        last = last < 1 && tail_last_percent_ > 0 && chunks > 1 ? 1 : last;
        const size_t evenly = last > 0 ? chunks - 1 : chunks;      // sub-batches that share the rest
        const size_t rest = batch_size - last;
        const size_t per_chunk = (rest + evenly - 1) / evenly;
        for (size_t c = 0; c <= evenly; ++c) {
            chunk_begin[c] = c * per_chunk < rest ? c * per_chunk : rest;
        }
        if (last > 0) {
            chunk_begin[chunks] = batch_size;
        }
    }
    if (L - tail > 0) {
        const GraphKey key{batch_size, 0, d_ids, d_mask, d_seg, kHeadLayers, 0, L - tail, plan_key()};
        run_graph(key, [&] { forward_layers(0, L - tail, 0, batch_size, batch_size, d_mask, 0); });
    }
    size_t used = 0;
    for (size_t c = 0; c < chunks; ++c) {
        const size_t b0 = chunk_begin[c];
        const size_t nb = chunk_begin[c + 1] - b0;
        used = c + 1;
        if (nb == 0) {
            continue;
        }
        if (tail > 0) {
            const GraphKey key{batch_size, 0, d_ids, d_mask, d_seg, kTailLayers, b0, nb, plan_key()};
            run_graph(key, [&] { forward_layers(L - tail, L, b0, nb, batch_size, d_mask, 0); });
        }
        if (out->sequence_output != nullptr) {
            if (convert) {
                KERNEL_CHECK(cubk_half_to_float(sequence_output_ + b0 * S * H,
                                                float_staging_.template as<float>() + b0 * S * H,
                                                (int64_t) (nb * S * H), stream_));
            }
            CUDA_CHECK(cudaEventRecord(chunk_ready_[c], stream_));
        }
    }
    {
        const GraphKey key{batch_size, 0, d_ids, d_mask, d_seg, kHeads, 0, 0, 0};
        run_graph(key, [&] { forward_heads(batch_size, d_mask, 0); });
    }
    auto small = [&](void *dst, const T *src, size_t count) {
        if (dst == nullptr || src == nullptr) {
            return;
        }
        if (convert) {
            KERNEL_CHECK(cubk_half_to_float(src, float_staging_small_.template as<float>(), (int64_t) count, stream_));
            CUDA_CHECK(cudaMemcpyAsync(dst, float_staging_small_.get(), sizeof(float) * count, cudaMemcpyDeviceToHost,
                                       stream_));
        } else {
            CUDA_CHECK(cudaMemcpyAsync(dst, src, sizeof(T) * count, cudaMemcpyDeviceToHost, stream_));
        }
    };

    // ---- ... then the large copies on the copy stream, each behind the event that makes its rows final
    // (a copy into pageable memory blocks the calling thread; by now the GPU has all its work)
    if (out->embedding_output != nullptr) {
        CUDA_CHECK(cudaStreamWaitEvent(copy_stream_, embed_ready_, 0));
        CUDA_CHECK(cudaMemcpyAsync(out->embedding_output, embedding_src, tokens * H * out_elem, cudaMemcpyDeviceToHost,
                                   copy_stream_));
    }
    if (out->sequence_output != nullptr) {
        const char *src = convert ? float_staging_.template as<char>() : reinterpret_cast<const char *>(sequence_output_);
        for (size_t c = 0; c < used; ++c) {
            const size_t b0 = chunk_begin[c];
            const size_t nb = chunk_begin[c + 1] - b0;
            if (nb == 0) {
                continue;
            }
            const size_t off = b0 * S * H * out_elem;
            CUDA_CHECK(cudaStreamWaitEvent(copy_stream_, chunk_ready_[c], 0));
            CUDA_CHECK(cudaMemcpyAsync(static_cast<char *>(out->sequence_output) + off, src + off, nb * S * H * out_elem,
                                       cudaMemcpyDeviceToHost, copy_stream_));
        }
    }
    small(out->logits, has_classifier_ ? logits_.template as<T>() : nullptr, batch_size * num_labels);
    small(out->probs, has_classifier_ ? probs_.template as<T>() : nullptr, batch_size * num_labels);
    small(out->pooled_output, pooled_.template as<T>(), batch_size * H);
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    CUDA_CHECK(cudaStreamSynchronize(copy_stream_));
}

template <typename T>
void Bert<T>::synchronize() {
    CUDA_CHECK(cudaSetDevice(device_));
    CUDA_CHECK(cudaStreamSynchronize(stream_));
}

template <typename T>
cuBERT_Output Bert<T>::device_outputs() const {
    cuBERT_Output o;
    o.logits = has_classifier_ ? logits_.get() : nullptr;
    o.probs = has_classifier_ ? probs_.get() : nullptr;
    o.pooled_output = pooled_.get();
    o.sequence_output = sequence_output_;
    o.embedding_output = embedding_.get();
    return o;
}

template class Bert<float>;
template class Bert<__half>;

}  // namespace cubert
