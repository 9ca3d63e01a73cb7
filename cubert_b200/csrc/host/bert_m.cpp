#include "bert_m.h"

#include <chrono>
#include <iostream>

namespace cubert {

namespace {
// Name, compute capability, bus id and memory of a GPU, in the form the reference prints them
// (src/cuBERT/common.cpp:117-126).
void describe_device(int device) {
    cudaDeviceProp prop;
    CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
    std::cerr << "Found device " << device << " with properties:\n  name: " << prop.name << " major: " << prop.major
              << " minor: " << prop.minor << "\n  pciBusID: " << prop.pciBusID
              << "\n  totalMemory: " << prop.totalGlobalMem << std::endl;
}
}  // namespace

template <typename T>
BertM<T>::BertM(const char *model_file, size_t max_batch_size_, size_t seq_length_, size_t num_hidden_layers,
                size_t num_attention_heads)
    : seq_length(seq_length_), max_batch_size(max_batch_size_), weights_(model_file), calls_(0) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        (void) cudaGetLastError();
        count = 0;
    }
    if (count == 0) {
        throw std::invalid_argument("No GPU device detected");
    }
    std::cerr << "Found GPU count: " << count << std::endl;
    failing_replica = env_int("CUBERT_INJECT_REPLICA_FAILURE", -1);
    int per_gpu = env_int("CUBERT_NUM_MODELS_PER_GPU", 1);
    if (per_gpu < 1) {
        per_gpu = 1;
    }

    // every array a replica uploads has the size its geometry says, before anything reads it
    weights_.validate(seq_length, num_hidden_layers, num_attention_heads);

    std::unordered_map<std::string, const T *> var;
    for (auto &kv : weights_.var) {
        var[kv.first] = kv.second.data();
    }
    const size_t num_labels = weights_.has("output_weights") ? weights_.num_labels : 0;

    const int total = count * per_gpu;
    replicas_.reserve((size_t) total);
    busy_.assign((size_t) total, 0);
    strict_round_robin_ = env_int("CUBERT_STRICT_ROUND_ROBIN", 0) != 0;
    for (int replica = 0; replica < total; ++replica) {
        const int device = replica % count;  // the replicas of one GPU are spread over the rotation
        const auto t0 = std::chrono::steady_clock::now();
        if (replica < count) {
            describe_device(device);
        }
        replicas_.emplace_back(new Bert<T>(var, max_batch_size, seq_length, weights_.vocab_size,
                                                weights_.type_vocab_size, weights_.hidden_size, num_hidden_layers,
                                                num_attention_heads, weights_.intermediate_size, num_labels,
                                                device));
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0);
        // the reference's progress line (src/cuBERT/BertM.cpp:47-50), kept for tools that parse it
        std::cerr << "device setup: " << device << ". Took " << ms.count() << " milliseconds." << std::endl;
    }
}

template <typename T>
unsigned int BertM<T>::compute(size_t batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                               void *output, cuBERT_OutputType output_type) {
    // the output type selects one field of cuBERT_Output (enum values 0..4, include/cuBERT.h)
    static void *cuBERT_Output::*const kField[] = {&cuBERT_Output::logits, &cuBERT_Output::pooled_output,
                                                   &cuBERT_Output::sequence_output, &cuBERT_Output::embedding_output,
                                                   &cuBERT_Output::probs};
    const int which = (int) output_type;
    if (which < 0 || which >= (int) (sizeof(kField) / sizeof(kField[0]))) {
        throw std::invalid_argument("invalid output type");
    }
    cuBERT_Output out;
    out.*kField[which] = output;
    return compute(batch_size, input_ids, input_mask, segment_ids, &out, false);
}

template <typename T>
unsigned int BertM<T>::compute(size_t batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                               cuBERT_Output *output, bool output_to_float) {
    const size_t choice = acquire();
    struct Release {
        BertM<T> *self;
        size_t replica;
        ~Release() { self->release(replica); }
    } release_on_exit{this, choice};
    Bert<T> *bert = replicas_[choice].get();
    if ((int) choice == failing_replica) {
        throw RuntimeError("injected failure on replica " + std::to_string(choice));
    }
    // Only when no per-position output is wanted may the replica skip padding tokens; when one is
    // wanted, its device-to-host copy overlaps the computation (Bert::compute_output).
    bert->compute_output(batch_size, input_ids, input_mask, segment_ids, output, output_to_float);
    return (unsigned int) choice;
}

// The replica this call may use, marked busy: see the header for the order of preference. Callers that
// have to wait are served first come, first served: a replica that comes free goes to the longest waiter,
// not to whoever asks next (a closed-loop caller that has just released would otherwise take it again
// before any waiter wakes, and starve them: measured, 0.9 s of waiting at four callers on two replicas).
template <typename T>
size_t BertM<T>::acquire() {
    const size_t n = replicas_.size();
    const size_t dealt = (size_t) (calls_.fetch_add(1) % n);
    std::unique_lock<std::mutex> lock(pool_mutex_);
    auto take_free = [&](size_t candidates) -> size_t {
        for (size_t k = 0; k < candidates; ++k) {
            const size_t replica = (dealt + k) % n;
            if (!busy_[replica]) {
                busy_[replica] = 1;
                return replica;
            }
        }
        return n;
    };
    if (strict_round_robin_) {   // the reference's behaviour: wait for the dealt replica, whoever else is free
        size_t replica;
        while ((replica = take_free(1)) == n) {
            pool_cv_.wait(lock);
        }
        return replica;
    }
    if (waiters_.empty()) {
        const size_t replica = take_free(n);
        if (replica != n) {
            return replica;
        }
    }
    const uint64_t ticket = next_ticket_++;
    waiters_.push_back(ticket);
    size_t replica = n;
    pool_cv_.wait(lock, [&] { return waiters_.front() == ticket && (replica = take_free(n)) != n; });
    waiters_.pop_front();
    if (!waiters_.empty()) {
        pool_cv_.notify_all();   // the next in line may find another free replica
    }
    return replica;
}

template <typename T>
void BertM<T>::release(size_t replica) {
    {
        std::lock_guard<std::mutex> lock(pool_mutex_);
        busy_[replica] = 0;
    }
    pool_cv_.notify_all();   // every waiter re-checks; only the one whose turn it is proceeds
}

template class BertM<float>;
template class BertM<__half>;

}  // namespace cubert
