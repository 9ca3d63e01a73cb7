// Replica manager: one Bert per GPU (times CUBERT_NUM_MODELS_PER_GPU), at most one call per replica at a
// time, as the reference's BertM<T> (src/cuBERT/BertM.h:15-45, BertM.cpp:12-121). Dispatch: a call takes the
// replica the rotation deals it when that one is free (so one caller at a time sees the reference's
// round-robin exactly), the next free one in rotation otherwise, and waits, first come first served, for ANY
// replica to come free when all are busy. The reference blocks on the mutex of the dealt replica even while others idle, which
// with more callers than replicas stretched the tail of the serving mix to 11 ms at p99;
// CUBERT_STRICT_ROUND_ROBIN=1 restores that.
// The replicas share nothing on the device and never communicate: the batch dimension is the
// only parallel axis, so there is no collective anywhere.
#pragma once

#include <atomic>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <vector>

#include "bert.h"
#include "frozen_graph.h"

namespace cubert {

template <typename T>
class BertM {
public:
    BertM(const char *model_file, size_t max_batch_size, size_t seq_length, size_t num_hidden_layers,
          size_t num_attention_heads);

    // Single selected output (src/cuBERT/BertM.cpp:65-99). Returns the replica that served the call.
    unsigned int compute(size_t batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids, void *output,
                         cuBERT_OutputType output_type);

    // Every non-NULL field of `output` (src/cuBERT/BertM.cpp:101-121).
    unsigned int compute(size_t batch_size, int *input_ids, int8_t *input_mask, int8_t *segment_ids,
                         cuBERT_Output *output, bool output_to_float);

    size_t replicas() const { return replicas_.size(); }
    Bert<T> *replica(size_t i) { return replicas_.at(i).get(); }

    size_t seq_length;
    size_t max_batch_size;

private:
    FrozenGraph<T> weights_;
    std::vector<std::unique_ptr<Bert<T>>> replicas_;
    // which replicas are serving a call; guarded by pool_mutex_, waited on through pool_cv_
    std::vector<char> busy_;
    std::mutex pool_mutex_;
    std::condition_variable pool_cv_;
    std::deque<uint64_t> waiters_;   // tickets of the callers that wait for a replica, oldest first
    uint64_t next_ticket_ = 0;
    bool strict_round_robin_ = false;
    size_t acquire();
    void release(size_t replica);
    // The reference counts in a uint8_t, which skews the rotation whenever 256 is not a multiple
    // of the replica count (src/cuBERT/BertM.h:44); a wide counter keeps it even.
    std::atomic<uint64_t> calls_;
    // Host-side fault injection for tests: calls routed to this replica fail with a RuntimeError before
    // anything reaches its GPU (CUBERT_INJECT_REPLICA_FAILURE=<replica>; -1, the default, injects nothing).
    int failing_replica = -1;
};

}  // namespace cubert
