// Closed-loop serving client for the cuBERT C API, in native code: what the Python driver
// (cubert_b200/serve_bench.py) does with threads that share one interpreter, done with plain threads,
// so that request latency holds nothing but the library and the driver.
//
//   serve_mix <model.pb> <requests> <clients (0 = one per replica)> <seed> <half 0|1>
//             <layers> <heads> <vocab> [seq_length = 32]
//
// The request stream: batch size 1, 8 or 32 with probabilities 0.5 / 0.3 / 0.2, every sequence's valid
// length uniform in [4, seq_length] (prefix mask), token ids uniform in [1, vocab), segment ids 0;
// 2048 distinct requests drawn from std::mt19937_64(seed), cycled. Each client thread takes the next
// request index from a shared counter, calls cuBERT_compute(..., cuBERT_PROBS) and records the call's
// wall time. One in-flight request per replica is the reference's threading contract
// (README.md:181-199, src/cuBERT/BertM.cpp:65-76). Prints one JSON line.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include "cuBERT.h"
#include "cubert_b200.h"

namespace {

struct Request {
    int batch;
    std::vector<int> ids;
    std::vector<int8_t> mask, seg;
};

double percentile(const std::vector<double> &sorted, double p) {
    if (sorted.empty()) {
        return 0.0;
    }
    size_t i = (size_t) (p * (double) sorted.size());
    return sorted[i < sorted.size() ? i : sorted.size() - 1];
}

}  // namespace

int main(int argc, char **argv) {
    if (argc < 9) {
        std::fprintf(stderr, "usage: %s model.pb requests clients seed half layers heads vocab [seq]\n", argv[0]);
        return 2;
    }
    const char *path = argv[1];
    const long requests = std::atol(argv[2]);
    int clients = std::atoi(argv[3]);
    const uint64_t seed = std::strtoull(argv[4], nullptr, 10);
    const int half = std::atoi(argv[5]);
    const int layers = std::atoi(argv[6]), heads = std::atoi(argv[7]), vocab = std::atoi(argv[8]);
    const int seq = argc > 9 ? std::atoi(argv[9]) : 32;
    const cuBERT_ComputeType ct = half ? cuBERT_COMPUTE_HALF : cuBERT_COMPUTE_FLOAT;
    const size_t out_elem = half ? 2 : 4;

    void *model = nullptr;
    if (cubert_b200_open(path, 32, seq, layers, heads, (int) ct, &model) != CUBERT_B200_OK) {
        std::fprintf(stderr, "open failed: %s\n", cubert_b200_last_error());
        return 1;
    }
    cubert_b200_info info;
    cubert_b200_model_info(model, (int) ct, &info);
    if (clients <= 0) {
        clients = info.replicas;
    }

    std::mt19937_64 rng(seed);
    const int distinct = 2048;
    std::vector<Request> reqs((size_t) distinct);
    for (Request &r : reqs) {
        const double u = std::uniform_real_distribution<double>(0.0, 1.0)(rng);
        r.batch = u < 0.5 ? 1 : (u < 0.8 ? 8 : 32);
        r.ids.resize((size_t) r.batch * seq);
        r.mask.assign((size_t) r.batch * seq, 0);
        r.seg.assign((size_t) r.batch * seq, 0);
        for (int b = 0; b < r.batch; ++b) {
            const int len = std::uniform_int_distribution<int>(4, seq)(rng);
            for (int s = 0; s < seq; ++s) {
                r.ids[(size_t) b * seq + s] = std::uniform_int_distribution<int>(1, vocab - 1)(rng);
                r.mask[(size_t) b * seq + s] = s < len ? 1 : 0;
            }
        }
    }

    // warm every replica on every batch size (the first uses of a shape run eagerly, then capture a graph)
    {
        std::vector<unsigned char> out(32 * 2 * out_elem);
        for (int want : {1, 8, 32}) {
            for (Request &r : reqs) {
                if (r.batch == want) {
                    for (int i = 0; i < 3 * info.replicas; ++i) {
                        cuBERT_compute(model, r.batch, r.ids.data(), r.mask.data(), r.seg.data(), out.data(), cuBERT_PROBS, ct);
                    }
                    break;
                }
            }
        }
    }

    std::atomic<long> next(0);
    std::vector<std::vector<double>> lat((size_t) clients);
    std::vector<long> seqs((size_t) clients, 0);
    auto client = [&](int k) {
        std::vector<unsigned char> out(32 * 2 * out_elem);
        lat[(size_t) k].reserve((size_t) (requests / clients + 16));
        for (;;) {
            const long i = next.fetch_add(1);
            if (i >= requests) {
                return;
            }
            Request &r = reqs[(size_t) (i % distinct)];
            const auto t0 = std::chrono::steady_clock::now();
            cuBERT_compute(model, r.batch, r.ids.data(), r.mask.data(), r.seg.data(), out.data(), cuBERT_PROBS, ct);
            const auto t1 = std::chrono::steady_clock::now();
            lat[(size_t) k].push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
            seqs[(size_t) k] += r.batch;
        }
    };
    const auto w0 = std::chrono::steady_clock::now();
    std::vector<std::thread> threads;
    for (int k = 0; k < clients; ++k) {
        threads.emplace_back(client, k);
    }
    for (std::thread &t : threads) {
        t.join();
    }
    const double wall = std::chrono::duration<double>(std::chrono::steady_clock::now() - w0).count();

    std::vector<double> all;
    long total_seqs = 0;
    for (int k = 0; k < clients; ++k) {
        all.insert(all.end(), lat[(size_t) k].begin(), lat[(size_t) k].end());
        total_seqs += seqs[(size_t) k];
    }
    std::sort(all.begin(), all.end());
    double mean = 0.0;
    for (double v : all) {
        mean += v;
    }
    mean /= all.empty() ? 1.0 : (double) all.size();
    std::printf("{\"metric\": \"BERT-base seq%d serving mix\", \"client\": \"native threads\", \"requests\": %ld, "
                "\"clients\": %d, \"replicas\": %d, \"gpus\": %d, \"dtype\": \"%s\", \"sequences_per_s\": %.1f, "
                "\"requests_per_s\": %.1f, \"latency_ms\": {\"p50\": %.4f, \"p90\": %.4f, \"p99\": %.4f, \"p999\": %.4f, "
                "\"mean\": %.4f, \"max\": %.4f}, \"mix\": \"batch 1/8/32 with p 0.5/0.3/0.2, valid length U[4,%d], "
                "seed %llu\", \"wall_s\": %.3f}\n",
                seq, requests, clients, info.replicas, cuBERT_get_gpu_count(), half ? "f16" : "f32",
                (double) total_seqs / wall, (double) requests / wall, percentile(all, 0.5), percentile(all, 0.9),
                percentile(all, 0.99), percentile(all, 0.999), mean, all.empty() ? 0.0 : all.back(), seq,
                (unsigned long long) seed, wall);
    cubert_b200_close(model, (int) ct);
    return 0;
}
