// Host-only harness for the model-file reader and the tokenizer, built by tests/test_host_sanitizers.py
// with -fsanitize=address,undefined. It reads a list of commands from stdin, one per line:
//   graph <float|half> <path>      open a frozen graph; prints "ok <tensors> <checksum>" or "rejected: <why>"
//   model <float|half> <path> <seq_length> <layers> <heads>   open it and check every tensor's size against the
//                                  geometry, as cuBERT_open does before building replicas; "ok" or "rejected: <why>"
//   extents <seq> <granule> <max_groups> <hex of the int8 mask, batch * seq bytes>
//                                  key extents of every row and their grouping; prints "ok e0 e1 ... | order ... | start ... | extent ..."
//   tok <lower 0|1> <vocab path> <max_seq_length> <hex of UTF-8 text>    prints "ok <ids...>" or "rejected: <why>"
// A malformed input must end in "rejected" (a C++ exception), never in a sanitizer report or a crash.
#include <cstdint>
#include <cstdio>
#include <exception>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "frozen_graph.h"
#include "key_extents.h"
#include "runtime.h"
#include "tokenizer.h"

// runtime.cpp names this symbol of the kernel library, which this host-only program does not link
extern "C" const char *cubk_last_cuda_error(void) {
    return "";
}

namespace {

template <typename T>
void open_graph(const std::string &path) {
    cubert::FrozenGraph<T> g(path.c_str());
    double sum = 0.0;
    size_t n = 0;
    for (const auto &kv : g.var) {
        std::vector<float> f(kv.second.size());
        cubert::convert(kv.second.data(), f.data(), f.size());
        for (float v : f) {
            sum += v;
        }
        ++n;
    }
    std::printf("ok %zu %.6e %zu %zu %zu %zu %zu\n", n, sum, g.vocab_size, g.type_vocab_size, g.hidden_size,
                g.intermediate_size, g.num_labels);
}

template <typename T>
void open_model(const std::string &path, size_t seq_length, size_t layers, size_t heads) {
    cubert::FrozenGraph<T> g(path.c_str());
    g.validate(seq_length, layers, heads);
    std::printf("ok\n");
}

std::string unhex(const std::string &h) {
    std::string out;
    for (size_t i = 0; i + 1 < h.size(); i += 2) {
        out.push_back((char) std::stoi(h.substr(i, 2), nullptr, 16));
    }
    return out;
}

}  // namespace

int main() {
    std::string line;
    std::unique_ptr<cubert::FullTokenizer> tokenizer;
    std::string tokenizer_key;
    while (std::getline(std::cin, line)) {
        std::istringstream in(line);
        std::string cmd;
        in >> cmd;
        try {
            if (cmd == "graph") {
                std::string type, path;
                in >> type >> path;
                if (type == "half") {
                    open_graph<__half>(path);
                } else {
                    open_graph<float>(path);
                }
            } else if (cmd == "model") {
                std::string type, path;
                size_t seq_length = 0, layers = 0, heads = 0;
                in >> type >> path >> seq_length >> layers >> heads;
                if (type == "half") {
                    open_model<__half>(path, seq_length, layers, heads);
                } else {
                    open_model<float>(path, seq_length, layers, heads);
                }
            } else if (cmd == "extents") {
                int seq = 0, granule = 0, max_groups = 0;
                std::string hex;
                in >> seq >> granule >> max_groups >> hex;
                const std::string raw = unhex(hex);
                if (seq <= 0 || granule <= 0 || raw.size() % (size_t) seq != 0) {
                    throw std::invalid_argument("bad extents command");
                }
                const size_t batch = raw.size() / (size_t) seq;
                std::vector<int32_t> extents(batch), order(batch);
                std::vector<int> start((size_t) max_groups + 2), group_extent((size_t) max_groups + 1);
                for (size_t b = 0; b < batch; ++b) {
                    extents[b] = cubert::key_extent(reinterpret_cast<const int8_t *>(raw.data()) + b * (size_t) seq, seq, granule);
                }
                const int groups = cubert::group_by_extent(extents.data(), batch, seq, granule, max_groups, order.data(),
                                                           start.data(), group_extent.data());
                std::printf("ok");
                for (int32_t e : extents) std::printf(" %d", e);
                std::printf(" | order");
                for (size_t i = 0; groups > 0 && i < batch; ++i) std::printf(" %d", order[i]);
                std::printf(" | start");
                for (int g = 0; groups > 0 && g <= groups; ++g) std::printf(" %d", start[(size_t) g]);
                std::printf(" | extent");
                for (int g = 0; g < groups; ++g) std::printf(" %d", group_extent[(size_t) g]);
                std::printf("\n");
            } else if (cmd == "tok") {
                int lower = 1;
                std::string vocab, hex;
                size_t max_len = 0;
                in >> lower >> vocab >> max_len >> hex;
                const std::string key = vocab + (lower ? "|1" : "|0");
                if (key != tokenizer_key) {
                    tokenizer.reset(new cubert::FullTokenizer(vocab.c_str(), lower != 0));
                    tokenizer_key = key;
                }
                const std::string text = unhex(hex);
                std::vector<int> ids(max_len);
                std::vector<int8_t> mask(max_len), seg(max_len);
                tokenizer->encode(max_len, text.c_str(), nullptr, ids.data(), mask.data(), seg.data());
                std::printf("ok");
                for (int id : ids) {
                    std::printf(" %d", id);
                }
                std::printf("\n");
            } else if (!cmd.empty()) {
                std::printf("rejected: unknown command\n");
            }
        } catch (const std::exception &e) {
            std::printf("rejected: %s\n", e.what());
        }
        std::fflush(stdout);
    }
    return 0;
}
