#include "frozen_graph.h"

#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>

#include "runtime.h"

namespace cubert {
namespace {

constexpr int kDtFloat = 1;  // tensorflow/core/framework/types.proto:18
constexpr int kDtHalf = 19;  // tensorflow/core/framework/types.proto:36

struct Malformed {};

// Cursor over a protobuf-encoded byte range.
struct Wire {
    const uint8_t *p;
    const uint8_t *end;

    bool done() const { return p >= end; }

    uint64_t varint() {
        uint64_t v = 0;
        for (int shift = 0; shift < 64; shift += 7) {
            if (p >= end) {
                throw Malformed();
            }
            const uint8_t b = *p++;
            v |= (uint64_t) (b & 0x7f) << shift;
            if ((b & 0x80) == 0) {
                return v;
            }
        }
        throw Malformed();
    }

    // Reads a field key; returns the field number and sets the wire type.
    uint32_t key(int &wire_type) {
        const uint64_t k = varint();
        wire_type = (int) (k & 7);
        return (uint32_t) (k >> 3);
    }

    Wire sub() {  // length-delimited payload
        const uint64_t n = varint();
        if (n > (uint64_t) (end - p)) {
            throw Malformed();
        }
        Wire w{p, p + n};
        p += n;
        return w;
    }

    void skip(int wire_type) {
        switch (wire_type) {
            case 0:
                varint();
                break;
            case 1:
                if (end - p < 8) throw Malformed();
                p += 8;
                break;
            case 2:
                sub();
                break;
            case 5:
                if (end - p < 4) throw Malformed();
                p += 4;
                break;
            default:
                throw Malformed();  // groups are not used by GraphDef
        }
    }
};

struct Tensor {
    int dtype = 0;
    std::vector<int64_t> dims;
    const uint8_t *content = nullptr;
    size_t content_len = 0;
    bool present = false;
};

// TensorShapeProto { repeated Dim dim = 2 { int64 size = 1 } }
void parse_shape(Wire w, std::vector<int64_t> &dims) {
    while (!w.done()) {
        int wt;
        const uint32_t f = w.key(wt);
        if (f == 2 && wt == 2) {
            Wire d = w.sub();
            int64_t size = 0;
            while (!d.done()) {
                int dwt;
                const uint32_t df = d.key(dwt);
                if (df == 1 && dwt == 0) {
                    size = (int64_t) d.varint();
                } else {
                    d.skip(dwt);
                }
            }
            dims.push_back(size);
        } else {
            w.skip(wt);
        }
    }
}

// TensorProto { DataType dtype = 1; TensorShapeProto tensor_shape = 2; bytes tensor_content = 4 }
void parse_tensor(Wire w, Tensor &t) {
    t.present = true;
    while (!w.done()) {
        int wt;
        const uint32_t f = w.key(wt);
        if (f == 1 && wt == 0) {
            t.dtype = (int) w.varint();
        } else if (f == 2 && wt == 2) {
            parse_shape(w.sub(), t.dims);
        } else if (f == 4 && wt == 2) {
            Wire c = w.sub();
            t.content = c.p;
            t.content_len = (size_t) (c.end - c.p);
        } else {
            w.skip(wt);
        }
    }
}

// AttrValue { oneof value { ... TensorProto tensor = 8 ... } }
void parse_attr_value(Wire w, Tensor &t) {
    while (!w.done()) {
        int wt;
        const uint32_t f = w.key(wt);
        if (f == 8 && wt == 2) {
            parse_tensor(w.sub(), t);
        } else {
            w.skip(wt);
        }
    }
}

// NodeDef { string name = 1; map<string, AttrValue> attr = 5 } ; map entry { key = 1; value = 2 }
void parse_node(Wire w, std::string &name, Tensor &value) {
    while (!w.done()) {
        int wt;
        const uint32_t f = w.key(wt);
        if (f == 1 && wt == 2) {
            Wire s = w.sub();
            name.assign(reinterpret_cast<const char *>(s.p), (size_t) (s.end - s.p));
        } else if (f == 5 && wt == 2) {
            Wire entry = w.sub();
            std::string key;
            Wire val{nullptr, nullptr};
            while (!entry.done()) {
                int ewt;
                const uint32_t ef = entry.key(ewt);
                if (ef == 1 && ewt == 2) {
                    Wire s = entry.sub();
                    key.assign(reinterpret_cast<const char *>(s.p), (size_t) (s.end - s.p));
                } else if (ef == 2 && ewt == 2) {
                    val = entry.sub();
                } else {
                    entry.skip(ewt);
                }
            }
            if (key == "value" && val.p != nullptr) {  // only this attribute matters (Graph.cpp:34-36)
                Tensor t;
                parse_attr_value(val, t);
                if (t.present) {
                    value = t;
                }
            }
        } else {
            w.skip(wt);
        }
    }
}

}  // namespace

template <typename T>
FrozenGraph<T>::FrozenGraph(const char *filename) {
    std::ifstream input(filename, std::ios::binary | std::ios::ate);
    if (!input) {
        throw std::invalid_argument("model file not found");
    }
    const std::streamsize size = input.tellg();
    input.seekg(0);
    std::vector<uint8_t> buffer((size_t) (size > 0 ? size : 0));
    if (size > 0 && !input.read(reinterpret_cast<char *>(buffer.data()), size)) {
        throw std::invalid_argument("model file not found");
    }
    input.close();
    std::cerr << "model loaded from: " << filename << std::endl;

    try {
        Wire g{buffer.data(), buffer.data() + buffer.size()};
        while (!g.done()) {
            int wt;
            const uint32_t f = g.key(wt);
            if (!(f == 1 && wt == 2)) {  // GraphDef.node = 1
                g.skip(wt);
                continue;
            }
            std::string name;
            Tensor t;
            parse_node(g.sub(), name, t);
            if (!t.present || (t.dtype != kDtFloat && t.dtype != kDtHalf)) {
                continue;
            }
            std::vector<T> data;
            if (t.dtype == kDtFloat) {
                const size_t len = t.content_len / sizeof(float);
                std::vector<float> tmp(len);
                std::memcpy(tmp.data(), t.content, len * sizeof(float));
                data.resize(len);
                convert(tmp.data(), data.data(), len);
            } else {
                const size_t len = t.content_len / sizeof(__half);
                std::vector<__half> tmp(len);
                std::memcpy(static_cast<void *>(tmp.data()), t.content, len * sizeof(__half));
                data.resize(len);
                convert(tmp.data(), data.data(), len);
            }
            var[name] = std::move(data);
            shape[name] = t.dims;

            // geometry sniffed from tensor shapes (tensorflow/Graph.cpp:65-78)
            auto dim = [&](size_t i) -> size_t { return i < t.dims.size() ? (size_t) t.dims[i] : 0; };
            if (name == "bert/embeddings/word_embeddings") {
                vocab_size = dim(0);
                hidden_size = dim(1);
            } else if (name == "bert/embeddings/token_type_embeddings") {
                type_vocab_size = dim(0);
                hidden_size = dim(1);
            } else if (name == "bert/encoder/layer_0/intermediate/dense/bias") {
                intermediate_size = dim(0);
            } else if (name == "output_weights") {
                num_labels = dim(0);
            }
        }
    } catch (const Malformed &) {
        throw std::invalid_argument("model file invalid");
    }

    if (var.empty()) {
        throw std::invalid_argument("model file invalid");
    }
    std::cerr << "model param: {vocab_size=" << vocab_size << ";type_vocab_size=" << type_vocab_size
              << ";hidden_size=" << hidden_size << ";intermediate_size=" << intermediate_size
              << ";num_labels=" << num_labels << "}" << std::endl;
}

template <typename T>
void FrozenGraph<T>::validate(size_t seq_length, size_t num_hidden_layers, size_t num_attention_heads) const {
    const size_t H = hidden_size, I = intermediate_size;
    auto fail = [](const std::string &why) { throw std::invalid_argument("model file invalid: " + why); };
    if (H == 0 || vocab_size == 0 || type_vocab_size == 0 || seq_length == 0 || num_attention_heads == 0 ||
        H % num_attention_heads != 0 || (num_hidden_layers > 0 && I == 0)) {
        fail("geometry");
    }
    auto count_of = [&](const std::string &name) -> size_t {
        auto it = var.find(name);
        if (it == var.end()) {
            fail("no tensor named " + name);
        }
        return it->second.size();
    };
    auto expect = [&](const std::string &name, size_t count) {
        if (count_of(name) != count) {
            fail(name + " has " + std::to_string(count_of(name)) + " elements, expected " + std::to_string(count));
        }
    };
    expect("bert/embeddings/word_embeddings", vocab_size * H);
    expect("bert/embeddings/token_type_embeddings", type_vocab_size * H);
    const size_t positions = count_of("bert/embeddings/position_embeddings");
    if (positions % H != 0 || positions / H < seq_length) {
        fail("position_embeddings holds " + std::to_string(positions / H) + " rows, seq_length is " +
             std::to_string(seq_length));
    }
    expect("bert/embeddings/LayerNorm/gamma", H);
    expect("bert/embeddings/LayerNorm/beta", H);
    for (size_t l = 0; l < num_hidden_layers; ++l) {
        const std::string p = "bert/encoder/layer_" + std::to_string(l);
        for (const char *which : {"query", "key", "value"}) {
            expect(p + "/attention/self/" + which + "/kernel", H * H);
            expect(p + "/attention/self/" + which + "/bias", H);
        }
        expect(p + "/attention/output/dense/kernel", H * H);
        expect(p + "/attention/output/dense/bias", H);
        expect(p + "/attention/output/LayerNorm/gamma", H);
        expect(p + "/attention/output/LayerNorm/beta", H);
        expect(p + "/intermediate/dense/kernel", H * I);
        expect(p + "/intermediate/dense/bias", I);
        expect(p + "/output/dense/kernel", I * H);
        expect(p + "/output/dense/bias", H);
        expect(p + "/output/LayerNorm/gamma", H);
        expect(p + "/output/LayerNorm/beta", H);
    }
    if (has("bert/pooler/dense/kernel")) {
        expect("bert/pooler/dense/kernel", H * H);
        expect("bert/pooler/dense/bias", H);
    }
    if (has("output_weights")) {
        if (num_labels == 0) {
            fail("output_weights without labels");
        }
        expect("output_weights", num_labels * H);
        if (has("output_bias")) {
            expect("output_bias", num_labels);
        }
    }
}

template <typename T>
const T *FrozenGraph<T>::data(const std::string &name) const {
    auto it = var.find(name);
    if (it == var.end()) {
        throw std::invalid_argument("model file has no tensor named " + name);
    }
    return it->second.data();
}

template class FrozenGraph<float>;
template class FrozenGraph<__half>;

}  // namespace cubert
