// Reader for TensorFlow frozen graphs (GraphDef protobuf), the model format cuBERT_open takes.
//
// Same observable behaviour as the reference's loader (src/cuBERT/tensorflow/Graph.cpp:13-91):
// every node that carries an attribute "value" holding a DT_FLOAT or DT_HALF tensor becomes
// var[node name], converted to the model's storage type with round-to-nearest; vocabulary,
// hidden, intermediate and label sizes are sniffed from four named tensors; a missing file or a
// file without such tensors raises std::invalid_argument. The protobuf wire format is decoded
// by hand (no protobuf library): only GraphDef.node, NodeDef.name/attr, AttrValue.tensor and
// TensorProto.dtype/tensor_shape/tensor_content are read, everything else is skipped.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace cubert {

template <typename T>
class FrozenGraph {
public:
    explicit FrozenGraph(const char *filename);

    std::unordered_map<std::string, std::vector<T>> var;
    std::unordered_map<std::string, std::vector<int64_t>> shape;
    size_t vocab_size = 0;
    size_t type_vocab_size = 0;
    size_t hidden_size = 0;
    size_t intermediate_size = 0;
    size_t num_labels = 1;  // reference default when there is no output_weights (tensorflow/Graph.h:23)

    bool has(const std::string &name) const { return var.count(name) != 0; }

    // Checks that every tensor a BERT of this geometry reads is present with exactly the element count
    // the geometry implies (the shapes in the file and the caller's seq_length, layer and head counts
    // are otherwise taken on trust, and a replica copies `count` elements from each array): throws
    // std::invalid_argument("model file invalid: ...") on the first mismatch. The position table may
    // have more rows than seq_length. The reference does not check (src/cuBERT/Bert.cpp:17-53).
    void validate(size_t seq_length, size_t num_hidden_layers, size_t num_attention_heads) const;
    const T *data(const std::string &name) const;  // throws std::invalid_argument if absent
};

}  // namespace cubert
