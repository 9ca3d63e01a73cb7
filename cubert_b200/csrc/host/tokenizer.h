// BERT text front end: basic tokenization (clean-up, lower-casing with accent stripping, CJK and
// punctuation splitting) followed by greedy longest-match WordPiece, and the packing of one or two
// texts into input_ids / input_mask / segment_ids.
//
// Same behaviour as the reference's tokenizer (src/cuBERT/tokenization.{h,cpp}) and its
// convert_single_example (src/cuBERT.cpp:141-208), written without the utf8proc dependency:
// the Unicode data comes from unicode_tables.inc (see gen_unicode_tables.py). CPU only.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace cubert {

// Character classes as the reference defines them (tokenization.cpp:55-92).
bool is_whitespace(uint32_t cp);
bool is_control(uint32_t cp);
bool is_punctuation(uint32_t cp);
bool is_chinese_char(uint32_t cp);

// Canonical decomposition (NFD) of valid UTF-8; returns false on malformed input.
bool utf8_nfd(const char *text, std::u32string *out);

class BasicTokenizer {
public:
    explicit BasicTokenizer(bool do_lower_case = true) : do_lower_case_(do_lower_case) {}
    // Appends tokens; stops early once `max_length` tokens exist (tokenization.cpp:176-179).
    void tokenize(const char *text, std::vector<std::string> *output_tokens, size_t max_length) const;

private:
    bool do_lower_case_;
};

class WordpieceTokenizer {
public:
    explicit WordpieceTokenizer(const std::unordered_map<std::string, uint64_t> *vocab,
                                std::string unk_token = "[UNK]", size_t max_input_chars_per_word = 200)
        : vocab_(vocab), unk_token_(std::move(unk_token)), max_input_chars_per_word_(max_input_chars_per_word) {}
    void tokenize(const std::string &token, std::vector<std::string> *output_tokens) const;

private:
    const std::unordered_map<std::string, uint64_t> *vocab_;
    std::string unk_token_;
    size_t max_input_chars_per_word_;
};

class FullTokenizer {
public:
    // Throws std::invalid_argument("Unable to open vocab file") as the reference does.
    explicit FullTokenizer(const char *vocab_file, bool do_lower_case = true);

    void tokenize(const char *text, std::vector<std::string> *output_tokens, size_t max_length) const;
    uint64_t convert_token_to_id(const std::string &token) const;  // 0 and a stderr line if missing

    // One example -> one row of ids / mask / segment ids of length max_seq_length:
    // [CLS] a [SEP] (b [SEP]) then zero padding (src/cuBERT.cpp:141-208). text_b may be NULL.
    void encode(size_t max_seq_length, const char *text_a, const char *text_b, int *input_ids, int8_t *input_mask,
                int8_t *segment_ids) const;

private:
    std::unordered_map<std::string, uint64_t> vocab_;
    BasicTokenizer basic_;
    WordpieceTokenizer wordpiece_;
};

}  // namespace cubert
