#include "tokenizer.h"

#include <algorithm>
#include <cctype>
#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>

namespace cubert {

namespace {

struct CategoryRange {
    uint32_t first, last;
    int value;
};
struct CodePair {
    uint32_t from, to;
};
struct DecompEntry {
    uint32_t cp;
    int offset, length;
};

#include "unicode_tables.inc"

enum { CLS_OTHER = 0, CLS_ZS = 1, CLS_MN = 2, CLS_P = 3, CLS_C = 4 };

template <size_t N>
int range_lookup(const CategoryRange (&table)[N], uint32_t cp) {
    size_t lo = 0, hi = N;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (cp < table[mid].first) {
            hi = mid;
        } else if (cp > table[mid].last) {
            lo = mid + 1;
        } else {
            return table[mid].value;
        }
    }
    return 0;
}

int category_class(uint32_t cp) {
    if (cp < 0x80) {  // ASCII: looked up once per process
        static const struct AsciiClasses {
            unsigned char cls[0x80];
            AsciiClasses() {
                for (uint32_t c = 0; c < 0x80; ++c) {
                    cls[c] = (unsigned char) range_lookup(kCategoryRanges, c);
                }
            }
        } ascii;
        return ascii.cls[cp];
    }
    if (cp >= 0x110000) {
        return CLS_C;
    }
    return range_lookup(kCategoryRanges, cp);
}

// combining class; nothing below U+0300 has one
inline int combining_class(uint32_t cp) {
    return cp < 0x300 ? 0 : range_lookup(kCcc, cp);
}

uint32_t to_lower(uint32_t cp) {
    if (cp < 0x80) {
        return (cp >= 'A' && cp <= 'Z') ? cp + 32 : cp;
    }
    const CodePair *end = kLower + sizeof(kLower) / sizeof(kLower[0]);
    const CodePair *it = std::lower_bound(kLower, end, cp, [](const CodePair &p, uint32_t v) { return p.from < v; });
    return (it != end && it->from == cp) ? it->to : cp;
}

// Decodes one code point; returns the number of bytes used or -1 on malformed input
// (overlong forms, surrogates, values above U+10FFFF and truncated sequences are malformed).
int utf8_decode(const unsigned char *s, size_t n, uint32_t *cp) {
    if (n == 0) {
        return -1;
    }
    const unsigned char c = s[0];
    if (c < 0x80) {
        *cp = c;
        return 1;
    }
    int len;
    uint32_t v, min;
    if ((c & 0xE0) == 0xC0) {
        len = 2, v = c & 0x1F, min = 0x80;
    } else if ((c & 0xF0) == 0xE0) {
        len = 3, v = c & 0x0F, min = 0x800;
    } else if ((c & 0xF8) == 0xF0) {
        len = 4, v = c & 0x07, min = 0x10000;
    } else {
        return -1;
    }
    if ((size_t) len > n) {
        return -1;
    }
    for (int i = 1; i < len; ++i) {
        if ((s[i] & 0xC0) != 0x80) {
            return -1;
        }
        v = (v << 6) | (s[i] & 0x3F);
    }
    if (v < min || v > 0x10FFFF || (v >= 0xD800 && v <= 0xDFFF)) {
        return -1;
    }
    *cp = v;
    return len;
}

void utf8_append(uint32_t cp, std::string *out) {
    if (cp < 0x80) {
        out->push_back((char) cp);
    } else if (cp < 0x800) {
        out->push_back((char) (0xC0 | (cp >> 6)));
        out->push_back((char) (0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
        out->push_back((char) (0xE0 | (cp >> 12)));
        out->push_back((char) (0x80 | ((cp >> 6) & 0x3F)));
        out->push_back((char) (0x80 | (cp & 0x3F)));
    } else {
        out->push_back((char) (0xF0 | (cp >> 18)));
        out->push_back((char) (0x80 | ((cp >> 12) & 0x3F)));
        out->push_back((char) (0x80 | ((cp >> 6) & 0x3F)));
        out->push_back((char) (0x80 | (cp & 0x3F)));
    }
}

void decompose(uint32_t cp, std::u32string *out) {
    if (cp < 0xC0) {  // no canonical decomposition below U+00C0
        out->push_back(cp);
        return;
    }
    // Hangul syllables decompose arithmetically (Unicode chapter 3.12)
    if (cp >= 0xAC00 && cp <= 0xD7A3) {
        const uint32_t s = cp - 0xAC00;
        out->push_back(0x1100 + s / 588);
        out->push_back(0x1161 + (s % 588) / 28);
        if (s % 28 != 0) {
            out->push_back(0x11A7 + s % 28);
        }
        return;
    }
    const DecompEntry *end = kDecomp + sizeof(kDecomp) / sizeof(kDecomp[0]);
    const DecompEntry *it =
        std::lower_bound(kDecomp, end, cp, [](const DecompEntry &e, uint32_t v) { return e.cp < v; });
    if (it != end && it->cp == cp) {
        for (int i = 0; i < it->length; ++i) {
            out->push_back(kDecompPool[it->offset + i]);
        }
    } else {
        out->push_back(cp);
    }
}

inline void trim(std::string &s) {
    s.erase(s.begin(), std::find_if(s.begin(), s.end(), [](unsigned char ch) { return !std::isspace(ch); }));
    s.erase(std::find_if(s.rbegin(), s.rend(), [](unsigned char ch) { return !std::isspace(ch); }).base(), s.end());
}

}  // namespace

bool is_whitespace(uint32_t cp) {
    if (cp == ' ' || cp == '\t' || cp == '\n' || cp == '\r') {
        return true;
    }
    return category_class(cp) == CLS_ZS;
}

bool is_control(uint32_t cp) {
    // tab, newline and carriage return count as whitespace, not control (tokenization.cpp:62-68)
    if (cp == '\t' || cp == '\n' || cp == '\r') {
        return false;
    }
    return category_class(cp) == CLS_C;
}

bool is_punctuation(uint32_t cp) {
    // every non-letter, non-digit ASCII character counts as punctuation (tokenization.cpp:70-81)
    if ((cp >= 33 && cp <= 47) || (cp >= 58 && cp <= 64) || (cp >= 91 && cp <= 96) || (cp >= 123 && cp <= 126)) {
        return true;
    }
    return category_class(cp) == CLS_P;
}

bool is_chinese_char(uint32_t cp) {
    // the CJK ideograph blocks of tokenization.cpp:95-113
    return (cp >= 0x4E00 && cp <= 0x9FFF) || (cp >= 0x3400 && cp <= 0x4DBF) || (cp >= 0x20000 && cp <= 0x2A6DF) ||
           (cp >= 0x2A700 && cp <= 0x2B73F) || (cp >= 0x2B740 && cp <= 0x2B81F) || (cp >= 0x2B820 && cp <= 0x2CEAF) ||
           (cp >= 0xF900 && cp <= 0xFAFF) || (cp >= 0x2F800 && cp <= 0x2FA1F);
}

bool utf8_nfd(const char *text, std::u32string *out) {
    out->clear();
    const unsigned char *s = reinterpret_cast<const unsigned char *>(text);
    size_t n = std::strlen(text);
    while (n > 0) {
        uint32_t cp;
        const int len = utf8_decode(s, n, &cp);
        if (len < 0) {
            return false;
        }
        decompose(cp, out);
        s += len;
        n -= len;
    }
    // canonical ordering: stable sort of every run of non-starters by combining class
    size_t i = 0;
    while (i < out->size()) {
        if (combining_class((*out)[i]) == 0) {
            ++i;
            continue;
        }
        size_t j = i;
        while (j < out->size() && combining_class((*out)[j]) != 0) {
            ++j;
        }
        std::stable_sort(out->begin() + i, out->begin() + j,
                         [](char32_t a, char32_t b) { return combining_class(a) < combining_class(b); });
        i = j;
    }
    return true;
}

// tokenization.cpp:115-185: with lower-casing the text is NFD-normalised first, every code point is
// lower-cased, controls / U+0000 / U+FFFD and (when lower-casing) non-spacing marks are dropped,
// whitespace ends a token, punctuation and CJK ideographs are tokens of their own.
void BasicTokenizer::tokenize(const char *text, std::vector<std::string> *output_tokens, size_t max_length) const {
    std::u32string cps;
    if (do_lower_case_) {
        if (!utf8_nfd(text, &cps)) {
            std::cerr << "UTF-8 decode error: " << text << std::endl;
            return;
        }
    } else {
        const unsigned char *s = reinterpret_cast<const unsigned char *>(text);
        size_t n = std::strlen(text);
        while (n > 0) {
            uint32_t cp;
            const int len = utf8_decode(s, n, &cp);
            if (len < 0) {
                std::cerr << "UTF-8 decode error: " << text << std::endl;
                break;  // what was decoded so far is still tokenized, as in the reference
            }
            cps.push_back(cp);
            s += len;
            n -= len;
        }
    }

    bool new_token = true;
    for (char32_t raw : cps) {
        uint32_t cp = raw;
        if (do_lower_case_) {
            cp = to_lower(cp);
        }
        const int cls = category_class(cp);  // the four tests below are is_control / is_whitespace / is_punctuation
        const bool space_char = cp == ' ' || cp == '\t' || cp == '\n' || cp == '\r';
        const bool ascii_punct = (cp >= 33 && cp <= 47) || (cp >= 58 && cp <= 64) || (cp >= 91 && cp <= 96) ||
                                 (cp >= 123 && cp <= 126);
        if (cp == 0 || cp == 0xfffd || (cls == CLS_C && !space_char)) {
            // dropped
        } else if (do_lower_case_ && cls == CLS_MN) {
            // accent stripped
        } else if (space_char || cls == CLS_ZS) {
            new_token = true;
        } else if (ascii_punct || cls == CLS_P || is_chinese_char(cp)) {
            output_tokens->emplace_back();
            utf8_append(cp, &output_tokens->back());
            new_token = true;
        } else {
            if (new_token) {
                output_tokens->emplace_back();
                new_token = false;
            }
            utf8_append(cp, &output_tokens->back());
        }
        if (output_tokens->size() >= max_length) {
            break;
        }
    }
}

// tokenization.cpp:188-217: greedy longest match first; the length limit counts bytes and the
// candidate ends move byte by byte, as in the reference.
void WordpieceTokenizer::tokenize(const std::string &token, std::vector<std::string> *output_tokens) const {
    if (token.size() > max_input_chars_per_word_) {
        output_tokens->push_back(unk_token_);
        return;
    }
    const size_t mark = output_tokens->size();
    for (size_t start = 0; start < token.size();) {
        bool is_bad = true;
        std::string piece = start > 0 ? "##" : "";
        piece.append(token, start, std::string::npos);  // the longest candidate; one byte shorter every round
        for (size_t end = token.size(); start < end; --end) {
            if (vocab_->count(piece)) {
                is_bad = false;
                output_tokens->push_back(std::move(piece));
                start = end;
                break;
            }
            piece.pop_back();
        }
        if (is_bad) {
            output_tokens->resize(mark);
            output_tokens->push_back(unk_token_);
            return;
        }
    }
}

FullTokenizer::FullTokenizer(const char *vocab_file, bool do_lower_case)
    : basic_(do_lower_case), wordpiece_(&vocab_) {
    std::ifstream file(vocab_file);
    if (!file) {
        throw std::invalid_argument("Unable to open vocab file");
    }
    uint64_t index = 0;
    std::string line;
    while (std::getline(file, line)) {  // tokenization.cpp:38-53: one token per line, id = line number
        trim(line);
        vocab_[line] = index++;
    }
}

void FullTokenizer::tokenize(const char *text, std::vector<std::string> *output_tokens, size_t max_length) const {
    std::vector<std::string> tokens;
    tokens.reserve(max_length);
    basic_.tokenize(text, &tokens, max_length);
    for (const std::string &token : tokens) {
        wordpiece_.tokenize(token, output_tokens);
        if (output_tokens->size() >= max_length) {
            break;
        }
    }
}

uint64_t FullTokenizer::convert_token_to_id(const std::string &token) const {
    auto it = vocab_.find(token);
    if (it == vocab_.end()) {
        std::cerr << "vocab missing key: " << token << std::endl;
        return 0;
    }
    return it->second;
}

void FullTokenizer::encode(size_t max_seq_length, const char *text_a, const char *text_b, int *input_ids,
                           int8_t *input_mask, int8_t *segment_ids) const {
    if (max_seq_length < 3) {
        throw std::invalid_argument("seq_length too short for [CLS] and [SEP]");
    }
    std::vector<std::string> a, b;
    a.reserve(max_seq_length);
    b.reserve(max_seq_length);
    tokenize(text_a, &a, max_seq_length);
    if (text_b != nullptr) {
        tokenize(text_b, &b, max_seq_length);
        // trim the longer of the two, one token at a time, to leave room for [CLS] [SEP] [SEP]
        while (a.size() + b.size() > max_seq_length - 3) {
            if (a.size() > b.size()) {
                a.pop_back();
            } else {
                b.pop_back();
            }
        }
    } else if (a.size() > max_seq_length - 2) {
        a.resize(max_seq_length - 2);
    }

    size_t n = 0;
    auto put = [&](const std::string &token, int8_t segment) {
        input_ids[n] = (int) convert_token_to_id(token);
        segment_ids[n] = segment;
        ++n;
    };
    put("[CLS]", 0);
    for (const std::string &t : a) {
        put(t, 0);
    }
    put("[SEP]", 0);
    if (text_b != nullptr) {
        for (const std::string &t : b) {
            put(t, 1);
        }
        put("[SEP]", 1);
    }
    std::fill_n(input_mask, n, (int8_t) 1);
    std::fill_n(input_ids + n, max_seq_length - n, 0);
    std::fill_n(input_mask + n, max_seq_length - n, (int8_t) 0);
    std::fill_n(segment_ids + n, max_seq_length - n, (int8_t) 0);
}

}  // namespace cubert
