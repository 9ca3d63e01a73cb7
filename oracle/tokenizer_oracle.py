"""Python restatement of the reference's BERT tokenizer. TEST INFRASTRUCTURE ONLY.

Follows src/cuBERT/tokenization.cpp (BasicTokenizer::tokenize :115-185, WordpieceTokenizer::tokenize
:188-217, FullTokenizer::tokenize :220-233) and convert_single_example (src/cuBERT.cpp:141-208), with
Python's `unicodedata` standing in for utf8proc (NFD, general category, lower-casing). Pinned by the
known answers of test/cuBERT/tokenization_test.cpp (tests/test_tokenizer.py).
"""
import unicodedata


def _is_whitespace(ch):
    return ch in " \t\n\r" or unicodedata.category(ch) == "Zs"


def _is_control(ch):
    if ch in "\t\n\r":
        return False
    return unicodedata.category(ch).startswith("C")


def _is_punctuation(ch):
    cp = ord(ch)
    if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
        return True
    return unicodedata.category(ch).startswith("P")


def _is_chinese_char(cp):
    return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF or
            0x2A700 <= cp <= 0x2B73F or 0x2B740 <= cp <= 0x2B81F or 0x2B820 <= cp <= 0x2CEAF or
            0xF900 <= cp <= 0xFAFF or 0x2F800 <= cp <= 0x2FA1F)


def _lower(ch):
    lo = ch.lower()
    return lo[0] if lo else ch  # simple (single code point) mapping, as utf8proc_tolower


def basic_tokenize(text, do_lower_case=True, max_length=1 << 30):
    if do_lower_case:
        text = unicodedata.normalize("NFD", text)
    tokens = []
    new_token = True
    for ch in text:
        if do_lower_case:
            ch = _lower(ch)
        cp = ord(ch)
        if cp == 0 or cp == 0xFFFD or _is_control(ch):
            pass
        elif do_lower_case and unicodedata.category(ch) == "Mn":
            pass
        elif _is_whitespace(ch):
            new_token = True
        elif _is_punctuation(ch) or _is_chinese_char(cp):
            tokens.append(ch)
            new_token = True
        elif new_token:
            tokens.append(ch)
            new_token = False
        else:
            tokens[-1] += ch
        if len(tokens) >= max_length:
            break
    return tokens


def wordpiece(token, vocab, unk="[UNK]", max_bytes=200):
    raw = token.encode("utf8")
    if len(raw) > max_bytes:      # the reference compares the byte length (tokenization.cpp:189)
        return [unk]
    out = []
    start = 0
    while start < len(raw):
        end = len(raw)
        piece = None
        while start < end:        # candidate ends move byte by byte, as in the reference
            cand = (b"##" if start > 0 else b"") + raw[start:end]
            try:
                key = cand.decode("utf8")
            except UnicodeDecodeError:
                key = None
            if key is not None and key in vocab:
                piece = key
                break
            end -= 1
        if piece is None:
            return [unk]
        out.append(piece)
        start = end
    return out


def full_tokenize(text, vocab, do_lower_case=True, max_length=1 << 30):
    out = []
    for tok in basic_tokenize(text, do_lower_case, max_length):
        out.extend(wordpiece(tok, vocab))
        if len(out) >= max_length:
            break
    return out


def encode(text_a, text_b, vocab, max_seq_length, do_lower_case=True):
    a = full_tokenize(text_a, vocab, do_lower_case, max_seq_length)
    b = []
    if text_b is not None:
        b = full_tokenize(text_b, vocab, do_lower_case, max_seq_length)
        while len(a) + len(b) > max_seq_length - 3:
            if len(a) > len(b):
                a.pop()
            else:
                b.pop()
    elif len(a) > max_seq_length - 2:
        a = a[:max_seq_length - 2]
    toks = ["[CLS]"] + a + ["[SEP]"]
    segs = [0] * len(toks)
    if text_b is not None:
        toks += b + ["[SEP]"]
        segs += [1] * (len(b) + 1)
    ids = [vocab.get(t, 0) for t in toks]
    n = len(ids)
    pad = max_seq_length - n
    return ids + [0] * pad, [1] * n + [0] * pad, segs + [0] * pad
