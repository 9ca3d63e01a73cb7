"""The text front end (cuBERT_open_tokenizer / cuBERT_tokenize_compute*): known answers of the
reference's test/cuBERT/tokenization_test.cpp, and the C++ tokenizer against a Python restatement
(oracle/tokenizer_oracle.py, Python's unicodedata in place of utf8proc) on generated text. CPU only
except the last test."""
import random

import numpy as np
import pytest

from cubert_b200 import model
from oracle import tokenizer_oracle as T

# test_vocab.txt of the reference (one token per line; the id is the line number)
VOCAB = ["[UNK]", "[CLS]", "[SEP]", "want", "##want", "##ed", "wa", "un", "runn", "##ing", ","]


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    path = tmp_path_factory.mktemp("vocab") / "vocab.txt"
    path.write_text("\n".join(VOCAB) + "\n")
    t = model.Tokenizer(str(path))
    yield t
    t.close()


def test_known_answers_of_the_reference_tests(tok):
    # tokenization_test.cpp:12-34 full_tokenizer
    pieces = tok.tokenize("UNwantéd,running", 32)
    assert pieces == ["un", "##want", "##ed", ",", "runn", "##ing"]
    ids, mask, seg = tok.encode("UNwantéd,running", None, 10)
    assert list(ids) == [1, 7, 4, 5, 10, 8, 9, 2, 0, 0]
    assert list(mask) == [1] * 8 + [0, 0] and list(seg) == [0] * 10
    # :36-46 chinese
    assert model.basic_tokenize("ah博推zz") == ["ah", "博", "推", "zz"]
    # :48-64 basic_tokenizer_lower
    assert model.basic_tokenize(" \tHeLLo!how  \n Are yoU?  ") == ["hello", "!", "how", "are", "you", "?"]
    assert model.basic_tokenize("Héllo") == ["hello"]
    # :66-78 basic_tokenizer_no_lower
    assert model.basic_tokenize(" \tHeLLo!how  \n Are yoU?  ", do_lower_case=False) == \
        ["HeLLo", "!", "how", "Are", "yoU", "?"]
    # :80-108 wordpiece_tokenizer
    assert tok.tokenize("") == []
    assert tok.tokenize("unwanted running") == ["un", "##want", "##ed", "runn", "##ing"]
    assert tok.tokenize("unwantedX running") == ["[UNK]", "runn", "##ing"]
    # :124-152 character classes, seen through the basic tokenizer
    assert model.basic_tokenize("a b") == ["a", "b"]            # U+00A0 is whitespace
    assert model.basic_tokenize("a\u0005b") == ["ab"]                # U+0005 is a control character: dropped
    assert model.basic_tokenize("a-b$c`d.e") == ["a", "-", "b", "$", "c", "`", "d", ".", "e"]


def test_pairs_and_truncation_match_the_restatement(tok):
    vocab = {t: i for i, t in enumerate(VOCAB)}
    cases = [("unwanted running", "wa , un", 16), ("unwanted " * 10, "running " * 3, 12), ("runn", None, 5),
             ("unwanted " * 10, None, 8), ("", "", 4), ("wa", "unwanted unwanted unwanted", 9)]
    for a, b, seq in cases:
        ids, mask, seg = tok.encode(a, b, seq)
        rid, rmask, rseg = T.encode(a, b, vocab, seq)
        assert list(ids) == rid and list(mask) == rmask and list(seg) == rseg, (a, b, seq)


def _random_text(rng, n):
    pools = [
        "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789",
        " \t\n\r  　",
        "!\"#$%&'()*+,-./:;<=>?@[\\]^_`{|}~—。，¿“",
        "ÉéüñÅİǅẞΑΣЖёệß",
        "中文博推知乎あア한글\U00020000",
        "ְ̧̣́̈ั​‍﻿\u0000�\u0005­",
        "กิकिאا\U0001f600①",
    ]
    return "".join(rng.choice(rng.choice(pools)) for _ in range(n)).replace("\x00", "")


def test_basic_tokenizer_matches_the_restatement_on_generated_text():
    rng = random.Random(7)
    for i in range(400):
        text = _random_text(rng, rng.randint(0, 60))
        for lower in (True, False):
            assert model.basic_tokenize(text, lower) == T.basic_tokenize(text, lower), (repr(text), lower)
        limit = rng.randint(1, 8)
        assert model.basic_tokenize(text, True, limit) == T.basic_tokenize(text, True, limit)


def test_nfd_covers_every_decomposable_code_point():
    """Lower-casing runs NFD first: every code point with a canonical decomposition must come out as
    Python's NFD does (accents then vanish, Hangul falls apart into jamo)."""
    import unicodedata
    for cp in list(range(0xC0, 0x250)) + list(range(0x1E00, 0x1F00)) + [0x0958, 0x0F43, 0x1109A, 0x1D15E, 0xAC01,
                                                                         0xD4DB, 0x2126, 0x212B, 0xFB1D, 0x0344]:
        ch = chr(cp)
        if unicodedata.category(ch)[0] == "C":
            continue
        text = "x" + ch + "y"
        assert model.basic_tokenize(text, True) == T.basic_tokenize(text, True), hex(cp)


def test_errors():
    with pytest.raises(ValueError, match="Unable to open vocab file"):
        model.Tokenizer("/no/such/vocab.txt")
    assert model.basic_tokenize(b"ab\xff\xfecd", True) == []            # malformed UTF-8: nothing, no crash
    assert model.basic_tokenize(b"ab \xff\xfecd", False) == ["ab"]      # what was decoded before the error


@pytest.mark.gpu
def test_tokenize_compute_equals_compute_on_the_encoded_ids(tmp_path):
    """cuBERT_tokenize_compute_m = convert_single_example per row + cuBERT_compute_m (src/cuBERT.cpp:210-280)."""
    from cubert_b200 import frozen_graph, synthetic
    cfg = synthetic.config("tiny", vocab=len(VOCAB))
    var = synthetic.random_weights(cfg, 21)
    path = str(tmp_path / "m.pb")
    frozen_graph.write_frozen_graph(path, var)
    (tmp_path / "vocab.txt").write_text("\n".join(VOCAB) + "\n")
    tk = model.Tokenizer(str(tmp_path / "vocab.txt"))
    m = model.Model(path, 4, 12, cfg["layers"], cfg["heads"])
    text_a = ["UNwantéd,running", "wa", "running unwanted running"]
    text_b = ["wa , un", "unwanted", "wa"]
    rows = [tk.encode(a, b, 12) for a, b in zip(text_a, text_b)]
    ids = np.stack([r[0] for r in rows])
    mask = np.stack([r[1] for r in rows])
    seg = np.stack([r[2] for r in rows])
    want = model.Output()
    want.logits = np.zeros((3, 3), np.float32)
    want.sequence_output = np.zeros((3, 12, 64), np.float32)
    m.compute_m(ids, mask, seg, want)
    got = model.Output()
    got.logits = np.zeros((3, 3), np.float32)
    got.sequence_output = np.zeros((3, 12, 64), np.float32)
    m.tokenize_compute_m(tk, text_a, text_b, got)
    assert np.array_equal(got.logits, want.logits) and np.array_equal(got.sequence_output, want.sequence_output)
    m.close()
    tk.close()


@pytest.mark.gpu
def test_large_batches_are_tokenized_on_several_threads_with_the_same_result(tmp_path, monkeypatch):
    """Batches of 16 texts or more are split over host threads; every row must equal the single-text
    encoding, pairs and single sentences, with CUBERT_TOKENIZER_THREADS at its default and at 1."""
    from cubert_b200 import frozen_graph, synthetic
    cfg = synthetic.config("tiny", vocab=len(VOCAB))
    path = str(tmp_path / "m.pb")
    frozen_graph.write_frozen_graph(path, synthetic.random_weights(cfg, 22))
    (tmp_path / "vocab.txt").write_text("\n".join(VOCAB) + "\n")
    tk = model.Tokenizer(str(tmp_path / "vocab.txt"))
    rng = np.random.default_rng(5)
    pieces = ["un", "want", "wanted", "running", "runn", "wa", ",", "é", "UNwantéd", "x"]
    B, S = 203, 24
    text_a = [" ".join(rng.choice(pieces, size=int(rng.integers(1, 30)))) for _ in range(B)]
    text_b = [" ".join(rng.choice(pieces, size=int(rng.integers(1, 10)))) for _ in range(B)]
    rows = [tk.encode(a, b, S) for a, b in zip(text_a, text_b)]
    ids, mask, seg = (np.stack([r[i] for r in rows]) for i in range(3))
    for threads in (None, "1", "3"):
        if threads is None:
            monkeypatch.delenv("CUBERT_TOKENIZER_THREADS", raising=False)
        else:
            monkeypatch.setenv("CUBERT_TOKENIZER_THREADS", threads)
        m = model.Model(path, B, S, cfg["layers"], cfg["heads"])
        want, got = model.Output(), model.Output()
        want.pooled_output = np.zeros((B, 64), np.float32)
        got.pooled_output = np.zeros((B, 64), np.float32)
        m.compute_m(ids, mask, seg, want)
        m.tokenize_compute_m(tk, text_a, text_b, got)
        assert np.array_equal(got.pooled_output, want.pooled_output), threads
        single = model.Output()
        single.pooled_output = np.zeros((B, 64), np.float32)
        rows_a = [tk.encode(a, None, S) for a in text_a]
        m.compute_m(*(np.stack([r[i] for r in rows_a]) for i in range(3)), single)
        got_a = model.Output()
        got_a.pooled_output = np.zeros((B, 64), np.float32)
        m.tokenize_compute_m(tk, text_a, None, got_a)
        assert np.array_equal(got_a.pooled_output, single.pooled_output), threads
        m.close()
    tk.close()
