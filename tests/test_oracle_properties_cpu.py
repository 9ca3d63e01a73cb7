"""The C oracle against an independent float64 NumPy restatement of the same formulas, on randomised
shapes and values (hypothesis, derandomised). The known-answer vectors pin the oracle at a handful of
points; this pins it everywhere else, so that a GPU/oracle disagreement can be attributed."""
import math

import numpy as np
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

SETTINGS = dict(max_examples=80, deadline=None, derandomize=True, database=None,
                suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])
SEED = st.integers(0, 2 ** 31 - 1)
erf = np.vectorize(math.erf)


def rel(got, ref, floor):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), floor)))


@settings(**SETTINGS)
@given(rows=st.integers(1, 12), ch=st.integers(2, 200), seed=SEED)
def test_layer_norm(oracle, rows, ch, seed):
    rng = np.random.default_rng(seed)
    x, r = rng.standard_normal((rows, ch)).astype(np.float32), rng.standard_normal((rows, ch)).astype(np.float32)
    g, b = (1 + 0.2 * rng.standard_normal(ch)).astype(np.float32), rng.standard_normal(ch).astype(np.float32)
    t = x.astype(np.float64) + r
    if np.any(t.std(axis=1) < 0.05):
        return
    mean, var = t.mean(axis=1, keepdims=True), t.var(axis=1, keepdims=True)
    ref = b + g * (t - mean) / np.sqrt(var + 1e-12)          # src/cuBERT/op/LayerNorm.cpp:22-45
    assert rel(oracle.layer_norm_(r, x, b, g), ref, 1.0) < 2e-5


@settings(**SETTINGS)
@given(batch=st.integers(1, 3), heads=st.integers(1, 3), seq=st.integers(1, 40), seed=SEED, scale=st.sampled_from([1.0, 0.125]))
def test_masked_softmax(oracle, batch, heads, seq, seed, scale):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((batch, seq, heads, seq)) * 3).astype(np.float32)
    mask = (rng.random((batch, seq)) < 0.7).astype(np.int8)
    mask[:, 0] = 1
    v = scale * x.astype(np.float64) + np.where(mask[:, None, None, :] == 0, -10000.0, 0.0)   # op_att/AttentionSelf.cpp:58-60
    e = np.exp(v - v.max(axis=-1, keepdims=True))
    ref = e / e.sum(axis=-1, keepdims=True)
    got = oracle.masked_softmax(x, mask, scale)
    assert rel(got, ref, 1e-4) < 2e-5
    assert np.all(got[np.broadcast_to(mask[:, None, None, :] == 0, got.shape)] == 0)


@settings(**SETTINGS)
@given(n=st.integers(1, 500), seed=SEED, spread=st.sampled_from([0.5, 3.0, 8.0]))
def test_gelu_and_tanh(oracle, n, seed, spread):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * spread).astype(np.float32)
    ref = x.astype(np.float64) * 0.5 * (1.0 + erf(x.astype(np.float64) / math.sqrt(2.0)))       # op/GELU.cpp:10-21
    assert rel(oracle.gelu(x), ref, np.maximum(2e-2 * np.abs(x), 1e-3)) < 1e-5
    assert rel(oracle.tanh_(x), np.tanh(x.astype(np.float64)), 1e-3) < 1e-5


@settings(**SETTINGS)
@given(batch=st.integers(1, 4), seq=st.integers(1, 30), hidden=st.integers(1, 70), labels=st.integers(1, 6), seed=SEED)
def test_pooling_and_classifier(oracle, batch, seq, hidden, labels, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, seq, hidden)).astype(np.float32)
    assert rel(oracle.reduce_mean_1(x), x.astype(np.float64).mean(axis=1), 1e-2) < 1e-5          # op_bert/BertPooler.cpp:18-32
    k = (rng.standard_normal((hidden, hidden)) / math.sqrt(hidden)).astype(np.float32)
    kb = rng.standard_normal(hidden).astype(np.float32)
    pooled = np.tanh(x[:, 0, :].astype(np.float64) @ k + kb)                                     # op_bert/BertPooler.cpp:62-77
    got_pooled = oracle.bert_pooler(x, k, kb)
    assert rel(got_pooled, pooled, 1.0) < 1e-5          # a float32 dot product of O(1) terms in front of the tanh
    w = rng.standard_normal((labels, hidden)).astype(np.float32)
    b = rng.standard_normal(labels).astype(np.float32)
    logits = got_pooled.astype(np.float64) @ w.T.astype(np.float64) + b                          # op_out/AdditionalOutputLayer.cpp:44-66
    e = np.exp(logits - logits.max(axis=1, keepdims=True))
    got_logits, got_probs = oracle.classifier(got_pooled, w, b)
    assert rel(got_logits, logits, 1.0) < 2e-5
    assert rel(got_probs, e / e.sum(axis=1, keepdims=True), 1e-2) < 2e-5


@settings(**SETTINGS)
@given(batch=st.integers(1, 4), seq=st.integers(1, 12), hidden=st.integers(2, 64), vocab=st.integers(1, 20), seed=SEED)
def test_embeddings(oracle, batch, seq, hidden, vocab, seed):
    rng = np.random.default_rng(seed)
    word = rng.standard_normal((vocab, hidden)).astype(np.float32)
    pos = rng.standard_normal((seq, hidden)).astype(np.float32)
    typ = rng.standard_normal((2, hidden)).astype(np.float32)
    g, b = (1 + 0.2 * rng.standard_normal(hidden)).astype(np.float32), rng.standard_normal(hidden).astype(np.float32)
    ids = rng.integers(0, vocab, (batch, seq), dtype=np.int32)
    seg = rng.integers(0, 2, (batch, seq)).astype(np.int8)
    t = word[ids].astype(np.float64) + pos[None, :, :] + typ[seg.astype(np.int64)]               # op_bert/BertEmbeddings.cpp:50-66
    if np.any(t.std(axis=-1) < 0.05):
        return
    ref = b + g * (t - t.mean(axis=-1, keepdims=True)) / np.sqrt(t.var(axis=-1, keepdims=True) + 1e-12)
    assert rel(oracle.bert_embeddings(ids, seg, word, pos, typ, b, g), ref, 1.0) < 2e-5
    assert np.array_equal(oracle.embedding(ids.reshape(-1), word), word[ids.reshape(-1)])         # the gather is a copy
