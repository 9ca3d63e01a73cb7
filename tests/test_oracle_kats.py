"""Pin the CPU oracle: every known-answer vector the reference's own unit tests hold for
the fused-kernel path (tests/golden/reference_kats.json, extracted from test/cuBERT/**),
and, where oracle/_ref could be built, the reference's own CPU code on seeded inputs.
CPU only.
"""
import numpy as np
import pytest

from conftest import assert_kat
from cubert_b200 import synthetic


def A(entry, name, dtype=np.float32, shape=None):
    a = np.asarray(entry["arrays"][name], dtype=dtype)
    return a.reshape(shape) if shape else a


# ------------------------------------------------------------------ op-level KATs

def test_embedding_kat(oracle, kats):
    e = kats["op/EmbeddingTest.cpp::embedding"]
    out = oracle.embedding(A(e, "input_ids", np.int32), A(e, "embedding_table", shape=(4, 3)))
    assert_kat(e, out)
    assert np.array_equal(out, A(e, "embedding_table", shape=(4, 3))[[2, 2, 1]])


def test_layer_norm_kat(oracle, kats):
    e = kats["op/LayerNormTest.cpp::layer_norm_ext"]
    out = oracle.layer_norm_(A(e, "in", shape=(2, 3)), A(e, "inout", shape=(2, 3)), A(e, "beta"), A(e, "gamma"))
    assert_kat(e, out)


def test_softmax_kat(oracle, kats):
    e = kats["op/SoftmaxTest.cpp::softmax_"]
    assert_kat(e, oracle.softmax_(A(e, "inout", shape=(2, 3))))


def test_gelu_kat(oracle, kats):
    e = kats["op/GELUTest.cpp::gelu"]
    assert_kat(e, oracle.gelu(A(e, "inout")))


def test_dense_kat(oracle, kats):
    e = kats["op/DenseTest.cpp::dense"]
    # test/cuBERT/op/DenseTest.cpp:5-34: inputs=2, units=3, 3 rows
    out = oracle.dense(A(e, "input", shape=(3, 2)), A(e, "kernel", shape=(2, 3)), A(e, "bias"))
    assert_kat(e, out)


def test_attention_mask_kat(oracle, kats):
    e = kats["op_att/AttentionMaskTest.cpp::attention_mask"]
    out = oracle.attention_mask(A(e, "in", np.int8, (2, 2)), heads=3)
    assert_kat(e, out)


def test_batch_matmul_kats(oracle, kats):
    e = kats["op_att/BatchMatMulTest.cpp::q_k"]
    out = oracle.att_q_k(A(e, "query", shape=(2, 2, 4, 3)), A(e, "key", shape=(2, 2, 4, 3)))
    assert_kat(e, out)
    e = kats["op_att/BatchMatMulTest.cpp::qk_v"]
    out = oracle.att_qk_v(A(e, "qk", shape=(2, 2, 4, 2)), A(e, "value", shape=(2, 2, 4, 3)))
    assert_kat(e, out)


def test_attention_self_kat(oracle, kats):
    e = kats["op_att/AttentionSelfTest.cpp::attention_self"]
    qkv = [A(e, "query_kernel", shape=(6, 6)), A(e, "query_bias"), A(e, "key_kernel", shape=(6, 6)),
           A(e, "key_bias"), A(e, "value_kernel", shape=(6, 6)), A(e, "value_bias")]
    neg = np.zeros(64, np.float32)
    neg[0] = 1  # test/cuBERT/op_att/AttentionSelfTest.cpp:55-57
    out = oracle.attention_self(A(e, "tensor", shape=(8, 6)), qkv, 2, 4, 2, 3, neg)
    assert_kat(e, out)


def _transformer_var(kats, layers):
    g = kats["op_att/TransformerTest.cpp::<globals>"]["arrays"]
    names = {
        "attention/self/query/kernel": ("query_kernel", (6, 6)), "attention/self/query/bias": ("query_bias", None),
        "attention/self/key/kernel": ("key_kernel", (6, 6)), "attention/self/key/bias": ("key_bias", None),
        "attention/self/value/kernel": ("value_kernel", (6, 6)), "attention/self/value/bias": ("value_bias", None),
        "attention/output/dense/kernel": ("attention_output_kernel", (6, 6)),
        "attention/output/dense/bias": ("attention_output_bias", None),
        "attention/output/LayerNorm/beta": ("attention_norm_beta", None),
        "attention/output/LayerNorm/gamma": ("attention_norm_gamma", None),
        "intermediate/dense/kernel": ("intermediate_kernel", (6, 5)),
        "intermediate/dense/bias": ("intermediate_bias", None),
        "output/dense/kernel": ("output_kernel", (5, 6)), "output/dense/bias": ("output_bias", None),
        "output/LayerNorm/beta": ("output_norm_beta", None), "output/LayerNorm/gamma": ("output_norm_gamma", None),
    }
    var = {}
    for l in range(layers):
        for tf_name, (arr, shape) in names.items():
            a = np.asarray(g[arr], np.float32)
            var["encoder/layer_%d/%s" % (l, tf_name)] = a.reshape(shape) if shape else a
    return var


TRANSFORMER_CFG = dict(seq=4, hidden=6, heads=2, intermediate=5)


@pytest.mark.parametrize("test,layers", [("transformer", 1), ("transformer_complex", 2)])
def test_transformer_kats(oracle, kats, test, layers):
    e = kats["op_att/TransformerTest.cpp::" + test]
    var = _transformer_var(kats, layers)
    mask = np.ones((2, 4), np.int8)
    mask[0, 0] = 0  # test/cuBERT/op_att/TransformerTest.cpp:99-101
    cfg = dict(TRANSFORMER_CFG, layers=layers)
    out = oracle.transformer(var, cfg, A(e, "tensor", shape=(8, 6)), mask, prefix="encoder")
    assert_kat(e, out)


def test_bert_embeddings_kat(oracle, kats):
    e = kats["op_bert/BertEmbeddingsTest.cpp::bert_embedding"]
    out = oracle.bert_embeddings(A(e, "input_ids", np.int32, (2, 4)), A(e, "segment_ids", np.int8, (2, 4)),
                                 A(e, "word_embeddings", shape=(5, 3)), A(e, "position_embeddings", shape=(4, 3)),
                                 A(e, "token_type_embeddings", shape=(2, 3)), A(e, "beta"), A(e, "gamma"))
    assert_kat(e, out, float_eq_ulps=4)


def test_pooler_kats(oracle, kats):
    e = kats["op_bert/BertPoolerTest.cpp::bert_pooler"]
    out = oracle.bert_pooler(A(e, "in", shape=(2, 3, 2)), A(e, "kernel", shape=(2, 2)), A(e, "bias"))
    assert_kat(e, out)
    e = kats["op_bert/BertPoolerTest.cpp::mean_pooler"]
    assert_kat(e, oracle.reduce_mean_1(A(e, "in", shape=(2, 3, 2))))


def test_classifier_kat(oracle, kats):
    e = kats["op_out/AdditionalOutputLayerTest.cpp::additional_output"]
    logits, _ = oracle.classifier(A(e, "in", shape=(2, 3)), A(e, "output_weights", shape=(1, 3)), None,
                                  want_probs=False)
    assert_kat(e, logits)


# ------------------------------------------------------------------ the reference's own KATs on oracle/_ref

def test_reference_cpu_reproduces_kats(reference_cpu, kats):
    """Sanity of the _ref build itself: it must pass its own known answers."""
    ref = reference_cpu
    e = kats["op/LayerNormTest.cpp::layer_norm_ext"]
    assert_kat(e, ref.layer_norm_(A(e, "in", shape=(2, 3)), A(e, "inout", shape=(2, 3)), A(e, "beta"), A(e, "gamma")))
    e = kats["op/SoftmaxTest.cpp::softmax_"]
    assert_kat(e, ref.softmax_(A(e, "inout", shape=(2, 3))))
    e = kats["op_att/AttentionMaskTest.cpp::attention_mask"]
    assert_kat(e, ref.attention_mask(A(e, "in", np.int8, (2, 2)), heads=3))
    e = kats["op_bert/BertPoolerTest.cpp::bert_pooler"]
    assert_kat(e, ref.bert_pooler(A(e, "in", shape=(2, 3, 2)), A(e, "kernel", shape=(2, 2)), A(e, "bias")))
    e = kats["op_att/TransformerTest.cpp::transformer_complex"]
    mask = np.ones((2, 4), np.int8)
    mask[0, 0] = 0
    out = ref.transformer(_transformer_var(kats, 2), dict(TRANSFORMER_CFG, layers=2),
                          A(e, "tensor", shape=(8, 6)), mask, prefix="encoder")
    assert_kat(e, out)


# ------------------------------------------------------------------ oracle vs reference on seeded inputs

def _rel(a, b):
    return float(np.max(np.abs(a - b)) / (np.max(np.abs(b)) + 1e-30))


def test_oracle_ops_match_reference_bitwise(oracle, reference_cpu):
    """The scalar ops restate the reference loops exactly: results must be bit-identical."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal((37, 129), dtype=np.float32)
    y = rng.standard_normal((37, 129), dtype=np.float32)
    beta = rng.standard_normal(129, dtype=np.float32)
    gamma = rng.standard_normal(129, dtype=np.float32)
    assert np.array_equal(oracle.layer_norm_(x, y, beta, gamma), reference_cpu.layer_norm_(x, y, beta, gamma))
    s = (rng.standard_normal((53, 33), dtype=np.float32) * 3).astype(np.float32)
    assert np.array_equal(oracle.softmax_(s), reference_cpu.softmax_(s))
    g = (rng.standard_normal(1000, dtype=np.float32) * 3).astype(np.float32)
    assert np.array_equal(oracle.gelu(g), reference_cpu.gelu(g))
    assert np.array_equal(oracle.tanh_(g), reference_cpu.tanh_(g))
    t = rng.standard_normal((5, 7, 19), dtype=np.float32)
    assert np.array_equal(oracle.reduce_mean_1(t), reference_cpu.reduce_mean_1(t))
    table = rng.standard_normal((50, 24), dtype=np.float32)
    ids = rng.integers(0, 50, 91, dtype=np.int32)
    assert np.array_equal(oracle.embedding(ids, table), reference_cpu.embedding(ids, table))
    seg = rng.integers(0, 2, 91).astype(np.int8)
    assert np.array_equal(oracle.embedding(seg, table), reference_cpu.embedding(seg, table))
    m = rng.integers(0, 2, (4, 9)).astype(np.int8)
    assert np.array_equal(oracle.not_(m), reference_cpu.not_(m))
    assert np.array_equal(oracle.attention_mask(m, 3), reference_cpu.attention_mask(m, 3))


def test_oracle_embeddings_match_reference(oracle, reference_cpu):
    cfg = synthetic.config("tiny")
    var = synthetic.random_weights(cfg, 5)
    ids, mask, seg, _ = synthetic.random_inputs(cfg, 6, 24, 5, segments="random")
    args = (ids, seg, var["bert/embeddings/word_embeddings"], var["bert/embeddings/position_embeddings"],
            var["bert/embeddings/token_type_embeddings"],
            np.random.default_rng(1).standard_normal(cfg["hidden"], dtype=np.float32),
            np.random.default_rng(2).standard_normal(cfg["hidden"], dtype=np.float32))
    a, b = oracle.bert_embeddings(*args), reference_cpu.bert_embeddings(*args)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("name,batch,seq,lengths", [
    ("tiny", 5, 16, (3, 16)),
    ("tiny_mean", 3, 48, "full"),
    ("small", 4, 32, (8, 32)),
])
def test_oracle_forward_matches_reference(oracle, reference_cpu, name, batch, seq, lengths):
    """Whole forward pass: identical algorithm, only the GEMM summation order (MKL vs loop
    nest) differs, so agreement is at float32 rounding level."""
    cfg = synthetic.config(name)
    var = synthetic.random_weights(cfg, 7)
    geo = synthetic.model_geometry(cfg, seq)
    ids, mask, seg, _ = synthetic.random_inputs(cfg, batch, seq, 7, lengths=lengths)
    a = oracle.bert_forward(var, geo, ids, mask, seg)
    b = reference_cpu.bert_forward(var, geo, ids, mask, seg)
    assert set(a) == set(b)
    assert np.array_equal(a["embedding_output"], b["embedding_output"])
    for k in a:
        assert _rel(a[k], b[k]) < 2e-6, (k, _rel(a[k], b[k]))
