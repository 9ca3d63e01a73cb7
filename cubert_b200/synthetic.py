"""Seeded synthetic BERT weights and inputs.

The reference measures on random token ids (benchmark/benchmark_cu.cpp:25-34) and its
test model file is not redistributable, so every whole-model test and benchmark here
uses random-init weights of the named architecture: N(0, 0.02) for every kernel,
embedding table and bias, LayerNorm gamma = 1 and beta = 0. One generator
(``numpy.random.default_rng(seed)``) drives everything so that the CPU checker and the
CUDA path see identical bits.

Variable names and shapes are the TensorFlow ones the reference's loader expects
(src/cuBERT/Bert.cpp:34-47, op_bert/BertEmbeddings.cpp:19-27, op_att/Transformer.cpp:45-103,
op_att/AttentionSelf.cpp:27-44).
"""
import numpy as np

CONFIGS = {
    # BERT-base as the reference's benchmark uses it (vocab 21128 = Chinese BERT)
    "base": dict(layers=12, hidden=768, heads=12, intermediate=3072, vocab=21128,
                 max_position=512, type_vocab=2, num_labels=2, pooler=True),
    # BERT-large with the mean pooler and no classifier head
    "large": dict(layers=24, hidden=1024, heads=16, intermediate=4096, vocab=30522,
                  max_position=512, type_vocab=2, num_labels=0, pooler=False),
    # small geometries for CPU-checkable parity tests
    "tiny": dict(layers=2, hidden=64, heads=4, intermediate=256, vocab=97,
                 max_position=64, type_vocab=2, num_labels=3, pooler=True),
    "tiny_mean": dict(layers=2, hidden=96, heads=3, intermediate=160, vocab=61,
                      max_position=48, type_vocab=2, num_labels=0, pooler=False),
    "small": dict(layers=3, hidden=256, heads=4, intermediate=1024, vocab=1000,
                  max_position=128, type_vocab=2, num_labels=2, pooler=True),
}


def config(name, **overrides):
    cfg = dict(CONFIGS[name])
    cfg.update(overrides)
    return cfg


def random_weights(cfg, seed, std=0.02):
    """name -> float32 array, in a fixed generation order."""
    rng = np.random.default_rng(seed)
    H, I = cfg["hidden"], cfg["intermediate"]

    def normal(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)

    var = {}
    var["bert/embeddings/word_embeddings"] = normal(cfg["vocab"], H)
    var["bert/embeddings/token_type_embeddings"] = normal(cfg["type_vocab"], H)
    var["bert/embeddings/position_embeddings"] = normal(cfg["max_position"], H)
    var["bert/embeddings/LayerNorm/beta"] = np.zeros(H, np.float32)
    var["bert/embeddings/LayerNorm/gamma"] = np.ones(H, np.float32)
    for l in range(cfg["layers"]):
        p = "bert/encoder/layer_%d/" % l
        for name in ("query", "key", "value"):
            var[p + "attention/self/%s/kernel" % name] = normal(H, H)
            var[p + "attention/self/%s/bias" % name] = normal(H)
        var[p + "attention/output/dense/kernel"] = normal(H, H)
        var[p + "attention/output/dense/bias"] = normal(H)
        var[p + "attention/output/LayerNorm/beta"] = np.zeros(H, np.float32)
        var[p + "attention/output/LayerNorm/gamma"] = np.ones(H, np.float32)
        var[p + "intermediate/dense/kernel"] = normal(H, I)
        var[p + "intermediate/dense/bias"] = normal(I)
        var[p + "output/dense/kernel"] = normal(I, H)
        var[p + "output/dense/bias"] = normal(H)
        var[p + "output/LayerNorm/beta"] = np.zeros(H, np.float32)
        var[p + "output/LayerNorm/gamma"] = np.ones(H, np.float32)
    if cfg.get("pooler", True):
        var["bert/pooler/dense/kernel"] = normal(H, H)
        var["bert/pooler/dense/bias"] = normal(H)
    if cfg.get("num_labels", 0) > 0:
        var["output_weights"] = normal(cfg["num_labels"], H)
        var["output_bias"] = normal(cfg["num_labels"])
    return var


def random_inputs(cfg, batch, seq, seed, lengths="full", segments="half"):
    """(input_ids int32 [B,S], input_mask int8 [B,S], segment_ids int8 [B,S], lengths).

    lengths: "full" (mask all ones) or (lo, hi) for a per-sequence valid length uniform in
    [lo, hi] with a prefix mask. segments: "half" (0 for the first S/2 positions, 1 after),
    "zero", or "random".
    """
    rng = np.random.default_rng(seed)
    ids = rng.integers(1, cfg["vocab"], size=(batch, seq), dtype=np.int32)
    if lengths == "full":
        lens = np.full(batch, seq, np.int32)
    else:
        lo, hi = lengths
        lens = rng.integers(lo, hi + 1, size=batch, dtype=np.int32)
    mask = (np.arange(seq, dtype=np.int32)[None, :] < lens[:, None]).astype(np.int8)
    if segments == "half":
        seg = np.broadcast_to((np.arange(seq) >= seq // 2).astype(np.int8), (batch, seq)).copy()
    elif segments == "zero":
        seg = np.zeros((batch, seq), np.int8)
    else:
        seg = rng.integers(0, cfg["type_vocab"], size=(batch, seq), dtype=np.int8)
    return ids, mask, seg, lens


def model_geometry(cfg, seq):
    """The geometry dict the CPU checkers take."""
    return dict(vocab=cfg["vocab"], type_vocab=cfg["type_vocab"], hidden=cfg["hidden"],
                layers=cfg["layers"], heads=cfg["heads"], intermediate=cfg["intermediate"],
                num_labels=max(cfg.get("num_labels", 0), 1), seq=seq)
