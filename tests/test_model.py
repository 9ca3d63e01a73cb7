"""The host library (include/cuBERT.h, include/cubert_b200.h): model-file codec on CPU; whole
forward pass, outputs, error behaviour, replica manager and device-resident entry points on GPU.

Whole-model parity, float32: our result against the reference's own CPU output (golden
fixtures written by tests/golden/make_reference_fixtures.py, plus oracle/_ref run live where
it exists) and against the C oracle. The algorithm is identical; the GEMMs are summed in a
different order by cuBLAS than by MKL, so the bar is 1e-5 relative to the tensor's scale
(see `rel_err`). binary16: weights rounded to binary16, float32 oracle on the rounded weights;
bar 1e-2 absolute on probs and pooled output.
"""
import os
import threading

import numpy as np
import pytest

from cubert_b200 import frozen_graph, model, synthetic
from tests.golden.make_reference_fixtures import CASES, weight_checksum

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel_err(got, ref):
    """max |got - ref| relative to the root-mean-square magnitude of the reference tensor."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(got - ref)) / (np.sqrt(np.mean(ref * ref)) + 1e-30))


@pytest.fixture(scope="module")
def model_files(tmp_path_factory):
    """name -> (path, cfg, var) of frozen graphs holding the seeded fixture models."""
    d = tmp_path_factory.mktemp("models")
    out = {}
    for name, (cfg_name, seed, batch, seq, lengths, segments) in CASES.items():
        cfg = synthetic.config(cfg_name)
        var = synthetic.random_weights(cfg, seed)
        path = str(d / (name + ".pb"))
        frozen_graph.write_frozen_graph(path, var, extra_nodes=["bert/encoder/Reshape", "loss/Softmax"])
        out[name] = (path, cfg, var)
    return out


def golden(name):
    return np.load(os.path.join(GOLDEN, "reference_forward_%s.npz" % name))


# ============================================================================ CPU: model-file codec

def test_frozen_graph_round_trip_python(model_files):
    path, cfg, var = model_files["tiny"]
    back = frozen_graph.read_frozen_graph(path)
    assert set(back) == set(var)
    for k in var:
        assert back[k].dtype == np.float32 and np.array_equal(back[k], var[k])


@pytest.mark.parametrize("ct,dtype", [(model.ComputeType.FLOAT, np.float32), (model.ComputeType.HALF, np.float16)])
def test_frozen_graph_cpp_reader(model_files, ct, dtype):
    """The C++ loader sees every tensor, converts with round-to-nearest and sniffs the geometry
    (src/cuBERT/tensorflow/Graph.cpp:28-79)."""
    for name in ("tiny", "tiny_mean"):
        path, cfg, var = model_files[name]
        g = model.FrozenGraph(path, ct)
        assert g.info["vocab_size"] == cfg["vocab"] and g.info["hidden_size"] == cfg["hidden"]
        assert g.info["type_vocab_size"] == cfg["type_vocab"] and g.info["intermediate_size"] == cfg["intermediate"]
        assert g.info["num_labels"] == cfg["num_labels"] and g.info["has_pooler_dense"] == int(cfg["pooler"])
        for k, v in var.items():
            assert np.array_equal(g.tensor(k), v.astype(dtype).ravel()), k
        with pytest.raises(ValueError):
            g.tensor("no/such/tensor")
        g.close()


def test_frozen_graph_half_file_and_errors(tmp_path):
    cfg = synthetic.config("tiny")
    var = {k: v.astype(np.float16) for k, v in synthetic.random_weights(cfg, 3).items()}
    path = str(tmp_path / "half.pb")
    frozen_graph.write_frozen_graph(path, var)
    g = model.FrozenGraph(path, model.ComputeType.FLOAT)  # DT_HALF file opened as a float32 model
    assert np.array_equal(g.tensor("output_bias"), var["output_bias"].astype(np.float32))
    g.close()
    with pytest.raises(ValueError, match="model file not found"):
        model.FrozenGraph(str(tmp_path / "missing.pb"))
    (tmp_path / "empty.pb").write_bytes(b"")
    with pytest.raises(ValueError, match="model file invalid"):
        model.FrozenGraph(str(tmp_path / "empty.pb"))
    (tmp_path / "garbage.pb").write_bytes(b"\x0a\xff\xff\xff\xff\x0f not a graph")
    with pytest.raises(ValueError, match="model file invalid"):
        model.FrozenGraph(str(tmp_path / "garbage.pb"))


def test_golden_fixtures_match_the_weight_generator():
    for name, (cfg_name, seed, batch, seq, lengths, segments) in CASES.items():
        g = golden(name)
        cfg = synthetic.config(cfg_name)
        assert abs(float(g["weight_checksum"]) - weight_checksum(synthetic.random_weights(cfg, seed))) < 1e-9
        ids, mask, seg, _ = synthetic.random_inputs(cfg, batch, seq, seed, lengths=lengths, segments=segments)
        assert np.array_equal(g["ids"], ids) and np.array_equal(g["mask"], mask) and np.array_equal(g["seg"], seg)


def test_oracle_reproduces_reference_fixtures(oracle):
    """The C oracle against the reference's recorded outputs (runs without the reference tree)."""
    for name, (cfg_name, seed, batch, seq, lengths, segments) in CASES.items():
        g = golden(name)
        cfg = synthetic.config(cfg_name)
        out = oracle.bert_forward(synthetic.random_weights(cfg, seed), synthetic.model_geometry(cfg, seq),
                                  g["ids"], g["mask"], g["seg"])
        for k, v in out.items():
            assert rel_err(v, g[k]) < 5e-6, (name, k)


# ============================================================================ GPU: whole model

def _run(m, ids, mask, seg, cfg, to_float=False):
    b, s = ids.shape
    h = cfg["hidden"]
    dt = np.float32 if (to_float or m.dtype == np.float32) else np.float16
    out = model.Output()
    out.embedding_output = np.zeros((b, s, h), dt)
    out.sequence_output = np.zeros((b, s, h), dt)
    out.pooled_output = np.zeros((b, h), dt)
    if m.info["num_labels"] > 0:
        out.logits = np.zeros((b, m.info["num_labels"]), dt)
        out.probs = np.zeros((b, m.info["num_labels"]), dt)
    m.compute_m(ids, mask, seg, out, output_to_float=to_float)
    return {f: getattr(out, f) for f in model.Output.FIELDS if getattr(out, f) is not None}


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_forward_f32_matches_reference(model_files, oracle, name):
    path, cfg, var = model_files[name]
    g = golden(name)
    ids, mask, seg = g["ids"], g["mask"], g["seg"]
    m = model.Model(path, ids.shape[0] + 3, ids.shape[1], cfg["layers"], cfg["heads"], model.ComputeType.FLOAT)
    assert m.info["hidden_size"] == cfg["hidden"] and m.info["num_labels"] == cfg["num_labels"]
    got = _run(m, ids, mask, seg, cfg)
    ref = oracle.bert_forward(var, synthetic.model_geometry(cfg, ids.shape[1]), ids, mask, seg)
    assert set(got) == {k for k in g.files if k not in ("ids", "mask", "seg", "weight_checksum")}
    # embeddings involve no GEMM: 1e-5 of the element itself (floor at the tensor scale * 1e-0)
    assert rel_err(got["embedding_output"], g["embedding_output"]) < 1e-5
    for k in got:
        assert rel_err(got[k], g[k]) < 1e-5, (k, rel_err(got[k], g[k]))      # the reference's own output
        assert rel_err(got[k], ref[k]) < 1e-5, (k, rel_err(got[k], ref[k]))  # the C oracle
    m.close()


@pytest.mark.gpu
def test_forward_f32_matches_reference_live(model_files, reference_cpu):
    """Same comparison with oracle/_ref executed now, on a batch the fixtures do not hold."""
    path, cfg, var = model_files["small"]
    ids, mask, seg, _ = synthetic.random_inputs(cfg, 7, 32, 123, lengths=(1, 32), segments="random")
    m = model.Model(path, 8, 32, cfg["layers"], cfg["heads"], model.ComputeType.FLOAT)
    got = _run(m, ids, mask, seg, cfg)
    ref = reference_cpu.bert_forward(var, synthetic.model_geometry(cfg, 32), ids, mask, seg)
    for k in got:
        assert rel_err(got[k], ref[k]) < 1e-5, (k, rel_err(got[k], ref[k]))
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_forward_f16_within_tolerance(model_files, oracle, name):
    path, cfg, var = model_files[name]
    g = golden(name)
    ids, mask, seg = g["ids"], g["mask"], g["seg"]
    var16 = {k: v.astype(np.float16).astype(np.float32) for k, v in var.items()}
    ref = oracle.bert_forward(var16, synthetic.model_geometry(cfg, ids.shape[1]), ids, mask, seg)
    m = model.Model(path, ids.shape[0], ids.shape[1], cfg["layers"], cfg["heads"], model.ComputeType.HALF)
    raw = _run(m, ids, mask, seg, cfg)                      # binary16 outputs
    conv = _run(m, ids, mask, seg, cfg, to_float=True)      # converted on the device
    for k in raw:
        assert raw[k].dtype == np.float16 and conv[k].dtype == np.float32
        assert np.array_equal(raw[k].astype(np.float32), conv[k]), k
    # embeddings: the reference accepts 3e-4 (test/cuBERT/BertTest.cpp:96-101); outputs are O(1)
    assert np.max(np.abs(conv["embedding_output"] - ref["embedding_output"])) < 4e-3
    # encoder output: the reference accepts up to 1e-2 after 2 layers (op_att/TransformerTest.cpp:330-341)
    assert np.max(np.abs(conv["sequence_output"] - ref["sequence_output"])) < 3e-2
    assert np.max(np.abs(conv["pooled_output"] - ref["pooled_output"])) < 1e-2
    if "probs" in conv:
        assert np.max(np.abs(conv["probs"] - ref["probs"])) < 1e-2
        assert np.max(np.abs(conv["logits"] - ref["logits"])) < 1e-2
    m.close()


@pytest.mark.gpu
def test_single_output_api_and_repeatability(model_files):
    """cuBERT_compute with each cuBERT_OutputType; four consecutive calls give identical results
    (test/cuBERT/BertMTest.cpp:5-38 checks that the round-robin and buffer reuse do not leak state)."""
    path, cfg, var = model_files["tiny"]
    g = golden("tiny")
    ids, mask, seg = g["ids"], g["mask"], g["seg"]
    b, s = ids.shape
    m = model.Model(path, 8, s, cfg["layers"], cfg["heads"])
    shapes = {model.OutputType.LOGITS: ("logits", (b, 3)), model.OutputType.PROBS: ("probs", (b, 3)),
              model.OutputType.POOLED_OUTPUT: ("pooled_output", (b, 64)),
              model.OutputType.SEQUENCE_OUTPUT: ("sequence_output", (b, s, 64)),
              model.OutputType.EMBEDDING_OUTPUT: ("embedding_output", (b, s, 64))}
    for ot, (key, shape) in shapes.items():
        first = None
        for _ in range(4):
            out = np.zeros(shape, np.float32)
            m.compute(ids, mask, seg, out, ot)
            assert rel_err(out, g[key]) < 1e-5
            if first is None:
                first = out
            assert np.array_equal(out, first)
    # a smaller batch after a larger one must not see stale rows
    out = np.zeros((2, 3), np.float32)
    m.compute(ids[:2].copy(), mask[:2].copy(), seg[:2].copy(), out, model.OutputType.LOGITS)
    assert rel_err(out, g["logits"][:2]) < 1e-5
    m.close()


@pytest.mark.gpu
def test_error_behaviour(model_files, tmp_path):
    """What the reference reports as std::invalid_argument (src/cuBERT/Bert.cpp:100-103,
    BertM.cpp:95, tensorflow/Graph.cpp:18,84)."""
    path, cfg, var = model_files["tiny"]
    with pytest.raises(ValueError, match="model file not found"):
        model.Model(str(tmp_path / "nope.pb"), 4, 16, 2, 4)
    partial = {k: v for k, v in var.items() if "layer_1" not in k}
    frozen_graph.write_frozen_graph(str(tmp_path / "partial.pb"), partial)
    with pytest.raises(ValueError, match="layer_1"):
        model.Model(str(tmp_path / "partial.pb"), 4, 16, 2, 4)
    m = model.Model(path, 4, 16, cfg["layers"], cfg["heads"])
    ids, mask, seg, _ = synthetic.random_inputs(cfg, 5, 16, 0)
    out = np.zeros((5, 3), np.float32)
    with pytest.raises(ValueError, match="batch_size > max_batch_size"):
        m.compute(ids, mask, seg, out)
    with pytest.raises(ValueError, match="invalid output type"):
        m.compute(ids[:4].copy(), mask[:4].copy(), seg[:4].copy(), out, 17)
    # batch 0 returns silently and writes nothing
    sentinel = np.full((1, 3), 7.0, np.float32)
    m.compute(ids[:0].copy(), mask[:0].copy(), seg[:0].copy(), sentinel)
    assert np.all(sentinel == 7.0)
    # the model is still usable after the errors
    ok = np.zeros((4, 3), np.float32)
    m.compute(ids[:4].copy(), mask[:4].copy(), seg[:4].copy(), ok)
    assert np.all(np.isfinite(ok)) and np.any(ok != 0)
    m.close()


@pytest.mark.gpu
def test_a_failing_replica_does_not_stop_the_others(model_files, oracle, monkeypatch):
    """Failure made on the host (no GPU fault): with three replicas on the GPU and replica 1 set to fail,
    every third call reports a runtime error through the status API, the other calls keep giving the
    right answers, and the model closes cleanly."""
    path, cfg, var = model_files["tiny"]
    monkeypatch.setenv("CUBERT_NUM_MODELS_PER_GPU", "3")
    monkeypatch.setenv("CUBERT_INJECT_REPLICA_FAILURE", "1")
    m = model.Model(path, 4, 16, cfg["layers"], cfg["heads"])
    replicas = m.info["replicas"]
    assert replicas % 3 == 0
    ids, mask, seg, _ = synthetic.random_inputs(cfg, 4, 16, 3, lengths=(2, 16))
    ref = oracle.bert_forward(var, synthetic.model_geometry(cfg, 16), ids, mask, seg)
    outcomes = []
    for call in range(4 * replicas):
        out = np.zeros((4, cfg["num_labels"]), np.float32)
        try:
            m.compute(ids, mask, seg, out, model.OutputType.PROBS)
            assert rel_err(out, ref["probs"]) < 1e-5
            outcomes.append("ok")
        except RuntimeError as e:
            assert "injected failure on replica 1" in str(e)
            outcomes.append("failed")
    assert outcomes == [("failed" if c % replicas == 1 else "ok") for c in range(4 * replicas)]
    m.close()


@pytest.mark.gpu
def test_device_resident_forward_and_profile(model_files):
    import torch
    path, cfg, var = model_files["small"]
    g = golden("small")
    ids, mask, seg = g["ids"], g["mask"], g["seg"]
    b, s = ids.shape
    m = model.Model(path, b, s, cfg["layers"], cfg["heads"])
    want = _run(m, ids, mask, seg, cfg)
    m.profile_read()  # clear counters
    m.profile_enable(True)
    d_ids, d_mask, d_seg = (torch.from_numpy(a).cuda() for a in (ids, mask, seg))
    torch.cuda.synchronize()
    m.forward_device(0, b, d_ids.data_ptr(), d_mask.data_ptr(), d_seg.data_ptr())
    m.synchronize(0)
    prof = m.profile_read()
    m.profile_enable(False)
    L = cfg["layers"]
    assert prof["embed_ln"]["launches"] == 1 and prof["bias_residual_ln"]["launches"] == 2 * L
    assert prof["bias_gelu"]["launches"] == L and prof["masked_softmax"]["launches"] == L
    # pooler activation and the two-label classifier run as one launch, counted with the former
    assert prof["bias_tanh"]["launches"] == 1 and prof["logits_probs"]["launches"] == 0
    # a request this small runs each layer's attention as one launch (counted with the softmax) in place of the
    # two batched products: four library products per layer, not six
    small = s <= 64 and cfg["hidden"] == 64 * cfg["heads"] and b * s <= 512
    assert prof["gemm"]["launches"] == (4 if small else 6) * L + 1 and prof["event_overhead"]["launches"] == 1
    assert prof["bias_gelu"]["ms"] > 0
    assert prof["bias_gelu"]["bytes"] == L * (2 * b * s * cfg["intermediate"] * 4 + cfg["intermediate"] * 4)
    # the results stayed in the replica's device buffers
    ptrs = m.device_outputs(0)
    import gpu_harness as G
    seq_out = G.copy_from_device(ptrs["sequence_output"], (b, s, cfg["hidden"]), np.float32)
    assert np.array_equal(seq_out, want["sequence_output"])
    probs = G.copy_from_device(ptrs["probs"], (b, cfg["num_labels"]), np.float32)
    assert np.array_equal(probs, want["probs"])
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("per_gpu,strict", [("1", "0"), ("3", "0"), ("3", "1")])
def test_concurrent_callers_are_serialised_per_replica(model_files, per_gpu, strict, monkeypatch):
    """Several threads on one model, more threads than replicas: every call must return the right answer
    (src/cuBERT/BertM.cpp:69-76 locks the chosen replica; here a caller takes any free replica and waits only
    when all are busy, or, with CUBERT_STRICT_ROUND_ROBIN=1, waits for the replica the rotation dealt it)."""
    monkeypatch.setenv("CUBERT_NUM_MODELS_PER_GPU", per_gpu)
    monkeypatch.setenv("CUBERT_STRICT_ROUND_ROBIN", strict)
    path, cfg, var = model_files["tiny"]
    g = golden("tiny")
    ids, mask, seg, want = g["ids"], g["mask"], g["seg"], g["probs"]  # read the archive before threading
    m = model.Model(path, 8, ids.shape[1], cfg["layers"], cfg["heads"])
    errors = []

    def worker(k):
        try:
            for _ in range(10):
                n = 1 + (k % ids.shape[0])
                out = np.zeros((n, 3), np.float32)
                m.compute(ids[:n].copy(), mask[:n].copy(), seg[:n].copy(), out, model.OutputType.PROBS)
                if rel_err(out, want[:n]) > 1e-5:
                    errors.append((k, rel_err(out, want[:n])))
        except Exception as e:  # pragma: no cover
            errors.append((k, repr(e)))

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("ct", [model.ComputeType.FLOAT, model.ComputeType.HALF])
def test_padding_is_skipped_without_changing_the_results(model_files, oracle, ct):
    """When only pooled_output / logits / probs are asked for, the library works on the non-padding
    tokens only. A masked position never influences an unmasked one, so the answers must be those of
    the full computation -- including masks that are not prefixes and a masked first position."""
    path, cfg, var = model_files["small"]
    B, S = 64, 32       # 2048 positions: the smallest request the library packs
    rng = np.random.default_rng(17)
    ids, _, seg, _ = synthetic.random_inputs(cfg, B, S, 17, segments="random")
    mask = np.zeros((B, S), np.int8)
    for b in range(B):
        keep = rng.choice(S, size=rng.integers(2, 12), replace=False)
        mask[b, keep] = rng.integers(1, 5, size=keep.size)      # scattered, any non-zero value
    mask[3, 0] = 0                                               # first token masked as a key, still pooled
    mask[5, :] = 0
    mask[5, 7] = 1
    dt = np.float32 if ct == model.ComputeType.FLOAT else np.float16
    m = model.Model(path, B, S, cfg["layers"], cfg["heads"], ct)

    def heads_only():
        out = model.Output()
        out.pooled_output = np.zeros((B, cfg["hidden"]), dt)
        out.logits = np.zeros((B, 2), dt)
        out.probs = np.zeros((B, 2), dt)
        m.compute_m(ids, mask, seg, out)
        return out

    m.profile_read()
    m.profile_enable(True)
    packed = heads_only()
    prof = m.profile_read()
    m.profile_enable(False)
    kept = int(np.count_nonzero(mask[:, 1:])) + B
    step = max(64, (B * S // 16 + 63) // 64 * 64)      # packed lengths come in sixteenths of the request
    rows = (kept + step - 1) // step * step
    assert rows < B * S
    e = 4 if ct == model.ComputeType.FLOAT else 2
    # packed rows in every layer but the last, which runs on the B first tokens only
    assert prof["bias_gelu"]["bytes"] == (cfg["layers"] - 1) * (2 * rows * cfg["intermediate"] * e + cfg["intermediate"] * e) + \
        (2 * B * cfg["intermediate"] * e + cfg["intermediate"] * e)

    full = _run(m, ids, mask, seg, cfg)                         # asks for sequence_output: no skipping
    tol = 1e-5 if ct == model.ComputeType.FLOAT else 4e-3
    for k in ("pooled_output", "logits", "probs"):
        assert rel_err(getattr(packed, k), full[k]) < tol, k
    again = heads_only()                                         # replayed from the captured graph
    for k in ("pooled_output", "logits", "probs"):
        assert np.array_equal(getattr(again, k), getattr(packed, k))
    if ct == model.ComputeType.FLOAT:
        ref = oracle.bert_forward(var, synthetic.model_geometry(cfg, S), ids, mask, seg)
        for k in ("pooled_output", "logits", "probs"):
            assert rel_err(getattr(packed, k), ref[k]) < 1e-5, k
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("ct", [model.ComputeType.FLOAT, model.ComputeType.HALF])
def test_a_sequence_without_any_kept_key_is_not_packed(model_files, oracle, ct):
    """A mask row of zeros (the empty rows that fill a fixed batch): the reference gives every key of that
    sequence the same -10000, i.e. uniform attention over ALL its positions, so none may be dropped. The
    request must give what the full pass gives, also right after a different request has left its rows in
    the replica's buffers."""
    path, cfg, var = model_files["small"]
    B, S = 64, 32
    rng = np.random.default_rng(29)
    ids, full_mask, seg, _ = synthetic.random_inputs(cfg, B, S, 29, lengths="full", segments="random")
    ids2, _, seg2, _ = synthetic.random_inputs(cfg, B, S, 31, segments="random")
    mask = np.zeros((B, S), np.int8)
    for b in range(B):
        mask[b, :rng.integers(2, 9)] = 1
    mask[7, :] = 0
    mask[40, :] = 0
    dt = np.float32 if ct == model.ComputeType.FLOAT else np.float16
    m = model.Model(path, B, S, cfg["layers"], cfg["heads"], ct)
    full = _run(m, ids2, mask, seg2, cfg)          # every position computed: the answer to match
    _run(m, ids, full_mask, seg, cfg)              # a different request: its rows stay behind in the buffers
    out = model.Output()
    out.pooled_output = np.zeros((B, cfg["hidden"]), dt)
    out.probs = np.zeros((B, 2), dt)
    m.compute_m(ids2, mask, seg2, out)             # pooled outputs only: the request that may skip padding
    tol = 1e-5 if ct == model.ComputeType.FLOAT else 4e-3
    assert rel_err(out.pooled_output, full["pooled_output"]) < tol
    assert rel_err(out.probs, full["probs"]) < tol
    if ct == model.ComputeType.FLOAT:
        ref = oracle.bert_forward(var, synthetic.model_geometry(cfg, S), ids2, mask, seg2)
        assert rel_err(out.pooled_output, ref["pooled_output"]) < 1e-5
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("ct", [model.ComputeType.FLOAT, model.ComputeType.HALF])
@pytest.mark.parametrize("batch", [24, 130])     # 130 x 128 positions: per-position outputs leave in sub-batches
@pytest.mark.parametrize("how", ["softmax_only", "products_too", "one_launch"])
def test_masked_key_columns_are_left_out_of_the_attention(model_files, oracle, ct, batch, how, monkeypatch):
    """With the mask visible on the host, the softmax (and with CUBERT_KEY_GEMM=1 the two attention products as
    well, per group of sequences) works only on the key columns below each sequence's last kept key, rounded
    up to 8 (32 with the products). Those columns carry probability exactly 0 in the full computation, so every
    output must be what the library gives with the feature off -- for ragged prefixes, masks with holes, a full
    sequence, a sequence without any kept key -- eagerly, captured and replayed, for per-position requests,
    pooled-only requests and device-resident inputs."""
    # "one_launch": binary16 models of up to 128 positions run the attention as one kernel, which finds each
    # sequence's last kept key itself and neither loads nor multiplies the keys behind it
    if how == "one_launch" and ct == model.ComputeType.FLOAT:
        pytest.skip("binary16 only")
    products_too = "1" if how == "products_too" else "0"
    monkeypatch.setenv("CUBERT_KEY_GEMM", products_too)
    monkeypatch.setenv("CUBERT_SMALL_ATTENTION", "0")
    step = 32 if products_too == "1" else 8
    import torch
    path, cfg, var = model_files["small"]
    S = 128
    rng = np.random.default_rng(41 + batch)
    ids, mask, seg, _ = synthetic.random_inputs(cfg, batch, S, 41, lengths=(1, S), segments="random")
    mask[0, :] = 1                                   # a full sequence
    mask[1, :] = 0                                   # no kept key at all: uniform attention over every position
    mask[2, :] = 0
    mask[2, [3, 40, 77]] = [1, 9, -3]                # holes; any non-zero value keeps
    mask[3, :] = 0
    mask[3, 0] = 1                                   # a single kept key
    dt = np.float32 if ct == model.ComputeType.FLOAT else np.float16
    tol = 1e-5 if ct == model.ComputeType.FLOAT else 4e-3

    monkeypatch.setenv("CUBERT_SKIP_MASKED_KEYS", "0")
    plain = model.Model(path, batch, S, cfg["layers"], cfg["heads"], ct)
    want = _run(plain, ids, mask, seg, cfg)
    mask_b = mask.copy()
    mask_b[1, 5] = 1                                 # every sequence keeps a key: pooled-only requests get packed
    want_b = _run(plain, ids, mask_b, seg, cfg)
    plain.close()
    monkeypatch.delenv("CUBERT_SKIP_MASKED_KEYS")
    if how == "one_launch":
        monkeypatch.delenv("CUBERT_SMALL_ATTENTION")

    m = model.Model(path, batch, S, cfg["layers"], cfg["heads"], ct)
    for _ in range(3):                               # eager, captured, replayed
        got = _run(m, ids, mask, seg, cfg)
        for k, ref in want.items():
            assert rel_err(got[k], ref) < tol, (k, rel_err(got[k], ref))
    # the feature is on for this request: less than nine tenths of the key columns are kept
    last = np.where(mask.any(axis=1), S - np.argmax(mask[:, ::-1] != 0, axis=1), S)
    extents = np.minimum((last + step - 1) // step * step, S)
    assert int(extents.sum()) < 0.9 * batch * S
    # pooled outputs only (padding rows skipped as well)
    for _ in range(3):
        out = model.Output()
        out.pooled_output = np.zeros((batch, cfg["hidden"]), dt)
        out.probs = np.zeros((batch, 2), dt)
        m.compute_m(ids, mask_b, seg, out)
        assert rel_err(out.pooled_output, want_b["pooled_output"]) < tol
        assert rel_err(out.probs, want_b["probs"]) < tol
    # a different request in between, then inputs resident on the device with the host's copy of the mask
    ids2, mask2, seg2, _ = synthetic.random_inputs(cfg, batch, S, 43, lengths=(90, S))
    _run(m, ids2, mask2, seg2, cfg)
    d_ids, d_mask, d_seg = (torch.from_numpy(a).cuda() for a in (ids, mask, seg))
    torch.cuda.synchronize()
    import gpu_harness as G
    for host_mask in (mask, None, mask):
        m.forward_device(0, batch, d_ids.data_ptr(), d_mask.data_ptr(), d_seg.data_ptr(), host_mask=host_mask)
        m.synchronize(0)
        ptrs = m.device_outputs(0)
        seq_out = G.copy_from_device(ptrs["sequence_output"], (batch, S, cfg["hidden"]), dt)
        assert rel_err(seq_out, want["sequence_output"]) < tol
    if ct == model.ComputeType.FLOAT:
        truth = oracle.bert_forward(var, synthetic.model_geometry(cfg, S), ids, mask, seg)
        for k in ("sequence_output", "pooled_output", "probs"):
            assert rel_err(got[k], truth[k]) < 1e-5, (k, rel_err(got[k], truth[k]))
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("ct", [model.ComputeType.FLOAT, model.ComputeType.HALF])
@pytest.mark.parametrize("batch,seq", [(1, 32), (8, 32), (16, 32), (5, 64), (3, 20), (40, 32), (4, 128), (3, 100)])
def test_small_requests_run_each_layers_attention_as_one_launch(tmp_path, oracle, ct, batch, seq, monkeypatch):
    """With heads of 64, binary16 models of up to 128 positions (any request) and float32 models of up to 64
    positions (requests of up to 512 tokens) take cubk_attention_small_* in place of two batched products and the
    softmax kernel: same outputs as with the switch off, and as the oracle."""
    if ct == model.ComputeType.FLOAT and (seq > 64 or batch * seq > 512):
        pytest.skip("float32: the one-launch attention stops at 64 positions and 512 tokens")
    cfg = synthetic.config("small", hidden=128, heads=2, intermediate=256, layers=2)    # heads of 64
    var = synthetic.random_weights(cfg, 7)
    path = str(tmp_path / "m.pb")
    frozen_graph.write_frozen_graph(path, var)
    ids, mask, seg, _ = synthetic.random_inputs(cfg, batch, seq, 13, lengths=(1, seq), segments="random")
    tol = 1e-5 if ct == model.ComputeType.FLOAT else 4e-3
    monkeypatch.setenv("CUBERT_SMALL_ATTENTION", "0")
    plain = model.Model(path, batch, seq, cfg["layers"], cfg["heads"], ct)
    want = _run(plain, ids, mask, seg, cfg)
    plain.close()
    monkeypatch.delenv("CUBERT_SMALL_ATTENTION")
    m = model.Model(path, batch, seq, cfg["layers"], cfg["heads"], ct)
    m.profile_read()
    m.profile_enable(True)
    got = _run(m, ids, mask, seg, cfg)
    prof = m.profile_read()
    m.profile_enable(False)
    assert prof["gemm"]["launches"] == 4 * cfg["layers"] + 1 and prof["masked_softmax"]["launches"] == cfg["layers"]
    for _ in range(2):                                   # captured, replayed
        again = _run(m, ids, mask, seg, cfg)
    for k, ref in want.items():
        assert rel_err(got[k], ref) < tol, (k, rel_err(got[k], ref))
        assert np.array_equal(again[k], got[k]), k
    if ct == model.ComputeType.FLOAT:
        truth = oracle.bert_forward(var, synthetic.model_geometry(cfg, seq), ids, mask, seg)
        for k in ("sequence_output", "pooled_output", "probs"):
            assert rel_err(got[k], truth[k]) < 1e-5, (k, rel_err(got[k], truth[k]))
    m.close()


@pytest.mark.gpu
def test_through_the_references_own_python_wrapper(model_files, reference_python_wrapper):
    """The calls of the reference's python/cuBERT_test.py:35-51, made through its unmodified Cython
    wrapper, served by this library; checked against the reference CPU build's recorded outputs."""
    cuBERT = reference_python_wrapper
    path, cfg, var = model_files["tiny"]
    g = golden("tiny")
    ids, mask, seg = g["ids"], g["mask"], g["seg"]
    b, s = ids.shape
    m = cuBERT.Model(path, 8, s, cfg["layers"], cfg["heads"], compute_type=cuBERT.ComputeType.FLOAT)
    output = np.zeros((b, 3), dtype=np.float32, order="C")
    m.compute(ids, mask, seg, output, output_type=cuBERT.OutputType.LOGITS)
    assert rel_err(output, g["logits"]) < 1e-5
    new_output = cuBERT.Output()
    new_output.logits = np.zeros((b, 3), dtype=np.float32, order="C")
    new_output.sequence_output = np.zeros((b, s, 64), dtype=np.float32, order="C")
    m.compute_m(ids, mask, seg, new_output)
    assert rel_err(new_output.logits, g["logits"]) < 1e-5
    assert rel_err(new_output.sequence_output, g["sequence_output"]) < 1e-5
    del m


@pytest.mark.gpu
@pytest.mark.parametrize("ct", [model.ComputeType.FLOAT, model.ComputeType.HALF])
@pytest.mark.parametrize("name,batch,seq,skip", [("small", 80, 32, "0"), ("small", 67, 32, "1"), ("tiny", 40, 64, "0")])
def test_last_layer_on_first_tokens_only(model_files, oracle, ct, name, batch, seq, skip, monkeypatch):
    """When only pooled_output / logits / probs are asked for, the last encoder layer runs for the first
    token of every sequence alone (one attention query per sequence, batch rows through the feed-forward
    part). Same operations on fewer rows: the answers must be those of the full pass, with and without
    padding skipping, full and ragged masks, and after graph replay."""
    path, cfg, var = model_files[name]
    lengths = (3, seq) if skip == "1" else "full"
    ids, mask, seg, _ = synthetic.random_inputs(cfg, batch, seq, 29, lengths=lengths, segments="random")
    dt = np.float32 if ct == model.ComputeType.FLOAT else np.float16
    tol = 1e-5 if ct == model.ComputeType.FLOAT else 4e-3
    monkeypatch.setenv("CUBERT_SKIP_PADDING", skip)
    m = model.Model(path, batch, seq, cfg["layers"], cfg["heads"], ct)
    monkeypatch.setenv("CUBERT_PRUNE_LAST_LAYER", "0")
    full = model.Model(path, batch, seq, cfg["layers"], cfg["heads"], ct)

    def heads(mm):
        out = model.Output()
        out.pooled_output = np.zeros((batch, cfg["hidden"]), dt)
        out.logits = np.zeros((batch, cfg["num_labels"]), dt)
        out.probs = np.zeros((batch, cfg["num_labels"]), dt)
        mm.compute_m(ids, mask, seg, out)
        return out

    m.profile_read()
    m.profile_enable(True)
    heads(m)
    prof = m.profile_read()
    m.profile_enable(False)
    e = 4 if ct == model.ComputeType.FLOAT else 2
    last = 2 * batch * cfg["intermediate"] * e + cfg["intermediate"] * e
    assert (prof["bias_gelu"]["bytes"] - last) % (cfg["layers"] - 1) == 0      # the last layer saw `batch` rows
    want = heads(full)
    for _ in range(3):
        got = heads(m)
        for k in ("pooled_output", "logits", "probs"):
            assert rel_err(getattr(got, k), getattr(want, k)) < tol, k
    if ct == model.ComputeType.FLOAT:
        truth = oracle.bert_forward(var, synthetic.model_geometry(cfg, seq), ids, mask, seg)
        for k in ("pooled_output", "logits", "probs"):
            assert rel_err(getattr(got, k), truth[k]) < 1e-5, k
    # asking for a per-position output afterwards takes the full pass again
    allout = _run(m, ids, mask, seg, cfg)
    assert rel_err(allout["pooled_output"], want.pooled_output) < tol
    m.close()
    full.close()


@pytest.mark.gpu
@pytest.mark.parametrize("ct", [model.ComputeType.FLOAT, model.ComputeType.HALF])
@pytest.mark.parametrize("chunks,layers,batch", [("4", "2", 601), ("3", "1", 600), ("8", "5", 515), ("1", "2", 600),
                                                  ("4", "0", 520)])
def test_output_copies_overlap_the_computation(model_files, oracle, ct, chunks, layers, batch, monkeypatch):
    """A large request that wants per-position outputs runs its last encoder layers sub-batch by sub-batch
    and copies each sub-batch's rows out while the next is computed; embedding_output leaves right after
    the embedding kernel. Every output of every sequence must be what the plain pass gives: uneven
    splits, more tail layers than the model has, no tail layers, repeated calls (graphs replayed),
    float32 conversion, and a smaller request afterwards."""
    path, cfg, var = model_files["small"]
    S = 32
    ids, mask, seg, _ = synthetic.random_inputs(cfg, batch, S, 23, lengths=(3, S), segments="random")
    dt = np.float32 if ct == model.ComputeType.FLOAT else np.float16
    tol = 1e-5 if ct == model.ComputeType.FLOAT else 4e-3

    monkeypatch.setenv("CUBERT_TAIL_CHUNKS", "1")
    plain = model.Model(path, batch, S, cfg["layers"], cfg["heads"], ct)
    want = {}
    for name, kind, shape in (("sequence_output", model.OutputType.SEQUENCE_OUTPUT, (batch, S, cfg["hidden"])),
                              ("pooled_output", model.OutputType.POOLED_OUTPUT, (batch, cfg["hidden"])),
                              ("logits", model.OutputType.LOGITS, (batch, 2)),
                              ("probs", model.OutputType.PROBS, (batch, 2))):
        want[name] = np.zeros(shape, dt)
        plain.compute(ids, mask, seg, want[name], kind)     # one output at a time: the plain path
    plain.close()

    monkeypatch.setenv("CUBERT_TAIL_CHUNKS", chunks)
    monkeypatch.setenv("CUBERT_TAIL_LAYERS", layers)
    m = model.Model(path, batch, S, cfg["layers"], cfg["heads"], ct)
    for to_float in (False, True):
        for _ in range(3):   # eager, captured, replayed
            got = _run(m, ids, mask, seg, cfg, to_float=to_float)
            for k, ref in want.items():
                assert got[k].dtype == (np.float32 if to_float else dt)
                assert rel_err(got[k], ref) < tol, (k, to_float, rel_err(got[k], ref))
    if ct == model.ComputeType.FLOAT:
        truth = oracle.bert_forward(var, synthetic.model_geometry(cfg, S), ids, mask, seg)
        for k in got:
            assert rel_err(got[k], truth[k]) < 1e-5, (k, rel_err(got[k], truth[k]))
    else:
        r16 = lambda n: var["bert/embeddings/" + n].astype(np.float16).astype(np.float32)  # noqa: E731
        truth = oracle.bert_embeddings(ids, seg, r16("word_embeddings"), r16("position_embeddings")[:S],
                                       r16("token_type_embeddings"), r16("LayerNorm/beta"), r16("LayerNorm/gamma"))
        assert rel_err(got["embedding_output"], truth.reshape(batch, S, -1)) < 2e-3
    # a smaller request afterwards, sequence_output alone
    nb = batch // 2 + 1
    out = model.Output()
    out.sequence_output = np.zeros((nb, S, cfg["hidden"]), dt)
    m.compute_m(ids[:nb], mask[:nb], seg[:nb], out)
    assert rel_err(out.sequence_output, want["sequence_output"][:nb]) < tol
    m.close()


@pytest.mark.gpu
def test_float32_products_on_tensor_cores_keep_float32_accuracy(tmp_path, oracle, monkeypatch):
    """A float32 model's cuBLAS products run, where cuBLAS offers it, as three-way bfloat16 splits on the
    tensor cores. Both ways must stay within the float32 bar of the oracle, on BERT-base geometry
    (sums over 768 and 3072 terms)."""
    cfg = synthetic.config("base", layers=2)
    var = synthetic.random_weights(cfg, 5)
    path = str(tmp_path / "base2.pb")
    frozen_graph.write_frozen_graph(path, var)
    B, S = 16, 32
    ids, mask, seg, _ = synthetic.random_inputs(cfg, B, S, 5, lengths=(5, S), segments="random")
    ref = oracle.bert_forward(var, synthetic.model_geometry(cfg, S), ids, mask, seg)
    errs = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("CUBERT_FP32_EMULATION", mode)
        m = model.Model(path, B, S, cfg["layers"], cfg["heads"], model.ComputeType.FLOAT)
        if mode == "0":
            assert m.info["fp32_gemm_emulation"] == 0
        active = m.info["fp32_gemm_emulation"]
        for _ in range(3):   # eager, captured, replayed
            got = _run(m, ids, mask, seg, cfg)
        errs[mode] = (active, {k: rel_err(got[k], ref[k]) for k in got})
        m.close()
        for k, e in errs[mode][1].items():
            assert e < 1e-5, (mode, k, e)
    if errs["1"][0] == 0:
        pytest.skip("this cuBLAS has no float32 emulation; the float32 pipes were checked")


@pytest.mark.gpu
def test_the_references_own_benchmark_program(tmp_path):
    """benchmark/benchmark_cu.cpp of the reference, compiled unchanged against this library (make -C
    oracle ref_benchmark): BERT-base float32, batch 128, seq 32, cuBERT_POOLED_OUTPUT, 10 warm-up + 10
    timed calls with random ids, masks and segments. It must run to the end and write finite tanh values."""
    import subprocess
    from cubert_b200 import build as native
    from oracle import bindings
    native.build_all(verbose=False)
    binary = bindings.build_benchmark()
    if binary is None:
        pytest.skip("reference benchmark not built (reference tree absent)")
    cfg = synthetic.config("base")
    frozen_graph.write_frozen_graph(str(tmp_path / "bert_frozen_seq32.pb"), synthetic.random_weights(cfg, 0))
    proc = subprocess.run([binary], cwd=str(tmp_path), stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          timeout=600, universal_newlines=True)
    assert proc.returncode == 0, proc.stdout[-2000:]
    times = [int(l.split()[1][:-2]) for l in proc.stdout.splitlines() if l.startswith("cuBERT: ") and l.endswith("ms")]
    assert len(times) == 20, proc.stdout[-2000:]
    assert max(times[10:]) < 100          # the reference publishes 184.6 ms per call on a Tesla P4
    values = np.loadtxt(str(tmp_path / "cuBERT.txt"), dtype=np.float64)
    assert values.size == 20 * 128 * 768
    assert np.all(np.isfinite(values)) and np.all(np.abs(values) <= 1.0) and values.std() > 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_the_references_own_host_code_on_our_kernels(model_files, oracle, name):
    """The inner drop-in boundary: the reference's unmodified GPU host code (Bert, Transformer,
    AttentionSelf, Dense, BatchMatMul, its cuBLAS wrappers) linked with oracle/ref_host_b200_ops.cu, which
    defines the reference's operator templates (layer_norm_, softmax_, gelu, embedding, _not, tanh_,
    reduce_mean_1) as calls into this repository's launch layer. float32 must reproduce the reference's
    CPU results (golden fixtures) to 1e-5; binary16 must stay within the binary16 bars."""
    from cubert_b200 import build as native
    from oracle import bindings
    native.build_all(verbose=False)
    if bindings.build_host_b200() is None:
        pytest.skip("reference host library not built (reference tree absent)")
    host = bindings.ReferenceHost(bindings.REF_HOST_B200_SO)
    path, cfg, var = model_files[name]
    g = golden(name)
    ids, mask, seg = g["ids"], g["mask"], g["seg"]
    geo = synthetic.model_geometry(cfg, ids.shape[1])
    got = host.forward(var, geo, ids, mask, seg)
    for k in got:
        assert rel_err(got[k], g[k]) < 1e-5, (k, rel_err(got[k], g[k]))
    var16 = {k: v.astype(np.float16).astype(np.float32) for k, v in var.items()}
    ref16 = oracle.bert_forward(var16, geo, ids, mask, seg)
    got16 = host.forward(var, geo, ids, mask, seg, half=True)
    for k in got16:
        assert got16[k].dtype == np.float16
        assert np.max(np.abs(got16[k].astype(np.float32) - ref16[k])) < (1e-2 if k in ("probs", "pooled_output") else 6e-2), k
