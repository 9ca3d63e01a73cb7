"""Parity at the benchmark's full sizes.

Kernels at the largest shapes of the isolated sweep (more than 2^31 elements per tensor, which the
reference's `int` indices cannot address): the CPU oracle checks a random sample of rows, and
size-independent properties cover every row (LayerNorm rows have mean beta-weighted 0 and unit
variance, softmax rows sum to 1 with zeros exactly where the mask is 0, GELU is bounded by its input).
Whole model at the sizes of the three full-model benchmark workloads against the reference's CPU code.
"""
import numpy as np
import pytest
import torch

import gpu_harness as G
from cubert_b200 import frozen_graph, model, synthetic

pytestmark = pytest.mark.gpu


def _sample_rows(n, k, seed):
    rng = np.random.default_rng(seed)
    idx = np.unique(np.concatenate([[0, 1, n - 2, n - 1, n // 2], rng.integers(0, n, k)]))
    return idx


@pytest.mark.parametrize("t", ["f16", "f32"])
def test_layernorm_and_gelu_beyond_2_to_31_elements(oracle, t):
    rows, ch = 1048576, 3072 if t == "f16" else 2304   # 3.2e9 / 2.4e9 elements per tensor
    dt = G.TORCH_DTYPE[t]
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.empty((rows, ch), device="cuda", dtype=dt)
    r = torch.empty((rows, ch), device="cuda", dtype=dt)
    for part in range(8):  # fill in slices to bound temporary memory
        sl = slice(part * rows // 8, (part + 1) * rows // 8)
        x[sl] = torch.randn((rows // 8, ch), device="cuda", generator=g).to(dt)
        r[sl] = torch.randn((rows // 8, ch), device="cuda", generator=g).to(dt)
    bias = torch.randn(ch, device="cuda", generator=g).to(dt)
    gamma = (1 + 0.1 * torch.randn(ch, device="cuda", generator=g)).to(dt)
    beta = (0.1 * torch.randn(ch, device="cuda", generator=g)).to(dt)
    idx = _sample_rows(rows, 500, 2)
    tidx = torch.from_numpy(idx).cuda()
    xs, rs = G.host(x[tidx]), G.host(r[tidx])
    bh, gh, beh = G.host(bias), G.host(gamma), G.host(beta)

    out = G.bias_residual_ln(x, bias, r, gamma, beta, t)
    ref = oracle.layer_norm_(rs, xs + bh[None, :], beh, gh)
    got = G.host(out[tidx])
    if t == "f32":
        G.assert_close(got, ref, G.F32_RTOL, 1.0, "ln sample")
    else:
        G.assert_close(got, ref, G.F16_RTOL, 1.0, "ln sample")
    # property over ALL rows: ((out - beta) / gamma) has mean 0 and variance 1 per row
    for part in range(8):
        sl = slice(part * rows // 8, (part + 1) * rows // 8)
        z = (out[sl].float() - beta.float()) / gamma.float()
        assert z.mean(dim=1).abs().max().item() < (2e-3 if t == "f16" else 1e-4)
        assert (z.var(dim=1, unbiased=False) - 1).abs().max().item() < (1e-2 if t == "f16" else 1e-3)
        del z
    del out

    act = G.bias_gelu(x, bias, t)
    ref = oracle.gelu(xs + bh[None, :])
    floor = np.maximum(2e-2 * np.abs(xs + bh[None, :]), 1e-3)
    G.assert_close(G.host(act[tidx]), ref, G.F32_RTOL if t == "f32" else G.F16_RTOL, floor, "gelu sample")
    for part in range(8):  # -0.17 <= gelu(y) and |gelu(y)| <= |y| for every element
        sl = slice(part * rows // 8, (part + 1) * rows // 8)
        y = x[sl].float() + bias.float()
        a = act[sl].float()
        assert a.min().item() >= -0.1701 and bool(torch.all(a.abs() <= y.abs() * 1.001 + 1e-6))
        del y, a


@pytest.mark.parametrize("t", ["f16", "f32"])
@pytest.mark.parametrize("batch,seq", [(64, 512), (256, 128), (128, 32)])
def test_softmax_full_size(oracle, t, batch, seq):
    heads = 12
    dt = G.TORCH_DTYPE[t]
    g = torch.Generator(device="cuda").manual_seed(batch + seq)
    scores = (torch.randn((batch, seq, heads, seq), device="cuda", generator=g) * 3).to(dt)
    lens = torch.randint(1, seq + 1, (batch,), device="cuda", generator=g)
    mask = (torch.arange(seq, device="cuda")[None, :] < lens[:, None]).to(torch.int8).contiguous()
    out = G.masked_softmax(scores.view(-1, seq), mask, seq * heads, 0.125, t).view(batch, seq, heads, seq)
    # every row sums to 1 and is exactly 0 where the key is masked
    sums = out.float().sum(dim=-1)
    assert (sums - 1).abs().max().item() < (2e-3 if t == "f16" else 1e-5)
    assert bool(torch.all(out.masked_select((mask == 0)[:, None, None, :].expand_as(out)) == 0))
    # a sample of sequences against the oracle
    sel = _sample_rows(batch, 6, 5)
    tsel = torch.from_numpy(sel).cuda()
    ref = oracle.masked_softmax(G.host(scores[tsel]), G.host(mask[tsel]).astype(np.int8), 0.125)
    G.assert_close(G.host(out[tsel]), ref, G.F32_RTOL if t == "f32" else G.F16_RTOL, 1e-4 if t == "f32" else 1e-1,
                   "softmax sample")


@pytest.fixture(scope="module")
def base_model_file(tmp_path_factory):
    cfg = synthetic.config("base")
    var = synthetic.random_weights(cfg, 0)
    path = str(tmp_path_factory.mktemp("base") / "bert_base.pb")
    frozen_graph.write_frozen_graph(path, var)
    return path, cfg, var


def _rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / (np.sqrt(np.mean(b * b)) + 1e-30))


def test_bert_base_f32_seq32_batch128(base_model_file, reference_cpu):
    """The reference's published case: BERT-base float32, seq 32, batch 128, logits and probs, against the
    reference's CPU build on the same weights and inputs (seed 0, ids in [1, 21128), full mask,
    segment 0 for the first 16 positions)."""
    path, cfg, var = base_model_file
    ids, mask, seg, _ = synthetic.random_inputs(cfg, 128, 32, 0, lengths="full", segments="half")
    ref = reference_cpu.bert_forward(var, synthetic.model_geometry(cfg, 32), ids, mask, seg)
    m = model.Model(path, 128, 32, cfg["layers"], cfg["heads"], model.ComputeType.FLOAT)
    out = model.Output()
    out.logits = np.zeros((128, 2), np.float32)
    out.probs = np.zeros((128, 2), np.float32)
    out.pooled_output = np.zeros((128, 768), np.float32)
    out.sequence_output = np.zeros((128, 32, 768), np.float32)
    out.embedding_output = np.zeros((128, 32, 768), np.float32)
    m.compute_m(ids, mask, seg, out)
    m.close()
    assert _rel(out.embedding_output, ref["embedding_output"]) < 1e-5
    assert _rel(out.sequence_output, ref["sequence_output"]) < 2e-5   # 12 layers of GEMM reordering
    assert _rel(out.pooled_output, ref["pooled_output"]) < 2e-5
    assert np.max(np.abs(out.logits - ref["logits"])) < 1e-5          # the bar of test/cuBERT/BertTest.cpp:43-53
    assert np.max(np.abs(out.probs - ref["probs"])) < 1e-5


def test_bert_base_f16_seq128_variable_length(base_model_file, reference_cpu):
    """The headline benchmark workload (BERT-base, seq 128, ragged masks) on a 32-sequence slice: binary16 storage against the
    float32 reference on binary16-rounded weights."""
    path, cfg, var = base_model_file
    var16 = {k: v.astype(np.float16).astype(np.float32) for k, v in var.items()}
    ids, mask, seg, _ = synthetic.random_inputs(cfg, 32, 128, 2, lengths=(8, 128))
    ref = reference_cpu.bert_forward(var16, synthetic.model_geometry(cfg, 128), ids, mask, seg)
    m = model.Model(path, 256, 128, cfg["layers"], cfg["heads"], model.ComputeType.HALF)
    out = model.Output()
    out.sequence_output = np.zeros((32, 128, 768), np.float32)
    out.pooled_output = np.zeros((32, 768), np.float32)
    out.probs = np.zeros((32, 2), np.float32)
    m.compute_m(ids, mask, seg, out, output_to_float=True)
    m.close()
    assert np.max(np.abs(out.probs - ref["probs"])) < 1e-2
    assert np.max(np.abs(out.pooled_output - ref["pooled_output"])) < 1e-2
    # 12 layers in binary16 storage: the reference accepts 1e-2 after 2 layers on O(1) outputs
    err = np.abs(out.sequence_output - ref["sequence_output"])
    assert np.sqrt(np.mean(err ** 2)) < 1e-2 and err.max() < 1e-1


def test_bert_large_f16_seq512_mean_pooler(tmp_path, reference_cpu):
    """The BERT-large workload on a 4-sequence slice: BERT-large geometry, seq 512, no pooler weights
    (mean pooler) and no classifier, cuBERT_POOLED_OUTPUT."""
    cfg = synthetic.config("large", layers=4)   # 4 of the 24 layers keep the CPU reference to seconds
    var = synthetic.random_weights(cfg, 3)
    var16 = {k: v.astype(np.float16).astype(np.float32) for k, v in var.items()}
    path = str(tmp_path / "large.pb")
    frozen_graph.write_frozen_graph(path, {k: v.astype(np.float16) for k, v in var.items()})
    ids, mask, seg, _ = synthetic.random_inputs(cfg, 4, 512, 3, lengths="full")
    ref = reference_cpu.bert_forward(var16, synthetic.model_geometry(cfg, 512), ids, mask, seg)
    m = model.Model(path, 4, 512, cfg["layers"], cfg["heads"], model.ComputeType.HALF)
    assert m.info["has_pooler_dense"] == 0 and m.info["num_labels"] == 0
    pooled = np.zeros((4, 1024), np.float16)
    m.compute(ids, mask, seg, pooled, model.OutputType.POOLED_OUTPUT)
    m.close()
    assert np.max(np.abs(pooled.astype(np.float32) - ref["pooled_output"])) < 1e-2
