"""Randomised property tests (hypothesis): shapes, alignments, masks and value ranges that nobody wrote
down by hand, each checked against the C oracle and against properties the operation must have whatever
the input (probabilities sum to one, masked keys get nothing, gather then scatter is the identity, a mean
is linear). The reference's tests hold fixed known answers only."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

import gpu_harness as G
from cubert_b200 import kernels

pytestmark = pytest.mark.gpu

SETTINGS = dict(max_examples=150, deadline=None, derandomize=True, database=None, suppress_health_check=[HealthCheck.function_scoped_fixture,
                                                                      HealthCheck.too_slow, HealthCheck.data_too_large])
DT = st.sampled_from(["f32", "f16"])
# widths that take the vector kernels (multiples of 8), the block-per-row kernels and the generic ones
WIDTH = st.one_of(st.integers(1, 70), st.sampled_from([8, 64, 96, 256, 768, 776, 1024, 2056, 3072, 4104, 8200]))


def _prep(a, t):
    a = np.asarray(a, np.float32)
    if t == "f16":
        a = G.round_f16(a)
    return G.dev(a, G.TORCH_DTYPE[t]), a


def _close(got, ref, t, floor=1.0):
    g = G.host(got)
    G.assert_close(g, ref, G.F32_RTOL if t == "f32" else G.F16_RTOL, floor, "property")
    if t == "f16":
        assert np.max(np.abs(g - ref)) <= G.F16_ATOL


@settings(**SETTINGS)
@given(t=DT, rows=st.integers(1, 33), ch=WIDTH, seed=st.integers(0, 2 ** 31 - 1), with_bias=st.booleans(),
       with_residual=st.booleans(), scale=st.sampled_from([1e-3, 1.0, 30.0]))
def test_layer_norm_family(oracle, t, rows, ch, seed, with_bias, with_residual, scale):
    rng = np.random.default_rng(seed)
    x, xh = _prep(rng.standard_normal((rows, ch)) * scale + rng.standard_normal() * scale, t)
    res, resh = _prep(rng.standard_normal((rows, ch)) * scale, t) if with_residual else (None, np.zeros((rows, ch), np.float32))
    bias, biash = _prep(rng.standard_normal(ch) * scale, t) if with_bias else (None, np.zeros(ch, np.float32))
    g, gh = _prep(1 + 0.3 * rng.standard_normal(ch), t)
    be, beh = _prep(0.3 * rng.standard_normal(ch), t)
    ref = oracle.layer_norm_(resh, xh + biash, beh, gh)     # float32 sum of the inputs, then the reference's LN
    total = (xh + biash + resh).astype(np.float64)
    std, mean = total.std(axis=1), np.abs(total.mean(axis=1))
    if ch == 1 or np.any(std < 0.05 * (mean + std)):
        return    # rows that are nearly constant relative to their mean: float32 cancellation on both sides, documented
    got = G.bias_residual_ln(x, bias, res, g, be, t)
    # inputs of very different magnitudes lose digits in the float32 pre-sum on both sides alike
    _close(got, ref, t, floor=max(1.0, float(np.max(np.abs(gh))) * 2))


@settings(**SETTINGS)
@given(t=DT, rows=st.integers(1, 40), ch=WIDTH, seed=st.integers(0, 2 ** 31 - 1), spread=st.sampled_from([0.5, 3.0, 9.0]))
def test_bias_gelu_and_tanh(oracle, t, rows, ch, seed, spread):
    rng = np.random.default_rng(seed)
    x, xh = _prep(rng.standard_normal((rows, ch)) * spread, t)
    b, bh = _prep(rng.standard_normal(ch), t)
    xb = (xh + bh).astype(np.float32)
    got = G.host(G.bias_gelu(x, b, t))
    ref = oracle.gelu(xb)
    G.assert_close(got, ref, G.F32_RTOL if t == "f32" else G.F16_RTOL, np.maximum(2e-2 * np.abs(xb), 1e-3), "gelu")
    assert np.all(got[xb > 6] > 0) and np.all(np.abs(got[xb < -9]) <= 1e-6)        # the two tails
    tanh = G.host(G.bias_tanh(x, b, t))
    assert np.max(np.abs(tanh - np.tanh(xb.astype(np.float64)))) <= (2e-6 if t == "f32" else 1e-3)
    assert np.all(np.abs(tanh) <= 1.0)


@settings(**SETTINGS)
@given(t=DT, batch=st.integers(1, 4), heads=st.integers(1, 3),
       seq=st.one_of(st.integers(1, 72), st.sampled_from([128, 256, 264, 512, 1024])), seed=st.integers(0, 2 ** 31 - 1),
       keep=st.sampled_from([0.0, 0.3, 0.9, 1.0]), scale=st.sampled_from([1.0, 0.125]))
def test_masked_softmax(oracle, t, batch, heads, seq, seed, keep, scale):
    rng = np.random.default_rng(seed)
    x, xh = _prep(rng.standard_normal((batch, seq, heads, seq)) * 3, t)
    mask = (rng.random((batch, seq)) < keep).astype(np.int8) * rng.integers(1, 100, (batch, seq)).astype(np.int8)
    got = G.host(G.masked_softmax(x.view(-1, seq), G.dev(mask), seq * heads, scale, t)).reshape(batch, seq, heads, seq)
    tol = 2e-2 if t == "f16" else 1e-4
    assert np.all(np.abs(got.sum(axis=-1) - 1.0) <= tol)                           # rows are distributions
    assert np.all(got >= 0)
    for b in range(batch):
        if mask[b].any():                                                          # masked keys get nothing
            assert np.all(got[b][:, :, mask[b] == 0] == 0)
    if seq <= 512 and all(m.any() for m in mask):
        ref = oracle.masked_softmax(xh, mask, scale)
        G.assert_close(got, ref, G.F32_RTOL if t == "f32" else G.F16_RTOL, 1e-4 if t == "f32" else 1e-1, "softmax")


@settings(**SETTINGS)
@given(t=DT, batch=st.integers(1, 5), seq=st.integers(1, 40), hidden=WIDTH, seed=st.integers(0, 2 ** 31 - 1))
def test_mean_pool_is_a_linear_mean(t, batch, seq, hidden, seed):
    rng = np.random.default_rng(seed)
    a, ah = _prep(rng.standard_normal((batch, seq, hidden)), t)
    b, bh = _prep(rng.standard_normal((batch, seq, hidden)), t)
    pa, pb = G.host(G.mean_pool(a, t)), G.host(G.mean_pool(b, t))
    tol = 2e-6 if t == "f32" else 2e-3
    assert np.max(np.abs(pa - ah.astype(np.float64).mean(axis=1))) <= tol
    s, sh = _prep(ah + bh, t)
    ps = G.host(G.mean_pool(s, t))
    assert np.max(np.abs(ps - (pa + pb))) <= (1e-5 if t == "f32" else 1e-2)         # mean(a + b) = mean(a) + mean(b)


@settings(**SETTINGS)
@given(dtype=st.sampled_from([torch.float32, torch.float16]), rows=st.integers(1, 60), width=WIDTH,
       n=st.integers(1, 90), seed=st.integers(0, 2 ** 31 - 1))
def test_gather_then_scatter_is_the_identity(dtype, rows, width, n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    table = torch.randn((rows, width), device="cuda", generator=g).to(dtype)
    idx = torch.randint(0, rows, (n,), device="cuda", generator=g, dtype=torch.int32)
    picked = G.embed_gather(idx, table)
    assert torch.equal(picked, table[idx.long()])                                   # bit-exact gather
    back = torch.full_like(table, 7)
    kernels.check(kernels.load().cubk_scatter_rows(G.ptr(idx), n, G.ptr(picked), width, table.element_size(),
                                                   G.ptr(back), rows, G.stream()))
    touched = torch.zeros(rows, dtype=torch.bool, device="cuda")
    touched[idx.long()] = True
    assert torch.equal(back[touched], table[touched]) and bool((back[~touched] == 7).all())


@settings(**SETTINGS)
@given(t=DT, batch=st.integers(1, 6), seq=st.integers(1, 20), hidden=st.sampled_from([8, 64, 200, 768, 1000, 4096]),
       vocab=st.integers(1, 50), seed=st.integers(0, 2 ** 31 - 1),
       staged=st.sampled_from(["general", "exact", "staged"]))
def test_embed_ln(oracle, t, batch, seq, hidden, vocab, seed, staged):
    saved = (kernels.set_option(kernels.OPT_EMBED_STAGED_ROWS, 1 if staged == "staged" else 0),
             kernels.set_option(kernels.OPT_EXACT_WIDTH_EMBED, 0 if staged == "general" else 1))
    try:
        rng = np.random.default_rng(seed)
        word, wh = _prep(rng.standard_normal((vocab, hidden)) * 0.05, t)
        pos, ph = _prep(rng.standard_normal((seq, hidden)) * 0.05, t)
        typ, th = _prep(rng.standard_normal((2, hidden)) * 0.05, t)
        g, gh = _prep(1 + 0.1 * rng.standard_normal(hidden), t)
        be, beh = _prep(0.1 * rng.standard_normal(hidden), t)
        ids = rng.integers(0, vocab, (batch, seq), dtype=np.int32)
        seg = rng.integers(0, 2, (batch, seq)).astype(np.int8)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = G.embed_ln(G.dev(ids), G.dev(seg), word, pos, typ, g, be, t, status)
        _close(got, oracle.bert_embeddings(ids, seg, wh, ph, th, beh, gh), t)
        assert int(status.item()) == 0
    finally:
        kernels.set_option(kernels.OPT_EMBED_STAGED_ROWS, saved[0])
        kernels.set_option(kernels.OPT_EXACT_WIDTH_EMBED, saved[1])


@settings(**SETTINGS)
@given(t=DT, batch=st.integers(1, 5), heads=st.integers(1, 3), seq=st.one_of(st.integers(1, 72), st.sampled_from([128, 264, 512])),
       seed=st.integers(0, 2 ** 31 - 1), zero_to=st.sampled_from(["own", "common", "full"]))
def test_masked_softmax_with_key_extents(t, batch, heads, seq, seed, zero_to):
    """Any extents that cover every kept key: below them the extents call equals the plain call bit for bit,
    from there to zero_to it writes zeros, beyond it touches nothing; rows stay distributions."""
    rng = np.random.default_rng(seed)
    x, _ = _prep(rng.standard_normal((batch, seq, heads, seq)) * 3, t)
    lengths = rng.integers(1, seq + 1, batch)
    mask = np.zeros((batch, seq), np.int8)
    for b, n in enumerate(lengths):
        mask[b, :n] = rng.integers(0, 2, n) * 3
        mask[b, n - 1] = 1
    slack = rng.integers(0, 20, batch)                      # an extent may lie beyond the last kept key
    extents = np.minimum(lengths + slack, seq).astype(np.int32)
    z = {"own": 0, "common": int(extents.max()), "full": seq}[zero_to]
    plain = G.masked_softmax(x.view(-1, seq), G.dev(mask), seq * heads, 0.125, t).view(batch, seq, heads, seq)
    got = G.masked_softmax_extents(x.view(-1, seq), G.dev(mask), G.dev(extents), z, seq * heads, 0.125, t)
    got = got.view(batch, seq, heads, seq)
    epv = 4 if t == "f32" else 8
    vector_path = seq % epv == 0 and seq // epv <= 256
    for b in range(batch):
        n, w = int(extents[b]), max(int(extents[b]), z)
        if vector_path:      # whole 16-byte vectors: the boundaries move up to the next vector
            n, w = min(seq, -(-n // epv) * epv), min(seq, -(-w // epv) * epv)
        assert torch.equal(got[b, :, :, :n], plain[b, :, :, :n])
        assert bool((got[b, :, :, n:w] == 0).all())
        assert bool(torch.isnan(got[b, :, :, w:]).all())
        sums = got[b, :, :, :n].float().sum(-1)
        assert bool(((sums - 1).abs() < (1e-4 if t == "f32" else 5e-3)).all())


@settings(**SETTINGS)
@given(t=DT, batch=st.integers(1, 6), heads=st.integers(1, 3), seq=st.integers(1, 128), seed=st.integers(0, 2 ** 31 - 1),
       keep=st.sampled_from([0.0, 0.4, 1.0]), tail=st.integers(0, 100), tensor_memory=st.sampled_from([0, 1]))
def test_attention_of_short_sequences(oracle, t, batch, heads, seq, seed, keep, tail, tensor_memory):
    """The one-launch attention against its three steps on the host (reference softmax), for any short shape
    and any mask, fully masked sequences included."""
    rng = np.random.default_rng(seed)
    hidden = heads * 64
    qkv, qkvh = _prep(rng.standard_normal((batch * seq, 3 * hidden)), t)
    mask = (rng.random((batch, seq)) < keep).astype(np.int8) * rng.integers(1, 100, (batch, seq)).astype(np.int8)
    mask[:, seq - min(tail, seq - 1):] = 0   # a masked tail, which the binary16 kernel past 64 positions skips
    if t == "f32":
        seq_ok = seq <= 64
    else:
        seq_ok = True
    saved = kernels.set_option(kernels.OPT_ATTENTION_TENSOR_MEMORY, tensor_memory)   # binary16 past 64 positions
    try:
        rc, ctx = G.attention_small(qkv, G.dev(mask), batch, seq, heads, 0.125, t)
    finally:
        kernels.set_option(kernels.OPT_ATTENTION_TENSOR_MEMORY, saved)
    if not seq_ok:
        assert rc == kernels.CUBK_ERR_UNSUPPORTED
        return
    assert rc == kernels.CUBK_OK
    dt = np.float32 if t == "f32" else np.float16
    x = qkvh.reshape(batch, seq, 3, heads, 64).astype(np.float64)
    scores = (0.125 * np.einsum("bihc,bjhc->bihj", x[:, :, 0], x[:, :, 1])).astype(np.float32).astype(dt).astype(np.float32)
    probs = oracle.masked_softmax(scores, mask, 1.0).astype(dt).astype(np.float64)
    ref = np.einsum("bihj,bjhc->bihc", probs, x[:, :, 2]).reshape(batch * seq, hidden)
    got = G.host(ctx).astype(np.float64)
    assert np.all(np.isfinite(got))
    # sequences without a kept key sit at -10000, where float32 resolves 1e-3 (see the softmax tests)
    loose = np.repeat(~mask.any(axis=1), seq)
    tol = 2e-5 if t == "f32" else 4e-3
    scale = max(1.0, float(np.max(np.abs(ref))))
    if (~loose).any():
        assert np.max(np.abs(got[~loose] - ref[~loose])) <= tol * scale
    if loose.any():
        assert np.max(np.abs(got[loose] - ref[loose])) <= 5e-3 * scale


@settings(**SETTINGS)
@given(t=DT, batch=st.integers(1, 40), hidden=st.sampled_from([8, 64, 256, 768, 1024, 2048]), labels=st.integers(1, 8),
       seed=st.integers(0, 2 ** 31 - 1), bias=st.booleans())
def test_pooler_head_in_one_launch(oracle, t, batch, hidden, labels, seed, bias):
    """pooled row bit-equal to bias+tanh; logits and probs as the classifier gives them on the stored pooled row."""
    rng = np.random.default_rng(seed)
    x, _ = _prep(rng.standard_normal((batch, hidden)) * 2, t)
    pb, _ = _prep(rng.standard_normal(hidden), t)
    w, wh = _prep(rng.standard_normal((labels, hidden)) * 0.1, t)
    b, bh = _prep(rng.standard_normal(labels), t) if bias else (None, None)
    rc, pooled, logits, probs = G.pooler_head(x, pb, w, b, t)
    assert rc == kernels.CUBK_OK
    assert torch.equal(pooled, G.bias_tanh(x, pb, t))
    ref_logits, ref_probs = oracle.classifier(G.host(pooled), wh, bh)
    _close(logits, ref_logits, t)
    p = G.host(probs)
    assert np.max(np.abs(p - ref_probs)) <= (1e-5 if t == "f32" else G.F16_ATOL)
    assert np.all(np.abs(p.sum(-1) - 1) <= (1e-5 if t == "f32" else 5e-3))
