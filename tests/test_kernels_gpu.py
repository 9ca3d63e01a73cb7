"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle.

float32 storage: within 1e-5 relative. binary16 storage: the oracle runs in float32 on the
binary16-rounded inputs; the kernel output must be within 1e-3 relative / 1e-2 absolute.
Gathers and index handling: bit-exact.
"""
import numpy as np
import pytest
import torch

import gpu_harness as G
from conftest import assert_kat
from cubert_b200 import kernels

pytestmark = pytest.mark.gpu

DTYPES = ["f32", "f16"]


def _prep(a, t):
    """(device tensor in storage type, float32 host copy of what the kernel sees)."""
    a = np.asarray(a, np.float32)
    if t == "f16":
        a = G.round_f16(a)
    return G.dev(a, G.TORCH_DTYPE[t]), a


def _check(got, ref, t, floor, what):
    if t == "f32":
        G.assert_close(G.host(got), ref, G.F32_RTOL, floor, what)
    else:
        g = G.host(got)
        G.assert_close(g, ref, G.F16_RTOL, floor, what)
        assert np.max(np.abs(g - ref)) <= G.F16_ATOL


def A(entry, name, dtype=np.float32, shape=None):
    a = np.asarray(entry["arrays"][name], dtype=dtype)
    return a.reshape(shape) if shape else a


# ============================================================================ known answers of the reference tests

def test_kat_layer_norm(kats):
    e = kats["op/LayerNormTest.cpp::layer_norm_ext"]
    out = G.bias_residual_ln(G.dev(A(e, "inout", shape=(2, 3))), None, G.dev(A(e, "in", shape=(2, 3))),
                             G.dev(A(e, "gamma")), G.dev(A(e, "beta")), inplace=True)
    assert_kat(e, G.host(out))


def test_kat_softmax(kats):
    e = kats["op/SoftmaxTest.cpp::softmax_"]
    out = G.masked_softmax(G.dev(A(e, "inout", shape=(2, 3))), None, 2, inplace=True)
    assert_kat(e, G.host(out))


def test_kat_gelu(kats):
    e = kats["op/GELUTest.cpp::gelu"]
    out = G.bias_gelu(G.dev(A(e, "inout", shape=(1, 5))), None, inplace=True)
    assert_kat(e, G.host(out))
    # binary16 storage variant of the same vector: within binary16 rounding of the double answer
    out16 = G.bias_gelu(G.dev(A(e, "inout", shape=(1, 5)), torch.float16), None, t="f16")
    want = np.array([v for (_, _, v, _) in e["expect"]])
    assert np.max(np.abs(G.host(out16).ravel() - want)) < 1e-3


def test_kat_embedding(kats):
    e = kats["op/EmbeddingTest.cpp::embedding"]
    out = G.embed_gather(G.dev(A(e, "input_ids", np.int32)), G.dev(A(e, "embedding_table", shape=(4, 3))))
    assert_kat(e, G.host(out))


def test_kat_bert_embeddings(kats):
    e = kats["op_bert/BertEmbeddingsTest.cpp::bert_embedding"]
    out = G.embed_ln(G.dev(A(e, "input_ids", np.int32, (2, 4))), G.dev(A(e, "segment_ids", np.int8, (2, 4))),
                     G.dev(A(e, "word_embeddings", shape=(5, 3))), G.dev(A(e, "position_embeddings", shape=(4, 3))),
                     G.dev(A(e, "token_type_embeddings", shape=(2, 3))), G.dev(A(e, "gamma")), G.dev(A(e, "beta")))
    # EXPECT_FLOAT_EQ(out, 0) lines: our centred two-pass mean gives exactly 0 there as well
    assert_kat(e, G.host(out))


def test_kat_attention_mask(kats, oracle):
    """The reference materialises neg mask [B, S*H, S]; our softmax applies the int8 mask directly.
    Check that the rows our kernel treats as masked are exactly the reference tensor's ones."""
    e = kats["op_att/AttentionMaskTest.cpp::attention_mask"]
    mask = A(e, "in", np.int8, (2, 2))
    neg = G.host(G.logical_not(G.dev(mask)))
    assert np.array_equal(neg, oracle.not_(mask))
    expect = np.array([v for (_, _, v, _) in e["expect"]], np.float32).reshape(2, 6, 2)
    assert np.array_equal(np.broadcast_to(neg[:, None, :], (2, 6, 2)), expect)
    # and through the kernel: zero scores, masked keys get ~0 probability unless the whole row is masked
    probs = G.host(G.masked_softmax(torch.zeros((12, 2), device="cuda"), G.dev(mask), 6))
    assert np.allclose(probs[:6], [[1, 0]] * 6) and np.allclose(probs[6:], 0.5)


def test_kat_poolers(kats):
    e = kats["op_bert/BertPoolerTest.cpp::bert_pooler"]
    x = A(e, "in", shape=(2, 3, 2))
    pre = x[:, 0, :] @ A(e, "kernel", shape=(2, 2))  # the GEMM stays outside the kernels
    out = G.bias_tanh(G.dev(pre), G.dev(A(e, "bias")))
    assert_kat(e, G.host(out))
    e = kats["op_bert/BertPoolerTest.cpp::mean_pooler"]
    assert_kat(e, G.host(G.mean_pool(G.dev(A(e, "in", shape=(2, 3, 2))))))


def test_kat_classifier(kats):
    e = kats["op_out/AdditionalOutputLayerTest.cpp::additional_output"]
    logits, _ = G.logits_probs(G.dev(A(e, "in", shape=(2, 3))), G.dev(A(e, "output_weights", shape=(1, 3))), None,
                               want_probs=False)
    assert_kat(e, G.host(logits))


# ============================================================================ K2 bias + residual + LayerNorm

LN_SHAPES = [(2, 3), (5, 5), (7, 6), (1, 8), (33, 768), (17, 1024), (9, 3072), (5, 4096), (6, 200), (3, 1000),
             (4, 8192), (3, 8200), (130, 64), (257, 96), (9001, 768), (4099, 1024), (5003, 256), (1, 1536), (7, 2048)]


@pytest.mark.parametrize("exact_width", [1, 0])   # the kernel for rows that fill a warp exactly / the general one
@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("rows,ch", LN_SHAPES)
def test_bias_residual_ln(oracle, t, rows, ch, exact_width, kernel_options):
    vectors = ch // (4 if t == "f32" else 8)
    if exact_width == 0 and not (ch % 8 == 0 and vectors % 32 == 0 and vectors // 32 in (1, 2, 3, 4, 6, 8)):
        pytest.skip("this width takes the general kernel either way")
    kernel_options(kernels.OPT_EXACT_WIDTH_ROWS, exact_width)
    rng = np.random.default_rng(rows * 7919 + ch)
    x, xh = _prep(rng.standard_normal((rows, ch)), t)
    r, rh = _prep(rng.standard_normal((rows, ch)), t)
    b, bh = _prep(rng.standard_normal(ch) * 0.5, t)
    g, gh = _prep(1 + 0.1 * rng.standard_normal(ch), t)
    be, beh = _prep(0.1 * rng.standard_normal(ch), t)
    ref = oracle.layer_norm_(rh, xh + bh[None, :], beh, gh)
    _check(G.bias_residual_ln(x, b, r, g, be, t), ref, t, 1.0, "ln")
    _check(G.bias_residual_ln(x.clone(), b, r, g, be, t, inplace=True), ref, t, 1.0, "ln in place, all operands")
    # in place, and without bias / residual
    ref2 = oracle.layer_norm_(rh, xh, beh, gh)
    _check(G.bias_residual_ln(x.clone(), None, r, g, be, t, inplace=True), ref2, t, 1.0, "ln in place")
    ref3 = oracle.layer_norm_(np.zeros_like(xh), xh, beh, gh)
    _check(G.bias_residual_ln(x, None, None, g, be, t), ref3, t, 1.0, "ln plain")


@pytest.mark.parametrize("t", DTYPES)
def test_ln_unaligned_pointers_take_generic_path(oracle, t):
    rng = np.random.default_rng(3)
    rows, ch = 6, 768
    big, _ = _prep(rng.standard_normal(rows * ch + 1), t)
    x = big[1:].view(rows, ch)  # 4- or 2-byte aligned only
    xh = G.host(x)
    g, gh = _prep(np.ones(ch), t)
    be, beh = _prep(np.zeros(ch), t)
    ref = oracle.layer_norm_(np.zeros_like(xh), xh, beh, gh)
    _check(G.bias_residual_ln(x, None, None, g, be, t), ref, t, 1.0, "ln unaligned")


def test_ln_constant_rows_are_finite():
    """A constant row has (nearly) zero variance. The centred two-pass variance is never negative, so
    the result is finite and within |gamma| of beta; the reference's E[t^2] - mean^2 can go negative
    there and produce NaN (src/cuBERT/op/LayerNorm.cpp:32-35)."""
    for value in (3.14159, 0.0, -1e4):
        x = torch.full((4, 768), value, device="cuda")
        g = torch.full((768,), 2.0, device="cuda")
        be = torch.full((768,), 0.25, device="cuda")
        out = G.host(G.bias_residual_ln(x, None, None, g, be))
        assert np.all(np.isfinite(out))
        assert np.all(np.abs(out - 0.25) <= 2.0 * 1.0001)
    out = G.host(G.bias_residual_ln(torch.zeros((4, 768), device="cuda"), None, None, g, be))
    assert np.array_equal(out, np.full((4, 768), 0.25, np.float32))


# ============================================================================ K3 bias + GELU, K5a bias + tanh

ACT_SHAPES = [(1, 5), (3, 7), (5, 768), (4, 3072), (9, 1024), (2, 2048), (3, 4096), (6, 200), (5, 1001), (1000, 96)]


def _gelu_floor(xb):
    # |gelu| is tiny for very negative inputs, where the reference's 1 + erf cancels (its erff is
    # good to about 1e-7 absolute, i.e. |x| * 1e-7 in the result); bound the error there relative
    # to max(|y|, 2e-2 * |x|) instead of |y| alone.
    return np.maximum(2e-2 * np.abs(xb), 1e-3)


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("rows,ch", ACT_SHAPES)
def test_bias_gelu(oracle, t, rows, ch):
    rng = np.random.default_rng(rows * 31 + ch)
    x, xh = _prep(rng.standard_normal((rows, ch)) * 2, t)
    b, bh = _prep(rng.standard_normal(ch) * 0.5, t)
    ref = oracle.gelu(xh + bh[None, :])
    _check(G.bias_gelu(x, b, t), ref, t, _gelu_floor(xh + bh[None, :]), "gelu")
    ref2 = oracle.gelu(xh)
    _check(G.bias_gelu(x.clone(), None, t, inplace=True), ref2, t, _gelu_floor(xh), "gelu in place")


@pytest.mark.parametrize("t", DTYPES)
def test_gelu_full_input_range(t):
    """Every interesting input (dense grid on [-12, 12] plus huge values) against double erf."""
    from scipy.special import ndtr
    xs = np.concatenate([np.linspace(-12, 12, 48001), [-65504, -100, 100, 65504, 0.0, -0.0]]).astype(np.float32)
    pad = (-len(xs)) % 8
    xs = np.concatenate([xs, np.zeros(pad, np.float32)])
    x, xh = _prep(xs.reshape(1, -1), t)
    got = G.host(G.bias_gelu(x, None, t)).ravel().astype(np.float64)
    want = xh.ravel().astype(np.float64) * ndtr(xh.ravel().astype(np.float64))
    tol = 1e-5 if t == "f32" else 1e-3
    err = np.abs(got - want) / np.maximum(np.abs(want), np.maximum(2e-2 * np.abs(xh.ravel()), 1e-3))
    assert err.max() < tol, (err.max(), xh.ravel()[err.argmax()])


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("rows,ch", [(2, 2), (128, 768), (7, 1024), (3, 13)])
def test_bias_tanh(oracle, t, rows, ch):
    rng = np.random.default_rng(rows + ch)
    x, xh = _prep(rng.standard_normal((rows, ch)) * 2, t)
    b, bh = _prep(rng.standard_normal(ch), t)
    _check(G.bias_tanh(x, b, t), oracle.tanh_(xh + bh[None, :]), t, 1e-2, "tanh")


# ============================================================================ K4 masked scaled softmax

SOFTMAX_SHAPES = [  # (batch, heads, seq)
    (2, 3, 2), (1, 1, 3), (3, 2, 5), (2, 2, 8), (4, 12, 32), (2, 12, 128), (1, 16, 512), (2, 3, 64), (2, 2, 48),
    (1, 2, 1024), (1, 1, 2048), (2, 2, 200), (1, 2, 1000), (1, 1, 4096), (5, 2, 256), (3, 1, 512), (7, 1, 128),
]


def _mask(rng, batch, seq, kind):
    if kind == "prefix":
        lens = rng.integers(1, seq + 1, batch)
        return (np.arange(seq)[None, :] < lens[:, None]).astype(np.int8)
    if kind == "random":
        m = rng.integers(0, 2, (batch, seq)).astype(np.int8)
        m[:, 0] = 1
        return m * rng.integers(1, 100, (batch, seq)).astype(np.int8)  # any non-zero value keeps
    if kind == "empty_row":
        m = np.ones((batch, seq), np.int8)
        m[0, :] = 0  # a sequence with every key masked
        return m
    return None


@pytest.mark.parametrize("mask_terms", ["shared", "registers"])   # where long rows keep the additive mask terms
@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("kind", ["prefix", "random", "empty_row", "none"])
@pytest.mark.parametrize("batch,heads,seq", SOFTMAX_SHAPES)
def test_masked_softmax(oracle, t, kind, batch, heads, seq, mask_terms, kernel_options):
    if mask_terms == "registers":
        if seq // (4 if t == "f32" else 8) <= 8:
            pytest.skip("rows this short keep their mask terms in registers either way")
        kernel_options(kernels.OPT_SOFTMAX_MASK_SMEM, 0)
    else:
        kernel_options(kernels.OPT_SOFTMAX_MASK_SMEM, 1)
    rng = np.random.default_rng(batch * 1000 + heads * 100 + seq)
    x, xh = _prep(rng.standard_normal((batch, seq, heads, seq)) * 3, t)
    mask = _mask(rng, batch, seq, kind)
    scale = 0.125 if kind != "none" else 1.0
    if seq > 512:
        # The reference sums a row sequentially in float32; for rows this long that sum is itself off
        # by more than 1e-5 (n * eps / 2 systematic rounding). Judge long rows against float64 (with
        # the masked score rounded to float32 once, as the kernel's fused multiply-add does).
        v = scale * xh.astype(np.float64)
        if mask is not None:
            v = v + np.where(mask[:, None, None, :] == 0, -10000.0, 0.0)
        v = v.astype(np.float32).astype(np.float64)
        ev = np.exp(v - v.max(axis=-1, keepdims=True))
        ref = ev / ev.sum(axis=-1, keepdims=True)
    else:
        ref = oracle.masked_softmax(xh, mask, scale)
    got = G.masked_softmax(x.view(-1, seq), None if mask is None else G.dev(mask), seq * heads, scale, t)
    got4 = got.view(batch, seq, heads, seq)
    first = 0
    if kind == "empty_row":
        # Sequence 0 has every key masked: all scores sit near -10000, where float32 resolves only
        # 1e-3, so each probability carries a relative error of that order and whether the score was
        # rounded once (fused multiply-add) or twice decides single elements. The reference's own
        # backends differ from each other here; hold the degenerate sequence to 2e-3 instead.
        r0 = G.host(got4[:1])
        G.assert_close(r0, ref[:1], 2e-3, 1e-4, "softmax fully masked sequence")
        assert np.allclose(r0.sum(-1), 1.0, atol=2e-3)
        first = 1
    # probabilities: relative to max(|p|, 1e-4) -- a masked key is exactly 0 on both sides
    if batch > first:
        _check(got4[first:], ref[first:], t, 1e-4 if t == "f32" else 1e-1, "softmax " + kind)
    if kind == "prefix":
        p = G.host(got).reshape(batch, seq, heads, seq)
        assert np.all(p[np.broadcast_to(mask[:, None, None, :] == 0, p.shape)] == 0)
    # in place
    got2 = G.masked_softmax(x.view(-1, seq).clone(), None if mask is None else G.dev(mask), seq * heads, scale, t,
                            inplace=True)
    assert torch.equal(got, got2)


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("seq", [32, 128, 37])
def test_masked_softmax_keeps_nan_and_infinity_visible(t, seq):
    """A NaN score makes its whole row NaN, a row of -inf scores becomes NaN (-inf minus -inf), a +inf score
    as well (inf minus inf): what the reference's max-subtracted softmax yields (src/cuBERT/op/Softmax.cpp:19-35).
    Rows next to them are untouched."""
    x = torch.zeros((4, seq), dtype=G.TORCH_DTYPE[t], device="cuda")
    x[0, 3] = float("nan")
    x[1, :] = -float("inf")
    x[2, 5] = float("inf")
    got = G.host(G.masked_softmax(x, None, 4, 1.0, t))
    assert np.all(np.isnan(got[0])) and np.all(np.isnan(got[1])) and np.all(np.isnan(got[2]))
    assert np.allclose(got[3], 1.0 / seq, rtol=2e-3)


@pytest.mark.parametrize("zero_to", ["own", "common", "full"])
@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("batch,heads,seq", [(6, 3, 128), (3, 2, 512), (5, 2, 32), (4, 2, 64), (3, 1, 37), (2, 1, 1024),
                                             (3, 2, 2056), (70, 2, 128)])
def test_masked_softmax_with_key_extents(t, batch, heads, seq, zero_to):
    """The call that is told where each sequence's kept keys end: below the extent it must equal the plain call
    bit for bit (the columns it skips contribute exact zeros there), from the extent up to zero_to it writes
    zeros, and beyond that it touches nothing."""
    rng = np.random.default_rng(batch * 131 + seq)
    vector_path = seq % 8 == 0 and seq // (4 if t == "f32" else 8) <= 256
    step = 32 if vector_path and seq >= 32 else 1
    x, _ = _prep(rng.standard_normal((batch, seq, heads, seq)) * 3, t)
    lengths = rng.integers(1, seq + 1, batch)
    lengths[0] = seq                      # a full sequence
    lengths[-1] = 1                       # and one with a single kept key
    mask = np.zeros((batch, seq), np.int8)
    for b, n in enumerate(lengths):
        mask[b, :n] = rng.integers(0, 2, n) * 5     # any non-zero value keeps
        mask[b, n - 1] = 1                          # the last kept key sits at n - 1
    extents = np.minimum((lengths + step - 1) // step * step, seq).astype(np.int32)
    common = int(extents.max())
    z = {"own": 0, "common": common, "full": seq}[zero_to]
    plain = G.masked_softmax(x.view(-1, seq), G.dev(mask), seq * heads, 0.125, t).view(batch, seq, heads, seq)
    got = G.masked_softmax_extents(x.view(-1, seq), G.dev(mask), G.dev(extents), z, seq * heads, 0.125, t)
    got = got.view(batch, seq, heads, seq)
    for b in range(batch):
        n, w = int(extents[b]), max(int(extents[b]), z)
        assert torch.equal(got[b, :, :, :n], plain[b, :, :, :n]), (b, n)
        assert bool((got[b, :, :, n:w] == 0).all()) and bool((plain[b, :, :, n:w] == 0).all())
        assert bool(torch.isnan(got[b, :, :, w:]).all()), (b, w)
    # in place
    again = x.clone().view(-1, seq)
    G.masked_softmax_extents(again, G.dev(mask), G.dev(extents), seq, seq * heads, 0.125, t, out=again)
    assert torch.equal(again.view(batch, seq, heads, seq), plain)
    lib = kernels.load()
    f = getattr(lib, "cubk_masked_softmax_extents_" + t)
    assert f(x.data_ptr(), G.dev(mask).data_ptr(), None, 0, batch * seq * heads, seq * heads, seq, 1.0, x.data_ptr(),
             G.stream()) == kernels.CUBK_ERR_INVALID_ARG
    assert f(x.data_ptr(), None, G.dev(extents).data_ptr(), 0, batch * seq * heads, seq * heads, seq, 1.0,
             x.data_ptr(), G.stream()) == kernels.CUBK_ERR_INVALID_ARG


@pytest.mark.parametrize("t", DTYPES)
def test_gelu_hands_on_nan_and_infinity(t):
    """A NaN or +inf that reaches the activation (a binary16 overflow upstream) must stay visible, as in the
    reference's x * 0.5 * (1 + erf(x / sqrt 2)). For -inf the reference yields NaN (-inf * 0); this kernel
    gives the limit of GELU there, a zero: the one non-finite input on which the two differ."""
    x = torch.tensor([[float("nan"), float("inf"), -float("inf"), 1.0, -1.0, 0.0, float("nan"), 2.0]],
                     dtype=G.TORCH_DTYPE[t], device="cuda")
    got = G.host(G.bias_gelu(x, None, t))[0]
    assert np.isnan(got[0]) and np.isnan(got[6])
    assert got[1] == np.inf
    assert abs(got[2]) <= 1e-6
    assert np.all(np.isfinite(got[3:6])) and abs(got[3] - 0.8413447) < 2e-3 and abs(got[4] + 0.1586553) < 2e-3


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("batch,seq,heads,kind", [(1, 32, 12, "prefix"), (8, 32, 12, "random"), (32, 32, 12, "prefix"),
                                                  (3, 64, 16, "random"), (5, 17, 2, "prefix"), (2, 49, 3, "none"),
                                                  (4, 1, 1, "none"), (3, 32, 4, "empty_row"), (4, 128, 12, "prefix"),
                                                  (3, 100, 2, "random"), (2, 128, 3, "empty_row"), (2, 77, 2, "none"),
                                                  (5, 65, 1, "prefix")])
@pytest.mark.parametrize("tensor_memory", [0, 1])   # binary16 past 64 positions: mma.sync or tcgen05
def test_attention_of_short_sequences_in_one_launch(oracle, t, batch, seq, heads, kind, tensor_memory, kernel_options):
    """cubk_attention_small_* against the three steps it stands for, computed on the host with the reference's
    softmax: scores = scale * Q.K^T rounded to the storage type, masked softmax rounded to the storage type, P.V."""
    if tensor_memory == 1 and not (t == "f16" and seq > 64):
        pytest.skip("the same kernel either way")
    kernel_options(kernels.OPT_ATTENTION_TENSOR_MEMORY, tensor_memory)
    rng = np.random.default_rng(batch * 100 + seq + heads)
    hidden = heads * 64
    qkv, qkvh = _prep(rng.standard_normal((batch * seq, 3 * hidden)), t)
    mask = _mask(rng, batch, seq, kind)
    scale = 0.125
    rc, ctx = G.attention_small(qkv, None if mask is None else G.dev(mask), batch, seq, heads, scale, t)
    if t == "f32" and seq > 64:
        assert rc == kernels.CUBK_ERR_UNSUPPORTED   # 65 to 128 positions: binary16 only
        return
    assert rc == kernels.CUBK_OK
    dt = np.float32 if t == "f32" else np.float16
    x = qkvh.reshape(batch, seq, 3, heads, 64).astype(np.float64)
    q, k, v = x[:, :, 0], x[:, :, 1], x[:, :, 2]
    scores = (scale * np.einsum("bihc,bjhc->bihj", q, k)).astype(np.float32).astype(dt).astype(np.float32)
    probs = oracle.masked_softmax(scores, mask, 1.0).astype(dt).astype(np.float64)
    ref = np.einsum("bihj,bjhc->bihc", probs, v).reshape(batch * seq, hidden)
    got = G.host(ctx).astype(np.float64)
    assert np.all(np.isfinite(got))
    # a probability that falls on the other side of a rounding boundary of the storage type moves one term
    tol = 2e-5 if t == "f32" else 4e-3
    first = 0
    if kind == "empty_row":
        # sequence 0 has every key masked: scores near -10000, where float32 resolves 1e-3 (see test_masked_softmax)
        assert np.max(np.abs(got[:seq] - ref[:seq])) <= 5e-3 * max(1.0, float(np.max(np.abs(ref))))
        first = seq
    err = float(np.max(np.abs(got[first:] - ref[first:])))
    assert err <= tol * max(1.0, float(np.max(np.abs(ref)))), err


@pytest.mark.parametrize("batch,seq,heads", [(2, 32, 3), (3, 50, 2)])
def test_attention_small_binary16_kernels_agree(batch, seq, heads):
    """Binary16 inputs on a 16-byte boundary take the matrix-instruction kernel, any other address the float32-pipe
    kernel: the same rounding points, so the two differ by the order of additions only."""
    rng = np.random.default_rng(seq)
    hidden = heads * 64
    n = batch * seq * 3 * hidden
    flat = torch.zeros(n + 8, dtype=torch.float16, device="cuda")
    vals = G.dev(G.round_f16(rng.standard_normal(n).astype(np.float32)), torch.float16)
    mask = G.dev(_mask(rng, batch, seq, "random"))
    flat[:n] = vals
    rc, aligned = G.attention_small(flat[:n].view(batch * seq, 3 * hidden), mask, batch, seq, heads, 0.125, "f16")
    assert rc == kernels.CUBK_OK and flat.data_ptr() % 16 == 0
    flat[1:n + 1] = vals
    rc, shifted = G.attention_small(flat[1:n + 1].view(batch * seq, 3 * hidden), mask, batch, seq, heads, 0.125, "f16")
    assert rc == kernels.CUBK_OK
    a, b = G.host(aligned).astype(np.float64), G.host(shifted).astype(np.float64)
    assert np.all(np.isfinite(a)) and np.all(np.isfinite(b))
    assert np.max(np.abs(a - b)) <= 4e-3 * max(1.0, float(np.max(np.abs(a))))


def test_attention_small_declines_what_it_does_not_cover():
    lib = kernels.load()
    x = torch.zeros(65 * 3 * 128, device="cuda")
    p, s = x.data_ptr(), G.stream()
    assert lib.cubk_attention_small_f32(p, None, 1, 65, 2, 128, 1.0, p, s) == kernels.CUBK_ERR_UNSUPPORTED   # too long
    assert lib.cubk_attention_small_f16(p, None, 1, 129, 2, 128, 1.0, p, s) == kernels.CUBK_ERR_UNSUPPORTED  # too long
    assert lib.cubk_attention_small_f16(p + 2, None, 1, 65, 2, 128, 1.0, p, s) == kernels.CUBK_ERR_UNSUPPORTED  # past 64: 16-byte rows only
    assert lib.cubk_attention_small_f32(p, None, 1, 32, 2, 96, 1.0, p, s) == kernels.CUBK_ERR_UNSUPPORTED    # head size
    assert lib.cubk_attention_small_f32(None, None, 1, 32, 2, 128, 1.0, p, s) == kernels.CUBK_ERR_INVALID_ARG
    assert lib.cubk_attention_small_f32(p, None, 0, 32, 2, 128, 1.0, p, s) == kernels.CUBK_OK


# ============================================================================ K1 embedding + add + LayerNorm

def _choose_embed_kernel(kernel_options, which):
    kernel_options(kernels.OPT_EMBED_STAGED_ROWS, 1 if which == "staged" else 0)
    kernel_options(kernels.OPT_EXACT_WIDTH_EMBED, 0 if which == "general" else 1)


# which kernel takes the shapes that fit it: the general register-resident one, the one for rows that fill a warp
# exactly, or the one with word rows staged through shared memory
@pytest.mark.parametrize("staged", ["general", "exact", "staged"])
@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("batch,seq,hidden,vocab", [(2, 4, 3, 5), (3, 7, 10, 11), (4, 32, 768, 2000), (2, 128, 1024, 3000),
                                                    (1, 16, 200, 50), (2, 5, 4096, 30), (5, 9, 32, 7), (300, 64, 256, 999),
                                                    (7, 33, 1536, 100)])
def test_embed_ln(oracle, t, batch, seq, hidden, vocab, staged, kernel_options):
    _choose_embed_kernel(kernel_options, staged)
    gave_up_before = kernels.copy_timeouts()
    rng = np.random.default_rng(hidden + vocab)
    word, wh = _prep(rng.standard_normal((vocab, hidden)) * 0.02, t)
    pos, ph = _prep(rng.standard_normal((seq + 3, hidden)) * 0.02, t)
    typ, th = _prep(rng.standard_normal((2, hidden)) * 0.02, t)
    g, gh = _prep(1 + 0.1 * rng.standard_normal(hidden), t)
    be, beh = _prep(0.1 * rng.standard_normal(hidden), t)
    ids = rng.integers(0, vocab, (batch, seq), dtype=np.int32)
    seg = rng.integers(0, 2, (batch, seq)).astype(np.int8)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = G.embed_ln(G.dev(ids), G.dev(seg), word, pos, typ, g, be, t, status)
    ref = oracle.bert_embeddings(ids, seg, wh, ph[:seq], th, beh, gh)
    _check(got, ref, t, 1.0, "embed_ln")
    assert int(status.item()) == 0
    assert kernels.copy_timeouts() == gave_up_before


@pytest.mark.parametrize("t", DTYPES)
def test_embed_ln_sweep_shape_with_the_default_kernel_choice(oracle, t, kernel_options):
    """256 x 128 tokens, hidden 768, vocabulary 21128: float32 takes the staged kernel by default,
    binary16 the register-resident one; every token of the even split over warps is checked."""
    kernel_options(kernels.OPT_EMBED_STAGED_ROWS, -1)
    kernel_options(kernels.OPT_EXACT_WIDTH_EMBED, 1)
    gave_up_before = kernels.copy_timeouts()
    batch, seq, hidden, vocab = 256, 128, 768, 21128
    rng = np.random.default_rng(1)
    word, wh = _prep(rng.standard_normal((vocab, hidden)) * 0.02, t)
    pos, ph = _prep(rng.standard_normal((512, hidden)) * 0.02, t)
    typ, th = _prep(rng.standard_normal((2, hidden)) * 0.02, t)
    g, gh = _prep(1 + 0.1 * rng.standard_normal(hidden), t)
    be, beh = _prep(0.1 * rng.standard_normal(hidden), t)
    ids = rng.integers(0, vocab, (batch, seq), dtype=np.int32)
    seg = rng.integers(0, 2, (batch, seq)).astype(np.int8)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = G.embed_ln(G.dev(ids), G.dev(seg), word, pos, typ, g, be, t, status)
    ref = oracle.bert_embeddings(ids, seg, wh, ph[:seq], th, beh, gh)
    _check(got, ref, t, 1.0, "embed_ln 256x128")
    assert int(status.item()) == 0
    assert kernels.copy_timeouts() == gave_up_before


def test_a_copy_wait_that_runs_out_is_reported_and_leaves_the_context_usable():
    """The staged kernels bound every wait for an asynchronous copy. Here a warp waits (200 polls) for a
    barrier that nothing completes: the kernel must return, set CUBK_STATUS_COPY_TIMEOUT, count the
    give-up, and the next launches on the same context must work."""
    before = kernels.copy_timeouts()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.check(kernels.load().cubk_selftest_copy_wait_timeout(200, G.ptr(status), G.stream()))
    torch.cuda.synchronize()
    assert int(status.item()) == kernels.STATUS_COPY_TIMEOUT
    assert kernels.copy_timeouts() == before + 1
    assert kernels.load().cubk_selftest_copy_wait_timeout(0, None, G.stream()) == kernels.CUBK_ERR_INVALID_ARG
    x = torch.randn(64, 768, device="cuda")
    y = G.bias_gelu(x, None, "f32")
    assert torch.isfinite(y).all() and torch.cuda.current_stream().query() is not None


@pytest.mark.parametrize("staged", ["general", "exact", "staged"])
def test_embed_out_of_range_ids_are_clamped_and_flagged(oracle, staged, kernel_options):
    _choose_embed_kernel(kernel_options, staged)
    rng = np.random.default_rng(0)
    vocab, hidden, seq = 10, 768, 4
    word = rng.standard_normal((vocab, hidden)).astype(np.float32)
    pos = rng.standard_normal((seq, hidden)).astype(np.float32)
    typ = rng.standard_normal((2, hidden)).astype(np.float32)
    g, be = np.ones(hidden, np.float32), np.zeros(hidden, np.float32)
    ids = np.array([[1, 99, -5, 3]], np.int32)
    seg = np.array([[0, 1, 7, -1]], np.int8)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = G.embed_ln(G.dev(ids), G.dev(seg), G.dev(word), G.dev(pos), G.dev(typ), G.dev(g), G.dev(be), "f32", status)
    ref = oracle.bert_embeddings(np.array([[1, 9, 0, 3]], np.int32), np.array([[0, 1, 1, 0]], np.int8),
                                 word, pos, typ, be, g)
    G.assert_close(G.host(got), ref, G.F32_RTOL, 1.0, "clamped")
    assert int(status.item()) == (kernels.STATUS_BAD_TOKEN_ID | kernels.STATUS_BAD_SEGMENT_ID)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("width", [3, 8, 768, 1000])
@pytest.mark.parametrize("idt", [np.int32, np.int8])
def test_embed_gather_bit_exact(dtype, width, idt):
    rng = np.random.default_rng(width)
    vocab = 100
    table = torch.from_numpy(rng.standard_normal((vocab, width)).astype(np.float32)).to(dtype).cuda()
    ids = rng.integers(0, vocab, 777).astype(idt)
    got = G.embed_gather(G.dev(ids), table)
    assert torch.equal(got, table[torch.from_numpy(ids.astype(np.int64)).cuda()])


# ============================================================================ K5b mean pool, K5c classifier head

@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("batch,seq,hidden", [(2, 3, 2), (3, 5, 7), (4, 32, 768), (2, 512, 1024), (64, 512, 1024),
                                              (1, 128, 768), (300, 16, 64), (2, 100, 200), (80, 200, 1000), (700, 128, 24)])
def test_mean_pool(oracle, t, batch, seq, hidden):
    rng = np.random.default_rng(batch + seq + hidden)
    x, xh = _prep(rng.standard_normal((batch, seq, hidden)), t)
    got = G.mean_pool(x, t)
    _check(got, oracle.reduce_mean_1(xh), t, 0.1, "mean_pool")


def test_mean_pool_scratch_contract():
    lib = kernels.load()
    assert lib.cubk_mean_pool_scratch_bytes(512, 512, 1024) == 0      # enough blocks without splitting
    need = lib.cubk_mean_pool_scratch_bytes(2, 512, 1024)
    assert need > 0
    x = torch.randn((2, 512, 1024), device="cuda")
    out = torch.empty((2, 1024), device="cuda")
    rc = lib.cubk_mean_pool_f32(x.data_ptr(), 2, 512, 1024, out.data_ptr(), None, 0, G.stream())
    assert rc == kernels.CUBK_ERR_SCRATCH
    small = torch.empty(need - 4, dtype=torch.uint8, device="cuda")
    rc = lib.cubk_mean_pool_f32(x.data_ptr(), 2, 512, 1024, out.data_ptr(), small.data_ptr(), need - 4, G.stream())
    assert rc == kernels.CUBK_ERR_SCRATCH


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("batch,hidden,labels,bias", [(1, 768, 2, True), (256, 768, 2, True), (7, 1024, 8, False),
                                                      (33, 64, 1, True), (5, 2048, 3, True), (3, 8, 5, True)])
def test_pooler_activation_and_classifier_in_one_launch(oracle, t, batch, hidden, labels, bias):
    """cubk_pooler_head_* against the two calls it stands for: the pooled row bit for bit, logits and probs as
    the classifier gives them on the STORED pooled row (only the order of the dot product's additions differs)."""
    rng = np.random.default_rng(batch * 7 + hidden + labels)
    x, _ = _prep(rng.standard_normal((batch, hidden)) * 2, t)
    pb, _ = _prep(rng.standard_normal(hidden), t)
    w, wh = _prep(rng.standard_normal((labels, hidden)) * 0.1, t)
    b, bh = _prep(rng.standard_normal(labels), t) if bias else (None, None)
    rc, pooled, logits, probs = G.pooler_head(x, pb, w, b, t)
    assert rc == kernels.CUBK_OK
    assert torch.equal(pooled, G.bias_tanh(x, pb, t))
    two_l, two_p = G.logits_probs(pooled, w, b, t)
    ref_logits, ref_probs = oracle.classifier(G.host(pooled), wh, bh)
    _check(logits, ref_logits, t, 1.0, "logits")
    _check(logits, G.host(two_l), t, 1.0, "logits against the separate call")
    if t == "f32":
        _check(probs, ref_probs, t, 1e-3, "probs")
    else:
        _check(probs, oracle.softmax_(G.host(logits)), t, 1e-1, "probs of stored logits")
        assert np.max(np.abs(G.host(probs) - ref_probs)) <= G.F16_ATOL
    # in place, and without probs
    x2 = x.clone()
    lib = kernels.load()
    f = getattr(lib, "cubk_pooler_head_" + t)
    logits2 = torch.empty_like(logits)
    assert f(x2.data_ptr(), pb.data_ptr(), w.data_ptr(), G.ptr(b), batch, hidden, labels, x2.data_ptr(),
             logits2.data_ptr(), None, G.stream()) == kernels.CUBK_OK
    assert torch.equal(x2, pooled) and torch.equal(logits2, logits)


def test_pooler_head_declines_what_it_does_not_cover():
    lib = kernels.load()
    x = torch.zeros((2, 4096), device="cuda")
    s = G.stream()
    p = x.data_ptr()
    assert lib.cubk_pooler_head_f32(p, p, p, None, 2, 768, 9, p, p, None, s) == kernels.CUBK_ERR_UNSUPPORTED      # labels
    assert lib.cubk_pooler_head_f32(p, p, p, None, 2, 770, 2, p, p, None, s) == kernels.CUBK_ERR_UNSUPPORTED      # width
    assert lib.cubk_pooler_head_f32(p, p, p, None, 2, 4096, 2, p, p, None, s) == kernels.CUBK_ERR_UNSUPPORTED     # too wide
    assert lib.cubk_pooler_head_f32(p + 4, p, p, None, 2, 768, 2, p, p, None, s) == kernels.CUBK_ERR_UNSUPPORTED  # alignment
    assert lib.cubk_pooler_head_f32(None, p, p, None, 2, 768, 2, p, p, None, s) == kernels.CUBK_ERR_INVALID_ARG
    assert lib.cubk_pooler_head_f32(p, p, p, None, 2, 768, 0, p, p, None, s) == kernels.CUBK_ERR_INVALID_ARG
    torch.cuda.synchronize()
    assert bool((x == 0).all())


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("batch,hidden,labels,bias", [(2, 3, 1, False), (128, 768, 2, True), (5, 1024, 3, True),
                                                      (3, 100, 37, True), (2, 64, 1000, False)])
def test_logits_probs(oracle, t, batch, hidden, labels, bias):
    rng = np.random.default_rng(batch + hidden + labels)
    x, xh = _prep(rng.standard_normal((batch, hidden)), t)
    w, wh = _prep(rng.standard_normal((labels, hidden)) * 0.1, t)
    b, bh = _prep(rng.standard_normal(labels), t) if bias else (None, None)
    logits, probs = G.logits_probs(x, w, b, t)
    ref_logits, ref_probs = oracle.classifier(xh, wh, bh)
    _check(logits, ref_logits, t, 1.0, "logits")
    if t == "f32":
        _check(probs, ref_probs, t, 1e-3, "probs")
    else:
        # As in the reference, the softmax reads the logits back in storage precision
        # (src/cuBERT/op_out/AdditionalOutputLayer.cpp:61-64): probs must be the softmax of the
        # binary16 logits we stored, and within the 1e-2 bar of the float32 oracle.
        _check(probs, oracle.softmax_(G.host(logits)), t, 1e-1, "probs of stored logits")
        assert np.max(np.abs(G.host(probs) - ref_probs)) <= G.F16_ATOL


# ============================================================================ helpers and argument checking

def test_half_to_float_and_not():
    rng = np.random.default_rng(1)
    for n in (1, 7, 8, 1000, 4099):
        h = torch.from_numpy(rng.standard_normal(n).astype(np.float16)).cuda()
        assert torch.equal(G.half_to_float(h), h.float())
        m = torch.from_numpy(rng.integers(-2, 3, n).astype(np.int8)).cuda()
        assert torch.equal(G.logical_not(m, "f16").float(), (m == 0).float())


def test_argument_checks_and_empty_inputs():
    lib = kernels.load()
    x = torch.zeros((4, 8), device="cuda")
    s = G.stream()
    assert lib.cubk_bias_residual_ln_f32(None, None, None, x.data_ptr(), x.data_ptr(), 4, 8, x.data_ptr(), s) \
        == kernels.CUBK_ERR_INVALID_ARG
    assert lib.cubk_bias_gelu_f32(x.data_ptr(), None, 4, 0, x.data_ptr(), s) == kernels.CUBK_ERR_INVALID_ARG
    assert lib.cubk_masked_softmax_f32(x.data_ptr(), x.data_ptr(), 4, 0, 8, 1.0, x.data_ptr(), s) \
        == kernels.CUBK_ERR_INVALID_ARG
    assert lib.cubk_logits_probs_f32(x.data_ptr(), x.data_ptr(), None, 4, 8, 5000, x.data_ptr(), None, s) \
        == kernels.CUBK_ERR_UNSUPPORTED
    # batch 0 / rows 0: success, nothing launched (src/cuBERT/Bert.cpp:102-103 returns silently)
    assert lib.cubk_bias_residual_ln_f32(x.data_ptr(), None, None, x.data_ptr(), x.data_ptr(), 0, 8, x.data_ptr(), s) == 0
    assert lib.cubk_bias_gelu_f32(x.data_ptr(), None, 0, 8, x.data_ptr(), s) == 0
    assert lib.cubk_masked_softmax_f32(x.data_ptr(), None, 0, 1, 8, 1.0, x.data_ptr(), s) == 0
    assert lib.cubk_mean_pool_f32(x.data_ptr(), 0, 4, 8, x.data_ptr(), None, 0, s) == 0
    torch.cuda.synchronize()


# ============================================================================ guard bands around every buffer
# compute-sanitizer is not available for these kernels, so out-of-bounds writes are looked for the
# plain way: every input and output sits between two bands of a sentinel value, and the bands (and the
# inputs) must be untouched after the launch.

class _Guarded:
    PAD = 128          # elements; keeps the payload 16-byte aligned for every dtype used here

    def __init__(self, shape, dtype, fill=None, misalign=0):
        n = int(np.prod(shape))
        self.sentinel = 113
        self.buf = torch.full((n + 2 * self.PAD + misalign,), self.sentinel, dtype=dtype, device="cuda")
        self.view = self.buf[self.PAD + misalign: self.PAD + misalign + n].view(*shape)
        if fill is not None:
            self.view.copy_(fill.to(dtype))
        self.before = self.view.clone()
        self.lo, self.hi = self.PAD + misalign, self.PAD + misalign + n

    def bands_intact(self):
        return bool((self.buf[:self.lo] == self.sentinel).all() and (self.buf[self.hi:] == self.sentinel).all())

    def unchanged(self):
        return self.bands_intact() and torch.equal(self.view, self.before)


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("rows,ch,misalign", [(1, 8, 0), (3, 768, 0), (37, 776, 0), (5, 3072, 0), (9, 4096, 0), (2, 8200, 0),
                                              (7, 33, 0), (4, 100, 1), (3, 768, 1)])
def test_row_kernels_stay_inside_their_buffers(t, rows, ch, misalign):
    dt = G.TORCH_DTYPE[t]
    g = torch.Generator(device="cuda").manual_seed(rows * 7919 + ch)
    rnd = lambda *shape: torch.randn(*shape, device="cuda", generator=g)  # noqa: E731
    x, res = _Guarded((rows, ch), dt, rnd(rows, ch), misalign), _Guarded((rows, ch), dt, rnd(rows, ch), misalign)
    bias, gamma, beta = (_Guarded((ch,), dt, rnd(ch), misalign) for _ in range(3))
    out = _Guarded((rows, ch), dt, None, misalign)
    inputs = (x, res, bias, gamma, beta)
    kernels.check(G.fn("bias_residual_ln", t)(G.ptr(x.view), G.ptr(bias.view), G.ptr(res.view), G.ptr(gamma.view),
                                              G.ptr(beta.view), rows, ch, G.ptr(out.view), G.stream()))
    torch.cuda.synchronize()
    assert out.bands_intact() and all(i.unchanged() for i in inputs), "bias_residual_ln"
    assert torch.isfinite(out.view.float()).all()
    for name in ("bias_gelu", "bias_tanh"):
        out = _Guarded((rows, ch), dt, None, misalign)
        kernels.check(G.fn(name, t)(G.ptr(x.view), G.ptr(bias.view), rows, ch, G.ptr(out.view), G.stream()))
        torch.cuda.synchronize()
        assert out.bands_intact() and all(i.unchanged() for i in inputs), name
    # in place: the bands of the one buffer
    y = _Guarded((rows, ch), dt, x.view, misalign)
    kernels.check(G.fn("bias_gelu", t)(G.ptr(y.view), G.ptr(bias.view), rows, ch, G.ptr(y.view), G.stream()))
    torch.cuda.synchronize()
    assert y.bands_intact() and bias.unchanged()


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("batch,heads,seq", [(1, 1, 8), (3, 2, 32), (2, 12, 128), (2, 3, 512), (1, 2, 2048), (2, 2, 40),
                                             (5, 1, 7), (2, 2, 264)])
def test_softmax_and_pool_stay_inside_their_buffers(t, batch, heads, seq):
    dt = G.TORCH_DTYPE[t]
    g = torch.Generator(device="cuda").manual_seed(batch * 31 + seq)
    rows = batch * seq * heads
    scores = _Guarded((rows, seq), dt, torch.randn(rows, seq, device="cuda", generator=g) * 3)
    mask = _Guarded((batch, seq), torch.int8, (torch.rand(batch, seq, device="cuda", generator=g) > 0.3).to(torch.int8))
    out = _Guarded((rows, seq), dt)
    kernels.check(G.fn("masked_softmax", t)(G.ptr(scores.view), G.ptr(mask.view), rows, seq * heads, seq, 0.125,
                                            G.ptr(out.view), G.stream()))
    torch.cuda.synchronize()
    assert out.bands_intact() and scores.unchanged() and mask.unchanged()
    assert torch.allclose(out.view.float().sum(dim=1), torch.ones(rows, device="cuda"), atol=2e-2 if t == "f16" else 1e-4)
    # mean pool over [batch, seq, hidden] with the library's own scratch sizing
    hidden = 8 * heads * 4
    x = _Guarded((batch, seq, hidden), dt, torch.randn(batch, seq, hidden, device="cuda", generator=g))
    pooled = _Guarded((batch, hidden), dt)
    need = kernels.load().cubk_mean_pool_scratch_bytes(batch, seq, hidden)
    scratch = _Guarded((max(need // 4, 1),), torch.float32)
    kernels.check(G.fn("mean_pool", t)(G.ptr(x.view), batch, seq, hidden, G.ptr(pooled.view), G.ptr(scratch.view), need,
                                       G.stream()))
    torch.cuda.synchronize()
    assert pooled.bands_intact() and scratch.bands_intact() and x.unchanged()


@pytest.mark.parametrize("t", DTYPES)
@pytest.mark.parametrize("staged", ["general", "exact", "staged"])
@pytest.mark.parametrize("batch,seq,hidden,vocab", [(1, 1, 8, 3), (3, 5, 768, 50), (2, 7, 1024, 9), (9, 3, 40, 4), (4, 4, 4096, 6)])
def test_embedding_kernels_stay_inside_their_buffers(t, staged, batch, seq, hidden, vocab, kernel_options):
    _choose_embed_kernel(kernel_options, staged)
    dt = G.TORCH_DTYPE[t]
    g = torch.Generator(device="cuda").manual_seed(hidden + vocab)
    rnd = lambda *shape: torch.randn(*shape, device="cuda", generator=g) * 0.1  # noqa: E731
    word, pos, typ = _Guarded((vocab, hidden), dt, rnd(vocab, hidden)), _Guarded((seq, hidden), dt, rnd(seq, hidden)), \
        _Guarded((2, hidden), dt, rnd(2, hidden))
    gamma, beta = _Guarded((hidden,), dt, 1 + rnd(hidden)), _Guarded((hidden,), dt, rnd(hidden))
    ids = _Guarded((batch, seq), torch.int32, torch.randint(-2, vocab + 2, (batch, seq), device="cuda", generator=g))
    seg = _Guarded((batch, seq), torch.int8, torch.randint(-1, 3, (batch, seq), device="cuda", generator=g))
    status = _Guarded((1,), torch.int32, torch.zeros(1))
    out = _Guarded((batch, seq, hidden), dt)
    kernels.check(G.fn("embed_ln", t)(G.ptr(ids.view), G.ptr(seg.view), G.ptr(word.view), G.ptr(pos.view), G.ptr(typ.view),
                                      G.ptr(gamma.view), G.ptr(beta.view), batch, seq, hidden, vocab, 2, G.ptr(out.view),
                                      G.ptr(status.view), G.stream()))
    torch.cuda.synchronize()
    assert out.bands_intact() and status.bands_intact()
    assert all(i.unchanged() for i in (word, pos, typ, gamma, beta, ids, seg))
    assert torch.isfinite(out.view.float()).all()
    # plain gather and its inverse
    rows = _Guarded((batch * seq, hidden), dt)
    kernels.check(kernels.load().cubk_embed_gather_i32(G.ptr(ids.view), batch * seq, G.ptr(word.view), vocab, hidden,
                                                       word.view.element_size(), G.ptr(rows.view), G.ptr(status.view),
                                                       G.stream()))
    table2 = _Guarded((vocab, hidden), dt, word.view)
    kernels.check(kernels.load().cubk_scatter_rows(G.ptr(ids.view), batch * seq, G.ptr(rows.view), hidden,
                                                   word.view.element_size(), G.ptr(table2.view), vocab, G.stream()))
    torch.cuda.synchronize()
    assert rows.bands_intact() and table2.bands_intact() and word.unchanged() and ids.unchanged()
