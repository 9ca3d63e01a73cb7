"""Test-side helpers that drive the CUDA kernels through the C ABI with torch device buffers.

torch is used for device memory and streams only; every computation under test goes
through ``libcubert_kernels.so``.
"""
import numpy as np
import torch

from cubert_b200 import kernels

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16}
NP_DTYPE = {"f32": np.float32, "f16": np.float16}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def ptr(t):
    return None if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def fn(name, t):
    return getattr(kernels.load(), "cubk_%s_%s" % (name, t))


def bias_residual_ln(x, bias, residual, gamma, beta, t="f32", inplace=False):
    """x, residual: torch [rows, C] on device (dtype of t). Returns torch tensor."""
    rows, ch = x.shape
    out = x if inplace else torch.empty_like(x)
    rc = fn("bias_residual_ln", t)(ptr(x), ptr(bias), ptr(residual), ptr(gamma), ptr(beta), rows, ch, ptr(out),
                                   stream())
    kernels.check(rc)
    return out


def bias_gelu(x, bias, t="f32", inplace=False):
    rows, ch = x.shape
    out = x if inplace else torch.empty_like(x)
    kernels.check(fn("bias_gelu", t)(ptr(x), ptr(bias), rows, ch, ptr(out), stream()))
    return out


def bias_tanh(x, bias, t="f32", inplace=False):
    rows, ch = x.shape
    out = x if inplace else torch.empty_like(x)
    kernels.check(fn("bias_tanh", t)(ptr(x), ptr(bias), rows, ch, ptr(out), stream()))
    return out


def masked_softmax(scores, mask, rows_per_batch, scale=1.0, t="f32", inplace=False):
    """scores: torch [rows, S]; mask: torch int8 [B, S] or None."""
    rows, seq = scores.shape
    out = scores if inplace else torch.empty_like(scores)
    kernels.check(fn("masked_softmax", t)(ptr(scores), ptr(mask), rows, rows_per_batch, seq, float(scale),
                                          ptr(out), stream()))
    return out


def masked_softmax_extents(scores, mask, extents, zero_to, rows_per_batch, scale=1.0, t="f32", out=None):
    """As masked_softmax, with per-batch-entry key extents (torch int32 [B]); `out` defaults to a new tensor
    filled with NaN so that untouched columns can be told apart."""
    rows, seq = scores.shape
    if out is None:
        out = torch.full_like(scores, float("nan"))
    kernels.check(fn("masked_softmax_extents", t)(ptr(scores), ptr(mask), ptr(extents), int(zero_to), rows,
                                                  rows_per_batch, seq, float(scale), ptr(out), stream()))
    return out


def pooler_head(x, pooler_bias, weights, bias, t="f32", want_probs=True):
    """(status, pooled, logits, probs) of the one-launch pooler activation + classifier."""
    batch, hidden = x.shape
    labels = weights.shape[0]
    pooled = torch.full_like(x, float("nan"))
    logits = torch.full((batch, labels), float("nan"), dtype=x.dtype, device="cuda")
    probs = torch.full((batch, labels), float("nan"), dtype=x.dtype, device="cuda") if want_probs else None
    rc = fn("pooler_head", t)(ptr(x), ptr(pooler_bias), ptr(weights), ptr(bias), batch, hidden, labels, ptr(pooled),
                              ptr(logits), ptr(probs), stream())
    return rc, pooled, logits, probs


def attention_small(qkv, mask, batch, seq, heads, scale, t="f32"):
    """qkv: torch [batch * seq, 3 * hidden]; returns (status, context [batch * seq, hidden])."""
    hidden = qkv.shape[1] // 3
    ctx = torch.full((batch * seq, hidden), float("nan"), dtype=qkv.dtype, device="cuda")
    rc = fn("attention_small", t)(ptr(qkv), ptr(mask), batch, seq, heads, hidden, float(scale), ptr(ctx), stream())
    return rc, ctx


def embed_ln(ids, seg, word, pos, typ, gamma, beta, t="f32", status=None):
    b, s = ids.shape
    vocab, hidden = word.shape
    out = torch.empty((b, s, hidden), dtype=word.dtype, device="cuda")
    kernels.check(fn("embed_ln", t)(ptr(ids), ptr(seg), ptr(word), ptr(pos), ptr(typ), ptr(gamma), ptr(beta),
                                    b, s, hidden, vocab, typ.shape[0], ptr(out), ptr(status), stream()))
    return out


def embed_gather(ids, table, status=None):
    n = ids.numel()
    vocab, width = table.shape
    out = torch.empty((n, width), dtype=table.dtype, device="cuda")
    name = "cubk_embed_gather_i8" if ids.dtype == torch.int8 else "cubk_embed_gather_i32"
    kernels.check(getattr(kernels.load(), name)(ptr(ids), n, ptr(table), vocab, width, table.element_size(),
                                                ptr(out), ptr(status), stream()))
    return out


def mean_pool(x, t="f32", scratch="auto"):
    b, s, h = x.shape
    out = torch.empty((b, h), dtype=x.dtype, device="cuda")
    need = kernels.load().cubk_mean_pool_scratch_bytes(b, s, h)
    buf = None
    if scratch == "auto" and need:
        buf = torch.empty(need, dtype=torch.uint8, device="cuda")
    rc = fn("mean_pool", t)(ptr(x), b, s, h, ptr(out), ptr(buf), need if buf is not None else 0, stream())
    kernels.check(rc)
    return out


def logits_probs(pooled, w, bias, t="f32", want_probs=True):
    b, h = pooled.shape
    labels = w.shape[0]
    logits = torch.empty((b, labels), dtype=pooled.dtype, device="cuda")
    probs = torch.empty((b, labels), dtype=pooled.dtype, device="cuda") if want_probs else None
    kernels.check(fn("logits_probs", t)(ptr(pooled), ptr(w), ptr(bias), b, h, labels, ptr(logits), ptr(probs),
                                        stream()))
    return logits, probs


def logical_not(mask, t="f32"):
    out = torch.empty(mask.shape, dtype=TORCH_DTYPE[t], device="cuda")
    kernels.check(fn("not", t)(ptr(mask), ptr(out), mask.numel(), stream()))
    return out


def half_to_float(x):
    out = torch.empty(x.shape, dtype=torch.float32, device="cuda")
    kernels.check(kernels.load().cubk_half_to_float(ptr(x), ptr(out), x.numel(), stream()))
    return out


def copy_from_device(address, shape, dtype):
    """numpy copy of a raw device allocation (cudaMemcpy device-to-host through the CUDA runtime)."""
    import ctypes
    out = np.empty(shape, dtype)
    cudart = ctypes.CDLL("libcudart.so.12")
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    torch.cuda.synchronize()
    rc = cudart.cudaMemcpy(out.ctypes.data, address, out.nbytes, 2)
    assert rc == 0, rc
    return out


def host(t):
    torch.cuda.synchronize()
    return t.detach().float().cpu().numpy()


# ---------------------------------------------------------------------------------- tolerances
# float32 storage: 1e-5 relative (the bar stated for this path). "Relative" is taken
# per element against max(|ref|, floor) where `floor` is a per-op magnitude floor that keeps
# results that are small only through cancellation (LayerNorm outputs near zero, GELU of very
# negative inputs) from demanding more digits than float32 arithmetic on O(1) operands has.
F32_RTOL = 1e-5
# binary16 storage: the inputs are rounded to binary16 first and the CPU checker runs on those
# rounded values in float32, so the only difference left is our float32 math plus one final
# rounding to binary16 (relative 2^-11 = 4.9e-4). The bar for this path is 1e-2 absolute.
F16_RTOL = 1e-3
F16_ATOL = 1e-2


def assert_close(got, ref, rtol, floor, what=""):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.all(np.isfinite(got)), "non-finite output " + what
    err = np.abs(got - ref)
    bound = rtol * np.maximum(np.abs(ref), floor)
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err / bound), err.shape)
        raise AssertionError("%s: %d of %d elements outside rtol=%g (floor %g); worst at %s: got %r want %r"
                             % (what, bad.sum(), bad.size, rtol, floor, i, got[i], ref[i]))


def round_f16(a):
    """float32 array rounded through binary16 (round to nearest even), back as float32."""
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
