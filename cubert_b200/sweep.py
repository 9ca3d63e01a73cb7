"""Isolated sweep of the fused kernels: achieved HBM GB/s per kernel and shape.

    python -m cubert_b200.sweep [--quick] [--large] [--only ln,gelu,softmax,embed,pool,attention] [--dtype f16,f32]
                                [--iters N] [--json out.json]

Each case is timed with CUDA events on the launching stream: `iters` back-to-back launches
rotating over enough distinct buffer sets to exceed the 126 MB L2 (or, for tensors that are
themselves larger than L2, a single set), after 3 warm-up launches. Reported bandwidth is
ALGORITHMIC bytes / time:

    bias+residual+LN   3*rows*C*e + 3*C*e
    bias+GELU          2*rows*C*e + C*e
    masked softmax     2*B*H*S*S*e + B*S
    embed+LN           2*B*S*H*e + 5*B*S + S*H*e + type_vocab*H*e + 2*H*e
    mean pool          B*S*H*e + B*H*e
    one-launch attention  4*B*S*H*e + B*S   (Q, K, V read, context written; latency-bound at its sizes)

torch provides device memory and the stream only.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

from cubert_b200 import kernels

L2_BYTES = 126 * 1024 * 1024
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


USE_GRAPH = True


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _time(launch, nsets, iters, warmup=3):
    """Seconds per launch. The `iters` launches are captured into one CUDA graph and replayed,
    so that the host's launch cost (Python + ctypes) is not part of the device time."""
    for i in range(warmup):
        launch(i % nsets)
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    if USE_GRAPH:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                launch(i % nsets)
        graph.replay()  # warm replay
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream()
        start.record(stream)
        graph.replay()
        stop.record(stream)
    else:
        stream = torch.cuda.current_stream()
        start.record(stream)
        for i in range(iters):
            launch(i % nsets)
        stop.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters * 1e-3


def _nsets(bytes_per_set, budget=8 << 30):
    if bytes_per_set >= 2 * L2_BYTES:
        return 1
    n = int(np.ceil(2.5 * L2_BYTES / bytes_per_set))
    return max(1, min(n, budget // max(bytes_per_set, 1)))


def _dt(t):
    return torch.float32 if t == "f32" else torch.float16


def _fn(name, t):
    return getattr(kernels.load(), "cubk_%s_%s" % (name, t))


def case_ln(t, rows, ch, iters):
    e = 4 if t == "f32" else 2
    per_set = 3 * rows * ch * e
    n = _nsets(per_set)
    g = torch.Generator(device="cuda").manual_seed(1)
    xs = [torch.randn((rows, ch), device="cuda", generator=g, dtype=torch.float32).to(_dt(t)) for _ in range(n)]
    rs = [torch.randn((rows, ch), device="cuda", generator=g, dtype=torch.float32).to(_dt(t)) for _ in range(n)]
    outs = [torch.empty((rows, ch), device="cuda", dtype=_dt(t)) for _ in range(n)]
    bias = torch.randn(ch, device="cuda").to(_dt(t))
    gamma = torch.ones(ch, device="cuda", dtype=_dt(t))
    beta = torch.zeros(ch, device="cuda", dtype=_dt(t))
    f = _fn("bias_residual_ln", t)

    def launch(i):
        kernels.check(f(xs[i].data_ptr(), bias.data_ptr(), rs[i].data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                        rows, ch, outs[i].data_ptr(), _stream()))

    sec = _time(launch, n, iters)
    return dict(kernel="bias_residual_ln", dtype=t, shape=[rows, ch], bytes=per_set + 3 * ch * e, sec=sec, sets=n)


def case_gelu(t, rows, ch, iters):
    e = 4 if t == "f32" else 2
    per_set = 2 * rows * ch * e
    n = _nsets(per_set)
    g = torch.Generator(device="cuda").manual_seed(1)
    xs = [torch.randn((rows, ch), device="cuda", generator=g, dtype=torch.float32).to(_dt(t)) for _ in range(n)]
    outs = [torch.empty((rows, ch), device="cuda", dtype=_dt(t)) for _ in range(n)]
    bias = torch.randn(ch, device="cuda").to(_dt(t))
    f = _fn("bias_gelu", t)

    def launch(i):
        kernels.check(f(xs[i].data_ptr(), bias.data_ptr(), rows, ch, outs[i].data_ptr(), _stream()))

    sec = _time(launch, n, iters)
    return dict(kernel="bias_gelu", dtype=t, shape=[rows, ch], bytes=per_set + ch * e, sec=sec, sets=n)


def case_softmax(t, batch, seq, iters, heads=12):
    e = 4 if t == "f32" else 2
    rows = batch * heads * seq
    per_set = 2 * rows * seq * e
    n = _nsets(per_set)
    g = torch.Generator(device="cuda").manual_seed(1)
    xs = [(torch.randn((rows, seq), device="cuda", generator=g, dtype=torch.float32) * 3).to(_dt(t)) for _ in range(n)]
    outs = [torch.empty((rows, seq), device="cuda", dtype=_dt(t)) for _ in range(n)]
    lens = torch.randint(max(1, seq // 16), seq + 1, (batch,), device="cuda", generator=g)
    mask = (torch.arange(seq, device="cuda")[None, :] < lens[:, None]).to(torch.int8).contiguous()
    f = _fn("masked_softmax", t)

    def launch(i):
        kernels.check(f(xs[i].data_ptr(), mask.data_ptr(), rows, heads * seq, seq, 0.125, outs[i].data_ptr(), _stream()))

    sec = _time(launch, n, iters)
    return dict(kernel="masked_softmax", dtype=t, shape=[batch, heads, seq, seq], bytes=per_set + batch * seq,
                sec=sec, sets=n)


def case_embed(t, batch, seq, iters, hidden=768, vocab=21128):
    e = 4 if t == "f32" else 2
    per_set = 2 * batch * seq * hidden * e
    n = _nsets(per_set)
    g = torch.Generator(device="cuda").manual_seed(1)
    word = (torch.randn((vocab, hidden), device="cuda", generator=g) * 0.02).to(_dt(t))
    pos = (torch.randn((512, hidden), device="cuda", generator=g) * 0.02).to(_dt(t))
    typ = (torch.randn((2, hidden), device="cuda", generator=g) * 0.02).to(_dt(t))
    gamma = torch.ones(hidden, device="cuda", dtype=_dt(t))
    beta = torch.zeros(hidden, device="cuda", dtype=_dt(t))
    ids = [torch.randint(0, vocab, (batch, seq), device="cuda", generator=g, dtype=torch.int32) for _ in range(n)]
    seg = torch.randint(0, 2, (batch, seq), device="cuda", generator=g).to(torch.int8)
    outs = [torch.empty((batch, seq, hidden), device="cuda", dtype=_dt(t)) for _ in range(n)]
    f = _fn("embed_ln", t)

    def launch(i):
        kernels.check(f(ids[i].data_ptr(), seg.data_ptr(), word.data_ptr(), pos.data_ptr(), typ.data_ptr(),
                        gamma.data_ptr(), beta.data_ptr(), batch, seq, hidden, vocab, 2, outs[i].data_ptr(),
                        None, _stream()))

    sec = _time(launch, n, iters)
    nbytes = per_set + 5 * batch * seq + seq * hidden * e + 2 * hidden * e + 2 * hidden * e
    return dict(kernel="embed_ln", dtype=t, shape=[batch, seq, hidden], bytes=nbytes, sec=sec, sets=n)


def case_pool(t, batch, seq, hidden, iters):
    e = 4 if t == "f32" else 2
    per_set = batch * seq * hidden * e
    n = _nsets(per_set)
    g = torch.Generator(device="cuda").manual_seed(1)
    xs = [torch.randn((batch, seq, hidden), device="cuda", generator=g, dtype=torch.float32).to(_dt(t)) for _ in range(n)]
    out = torch.empty((batch, hidden), device="cuda", dtype=_dt(t))
    need = kernels.load().cubk_mean_pool_scratch_bytes(batch, seq, hidden)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    f = _fn("mean_pool", t)

    def launch(i):
        kernels.check(f(xs[i].data_ptr(), batch, seq, hidden, out.data_ptr(), scratch.data_ptr(), need, _stream()))

    sec = _time(launch, n, iters)
    return dict(kernel="mean_pool", dtype=t, shape=[batch, seq, hidden], bytes=per_set + batch * hidden * e,
                sec=sec, sets=n)


def case_attention(t, batch, seq, iters, heads=12):
    """The one-launch attention (binary16: up to 128 positions; float32: up to 64)."""
    if t == "f32" and seq > 64:
        return None
    e = 4 if t == "f32" else 2
    hidden = 64 * heads
    per_set = 4 * batch * seq * hidden * e
    n = min(64, _nsets(per_set))
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = [torch.randn((batch * seq, 3 * hidden), device="cuda", generator=g, dtype=torch.float32).to(_dt(t))
           for _ in range(n)]
    outs = [torch.empty((batch * seq, hidden), device="cuda", dtype=_dt(t)) for _ in range(n)]
    lens = torch.randint(4, seq + 1, (batch,), device="cuda", generator=g)
    mask = (torch.arange(seq, device="cuda")[None, :] < lens[:, None]).to(torch.int8).contiguous()
    f = _fn("attention_small", t)

    def launch(i):
        kernels.check(f(qkv[i].data_ptr(), mask.data_ptr(), batch, seq, heads, hidden, 0.125, outs[i].data_ptr(),
                        _stream()))

    sec = _time(launch, n, iters)
    return dict(kernel="attention_small", dtype=t, shape=[batch, seq, hidden], bytes=per_set + batch * seq, sec=sec,
                sets=n)


def run(only=None, dtypes=("f16", "f32"), quick=False, iters=20, large=False):
    kernels.load()
    peak, peak_kind = measured_peak_gbs()
    rows_list = [4096, 65536] if quick else [4096, 32768, 65536, 1048576]
    results = []

    def want(k):
        return only is None or k in only

    if large:
        # the shapes of BERT-large at seq 512 (hidden 1024, intermediate 4096, 16 heads), 64 sequences
        for t in dtypes:
            if want("ln"):
                results.append(case_ln(t, 65536, 1024, iters))
            if want("gelu"):
                results.append(case_gelu(t, 65536, 4096, iters))
            if want("softmax"):
                results.append(case_softmax(t, 64, 512, iters, heads=16))
            if want("embed"):
                results.append(case_embed(t, 64, 512, iters, hidden=1024, vocab=30522))
            if want("pool"):
                results.append(case_pool(t, 64, 512, 1024, iters))
            torch.cuda.empty_cache()
        dtypes = ()
    for t in dtypes:
        if want("ln"):
            for ch in (768, 3072):
                for rows in rows_list:
                    results.append(case_ln(t, rows, ch, iters))
                    torch.cuda.empty_cache()
        if want("gelu"):
            for ch in (768, 3072):
                for rows in rows_list:
                    results.append(case_gelu(t, rows, ch, iters))
                    torch.cuda.empty_cache()
        if want("softmax"):
            for (b, s) in ((128, 32), (256, 128), (64, 512)):
                results.append(case_softmax(t, b, s, iters))
                torch.cuda.empty_cache()
        if want("embed"):
            for (b, s) in ((128, 32), (256, 128), (64, 512)):
                results.append(case_embed(t, b, s, iters))
                torch.cuda.empty_cache()
        if want("pool"):
            for (b, s, h) in ((64, 512, 1024), (512, 512, 1024)):
                results.append(case_pool(t, b, s, h, iters))
                torch.cuda.empty_cache()
        if want("attention"):
            for (b, s) in ((1, 32), (8, 32), (16, 32), (32, 32), (128, 32), (8, 64), (32, 64), (64, 128), (256, 128)):
                r = case_attention(t, b, s, iters)
                if r is not None:
                    results.append(r)
                torch.cuda.empty_cache()
    for r in results:
        r["gbs"] = r["bytes"] / r["sec"] / 1e9
        r["frac_of_%s_peak" % peak_kind] = r["gbs"] / peak
        r["us"] = r["sec"] * 1e6
    return results, peak, peak_kind


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default=None)
    ap.add_argument("--dtype", default="f16,f32")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--no-graph", action="store_true", help="time plain stream launches instead of a graph replay")
    ap.add_argument("--large", action="store_true", help="the BERT-large / seq 512 shapes instead of the BERT-base sweep")
    a = ap.parse_args()
    global USE_GRAPH
    USE_GRAPH = not a.no_graph
    if not torch.cuda.is_available():
        sys.exit("cubert_b200.sweep needs a CUDA device")
    results, peak, kind = run(a.only.split(",") if a.only else None, a.dtype.split(","), a.quick, a.iters, a.large)
    print("peak HBM %.0f GB/s (%s)" % (peak, kind))
    print("%-18s %-4s %-22s %10s %10s %8s %5s" % ("kernel", "dt", "shape", "us", "GB/s", "frac", "sets"))
    for r in results:
        print("%-18s %-4s %-22s %10.1f %10.0f %8.3f %5d" % (r["kernel"], r["dtype"], "x".join(map(str, r["shape"])),
                                                          r["us"], r["gbs"], r["gbs"] / peak, r["sets"]))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(dict(peak_gbs=peak, peak_kind=kind, results=results), f, indent=1)


if __name__ == "__main__":
    main()
