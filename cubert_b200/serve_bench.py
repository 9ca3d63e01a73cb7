"""Online-serving mix through the replica manager.

    CUBERT_NUM_MODELS_PER_GPU=2 python -m cubert_b200.serve_bench [--requests N] [--clients C]
                                                                   [--dtype f16|f32] [--seed S]

BERT-base, seq_length 32, two-class head, output cuBERT_PROBS. A seeded stream of requests: each
request's batch size is 1, 8 or 32 with probabilities 0.5 / 0.3 / 0.2 and each sequence's valid length
is uniform in [4, 32]. C closed-loop client threads share ONE model handle and call cuBERT_compute
through the C API (ctypes releases the GIL); the library spreads the calls round-robin over its
replicas (visible GPUs x CUBERT_NUM_MODELS_PER_GPU) and serialises them per replica, as the
reference's BertM does (src/cuBERT/BertM.cpp:65-76). Prints one JSON line with p50 / p99 request
latency and aggregate sequences/s.
"""
import argparse
import json
import os
import subprocess
import tempfile
import threading
import time

import numpy as np

from . import frozen_graph, model, synthetic


def request_stream(cfg, n, seq, seed):
    rng = np.random.default_rng(seed)
    sizes = rng.choice([1, 8, 32], size=n, p=[0.5, 0.3, 0.2])
    reqs = []
    for i, b in enumerate(sizes):
        ids = rng.integers(1, cfg["vocab"], size=(b, seq), dtype=np.int32)
        lens = rng.integers(4, seq + 1, size=b)
        mask = (np.arange(seq)[None, :] < lens[:, None]).astype(np.int8)
        seg = np.zeros((b, seq), np.int8)
        reqs.append((ids, mask, seg))
    return reqs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=100000)
    ap.add_argument("--clients", type=int, default=0,
                    help="closed-loop client threads (default: one per replica; more only queue behind the replicas)")
    ap.add_argument("--dtype", default="f16", choices=["f16", "f32"])
    ap.add_argument("--seed", type=int, default=5)
    ap.add_argument("--distinct", type=int, default=2048, help="distinct requests generated; the stream cycles over them")
    ap.add_argument("--native", action="store_true",
                    help="drive the C API from the native client (lib/serve_mix: C++ threads, its own seeded stream of "
                         "the same mix) instead of Python threads")
    a = ap.parse_args()

    cfg = synthetic.config("base")
    seq = 32
    var = synthetic.random_weights(cfg, a.seed)
    if a.dtype == "f16":
        var = {k: v.astype(np.float16) for k, v in var.items()}
    path = os.path.join(tempfile.mkdtemp(prefix="cubert_serve_"), "model.pb")
    frozen_graph.write_frozen_graph(path, var)
    if a.native:
        from . import build as native
        if not os.path.exists(native.SERVE_MIX):
            raise SystemExit("%s is missing: run `python -m cubert_b200.build`" % native.SERVE_MIX)
        proc = subprocess.run([native.SERVE_MIX, path, str(a.requests), str(a.clients), str(a.seed),
                               "1" if a.dtype == "f16" else "0", str(cfg["layers"]), str(cfg["heads"]), str(cfg["vocab"]),
                               str(seq)], stdout=subprocess.PIPE, universal_newlines=True)
        os.unlink(path)
        lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
        if proc.returncode != 0 or not lines:
            raise SystemExit("serve_mix failed (exit %d)" % proc.returncode)
        line = json.loads(lines[-1])
        line["models_per_gpu"] = int(os.environ.get("CUBERT_NUM_MODELS_PER_GPU", "1"))
        print(json.dumps(line), flush=True)
        return
    ct = model.ComputeType.HALF if a.dtype == "f16" else model.ComputeType.FLOAT
    m = model.Model(path, 32, seq, cfg["layers"], cfg["heads"], ct)
    os.unlink(path)
    replicas = m.info["replicas"]
    clients = a.clients or replicas
    reqs = request_stream(cfg, min(a.distinct, a.requests), seq, a.seed)
    out_dtype = np.float16 if a.dtype == "f16" else np.float32

    # warm every replica and every batch size (first use captures a CUDA graph per batch size)
    for b in (1, 8, 32):
        ids, mask, seg = next(r for r in reqs if r[0].shape[0] == b)
        for _ in range(3 * replicas):
            m.compute(ids, mask, seg, np.zeros((b, 2), out_dtype), model.OutputType.PROBS)

    counter = [0]
    lock = threading.Lock()
    lat = [[] for _ in range(clients)]
    seqs = [0] * clients

    def client(k):
        outs = {b: np.zeros((b, 2), out_dtype) for b in (1, 8, 32)}
        while True:
            with lock:
                i = counter[0]
                counter[0] += 1
            if i >= a.requests:
                return
            ids, mask, seg = reqs[i % len(reqs)]
            t0 = time.perf_counter()
            m.compute(ids, mask, seg, outs[ids.shape[0]], model.OutputType.PROBS)
            lat[k].append(time.perf_counter() - t0)
            seqs[k] += ids.shape[0]

    threads = [threading.Thread(target=client, args=(k,)) for k in range(clients)]
    t0 = time.perf_counter()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    all_lat = np.sort(np.concatenate([np.asarray(x) for x in lat]))
    line = {
        "metric": "BERT-base seq32 serving mix", "requests": int(a.requests), "clients": clients, "replicas": replicas,
        "gpus": model.get_gpu_count(), "models_per_gpu": int(os.environ.get("CUBERT_NUM_MODELS_PER_GPU", "1")),
        "dtype": a.dtype, "sequences_per_s": sum(seqs) / wall, "requests_per_s": a.requests / wall,
        "latency_ms": {"p50": float(all_lat[len(all_lat) // 2] * 1e3), "p99": float(all_lat[int(len(all_lat) * 0.99)] * 1e3),
                       "mean": float(all_lat.mean() * 1e3), "max": float(all_lat[-1] * 1e3)},
        "mix": "batch 1/8/32 with p 0.5/0.3/0.2, valid length U[4,32], seed %d" % a.seed,
        "wall_s": wall,
    }
    print(json.dumps(line), flush=True)
    m.close()


if __name__ == "__main__":
    main()
