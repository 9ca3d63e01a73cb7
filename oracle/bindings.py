"""ctypes bindings for the CPU checkers. TEST INFRASTRUCTURE ONLY.

Two libraries, both built by oracle/Makefile:

* ``liboracle.so``               -- our plain-C restatement (oracle/cubert_oracle.c)
* ``_ref/libcubert_ref_cpu.so``  -- the reference's own CPU sources compiled in place
                                     (only where the reference tree was present at build time)

Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
may import this module. The product never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_CPU_SO = os.path.join(HERE, "_ref", "libcubert_ref_cpu.so")
REF_GPU_SO = os.path.join(HERE, "_ref", "libcubert_ref_gpu.so")

LAYER_TENSORS = [
    "attention/self/query/kernel", "attention/self/query/bias",
    "attention/self/key/kernel", "attention/self/key/bias",
    "attention/self/value/kernel", "attention/self/value/bias",
    "attention/output/dense/kernel", "attention/output/dense/bias",
    "attention/output/LayerNorm/beta", "attention/output/LayerNorm/gamma",
    "intermediate/dense/kernel", "intermediate/dense/bias",
    "output/dense/kernel", "output/dense/bias",
    "output/LayerNorm/beta", "output/LayerNorm/gamma",
]


# Where the reference's sources are looked for (the same default as oracle/Makefile's REF).
REFERENCE_SRC = os.environ.get("CUBERT_REFERENCE_SRC", os.path.join(os.sep, "root", "reference", "src"))


def reference_tree_present():
    return os.path.isdir(os.path.join(REFERENCE_SRC, "cuBERT"))


def build(ref=False):
    """Compile the checkers (idempotent; make decides what is stale)."""
    targets = ["oracle"] + (["ref", "ref_gpu"] if ref else [])
    subprocess.run(["make", "-C", HERE, "REF=" + REFERENCE_SRC] + targets, check=True, stdout=subprocess.DEVNULL)


PYWRAP_DIR = os.path.join(HERE, "_ref", "pywrap")


def build_pywrap():
    """Compile the reference's own Cython wrapper against our libcuBERT.so (needs the reference tree and
    the native libraries). Returns the folder to put on sys.path, or None where it cannot be built."""
    import glob
    if not glob.glob(os.path.join(PYWRAP_DIR, "cuBERT*.so")):
        if not reference_tree_present():
            return None
        subprocess.run(["make", "-C", HERE, "REF=" + REFERENCE_SRC, "ref_pywrap"], check=True,
                       stdout=subprocess.DEVNULL)
    return PYWRAP_DIR


REF_HOST_B200_SO = os.path.join(HERE, "_ref", "libcubert_ref_host_b200.so")


def build_host_b200():
    """Link the reference's own GPU host code (HAVE_CUDA build of Bert, Transformer, Dense, ...) with
    ref_host_b200_ops.cu, which serves its operator templates from OUR kernel library. Returns the
    path of the library, or None where it cannot be built (reference tree absent)."""
    if not os.path.exists(REF_HOST_B200_SO):
        if not reference_tree_present():
            return None
        subprocess.run(["make", "-C", HERE, "REF=" + REFERENCE_SRC, "ref_host_b200"], check=True,
                       stdout=subprocess.DEVNULL)
    return REF_HOST_B200_SO


BENCHMARK_BIN = os.path.join(HERE, "_ref", "benchmark_cu")


def build_benchmark():
    """Compile the reference's own benchmark program (benchmark/benchmark_cu.cpp, unmodified) against our
    libcuBERT.so. Returns the path of the binary, or None where it cannot be built."""
    if not os.path.exists(BENCHMARK_BIN):
        if not os.path.exists(os.path.join(REFERENCE_SRC, "..", "benchmark", "benchmark_cu.cpp")):
            return None
        subprocess.run(["make", "-C", HERE, "REF=" + REFERENCE_SRC, "ref_benchmark"], check=True,
                       stdout=subprocess.DEVNULL)
    return BENCHMARK_BIN


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t=C.c_float):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


class _Weights(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("vocab", "type_vocab", "hidden", "layers", "heads", "intermediate", "num_labels", "seq")] + \
               [(n, C.POINTER(C.c_float)) for n in
                ("word_emb", "type_emb", "pos_emb", "emb_ln_beta", "emb_ln_gamma")] + \
               [("layer_tensors", C.POINTER(C.POINTER(C.c_float)))] + \
               [(n, C.POINTER(C.c_float)) for n in
                ("pooler_kernel", "pooler_bias", "output_weights", "output_bias")]


class Oracle:
    """Our C restatement."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build()
        self.lib = C.CDLL(ORACLE_SO)

    # ---- single ops -------------------------------------------------
    def embedding(self, ids, table):
        table = _f32(table)
        n, width = ids.size, table.shape[1]
        out = np.empty((n, width), np.float32)
        if ids.dtype == np.int8:
            self.lib.orc_embedding_i8(_p(np.ascontiguousarray(ids), C.c_int8), n, _p(table), width, _p(out))
        else:
            ids = np.ascontiguousarray(ids, np.int32)
            self.lib.orc_embedding_i32(_p(ids, C.c_int32), n, _p(table), width, _p(out))
        return out

    def layer_norm_(self, inp, inout, beta, gamma):
        inp, out = _f32(inp), _f32(inout).copy()
        rows, ch = out.shape
        self.lib.orc_layer_norm_(_p(inp), _p(out), rows, ch, _p(_f32(beta)), _p(_f32(gamma)))
        return out

    def gelu(self, x):
        out = _f32(x).copy()
        self.lib.orc_gelu(C.c_size_t(out.size), _p(out))
        return out

    def softmax_(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.orc_softmax_(_p(x), _p(out), x.shape[0], x.shape[1])
        return out

    def not_(self, mask):
        mask = np.ascontiguousarray(mask, np.int8)
        out = np.empty(mask.shape, np.float32)
        self.lib.orc_not(_p(mask, C.c_int8), _p(out), mask.size)
        return out

    def attention_mask(self, mask, heads):
        mask = np.ascontiguousarray(mask, np.int8)
        b, s = mask.shape
        out = np.empty((b, s * heads, s), np.float32)
        self.lib.orc_attention_mask(_p(mask, C.c_int8), b, s, heads, _p(out))
        return out

    def tanh_(self, x):
        out = _f32(x).copy()
        self.lib.orc_tanh_(_p(out), out.size)
        return out

    def reduce_mean_1(self, x):
        x = _f32(x)
        b, s, h = x.shape
        out = np.empty((b, h), np.float32)
        self.lib.orc_reduce_mean_1(_p(x), _p(out), b, s, h)
        return out

    def dense(self, x, w, bias):
        x, w = _f32(x), _f32(w)
        rows, inputs = x.shape
        units = w.shape[1]
        y = np.empty((rows, units), np.float32)
        b = _f32(bias) if bias is not None else None
        self.lib.orc_dense(_p(x), _p(w), _p(b), rows, inputs, units, _p(y))
        return y

    def bert_embeddings(self, ids, seg, word, pos, typ, beta, gamma):
        ids = np.ascontiguousarray(ids, np.int32)
        seg = np.ascontiguousarray(seg, np.int8)
        b, s = ids.shape
        word, pos, typ = _f32(word), _f32(pos), _f32(typ)
        h = word.shape[1]
        out = np.empty((b, s, h), np.float32)
        self.lib.orc_bert_embeddings(_p(ids, C.c_int32), _p(seg, C.c_int8), b, s, h,
                                     _p(word), _p(pos), _p(typ), _p(_f32(beta)), _p(_f32(gamma)), _p(out))
        return out

    def masked_softmax(self, scores, mask, scale=1.0):
        """scores [B, S, H, S]; mask int8 [B, S] or None."""
        scores = _f32(scores)
        b, s, h, s2 = scores.shape
        assert s == s2
        m = np.ascontiguousarray(mask, np.int8) if mask is not None else None
        out = np.empty_like(scores)
        self.lib.orc_masked_softmax(_p(scores), _p(m, C.c_int8), b, h, s, C.c_float(scale), _p(out))
        return out

    def bert_pooler(self, seq_out, kernel, bias):
        x = _f32(seq_out)
        b, s, h = x.shape
        out = np.empty((b, h), np.float32)
        self.lib.orc_bert_pooler(_p(x), b, s, h, _p(_f32(kernel)), _p(_f32(bias)), _p(out))
        return out

    def classifier(self, pooled, w, bias, want_probs=True):
        x, w = _f32(pooled), _f32(w)
        b, h = x.shape
        labels = w.shape[0]
        logits = np.empty((b, labels), np.float32)
        probs = np.empty((b, labels), np.float32) if want_probs else None
        bb = _f32(bias) if bias is not None else None
        self.lib.orc_classifier(_p(x), b, h, labels, _p(w), _p(bb), _p(logits), _p(probs))
        return logits, probs

    def att_q_k(self, q, k):
        q, k = _f32(q), _f32(k)
        b, s, h, d = q.shape
        out = np.empty((b, s, h, s), np.float32)
        self.lib.orc_att_q_k(_p(q), _p(k), b, s, h, d, _p(out))
        return out

    def att_qk_v(self, probs, v):
        probs, v = _f32(probs), _f32(v)
        b, s, h, d = v.shape
        out = np.empty((b, s, h, d), np.float32)
        self.lib.orc_att_qk_v(_p(probs), _p(v), b, s, h, d, _p(out))
        return out

    def attention_self(self, x, qkv, batch, seq, heads, d, neg_mask):
        x = _f32(x)
        keep = [_f32(t) for t in qkv]
        arr = (C.POINTER(C.c_float) * 6)(*[_p(t) for t in keep])
        neg = _f32(neg_mask)
        out = np.empty((batch, seq, heads * d), np.float32)
        self.lib.orc_attention_self(_p(x), arr, batch, seq, heads, d, _p(neg), _p(out))
        return out

    # ---- whole model ------------------------------------------------
    def _weights(self, var, cfg, prefix="bert/encoder"):
        """var: name -> float32 array (TF variable names); cfg: dict of geometry."""
        keep = []

        def ptr(name):
            if name not in var:
                return None
            a = _f32(var[name])
            keep.append(a)
            return _p(a)

        w = _Weights()
        for k in ("vocab", "type_vocab", "hidden", "layers", "heads", "intermediate", "num_labels", "seq"):
            setattr(w, k, int(cfg.get(k, 0)))
        w.word_emb = ptr("bert/embeddings/word_embeddings")
        w.type_emb = ptr("bert/embeddings/token_type_embeddings")
        w.pos_emb = ptr("bert/embeddings/position_embeddings")
        w.emb_ln_beta = ptr("bert/embeddings/LayerNorm/beta")
        w.emb_ln_gamma = ptr("bert/embeddings/LayerNorm/gamma")
        n = cfg["layers"] * len(LAYER_TENSORS)
        arr = (C.POINTER(C.c_float) * n)()
        for l in range(cfg["layers"]):
            for i, t in enumerate(LAYER_TENSORS):
                arr[l * len(LAYER_TENSORS) + i] = ptr("%s/layer_%d/%s" % (prefix, l, t))
        keep.append(arr)
        w.layer_tensors = C.cast(arr, C.POINTER(C.POINTER(C.c_float)))
        w.pooler_kernel = ptr("bert/pooler/dense/kernel")
        w.pooler_bias = ptr("bert/pooler/dense/bias")
        w.output_weights = ptr("output_weights")
        w.output_bias = ptr("output_bias")
        return w, keep

    def transformer(self, var, cfg, x, mask, prefix="bert/encoder"):
        w, keep = self._weights(var, cfg, prefix)
        x = _f32(x).copy()
        mask = np.ascontiguousarray(mask, np.int8)
        batch = mask.shape[0]
        self.lib.orc_transformer(C.byref(w), batch, _p(x), _p(mask, C.c_int8))
        return x

    def bert_forward(self, var, cfg, ids, mask, seg):
        w, keep = self._weights(var, cfg)
        ids = np.ascontiguousarray(ids, np.int32)
        mask = np.ascontiguousarray(mask, np.int8)
        seg = np.ascontiguousarray(seg, np.int8)
        b, s = ids.shape
        h, labels = cfg["hidden"], cfg.get("num_labels", 1)
        out = {
            "embedding_output": np.empty((b, s, h), np.float32),
            "sequence_output": np.empty((b, s, h), np.float32),
            "pooled_output": np.empty((b, h), np.float32),
        }
        has_cls = "output_weights" in var
        if has_cls:
            out["logits"] = np.empty((b, labels), np.float32)
            out["probs"] = np.empty((b, labels), np.float32)
        self.lib.orc_bert_forward(C.byref(w), b, _p(ids, C.c_int32), _p(mask, C.c_int8), _p(seg, C.c_int8),
                                  _p(out["embedding_output"]), _p(out["sequence_output"]),
                                  _p(out["pooled_output"]),
                                  _p(out.get("logits")), _p(out.get("probs")))
        return out


class Reference:
    """The reference's own CPU code (oracle/_ref). Raises FileNotFoundError if not built."""

    def __init__(self):
        if not os.path.exists(REF_CPU_SO):
            raise FileNotFoundError(REF_CPU_SO)
        self.lib = C.CDLL(REF_CPU_SO)
        self.lib.ref_bert_open.restype = C.c_void_p

    @staticmethod
    def _names(var):
        keep = {k: _f32(v).copy() for k, v in var.items()}
        names = (C.c_char_p * len(keep))(*[k.encode() for k in keep])
        ptrs = (C.POINTER(C.c_float) * len(keep))(*[_p(v) for v in keep.values()])
        return len(keep), names, ptrs, keep

    def layer_norm_(self, inp, inout, beta, gamma):
        inp, out = _f32(inp), _f32(inout).copy()
        self.lib.ref_layer_norm_(_p(inp), _p(out), out.shape[0], out.shape[1], _p(_f32(beta)), _p(_f32(gamma)))
        return out

    def softmax_(self, x):
        x = _f32(x).copy()
        out = np.empty_like(x)
        self.lib.ref_softmax_(_p(x), _p(out), x.shape[0], x.shape[1])
        return out

    def gelu(self, x):
        out = _f32(x).copy()
        self.lib.ref_gelu(C.c_size_t(out.size), _p(out))
        return out

    def embedding(self, ids, table):
        table = _f32(table)
        out = np.empty((ids.size, table.shape[1]), np.float32)
        if ids.dtype == np.int8:
            self.lib.ref_embedding_i8(_p(np.ascontiguousarray(ids), C.c_int8), ids.size, _p(table),
                                      table.shape[1], _p(out))
        else:
            ids = np.ascontiguousarray(ids, np.int32)
            self.lib.ref_embedding_i32(_p(ids, C.c_int32), ids.size, _p(table), table.shape[1], _p(out))
        return out

    def not_(self, mask):
        mask = np.ascontiguousarray(mask, np.int8)
        out = np.empty(mask.shape, np.float32)
        self.lib.ref_not(_p(mask, C.c_int8), _p(out), mask.size)
        return out

    def tanh_(self, x):
        out = _f32(x).copy()
        self.lib.ref_tanh_(_p(out), out.size)
        return out

    def reduce_mean_1(self, x):
        x = _f32(x)
        b, s, h = x.shape
        out = np.empty((b, h), np.float32)
        self.lib.ref_reduce_mean_1(_p(x), _p(out), b, s, h)
        return out

    def attention_mask(self, mask, heads):
        mask = np.ascontiguousarray(mask, np.int8).copy()
        b, s = mask.shape
        out = np.empty((b, s * heads, s), np.float32)
        self.lib.ref_attention_mask(_p(mask, C.c_int8), b, s, heads, _p(out))
        return out

    def bert_embeddings(self, ids, seg, word, pos, typ, beta, gamma):
        var = {"bert/embeddings/word_embeddings": word, "bert/embeddings/token_type_embeddings": typ,
               "bert/embeddings/position_embeddings": pos, "bert/embeddings/LayerNorm/beta": beta,
               "bert/embeddings/LayerNorm/gamma": gamma}
        n, names, ptrs, keep = self._names(var)
        ids = np.ascontiguousarray(ids, np.int32).copy()
        seg = np.ascontiguousarray(seg, np.int8).copy()
        b, s = ids.shape
        word = np.asarray(word)
        out = np.empty((b, s, word.shape[1]), np.float32)
        self.lib.ref_bert_embeddings(n, names, ptrs, b, s, word.shape[0], np.asarray(typ).shape[0],
                                     word.shape[1], _p(ids, C.c_int32), _p(seg, C.c_int8), _p(out))
        return out

    def transformer(self, var, cfg, x, mask, prefix="bert/encoder"):
        n, names, ptrs, keep = self._names(var)
        x = _f32(x).copy()
        mask = np.ascontiguousarray(mask, np.int8).copy()
        b = mask.shape[0]
        out = np.empty_like(x)
        self.lib.ref_transformer(n, names, ptrs, prefix.encode(), b, cfg["seq"], cfg["hidden"],
                                 cfg["layers"], cfg["heads"], cfg["intermediate"],
                                 _p(x), _p(mask, C.c_int8), _p(out))
        return out

    def bert_pooler(self, seq_out, kernel, bias):
        x = _f32(seq_out).copy()
        b, s, h = x.shape
        out = np.empty((b, h), np.float32)
        self.lib.ref_bert_pooler(_p(_f32(kernel).copy()), _p(_f32(bias).copy()), b, s, h, _p(x), _p(out))
        return out

    def classifier(self, pooled, w, bias, want_probs=True):
        x, w = _f32(pooled).copy(), _f32(w).copy()
        b, h = x.shape
        labels = w.shape[0]
        logits = np.empty((b, labels), np.float32)
        probs = np.empty((b, labels), np.float32) if want_probs else None
        bb = _f32(bias).copy() if bias is not None else None
        self.lib.ref_classifier(_p(w), _p(bb), b, h, labels, _p(x), _p(logits), _p(probs))
        return logits, probs

    def bert_open(self, var, cfg, max_batch):
        n, names, ptrs, keep = self._names(var)
        h = self.lib.ref_bert_open(n, names, ptrs, max_batch, cfg["seq"], cfg["vocab"], cfg["type_vocab"],
                                   cfg["hidden"], cfg["layers"], cfg["heads"], cfg["intermediate"],
                                   cfg.get("num_labels", 1))
        return C.c_void_p(h)

    def bert_compute(self, handle, ids, mask, seg):
        ids = np.ascontiguousarray(ids, np.int32).copy()
        mask = np.ascontiguousarray(mask, np.int8).copy()
        seg = np.ascontiguousarray(seg, np.int8).copy()
        self.lib.ref_bert_compute(handle, ids.shape[0], _p(ids, C.c_int32), _p(mask, C.c_int8),
                                  _p(seg, C.c_int8))

    def bert_output(self, handle, batch, cfg, has_classifier):
        s, h, labels = cfg["seq"], cfg["hidden"], cfg.get("num_labels", 1)
        out = {
            "embedding_output": np.empty((batch, s, h), np.float32),
            "sequence_output": np.empty((batch, s, h), np.float32),
            "pooled_output": np.empty((batch, h), np.float32),
        }
        if has_classifier:
            out["logits"] = np.empty((batch, labels), np.float32)
            out["probs"] = np.empty((batch, labels), np.float32)
        self.lib.ref_bert_output(handle, batch, _p(out.get("logits")), _p(out.get("probs")),
                                 _p(out["pooled_output"]), _p(out["sequence_output"]),
                                 _p(out["embedding_output"]))
        return out

    def bert_close(self, handle):
        self.lib.ref_bert_close(handle)

    def bert_forward(self, var, cfg, ids, mask, seg):
        h = self.bert_open(var, cfg, ids.shape[0])
        try:
            self.bert_compute(h, ids, mask, seg)
            return self.bert_output(h, ids.shape[0], cfg, "output_weights" in var)
        finally:
            self.bert_close(h)


class ReferenceGPU:
    """The reference's own CUDA operator bodies compiled for sm_100a (oracle/_ref). Every pointer is a
    raw device address; raises FileNotFoundError if the library was not built."""

    def __init__(self):
        if not os.path.exists(REF_GPU_SO):
            raise FileNotFoundError(REF_GPU_SO)
        self.lib = C.CDLL(REF_GPU_SO)
        P, I, Z = C.c_void_p, C.c_int, C.c_size_t
        for t in ("f32", "f16"):
            getattr(self.lib, "refgpu_layer_norm_" + t).argtypes = [P, P, I, I, P, P, P, P, P]
            getattr(self.lib, "refgpu_softmax_" + t).argtypes = [P, P, I, I, P, P]
            getattr(self.lib, "refgpu_gelu_" + t).argtypes = [Z, P, P]
            getattr(self.lib, "refgpu_embedding_i32_" + t).argtypes = [P, I, P, I, P, P]
            getattr(self.lib, "refgpu_embedding_i8_" + t).argtypes = [P, I, P, I, P, P]
            getattr(self.lib, "refgpu_not_" + t).argtypes = [P, P, I, P]
            getattr(self.lib, "refgpu_tanh_" + t).argtypes = [P, I, P]
            getattr(self.lib, "refgpu_reduce_mean_1_" + t).argtypes = [P, P, I, I, I, P]

    def fn(self, name, t):
        return getattr(self.lib, "refgpu_%s_%s" % (name, t))


REF_GPU_FULL_SO = os.path.join(HERE, "_ref", "libcubert_ref_gpu_full.so")


def build_gpu_full():
    """The reference's complete GPU build (its host code and its own .cu files) for sm_100a. Returns the
    path of the library, or None where it cannot be built (reference tree absent)."""
    if not os.path.exists(REF_GPU_FULL_SO):
        if not reference_tree_present():
            return None
        subprocess.run(["make", "-C", HERE, "REF=" + REFERENCE_SRC, "ref_gpu_full"], check=True,
                       stdout=subprocess.DEVNULL)
    return REF_GPU_FULL_SO


class ReferenceHost:
    """The reference's own Bert<T> host class in its GPU build, behind ref_host_b200_driver.cpp: either on
    this repository's kernels (REF_HOST_B200_SO) or on the reference's own (REF_GPU_FULL_SO).
    Host arrays in, host arrays out; needs a GPU."""

    def __init__(self, library):
        if not os.path.exists(library):
            raise FileNotFoundError(library)
        self.lib = C.CDLL(library)
        P, I = C.c_void_p, C.c_int
        self.lib.refhost_open.restype = P
        self.lib.refhost_open.argtypes = [I, C.POINTER(C.c_char_p), C.POINTER(P), I, I, I, I, I, I, I, I, I, I]
        self.lib.refhost_compute.argtypes = [P, I, I, P, P, P]
        self.lib.refhost_output.argtypes = [P, I, I, P, P, P, P, P]
        self.lib.refhost_close.argtypes = [P, I]

    def open(self, var, cfg, max_batch, half=False):
        """var: name -> float32 array (rounded to binary16 here when `half`); cfg as model_geometry()."""
        dt = np.float16 if half else np.float32
        keep = {k: np.ascontiguousarray(v, dtype=dt) for k, v in var.items()}
        names = (C.c_char_p * len(keep))(*[k.encode() for k in keep])
        ptrs = (C.c_void_p * len(keep))(*[v.ctypes.data for v in keep.values()])
        h = self.lib.refhost_open(len(keep), names, ptrs, int(half), max_batch, cfg["seq"], cfg["vocab"],
                                  cfg["type_vocab"], cfg["hidden"], cfg["layers"], cfg["heads"],
                                  cfg["intermediate"], cfg.get("num_labels", 1))
        return dict(handle=h, half=int(half), dtype=dt, cfg=cfg, classifier="output_weights" in var, keep=keep)

    def compute(self, m, ids, mask, seg):
        """ids int32, mask int8, seg int8, C-contiguous [batch, seq]."""
        self.lib.refhost_compute(m["handle"], m["half"], ids.shape[0], ids.ctypes.data, mask.ctypes.data, seg.ctypes.data)

    def output(self, m, batch, names=("embedding_output", "sequence_output", "pooled_output", "logits", "probs")):
        cfg, dt = m["cfg"], m["dtype"]
        s, hid, labels = cfg["seq"], cfg["hidden"], cfg.get("num_labels", 1)
        shapes = {"embedding_output": (batch, s, hid), "sequence_output": (batch, s, hid), "pooled_output": (batch, hid),
                  "logits": (batch, labels), "probs": (batch, labels)}
        out = {n: np.empty(shapes[n], dt) for n in names if m["classifier"] or n not in ("logits", "probs")}
        addr = lambda n: out[n].ctypes.data if n in out else None  # noqa: E731
        self.lib.refhost_output(m["handle"], m["half"], batch, addr("logits"), addr("probs"), addr("pooled_output"),
                                addr("sequence_output"), addr("embedding_output"))
        return out

    def close(self, m):
        self.lib.refhost_close(m["handle"], m["half"])

    def forward(self, var, cfg, ids, mask, seg, half=False):
        ids = np.ascontiguousarray(ids, np.int32).copy()
        mask = np.ascontiguousarray(mask, np.int8).copy()
        seg = np.ascontiguousarray(seg, np.int8).copy()
        m = self.open(var, cfg, ids.shape[0], half)
        try:
            self.compute(m, ids, mask, seg)
            return self.output(m, ids.shape[0])
        finally:
            self.close(m)
