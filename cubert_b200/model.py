"""Python binding of the cuBERT C API served by ``lib/libcuBERT.so`` (ctypes).

The classes mirror the reference's Cython wrapper (python/cuBERT.pyx): ``ComputeType``,
``OutputType``, ``Output`` and ``Model`` with ``compute`` / ``compute_m``, taking C-contiguous
numpy arrays (int32 ids, int8 mask and segments) and filling caller-provided output arrays.
Calls go through the status-returning entry points of include/cubert_b200.h, because a C++
exception cannot cross ctypes; a non-zero status is raised as ``ValueError`` (what the
reference throws as std::invalid_argument) or ``RuntimeError``.

The native library is mandatory. There is no CPU implementation behind this module.
"""
import ctypes as C
import os

import numpy as np

from . import kernels

HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB = os.path.join(HERE, "lib", "libcuBERT.so")

K_NAMES = ["embed_ln", "bias_residual_ln", "bias_gelu", "masked_softmax", "bias_tanh", "mean_pool",
           "logits_probs", "half_to_float", "gemm", "event_overhead"]


class ComputeType:
    FLOAT = 0
    HALF = 1


class OutputType:
    LOGITS = 0
    POOLED_OUTPUT = 1
    SEQUENCE_OUTPUT = 2
    EMBEDDING_OUTPUT = 3
    PROBS = 4


class _COutput(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("pooled_output", C.c_void_p), ("sequence_output", C.c_void_p),
                ("embedding_output", C.c_void_p), ("probs", C.c_void_p)]


class _CInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("replicas", "max_batch_size", "seq_length", "hidden_size", "num_labels", "vocab_size",
                 "type_vocab_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                 "has_pooler_dense", "fp32_gemm_emulation")]


class _CProfile(C.Structure):
    _fields_ = [("ms", C.c_double * len(K_NAMES)), ("launches", C.c_int64 * len(K_NAMES)),
                ("bytes", C.c_int64 * len(K_NAMES))]


_REFERENCE_API = ["cuBERT_initialize", "cuBERT_finalize", "cuBERT_get_gpu_count", "cuBERT_open", "cuBERT_compute",
                  "cuBERT_compute_m", "cuBERT_close", "cuBERT_open_tokenizer", "cuBERT_close_tokenizer",
                  "cuBERT_tokenize_compute", "cuBERT_tokenize_compute_m"]
_EXTENSION_API = ["cubert_b200_last_error", "cubert_b200_open", "cubert_b200_compute", "cubert_b200_compute_m",
                  "cubert_b200_close", "cubert_b200_model_info", "cubert_b200_graph_open",
                  "cubert_b200_graph_info", "cubert_b200_graph_tensor", "cubert_b200_graph_close",
                  "cubert_b200_open_tokenizer", "cubert_b200_close_tokenizer", "cubert_b200_encode",
                  "cubert_b200_tokenize", "cubert_b200_tokenize_compute_m",
                  "cubert_b200_replica_device",
                  "cubert_b200_replica_stream", "cubert_b200_forward_device", "cubert_b200_forward_device_masked",
                  "cubert_b200_device_outputs",
                  "cubert_b200_synchronize", "cubert_b200_profile_enable", "cubert_b200_profile_read"]


def exported_symbols():
    return _REFERENCE_API + _EXTENSION_API


_lib = None


def load():
    """Load libcuBERT.so (and the kernel library it links); raises if either is missing.

    The library is linked against the CUDA toolkit's cuBLAS. A process binds ONE libcublas.so.12: the
    first one loaded. Call this before `import torch` to get the toolkit's (12.9.1 here, 6 % faster on
    BERT-base than the 12.8.4 bundled with torch); after it, the library runs on torch's copy."""
    global _lib
    if _lib is not None:
        return _lib
    kernels.load()
    if not os.path.exists(HOST_LIB):
        raise RuntimeError("%s is missing: run `python -m cubert_b200.build` (there is no CPU fallback)" % HOST_LIB)
    lib = C.CDLL(HOST_LIB)
    lib.cubert_b200_last_error.restype = C.c_char_p
    lib.cuBERT_get_gpu_count.restype = C.c_int
    lib.cubert_b200_open.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
    lib.cubert_b200_compute.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_int, C.c_int]
    lib.cubert_b200_compute_m.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.POINTER(_COutput), C.c_int, C.c_int]
    lib.cubert_b200_close.argtypes = [C.c_void_p, C.c_int]
    lib.cubert_b200_model_info.argtypes = [C.c_void_p, C.c_int, C.POINTER(_CInfo)]
    lib.cubert_b200_graph_open.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]
    lib.cubert_b200_graph_info.argtypes = [C.c_void_p, C.c_int, C.POINTER(_CInfo)]
    lib.cubert_b200_graph_tensor.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.POINTER(C.c_void_p),
                                             C.POINTER(C.c_int64)]
    lib.cubert_b200_graph_close.argtypes = [C.c_void_p, C.c_int]
    lib.cubert_b200_open_tokenizer.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]
    lib.cubert_b200_close_tokenizer.argtypes = [C.c_void_p]
    lib.cubert_b200_encode.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.cubert_b200_tokenize.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.c_char_p, C.c_size_t,
                                         C.POINTER(C.c_int)]
    lib.cubert_b200_tokenize_compute_m.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_char_p),
                                                   C.POINTER(C.c_char_p), C.POINTER(_COutput), C.c_int, C.c_int]
    lib.cubert_b200_replica_device.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int)]
    lib.cubert_b200_replica_stream.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
    lib.cubert_b200_forward_device.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                               C.c_void_p]
    lib.cubert_b200_forward_device_masked.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                                      C.c_void_p, C.c_void_p]
    lib.cubert_b200_device_outputs.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(_COutput)]
    lib.cubert_b200_synchronize.argtypes = [C.c_void_p, C.c_int, C.c_int]
    lib.cubert_b200_profile_enable.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    lib.cubert_b200_profile_read.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(_CProfile)]
    _lib = lib
    return lib


def _check(rc):
    if rc == 0:
        return
    msg = load().cubert_b200_last_error().decode()
    if rc == -1:
        raise ValueError(msg)
    raise RuntimeError(msg)


def get_gpu_count():
    return load().cuBERT_get_gpu_count()


class FrozenGraph:
    """The C++ model-file reader on its own (works without a GPU)."""

    def __init__(self, model_file, compute_type=ComputeType.FLOAT):
        self._lib = load()
        self._handle = C.c_void_p()
        self._compute_type = compute_type
        _check(self._lib.cubert_b200_graph_open(model_file.encode("utf8"), compute_type, C.byref(self._handle)))
        info = _CInfo()
        _check(self._lib.cubert_b200_graph_info(self._handle, compute_type, C.byref(info)))
        self.info = {n: getattr(info, n) for n, _ in _CInfo._fields_}

    def tensor(self, name):
        data = C.c_void_p()
        count = C.c_int64()
        _check(self._lib.cubert_b200_graph_tensor(self._handle, self._compute_type, name.encode("utf8"),
                                                  C.byref(data), C.byref(count)))
        dtype = np.float32 if self._compute_type == ComputeType.FLOAT else np.float16
        buf = (C.c_char * (count.value * np.dtype(dtype).itemsize)).from_address(data.value)
        return np.frombuffer(buf, dtype=dtype).copy()

    def close(self):
        if self._handle:
            _check(self._lib.cubert_b200_graph_close(self._handle, self._compute_type))
            self._handle = C.c_void_p()


def _utf8(text):
    return text if isinstance(text, bytes) else text.encode("utf8")


class Tokenizer:
    """BERT basic + WordPiece tokenizer of the library (CPU only)."""

    def __init__(self, vocab_file, do_lower_case=True):
        self._lib = load()
        self._handle = C.c_void_p()
        _check(self._lib.cubert_b200_open_tokenizer(_utf8(vocab_file), 1 if do_lower_case else 0,
                                                    C.byref(self._handle)))

    def close(self):
        if self._handle:
            _check(self._lib.cubert_b200_close_tokenizer(self._handle))
            self._handle = C.c_void_p()

    def tokenize(self, text, max_tokens=1 << 20):
        return _tokenize(self._handle, text, True, max_tokens)

    def encode(self, text_a, text_b, max_seq_length):
        ids = np.zeros(max_seq_length, np.int32)
        mask = np.zeros(max_seq_length, np.int8)
        seg = np.zeros(max_seq_length, np.int8)
        _check(self._lib.cubert_b200_encode(self._handle, max_seq_length, _utf8(text_a),
                                            None if text_b is None else _utf8(text_b),
                                            ids.ctypes.data, mask.ctypes.data, seg.ctypes.data))
        return ids, mask, seg


def _tokenize(handle, text, do_lower_case, max_tokens):
    lib = load()
    raw = _utf8(text)
    size = 8 * len(raw) + 64
    buf = C.create_string_buffer(size)
    count = C.c_int()
    _check(lib.cubert_b200_tokenize(handle, raw, 1 if do_lower_case else 0, max_tokens, buf, size, C.byref(count)))
    return buf.value.decode("utf8").split("\n") if count.value else []


def basic_tokenize(text, do_lower_case=True, max_tokens=1 << 20):
    """The basic tokenizer alone (clean-up, lower-casing, punctuation and CJK splitting)."""
    return _tokenize(None, text, do_lower_case, max_tokens)


class Output:
    """Set of output arrays for ``Model.compute_m`` (python/cuBERT.pyx:46-121)."""

    FIELDS = ("logits", "pooled_output", "sequence_output", "embedding_output", "probs")

    def __init__(self, output=None, output_type=OutputType.LOGITS):
        for f in self.FIELDS:
            setattr(self, f, None)
        if output is not None:
            name = {OutputType.LOGITS: "logits", OutputType.POOLED_OUTPUT: "pooled_output",
                    OutputType.SEQUENCE_OUTPUT: "sequence_output", OutputType.EMBEDDING_OUTPUT: "embedding_output",
                    OutputType.PROBS: "probs"}[output_type]
            setattr(self, name, output)

    def _c(self):
        c = _COutput()
        for f in self.FIELDS:
            a = getattr(self, f)
            if a is not None:
                if not a.flags["C_CONTIGUOUS"]:
                    raise ValueError("output array %s must be C-contiguous" % f)
                setattr(c, f, a.ctypes.data)
        return c


def _input(a, dtype, name):
    if not isinstance(a, np.ndarray) or a.dtype != dtype or a.ndim != 2 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError("%s must be a C-contiguous 2-d numpy array of %s" % (name, np.dtype(dtype).name))
    return a.ctypes.data


class Model:
    """An open model (python/cuBERT.pyx:123-257 without the tokenizer half)."""

    def __init__(self, model_file, max_batch_size, seq_length, num_hidden_layers, num_attention_heads,
                 compute_type=ComputeType.FLOAT):
        self._lib = load()
        self._handle = C.c_void_p()
        self._compute_type = compute_type
        if isinstance(model_file, str):
            model_file = model_file.encode("utf8")
        _check(self._lib.cubert_b200_open(model_file, max_batch_size, seq_length, num_hidden_layers,
                                          num_attention_heads, compute_type, C.byref(self._handle)))
        info = _CInfo()
        _check(self._lib.cubert_b200_model_info(self._handle, compute_type, C.byref(info)))
        self.info = {n: getattr(info, n) for n, _ in _CInfo._fields_}

    def close(self):
        if self._handle:
            _check(self._lib.cubert_b200_close(self._handle, self._compute_type))
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def dtype(self):
        return np.float32 if self._compute_type == ComputeType.FLOAT else np.float16

    def compute(self, input_ids, input_mask, segment_ids, output, output_type=OutputType.LOGITS):
        batch = input_ids.shape[0]
        _check(self._lib.cubert_b200_compute(self._handle, batch, _input(input_ids, np.int32, "input_ids"),
                                             _input(input_mask, np.int8, "input_mask"),
                                             _input(segment_ids, np.int8, "segment_ids"), output.ctypes.data,
                                             output_type, self._compute_type))

    def compute_m(self, input_ids, input_mask, segment_ids, output, output_to_float=False):
        batch = input_ids.shape[0]
        c = output._c()
        _check(self._lib.cubert_b200_compute_m(self._handle, batch, _input(input_ids, np.int32, "input_ids"),
                                               _input(input_mask, np.int8, "input_mask"),
                                               _input(segment_ids, np.int8, "segment_ids"), C.byref(c),
                                               self._compute_type, 1 if output_to_float else 0))

    def tokenize_compute_m(self, tokenizer, text_a, text_b, output, output_to_float=False):
        """python/cuBERT.pyx:214-257: tokenise the texts, then compute_m."""
        n = len(text_a)
        a = (C.c_char_p * n)(*[_utf8(t) for t in text_a])
        b = (C.c_char_p * n)(*[_utf8(t) for t in text_b]) if text_b else None
        c = output._c()
        _check(self._lib.cubert_b200_tokenize_compute_m(self._handle, tokenizer._handle, n, a, b, C.byref(c),
                                                        self._compute_type, 1 if output_to_float else 0))

    # ---- additions of include/cubert_b200.h -------------------------------------------------
    def forward_device(self, replica, batch, d_ids, d_mask, d_segments, host_mask=None):
        """Forward pass on device-resident inputs (raw device addresses); asynchronous. host_mask: the
        caller's host copy of the mask (int8 numpy array), which lets the replica leave masked key columns
        out of the attention."""
        if host_mask is None:
            _check(self._lib.cubert_b200_forward_device(self._handle, self._compute_type, replica, batch, d_ids,
                                                        d_mask, d_segments))
        else:
            assert host_mask.dtype == np.int8 and host_mask.flags["C_CONTIGUOUS"]
            _check(self._lib.cubert_b200_forward_device_masked(self._handle, self._compute_type, replica, batch, d_ids,
                                                               d_mask, d_segments, host_mask.ctypes.data))

    def device_outputs(self, replica=0):
        c = _COutput()
        _check(self._lib.cubert_b200_device_outputs(self._handle, self._compute_type, replica, C.byref(c)))
        return {f: getattr(c, f) for f in Output.FIELDS}

    def synchronize(self, replica=0):
        _check(self._lib.cubert_b200_synchronize(self._handle, self._compute_type, replica))

    def replica_stream(self, replica=0):
        s = C.c_void_p()
        _check(self._lib.cubert_b200_replica_stream(self._handle, self._compute_type, replica, C.byref(s)))
        return s.value

    def replica_device(self, replica=0):
        d = C.c_int()
        _check(self._lib.cubert_b200_replica_device(self._handle, self._compute_type, replica, C.byref(d)))
        return d.value

    def profile_enable(self, enable=True, replica=0):
        _check(self._lib.cubert_b200_profile_enable(self._handle, self._compute_type, replica, 1 if enable else 0))

    def profile_read(self, replica=0):
        """{family: {"ms", "launches", "bytes"}} accumulated since the previous read."""
        p = _CProfile()
        _check(self._lib.cubert_b200_profile_read(self._handle, self._compute_type, replica, C.byref(p)))
        return {n: dict(ms=p.ms[i], launches=p.launches[i], bytes=p.bytes[i]) for i, n in enumerate(K_NAMES)}
