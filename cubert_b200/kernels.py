"""ctypes binding of the kernel C ABI (include/cubert_kernels.h).

This is the Python-side stub a maintainer of a Python host would use; the C++ host
library links the same symbols directly. The CUDA library is mandatory: importing
this module never builds or substitutes anything, and `load()` raises if
``lib/libcubert_kernels.so`` is missing. There is no CPU path.

All pointer arguments are raw device addresses (ints), e.g. ``tensor.data_ptr()``.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB = os.path.join(HERE, "lib", "libcubert_kernels.so")

CUBK_OK = 0
CUBK_ERR_INVALID_ARG = -1
CUBK_ERR_UNSUPPORTED = -2
CUBK_ERR_LAUNCH = -3
CUBK_ERR_SCRATCH = -4
STATIC_POOL_SCRATCH_BYTES = 512 * 1024
STATUS_BAD_TOKEN_ID = 1
STATUS_BAD_SEGMENT_ID = 2
STATUS_COPY_TIMEOUT = 4
OPT_EMBED_STAGED_ROWS = 0
OPT_SOFTMAX_MASK_SMEM = 1
OPT_EXACT_WIDTH_ROWS = 2
OPT_EXACT_WIDTH_EMBED = 3
OPT_ATTENTION_TENSOR_MEMORY = 4

_P = C.c_void_p
_I = C.c_int
_L = C.c_int64
_F = C.c_float
_Z = C.c_size_t

# name -> (restype, argtypes); `{t}` expands to f32 and f16
_SIGNATURES = {
    "cubk_version": (_I, []),
    "cubk_last_cuda_error": (C.c_char_p, []),
    "cubk_set_option": (_I, [_I, _I]),
    "cubk_get_option": (_I, [_I, _P]),
    "cubk_copy_timeouts": (_I, [_P]),
    "cubk_selftest_copy_wait_timeout": (_I, [C.c_uint, _P, _P]),
    "cubk_embed_ln_{t}": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P]),
    "cubk_embed_gather_i32": (_I, [_P, _L, _P, _I, _I, _I, _P, _P, _P]),
    "cubk_embed_gather_i8": (_I, [_P, _L, _P, _I, _I, _I, _P, _P, _P]),
    "cubk_scatter_rows": (_I, [_P, _L, _P, _I, _I, _P, _I, _P]),
    "cubk_bias_residual_ln_{t}": (_I, [_P, _P, _P, _P, _P, _L, _I, _P, _P]),
    "cubk_bias_gelu_{t}": (_I, [_P, _P, _L, _I, _P, _P]),
    "cubk_masked_softmax_{t}": (_I, [_P, _P, _L, _L, _I, _F, _P, _P]),
    "cubk_masked_softmax_extents_{t}": (_I, [_P, _P, _P, _I, _L, _L, _I, _F, _P, _P]),
    "cubk_attention_small_{t}": (_I, [_P, _P, _I, _I, _I, _I, _F, _P, _P]),
    "cubk_bias_tanh_{t}": (_I, [_P, _P, _L, _I, _P, _P]),
    "cubk_mean_pool_scratch_bytes": (_Z, [_I, _I, _I]),
    "cubk_mean_pool_{t}": (_I, [_P, _I, _I, _I, _P, _P, _Z, _P]),
    "cubk_mean_pool_static_scratch": (_I, [_P, _I, _I, _I, _I, _P, _P]),
    "cubk_logits_probs_{t}": (_I, [_P, _P, _P, _I, _I, _I, _P, _P, _P]),
    "cubk_pooler_head_{t}": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P]),
    "cubk_not_{t}": (_I, [_P, _P, _L, _P]),
    "cubk_half_to_float": (_I, [_P, _P, _L, _P]),
}


def exported_symbols():
    """Every symbol include/cubert_kernels.h declares."""
    names = []
    for pattern in _SIGNATURES:
        if "{t}" in pattern:
            names += [pattern.format(t="f32"), pattern.format(t="f16")]
        else:
            names.append(pattern)
    return names


_lib = None


def load():
    """Load the kernel library; raises RuntimeError if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(KERNEL_LIB):
        raise RuntimeError("%s is missing: run `python -m cubert_b200.build` (there is no CPU fallback)"
                           % KERNEL_LIB)
    lib = C.CDLL(KERNEL_LIB, mode=C.RTLD_GLOBAL)
    for pattern, (res, args) in _SIGNATURES.items():
        for t in (("f32", "f16") if "{t}" in pattern else ("",)):
            fn = getattr(lib, pattern.format(t=t))
            fn.restype = res
            fn.argtypes = args
    _lib = lib
    return lib


class KernelError(RuntimeError):
    pass


def check(rc):
    if rc != CUBK_OK:
        detail = load().cubk_last_cuda_error().decode() if rc == CUBK_ERR_LAUNCH else ""
        raise KernelError("cubk call failed with status %d %s" % (rc, detail))


def set_option(option, value):
    """Change a process-wide tuning switch (OPT_*); returns the value it had."""
    old = C.c_int(0)
    check(load().cubk_get_option(option, C.byref(old)))
    check(load().cubk_set_option(option, int(value)))
    return old.value


def get_option(option):
    v = C.c_int(0)
    check(load().cubk_get_option(option, C.byref(v)))
    return v.value


def copy_timeouts():
    """Warps on the current device that gave up waiting for a shared-memory copy (expected: 0)."""
    n = C.c_uint(0)
    check(load().cubk_copy_timeouts(C.byref(n)))
    return n.value
