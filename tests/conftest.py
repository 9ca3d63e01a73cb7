"""Shared pytest configuration.

Markers:
  gpu -- needs a CUDA device (the parity tests proper; they call the CUDA kernels
         through the C-ABI). Everything else runs on CPU only.
"""
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device")
    # Bind the CUDA toolkit's cuBLAS (what a C or C++ host of libcuBERT.so gets) before torch loads the
    # older copy it bundles; harmless when the native libraries are not built yet.
    try:
        from cubert_b200 import model
        model.load()
    except Exception:
        pass


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def kernel_options():
    """Setter for the kernel library's tuning switches (cubk_set_option); the values a test changes are put
    back when it ends."""
    from cubert_b200 import kernels
    saved = {}

    def set_option(option, value):
        old = kernels.set_option(option, value)
        saved.setdefault(option, old)

    yield set_option
    for option, old in saved.items():
        kernels.set_option(option, old)


@pytest.fixture(scope="session")
def oracle():
    from oracle import bindings
    bindings.build()
    return bindings.Oracle()


@pytest.fixture(scope="session")
def reference_cpu():
    """The reference's own CPU code, where oracle/_ref could be built."""
    from oracle import bindings
    if not os.path.exists(bindings.REF_CPU_SO):
        if bindings.reference_tree_present():
            bindings.build(ref=True)
        else:
            pytest.skip("oracle/_ref not built (reference tree absent)")
    return bindings.Reference()


@pytest.fixture(scope="session")
def reference_python_wrapper():
    """The reference's own Cython module (python/cuBERT.pyx, unmodified) linked against OUR library."""
    from cubert_b200 import build as native
    from oracle import bindings
    native.build_all(verbose=False)
    folder = bindings.build_pywrap()
    if folder is None:
        pytest.skip("reference wrapper not built (reference tree absent)")
    if folder not in sys.path:
        sys.path.insert(0, folder)
    import cuBERT
    return cuBERT


@pytest.fixture(scope="session")
def kats():
    with open(os.path.join(ROOT, "tests", "golden", "reference_kats.json")) as f:
        return json.load(f)


def kat_expect(entry, name=None):
    """[(index, value, tol)] of one known-answer test, optionally for one array name."""
    return [(i, v, t) for (n, i, v, t) in entry["expect"] if name is None or n == name]


def assert_kat(entry, got, name=None, float_eq_ulps=4):
    """Apply a reference test's EXPECT_NEAR / EXPECT_FLOAT_EQ lines to `got`."""
    got = np.asarray(got, np.float32).ravel()
    for idx, val, tol in kat_expect(entry, name):
        if tol is None:  # EXPECT_FLOAT_EQ: within 4 ULPs
            want = np.float32(val)
            ulp = np.spacing(np.abs(want)) if want != 0 else np.float32(1e-37)
            assert abs(got[idx] - want) <= float_eq_ulps * ulp, (idx, got[idx], val)
        else:
            assert abs(float(got[idx]) - val) <= tol, (idx, got[idx], val, tol)
