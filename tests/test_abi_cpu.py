"""CPU-only checks of the drop-in boundary: the shared libraries load without a GPU and export
every symbol their public headers declare. No compute call is made here."""
import ctypes
import os
import re

from cubert_b200 import build, kernels

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header, prefix):
    with open(os.path.join(ROOT, "include", header)) as f:
        src = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(%s\w+)\s*\(" % prefix, src)))


def test_kernel_library_exports_every_declared_symbol():
    build.build_kernels(verbose=False)
    lib = ctypes.CDLL(kernels.KERNEL_LIB)
    declared = _declared("cubert_kernels.h", "cubk_")
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(kernels.exported_symbols()) == declared
    assert kernels.load().cubk_version() >= 100


def test_kernel_binding_fails_loudly_without_the_library(monkeypatch):
    monkeypatch.setattr(kernels, "KERNEL_LIB", "/nonexistent/libcubert_kernels.so")
    monkeypatch.setattr(kernels, "_lib", None)
    try:
        kernels.load()
    except RuntimeError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("load() must raise when the CUDA library is missing")
