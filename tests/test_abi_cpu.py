"""CPU-only checks of the drop-in boundary: the shared libraries load without a GPU and export
every symbol their public headers declare. No compute call is made here."""
import ctypes
import os
import re

import pytest

from cubert_b200 import build, kernels, model

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


def test_host_library_exports_the_reference_api_and_the_additions():
    build.build_all(verbose=False)
    lib = ctypes.CDLL(model.HOST_LIB)
    declared = _declared("cuBERT.h", "cuBERT_") + _declared("cubert_b200.h", "cubert_b200_")
    assert {"cuBERT_open", "cuBERT_compute", "cuBERT_compute_m", "cuBERT_close", "cuBERT_get_gpu_count",
            "cuBERT_tokenize_compute"} <= set(declared)
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(model.exported_symbols()) == sorted(set(declared))


def test_reference_cython_wrapper_binds_to_this_library(reference_python_wrapper):
    """python/cuBERT.pyx + python/_cuBERT.pxd + the reference's src/cuBERT.h, compiled unchanged, link
    and load against our libcuBERT.so; enum values and exception translation come through."""
    cuBERT = reference_python_wrapper
    assert cuBERT.get_gpu_count() == model.get_gpu_count()
    assert (cuBERT.ComputeType.FLOAT, cuBERT.ComputeType.HALF) == (0, 1)
    assert (cuBERT.OutputType.LOGITS, cuBERT.OutputType.POOLED_OUTPUT, cuBERT.OutputType.SEQUENCE_OUTPUT,
            cuBERT.OutputType.EMBEDDING_OUTPUT, cuBERT.OutputType.PROBS) == (0, 1, 2, 3, 4)
    with pytest.raises(ValueError, match="model file not found"):   # std::invalid_argument through `except +`
        cuBERT.Model("/no/such/model.pb", 8, 32, 12, 12)


def test_headers_are_plain_c_and_a_c_program_links(tmp_path):
    """The boundary is a C ABI: every header under include/ must compile as C99 (and as C++), and a C
    program that names entry points of both libraries must link against them (no GPU needed to link)."""
    import shutil
    import subprocess
    from cubert_b200 import build as native
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    native.build_all(verbose=False)
    inc = os.path.join(ROOT, "include")
    for header in sorted(os.listdir(inc)):
        for compiler, std in (("gcc", "-std=c99"), ("g++", "-std=c++11")):
            proc = subprocess.run([compiler, std, "-pedantic", "-Wall", "-Werror", "-I" + inc, "-x",
                                   "c" if compiler == "gcc" else "c++", "-fsyntax-only", "-"],
                                  input='#include "%s"\n' % header, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                  universal_newlines=True)
            assert proc.returncode == 0, (header, compiler, proc.stdout)
    src = tmp_path / "link.c"
    src.write_text('#include <stdio.h>\n#include "cuBERT.h"\n#include "cubert_b200.h"\n#include "cubert_kernels.h"\n'
                   "int main(void) {\n"
                   '    printf("%d %p %p %p\\n", cubk_version(), (void *) cuBERT_open, (void *) cubert_b200_compute_m,\n'
                   "           (void *) cubk_masked_softmax_f16);\n"
                   "    return cubk_bias_gelu_f32(0, 0, 0, 0, 0, 0) == CUBK_ERR_INVALID_ARG ? 0 : 1;\n}\n")
    exe = str(tmp_path / "link")
    lib = os.path.join(ROOT, "cubert_b200", "lib")
    proc = subprocess.run(["gcc", "-std=c99", "-I" + inc, str(src), "-L" + lib, "-lcuBERT", "-lcubert_kernels",
                           "-Wl,-rpath," + lib, "-o", exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          universal_newlines=True)
    assert proc.returncode == 0, proc.stdout
    run = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, universal_newlines=True)
    assert run.returncode == 0, run.stdout          # argument validation happens before any CUDA call
