"""In-tree build of the native libraries for sm_100a.

    python -m cubert_b200.build          # build what is stale
    python -m cubert_b200.build --force  # rebuild everything

Produces, next to this file:
    lib/libcubert_kernels.so  -- the fused kernels and their C ABI (include/cubert_kernels.h)
    lib/libcuBERT.so          -- the host library with the cuBERT C API (include/cuBERT.h),
                                 linked against libcubert_kernels.so, cuBLAS and cuBLASLt
    lib/serve_mix             -- closed-loop serving client in native code (csrc/bench/serve_mix.cpp),
                                 a C++ program that uses nothing but the C API

nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
INCLUDE = os.path.join(ROOT, "include")

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
HOST_CXX = "g++"  # the image's $CXX points at a compiler without OpenMP specs; use the system one

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-ccbin", HOST_CXX, "-cudart", "shared",
                           "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-I" + INCLUDE]

KERNEL_LIB = os.path.join(LIBDIR, "libcubert_kernels.so")
HOST_LIB = os.path.join(LIBDIR, "libcuBERT.so")
SERVE_MIX = os.path.join(LIBDIR, "serve_mix")


def _sources(sub):
    d = os.path.join(CSRC, sub)
    if not os.path.isdir(d):
        return [], []
    files = sorted(os.listdir(d))
    srcs = [os.path.join(d, f) for f in files if f.endswith((".cu", ".cpp"))]
    hdrs = [os.path.join(d, f) for f in files if f.endswith((".cuh", ".h", ".hpp", ".inc"))]
    return srcs, hdrs


def _mtime(p):
    return os.path.getmtime(p) if os.path.exists(p) else 0.0


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), proc.stdout))
    return proc.stdout


def _compile(sub, extra_flags, force, verbose):
    srcs, hdrs = _sources(sub)
    public = [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    newest_hdr = max([_mtime(h) for h in hdrs + public] + [_mtime(os.path.abspath(__file__))])
    os.makedirs(os.path.join(OBJDIR, sub), exist_ok=True)
    jobs, objs = [], []
    for src in srcs:
        obj = os.path.join(OBJDIR, sub, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _mtime(obj) < max(_mtime(src), newest_hdr):
            jobs.append([NVCC] + NVCC_FLAGS + extra_flags + ["-x", "cu", "-c", src, "-o", obj])
    if jobs:
        if verbose:
            print("[build] compiling %d file(s) in csrc/%s" % (len(jobs), sub), file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(_run, jobs))
    return objs, bool(jobs)


def _up_to_date(lib, subs, extra=()):
    """True when `lib` exists and is newer than every source and header it is built from (the object
    files need not exist: a tree that was copied without its build folder is not recompiled)."""
    if not os.path.exists(lib):
        return False
    deps = [os.path.abspath(__file__)] + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)] + list(extra)
    for sub in subs:
        srcs, hdrs = _sources(sub)
        deps += srcs + hdrs
    return _mtime(lib) >= max(_mtime(d) for d in deps)


def build_kernels(force=False, verbose=True):
    if not force and _up_to_date(KERNEL_LIB, ["kernels"]):
        return KERNEL_LIB
    objs, changed = _compile("kernels", [], force, verbose)
    if not objs:
        raise RuntimeError("no kernel sources under %s" % CSRC)
    if changed or not os.path.exists(KERNEL_LIB):
        os.makedirs(LIBDIR, exist_ok=True)
        _run([NVCC] + ARCH_FLAGS + ["-shared", "-cudart", "shared", "-ccbin", HOST_CXX, "-o", KERNEL_LIB] + objs +
             ["-Xlinker", "-rpath," + os.path.join(CUDA_HOME, "lib64")])
    return KERNEL_LIB


def build_host(force=False, verbose=True):
    srcs, _ = _sources("host")
    if not srcs:
        return None
    kernel_lib = build_kernels(force=False, verbose=verbose)
    if not force and _up_to_date(HOST_LIB, ["host"], [kernel_lib]):
        return HOST_LIB
    objs, changed = _compile("host", ["-I" + os.path.join(CSRC, "host")], force, verbose)
    if changed or _mtime(HOST_LIB) < _mtime(kernel_lib):
        _run([NVCC] + ARCH_FLAGS + ["-shared", "-cudart", "shared", "-ccbin", HOST_CXX, "-o", HOST_LIB] + objs +
             ["-L" + LIBDIR, "-lcubert_kernels", "-lcublas", "-lcublasLt", "-ldl",
              "-Xlinker", "-rpath,$ORIGIN", "-Xlinker", "-rpath," + os.path.join(CUDA_HOME, "lib64")])
    return HOST_LIB


def build_serve_mix(force=False, verbose=True):
    src = os.path.join(CSRC, "bench", "serve_mix.cpp")
    if not os.path.exists(src):
        return None
    host_lib = build_host(force=False, verbose=verbose)
    if not force and os.path.exists(SERVE_MIX) and _mtime(SERVE_MIX) >= max(_mtime(src), _mtime(host_lib)):
        return SERVE_MIX
    if verbose:
        print("[build] compiling csrc/bench/serve_mix.cpp", file=sys.stderr)
    _run([HOST_CXX, "-O2", "-std=c++17", "-pthread", "-I" + INCLUDE, src, "-o", SERVE_MIX, "-L" + LIBDIR, "-lcuBERT",
          "-lcubert_kernels", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64")])
    return SERVE_MIX


def build_all(force=False, verbose=True):
    out = [build_kernels(force, verbose)]
    host = build_host(force, verbose)
    if host:
        out.append(host)
        client = build_serve_mix(force, verbose)
        if client:
            out.append(client)
    return out


if __name__ == "__main__":
    for lib in build_all(force="--force" in sys.argv):
        print(lib)
