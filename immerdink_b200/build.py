"""In-tree build of the two shared libraries (no cmake):

    libimmerdink_host.so   CUDA-free host queries        (g++)
    libimmerdink.so        C ABI + sm_100a kernels       (nvcc -gencode arch=compute_100a,code=sm_100a)

    python -m immerdink_b200.build [--force]

The libraries land next to this file so that they travel with the source tree.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
HOST_LIB = os.path.join(HERE, "libimmerdink_host.so")
CUDA_LIB = os.path.join(HERE, "libimmerdink.so")

HOST_SOURCES = [os.path.join(CSRC, "host", f)
                for f in ("lowering.cpp", "plan.cpp", "pack.cpp", "host_api.cpp", "accuracy.cpp", "perf.cpp",
                          "perf_text.cpp")]
CUDA_SOURCES = [os.path.join(CSRC, "cuda", f)
                for f in ("api.cpp", "pipeline.cu", "gemm_tcgen05.cu")]


def _cxx():
    for c in ("/usr/bin/g++", "g++"):
        if os.path.exists(c) or c == "g++":
            return c


def _nvcc():
    for c in ("/usr/local/cuda/bin/nvcc", "nvcc"):
        if os.path.exists(c) or c == "nvcc":
            return c


def _newest(paths):
    t = 0.0
    for p in paths:
        for base, _, files in os.walk(p) if os.path.isdir(p) else [(os.path.dirname(p), [], [os.path.basename(p)])]:
            for f in files:
                t = max(t, os.path.getmtime(os.path.join(base, f)))
    return t


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build failed: " + os.path.basename(cmd[0]))
    return r.stdout + r.stderr


def build_host(force=False):
    src_time = _newest([os.path.join(CSRC, "host"), os.path.join(CSRC, "common"), INCLUDE])
    if not force and os.path.exists(HOST_LIB) and os.path.getmtime(HOST_LIB) >= src_time:
        return HOST_LIB
    _run([_cxx(), "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-Wextra",
          "-I" + INCLUDE, *HOST_SOURCES, "-o", HOST_LIB])
    return HOST_LIB


def build_cuda(force=False, verbose=False):
    build_host(force)
    src_time = _newest([CSRC, INCLUDE])
    if not force and os.path.exists(CUDA_LIB) and os.path.getmtime(CUDA_LIB) >= src_time:
        return CUDA_LIB
    cmd = [_nvcc(), "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-ccbin", _cxx(),
           "-I" + INCLUDE, "-I" + CSRC, *CUDA_SOURCES, "-o", CUDA_LIB,
           "-L" + HERE, "-limmerdink_host", "-Xlinker", "-rpath=$ORIGIN"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    out = _run(cmd)
    if verbose:
        print(out)
    return CUDA_LIB


def build_all(force=False, verbose=False):
    build_host(force)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(HOST_LIB)
    print(CUDA_LIB)
