"""In-tree build of the two shared libraries (no cmake):

    libimmerdink_host.so   CUDA-free host queries        (g++)
    libimmerdink.so        C ABI + sm_100a kernels       (nvcc -gencode arch=compute_100a,code=sm_100a)
    libimmerdink_hooks.so  the same objects + the imd_test_* / imd_prof_* entry points (tests, phase timing)

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
HOOKS_LIB = os.path.join(HERE, "libimmerdink_hooks.so")
OBJ_DIR = os.path.join(HERE, "build")

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
    """Kernel and ABI objects are compiled once; hooks.cpp twice (with and without IMD_HOOKS); the
    two libraries differ only in that object."""
    build_host(force)
    src_time = _newest([CSRC, INCLUDE])
    if (not force and all(os.path.exists(p) and os.path.getmtime(p) >= src_time
                          for p in (CUDA_LIB, HOOKS_LIB))):
        return CUDA_LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    common = [_nvcc(), "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-ccbin", _cxx(), "-I" + INCLUDE, "-I" + CSRC]
    if verbose:
        common[1:1] = ["-Xptxas", "-v"]
    objs, out = [], ""
    for src in CUDA_SOURCES:
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < src_time:
            out += _run(common + ["-c", src, "-o", obj])
        objs.append(obj)
    hooks_src = os.path.join(CSRC, "cuda", "hooks.cpp")
    flavours = []
    for lib, flag in ((CUDA_LIB, None), (HOOKS_LIB, "-DIMD_HOOKS")):
        obj = os.path.join(OBJ_DIR, "hooks" + ("_on" if flag else "_off") + ".o")
        out += _run(common + ([flag] if flag else []) + ["-c", hooks_src, "-o", obj])
        flavours.append((lib, obj))
    for lib, obj in flavours:
        out += _run([_nvcc(), "-shared", "-ccbin", _cxx(), *objs, obj, "-o", lib,
                     "-L" + HERE, "-limmerdink_host", "-Xlinker", "-rpath=$ORIGIN"])
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
    print(HOOKS_LIB)
