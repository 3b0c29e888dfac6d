"""The C-ABI libraries load and export every symbol the headers declare (no GPU needed)."""
import ctypes
import os
import re

from immerdink_b200 import _capi, build, host

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared(header):
    text = open(os.path.join(ROOT, "include", "immerdink", header)).read()
    return sorted(set(re.findall(r"IMD_API[^;]*?\b(imd_[a-z0-9_]+)\s*\(", text)))


def test_host_library_exports_header():
    build.build_host()
    lib = ctypes.CDLL(build.HOST_LIB)
    names = declared("immerdink_host.h")
    assert len(names) == 29 and sorted(host.HOST_SYMBOLS) == names
    for n in names:
        getattr(lib, n)


def test_cuda_library_exports_header_and_refuses_without_gpu():
    build.build_cuda()
    lib = ctypes.CDLL(build.CUDA_LIB)
    names = declared("immerdink.h")
    assert len(names) == 20 and sorted(_capi.SIGNATURES) == names  # the reference's 12 + eight
    for n in names + declared("immerdink_host.h"):
        getattr(lib, n)          # host symbols reachable through DT_NEEDED
    # the production library exports no verification or profiling hook; the instrumented one does
    import subprocess
    def exported(path):
        out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True).stdout
        return {ln.split()[-1] for ln in out.splitlines() if " T " in ln and "imd_" in ln}
    plain, hooked = exported(build.CUDA_LIB), exported(build.HOOKS_LIB)
    assert plain == set(names)
    extra = hooked - plain
    assert extra and all(n.startswith(("imd_test_", "imd_prof_")) for n in extra)
    try:
        import torch
        if torch.cuda.is_available():
            return
    except Exception:
        pass
    h = ctypes.c_void_p()
    assert lib.imd_create(ctypes.byref(h)) == 6   # IMD_STATUS_CUDA_ERROR: no silent CPU path


def test_python_front_end_has_no_cpu_fallback(monkeypatch, tmp_path):
    monkeypatch.setenv("IMMERDINK_LIB", str(tmp_path / "missing.so"))
    monkeypatch.setattr(_capi, "_candidates", lambda: iter([str(tmp_path / "missing.so")]))
    try:
        _capi.Library()
    except OSError as exc:
        assert "no CPU fallback" in str(exc)
    else:
        raise AssertionError("loading must fail loudly")
