"""ctypes declarations of include/immerdink/immerdink.h and the loading of libimmerdink.so.

Search order: `path`, $IMMERDINK_LIB, $IMMERDINK_LIB_DIR/libimmerdink.so, the package directory.
There is no fallback: when the CUDA library is missing, loading raises OSError."""
import ctypes as C
import os
import threading

from . import host

Tensor, Options = host.CTensor, host.COptions


class Operand(C.Structure):
    _fields_ = [("data", C.c_void_p), ("packed", C.c_void_p), ("packed_bytes", C.c_size_t),
                ("pack", C.c_void_p)]


assert C.sizeof(Operand) == 32

_T, _O, _P = C.POINTER(Tensor), C.POINTER(Options), C.c_void_p
_SZ = C.POINTER(C.c_size_t)
SIGNATURES = {
    "imd_create": [C.POINTER(C.c_void_p)],
    "imd_destroy": [_P],
    "imd_plan_create": [_P, _T, _T, _T, _O, C.POINTER(C.c_void_p)],
    "imd_plan_destroy": [_P],
    "imd_plan_device_bytes": [_P, _SZ],
    "imd_contract": [_P, C.c_double, _P, _P, C.c_double, _P, _P, C.c_size_t, _P],
    "imd_pack_create": [_P, _P, C.POINTER(C.c_void_p)],
    "imd_pack_destroy": [_P],
    "imd_pack_bytes": [_P, _SZ, _SZ],
    "imd_pack": [_P, _P, _P, C.c_size_t, _P, C.c_size_t, _P],
    "imd_plan_create_packed": [_P, _T, _T, _T, _O, _P, _P, C.POINTER(C.c_void_p)],
    "imd_contract_builtin_ws": [_P, C.c_double, _P, _P, C.c_double, _P, _P],
    "imd_contract_packed_part": [_P, C.c_double, C.POINTER(Operand), C.POINTER(Operand), C.c_double,
                                 _P, _P, C.c_size_t, _P, C.c_int32],
    "imd_pack_scatter": [_P, _P, C.c_int64, C.c_int64, C.c_int32, C.POINTER(C.c_void_p), C.c_size_t, _P,
                         C.c_size_t, _P],
    "imd_contract_packed": [_P, C.c_double, C.POINTER(Operand), C.POINTER(Operand), C.c_double,
                            _P, _P, C.c_size_t, _P],
    "imd_wait_flags": [C.POINTER(C.c_void_p), C.c_int, C.c_uint, C.c_uint64, _P],
    "imd_device_error": [C.POINTER(C.c_uint)],
    "imd_device_error_peek": [C.c_void_p, _P],
    "imd_push_ranges": [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.c_int32,
                        C.POINTER(C.c_void_p), C.c_int32, C.c_uint, C.c_int32, _P],
    "imd_copy_if_flagged": [C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_void_p),
                            C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.c_int32, _P],
}


def _candidates():
    if os.environ.get("IMMERDINK_LIB"):
        yield os.environ["IMMERDINK_LIB"]
    if os.environ.get("IMMERDINK_LIB_DIR"):
        yield os.path.join(os.environ["IMMERDINK_LIB_DIR"], "libimmerdink.so")
    yield os.path.join(os.path.dirname(os.path.abspath(__file__)), "libimmerdink.so")


class Library:
    def __init__(self, path=None):
        if path is None:
            for cand in _candidates():
                if os.path.exists(cand):
                    path = cand
                    break
        if path is None:
            raise OSError("libimmerdink.so not found (build it with `python -m immerdink_b200.build`, "
                          "or set IMMERDINK_LIB); there is no CPU fallback")
        self.path = path
        sib = os.path.join(os.path.dirname(os.path.abspath(path)), "libimmerdink_host.so")
        self.host = host.load(sib if os.path.exists(sib) else None)
        lib = self.lib = C.CDLL(path)
        for name, args in SIGNATURES.items():
            f = getattr(lib, name)
            f.restype, f.argtypes = C.c_int, args
        self.cudart = None
        for name in ("libcudart.so.12", "libcudart.so.13", "libcudart.so"):
            try:
                self.cudart = C.CDLL(name)
                break
            except OSError:
                continue

    def device_error(self):
        """imd_device_error: the sticky device error word, read and cleared (synchronises)."""
        v = C.c_uint(0)
        st = self.lib.imd_device_error(C.byref(v))
        if st:
            raise RuntimeError(f"imd_device_error: status {st}")
        return int(v.value)

    def current_device(self):
        if self.cudart is None:
            return 0
        d = C.c_int(0)
        if self.cudart.cudaGetDevice(C.byref(d)) != 0:
            raise RuntimeError("cudaGetDevice failed")
        return d.value

    def sm_count(self, device=None):
        if self.cudart is None:
            return 0
        v = C.c_int(0)
        dev = self.current_device() if device is None else device
        if self.cudart.cudaDeviceGetAttribute(C.byref(v), 16, dev) != 0:
            raise RuntimeError("cudaDeviceGetAttribute failed")
        return v.value


_loaded, _lock = {}, threading.Lock()


def load(path=None):
    with _lock:
        if path not in _loaded:
            _loaded[path] = Library(path)
        return _loaded[path]
