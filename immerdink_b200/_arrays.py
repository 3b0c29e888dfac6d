"""Reading CUDA arrays without any array library: `__cuda_array_interface__` (v2 / v3), DLPack
capsules (0.x and 1.x), raw pointers (`DeviceArray`) and stream objects. ctypes only: no CUDA
call, no copy, no allocation. Same protocol rules as the reference front end
(python/immerdink/_arrays.py:118-240): float64 is checked by the caller, byte strides are
returned as given (None = C-contiguous), a v3 "stream" other than the call's stream is refused
under the "check" policy."""
import ctypes as C
import math
import os

_check_streams = os.environ.get("IMMERDINK_CAI_SYNC", "1").strip() != "0"


def set_cai_stream_policy(policy):
    """"check" (default) or "ignore": what to do with a producer stream that differs from the
    call's stream. The library never synchronises streams itself."""
    global _check_streams
    if policy not in ("check", "ignore"):
        raise ValueError("policy must be 'check' or 'ignore'")
    _check_streams = policy == "check"


def get_cai_stream_policy():
    return "check" if _check_streams else "ignore"


class DeviceArray:
    """A raw device pointer seen as an array. `ptr` addresses element (0, ..., 0); `strides`
    in ELEMENTS (None = dense, last mode fastest). Never dereferenced or freed here."""

    def __init__(self, ptr, shape, strides=None, dtype="f8", readonly=False):
        if isinstance(ptr, C.c_void_p):
            ptr = ptr.value
        self.ptr = int(ptr or 0)
        self.shape = tuple(int(e) for e in shape)
        self.dtype = dtype.lstrip("<|=")
        self.readonly = bool(readonly)
        item = int(self.dtype[1:])
        self.strides = None if strides is None else tuple(int(s) for s in strides)
        if self.strides is not None and len(self.strides) != len(self.shape):
            raise ValueError("one stride per mode")
        self.__cuda_array_interface__ = {
            "shape": self.shape, "typestr": ("|" if item == 1 else "<") + self.dtype,
            "data": (self.ptr, self.readonly), "version": 3, "stream": None,
            "strides": None if self.strides is None else tuple(s * item for s in self.strides)}

    @property
    def nbytes(self):
        return math.prod(self.shape) * int(self.dtype[1:])


class _DLTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("device_type", C.c_int32), ("device_id", C.c_int32),
                ("ndim", C.c_int32), ("code", C.c_uint8), ("bits", C.c_uint8),
                ("lanes", C.c_uint16), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("byte_offset", C.c_uint64)]


_py = C.pythonapi
_py.PyCapsule_GetPointer.argtypes = [C.py_object, C.c_char_p]
_py.PyCapsule_GetPointer.restype = C.c_void_p
_py.PyCapsule_GetName.argtypes = [C.py_object]
_py.PyCapsule_GetName.restype = C.c_char_p


def _from_dlpack(x, stream, device):
    kind, dev_id = (int(v) for v in x.__dlpack_device__())
    if kind not in (2, 13):  # kDLCUDA, kDLCUDAManaged
        raise TypeError(f"{type(x).__name__} is not in CUDA memory (DLPack device type {kind})")
    if device is not None and kind == 2 and dev_id != device:
        raise ValueError(f"{type(x).__name__} is on CUDA device {dev_id}, the plan on {device}")
    s = -1 if stream is None else 1 if stream == 0 else stream
    try:
        cap = x.__dlpack__(stream=s, max_version=(1, 0))
    except TypeError:
        cap = x.__dlpack__(stream=s)
    name = _py.PyCapsule_GetName(cap)
    base = _py.PyCapsule_GetPointer(cap, name)
    readonly = False
    if name == b"dltensor_versioned":
        # version (2 x u32), manager_ctx, deleter, flags (u64), then the DLTensor
        readonly = bool(C.c_uint64.from_address(base + 24).value & 1)
        base += 32
    elif name != b"dltensor":
        raise TypeError("__dlpack__ did not return a DLPack capsule")
    t = _DLTensor.from_address(base)
    nd = t.ndim
    shape = tuple(t.shape[i] for i in range(nd))
    item = t.bits * t.lanes // 8
    strides = None if not t.strides else tuple(t.strides[i] * item for i in range(nd))
    f8 = t.code == 2 and t.bits == 64 and t.lanes == 1
    return (t.data or 0) + t.byte_offset, shape, strides, f8, readonly, item


def view(x, stream=None, device=None):
    """(ptr, shape, byte strides or None, is_float64, readonly, itemsize) of a CUDA array."""
    cai = getattr(x, "__cuda_array_interface__", None)
    if cai is None:
        if hasattr(x, "__dlpack__"):
            return _from_dlpack(x, stream, device)
        raise TypeError(f"{type(x).__name__} is not a CUDA array: it has neither "
                        "__cuda_array_interface__ nor __dlpack__ (nothing is copied from the host)")
    if cai.get("mask") is not None:
        raise TypeError("masked arrays are not supported")
    if _check_streams and stream is not None:
        theirs = cai.get("stream")
        if theirs is not None and theirs != stream and not (theirs == 1 and stream == 0):
            raise ValueError(f"{type(x).__name__} was produced on stream {theirs}, the call runs on "
                             f"{stream}: pass stream=..., or set_cai_stream_policy('ignore')")
    ts = cai["typestr"]
    ptr, readonly = cai["data"]
    return ptr or 0, cai["shape"], cai.get("strides"), ts == "<f8", readonly, int(ts[2:])


def buffer(x, what, writable=True, stream=None, device=None):
    """(ptr, nbytes) of a byte buffer: None, an (int ptr, nbytes) tuple or a contiguous array."""
    if x is None:
        return None, 0
    if isinstance(x, tuple):
        return int(x[0] or 0), int(x[1])
    ptr, shape, strides, _, readonly, item = view(x, stream, device)
    if writable and readonly:
        raise ValueError(f"{what} is read-only")
    n = math.prod(shape)
    if strides is not None and n > 1:
        acc = item
        for e, s in zip(reversed(shape), reversed(strides)):
            if e > 1 and s != acc:
                raise ValueError(f"{what} must be contiguous")
            acc *= e
    return ptr, n * item


def stream_handle(s):
    """cudaStream_t value: None / 0 = the default stream, ints as is, `__cuda_stream__`,
    `.cuda_stream` (PyTorch), `.ptr` (CuPy), c_void_p."""
    if s is None:
        return 0
    if isinstance(s, int):
        return s
    if hasattr(s, "__cuda_stream__"):
        return int(s.__cuda_stream__()[1])
    for attr in ("cuda_stream", "ptr"):
        h = getattr(s, attr, None)
        if isinstance(h, int):
            return h
    if isinstance(s, C.c_void_p):
        return s.value or 0
    raise TypeError(f"not a CUDA stream: {type(s).__name__}")
