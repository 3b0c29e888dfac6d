"""Host queries without a GPU: exact workspace footprints, the lowering summary and the error
estimates, straight from libimmerdink_host.so (ctypes). Nothing is recomputed in Python.

    from immerdink_b200 import host
    spec, ext = "kjbc,kiac->abij", dict(a=200, b=200, c=200, i=40, j=40, k=40)
    host.workspace_size(spec, ext, N=14, g=7)
    host.workspace_layout(spec, ext, N=14)
    host.lowering(spec, ext, N=14)
    host.err_estimate(N=14, k=8000)

Mirrors the reference's python/immerdink/host.py for the queries of the contraction path
(workspace_size, lowering, workspace_layout, plan_bytes, g_tradeoff, err_estimate, min_moduli) and
of packed operands (PackSpec, pack_layout, pack_desc_for, `packing=` of workspace_size and
lowering): same names, arguments (einsum spec + extents dict, or raw (extent, stride, label)
descriptors) and error type. The performance-model queries are not provided.

Library search: `lib=` path, $IMMERDINK_HOST_LIB, $IMMERDINK_LIB_DIR/libimmerdink_host.so, the
package directory.
"""
import ctypes as C
import os
from dataclasses import dataclass

API_VERSION = 13

STATUS = ["SUCCESS", "INVALID_VALUE", "NOT_SUPPORTED", "ALIASING", "INSUFFICIENT_WORKSPACE",
          "MISALIGNED", "CUDA_ERROR", "ALLOC_FAILED", "PACK_MISMATCH"]
REGIONS = ["sA", "sB", "fA", "fB", "vec", "RA", "RB", "W"]
DISPATCH = ["NOOP", "EMULATE", "DIRECT", "SCALE"]
ROUNDING = {"RN": 0, "TRUNC": 1}
MODE = {"EMULATE": 0, "DIRECT": 1}
VEC = {"GENERATE": 0, "RESIDENT": 1}
ERR_METRICS = {"NORMWISE": 0, "ELEMENTWISE": 1, "ABSOLUTE": 2}
ERR_BASES = {"BOUND": 0, "TYPICAL": 1}
ERR_STATUS = ["UNCHECKED", "MET", "MISSED"]


class ImmerdinkError(RuntimeError):
    """A non-SUCCESS status of the host library; `.status` is its name."""

    def __init__(self, status, what=""):
        self.status = STATUS[status] if 0 <= status < len(STATUS) else f"<{status}>"
        super().__init__(f"{what}: IMD_STATUS_{self.status}" if what else self.status)


class CTensor(C.Structure):
    _fields_ = [("rank", C.c_int32), ("extent", C.POINTER(C.c_int64)),
                ("stride", C.POINTER(C.c_int64)), ("label", C.POINTER(C.c_int32))]


class COptions(C.Structure):
    _fields_ = [("num_moduli", C.c_int32), ("residue_group", C.c_int32), ("rounding", C.c_int32),
                ("mode", C.c_int32), ("vec_mode", C.c_int32), ("k4_tune", C.c_int32)]


class CRegion(C.Structure):
    _fields_ = [("offset", C.c_uint64), ("bytes", C.c_uint64)]


class CLowering(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("status", C.c_int32), ("lowered", C.c_int32),
                ("dispatch", C.c_int32), ("swapped", C.c_int32), ("num_moduli", C.c_int32),
                ("residue_group", C.c_int32), ("num_groups", C.c_int32),
                ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("b", C.c_int64),
                ("n_hat", C.c_int64), ("k_hat", C.c_int64), ("vec_entries", C.c_int64),
                ("k_chunks", C.c_int64), ("gemm_launches", C.c_int64), ("kappa", C.c_uint64),
                ("workspace_bytes", C.c_uint64), ("plan_device_bytes", C.c_uint64),
                ("plan_host_bytes", C.c_uint64), ("fused", C.c_int32), ("reserved", C.c_int32),
                ("kernel_launches", C.c_int64), ("sm_count", C.c_int32), ("k4_config", C.c_int32),
                ("k4_tune_bytes", C.c_uint64), ("fused_large", C.c_int32), ("reserved4", C.c_int32),
                ("packed", C.c_int32), ("pack_mismatch", C.c_int32), ("k_align", C.c_int32),
                ("reserved6", C.c_int32)]


class CErrRequest(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("metric", C.c_int32), ("target", C.c_double),
                ("cond", C.c_double), ("norm_product", C.c_double), ("l1_ratio_a", C.c_double),
                ("l1_ratio_b", C.c_double), ("basis", C.c_int32), ("reserved", C.c_int32),
                ("fail_prob", C.c_double)]


class CErr(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("status", C.c_int32), ("num_moduli", C.c_int32),
                ("rounding", C.c_int32), ("dispatch", C.c_int32), ("err_status", C.c_int32),
                ("k", C.c_int64), ("outputs", C.c_int64), ("bound", C.c_double),
                ("typical", C.c_double), ("unit_bound", C.c_double), ("unit_typical", C.c_double)]


class CPackDesc(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("num_moduli", C.c_int32), ("rounding", C.c_int32),
                ("order", C.c_int32), ("tensor", C.POINTER(CTensor)),
                ("num_contracted", C.c_int32), ("contracted", C.POINTER(C.c_int32)),
                ("num_batch", C.c_int32), ("batch", C.POINTER(C.c_int32)),
                ("num_rows", C.c_int32), ("rows", C.POINTER(C.c_int32))]


class CPackLayout(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("status", C.c_int32), ("format", C.c_int32),
                ("num_moduli", C.c_int32), ("rounding", C.c_int32), ("reserved", C.c_int32),
                ("b", C.c_int64), ("r", C.c_int64), ("k", C.c_int64), ("k_hat", C.c_int64),
                ("kappa", C.c_uint64), ("sig", CRegion), ("flag", CRegion), ("res", CRegion),
                ("pack_bytes", C.c_uint64), ("pack_ws_bytes", C.c_uint64), ("key_digest", C.c_uint64)]


class CPacking(C.Structure):
    _fields_ = [("A", C.POINTER(CPackDesc)), ("B", C.POINTER(CPackDesc))]


assert C.sizeof(CPackDesc) == 72 and C.sizeof(CPackLayout) == 136 and C.sizeof(CPacking) == 16
assert C.sizeof(CTensor) == 32 and C.sizeof(COptions) == 24 and C.sizeof(CLowering) == 192
assert C.sizeof(CErrRequest) == 64 and C.sizeof(CErr) == 72

# Every symbol of the host ABI; a library missing one is not a drop-in.
HOST_SYMBOLS = (
    "imd_host_api_version", "imd_workspace_size", "imd_workspace_layout", "imd_region_name",
    "imd_plan_bytes", "imd_lowering", "imd_pack_layout", "imd_pack_desc_for",
    "imd_workspace_size_packed", "imd_workspace_layout_packed", "imd_lowering_packed",
    "imd_status_string", "imd_perf_kernel_name", "imd_perf_calib_default", "imd_perf_calib_parse",
    "imd_perf_calib_load", "imd_perf_calib_parse_ex", "imd_perf_calib_load_ex",
    "imd_perf_calib_default_ex", "imd_perf_calib_error_name", "imd_perf_calib_format",
    "imd_perf_class_name", "imd_perf_param_name", "imd_perf_phase_name", "imd_perf_predict",
    "imd_perf_predict_pack", "imd_perf_rank", "imd_err_estimate", "imd_err_min_moduli")


def _candidates():
    if os.environ.get("IMMERDINK_HOST_LIB"):
        yield os.environ["IMMERDINK_HOST_LIB"]
    if os.environ.get("IMMERDINK_LIB_DIR"):
        yield os.path.join(os.environ["IMMERDINK_LIB_DIR"], "libimmerdink_host.so")
    yield os.path.join(os.path.dirname(os.path.abspath(__file__)), "libimmerdink_host.so")


class HostLibrary:
    def __init__(self, path=None):
        if path is None:
            for cand in _candidates():
                if os.path.exists(cand):
                    path = cand
                    break
        if path is None:
            raise OSError("libimmerdink_host.so not found: build it with "
                          "`python -m immerdink_b200.build` or set IMMERDINK_HOST_LIB")
        self.path = path
        L = self.lib = C.CDLL(path)
        for name in HOST_SYMBOLS:
            getattr(L, name)
        T, O = C.POINTER(CTensor), C.POINTER(COptions)
        L.imd_host_api_version.restype = C.c_uint32
        L.imd_status_string.restype = C.c_char_p
        L.imd_region_name.restype = C.c_char_p
        L.imd_workspace_size.argtypes = [T, T, T, O, C.POINTER(C.c_size_t)]
        L.imd_workspace_layout.argtypes = [T, T, T, O, C.POINTER(CRegion), C.c_int32,
                                           C.POINTER(C.c_int32), C.POINTER(C.c_size_t)]
        L.imd_plan_bytes.argtypes = [T, T, T, O, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        L.imd_lowering.argtypes = [T, T, T, O, C.POINTER(CLowering)]
        L.imd_err_estimate.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64,
                                       C.POINTER(CErrRequest), C.POINTER(CErr)]
        L.imd_err_min_moduli.argtypes = [T, T, T, O, C.c_int32, C.c_int32,
                                         C.POINTER(CErrRequest), C.POINTER(CErr)]
        self.version = L.imd_host_api_version()
        if self.version < API_VERSION:
            raise OSError(f"{path}: host API {self.version} < {API_VERSION}")


_libs = {}


def load(path=None):
    if path not in _libs:
        _libs[path] = HostLibrary(path)
    return _libs[path]


@dataclass(frozen=True)
class Desc:
    """One tensor: extents, element strides (any sign), integer labels."""
    extent: tuple
    stride: tuple
    label: tuple

    def __post_init__(self):
        object.__setattr__(self, "extent", tuple(int(x) for x in self.extent))
        object.__setattr__(self, "stride", tuple(int(x) for x in self.stride))
        object.__setattr__(self, "label", tuple(int(x) for x in self.label))
        if not len(self.extent) == len(self.stride) == len(self.label):
            raise ValueError("extent, stride and label need one entry per mode")


def dense_strides(extent):
    st, acc = [], 1
    for e in reversed(extent):
        st.append(acc)
        acc *= max(int(e), 1)
    return tuple(reversed(st))


def parse_spec(spec):
    try:
        ins, out = spec.replace(" ", "").split("->")
        a, b = ins.split(",")
    except ValueError:
        raise ValueError(f"spec {spec!r}: expected 'A,B->C'") from None
    return a, b, out


def contraction(spec, extents, strides=None):
    """(A, B, C) descriptors of an einsum spec; dense last-mode-fastest strides by default."""
    labs = parse_spec(spec)
    out = []
    for x, lab in enumerate(labs):
        ext = tuple(extents[c] for c in lab)
        st = dense_strides(ext) if strides is None or strides[x] is None else strides[x]
        out.append(Desc(ext, st, tuple(ord(c) for c in lab)))
    return tuple(out)


class CDesc:
    """Keeps the ctypes arrays of one imd_tensor_t alive."""

    def __init__(self, d):
        n = len(d.extent)
        self.ext = (C.c_int64 * max(n, 1))(*d.extent)
        self.st = (C.c_int64 * max(n, 1))(*d.stride)
        self.lab = (C.c_int32 * max(n, 1))(*d.label)
        self.t = CTensor(n, self.ext, self.st, self.lab)


PACK_MISMATCH = ["NONE", "FORMAT", "MODULI", "ROUNDING", "CLASSES", "EXTENTS", "STRIDES", "ORDER"]


@dataclass(frozen=True)
class PackSpec:
    """What to pack: the operand X and its label classes. `contracted` (K) and `batch` (L) are
    always listed; `rows` (R) only with order "GIVEN" (every label of X listed, each class in
    canonical order, first fastest); with "AUTO" the rest of X's labels are the rows."""
    tensor: Desc
    contracted: tuple
    batch: tuple = ()
    rows: tuple = ()
    N: int = 14
    rounding: str = "RN"
    order: str = "AUTO"

    def with_moduli(self, N):
        from dataclasses import replace
        return replace(self, N=int(N))


class CPackSpec:
    """Keeps the ctypes memory of one imd_pack_desc_t alive."""

    def __init__(self, p):
        self.cd = CDesc(p.tensor)
        k, l, r = [tuple(int(x) for x in t) for t in (p.contracted, p.batch, p.rows)]
        self.k = (C.c_int32 * max(len(k), 1))(*k)
        self.l = (C.c_int32 * max(len(l), 1))(*l)
        self.r = (C.c_int32 * max(len(r), 1))(*r)
        self.d = CPackDesc(C.sizeof(CPackDesc), int(p.N), ROUNDING[p.rounding],
                           {"AUTO": 0, "GIVEN": 1}[p.order], C.pointer(self.cd.t),
                           len(k), self.k if k else None, len(l), self.l if l else None,
                           len(r), self.r if r else None)


def _packing(packing):
    """(CPacking or None, keep-alive objects) from (PackSpec or None, PackSpec or None)."""
    if packing is None or all(p is None for p in packing):
        return None, None
    keep = [None if p is None else CPackSpec(p) for p in packing]
    cp = CPacking(None if keep[0] is None else C.pointer(keep[0].d),
                  None if keep[1] is None else C.pointer(keep[1].d))
    return cp, keep


def pack_layout(spec, lib=None, check=True):
    """Sizes and regions of the packed buffer of a PackSpec, as a dict."""
    L = lib or load()
    cs = CPackSpec(spec)
    out = CPackLayout()
    out.struct_size = C.sizeof(CPackLayout)
    L.lib.imd_pack_layout.argtypes = [C.POINTER(CPackDesc), C.POINTER(CPackLayout)]
    st = L.lib.imd_pack_layout(C.byref(cs.d), C.byref(out))
    if st and check:
        raise ImmerdinkError(st, "imd_pack_layout")
    d = dict(status=STATUS[out.status], format=out.format, N=out.num_moduli,
             rounding="TRUNC" if out.rounding else "RN", b=out.b, r=out.r, k=out.k, k_hat=out.k_hat,
             kappa=out.kappa, sig=(out.sig.offset, out.sig.bytes), flag=(out.flag.offset, out.flag.bytes),
             res=(out.res.offset, out.res.bytes), pack_bytes=out.pack_bytes,
             pack_ws_bytes=out.pack_ws_bytes, key_digest=out.key_digest)
    return d


def pack_desc_for(spec, extents=None, *, operand, N, g=0, rounding="RN", mode="EMULATE",
                  vec_mode="GENERATE", strides=None, lib=None):
    """The GIVEN PackSpec of operand 0 (A) or 1 (B) with exactly the classes and canonical orders
    of the unpacked plan: a pack made from it reproduces that contraction bit for bit."""
    L, ds, o = _call(spec, extents, strides, lib, options(N, g, rounding, mode, vec_mode))
    descs = _descs(spec, extents, strides)
    out = CPackDesc()
    out.struct_size = C.sizeof(CPackDesc)
    cap = len(descs[operand].label)
    labels = (C.c_int32 * max(cap, 1))()
    L.lib.imd_pack_desc_for.argtypes = [C.POINTER(CTensor)] * 3 + [C.POINTER(COptions), C.c_int32,
                                                                    C.POINTER(CPackDesc),
                                                                    C.POINTER(C.c_int32), C.c_int32]
    st = L.lib.imd_pack_desc_for(ds[0].t, ds[1].t, ds[2].t, o, operand, C.byref(out), labels, cap)
    if st:
        raise ImmerdinkError(st, "imd_pack_desc_for")
    take = lambda ptr, n: tuple(ptr[i] for i in range(n))
    return PackSpec(descs[operand], take(out.contracted, out.num_contracted),
                    take(out.batch, out.num_batch), take(out.rows, out.num_rows), int(N), rounding,
                    "GIVEN")


def _descs(spec_or_descs, extents, strides):
    if isinstance(spec_or_descs, str):
        return contraction(spec_or_descs, extents, strides)
    return tuple(d if isinstance(d, Desc) else Desc(*d) for d in spec_or_descs)


def options(N, g=0, rounding="RN", mode="EMULATE", vec_mode="GENERATE", k4_tune=0):
    return COptions(int(N), int(g), ROUNDING[rounding] if isinstance(rounding, str) else rounding,
                    MODE[mode] if isinstance(mode, str) else mode,
                    VEC[vec_mode] if isinstance(vec_mode, str) else vec_mode, int(k4_tune))


def _call(spec, extents, strides, lib, opt):
    ds = [CDesc(d) for d in _descs(spec, extents, strides)]
    return (lib or load()), ds, opt


def workspace_size(spec, extents=None, *, N, g=0, rounding="RN", mode="EMULATE",
                   vec_mode="GENERATE", strides=None, packing=None, lib=None):
    """Bytes of workspace imd_contract needs for this contraction (exact). packing = (PackSpec or
    None, PackSpec or None): the caller's A / B read from packed buffers."""
    L, ds, o = _call(spec, extents, strides, lib, options(N, g, rounding, mode, vec_mode))
    out = C.c_size_t(0)
    cp, keep = _packing(packing)
    if cp is not None:
        L.lib.imd_workspace_size_packed.argtypes = [C.POINTER(CTensor)] * 3 + [
            C.POINTER(COptions), C.POINTER(CPacking), C.POINTER(C.c_size_t)]
        st = L.lib.imd_workspace_size_packed(ds[0].t, ds[1].t, ds[2].t, o, C.byref(cp), C.byref(out))
        if st:
            raise ImmerdinkError(st, "imd_workspace_size_packed")
        return out.value
    st = L.lib.imd_workspace_size(ds[0].t, ds[1].t, ds[2].t, o, C.byref(out))
    if st:
        raise ImmerdinkError(st, "imd_workspace_size")
    return out.value


def workspace_layout(spec, extents=None, *, N, g=0, rounding="RN", mode="EMULATE",
                     vec_mode="GENERATE", strides=None, lib=None):
    """{region name: (offset, bytes)} plus 'total'."""
    L, ds, o = _call(spec, extents, strides, lib, options(N, g, rounding, mode, vec_mode))
    regs = (CRegion * 8)()
    cnt, tot = C.c_int32(0), C.c_size_t(0)
    st = L.lib.imd_workspace_layout(ds[0].t, ds[1].t, ds[2].t, o, regs, 8, C.byref(cnt),
                                    C.byref(tot))
    if st:
        raise ImmerdinkError(st, "imd_workspace_layout")
    out = {REGIONS[r]: (regs[r].offset, regs[r].bytes) for r in range(8)}
    out["total"] = tot.value
    return out


def plan_bytes(spec, extents=None, *, N, g=0, rounding="RN", mode="EMULATE", vec_mode="GENERATE",
               strides=None, lib=None):
    """(device bytes, host bytes) a plan would own; raises the plan-time status."""
    L, ds, o = _call(spec, extents, strides, lib, options(N, g, rounding, mode, vec_mode))
    dv, hs = C.c_size_t(0), C.c_size_t(0)
    st = L.lib.imd_plan_bytes(ds[0].t, ds[1].t, ds[2].t, o, C.byref(dv), C.byref(hs))
    if st:
        raise ImmerdinkError(st, "imd_plan_bytes")
    return dv.value, hs.value


def lowering(spec, extents=None, *, N, g=0, rounding="RN", mode="EMULATE", vec_mode="GENERATE",
             strides=None, sm_count=0, packing=None, lib=None, check=True):
    """The lowering summary as a dict (status and dispatch as names)."""
    L, ds, o = _call(spec, extents, strides, lib, options(N, g, rounding, mode, vec_mode))
    out = CLowering()
    out.struct_size = C.sizeof(CLowering)
    out.sm_count = sm_count
    cp, keep = _packing(packing)
    if cp is not None:
        L.lib.imd_lowering_packed.argtypes = [C.POINTER(CTensor)] * 3 + [
            C.POINTER(COptions), C.POINTER(CPacking), C.POINTER(CLowering)]
        st = L.lib.imd_lowering_packed(ds[0].t, ds[1].t, ds[2].t, o, C.byref(cp), C.byref(out))
    else:
        st = L.lib.imd_lowering(ds[0].t, ds[1].t, ds[2].t, o, C.byref(out))
    if st and check:
        raise ImmerdinkError(st, "imd_lowering")
    d = {name: getattr(out, name) for name, _ in CLowering._fields_ if not name.startswith("reserved")}
    d["status"] = STATUS[out.status]
    d["dispatch"] = DISPATCH[out.dispatch]
    return d


def g_tradeoff(spec, extents=None, *, N, rounding="RN", mode="EMULATE", vec_mode="GENERATE",
               strides=None, lib=None):
    """Workspace bytes for every residue group size g = 1..N."""
    return {g: workspace_size(spec, extents, N=N, g=g, rounding=rounding, mode=mode,
                              vec_mode=vec_mode, strides=strides, lib=lib)
            for g in range(1, N + 1)}


def _err_request(metric, target, cond, norm_product, l1_ratio_a, l1_ratio_b, basis, fail_prob):
    return CErrRequest(C.sizeof(CErrRequest), ERR_METRICS[metric], float(target), float(cond),
                       float(norm_product), float(l1_ratio_a), float(l1_ratio_b), ERR_BASES[basis],
                       0, float(fail_prob))


def _err_dict(e):
    return dict(N=e.num_moduli, rounding="TRUNC" if e.rounding else "RN",
                dispatch=DISPATCH[e.dispatch], err_status=ERR_STATUS[e.err_status], k=e.k,
                outputs=e.outputs, bound=e.bound, typical=e.typical, unit_bound=e.unit_bound,
                unit_typical=e.unit_typical)


def err_estimate(*, N, k, outputs=1, rounding="RN", dispatch="EMULATE", metric="NORMWISE",
                 target=0.0, cond=1.0, norm_product=1.0, l1_ratio_a=0.0, l1_ratio_b=0.0,
                 basis="BOUND", fail_prob=0.0, lib=None):
    """Rigorous bound and typical estimate of |D - x| in the chosen metric."""
    L = lib or load()
    req = _err_request(metric, target, cond, norm_product, l1_ratio_a, l1_ratio_b, basis, fail_prob)
    out = CErr()
    out.struct_size = C.sizeof(CErr)
    st = L.lib.imd_err_estimate(N, ROUNDING[rounding], DISPATCH.index(dispatch), k, outputs,
                                C.byref(req), C.byref(out))
    if st:
        raise ImmerdinkError(st, "imd_err_estimate")
    return _err_dict(out)


def min_moduli(spec, extents=None, *, target, rounding="RN", mode="EMULATE", n_lo=0, n_hi=0,
               metric="NORMWISE", cond=1.0, norm_product=1.0, l1_ratio_a=0.0, l1_ratio_b=0.0,
               basis="BOUND", fail_prob=0.0, strides=None, lib=None):
    """Smallest N whose estimate meets `target`; raises NOT_SUPPORTED when none does."""
    L, ds, o = _call(spec, extents, strides, lib, options(2, 0, rounding, mode))
    req = _err_request(metric, target, cond, norm_product, l1_ratio_a, l1_ratio_b, basis, fail_prob)
    out = CErr()
    out.struct_size = C.sizeof(CErr)
    st = L.lib.imd_err_min_moduli(ds[0].t, ds[1].t, ds[2].t, o, n_lo, n_hi, C.byref(req),
                                  C.byref(out))
    if st:
        raise ImmerdinkError(st, "imd_err_min_moduli")
    return _err_dict(out)


# ------------------------------------------------------------------ performance model
PERF_REGIMES = {"DEFAULT": 0, "BURST": 1, "SUSTAINED": 2}
PERF_CACHES = {"COLD": 0, "WARM": 1, "REPEAT": 2, "CLEAN": 3}
PERF_ORDERS = {"TIME": 0, "TIES_BY_FOOTPRINT": 1}
_PERF_VEC = {"GENERATE": 1, "RESIDENT": 2}
_PERF_PACK = {"NONE": 1, "A": 2, "B": 4, "AB": 8}
PERF_CLASS_COUNT, PERF_PHASE_COUNT, PERF_KERNEL_COUNT, PERF_MAX_PARAMS = 12, 13, 90, 6


class CPerfKernel(C.Structure):
    _fields_ = [("resident", C.c_int32), ("regs", C.c_int32), ("smem_bytes", C.c_int32),
                ("threads", C.c_int32)]


class CPerfCalib(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("format", C.c_int32), ("sm_count", C.c_int32),
                ("reserved", C.c_int32), ("peak_dram_bytes_per_s", C.c_double),
                ("peak_int8_ops_per_s", C.c_double), ("peak_fp64_flops_per_s", C.c_double),
                ("l2_bytes", C.c_double), ("gpu", C.c_char * 64), ("date", C.c_char * 32),
                ("version", C.c_char * 64), ("clocks", C.c_char * 128), ("notes", C.c_char * 128),
                ("param", C.c_double * 96), ("kernel", CPerfKernel * 128),
                ("clock_eff_mhz", C.c_double), ("clock_min_mhz", C.c_double),
                ("power_cap_w", C.c_double), ("power_idle_w", C.c_double),
                ("energy_tc_pj", C.c_double), ("energy_alu_pj", C.c_double),
                ("energy_byte_pj", C.c_double), ("energy_gamma", C.c_double),
                ("warm_l2_bytes", C.c_double), ("warm_l2byte_ns", C.c_double),
                ("band_call", (C.c_double * 2) * 3), ("band_class", (C.c_double * 2) * 16),
                ("tie_ratio", C.c_double), ("energy_byte_f_pj", C.c_double),
                ("pack_l2_hit_bytes", C.c_double), ("clock_boost_mhz", C.c_double),
                ("power_act_w", C.c_double), ("power_act_gap_us", C.c_double),
                ("energy_dram_pj", C.c_double), ("warm_call_ns", C.c_double),
                ("warm_clean_byte_ns", C.c_double), ("pack_l2_planes", C.c_double)]


class CPerfCalibError(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("line", C.c_int32), ("reason", C.c_int32),
                ("reserved", C.c_int32), ("key", C.c_char * 64), ("message", C.c_char * 192)]


class CPerfRequest(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("flags", C.c_int32), ("k4_config", C.c_int32),
                ("reserved", C.c_int32), ("eps_fraction", C.c_double), ("regime", C.c_int32),
                ("cache", C.c_int32), ("clock_mhz", C.c_double), ("accuracy", C.POINTER(CErrRequest))]


class CPerfPhase(C.Structure):
    _fields_ = [("phase", C.c_int32), ("cls", C.c_int32), ("launches", C.c_int64),
                ("time_s", C.c_double), ("bytes", C.c_double), ("ops", C.c_double),
                ("bound_s", C.c_double), ("x", C.c_double * 6)]


class CPerf(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("status", C.c_int32), ("dispatch", C.c_int32),
                ("k4_config", C.c_int32), ("sm_count", C.c_int32), ("num_phases", C.c_int32),
                ("time_s", C.c_double), ("bound_s", C.c_double), ("flops_eq", C.c_double),
                ("tflops_eq", C.c_double), ("eps_s", C.c_double), ("eps_fraction", C.c_double),
                ("kernel_launches", C.c_int64), ("workspace_bytes", C.c_uint64),
                ("plan_device_bytes", C.c_uint64), ("pack_bytes", C.c_uint64),
                ("pack_ws_bytes", C.c_uint64), ("phase", CPerfPhase * 16), ("regime", C.c_int32),
                ("cache", C.c_int32), ("clock_mhz", C.c_double), ("power_w", C.c_double),
                ("warm_bytes", C.c_double), ("time_lo_s", C.c_double), ("time_hi_s", C.c_double),
                ("phase_lo_s", C.c_double * 16), ("phase_hi_s", C.c_double * 16),
                ("err_bound", C.c_double), ("err_typical", C.c_double), ("err_status", C.c_int32),
                ("err_metric", C.c_int32)]


class CRankRequest(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("candidate_size", C.c_uint32),
                ("num_moduli_count", C.c_int32), ("residue_group_count", C.c_int32),
                ("num_moduli", C.POINTER(C.c_int32)), ("residue_groups", C.POINTER(C.c_int32)),
                ("vec_modes", C.c_int32), ("pack_modes", C.c_int32), ("reuse", C.c_int32),
                ("flags", C.c_int32), ("budget_bytes", C.c_uint64), ("eps_fraction", C.c_double),
                ("regime", C.c_int32), ("cache", C.c_int32), ("order", C.c_int32),
                ("reserved", C.c_int32), ("clock_mhz", C.c_double),
                ("accuracy", C.POINTER(CErrRequest))]


class CCandidate(C.Structure):
    _fields_ = [("num_moduli", C.c_int32), ("residue_group", C.c_int32), ("vec_mode", C.c_int32),
                ("packed", C.c_int32), ("status", C.c_int32), ("feasible", C.c_int32),
                ("k4_config", C.c_int32), ("dispatch", C.c_int32), ("time_s", C.c_double),
                ("contract_s", C.c_double), ("pack_s", C.c_double), ("tflops_eq", C.c_double),
                ("eps_s", C.c_double), ("eps_fraction", C.c_double), ("workspace_bytes", C.c_uint64),
                ("plan_device_bytes", C.c_uint64), ("pack_bytes", C.c_uint64),
                ("pack_ws_bytes", C.c_uint64), ("total_bytes", C.c_uint64),
                ("kernel_launches", C.c_int64), ("time_lo_s", C.c_double), ("time_hi_s", C.c_double),
                ("clock_mhz", C.c_double), ("power_w", C.c_double), ("tie", C.c_int32),
                ("raw_rank", C.c_int32), ("err_bound", C.c_double), ("err_typical", C.c_double),
                ("err_status", C.c_int32), ("infeasible", C.c_int32)]


assert (C.sizeof(CPerfCalib), C.sizeof(CPerf), C.sizeof(CCandidate), C.sizeof(CRankRequest),
        C.sizeof(CPerfRequest), C.sizeof(CPerfCalibError)) == (3744, 1976, 192, 96, 48, 272)


class CalibrationError(ValueError):
    """A calibration text that does not parse: .line, .reason (name), .key."""

    def __init__(self, err):
        self.line, self.key = err.line, err.key.decode()
        self.reason = err.reason
        super().__init__(err.message.decode() or "calibration rejected")


def _names(fn, count):
    fn.restype = C.c_char_p
    return [fn(i).decode() for i in range(count)]


def phase_names(lib=None):
    return _names((lib or load()).lib.imd_perf_phase_name, PERF_PHASE_COUNT)


def class_names(lib=None):
    return _names((lib or load()).lib.imd_perf_class_name, PERF_CLASS_COUNT)


def kernel_names(lib=None):
    return _names((lib or load()).lib.imd_perf_kernel_name, PERF_KERNEL_COUNT)


def param_names(lib=None):
    """{class name: [parameter names by slot (None: unused)]}."""
    L = (lib or load()).lib
    L.imd_perf_param_name.restype = C.c_char_p
    L.imd_perf_param_name.argtypes = [C.c_int32, C.c_int32]
    out = {}
    for ci, cn in enumerate(class_names(lib)):
        out[cn] = [(lambda v: None if v is None else v.decode())(L.imd_perf_param_name(ci, j))
                   for j in range(PERF_MAX_PARAMS)]
    return out


def calib_default(lib=None):
    """The shipped calibration (B200) as a CPerfCalib struct."""
    L = (lib or load()).lib
    c, e = CPerfCalib(), CPerfCalibError()
    c.struct_size, e.struct_size = C.sizeof(CPerfCalib), C.sizeof(CPerfCalibError)
    L.imd_perf_calib_default_ex.argtypes = [C.POINTER(CPerfCalib), C.POINTER(CPerfCalibError)]
    if L.imd_perf_calib_default_ex(C.byref(c), C.byref(e)):
        raise CalibrationError(e)
    return c


def calib_parse(text, lib=None):
    """Calibration text -> CPerfCalib; CalibrationError with line, reason and key."""
    L = (lib or load()).lib
    raw = text.encode() if isinstance(text, str) else bytes(text)
    c, e = CPerfCalib(), CPerfCalibError()
    c.struct_size, e.struct_size = C.sizeof(CPerfCalib), C.sizeof(CPerfCalibError)
    L.imd_perf_calib_parse_ex.argtypes = [C.c_char_p, C.c_size_t, C.POINTER(CPerfCalib),
                                          C.POINTER(CPerfCalibError)]
    if L.imd_perf_calib_parse_ex(raw, len(raw), C.byref(c), C.byref(e)):
        raise CalibrationError(e)
    return c


def calib_load(path, lib=None):
    L = (lib or load()).lib
    c, e = CPerfCalib(), CPerfCalibError()
    c.struct_size, e.struct_size = C.sizeof(CPerfCalib), C.sizeof(CPerfCalibError)
    L.imd_perf_calib_load_ex.argtypes = [C.c_char_p, C.POINTER(CPerfCalib), C.POINTER(CPerfCalibError)]
    if L.imd_perf_calib_load_ex(os.fsencode(path), C.byref(c), C.byref(e)):
        raise CalibrationError(e)
    return c


def calib_format(calib=None, lib=None):
    """Canonical text of a calibration (None: the shipped one); parse(format(c)) == c."""
    L = (lib or load()).lib
    L.imd_perf_calib_format.argtypes = [C.POINTER(CPerfCalib), C.c_char_p, C.c_size_t,
                                        C.POINTER(C.c_size_t)]
    n = C.c_size_t(0)
    ptr = None if calib is None else C.byref(calib)
    st = L.imd_perf_calib_format(ptr, None, 0, C.byref(n))
    if st not in (0, 4):
        raise ImmerdinkError(st, "imd_perf_calib_format")
    buf = C.create_string_buffer(n.value + 1)
    st = L.imd_perf_calib_format(ptr, buf, n.value + 1, C.byref(n))
    if st:
        raise ImmerdinkError(st, "imd_perf_calib_format")
    return buf.value.decode()


def _perf_dict(r, lib):
    ph, cl = phase_names(lib), class_names(lib)
    phases = [dict(phase=ph[p.phase], cls=cl[p.cls], launches=p.launches, time_s=p.time_s,
                   bytes=p.bytes, ops=p.ops, bound_s=p.bound_s, x=list(p.x),
                   lo_s=r.phase_lo_s[i], hi_s=r.phase_hi_s[i])
              for i, p in enumerate(r.phase[:r.num_phases])]
    return dict(status=STATUS[r.status], dispatch=DISPATCH[r.dispatch], sm_count=r.sm_count,
                time_s=r.time_s, time_lo_s=r.time_lo_s, time_hi_s=r.time_hi_s, bound_s=r.bound_s,
                flops_eq=r.flops_eq, tflops_eq=r.tflops_eq, kernel_launches=r.kernel_launches,
                workspace_bytes=r.workspace_bytes, plan_device_bytes=r.plan_device_bytes,
                pack_bytes=r.pack_bytes, pack_ws_bytes=r.pack_ws_bytes, phases=phases,
                regime=r.regime, cache=r.cache, clock_mhz=r.clock_mhz, power_w=r.power_w,
                err_bound=r.err_bound, err_typical=r.err_typical,
                err_status=ERR_STATUS[r.err_status])


def _perf_request(beta, alpha_zero, regime, cache, clock_mhz, accuracy):
    flags = (1 if beta else 0) | (2 if alpha_zero else 0)
    acc = None if accuracy is None else C.pointer(accuracy)
    return CPerfRequest(C.sizeof(CPerfRequest), flags, -1, 0, -1.0, PERF_REGIMES[regime],
                        PERF_CACHES[cache], float(clock_mhz), acc)


def predict(spec, extents=None, *, N, g=0, rounding="RN", mode="EMULATE", vec_mode="GENERATE",
            strides=None, packing=None, beta=False, alpha_zero=False, regime="DEFAULT",
            cache="COLD", clock_mhz=0.0, accuracy=None, calib=None, lib=None):
    """imd_perf_predict: predicted time of one imd_contract per phase and in total, as a dict. A
    plan-time status comes back in ["status"]; a bad argument raises. packing = (PackSpec or None,
    PackSpec or None); accuracy: a CErrRequest; calib: a CPerfCalib (None: the shipped one)."""
    L, ds, o = _call(spec, extents, strides, lib, options(N, g, rounding, mode, vec_mode))
    cp, keep = _packing(packing)
    req = _perf_request(beta, alpha_zero, regime, cache, clock_mhz, accuracy)
    r = CPerf()
    r.struct_size = C.sizeof(CPerf)
    L.lib.imd_perf_predict.argtypes = [C.POINTER(CTensor)] * 3 + [
        C.POINTER(COptions), C.POINTER(CPacking), C.POINTER(CPerfRequest), C.POINTER(CPerfCalib),
        C.POINTER(CPerf)]
    st = L.lib.imd_perf_predict(ds[0].t, ds[1].t, ds[2].t, o, None if cp is None else C.byref(cp),
                                C.byref(req), None if calib is None else C.byref(calib), C.byref(r))
    if st and r.status == 0:
        raise ImmerdinkError(st, "imd_perf_predict")
    return _perf_dict(r, L)


def predict_pack(pack, *, regime="DEFAULT", cache="COLD", clock_mhz=0.0, calib=None, lib=None):
    """imd_perf_predict_pack: predicted time of one imd_pack of a PackSpec."""
    L = lib or load()
    cs = CPackSpec(pack)
    req = _perf_request(False, False, regime, cache, clock_mhz, None)
    r = CPerf()
    r.struct_size = C.sizeof(CPerf)
    L.lib.imd_perf_predict_pack.argtypes = [C.POINTER(CPackDesc), C.POINTER(CPerfRequest),
                                            C.POINTER(CPerfCalib), C.POINTER(CPerf)]
    st = L.lib.imd_perf_predict_pack(C.byref(cs.d), C.byref(req),
                                     None if calib is None else C.byref(calib), C.byref(r))
    if st and r.status == 0:
        raise ImmerdinkError(st, "imd_perf_predict_pack")
    return _perf_dict(r, L)


def rank(spec, extents=None, *, N, g=None, vec_modes=("GENERATE",), packs=("NONE",), reuse=1,
         budget=0, beta=False, rounding="RN", mode="EMULATE", strides=None, order="TIME",
         regime="DEFAULT", cache="COLD", clock_mhz=0.0, accuracy=None, calib=None, lib=None):
    """imd_perf_rank: the candidates N x g x vec mode x packs ranked by predicted time inside a
    device-memory budget (bytes; 0 = none), as a list of dicts. N: an int or a list; g: None
    (every g in 1..N) or a list; packs: any of "NONE", "A", "B", "AB"."""
    Ns = [int(N)] if hasattr(N, "__index__") else [int(x) for x in N]
    gs = [] if g is None else ([int(g)] if isinstance(g, int) else [int(x) for x in g])
    L, ds, o = _call(spec, extents, strides, lib, options(Ns[0], 0, rounding, mode, "GENERATE"))
    narr = (C.c_int32 * max(len(Ns), 1))(*Ns)
    garr = (C.c_int32 * max(len(gs), 1))(*gs)
    req = CRankRequest(C.sizeof(CRankRequest), C.sizeof(CCandidate), len(Ns), len(gs),
                       C.cast(narr, C.POINTER(C.c_int32)),
                       C.cast(garr, C.POINTER(C.c_int32)) if gs else None,
                       sum(_PERF_VEC[v] for v in set(vec_modes)),
                       sum(_PERF_PACK[p] for p in set(packs)), int(reuse), 1 if beta else 0,
                       int(budget), -1.0, PERF_REGIMES[regime], PERF_CACHES[cache],
                       PERF_ORDERS[order], 0, float(clock_mhz),
                       None if accuracy is None else C.pointer(accuracy))
    L.lib.imd_perf_rank.argtypes = [C.POINTER(CTensor)] * 3 + [
        C.POINTER(COptions), C.POINTER(CRankRequest), C.POINTER(CPerfCalib), C.POINTER(CCandidate),
        C.c_int32, C.POINTER(C.c_int32)]
    cal = None if calib is None else C.byref(calib)
    count = C.c_int32(0)
    st = L.lib.imd_perf_rank(ds[0].t, ds[1].t, ds[2].t, o, C.byref(req), cal, None, 0, C.byref(count))
    if st:
        raise ImmerdinkError(st, "imd_perf_rank")
    out = (CCandidate * max(count.value, 1))()
    st = L.lib.imd_perf_rank(ds[0].t, ds[1].t, ds[2].t, o, C.byref(req), cal, out, count.value,
                             C.byref(count))
    if st:
        raise ImmerdinkError(st, "imd_perf_rank")
    vec_name = {v: k for k, v in VEC.items()}
    return [dict(N=c.num_moduli, g=c.residue_group, vec_mode=vec_name[c.vec_mode],
                 packs=["NONE", "A", "B", "AB"][c.packed], status=STATUS[c.status],
                 feasible=bool(c.feasible), infeasible=c.infeasible, dispatch=DISPATCH[c.dispatch],
                 time_s=c.time_s, contract_s=c.contract_s, pack_s=c.pack_s, tflops_eq=c.tflops_eq,
                 workspace_bytes=c.workspace_bytes, plan_device_bytes=c.plan_device_bytes,
                 pack_bytes=c.pack_bytes, pack_ws_bytes=c.pack_ws_bytes, total_bytes=c.total_bytes,
                 kernel_launches=c.kernel_launches, time_lo_s=c.time_lo_s, time_hi_s=c.time_hi_s,
                 tie=bool(c.tie), raw_rank=c.raw_rank, err_bound=c.err_bound,
                 err_typical=c.err_typical, err_status=ERR_STATUS[c.err_status])
            for c in out[:count.value]]
