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
