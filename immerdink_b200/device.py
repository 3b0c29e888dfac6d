"""Device API: plans and einsum-style contractions on caller-owned float64 CUDA arrays.

Mirrors the reference front end (python/immerdink/device.py: `Plan` :511-728, `PlanCache`
:744-809, `contract` :819-868, `workspace_size` :871-): same names, arguments, exception types
and ownership rules. Nothing here allocates device memory, copies data or synchronises: a call
checks the arrays' layouts on the host and enqueues imd_contract on the caller's stream, so it
can be captured in a CUDA graph. The caller owns operands, output and workspace."""
import ctypes as ct
import threading
import weakref
from collections import namedtuple

from . import _arrays, _capi, host
from ._arrays import (DeviceArray, get_cai_stream_policy, set_cai_stream_policy,  # noqa: F401
                      stream_handle)


class ImmerdinkError(RuntimeError):
    """A non-SUCCESS imd_status_t; `.status` is its name."""
    status = "UNKNOWN"


class InvalidValueError(ImmerdinkError, ValueError):
    status = "INVALID_VALUE"


class NotSupportedError(ImmerdinkError):
    status = "NOT_SUPPORTED"


class AliasingError(ImmerdinkError, ValueError):
    status = "ALIASING"


class InsufficientWorkspaceError(ImmerdinkError, ValueError):
    status = "INSUFFICIENT_WORKSPACE"


class MisalignedError(ImmerdinkError, ValueError):
    status = "MISALIGNED"


class CudaError(ImmerdinkError):
    status = "CUDA_ERROR"


class AllocFailedError(ImmerdinkError, MemoryError):
    status = "ALLOC_FAILED"


class PackMismatchError(ImmerdinkError, ValueError):
    status = "PACK_MISMATCH"


_BY_STATUS = {1: InvalidValueError, 2: NotSupportedError, 3: AliasingError,
              4: InsufficientWorkspaceError, 5: MisalignedError, 6: CudaError,
              7: AllocFailedError, 8: PackMismatchError}


def _error(st, what, extra=""):
    cls = _BY_STATUS.get(st, ImmerdinkError)
    return cls(f"{what}: IMD_STATUS_{cls.status}{extra}")


def load_library(path=None):
    return path if isinstance(path, _capi.Library) else _capi.load(path)


def wait_flags(flags, expect, *, max_polls=0, stream=0, lib=None):
    """imd_wait_flags: enqueue a bounded wait on `stream` until every 32-bit word at the device
    addresses `flags` (at most 32) holds `expect`. A wait that runs out (max_polls polls per flag;
    0 = about a second) sets bit 2 of the device error word instead of blocking the stream."""
    lib = load_library(lib)
    arr = (ct.c_void_p * max(len(flags), 1))(*[int(f) for f in flags])
    st = lib.lib.imd_wait_flags(arr, len(flags), int(expect), int(max_polls), stream)
    if st:
        raise _error(st, "imd_wait_flags")


def push_ranges(copies, flags, value, *, ctas=0, stream=0, lib=None):
    """imd_push_ranges: enqueue one small copy kernel that performs `copies` = [(dst, src, nbytes),
    ...] (device addresses, 16-byte granular; destinations may be peers' memory) and then stores
    `value` into the 32-bit words at the addresses `flags`."""
    lib = load_library(lib)
    nc, nf = len(copies), len(flags)
    dst = (ct.c_void_p * max(nc, 1))(*[int(c[0]) for c in copies])
    src = (ct.c_void_p * max(nc, 1))(*[int(c[1]) for c in copies])
    nb = (ct.c_int64 * max(nc, 1))(*[int(c[2]) for c in copies])
    fl = (ct.c_void_p * max(nf, 1))(*[int(f) for f in flags])
    st = lib.lib.imd_push_ranges(dst, src, nb, nc, fl, nf, int(value), int(ctas), stream)
    if st:
        raise _error(st, "imd_push_ranges")


def copy_if_flagged(flag_ranges, copies, *, stream=0, lib=None):
    """imd_copy_if_flagged: enqueue one kernel that performs `copies` = [(dst, src, nbytes), ...]
    (device addresses, 8-byte granular) only if a byte of `flag_ranges` = [(ptr, nbytes), ...] is
    nonzero."""
    lib = load_library(lib)
    nr, nc = len(flag_ranges), len(copies)
    fp = (ct.c_void_p * max(nr, 1))(*[int(p) for p, _ in flag_ranges])
    fb = (ct.c_int64 * max(nr, 1))(*[int(n) for _, n in flag_ranges])
    dst = (ct.c_void_p * max(nc, 1))(*[int(c[0]) for c in copies])
    src = (ct.c_void_p * max(nc, 1))(*[int(c[1]) for c in copies])
    nb = (ct.c_int64 * max(nc, 1))(*[int(c[2]) for c in copies])
    st = lib.lib.imd_copy_if_flagged(fp, fb, nr, dst, src, nb, nc, stream)
    if st:
        raise _error(st, "imd_copy_if_flagged")


class Layout(namedtuple("Layout", "shape strides")):
    """Extents and ELEMENT strides of an operand (None = dense), to plan before arrays exist."""

    def __new__(cls, shape, strides=None):
        shape = tuple(int(e) for e in shape)
        strides = host.dense_strides(shape) if strides is None else tuple(int(s) for s in strides)
        if len(strides) != len(shape):
            raise ValueError("one stride per mode")
        return super().__new__(cls, shape, strides)


def _layout_of_view(v, what):
    _, shape, bstrides, f8, _, _ = v
    if not f8:
        raise TypeError(f"{what}: dtype must be float64")
    shape = tuple(int(e) for e in shape)
    if bstrides is None:
        return Layout(shape)
    if any(s % 8 for s in bstrides):
        raise TypeError(f"{what}: byte strides must be multiples of 8")
    return Layout(shape, tuple(s // 8 for s in bstrides))


def _layout(x, what):
    return x if isinstance(x, Layout) else _layout_of_view(_arrays.view(x), what)


def _descs(spec, layouts):
    labels = host.parse_spec(spec)
    out = []
    for name, lab, lay in zip("ABC", labels, layouts):
        if len(lab) != len(lay.shape):
            raise ValueError(f"{name}: {len(lab)} labels in the spec, rank {len(lay.shape)} array")
        out.append(host.Desc(lay.shape, lay.strides, tuple(ord(c) for c in lab)))
    return tuple(out)


class _Expected:
    """Shape and strides one operand of a plan must have at call time (modes of extent <= 1
    are free: the lowering drops them)."""

    def __init__(self, desc, what):
        self.shape, self.strides, self.what = tuple(desc.extent), tuple(desc.stride), what

    def check(self, shape, bstrides):
        shape = tuple(int(e) for e in shape)
        if shape != self.shape:
            raise ValueError(f"{self.what}: shape {shape} != the plan's {self.shape}")
        if 0 in shape:
            return
        got = host.dense_strides(shape) if bstrides is None else tuple(s / 8 for s in bstrides)
        if any(e > 1 and s != w for e, s, w in zip(shape, got, self.strides)):
            raise ValueError(f"{self.what}: strides {got} (elements) != the plan's {self.strides}")


def _pointer(x, expected, stream, out=False, device=None):
    ptr, shape, bstrides, f8, readonly, _ = _arrays.view(x, stream, device)
    if not f8:
        raise TypeError(f"{expected.what}: dtype must be float64")
    if out and readonly:
        raise ValueError(f"{expected.what} is read-only")
    expected.check(shape, bstrides)
    return ptr


class Handle:
    """A library handle (imd_create) bound to the device that is current when it is made. It is
    released by close() or when the object is collected, whichever comes first."""

    def __init__(self, lib=None):
        library = load_library(lib)
        raw = ct.c_void_p()
        status = library.lib.imd_create(ct.byref(raw))
        if status != 0:
            raise _error(status, "imd_create")
        self.lib, self.device, self._h = library, library.current_device(), raw.value
        self._fin = weakref.finalize(self, library.lib.imd_destroy, raw.value)

    def close(self):
        if self._h is not None:
            self._h = None
            self._fin()


_handles, _handles_lock = {}, threading.Lock()


def default_handle(lib=None):
    lib = load_library(lib)
    key = (id(lib), lib.current_device())
    with _handles_lock:
        if key not in _handles:
            _handles[key] = Handle(lib)
        return _handles[key]


def pack_spec(spec, A, B, C, *, operand, N, g=0, rounding="RN", mode="EMULATE",
              vec_mode="GENERATE", lib=None):
    """imd_pack_desc_for: the GIVEN host.PackSpec of operand 0 (A) or 1 (B) with the classes and
    orders the unpacked plan uses (a pack of it reproduces that contraction bit for bit).
    A, B, C: arrays or Layouts. (ref: python/immerdink/device.py:289-296)"""
    descs = _descs(spec, [_layout(x, n) for x, n in zip((A, B, C), "ABC")])
    return host.pack_desc_for(descs, operand=operand, N=N, g=g, rounding=rounding, mode=mode,
                              vec_mode=vec_mode, lib=load_library(lib).host)


class PackRecord(namedtuple("PackRecord", "N rounding pack_bytes key_digest")):
    """What a PackedBuffer remembers: N, rounding, pack_bytes and the key digest of a pack."""
    __slots__ = ()


class Pack:
    """imd_pack_create of a host.PackSpec: an immutable host object (key and layout).
    `.pack(X, out)` writes the packed operand into caller-owned device memory of `pack_bytes`
    bytes. (ref: python/immerdink/device.py:299-413)"""

    def __init__(self, spec, *, handle=None, lib=None):
        self.lib = load_library(lib if handle is None else handle.lib)
        self.handle = handle or default_handle(self.lib)
        self.spec = spec
        self._cd = host.CPackSpec(spec)
        h = ct.c_void_p()
        L = self.lib.lib
        st = L.imd_pack_create(self.handle._h, ct.byref(self._cd.d), ct.byref(h))
        if st:
            raise _error(st, "imd_pack_create")
        self._h = h.value
        self._fin = weakref.finalize(self, L.imd_pack_destroy, h.value)
        pb, wb = ct.c_size_t(0), ct.c_size_t(0)
        st = L.imd_pack_bytes(self._h, ct.byref(pb), ct.byref(wb))
        if st:
            raise _error(st, "imd_pack_bytes")
        self.pack_bytes, self.workspace_bytes = pb.value, wb.value
        self._x = _Expected(spec.tensor, "X")
        self._fn = L.imd_pack
        self._layout = self._rec = None
        self._lock = threading.Lock()
        self._users = 0      # open plans made with this pack: they keep passing its handle
        self.closed = False

    # A pack is destroyed (imd_pack_destroy) once it has been closed AND no open plan still
    # passes its handle; `_users` counts those plans.
    def _destroy_if_unused(self, unused):
        if unused and self._h is not None:
            self._h = None
            self._fin()

    def _acquire(self):
        """A plan starts using this pack."""
        with self._lock:
            if self.closed:
                raise ValueError(f"{self!r} is closed")
            self._users += 1

    def _release(self):
        """A plan made with this pack was closed or collected."""
        with self._lock:
            self._users -= 1
            unused = self.closed and self._users == 0
        self._destroy_if_unused(unused)

    @property
    def layout(self):
        """imd_pack_layout of the spec: regions and sizes of the packed buffer (a dict)."""
        if self._layout is None:
            self._layout = host.pack_layout(self.spec, lib=self.lib.host)
        return self._layout

    @property
    def record(self):
        if self._rec is None:
            self._rec = PackRecord(int(self.spec.N), self.spec.rounding, self.pack_bytes,
                                   self.layout["key_digest"])
        return self._rec

    def pack(self, X, out, *, workspace=None, stream=None):
        """imd_pack: X (float64, the spec's layout) -> `out` (>= pack_bytes, 256-byte aligned) on
        `stream`; `workspace` >= workspace_bytes. A PackedBuffer `out` records this pack.
        Returns out."""
        if self.closed:
            raise ValueError(f"{self!r} is closed")
        s = 0 if stream is None else stream_handle(stream)
        dev = self.handle.device
        px = _pointer(X, self._x, s, device=dev)
        pw, nw = _arrays.buffer(workspace, "workspace", stream=s, device=dev)
        if isinstance(out, PackedBuffer):
            po, no = out._resolve("packed buffer", True, s, dev)
            with out._lock:   # the record follows host enqueue order
                st = self._fn(self._h, px, po, no, pw, nw, s)
                if st == 0:
                    out._last = self.record
                elif st == 6:  # the launches may have run in part
                    out._last = None
        else:
            po, no = _arrays.buffer(out, "packed buffer", stream=s, device=dev)
            st = self._fn(self._h, px, po, no, pw, nw, s)
        if st:
            raise _error(st, "imd_pack", f" (pack {self.pack_bytes} bytes, workspace "
                                         f"{self.workspace_bytes} bytes needed; given {no}, {nw})")
        return out

    def scatter_ptr(self, X, slab_rows, row_offset, dests, dest_bytes, ws, ws_bytes, stream=0):
        """imd_pack_scatter with raw integers: this pack describes a PIECE of a slab; its rows go to
        rows [row_offset, row_offset + r) of every packed buffer in `dests` (pointers; dests[0] the
        caller's own), each laid out for a slab of `slab_rows` rows per batch."""
        if self.closed:
            raise ValueError(f"{self!r} is closed")
        arr = (ct.c_void_p * len(dests))(*[int(d) for d in dests])
        st = self.lib.lib.imd_pack_scatter(self._h, X, int(slab_rows), int(row_offset), len(dests), arr,
                                           int(dest_bytes), ws, int(ws_bytes), stream)
        if st:
            raise _error(st, "imd_pack_scatter")

    def pack_ptr(self, X, packed, packed_bytes, ws, ws_bytes, stream=0):
        """imd_pack on raw addresses: nothing is checked on the Python side and no PackedBuffer
        record is left; the C entry point's own checks still apply."""
        if self.closed:
            raise ValueError(f"{self!r} is closed")
        status = self._fn(self._h, X, packed, packed_bytes, ws, ws_bytes, stream)
        if status != 0:
            raise _error(status, "imd_pack")

    def close(self):
        """No new use from now on; the handle itself lives until the last plan made with this pack
        is closed or collected (such plans pass the handle at every call)."""
        with self._lock:
            self.closed = True
            unused = self._users == 0
        self._destroy_if_unused(unused)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.close()

    def __repr__(self):
        return (f"<immerdink_b200.Pack {self.pack_bytes} bytes, workspace {self.workspace_bytes}"
                f"{', closed' if self.closed else ''}>")


class PackedBuffer:
    """Caller-owned device memory for one packed operand, together with a host-side note of which
    pack Pack.pack last enqueued into it. A packed plan checks that note against its slot before
    every call and refuses (PackMismatchError) a buffer that was never packed or that holds a
    different pack. The note is written in host order at enqueue time, so it protects the usual
    single-stream use, not arbitrary multi-stream orderings.

    `buf` is a contiguous CUDA array, a (pointer, nbytes) pair, or a bare integer pointer with
    `nbytes`. Interface as in the reference's python/immerdink/device.py:422-495."""

    __slots__ = ("buf", "nbytes", "_last", "_lock")

    def __init__(self, buf, nbytes=None):
        if isinstance(buf, PackedBuffer):
            raise TypeError("wrap the underlying buffer, not another PackedBuffer")
        if buf is None:
            raise ValueError("a PackedBuffer wraps existing device memory; got None")
        size = None if nbytes is None else int(nbytes)
        if isinstance(buf, int):
            if size is None:
                raise ValueError("an integer pointer carries no size: pass nbytes as well")
            buf = (buf, size)
        self.buf, self.nbytes = buf, size
        self._last, self._lock = None, threading.Lock()

    @property
    def last_pack(self):
        """The PackRecord of the pack last written here by Pack.pack, or None."""
        return self._last

    def _resolve(self, what, writable, stream, device):
        """(pointer, usable bytes) of the wrapped memory; `nbytes`, when given, caps the size."""
        ptr, have = _arrays.buffer(self.buf, what, writable, stream, device)
        if self.nbytes is None:
            return ptr, have
        if have < self.nbytes:
            raise ValueError(f"{what}: declared {self.nbytes} bytes but the buffer has only {have}")
        return ptr, self.nbytes

    def _expect(self, rec, what):
        """Raises PackMismatchError unless the noted pack equals `rec` (the plan slot's record)."""
        with self._lock:
            seen = self._last
        if seen == rec:
            return
        if seen is None:
            why = "no pack recorded: only Pack.pack(X, this_buffer) leaves the record a plan looks for"
        elif seen.N != rec.N:
            why = f"holds a pack made with N={seen.N}, plan expects N={rec.N}"
        elif seen.rounding != rec.rounding:
            why = f"holds a pack made with rounding {seen.rounding}, plan expects {rec.rounding}"
        else:
            why = (f"holds the pack with key digest {seen.key_digest:#x} ({seen.pack_bytes} bytes), "
                   f"plan expects key digest {rec.key_digest:#x}")
        raise PackMismatchError(f"{what}: {why}")

    def __repr__(self):
        seen = self._last
        state = "empty" if seen is None else f"N={seen.N} {seen.rounding} pack of {seen.pack_bytes} bytes"
        return f"<immerdink_b200.PackedBuffer {state}>"


def _pack_specs(packs):
    """The two slots of a plan as host PackSpecs: each entry of `packs` may be a Pack, a PackSpec
    or None; None (or a pair of Nones) means a plan without packed slots."""
    if packs is None:
        return None
    slots = tuple(packs)
    if len(slots) != 2:
        raise ValueError("packs must have two entries: (for A, for B), each a Pack, PackSpec or None")
    specs = tuple(getattr(entry, "spec", entry) if isinstance(entry, Pack) else entry for entry in slots)
    return specs if any(sp is not None for sp in specs) else None


def _finalize_plan(destroy, h, packs):
    destroy(h)
    for pk in packs:
        pk._release()


class Plan:
    """imd_plan_create for fixed operand layouts (arrays or `Layout`s). Immutable; any number
    of threads may call `contract` at once, each with its own workspace. Footprints:
    `workspace_bytes` (per in-flight call, caller-owned), `device_bytes` (plan-owned)."""

    def __init__(self, spec, A, B, C, *, N, g=0, rounding="RN", mode="EMULATE",
                 vec_mode="GENERATE", k4_tune=False, packs=None, handle=None, lib=None):
        lays = [_layout(x, n) for x, n in zip((A, B, C), "ABC")]
        self.spec = spec
        self._create(_descs(spec, lays), N, g, rounding, mode, vec_mode, k4_tune, packs, handle, lib)

    @classmethod
    def from_descs(cls, A, B, C, *, N, g=0, rounding="RN", mode="EMULATE", vec_mode="GENERATE",
                   k4_tune=False, packs=None, handle=None, lib=None):
        self = cls.__new__(cls)
        self.spec = None
        descs = tuple(d if isinstance(d, host.Desc) else host.Desc(*d) for d in (A, B, C))
        self._create(descs, N, g, rounding, mode, vec_mode, k4_tune, packs, handle, lib)
        return self

    def _create(self, descs, N, g, rounding, mode, vec_mode, k4_tune, packs, handle, lib):
        self._h = None
        self.lib = load_library(lib if handle is None else handle.lib)
        self.packs = (None, None) if packs is None else tuple(packs)
        if len(self.packs) != 2 or any(p is not None and not isinstance(p, Pack) for p in self.packs):
            raise TypeError("packs = (Pack or None, Pack or None)")
        self._packed = self.packs != (None, None)
        self.handle = handle or default_handle(self.lib)
        self.device = self.handle.device
        self.descs = descs
        self.options = dict(N=int(N), g=int(g), rounding=rounding, mode=mode, vec_mode=vec_mode,
                            k4_tune=bool(k4_tune))
        self._opt = host.options(N, g, rounding, mode, vec_mode, 1 if k4_tune else 0)
        self._cd = [host.CDesc(d) for d in descs]
        h = ct.c_void_p()
        L = self.lib.lib
        held = []   # packs this plan has started to use: given back if creation fails
        try:
            for pk in filter(None, self.packs):
                pk._acquire()
                held.append(pk)
            if self._packed:
                hp = [None if p is None else p._h for p in self.packs]
                st = L.imd_plan_create_packed(self.handle._h, self._cd[0].t, self._cd[1].t,
                                              self._cd[2].t, self._opt, hp[0], hp[1], ct.byref(h))
            else:
                st = L.imd_plan_create(self.handle._h, self._cd[0].t, self._cd[1].t, self._cd[2].t,
                                       self._opt, ct.byref(h))
            if st != 0:
                failure = _error(st, "imd_plan_create_packed" if self._packed else "imd_plan_create")
                if isinstance(failure, PackMismatchError):   # say which part of the key differs
                    failure.reason = host.PACK_MISMATCH[self._lowering(check=False)["pack_mismatch"]]
                    failure.args = (f"{failure.args[0]} ({failure.reason})",)
                raise failure
        except BaseException:
            while held:
                held.pop()._release()
            raise
        self._h = h.value
        self._fin = weakref.finalize(self, _finalize_plan, L.imd_plan_destroy, h.value, tuple(held))
        self.workspace_bytes = host.workspace_size(descs, N=N, g=g, rounding=rounding, mode=mode,
                                                   vec_mode=vec_mode, packing=_pack_specs(self.packs),
                                                   lib=self.lib.host)
        nb = ct.c_size_t(0)
        L.imd_plan_device_bytes(self._h, ct.byref(nb))
        self.device_bytes = nb.value
        self._ex = [_Expected(d, n) for d, n in zip(descs, "ABC")]
        self._fn = L.imd_contract_packed if self._packed else L.imd_contract
        self._lw = None

    def _lowering(self, sm_count=0, check=True):
        o = self.options
        return host.lowering(self.descs, N=o["N"], g=o["g"], rounding=o["rounding"],
                             mode=o["mode"], vec_mode=o["vec_mode"], sm_count=sm_count,
                             packing=_pack_specs(self.packs), lib=self.lib.host, check=check)

    @property
    def lowering(self):
        if self._lw is None:
            self._lw = self._lowering(self.lib.sm_count(self.device))
        return self._lw

    def pack_spec(self, operand):
        """The pack spec (imd_pack_desc_for) under which operand 0 (A) or 1 (B) of THIS plan would
        be packed: its descriptors with this plan's N, g, rounding, mode and vector mode."""
        keep = ("N", "g", "rounding", "mode", "vec_mode")
        return host.pack_desc_for(self.descs, operand=operand, lib=self.lib.host,
                                  **{name: self.options[name] for name in keep})

    @property
    def host_bytes(self):
        return self.lowering["plan_host_bytes"]

    def contract(self, A, B, C, *, alpha=1.0, beta=0.0, workspace=None, stream=None, packed=None,
                 part=0):
        """C <- alpha A.B + beta C on `stream`. Arrays must have the plan's shapes and strides;
        workspace >= workspace_bytes, 256-byte aligned, one in-flight call per workspace.
        part (packed plans, an extension): 0 the whole call; 1 all outputs but those of the native
        path (A and B are not read); 2 only those (imd_contract_packed_part). Returns C."""
        if self._h is None:
            raise ValueError("plan is closed")
        s = 0 if stream is None else stream_handle(stream)
        dev = self.device
        pa = _pointer(A, self._ex[0], s, device=dev)
        pb = _pointer(B, self._ex[1], s, device=dev)
        pc = _pointer(C, self._ex[2], s, True, dev)
        pw, nw = (None, 0) if workspace is None else _arrays.buffer(workspace, "workspace",
                                                                    stream=s, device=dev)
        if self._packed:
            ops = self._operands(pa, pb, packed, s)
            if part:
                st = self.lib.lib.imd_contract_packed_part(self._h, alpha, *ops, beta, pc, pw, nw, s,
                                                           int(part))
            else:
                st = self._fn(self._h, alpha, *ops, beta, pc, pw, nw, s)
        else:
            if packed is not None and any(x is not None for x in packed):
                raise ValueError("packed buffers given to a plan without packs")
            if part:
                raise ValueError("parts are defined for plans with packs")
            st = self._fn(self._h, alpha, pa, pb, beta, pc, pw, nw, s)
        if st:
            raise self._fail(st, nw)
        return C

    def _operands(self, pa, pb, packed, s):
        """The two imd_operand_t of a packed call: FP64 pointer plus, for a packed slot, the
        packed memory (pointer, size) and the pack handle that names its layout."""
        given = (None, None) if packed is None else tuple(packed)
        if len(given) != 2:
            raise ValueError("packed must have two entries: (buffer of A or None, buffer of B or None)")
        records = []
        for slot, fp64_ptr in enumerate((pa, pb)):
            pack, buf, name = self.packs[slot], given[slot], f"packed[{slot}]"
            if pack is None:
                if buf is not None:
                    raise ValueError(f"{name} given for an in-line operand")
                records.append(_capi.Operand(fp64_ptr, None, 0, None))
            elif isinstance(buf, PackedBuffer):
                buf._expect(pack.record, name)
                ptr, size = buf._resolve(name, False, s, self.device)
                records.append(_capi.Operand(fp64_ptr, ptr, size, pack._h))
            else:
                raw = buf is None or isinstance(buf, tuple)   # (pointer, size) pairs need no stream check
                ptr, size = _arrays.buffer(buf, name) if raw else _arrays.buffer(buf, name, False, s, self.device)
                records.append(_capi.Operand(fp64_ptr, ptr, size, pack._h))
        return ct.byref(records[0]), ct.byref(records[1])

    def contract_ptr(self, alpha, A, B, beta, C, ws, ws_bytes, stream=0, packed=None, part=0):
        """The C entry point on raw addresses (integers; `stream` a CUDA stream handle): no layout
        or dtype check happens here, only those of the C side. For a packed plan, `packed` holds
        one (pointer, nbytes) pair or None per operand and `part` selects a part of the call
        (see contract())."""
        if not self._packed:
            status = self._fn(self._h, alpha, A, B, beta, C, ws, ws_bytes, stream)
        else:
            op_a, op_b = self._operands(A, B, packed, stream)
            if part:
                status = self.lib.lib.imd_contract_packed_part(self._h, alpha, op_a, op_b, beta, C, ws,
                                                               ws_bytes, stream, int(part))
            else:
                status = self._fn(self._h, alpha, op_a, op_b, beta, C, ws, ws_bytes, stream)
        if status != 0:
            raise self._fail(status, ws_bytes)

    def _fail(self, st, nw):
        extra = ""
        if st in (1, 4) and nw < self.workspace_bytes:
            extra = f" (workspace of {nw} bytes; the plan needs {self.workspace_bytes})"
        return _error(st, "imd_contract" + ("_packed" if self._packed else ""), extra)

    def close(self):
        self._h = None
        if hasattr(self, "_fin"):
            self._fin()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.close()

    def __repr__(self):
        state = "closed" if self._h is None else f"workspace {self.workspace_bytes} bytes"
        return f"<immerdink_b200.Plan {self.spec or self.descs!r} N={self.options['N']} {state}>"


class PlanCache:
    """Plans keyed by (spec, layouts, options, device). Thread-safe; never evicts.
    `freeze()`: a miss raises KeyError (assert that every plan exists before a capture)."""

    def __init__(self):
        self._plans, self._lock, self.frozen = {}, threading.Lock(), False

    def plans(self):
        return list({id(p): p for p in list(self._plans.values())}.values())

    def __len__(self):
        return len(self.plans())

    @property
    def device_bytes(self):
        return sum(p.device_bytes for p in self.plans())

    def freeze(self, frozen=True):
        self.frozen = bool(frozen)

    def _get(self, key, make):
        p = self._plans.get(key)
        if p is None:
            if self.frozen:
                raise KeyError(f"PlanCache is frozen and holds no plan for {key[0]!r}")
            new = make()
            with self._lock:
                p = self._plans.setdefault(key, new)
            if p is not new:
                new.close()
        return p

    def get(self, spec, A, B, C, *, N, g=0, rounding="RN", mode="EMULATE", vec_mode="GENERATE",
            k4_tune=False, packs=None, lib=None):
        lib = load_library(lib)
        lays = tuple(_layout(x, n) for x, n in zip((A, B, C), "ABC"))
        opts = (int(N), int(g), rounding, mode, vec_mode, bool(k4_tune))
        pk = None if packs is None else tuple(None if p is None else id(p) for p in packs)
        key = (spec, lays, opts, pk, id(lib), lib.current_device())
        return self._get(key, lambda: Plan(spec, *lays, N=N, g=g, rounding=rounding, mode=mode,
                                           vec_mode=vec_mode, k4_tune=k4_tune, packs=packs, lib=lib))

    def clear(self):
        """Forgets every plan. Plans that own device memory (RESIDENT vectors) are closed here;
        the others are left to their finalizers, since callers may still hold them."""
        with self._lock:
            dropped = self._plans
            self._plans = {}
        seen = set()
        for plan in dropped.values():
            if id(plan) not in seen and plan.options["vec_mode"] == "RESIDENT":
                plan.close()
            seen.add(id(plan))


default_plan_cache = PlanCache()


def contract(spec, A, B, out, *, alpha=1.0, beta=0.0, N, g=0, rounding="RN", mode="EMULATE",
             vec_mode="GENERATE", k4_tune=False, workspace=None, stream=None, plan_cache=None,
             packs=None, packed=None, lib=None):
    """einsum-style `out <- alpha sum A B + beta out` ("ik,kj->ij") on float64 CUDA arrays.
    The plan comes from `plan_cache` (default: the process-wide cache; False: a plan for this
    call only). `workspace`: caller-owned, >= workspace_size(...). Returns out."""
    lib = load_library(lib)
    if plan_cache is False:
        if vec_mode != "GENERATE":
            raise ValueError("plan_cache=False needs vec_mode GENERATE")
        with Plan(spec, A, B, out, N=N, g=g, rounding=rounding, mode=mode, vec_mode=vec_mode,
                  k4_tune=k4_tune, packs=packs, lib=lib) as plan:
            return plan.contract(A, B, out, alpha=alpha, beta=beta, workspace=workspace,
                                 stream=stream, packed=packed)
    cache = default_plan_cache if plan_cache is None else plan_cache
    plan = cache.get(spec, A, B, out, N=N, g=g, rounding=rounding, mode=mode, vec_mode=vec_mode,
                     k4_tune=k4_tune, packs=packs, lib=lib)
    return plan.contract(A, B, out, alpha=alpha, beta=beta, workspace=workspace, stream=stream,
                         packed=packed)


def workspace_size(spec, A, B, C, *, N, g=0, rounding="RN", mode="EMULATE", vec_mode="GENERATE",
                   packs=None, lib=None):
    """Exact workspace bytes for these operands (arrays or `Layout`s); host library only."""
    descs = _descs(spec, [_layout(x, n) for x, n in zip((A, B, C), "ABC")])
    return host.workspace_size(descs, N=N, g=g, rounding=rounding, mode=mode, vec_mode=vec_mode,
                               packing=_pack_specs(packs), lib=load_library(lib).host)
