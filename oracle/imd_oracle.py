"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY, never imported by the product).

`lower` restates the reference's index-map lowering (spec/oracle.py:751-860, normative text
docs/DESIGN.md:1526-1597): label classes I/J/K/L, the coalescing role swap, the canonical mode
orders, fusion and the additive int64 scatter vectors. `contract_tensor` restates
spec/oracle.py:871-960: it gathers each batch's canonical matrices through those vectors and
hands them to the C kernels of imd_oracle.c (ctypes), which hold the numerics.

Parity is pinned by tests/golden (outputs of the reference's own spec/oracle.py).
"""
import ctypes as C
import math
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libimd_oracle.so")
REF_HOST_PATH = os.path.join(HERE, "_ref", "libimmerdink_host_ref.so")

MODULI = (256, 255, 253, 251, 247, 241, 239, 233, 229, 227,
          223, 217, 211, 199, 197, 193, 191, 181, 179, 173)
INT64_MAX = 2**63 - 1
GEMM_DIM_MAX = 2**31 - 1


class InvalidValue(Exception):
    pass


class NotSupported(Exception):
    pass


def reference_tree():
    """Where the reference's source tree lies: $IMD_REFERENCE, else a directory `reference` beside
    this repository; None when there is none (then only prebuilt files under _ref are used)."""
    cand = os.environ.get("IMD_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src", "host")) else None


def build(force=False):
    """Compile the C oracle (and the reference host library when its tree is present)."""
    src = os.path.join(HERE, "imd_oracle.c")
    stale = (not os.path.exists(LIB_PATH)
             or os.path.getmtime(LIB_PATH) < os.path.getmtime(src))
    ref = reference_tree()
    if force or stale or (ref is not None and not os.path.exists(REF_HOST_PATH)):
        subprocess.run(["make", "-C", HERE] + ([f"REF={ref}"] if ref else []), check=True,
                       capture_output=True)


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        dp, i64 = C.c_void_p, C.c_int64
        L.imdo_gemm.restype = C.c_int
        L.imdo_gemm.argtypes = [C.c_int, C.c_int, i64, i64, i64, dp, i64, dp, i64, C.c_double,
                                C.c_double, dp, dp, i64, C.c_int, i64, dp, dp, dp, dp, dp]
        L.imdo_direct.restype = C.c_int
        L.imdo_direct.argtypes = [i64, i64, i64, dp, i64, dp, i64, C.c_double, C.c_double, dp,
                                  dp, i64]
        L.imdo_scale.restype = C.c_int
        L.imdo_scale.argtypes = [C.c_int, C.c_int, i64, dp, i64, i64, i64, i64, dp, dp]
        L.imdo_residues.restype = C.c_int
        L.imdo_residues.argtypes = [C.c_int, C.c_int, dp, i64, i64, i64, i64, dp, dp]
        L.imdo_constants.restype = C.c_int
        L.imdo_constants.argtypes = [C.c_int, dp, dp, dp, dp, dp]
        L.imdo_round_scaled.restype = C.c_double
        L.imdo_round_scaled.argtypes = [C.c_int, dp, C.c_int]
        L.imdo_crt.restype = C.c_int
        L.imdo_crt.argtypes = [C.c_int, dp, dp, dp]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data


def _raise(st):
    if st == 1:
        raise InvalidValue("oracle: invalid value")
    if st == 2:
        raise NotSupported("oracle: kappa >= T under RN")


# ----------------------------------------------------------------------------- constants
def constants(N):
    """P, H, T, [M_l], [q_l] as Python ints (from the C code: what the oracle really uses)."""
    P = np.zeros(6, np.uint64)
    H = np.zeros(6, np.uint64)
    T = np.zeros(6, np.uint64)
    M = np.zeros((N, 6), np.uint64)
    q = np.zeros(N, np.int32)
    _raise(lib().imdo_constants(N, _p(P), _p(H), _p(T), _p(M), _p(q)))

    def big(w):
        return sum(int(x) << (64 * i) for i, x in enumerate(w))
    return big(P), big(H), big(T), [big(r) for r in M], [int(x) for x in q]


def round_scaled(z, e):
    """RN-even binary64 of the integer z times 2^e (one rounding)."""
    mag = abs(z)
    w = np.array([(mag >> (64 * i)) & (2**64 - 1) for i in range(6)], np.uint64)
    return lib().imdo_round_scaled(1 if z < 0 else 0, _p(w), e)


def crt(N, residues):
    w = np.array(residues, np.uint8)
    neg = C.c_int(0)
    mag = np.zeros(6, np.uint64)
    _raise(lib().imdo_crt(N, _p(w), C.addressof(neg), _p(mag)))
    z = sum(int(x) << (64 * i) for i, x in enumerate(mag))
    return -z if neg.value else z


# ----------------------------------------------------------------------------- matrix level
def scale(X, N, rounding="RN", k_plan=None):
    """sigma (int16) and flags (u8) of the rows of the 2-D float64 array X."""
    X = np.ascontiguousarray(X, np.float64)
    rows, k = X.shape
    sig = np.zeros(rows, np.int16)
    fl = np.zeros(rows, np.uint8)
    _raise(lib().imdo_scale(N, int(rounding == "TRUNC"), k if k_plan is None else k_plan,
                            _p(X), rows, k, k, 1, _p(sig), _p(fl)))
    return sig, fl


def residues(X, sigma, N, rounding="RN"):
    """int8 residue planes [N][rows][k] of the rows of X under shifts sigma."""
    X = np.ascontiguousarray(X, np.float64)
    rows, k = X.shape
    R = np.zeros((N, rows, k), np.int8)
    sg = np.ascontiguousarray(sigma, np.int16)
    _raise(lib().imdo_residues(N, int(rounding == "TRUNC"), _p(X), rows, k, k, 1, _p(sg), _p(R)))
    return R


def gemm(A, Bt, N, alpha=1.0, beta=0.0, Cin=None, rounding="RN", literal=False, chunk=0,
         trace=None):
    """One batch. A: m x k rows, Bt: n x k (columns of B as rows). Returns the m x n result."""
    A = np.ascontiguousarray(A, np.float64)
    Bt = np.ascontiguousarray(Bt, np.float64)
    m, k = A.shape
    n = Bt.shape[0]
    out = np.zeros((m, n), np.float64)
    cin = None if Cin is None else np.ascontiguousarray(Cin, np.float64)
    t = {}
    if trace is not None:
        t = dict(sigma=np.zeros(m, np.int16), tau=np.zeros(n, np.int16),
                 fA=np.zeros(m, np.uint8), fB=np.zeros(n, np.uint8))
        if literal:
            t["W"] = np.zeros((N, m, n), np.uint8)
        trace.update(t)
    _raise(lib().imdo_gemm(N, int(rounding == "TRUNC"), m, n, k, _p(A), max(k, 1), _p(Bt),
                           max(k, 1), float(alpha), float(beta), _p(cin), _p(out), max(n, 1),
                           int(bool(literal)), int(chunk), _p(t.get("sigma")), _p(t.get("tau")),
                           _p(t.get("fA")), _p(t.get("fB")), _p(t.get("W"))))
    return out


# ----------------------------------------------------------------------------- lowering
class Desc:
    def __init__(self, extent, stride, label):
        assert len(extent) == len(stride) == len(label)
        self.extent, self.stride, self.label = list(extent), list(stride), list(label)

    def empty(self):
        return 0 in self.extent


class View:
    pass


def _stride_rule(d):
    below = 0
    for a, _, e in sorted((abs(s), p, e) for p, (e, s) in enumerate(zip(d.extent, d.stride))
                          if e > 1):
        if a <= below:
            return False
        below += a * (e - 1)
    return True


def _radix(modes, X):
    """Offsets of tensor X over fused modes [(extent, {X: stride})...], first mode fastest."""
    v = np.zeros(1, np.int64)
    for e, st in modes:
        v = (np.arange(e, dtype=np.int64)[:, None] * np.int64(st[X]) + v[None, :]).reshape(-1)
    return v


def lower(A, B, C, mode="EMULATE", orders=None):
    """The lowering with legality rows 1-5 in precedence order. `orders` ({post-swap class:
    [labels]}): canonical orders adopted from packed operands (spec/oracle.py:831-836)."""
    T = {"A": A, "B": B, "C": C}
    for d in T.values():
        if any(e < 0 for e in d.extent):
            raise InvalidValue("negative extent")
    ext, members, ms, first = {}, {}, {}, {}
    pos = 0
    for X in "ABC":
        d = T[X]
        for e, s, l in zip(d.extent, d.stride, d.label):
            if ext.setdefault(l, e) != e:
                raise InvalidValue("extent mismatch")
            members.setdefault(l, set()).add(X)
            ms[(X, l)] = ms.get((X, l), 0) + s
            first.setdefault(l, pos)
            pos += 1
    if len(set(C.label)) != len(C.label):
        raise NotSupported("repeated label in C")
    for l, mem in members.items():
        if mem == {"C"} and ext[l] > 1:
            raise NotSupported("label only in C")
    if not C.empty() and not _stride_rule(C):
        raise InvalidValue("C stride rule")
    if any(abs(v) > INT64_MAX for v in ms.values()):
        raise InvalidValue("diagonal stride")
    for d in T.values():
        if not d.empty() and sum(abs(s) * (e - 1) for e, s in zip(d.extent, d.stride)) > INT64_MAX:
            raise InvalidValue("span")
    cls = {}
    for l, mem in members.items():
        cls[l] = ("L" if mem == {"A", "B", "C"} else "I" if mem == {"A", "C"} else
                  "J" if mem == {"B", "C"} else "I" if mem == {"C"} else "K")
    size = {g: math.prod(ext[l] for l in cls if cls[l] == g and ext[l] != 1) for g in "IJKL"}
    if any(v > INT64_MAX for v in size.values()):
        raise InvalidValue("extent product")
    stride = {X: {l: ms.get((X, l), 0) for l in ext} for X in "ABC"}
    swapped = False
    if not C.empty():
        kept = [(abs(s), p) for p, (e, s) in enumerate(zip(C.extent, C.stride)) if e > 1]
        if kept:
            swapped = cls[C.label[min(kept)[1]]] == "I"
    if swapped:
        stride["A"], stride["B"] = stride["B"], stride["A"]
        cls = {l: {"I": "J", "J": "I"}.get(c, c) for l, c in cls.items()}
        size["I"], size["J"] = size["J"], size["I"]
    v = View()
    v.m, v.n, v.k, v.b = size["I"], size["J"], size["K"], size["L"]
    v.swapped = swapped
    for x, y in ((v.m, v.k), (v.k, v.n), (v.m, v.n)):
        if v.b * x * y > INT64_MAX:
            raise InvalidValue("operand size")
    v.empty_output = v.b == 0 or v.m == 0 or v.n == 0
    if mode == "EMULATE" and not v.empty_output and v.k >= 2 and \
            (v.m > GEMM_DIM_MAX or -(-v.n // 16) * 16 > GEMM_DIM_MAX):
        raise InvalidValue("gemm dims")
    big, oth = ("A", "B") if v.m >= v.n else ("B", "A")

    def a(X, l):
        return abs(stride[X][l])
    keys = {"I": lambda l: (a("C", l), a("A", l), first[l]),
            "J": lambda l: (a("C", l), a("B", l), first[l]),
            "L": lambda l: (a("C", l), a("A", l), a("B", l), first[l]),
            "K": lambda l: (a(big, l), a(oth, l), first[l])}
    v.order = {g: sorted((l for l in cls if cls[l] == g and ext[l] != 1), key=keys[g])
               for g in "IJKL"}
    for g, lst in (orders or {}).items():
        assert sorted(lst) == sorted(v.order[g]), "an adopted order permutes the class's labels"
        v.order[g] = list(lst)
    v.ext, v.stride = ext, stride
    v.fused = {}
    for g in "IJKL":
        fused = []
        for l in v.order[g]:
            if fused and all(stride[X][l] == fused[-1][1][X] * fused[-1][0] for X in "ABC"):
                fused[-1][0] *= ext[l]
            else:
                fused.append([ext[l], {X: stride[X][l] for X in "ABC"}])
        v.fused[g] = fused
    v.vec = {}
    if not v.empty_output:
        where = {"A_row": ("A", "I"), "A_k": ("A", "K"), "A_bat": ("A", "L"),
                 "B_k": ("B", "K"), "B_col": ("B", "J"), "B_bat": ("B", "L"),
                 "C_row": ("C", "I"), "C_col": ("C", "J"), "C_bat": ("C", "L")}
        v._where, v._cache = where, {}
    return v


def vec(view, name):
    if name not in view._cache:
        X, g = view._where[name]
        view._cache[name] = _radix(view.fused[g], X)
    return view._cache[name]


# ----------------------------------------------------------------------------- tensor level
def contract_tensor(A, B, Cbuf, dA, dB, dC, alpha, beta, N, rounding="RN", mode="EMULATE",
                    baseA=0, baseB=0, baseC=0, literal=False, chunk=0, rows=None, cols=None,
                    orders=None):
    """C <- alpha A B + beta C on flat float64 buffers with descriptors (extent, element stride,
    label); base* is the buffer index of the all-zero multi-index. Returns a new flat C buffer.

    rows / cols (index arrays into the canonical i-bar / j-bar spaces) restrict the computation
    to a block of outputs; untouched elements keep Cbuf's values. Raises like the reference:
    InvalidValue / NotSupported."""
    if not (2 <= N <= 20) or rounding not in ("RN", "TRUNC") or mode not in ("EMULATE", "DIRECT"):
        raise InvalidValue("option")
    view = lower(dA, dB, dC, mode, orders)
    out = np.array(Cbuf, dtype=np.float64, copy=True)
    if view.empty_output:
        return out
    m, n, k, b = view.m, view.n, view.k, view.b
    if mode == "EMULATE" and k > 1:
        P, H, T, _, _ = constants(N)
        kappa = math.isqrt(k)
        kappa += kappa * kappa != k
        if rounding == "RN" and kappa >= T:
            raise NotSupported("kappa >= T")
    opA, opB = (B, A) if view.swapped else (A, B)
    bA, bB = (baseB, baseA) if view.swapped else (baseA, baseB)
    reads_ab = alpha != 0.0 and k != 0
    kind = "SCALE" if not reads_ab else "DIRECT" if (mode == "DIRECT" or k == 1) else "GEMM"
    ri = np.arange(m) if rows is None else np.asarray(rows, np.int64)
    cj = np.arange(n) if cols is None else np.asarray(cols, np.int64)
    c_row, c_col, c_bat = vec(view, "C_row")[ri], vec(view, "C_col")[cj], vec(view, "C_bat")
    for lam in range(b):
        cidx = baseC + c_bat[lam] + c_row[:, None] + c_col[None, :]
        Cl = np.ascontiguousarray(out[cidx]) if beta != 0.0 else None
        if kind == "SCALE":
            res = np.zeros((len(ri), len(cj))) if beta == 0.0 else float(beta) * Cl
        else:
            Al = opA[bA + vec(view, "A_bat")[lam] + vec(view, "A_row")[ri][:, None]
                     + vec(view, "A_k")[None, :]]
            Bl = opB[bB + vec(view, "B_bat")[lam] + vec(view, "B_col")[cj][:, None]
                     + vec(view, "B_k")[None, :]]
            if kind == "DIRECT":
                Al = np.ascontiguousarray(Al, np.float64)
                Bl = np.ascontiguousarray(Bl, np.float64)
                res = np.zeros((len(ri), len(cj)))
                lib().imdo_direct(len(ri), len(cj), k, _p(Al), max(k, 1), _p(Bl), max(k, 1),
                                  float(alpha), float(beta), _p(Cl), _p(res), max(len(cj), 1))
            else:
                res = gemm(Al, Bl, N, alpha, beta, Cl, rounding, literal, chunk)
        out[cidx] = res
    return out


# ----------------------------------------------------------------------------- packed operands
K_PAD64_MIN = 96   # k > 96: K rows padded to 64 (pack format 2), else to 16 (format 1)


class PackView:
    pass


def pack_view(X, contracted, batch, rows=None, order="AUTO", N=14, rounding="RN"):
    """Lowering of one operand X for packing (spec/oracle.py:1122-1186): classes K (contracted),
    L (batch), R (rows: listed for GIVEN, the rest of X's labels for AUTO); extent-1 labels
    dropped; AUTO orders a class by (|merged stride|, first position); modes fused over X's
    strides alone; byte layout of spec/oracle.py:1085-1102."""
    if not (2 <= N <= 20) or rounding not in ("RN", "TRUNC") or order not in ("AUTO", "GIVEN"):
        raise InvalidValue("option")
    if any(e < 0 for e in X.extent):
        raise InvalidValue("negative extent")
    ext, ms, first = {}, {}, {}
    for p, (e, st, l) in enumerate(zip(X.extent, X.stride, X.label)):
        if ext.setdefault(l, e) != e:
            raise InvalidValue("extent mismatch")
        ms[l] = ms.get(l, 0) + st
        first.setdefault(l, p)
    K, L = list(contracted), list(batch)
    if order == "AUTO":
        if rows:
            raise InvalidValue("AUTO with rows")
        R = None
    else:
        R = list(rows or [])
    listed = K + L + (R or [])
    if any(l not in ext for l in listed) or len(set(listed)) != len(listed):
        raise InvalidValue("labels")
    if R is None:
        R = [l for l in ext if l not in K and l not in L]
    elif set(listed) != set(ext):
        raise InvalidValue("GIVEN without every label")
    if any(abs(v) > INT64_MAX for v in ms.values()):
        raise InvalidValue("merged stride")
    if not X.empty() and sum(abs(s) * (e - 1) for e, s in zip(X.extent, X.stride)) > INT64_MAX:
        raise InvalidValue("span")
    lists = {"K": K, "L": L, "R": R}
    size = {c: math.prod(ext[l] for l in lists[c] if ext[l] != 1) for c in "KLR"}
    if any(v > INT64_MAX for v in size.values()):
        raise InvalidValue("extent product")
    v = PackView()
    v.N, v.rounding = N, rounding
    v.b, v.r, v.k = size["L"], size["R"], size["K"]
    v.format = 2 if v.k > K_PAD64_MIN else 1
    align = 64 if v.format == 2 else 16
    v.k_hat = -(-v.k // align) * align
    v.regs, v.pack_bytes = {}, 0
    if v.b * v.r * v.k != 0:
        off = 0
        for name, nbytes in (("sig", 2 * v.b * v.r), ("flag", v.b * v.r),
                             ("res", N * v.b * v.r * v.k_hat + (-(-v.r // 16) * 16 - v.r) * v.k_hat)):
            v.regs[name] = (off, nbytes)
            off += -(-nbytes // 256) * 256
            if off > 2**64 - 1:
                raise InvalidValue("pack size")
        v.pack_bytes = off
    if not any(ext[l] != 1 for l in K):
        raise NotSupported("K empty after lowering")
    if rounding == "RN" and v.k >= 2:
        kappa = math.isqrt(v.k)
        kappa += kappa * kappa != v.k
        if kappa >= constants(N)[2]:
            raise NotSupported("kappa >= T")
    key = (lambda l: (abs(ms[l]), first[l])) if order == "AUTO" else None
    v.order = {c: [l for l in (sorted(lists[c], key=key) if key else lists[c]) if ext[l] != 1]
               for c in "KLR"}
    v.fused = {}
    for c in "LRK":
        fused = []
        for l in v.order[c]:
            if fused and ms[l] == fused[-1][1] * fused[-1][0]:
                fused[-1][0] *= ext[l]
            else:
                fused.append([ext[l], ms[l]])
        v.fused[c] = fused
    words = [v.format, N, 0 if rounding == "RN" else 1, v.b, v.r, v.k]
    for c in "LRK":
        words.append(len(v.fused[c]))
        for e, st in v.fused[c]:
            words += [e, st]
    v.key = tuple(words)
    h = 0xcbf29ce484222325
    for w in words:
        for byte in (w & (2**64 - 1)).to_bytes(8, "little"):
            h = ((h ^ byte) * 0x100000001b3) & (2**64 - 1)
    v.digest = h
    return v


def pack(Xbuf, base, v):
    """The packed bytes of X (spec/oracle.py:1193-1224): per row (batch, row) its shift and
    flag, then the N residue planes over the canonical K with zero K padding, a zero tail and
    zero alignment gaps."""
    out = np.zeros(v.pack_bytes, np.uint8)
    if v.pack_bytes == 0:
        return out
    vec_of = lambda c: _radix([(e, {"X": st}) for e, st in v.fused[c]], "X")
    vL, vR, vK = vec_of("L"), vec_of("R"), vec_of("K")
    rows = np.asarray(Xbuf, np.float64)[base + (vL[:, None] + vR[None, :]).reshape(-1)[:, None]
                                        + vK[None, :]]
    sig, fl = scale(rows, v.N, v.rounding)
    R = residues(rows, sig, v.N, v.rounding)            # [N][b r][k]
    so, fo, ro_ = v.regs["sig"][0], v.regs["flag"][0], v.regs["res"][0]
    out[so:so + 2 * len(sig)] = sig.astype("<i2").view(np.uint8)
    out[fo:fo + len(fl)] = fl
    planes = np.zeros((v.N, v.b * v.r, v.k_hat), np.int8)
    planes[:, :, :v.k] = R
    out[ro_:ro_ + planes.size] = planes.reshape(-1).view(np.uint8)
    return out


def ref_host():
    """The reference's own host library (lowering, legality, sizes), when it was built."""
    if not os.path.exists(REF_HOST_PATH):
        return None
    return C.CDLL(REF_HOST_PATH)
