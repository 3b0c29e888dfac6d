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


def build(force=False):
    """Compile the C oracle (and the reference host library when its tree is present)."""
    src = os.path.join(HERE, "imd_oracle.c")
    stale = (not os.path.exists(LIB_PATH)
             or os.path.getmtime(LIB_PATH) < os.path.getmtime(src))
    if force or stale or (os.path.isdir("/root/reference/src/host")
                          and not os.path.exists(REF_HOST_PATH)):
        subprocess.run(["make", "-C", HERE], check=True, capture_output=True)


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


def lower(A, B, C, mode="EMULATE"):
    """The lowering with legality rows 1-5 in precedence order."""
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
                    baseA=0, baseB=0, baseC=0, literal=False, chunk=0, rows=None, cols=None):
    """C <- alpha A B + beta C on flat float64 buffers with descriptors (extent, element stride,
    label); base* is the buffer index of the all-zero multi-index. Returns a new flat C buffer.

    rows / cols (index arrays into the canonical i-bar / j-bar spaces) restrict the computation
    to a block of outputs; untouched elements keep Cbuf's values. Raises like the reference:
    InvalidValue / NotSupported."""
    if not (2 <= N <= 20) or rounding not in ("RN", "TRUNC") or mode not in ("EMULATE", "DIRECT"):
        raise InvalidValue("option")
    view = lower(dA, dB, dC, mode)
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


def ref_host():
    """The reference's own host library (lowering, legality, sizes), when it was built."""
    if not os.path.exists(REF_HOST_PATH):
        return None
    return C.CDLL(REF_HOST_PATH)
