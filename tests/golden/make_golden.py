"""Generates tests/golden/*.npz by running the REFERENCE's executable specification
(spec/oracle.py of the reference tree, imported read-only) on seeded and adversarial inputs.

Run once where the reference tree is present:

    python tests/golden/make_golden.py [/path/to/reference [file names to regenerate...]]

The fixtures pin the CPU oracle in oracle/ (and through it the CUDA library): every array is
stored as raw bit patterns, so the comparison is bit for bit. The input constructions below
are this repository's own; only the outputs come from the reference.

Files written:
  matrix.npz   one-batch cases through oracle.contract with full traces
               (sigma, tau, flags, residue planes, W planes, z, output)
  tensor.npz   strided / permuted / batched / diagonal / swapped descriptors through
               oracle.contract_tensor, and the lowering summary of each (m, n, k, b, swapped,
               canonical orders, scatter vectors)
  status.npz   descriptor sets with the status the reference's lowering raises
  pack.npz     packed operands: pack descriptors, layouts, keys and the packed BYTES from
               oracle.pack, and oracle.contract_tensor(packs=...) outputs
"""
import json
import math
import os
import random
import struct
import sys

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("IMD_REFERENCE", "")
if not os.path.isdir(os.path.join(REF, "spec")):
    raise SystemExit("usage: make_golden.py <path of the reference tree>  (or set IMD_REFERENCE)")
sys.path.insert(0, os.path.join(REF, "spec"))
import oracle as ro  # noqa: E402  (the reference's spec/oracle.py)

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(x):
    return struct.unpack("<Q", struct.pack("<d", x))[0]


def arr_bits(rows):
    return np.array([[bits(v) for v in r] for r in rows], dtype=np.uint64)


# --------------------------------------------------------------------------- generators
def gen_uniform(rng, lo=-1.0, hi=1.0):
    return lambda: rng.uniform(lo, hi)


def gen_wide(rng, emin, emax):
    """sign * 2^e * u, e uniform integer, u in [1, 2)."""
    return lambda: rng.choice((-1.0, 1.0)) * math.ldexp(1.0 + rng.random(), rng.randint(emin, emax))


def gen_ints(rng, span):
    return lambda: float(rng.randint(-span, span))


def gen_bimodal(rng):
    return lambda: rng.choice((-1.0, 1.0)) * (1.0 if rng.random() < 0.5 else 1e-8) * (1 + rng.random())


def gen_subnormal(rng):
    return lambda: rng.choice((-1.0, 1.0)) * math.ldexp(rng.random(), -1022 - rng.randint(0, 40))


def matrix(gen, r, c):
    return [[gen() for _ in range(c)] for _ in range(r)]


def inject(rng, M, values, count):
    for _ in range(count):
        i = rng.randrange(len(M))
        j = rng.randrange(len(M[0]))
        M[i][j] = rng.choice(values)


# --------------------------------------------------------------------------- matrix cases
def matrix_cases():
    rng = random.Random(20251125)
    cases = []

    def add(name, A, B, C, alpha, beta, N, rounding="RN", chunk=None):
        cases.append(dict(name=name, A=A, B=B, C=C, alpha=alpha, beta=beta, N=N,
                          rounding=rounding, chunk=chunk))

    # seeded sweeps over N, rounding, data classes
    for N in (2, 3, 5, 8, 11, 12, 13, 14, 15, 16, 17, 20):
        m, n, k = rng.randint(2, 6), rng.randint(2, 6), rng.randint(2, 40)
        for rounding in ("RN", "TRUNC"):
            add(f"uniform_N{N}_{rounding}", matrix(gen_uniform(rng), m, k),
                matrix(gen_uniform(rng), k, n), None, 1.0, 0.0, N, rounding)
    for N in (8, 12, 14, 16, 20):
        m, n, k = 4, 5, 24
        add(f"wide_N{N}", matrix(gen_wide(rng, -20, 20), m, k), matrix(gen_wide(rng, -20, 20), k, n),
            matrix(gen_uniform(rng), m, n), 1.5, 0.5, N)
        add(f"verywide_N{N}", matrix(gen_wide(rng, -1000, 900), m, k),
            matrix(gen_wide(rng, -60, 60), k, n), matrix(gen_uniform(rng), m, n), -0.75, 1.0, N)
        add(f"ints_N{N}", matrix(gen_ints(rng, 1000), m, k), matrix(gen_ints(rng, 7), k, n),
            None, 1.0, 0.0, N, "TRUNC")
        add(f"bimodal_N{N}", matrix(gen_bimodal(rng), m, k), matrix(gen_bimodal(rng), k, n),
            None, 1.0, 0.0, N)
        add(f"subnormal_N{N}", matrix(gen_subnormal(rng), m, k), matrix(gen_uniform(rng), k, n),
            None, 1.0, 0.0, N)
        add(f"subnormal_both_N{N}", matrix(gen_subnormal(rng), m, k),
            matrix(gen_subnormal(rng), k, n), None, 2.0, 0.0, N)
    # zero rows / columns, signed zeros, non-finite entries (native path), alpha/beta corners
    for N in (9, 14, 16):
        A = matrix(gen_uniform(rng), 5, 12)
        B = matrix(gen_uniform(rng), 12, 6)
        A[1] = [0.0] * 12
        A[3] = [-0.0] * 12
        for h in range(12):
            B[h][2] = 0.0
        inject(rng, A, [math.inf, -math.inf, math.nan, 0.0, -0.0], 4)
        inject(rng, B, [math.inf, -math.inf, math.nan, 0.0, -0.0], 4)
        Cm = matrix(gen_uniform(rng), 5, 6)
        add(f"special_N{N}", A, B, Cm, 1.0, 0.0, N)
        add(f"special_ab_N{N}", A, B, Cm, -2.5, 0.25, N)
        add(f"alpha0_N{N}", A, B, Cm, 0.0, 0.5, N)
        add(f"alpha0_beta0_N{N}", A, B, Cm, 0.0, 0.0, N)
        add(f"negzero_alpha_N{N}", matrix(gen_uniform(rng), 3, 4), matrix(gen_uniform(rng), 4, 3),
            matrix(gen_uniform(rng), 3, 3), -0.0, -0.0, N)
    # native path order: overflow then -Inf in canonical order gives NaN, not -Inf
    big = 1.7976931348623157e308
    add("native_order", [[big, big, -math.inf], [-math.inf, big, big]], [[2.0], [2.0], [1.0]],
        None, 1.0, 0.0, 9)
    # single rounding into the subnormal range: a b with a half-ulp bit and a sticky bit
    for j in (0, 1, 7, 13, 25):
        a = math.ldexp(1 + 2.0 ** -(52 - j), -512)
        b = math.ldexp(1 + 2.0 ** -(52 - j), -512 - j)
        for sa in (1.0, -1.0):
            for N in (14, 16, 20):
                for rounding in ("RN", "TRUNC"):
                    add(f"subtie_j{j}_{sa}_N{N}_{rounding}", [[sa * a]], [[b]], None, 1.0, 0.0,
                        N, rounding)
    # rows exactly on the shift boundary (the ceiling in S decides), k = 2, real width
    for N in range(14, 21):
        for rounding in ("TRUNC", "RN"):
            pl = ro.Plan(N, 2, rounding)
            bud = pl.T if rounding == "TRUNC" else (2 * pl.T - pl.kappa) // 2
            U = bud.bit_length() - 1
            w1 = (bud >> (U - 52)) << (U - 52)
            w2 = math.isqrt(bud * bud - w1 * w1) + 1
            a1, a2 = math.ldexp(w1 >> (U - 52), -52), math.ldexp(w2, -U)
            add(f"boundary_N{N}_{rounding}", [[a1, a2]], [[a1], [a2]], None, 1.0, 0.0, N, rounding)
    # all entries round up (RN slack), small N
    for k in (5, 17, 33):
        row = [rng.randint(1, 60) + 0.5 + 2.0 ** -30 for _ in range(k)]
        add(f"roundup_k{k}", [row], [[v] for v in row], None, 1.0, 0.0, 2)
        add(f"roundup3_k{k}", [row], [[v] for v in row], None, 1.0, 0.0, 3)
    # beta epilogue is a single fma: cancellation cases
    e = -(1 + 2.0 ** -51)
    add("beta_fma", [[e]], [[1.0]], [[1 + 2.0 ** -52]], 1.0, 1 + 2.0 ** -52, 16)
    for t in range(6):
        beta = rng.uniform(-3, 3)
        ds = [rng.uniform(-1, 1) * 2.0 ** rng.randint(-30, 30) for _ in range(8)]
        Cs = [[-d / beta] for d in ds]
        add(f"beta_cancel_{t}", [[d] for d in ds], [[1.0]], Cs, 1.0, beta, 16)
    # overflow to +-Inf and large magnitudes in the emulated path
    add("overflow", [[1e200, 1e200], [-1e200, 3.0]], [[1e200, 1.0], [1e150, -1e200]], None, 1.0,
        0.0, 14)
    add("alpha_overflow", [[1e300, 1.0]], [[1.0], [1.0]], [[-1e300]], 1e10, 1e10, 14)
    # K chunking with an explicit small chunk (chunk invariance) and k = 1
    A = matrix(gen_uniform(rng), 3, 50)
    B = matrix(gen_uniform(rng), 50, 4)
    for chunk in (7, 16, 49, 50):
        add(f"chunk{chunk}", A, B, None, 1.0, 0.0, 14, "RN", chunk)
    add("k1", matrix(gen_uniform(rng), 4, 1), matrix(gen_uniform(rng), 1, 3), None, 1.0, 0.0, 14)
    return cases


def run_matrix(out):
    cases = matrix_cases()
    manifest = []
    for ci, c in enumerate(cases):
        t = {}
        kw = {} if c["chunk"] is None else {"chunk": c["chunk"]}
        res = ro.contract(c["A"], c["B"], c["C"], c["alpha"], c["beta"], c["N"], c["rounding"],
                          trace=t, **kw)
        key = f"c{ci}"
        m, k, n = len(c["A"]), len(c["B"]), len(c["B"][0])
        out[key + "_A"] = arr_bits(c["A"])
        out[key + "_Bt"] = arr_bits([[c["B"][h][j] for h in range(k)] for j in range(n)])
        if c["C"] is not None:
            out[key + "_C"] = arr_bits(c["C"])
        out[key + "_out"] = arr_bits(res)
        entry = dict(name=c["name"], key=key, N=c["N"], rounding=c["rounding"],
                     alpha=bits(c["alpha"]), beta=bits(c["beta"]), chunk=c["chunk"], m=m, n=n, k=k,
                     traced=bool(t))
        if t:
            out[key + "_sigma"] = np.array(t["sigma"], np.int16)
            out[key + "_tau"] = np.array(t["tau"], np.int16)
            out[key + "_fA"] = np.array(t["fA"], np.uint8)
            out[key + "_fB"] = np.array(t["fB"], np.uint8)
            out[key + "_RA"] = np.array(t["RA"], np.int8)      # [N][m][k]
            out[key + "_RB"] = np.array(t["RB"], np.int8)      # [N][n][k]
            out[key + "_W"] = np.array(t["W"], np.uint8)       # [N][m][n]
            entry["z"] = [[None if z is None else str(z) for z in row] for row in t["z"]]
        manifest.append(entry)
    out["manifest"] = np.frombuffer(json.dumps(manifest).encode(), np.uint8)
    print(f"matrix: {len(cases)} cases")


# --------------------------------------------------------------------------- tensor cases
def dense_strides(extent, order=None):
    """Element strides of a dense layout; order = mode positions from slowest to fastest."""
    order = list(range(len(extent))) if order is None else order
    st = [0] * len(extent)
    acc = 1
    for d in reversed(order):
        st[d] = acc
        acc *= extent[d]
    return st, acc


def tensor_cases():
    rng = random.Random(7)
    cases = []

    def add(name, spec, ext, layouts=None, N=14, alpha=1.0, beta=0.0, mode="EMULATE",
            rounding="RN", gen=None, pad=None, negate=None):
        """spec 'ab,bc->ac'; ext: label -> extent; layouts: per tensor the slowest-to-fastest
        mode order (None = as written); pad: per tensor {mode position: stride multiplier};
        negate: per tensor a list of mode positions whose stride is negated."""
        cases.append(dict(name=name, spec=spec, ext=ext, layouts=layouts or [None] * 3, N=N,
                          alpha=alpha, beta=beta, mode=mode, rounding=rounding, gen=gen,
                          pad=pad or [None] * 3, negate=negate or [None] * 3))

    add("c1_like", "ijk,kl->lij", dict(i=6, j=4, k=9, l=5))
    add("c1_like_N8", "ijk,kl->lij", dict(i=5, j=3, k=7, l=4), N=8)
    add("c2_like", "kjbc,kiac->abij", dict(a=3, b=2, c=4, i=2, j=3, k=2))
    add("c3_like", "ik,kj->ij", dict(i=5, j=6, k=11), alpha=1.5, beta=0.5, gen="wide")
    add("c3_like_N12", "ik,kj->ij", dict(i=4, j=5, k=9), N=12, alpha=1.5, beta=0.5, gen="wide")
    add("c3_like_N16", "ik,kj->ij", dict(i=4, j=5, k=9), N=16, alpha=1.5, beta=0.5, gen="wide")
    add("c4_like", "abcd,cdij->abij", dict(a=3, b=2, c=3, d=2, i=2, j=3), alpha=1.0, beta=1.0)
    add("c5_like", "pqrs,sq->pr", dict(p=4, q=3, r=5, s=2), layouts=[[3, 0, 1, 2], None, None],
        pad=[{1: 2}, None, None], N=16, gen="bimodal")
    add("batch", "bik,bkj->bij", dict(b=3, i=2, j=4, k=5))
    add("batch_fast", "ikb,kjb->ijb", dict(b=3, i=2, j=4, k=5), beta=0.5)
    add("two_batch", "xiyk,ykxj->xyij", dict(x=2, y=2, i=2, j=3, k=4))
    add("diag_a", "iik,kj->ij", dict(i=3, j=4, k=5))
    add("diag_k", "ikk,kj->ij", dict(i=3, j=4, k=5))
    add("a_only_sum", "ikx,kj->ij", dict(i=3, j=4, k=5, x=2))
    add("b_only_sum", "ik,kjx->ij", dict(i=3, j=4, k=5, x=3))
    add("outer", "i,j->ij", dict(i=4, j=5))
    add("outer_batch", "bi,bj->bij", dict(b=2, i=3, j=2), beta=2.0)
    add("dot", "k,k->", dict(k=17))
    add("matvec", "ik,k->i", dict(i=6, k=8))
    add("vecmat", "k,kj->j", dict(j=6, k=8))
    add("extent1", "iak,kbj->iabj", dict(i=3, a=1, k=4, b=1, j=2))
    add("k_empty_ext1", "ik,kj->ij", dict(i=3, j=4, k=1))
    add("k_zero", "ik,kj->ij", dict(i=3, j=4, k=0), beta=0.5)
    add("direct_mode", "ik,kj->ij", dict(i=3, j=4, k=6), mode="DIRECT", alpha=0.5, beta=0.25)
    add("trunc", "ijk,kl->lij", dict(i=3, j=2, k=6, l=3), rounding="TRUNC")
    add("permuted_c", "ik,kj->ji", dict(i=4, j=3, k=5))
    add("permuted_all", "kji,lk->jli", dict(i=3, j=2, k=4, l=3), layouts=[[1, 0, 2], [1, 0], [2, 0, 1]])
    add("neg_strides", "ik,kj->ij", dict(i=4, j=3, k=5), negate=[[1], [0, 1], None])
    add("padded", "ik,kj->ij", dict(i=4, j=3, k=5), pad=[{0: 2}, {0: 3}, {0: 2}], beta=1.0)
    add("fuse_split", "abk,kcd->abcd", dict(a=2, b=3, c=2, d=2, k=4))
    add("highrank", "abcxy,xydef->abcdef", dict(a=2, b=2, c=2, d=2, e=2, f=2, x=2, y=3), N=10)
    add("specials", "ik,kj->ij", dict(i=4, j=4, k=6), gen="specials", alpha=2.0, beta=0.5)
    add("m_gt_n_korder", "xyk,kj->xyj", dict(x=4, y=3, j=2, k=3), layouts=[[2, 0, 1], None, None],
        gen="specials")
    for t in range(10):
        labels = "abcdefg"
        ra, rb = rng.randint(1, 4), rng.randint(1, 4)
        la = rng.sample(labels, ra)
        lb = rng.sample(labels, rb)
        pool = sorted(set(la) | set(lb))
        lc = [x for x in pool if rng.random() < 0.6]
        rng.shuffle(lc)
        ext = {x: rng.randint(1, 3) for x in pool}
        lay = []
        for lab in (la, lb, lc):
            o = list(range(len(lab)))
            rng.shuffle(o)
            lay.append(o)
        add(f"random_{t}", f"{''.join(la)},{''.join(lb)}->{''.join(lc)}", ext, layouts=lay,
            N=rng.choice((6, 9, 14)), alpha=rng.choice((1.0, -0.5)), beta=rng.choice((0.0, 1.0, 0.3)))
    return cases


def build_tensor(rng, labels, ext, layout, pad, negate, gen):
    extent = [ext[l] for l in labels]
    st, size = dense_strides(extent, layout)
    if pad:
        # multiply the strides of every mode slower than the padded one
        for pos, mult in pad.items():
            base = st[pos]
            for d in range(len(st)):
                if st[d] > base:
                    st[d] *= mult
            size *= mult
    size = max(size, 1)
    buf = [gen() for _ in range(size)]
    base = 0
    if negate:
        for pos in negate:
            base += st[pos] * (extent[pos] - 1)
            st[pos] = -st[pos]
    return ro.Tensor(buf, base, ro.Desc(extent, st, [ord(l) for l in labels]))


def run_tensor(out):
    rng = random.Random(99)
    gens = dict(uniform=gen_uniform(rng), wide=gen_wide(rng, -20, 20), bimodal=gen_bimodal(rng))
    special_vals = [math.inf, -math.inf, math.nan, 0.0, -0.0, 1e308, -1e308]
    gens["specials"] = lambda: (rng.choice(special_vals) if rng.random() < 0.08
                                else rng.uniform(-1, 1))
    manifest = []
    for ci, c in enumerate(tensor_cases()):
        ins, outl = c["spec"].split("->")
        la, lb = ins.split(",")
        gen = gens[c["gen"] or "uniform"]
        tens = [build_tensor(rng, lab, c["ext"], c["layouts"][x], c["pad"][x], c["negate"][x], gen)
                for x, lab in enumerate((la, lb, outl))]
        entry = dict(name=c["name"], key=f"t{ci}", spec=c["spec"], N=c["N"], mode=c["mode"],
                     rounding=c["rounding"], alpha=bits(c["alpha"]), beta=bits(c["beta"]),
                     desc=[dict(extent=t.desc.extent, stride=t.desc.stride, label=t.desc.label,
                                base=t.base) for t in tens])
        key = entry["key"]
        for x, t in zip("ABC", tens):
            out[f"{key}_{x}"] = np.array([bits(v) for v in t.buf], np.uint64)
        try:
            tr = {}
            res = ro.contract_tensor(tens[0], tens[1], tens[2], c["alpha"], c["beta"], c["N"],
                                     c["rounding"], None, c["mode"], trace=tr)
            out[f"{key}_out"] = np.array([bits(v) for v in res], np.uint64)
            v = tr["view"]
            entry.update(status="SUCCESS", kind=tr["kind"], m=v.m, n=v.n, k=v.k, b=v.b,
                         swapped=bool(v.swapped), order={g: v.order[g] for g in "IJKL"},
                         fused={g: [[e, [st["A"], st["B"], st["C"]]] for _, e, st in v.fused[g]]
                                for g in "IJKL"})
            if not v.empty_output():
                out[f"{key}_vec"] = np.array(v.vec_region(), np.int64)
        except ro.NotSupported:
            entry["status"] = "NOT_SUPPORTED"
        except ro.InvalidValue:
            entry["status"] = "INVALID_VALUE"
        manifest.append(entry)
    out["manifest"] = np.frombuffer(json.dumps(manifest).encode(), np.uint8)
    print(f"tensor: {len(manifest)} cases; statuses:",
          {s: sum(1 for e in manifest if e['status'] == s) for s in {e['status'] for e in manifest}})


# --------------------------------------------------------------------------- status cases
def run_status(out):
    """Descriptor sets for the legality rows, with the status of the reference's lowering."""
    D = ro.Desc
    L = [ord(c) for c in "ijkxyz"]
    i, j, k, x = L[0], L[1], L[2], L[3]
    sets = [
        ("ok", D([3, 4], [4, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([3, 5], [5, 1], [i, j])),
        ("extent_mismatch", D([3, 4], [4, 1], [i, k]), D([5, 5], [5, 1], [k, j]), D([3, 5], [5, 1], [i, j])),
        ("repeat_c", D([3, 4], [4, 1], [i, k]), D([4, 3], [3, 1], [k, i]), D([3, 3], [3, 1], [i, i])),
        ("c_only", D([3, 4], [4, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([3, 5, 2], [10, 2, 1], [i, j, x])),
        ("c_only_ext1", D([3, 4], [4, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([3, 5, 1], [5, 1, 1], [i, j, x])),
        ("c_overlap", D([3, 4], [4, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([3, 5], [4, 1], [i, j])),
        ("c_stride0", D([3, 4], [4, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([3, 5], [0, 1], [i, j])),
        ("neg_extent", D([-1, 4], [4, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([3, 5], [5, 1], [i, j])),
        ("span_overflow", D([3, 4], [2**62, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([3, 5], [5, 1], [i, j])),
        ("empty_i", D([0, 4], [4, 1], [i, k]), D([4, 5], [5, 1], [k, j]), D([0, 5], [5, 1], [i, j])),
        ("repeat_c_first", D([3, 4], [4, 1], [i, k]), D([4, 3], [3, 1], [k, i]), D([3, 3, 2], [6, 2, 1], [i, i, x])),
        ("diag_overflow", D([2, 2, 4], [2**62, 2**62, 1], [i, i, k]), D([4, 5], [5, 1], [k, j]), D([2, 5], [5, 1], [i, j])),
        ("huge_m", D([2**31, 2], [0, 1], [i, k]), D([2, 5], [5, 1], [k, j]), D([2**31, 5], [5, 1], [i, j])),
        ("huge_n_ok_direct", D([2**31, 1], [0, 1], [i, k]), D([1, 5], [5, 1], [k, j]), D([2**31, 5], [5, 1], [i, j])),
    ]
    manifest = []
    for name, A, B, Cd in sets:
        try:
            ro.lower(A, B, Cd, build_vec=False)
            st = "SUCCESS"
        except ro.NotSupported:
            st = "NOT_SUPPORTED"
        except ro.InvalidValue:
            st = "INVALID_VALUE"
        manifest.append(dict(name=name, status=st,
                             desc=[dict(extent=d.extent, stride=d.stride, label=d.label)
                                   for d in (A, B, Cd)]))
    out["manifest"] = np.frombuffer(json.dumps(manifest).encode(), np.uint8)
    print("status:", [(e["name"], e["status"]) for e in manifest])


# --------------------------------------------------------------------------- packed operands
def pack_cases():
    cases = []

    def add(name, spec, ext, **kw):
        cases.append(dict(name=name, spec=spec, ext=ext, layouts=kw.get("layouts") or [None] * 3,
                          N=kw.get("N", 14), rounding=kw.get("rounding", "RN"), gen=kw.get("gen"),
                          alpha=kw.get("alpha", 1.0), beta=kw.get("beta", 0.0),
                          pad=kw.get("pad") or [None] * 3, negate=kw.get("negate") or [None] * 3))

    add("matrix", "ik,kj->ij", dict(i=5, j=6, k=11))
    add("matrix_N7_trunc", "ik,kj->ij", dict(i=4, j=3, k=9), N=7, rounding="TRUNC")
    add("matrix_N18", "ik,kj->ij", dict(i=3, j=4, k=7), N=18, alpha=1.5, beta=0.5)
    add("k_over_96", "ik,kj->ij", dict(i=3, j=2, k=99), N=6)
    add("swapped", "ik,kj->ji", dict(i=4, j=3, k=5))
    add("three_mode", "ijk,kl->lij", dict(i=3, j=2, k=6, l=3))
    add("two_k", "kjbc,kiac->abij", dict(a=2, b=2, c=3, i=2, j=2, k=2))
    add("batch", "bik,bkj->bij", dict(b=3, i=2, j=4, k=5), beta=1.0)
    add("batch_fast", "ikb,kjb->ijb", dict(b=2, i=3, j=4, k=5))
    add("permuted", "kji,lk->jli", dict(i=3, j=2, k=4, l=3), layouts=[[1, 0, 2], [1, 0], [2, 0, 1]])
    add("neg_padded", "ik,kj->ij", dict(i=4, j=3, k=5), negate=[[1], [0, 1], None],
        pad=[{1: 2}, None, None])
    add("specials", "ik,kj->ij", dict(i=4, j=4, k=6), gen="specials", alpha=2.0, beta=0.5)
    add("extent1", "iak,kbj->iabj", dict(i=3, a=1, k=4, b=1, j=2))
    add("diag", "iik,kj->ij", dict(i=3, j=4, k=5))
    add("k_orders_differ", "kci,ckj->ij", dict(i=3, j=2, k=3, c=4))
    add("k_extent1", "ik,kj->ij", dict(i=3, j=4, k=1))
    return cases


def run_pack(out):
    """Packed operands: for each case and caller operand, the AUTO and the GIVEN pack (its
    descriptor, layout, key and BYTES), and the contraction through packs of A, of B and of both."""
    rng = random.Random(4242)
    gens = dict(uniform=gen_uniform(rng))
    special_vals = [math.inf, -math.inf, math.nan, 0.0, -0.0, 1e308, -1e308]
    gens["specials"] = lambda: (rng.choice(special_vals) if rng.random() < 0.08
                                else rng.uniform(-1, 1))
    manifest = []
    for ci, c in enumerate(pack_cases()):
        ins, outl = c["spec"].split("->")
        la, lb = ins.split(",")
        gen = gens[c["gen"] or "uniform"]
        tens = [build_tensor(rng, lab, c["ext"], c["layouts"][x], c["pad"][x], c["negate"][x], gen)
                for x, lab in enumerate((la, lb, outl))]
        key = f"p{ci}"
        entry = dict(name=c["name"], key=key, spec=c["spec"], N=c["N"], rounding=c["rounding"],
                     alpha=bits(c["alpha"]), beta=bits(c["beta"]),
                     desc=[dict(extent=t.desc.extent, stride=t.desc.stride, label=t.desc.label,
                                base=t.base) for t in tens], packs=[], runs=[])
        for x, t in zip("ABC", tens):
            out[f"{key}_{x}"] = np.array([bits(v) for v in t.buf], np.uint64)
        made = {}
        for x, (lab, other) in enumerate(((la, lb), (lb, la))):
            for order in ("AUTO", "GIVEN"):
                if order == "AUTO":
                    kl = [ord(l) for l in dict.fromkeys(lab) if l not in outl]
                    bl = [ord(l) for l in dict.fromkeys(lab) if l in outl and l in other]
                    pd = ro.PackDesc(tens[x].desc, c["N"], c["rounding"], "AUTO", kl, bl, None)
                else:
                    pd = ro.pack_desc_for(tens[0].desc, tens[1].desc, tens[2].desc, "EMULATE", x,
                                          c["N"], c["rounding"])
                rec = dict(operand=x, order=order, contracted=pd.contracted, batch=pd.batch,
                           rows=pd.rows or [])
                try:
                    tr = {}
                    data = ro.pack(tens[x], pd, tr)
                    v = tr.get("view") or ro.pack_lower(pd)
                    tag = f"{key}_pack{x}{order[0]}"
                    out[tag] = np.frombuffer(bytes(data), np.uint8)
                    rec.update(status="SUCCESS", tag=tag, b=v.b, r=v.r, k=v.k, k_hat=v.k_hat,
                               format=v.format, pack_bytes=v.pack_bytes, key=list(v.key),
                               digest=v.digest, order_K=v.order["K"], order_L=v.order["L"],
                               order_R=v.order["R"],
                               regs={n: list(v.regs[n]) for n in v.regs})
                    made[(x, order)] = ro.PackedOperand(pd, data)
                except ro.NotSupported:
                    rec["status"] = "NOT_SUPPORTED"
                except ro.InvalidValue:
                    rec["status"] = "INVALID_VALUE"
                entry["packs"].append(rec)
        for order in ("AUTO", "GIVEN"):
            for which in ((0,), (1,), (0, 1)):
                if any((x, order) not in made for x in which):
                    continue
                packs = tuple(made[(x, order)] if x in which else None for x in (0, 1))
                run = dict(order=order, which=list(which))
                try:
                    tr = {}
                    res = ro.contract_tensor(tens[0], tens[1], tens[2], c["alpha"], c["beta"],
                                             c["N"], c["rounding"], None, "EMULATE", trace=tr,
                                             packs=packs)
                    tag = f"{key}_out{order[0]}{''.join(map(str, which))}"
                    out[tag] = np.array([bits(v) for v in res], np.uint64)
                    run.update(status="SUCCESS", tag=tag, kind=tr["kind"],
                               orders={g: lst for g, lst in tr["packed"]["orders"].items()})
                except ro.PackMismatch as e:
                    run.update(status="PACK_MISMATCH", reason=e.reason)
                except ro.NotSupported:
                    run["status"] = "NOT_SUPPORTED"
                entry["runs"].append(run)
        manifest.append(entry)
    out["manifest"] = np.frombuffer(json.dumps(manifest).encode(), np.uint8)
    print("pack:", len(manifest), "cases;",
          sum(len(e["packs"]) for e in manifest), "packs;",
          {s: sum(1 for e in manifest for r in e["runs"] if r["status"] == s)
           for s in ("SUCCESS", "PACK_MISMATCH", "NOT_SUPPORTED")})


if __name__ == "__main__":
    only = sys.argv[2:]   # e.g. "pack": regenerate that file alone
    for name, fn in (("matrix", run_matrix), ("tensor", run_tensor), ("status", run_status),
                     ("pack", run_pack)):
        if only and name not in only:
            continue
        data = {}
        fn(data)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **data)
