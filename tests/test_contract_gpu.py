"""GPU parity through the C ABI: every output bit equals the CPU oracle's / the committed
outputs of the reference specification. Stages (shifts, flags, residues, product planes) are
compared too, on a workspace poisoned with 0xA5 and fenced by guard zones."""
import numpy as np
import pytest

import imd_oracle as orc
from golden_util import f64, load, same_bits, scalar

pytestmark = pytest.mark.gpu

ZM, MANM = load("matrix")
ZT, MANT = load("tensor")


def _gpu():
    import gpu_util
    return gpu_util


@pytest.mark.parametrize("reference_gemm", [True, False], ids=["refgemm", "tcgen05"])
@pytest.mark.parametrize("case", MANM, ids=[c["name"] for c in MANM])
def test_golden_matrix(case, reference_gemm):
    gu = _gpu()
    key = case["key"]
    A, Bt = f64(ZM[key + "_A"]), f64(ZM[key + "_Bt"])
    m, k = A.shape
    n = Bt.shape[0]
    Cin = f64(ZM[key + "_C"]) if key + "_C" in ZM else np.full((m, n), np.nan)
    descs = gu.matrix_descs(m, n, k)
    N, rnd = case["N"], case["rounding"]
    out, plan, ws = gu.run_descs(descs, (A, Bt, Cin), (0, 0, 0), scalar(case["alpha"]),
                                 scalar(case["beta"]), N, rounding=rnd,
                                 reference_gemm=reference_gemm, want_ws=True)
    want = f64(ZM[key + "_out"])
    assert same_bits(out.reshape(m, n), want), (out.reshape(m, n), want)
    emulated = k >= 2 and scalar(case["alpha"]) != 0.0
    if case["traced"] and emulated:
        lay = gu.layout_of(descs, N, rounding=rnd)
        kh, nh = plan.lowering["k_hat"], plan.lowering["n_hat"]
        g = {x: ZM[key + "_" + x] for x in ("sigma", "tau", "fA", "fB", "RA", "RB", "W")}
        mm, nn = m, n
        if plan.lowering["swapped"]:  # the GEMM computes C^T: the roles of A and B are exchanged
            mm, nn = n, m
            g = dict(sigma=g["tau"], tau=g["sigma"], fA=g["fB"], fB=g["fA"], RA=g["RB"], RB=g["RA"],
                     W=g["W"].transpose(0, 2, 1))
        assert np.array_equal(ws.region(lay["sA"][0], 2 * mm, np.int16), g["sigma"])
        assert np.array_equal(ws.region(lay["sB"][0], 2 * nn, np.int16), g["tau"])
        assert np.array_equal(ws.region(lay["fA"][0], mm, np.uint8), g["fA"])
        assert np.array_equal(ws.region(lay["fB"][0], nn, np.uint8), g["fB"])
        RA = ws.region(lay["RA"][0], N * mm * kh, np.int8).reshape(N, mm, kh)
        RB = ws.region(lay["RB"][0], N * nh * kh, np.int8).reshape(N, nh, kh)
        assert np.array_equal(RA[:, :, :k], g["RA"]) and not RA[:, :, k:].any()
        assert np.array_equal(RB[:, :nn, :k], g["RB"])
        assert not RB[:, nn:, :].any() and not RB[:, :, k:].any()
        # the product planes hold the CRT digits y_l = (q_l W_l) mod p_l
        W = ws.region(lay["W"][0], N * mm * nh, np.uint8).reshape(N, mm, nh)
        q = np.array(orc.constants(N)[4], np.int64)[:, None, None]
        pm = np.array(orc.MODULI[:N], np.int64)[:, None, None]
        assert np.array_equal(W[:, :, :nn], (g["W"].astype(np.int64) * q) % pm)
    plan.close()


@pytest.mark.parametrize("case", MANT, ids=[c["name"] for c in MANT])
def test_golden_tensor(case):
    gu = _gpu()
    from immerdink_b200 import host
    key = case["key"]
    descs = [host.Desc(d["extent"], d["stride"], d["label"]) for d in case["desc"]]
    bases = [d["base"] for d in case["desc"]]
    bufs = [f64(ZT[f"{key}_{x}"]) for x in "ABC"]
    out = gu.run_descs(descs, bufs, bases, scalar(case["alpha"]), scalar(case["beta"]), case["N"],
                       rounding=case["rounding"], mode=case["mode"])
    assert same_bits(out, f64(ZT[key + "_out"]))
    # the resident-vector variant and a small residue group give the same bits
    out2 = gu.run_descs(descs, bufs, bases, scalar(case["alpha"]), scalar(case["beta"]), case["N"],
                        g=min(3, case["N"]), rounding=case["rounding"], mode=case["mode"],
                        vec_mode="RESIDENT")
    assert same_bits(out2, out)


def _random_case(seed, m, n, k, kind):
    rng = np.random.default_rng(seed)
    if kind == "uniform":
        A, Bt = rng.uniform(-1, 1, (m, k)), rng.uniform(-1, 1, (n, k))
    elif kind == "wide":
        A = rng.choice([-1.0, 1.0], (m, k)) * np.ldexp(rng.uniform(1, 2, (m, k)), rng.integers(-20, 21, (m, k)))
        Bt = rng.choice([-1.0, 1.0], (n, k)) * np.ldexp(rng.uniform(1, 2, (n, k)), rng.integers(-20, 21, (n, k)))
    else:  # bimodal
        A = rng.choice([-1.0, 1.0], (m, k)) * np.where(rng.random((m, k)) < 0.5, 1.0, 1e-8) * rng.uniform(1, 2, (m, k))
        Bt = rng.choice([-1.0, 1.0], (n, k)) * np.where(rng.random((n, k)) < 0.5, 1.0, 1e-8) * rng.uniform(1, 2, (n, k))
    return A, Bt, rng.uniform(-1, 1, (m, n))


@pytest.mark.parametrize("m,n,k,N,kind,alpha,beta", [
    (130, 270, 200, 14, "uniform", 1.0, 0.0),      # more than one tile in both directions
    (257, 515, 1000, 14, "wide", 1.5, 0.5),        # ragged tiles, K tail inside a 128-byte block
    (64, 48, 4100, 16, "bimodal", 1.0, 0.0),       # 5 limbs in the CRT
    (300, 300, 333, 8, "uniform", -1.0, 1.0),
    (129, 17, 97, 20, "wide", 1.0, 0.0),           # 3-word residues, k_align 64
    (31, 1000, 96, 12, "uniform", 1.0, 0.0),       # k_align 16
    (1, 700, 512, 14, "uniform", 1.0, 0.0),
    (700, 1, 512, 2, "uniform", 1.0, 0.0),
])
def test_random_against_oracle(m, n, k, N, kind, alpha, beta):
    gu = _gpu()
    A, Bt, Cin = _random_case(m * 7 + n, m, n, k, kind)
    descs = gu.matrix_descs(m, n, k)
    want = orc.gemm(A, Bt, N, alpha, beta, Cin)
    outs = []
    for g in (0, 5 if N > 5 else 1):
        out = gu.run_descs(descs, (A, Bt, Cin), (0, 0, 0), alpha, beta, N, g=g)
        assert same_bits(out.reshape(m, n), want)
        outs.append(out)
    ref = gu.run_descs(descs, (A, Bt, Cin), (0, 0, 0), alpha, beta, N, reference_gemm=True)
    assert same_bits(ref, outs[0])
    for variant in (1, 2):   # one CTA per tile / CTA pairs, whatever the shape rule would pick
        out = gu.run_descs(descs, (A, Bt, Cin), (0, 0, 0), alpha, beta, N, gemm_variant=variant)
        assert same_bits(out, outs[0])


def test_k_chunks_carry_mod_p():
    """k beyond one int32-safe chunk: the second chunk adds into the u8 planes mod p."""
    gu = _gpu()
    m, n, k, N = 5, 20, 131500, 5
    A, Bt, _ = _random_case(3, m, n, k, "uniform")
    descs = gu.matrix_descs(m, n, k)
    want = orc.gemm(A, Bt, N, 1.0, 0.0, None, "TRUNC")
    for refg, variant in ((True, 0), (False, 1), (False, 2)):
        out = gu.run_descs(descs, (A, Bt, np.zeros((m, n))), (0, 0, 0), 1.0, 0.0, N,
                           rounding="TRUNC", reference_gemm=refg, gemm_variant=variant)
        assert same_bits(out.reshape(m, n), want)


def test_baseline_config_1_in_full():
    """'ijk,kl->lij', A (64,32,48), B (48,40), uniform [0,1), N = 14: every output bit."""
    gu = _gpu()
    from immerdink_b200 import host
    rng = np.random.default_rng(1)
    A, B = rng.random(64 * 32 * 48), rng.random(48 * 40)
    Cb = np.full(40 * 64 * 32, np.nan)
    descs = host.contraction("ijk,kl->lij", dict(i=64, j=32, k=48, l=40))
    out = gu.run_descs(descs, (A, B, Cb), (0, 0, 0), 1.0, 0.0, 14)
    od = [orc.Desc(d.extent, d.stride, d.label) for d in descs]
    want = orc.contract_tensor(A, B, Cb, od[0], od[1], od[2], 1.0, 0.0, 14)
    assert same_bits(out, want)


def test_north_star_shape_scaled_down():
    """'kjbc,kiac->abij' with small extents: the whole C against the oracle."""
    gu = _gpu()
    from immerdink_b200 import host
    ext = dict(a=20, b=18, c=24, i=6, j=7, k=5)
    descs = host.contraction("kjbc,kiac->abij", ext)
    rng = np.random.default_rng(2)
    sizes = [int(np.prod(d.extent)) for d in descs]
    A, B = rng.uniform(-1, 1, sizes[0]), rng.uniform(-1, 1, sizes[1])
    Cb = np.full(sizes[2], np.nan)
    out = gu.run_descs(descs, (A, B, Cb), (0, 0, 0), 1.0, 0.0, 14, g=7)
    od = [orc.Desc(d.extent, d.stride, d.label) for d in descs]
    want = orc.contract_tensor(A, B, Cb, od[0], od[1], od[2], 1.0, 0.0, 14)
    assert same_bits(out, want)
