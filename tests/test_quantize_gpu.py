"""The quantise stage on the GPU (shifts, flags, residue planes read back from the workspace):

- the FP64 shortcut of the shift rule against the forced exact integer path and the CPU oracle
  on more than a million rows (uniform, wide exponents, subnormal, huge, sparse, boundary-heavy);
- the residue planes of both operand layouts (K contiguous: fused launch; rows contiguous: scale
  launch + row tiles) against the oracle, for two- and three-word quantised integers.
"""
import numpy as np
import pytest

import imd_oracle as orc

pytestmark = pytest.mark.gpu


def _descs(m, n, k, a_rows_contiguous):
    from immerdink_b200 import host
    i, j, h = ord("i"), ord("j"), ord("h")
    a = host.Desc((m, k), (1, m), (i, h)) if a_rows_contiguous else host.Desc((m, k), (k, 1), (i, h))
    return (a, host.Desc((n, k), (k, 1), (j, h)), host.Desc((m, n), (n, 1), (i, j)))


def _rows(kind, rows, k, seed):
    rng = np.random.default_rng(seed)
    sign = rng.choice([-1.0, 1.0], (rows, k))
    u = rng.uniform(1, 2, (rows, k))
    if kind == "uniform":
        return rng.uniform(-1, 1, (rows, k))
    if kind == "wide":
        return sign * np.ldexp(u, rng.integers(-20, 21, (rows, k)))
    if kind == "subnormal":      # entries around and below the normal range
        return sign * np.ldexp(u, rng.integers(-1074, -1000, (rows, k)))
    if kind == "huge":           # largest exponents far from 0: the shortcut must stand aside
        return sign * np.ldexp(u, rng.integers(-30, 1, (rows, k)) + rng.choice([-900, 700, 1000], (rows, 1)))
    if kind == "sparse":         # mostly zeros, some rows all zero, signed zeros
        x = np.where(rng.random((rows, k)) < 0.9, 0.0, sign * u)
        x[::7] = 0.0
        x[1::7] = -0.0
        return x
    if kind == "grid":           # few distinct magnitudes: sums of squares land on round values
        return sign * np.ldexp(rng.integers(1, 4, (rows, k)).astype(np.float64), rng.integers(-2, 3, (rows, 1)))
    raise ValueError(kind)


def _shifts(A, N, rounding, rows_contiguous, exact):
    """sigma and flags of the rows of A as the device computes them (operand A of a tiny GEMM)."""
    import gpu_util as gu
    m, k = A.shape
    n = 16
    descs = _descs(m, n, k, rows_contiguous)
    Abuf = np.ascontiguousarray(A.T) if rows_contiguous else A
    Bt = np.ones((n, k))
    L = gu.lib().lib
    L.imd_test_force_exact_shift(1 if exact else 0)
    try:
        out, plan, ws = gu.run_descs(descs, (Abuf, Bt, np.zeros((m, n))), (0, 0, 0), 1.0, 0.0, N,
                                     rounding=rounding, want_ws=True)
    finally:
        L.imd_test_force_exact_shift(0)
    lay = gu.layout_of(descs, N, rounding=rounding)
    swapped = plan.lowering["swapped"]
    sig = ws.region(lay["sB" if swapped else "sA"][0], 2 * m, np.int16).copy()
    fl = ws.region(lay["fB" if swapped else "fA"][0], m, np.uint8).copy()
    plan.close()
    return sig, fl


@pytest.mark.parametrize("kind,rows,k,N,rounding", [
    ("uniform", 131072, 64, 14, "RN"),
    ("uniform", 131072, 64, 14, "TRUNC"),
    ("wide", 131072, 48, 12, "RN"),
    ("grid", 262144, 16, 14, "RN"),
    ("grid", 262144, 16, 16, "TRUNC"),
    ("subnormal", 65536, 40, 14, "RN"),
    ("huge", 65536, 40, 14, "RN"),
    ("sparse", 65536, 72, 20, "RN"),
    ("uniform", 4096, 5000, 14, "RN"),       # eight warps per row
    ("wide", 2048, 9001, 8, "RN"),           # odd k: unaligned rows, ragged last chunk
])
def test_shift_shortcut_equals_exact_path_and_oracle(kind, rows, k, N, rounding):
    A = _rows(kind, rows, k, rows + k)
    want, want_fl = orc.scale(A, N, rounding)
    for rows_contiguous in (False, True):
        fast = _shifts(A, N, rounding, rows_contiguous, exact=False)
        exact = _shifts(A, N, rounding, rows_contiguous, exact=True)
        assert np.array_equal(fast[0], exact[0]) and np.array_equal(fast[1], exact[1])
        assert np.array_equal(exact[0], want) and np.array_equal(exact[1], want_fl)


def test_shift_with_non_finite_entries():
    rng = np.random.default_rng(5)
    A = rng.uniform(-1, 1, (4096, 300))
    A[rng.integers(0, 4096, 200), rng.integers(0, 300, 200)] = np.inf
    A[rng.integers(0, 4096, 200), rng.integers(0, 300, 200)] = np.nan
    want, want_fl = orc.scale(A, 14)
    assert want_fl.any()
    for rows_contiguous in (False, True):
        sig, fl = _shifts(A, 14, "RN", rows_contiguous, exact=False)
        assert np.array_equal(sig, want) and np.array_equal(fl, want_fl)


@pytest.mark.parametrize("m,k,N,rounding,kind", [
    (300, 1000, 14, "RN", "wide"),
    (77, 520, 16, "TRUNC", "uniform"),
    (130, 333, 20, "RN", "wide"),          # three-word integers: two mma per tile
    (64, 2500, 17, "RN", "uniform"),
    (9, 40, 7, "RN", "sparse"),            # k_align 16, odd number of moduli
    (500, 264, 5, "RN", "huge"),
])
def test_residue_planes_against_oracle(m, k, N, rounding, kind):
    import gpu_util as gu
    A = _rows(kind, m, k, m * k)
    if kind == "wide":
        A[3, 5] = np.inf            # a flagged row: non-finite entries count as zero
        A[m - 1, k - 1] = np.nan
    n = 24
    Bt = _rows("uniform", n, k, 1)
    sig, _ = orc.scale(A, N, rounding)
    want = orc.residues(A, sig, N, rounding)
    for rows_contiguous in (False, True):
        for g in (0, 3 if N > 3 else 1):
            descs = _descs(m, n, k, rows_contiguous)
            Abuf = np.ascontiguousarray(A.T) if rows_contiguous else A
            out, plan, ws = gu.run_descs(descs, (Abuf, Bt, np.zeros((m, n))), (0, 0, 0), 1.0, 0.0, N,
                                         g=g, rounding=rounding, want_ws=True)
            low = plan.lowering
            lay = gu.layout_of(descs, N, g=g, rounding=rounding)
            kh = low["k_hat"]
            gg = g if g else N
            # the workspace holds the LAST residue group
            first = (N - 1) // gg * gg
            name = "RB" if low["swapped"] else "RA"
            rows_pad = low["n_hat"] if low["swapped"] else m
            R = ws.region(lay[name][0], gg * rows_pad * kh, np.int8).reshape(gg, rows_pad, kh)
            cnt = N - first
            assert np.array_equal(R[:cnt, :m, :k], want[first:]), (rows_contiguous, g)
            assert not R[:cnt, :m, k:].any() and not R[:cnt, m:, :].any()
            plan.close()
