"""The CRT stage on the GPU: the FP64 shortcut (with its integer fallback) against the forced
integer path and the CPU oracle, on data that exercises both: dense random values (the shortcut
decides nearly everything), small integers and cancelling rows (tiny or exactly representable z:
the fallback decides), wide exponents, subnormal results, alpha / beta, both rounding modes."""
import numpy as np
import pytest

import imd_oracle as orc

pytestmark = pytest.mark.gpu


def _data(kind, m, n, k, seed):
    rng = np.random.default_rng(seed)
    if kind == "uniform":
        return rng.uniform(-1, 1, (m, k)), rng.uniform(-1, 1, (n, k))
    if kind == "integers":          # exact products: z small, every output exactly representable
        return (rng.integers(-9, 10, (m, k)).astype(np.float64),
                rng.integers(-9, 10, (n, k)).astype(np.float64))
    if kind == "cancelling":        # B's rows nearly orthogonal to A's: outputs far below the bound
        A = rng.uniform(-1, 1, (m, k))
        B = rng.uniform(-1, 1, (n, k))
        A[:, 1::2] = A[:, 0::2][:, :A[:, 1::2].shape[1]]
        B[:, 1::2] = -B[:, 0::2][:, :B[:, 1::2].shape[1]]
        B[:, 0] += np.ldexp(rng.uniform(1, 2, n), -40)
        return A, B
    if kind == "wide":
        s = lambda r: rng.choice([-1.0, 1.0], (r, k)) * np.ldexp(rng.uniform(1, 2, (r, k)),
                                                                  rng.integers(-25, 26, (r, k)))
        return s(m), s(n)
    if kind == "tiny":              # results in and around the subnormal range
        A = rng.uniform(-1, 1, (m, k)) * 2.0 ** -520
        B = rng.uniform(-1, 1, (n, k)) * 2.0 ** -520
        B[::3] *= 2.0 ** 30
        return A, B
    if kind == "powers":            # single nonzero per row: z a power of two times an odd number
        A = np.zeros((m, k))
        B = np.zeros((n, k))
        A[np.arange(m), rng.integers(0, k, m)] = np.ldexp(1.0, rng.integers(-30, 30, m))
        B[:, :] = np.ldexp(rng.integers(1, 4, (n, k)).astype(np.float64), rng.integers(-5, 5, (n, 1)))
        return A, B
    raise ValueError(kind)


def _run(A, Bt, N, alpha, beta, Cin, rounding, exact):
    import gpu_util as gu
    m, k = A.shape
    n = Bt.shape[0]
    L = gu.lib().lib
    L.imd_test_force_exact_crt(1 if exact else 0)
    try:
        out = gu.run_descs(gu.matrix_descs(m, n, k), (A, Bt, Cin.copy()), (0, 0, 0), alpha, beta, N,
                           rounding=rounding)
    finally:
        L.imd_test_force_exact_crt(0)
    return out.reshape(m, n)


@pytest.mark.parametrize("kind,m,n,k,N,rounding,alpha,beta", [
    ("uniform", 384, 520, 1000, 14, "RN", 1.0, 0.0),
    ("uniform", 200, 132, 4096, 12, "TRUNC", -0.75, 0.5),
    ("uniform", 130, 260, 700, 16, "RN", 1.0, 1.0),
    ("uniform", 64, 96, 512, 20, "RN", 2.0, 0.0),
    ("uniform", 96, 64, 300, 8, "RN", 1.0, 0.0),
    ("uniform", 40, 44, 64, 3, "RN", 1.0, 0.0),
    ("integers", 256, 256, 333, 14, "RN", 1.0, 0.0),
    ("integers", 100, 100, 50, 6, "RN", 3.0, -1.0),
    ("cancelling", 256, 260, 1024, 14, "RN", 1.0, 0.0),
    ("cancelling", 128, 128, 512, 18, "TRUNC", 1.0, 0.0),
    ("wide", 200, 200, 777, 14, "RN", 1.0, 0.0),
    ("wide", 120, 88, 400, 10, "RN", 0.5, 2.0),
    ("tiny", 128, 132, 256, 14, "RN", 1.0, 0.0),
    ("powers", 256, 128, 96, 14, "RN", 1.0, 0.0),
    ("powers", 64, 64, 40, 5, "RN", 1.0, 0.0),
])
def test_shortcut_equals_integer_path_and_oracle(kind, m, n, k, N, rounding, alpha, beta):
    A, Bt = _data(kind, m, n, k, m + n + k + N)
    Cin = np.random.default_rng(7).uniform(-1, 1, (m, n))
    fast = _run(A, Bt, N, alpha, beta, Cin, rounding, exact=False)
    exact = _run(A, Bt, N, alpha, beta, Cin, rounding, exact=True)
    assert np.array_equal(fast.view(np.uint64), exact.view(np.uint64))
    want = orc.gemm(A, Bt, N, alpha=alpha, beta=beta, Cin=Cin, rounding=rounding)
    assert np.array_equal(exact.view(np.uint64), want.view(np.uint64))
