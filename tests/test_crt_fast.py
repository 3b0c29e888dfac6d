"""The CRT kernel's floating-point shortcut against exact integer arithmetic, on the host: the
header that the CUDA kernel includes (immerdink_b200/csrc/common/crtfast.hpp) is compiled with g++
(tests/crt_fast_shim.cpp) and every value it vouches for must equal the correctly rounded
z 2^e, z the centred CRT value of the digits computed with Python integers. Inputs: random digits
(z anywhere in the range) and digits built from chosen z: ties, powers of two and their
neighbours, tiny values, values next to +-P/2, results at both ends of the normal range."""
import ctypes
import os
import subprocess
from fractions import Fraction

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODULI = [256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193, 191, 181,
          179, 173]


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    so = tmp_path_factory.mktemp("crtfast") / "crt_fast_shim.so"
    subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-shared", "-fPIC",
                    "-I" + os.path.join(ROOT, "immerdink_b200", "csrc"),
                    os.path.join(ROOT, "tests", "crt_fast_shim.cpp"), "-o", str(so)], check=True)
    lib = ctypes.CDLL(str(so))
    lib.crt_fast_batch.argtypes = [ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.crt_fast_constants.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 4
    return lib


def _run(lib, N, y, e, parts=False):
    y = np.ascontiguousarray(y, np.uint8)
    e = np.ascontiguousarray(e, np.int32)
    out, xh, xl = np.zeros(len(e)), np.zeros(len(e)), np.zeros(len(e))
    ok = np.zeros(len(e), np.uint8)
    assert lib.crt_fast_batch(N, len(e), y.ctypes.data, e.ctypes.data, out.ctypes.data,
                              ok.ctypes.data, xh.ctypes.data, xl.ctypes.data) == 0
    return (out, ok.astype(bool), xh, xl) if parts else (out, ok.astype(bool))


def _constants(N):
    p = MODULI[:N]
    P = 1
    for x in p:
        P *= x
    M = [P // x for x in p]
    return p, P, M


def _centred(y, p, P, M):
    x = sum(int(a) * b for a, b in zip(y, M)) % P
    return x if x <= P // 2 - 1 else x - P


def _digits(z, p):
    """The digits y_l = z / M_l mod p_l of a chosen centred value z."""
    _, P, M = _constants(len(p))
    return [(z % pl) * pow(Ml % pl, -1, pl) % pl for pl, Ml in zip(p, M)]


def _rounded(z, e):
    """RN-even binary64 of z 2^e (exact rational to float conversion), None outside the normals."""
    v = Fraction(z) * Fraction(2) ** e
    try:
        d = float(v)
    except OverflowError:
        return None
    return d


@pytest.mark.parametrize("N", list(range(2, 21)))
def test_random_digits(shim, N):
    p, P, M = _constants(N)
    rng = np.random.default_rng(N)
    cases = 20000
    y = np.stack([rng.integers(0, pl, cases) for pl in p], axis=1)
    e = rng.integers(-40, 41, cases)
    out, ok = _run(shim, N, y, e)
    assert ok.mean() > (0.95 if N >= 8 else 0.0)
    for c in np.flatnonzero(ok):
        z = _centred(y[c], p, P, M)
        assert out[c] == _rounded(z, int(e[c])), (N, c, z)


def _chosen_values(P, rng, count):
    H = P // 2 - 1
    B = H.bit_length()
    zs = [0, 1, -1, 2, 3, H, -H, H - 1, -(H - 1), H // 2, -(H // 2)]
    for _ in range(count):
        kind = rng.integers(0, 6)
        top = int(rng.integers(54, B)) if B > 55 else B - 1
        if kind == 0:      # exact ties: 53 random bits, a one, then zeros
            m = (int(rng.integers(1 << 52, 1 << 53)) << 1) | 1
            z = m << max(top - 54, 0)
        elif kind == 1:    # just beside a tie
            m = (int(rng.integers(1 << 52, 1 << 53)) << 1) | 1
            z = (m << max(top - 54, 0)) + int(rng.integers(-3, 4))
        elif kind == 2:    # powers of two and their neighbours
            z = (1 << int(rng.integers(0, B - 1))) + int(rng.integers(-2, 3))
        elif kind == 3:    # small values (exactly representable)
            z = int(rng.integers(0, 1 << 40))
        elif kind == 4:    # next to the ends of the range
            z = H - int(rng.integers(0, 1 << 20))
        else:              # a long run of ones: rounds up into the next binade
            z = (1 << top) - 1 - int(rng.integers(0, 4))
        z = min(max(z, 0), H)
        zs.append(z if rng.integers(0, 2) else -z)
    return zs


@pytest.mark.parametrize("N", [2, 3, 5, 7, 8, 10, 12, 13, 14, 15, 16, 17, 18, 20])
def test_chosen_values(shim, N):
    p, P, M = _constants(N)
    rng = np.random.default_rng(100 + N)
    zs = _chosen_values(P, rng, 6000)
    y = np.array([_digits(z, p) for z in zs])
    for z, row in zip(zs[:50], y[:50]):
        assert _centred(row, p, P, M) == z
    B = P.bit_length()
    # exponents: moderate ones, and ones that push the result to the ends of the normal range
    e = rng.integers(-60, 61, len(zs))
    far = rng.random(len(zs)) < 0.2
    e[far] = rng.choice([-1074 - B // 2, -1022 - B + 1, -1022 - B + 30, 1023 - B, 1024 - B, 1000 - B],
                        far.sum())
    out, ok = _run(shim, N, y, e)
    for c in np.flatnonzero(ok):
        want = _rounded(zs[c], int(e[c]))
        assert want is not None and out[c] == want, (N, zs[c], int(e[c]))
        assert abs(want) >= 2.0 ** -1022 and np.isfinite(want)


@pytest.mark.parametrize("N", list(range(2, 21)))
def test_error_bound_holds_and_is_not_wasteful(shim, N):
    """|xh + xl - z| stays below half of the plan's bound `eabs` (the bound carries a factor of two)
    on random and on extreme digits, and the bound leaves the shortcut usable: a value must exceed
    eabs 2^53 to be vouched for, which is far below typical |z| (2^-8 .. 2^-12 of P)."""
    p, P, M = _constants(N)
    eabs, Ph, Pl = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
    q = (ctypes.c_uint32 * 20)()
    assert shim.crt_fast_constants(N, ctypes.byref(eabs), ctypes.byref(Ph), ctypes.byref(Pl), q) == 0
    assert abs(Fraction(Ph.value) + Fraction(Pl.value) - P) <= Fraction(P, 1 << 105)
    assert eabs.value * 2.0 ** 53 < P * 2.0 ** -24
    rng = np.random.default_rng(N)
    cases = 6000
    y = np.stack([rng.integers(0, pl, cases) for pl in p], axis=1)
    y[:200] = np.array(p) - 1                      # largest digits: largest partial sums
    y[:200] -= rng.integers(0, 2, (200, N))
    y[200:400] = rng.integers(0, 2, (200, N))      # smallest digits
    out, ok, xh, xl = _run(shim, N, y, np.zeros(cases, np.int32), parts=True)
    worst = Fraction(0)
    for c in range(cases):
        f = sum(Fraction(int(a), pl) for a, pl in zip(y[c], p))
        f -= round(f)
        z = f * P                                   # an integer: the centred value (or +-P/2 ties)
        assert z.denominator == 1
        if abs(z) >= P // 2 - 1:
            continue
        assert int(z) == _centred(y[c], p, P, M)
        worst = max(worst, abs(Fraction(xh[c]) + Fraction(xl[c]) - z))
    assert worst <= Fraction(eabs.value) / 2, float(worst / Fraction(eabs.value))
    assert worst >= Fraction(eabs.value) / 4096     # a bound thousands of times too wide would cost coverage
