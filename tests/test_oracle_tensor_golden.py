"""The oracle's lowering and tensor front end against the reference's spec/oracle.py
(tests/golden/tensor.npz): GEMM view, canonical orders, scatter vectors and the whole C buffer."""
import numpy as np
import pytest

import imd_oracle as orc
from golden_util import f64, load, same_bits, scalar

Z, MAN = load("tensor")
ZS, MANS = load("status")


def descs(case):
    return [orc.Desc(d["extent"], d["stride"], d["label"]) for d in case["desc"]]


@pytest.mark.parametrize("case", MAN, ids=[c["name"] for c in MAN])
def test_tensor_case(case):
    key = case["key"]
    dA, dB, dC = descs(case)
    v = orc.lower(dA, dB, dC, case["mode"])
    assert (v.m, v.n, v.k, v.b, v.swapped) == (case["m"], case["n"], case["k"], case["b"],
                                               case["swapped"])
    for g in "IJKL":
        assert v.order[g] == case["order"][g]
        assert [[e, [st["A"], st["B"], st["C"]]] for e, st in v.fused[g]] == case["fused"][g]
    if key + "_vec" in Z:
        names = ("A_row", "A_k", "A_bat", "B_k", "B_col", "B_bat", "C_row", "C_col", "C_bat")
        got = np.concatenate([orc.vec(v, nm) for nm in names])
        assert np.array_equal(got, Z[key + "_vec"])
    bases = [d["base"] for d in case["desc"]]
    for literal in (True, False):
        out = orc.contract_tensor(f64(Z[key + "_A"]), f64(Z[key + "_B"]), f64(Z[key + "_C"]),
                                  dA, dB, dC, scalar(case["alpha"]), scalar(case["beta"]),
                                  case["N"], case["rounding"], case["mode"], bases[0], bases[1],
                                  bases[2], literal=literal)
        assert same_bits(out, f64(Z[key + "_out"]))


@pytest.mark.parametrize("case", MANS, ids=[c["name"] for c in MANS])
def test_status_case(case):
    dA, dB, dC = descs(case)
    try:
        orc.lower(dA, dB, dC)
        st = "SUCCESS"
    except orc.NotSupported:
        st = "NOT_SUPPORTED"
    except orc.InvalidValue:
        st = "INVALID_VALUE"
    assert st == case["status"]
