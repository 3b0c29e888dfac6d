"""Packed operands on the CPU: the oracle's pack lowering and packed BYTES, and the host library's
pack queries, against the reference's spec/oracle.py (tests/golden/pack.npz)."""
import numpy as np
import pytest

import imd_oracle as orc
from golden_util import f64, load, same_bits, scalar
from immerdink_b200 import host

Z, MAN = load("pack")
IDS = [c["name"] for c in MAN]


def descs(case):
    return [orc.Desc(d["extent"], d["stride"], d["label"]) for d in case["desc"]]


def oracle_view(case, rec):
    X = descs(case)[rec["operand"]]
    return orc.pack_view(X, rec["contracted"], rec["batch"], rec["rows"] or None, rec["order"],
                         case["N"], case["rounding"])


def adopted_orders(case, views):
    """{post-swap class: labels} a plan adopts from the packs (views by caller operand)."""
    v0 = orc.lower(*descs(case))
    orders = {}
    for x, pv in enumerate(views):
        if pv is None:
            continue
        role = ("A", "B")[x] if not v0.swapped else ("B", "A")[x]
        for c, lst in (("K", pv.order["K"]), ("L", pv.order["L"]),
                       ("I" if role == "A" else "J", pv.order["R"])):
            orders.setdefault(c, lst)
    return orders


@pytest.mark.parametrize("case", MAN, ids=IDS)
def test_pack_lowering_and_bytes(case):
    for rec in case["packs"]:
        try:
            v = oracle_view(case, rec)
            st = "SUCCESS"
        except orc.NotSupported:
            st = "NOT_SUPPORTED"
        except orc.InvalidValue:
            st = "INVALID_VALUE"
        assert st == rec["status"]
        if st != "SUCCESS":
            continue
        assert (v.b, v.r, v.k, v.k_hat, v.format, v.pack_bytes) == (
            rec["b"], rec["r"], rec["k"], rec["k_hat"], rec["format"], rec["pack_bytes"])
        assert list(v.key) == rec["key"] and v.digest == rec["digest"]
        assert (v.order["K"], v.order["L"], v.order["R"]) == (rec["order_K"], rec["order_L"],
                                                              rec["order_R"])
        assert {n: list(v.regs[n]) for n in v.regs} == rec["regs"]
        x = rec["operand"]
        got = orc.pack(f64(Z[f"{case['key']}_{'AB'[x]}"]), case["desc"][x]["base"], v)
        assert np.array_equal(got, Z[rec["tag"]])


@pytest.mark.parametrize("case", MAN, ids=IDS)
def test_host_library_pack_queries(case):
    """imd_pack_layout and imd_pack_desc_for of the product's host library."""
    ds = [host.Desc(tuple(d["extent"]), tuple(d["stride"]), tuple(d["label"])) for d in case["desc"]]
    for rec in case["packs"]:
        x = rec["operand"]
        spec = host.PackSpec(ds[x], tuple(rec["contracted"]), tuple(rec["batch"]), tuple(rec["rows"]),
                             case["N"], case["rounding"], rec["order"])
        lay = host.pack_layout(spec, check=False)
        assert lay["status"] == rec["status"]
        if rec["status"] != "SUCCESS":
            continue
        assert (lay["b"], lay["r"], lay["k"], lay["k_hat"], lay["format"], lay["pack_bytes"]) == (
            rec["b"], rec["r"], rec["k"], rec["k_hat"], rec["format"], rec["pack_bytes"])
        assert lay["key_digest"] == rec["digest"]
        assert {n: list(lay[n]) for n in ("sig", "flag", "res")} == rec["regs"]
        if rec["order"] == "GIVEN":
            got = host.pack_desc_for(tuple(ds), operand=x, N=case["N"], rounding=case["rounding"])
            assert (list(got.contracted), list(got.batch), list(got.rows)) == (
                rec["contracted"], rec["batch"], rec["rows"])


@pytest.mark.parametrize("case", MAN, ids=IDS)
def test_packed_contraction(case):
    """A contraction through packs = the contraction in the packs' adopted canonical orders."""
    by = {(r["operand"], r["order"]): r for r in case["packs"]}
    dA, dB, dC = descs(case)
    bases = [d["base"] for d in case["desc"]]
    ds = [host.Desc(tuple(d["extent"]), tuple(d["stride"]), tuple(d["label"])) for d in case["desc"]]
    for run in case["runs"]:
        recs = [by[(x, run["order"])] if x in run["which"] else None for x in (0, 1)]
        specs = tuple(None if r is None else
                      host.PackSpec(ds[r["operand"]], tuple(r["contracted"]), tuple(r["batch"]),
                                    tuple(r["rows"]), case["N"], case["rounding"], r["order"])
                      for r in recs)
        lw = host.lowering(tuple(ds), N=case["N"], rounding=case["rounding"], packing=specs,
                           check=False)
        assert lw["status"] == run["status"]
        if run["status"] == "PACK_MISMATCH":
            assert lw["pack_mismatch"] == run["reason"]
            continue
        views = [None if r is None else oracle_view(case, r) for r in recs]
        orders = adopted_orders(case, views)
        assert orders == {g: lst for g, lst in run["orders"].items()}
        out = orc.contract_tensor(f64(Z[case["key"] + "_A"]), f64(Z[case["key"] + "_B"]),
                                  f64(Z[case["key"] + "_C"]), dA, dB, dC, scalar(case["alpha"]),
                                  scalar(case["beta"]), case["N"], case["rounding"], "EMULATE",
                                  bases[0], bases[1], bases[2], orders=orders)
        assert same_bits(out, f64(Z[run["tag"]]))
