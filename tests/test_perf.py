"""The performance model behind the reference's imd_perf_* interface: names, calibration text,
argument checks, phase structure, ranking order; kernel-independent parts against the
reference's own host library when it is built (oracle/_ref)."""
import ctypes as C
import math
import random

import pytest

import imd_oracle as orc
from immerdink_b200 import host

SPEC, EXT = "kjbc,kiac->abij", dict(a=200, b=200, c=200, i=40, j=40, k=40)


def ref_lib():
    ref = orc.ref_host()
    if ref is None:
        pytest.skip("reference host library not built")
    return host.HostLibrary(orc.REF_HOST_PATH)


def test_names_match_the_reference():
    ref = ref_lib()
    assert host.class_names() == host.class_names(ref)
    assert host.phase_names() == host.phase_names(ref)
    assert host.kernel_names() == host.kernel_names(ref)
    assert host.param_names() == host.param_names(ref)
    ours, theirs = host.load().lib, ref.lib
    for L in (ours, theirs):
        L.imd_perf_calib_error_name.restype = C.c_char_p
    assert [ours.imd_perf_calib_error_name(i) for i in range(-1, 12)] == \
           [theirs.imd_perf_calib_error_name(i) for i in range(-1, 12)]


def test_names_out_of_range_are_null():
    L = host.load().lib
    for fn, n in ((L.imd_perf_class_name, 12), (L.imd_perf_phase_name, 13), (L.imd_perf_kernel_name, 90)):
        fn.restype = C.c_char_p
        assert fn(-1) is None and fn(n) is None and fn(n - 1) is not None
    assert host.kernel_names()[14:18] == ["k5_n2_e1", "k5_n2_e2", "k5_n2_e4", "k5b_n2"]
    assert host.kernel_names()[-1] == "k5b_n20"


def test_shipped_calibration_round_trips():
    text = host.calib_format()
    cal = host.calib_parse(text)
    assert host.calib_format(cal) == text
    assert bytes(cal) == bytes(host.calib_default())          # bit for bit
    assert cal.format == 2 and cal.sm_count == 148 and b"B200" in cal.gpu
    assert 1.0 <= cal.tie_ratio <= 1.25


@pytest.mark.parametrize("edit,reason,line", [
    (lambda t: t + "bogus = 1\n", 4, None),                                   # unknown key
    (lambda t: t + "sm_count = 148\n", 5, None),                              # repeated key
    (lambda t: t.replace("sm_count = 148", "sm_count = many"), 6, None),      # value
    (lambda t: t.replace("gpu = NVIDIA B200", "gpu = " + "x" * 70), 7, None),  # too long
    (lambda t: "\n".join(l for l in t.splitlines() if not l.startswith("k5.op")) + "\n", 8, 0),
    (lambda t: t.replace("format = 2", "format = 2\nthis is not a key value line"), 3, None),
    (lambda t: t.replace("rank.tie_ratio = ", "rank.tie_ratio = 2 #"), 6, None),
    (lambda t: t.replace("band.k5 = ", "band.k5 = 2 1 #"), 6, None),
])
def test_calibration_errors(edit, reason, line):
    text = edit(host.calib_format())
    with pytest.raises(host.CalibrationError) as e:
        host.calib_parse(text)
    assert e.value.reason == reason
    if line is not None:
        assert e.value.line == line
    else:
        assert e.value.line >= 1


def test_calibration_inconsistent_and_load(tmp_path):
    text = host.calib_format().replace("rank.tie_ratio = ", "rank.tie_ratio = 1.5\n# ")
    with pytest.raises(host.CalibrationError) as e:
        host.calib_parse(text)
    assert e.value.reason == 10
    p = tmp_path / "b200.calib"
    p.write_text(host.calib_format())
    assert bytes(host.calib_load(str(p))) == bytes(host.calib_default())
    with pytest.raises(host.CalibrationError) as e:
        host.calib_load(str(tmp_path / "missing.calib"))
    assert e.value.reason == 2


def test_prediction_structure():
    p = host.predict(SPEC, EXT, N=14, g=7)
    assert p["status"] == "SUCCESS" and p["dispatch"] == "EMULATE"
    assert [q["phase"] for q in p["phases"]] == ["K0 vec", "KL A", "KL B", "K2 pack A", "K3 pack B",
                                                 "K4 gemm", "K5 crt", "call"]
    assert math.isclose(sum(q["time_s"] for q in p["phases"]), p["time_s"], rel_tol=1e-12)
    low = host.lowering(SPEC, EXT, N=14, g=7)
    assert p["kernel_launches"] == low["kernel_launches"]
    assert p["workspace_bytes"] == low["workspace_bytes"]
    assert p["flops_eq"] == 2.0 * 8000 ** 3
    assert p["time_lo_s"] <= p["time_s"] <= p["time_hi_s"]
    gemm = next(q for q in p["phases"] if q["phase"] == "K4 gemm")
    assert gemm["ops"] == 2.0 * 14 * 8000 ** 3 and gemm["launches"] == 2
    assert p["bound_s"] < p["time_s"]
    # the shipped calibration reproduces the measured benchmark within its band
    assert 6.5e-3 < p["time_s"] < 9.0e-3
    # error estimate of the configuration, as imd_err_estimate
    e = host.err_estimate(N=14, k=8000, outputs=8000 * 8000)
    assert p["err_bound"] == e["bound"] and p["err_typical"] == e["typical"]


def test_prediction_variants():
    base = host.predict(SPEC, EXT, N=14, g=7)["time_s"]
    assert host.predict(SPEC, EXT, N=14, g=14)["time_s"] < base            # one residue pass
    assert host.predict(SPEC, EXT, N=8, g=8)["time_s"] < base
    assert host.predict(SPEC, EXT, N=14, g=7, beta=True)["time_s"] >= base
    res = host.predict(SPEC, EXT, N=14, g=7, vec_mode="RESIDENT")
    assert [q["phase"] for q in res["phases"]][0] == "KL A" and res["plan_device_bytes"] > 0
    d = host.predict(SPEC, EXT, N=14, mode="DIRECT")
    assert d["dispatch"] == "DIRECT" and [q["phase"] for q in d["phases"]] == ["K0 vec", "DIRECT", "call"]
    z = host.predict(SPEC, EXT, N=14, alpha_zero=True, beta=True)
    assert [q["phase"] for q in z["phases"]] == ["K0 vec", "K5 beta-only", "call"]
    noop = host.predict("ik,kj->ij", dict(i=0, j=4, k=3), N=14)
    assert noop["dispatch"] == "NOOP" and noop["phases"] == [] and noop["time_s"] == 0
    # a packed operand drops its scale and residue phases and its workspace regions
    descs = host._descs(SPEC, EXT, None)
    ps = host.pack_desc_for(SPEC, EXT, operand=1, N=14, g=7)
    pk = host.predict(SPEC, EXT, N=14, g=7, packing=(None, ps))
    names = [q["phase"] for q in pk["phases"]]
    assert len(names) == 6 and pk["time_s"] < base and pk["workspace_bytes"] < \
        host.workspace_size(SPEC, EXT, N=14, g=7)
    pp = host.predict_pack(ps)
    assert [q["phase"] for q in pp["phases"]] == ["pack prep", "pack KL", "K2 pack A", "call"]
    assert pp["pack_bytes"] == host.pack_layout(ps)["pack_bytes"] and pp["kernel_launches"] == 3   # vectors, gaps, one fused quantise launch
    assert descs is not None


def test_plan_time_status_comes_back_zeroed():
    p = host.predict("ik,kj->ij", dict(i=4, j=4, k=2 ** 40), N=2)      # kappa >= T at N = 2
    assert p["status"] == "NOT_SUPPORTED" and p["time_s"] == 0 and p["phases"] == []
    with pytest.raises(host.ImmerdinkError):
        host.predict(SPEC, EXT, N=14, clock_mhz=-1.0)
    with pytest.raises(KeyError):
        host.predict(SPEC, EXT, N=14, regime="TURBO")


def test_struct_size_versions():
    """A caller compiled against the first version of imd_perf_t gets that prefix only."""
    L, ds, o = host._call(SPEC, EXT, None, None, host.options(14, 7))
    r = host.CPerf()
    C.memset(C.byref(r), 0xEE, C.sizeof(r))
    r.struct_size = 1648
    L.lib.imd_perf_predict.argtypes = [C.POINTER(host.CTensor)] * 3 + [
        C.POINTER(host.COptions), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(host.CPerf)]
    assert L.lib.imd_perf_predict(ds[0].t, ds[1].t, ds[2].t, o, None, None, None, C.byref(r)) == 0
    assert r.num_phases == 8 and r.regime == C.c_int32(0xEEEEEEEE).value   # beyond 1648: untouched
    r.struct_size = 100
    assert L.lib.imd_perf_predict(ds[0].t, ds[1].t, ds[2].t, o, None, None, None, C.byref(r)) == 1


def test_rank_order_and_budget():
    cands = host.rank(SPEC, EXT, N=[12, 14], g=[4, 7, 14], packs=("NONE", "A", "B", "AB"), reuse=8)
    assert len(cands) == 2 * 3 * 4 - 4        # g = 14 > N = 12 is skipped
    feas = [c for c in cands if c["feasible"]]
    assert feas == cands and all(a["time_s"] <= b["time_s"] for a, b in zip(cands, cands[1:]))
    assert [c["raw_rank"] for c in cands] == list(range(len(cands)))
    assert cands[0]["tie"] and cands[0]["packs"] == "AB"        # both operands reused 8 times
    for c in cands:
        assert c["total_bytes"] == (c["workspace_bytes"] + c["plan_device_bytes"] + c["pack_bytes"] +
                                    c["pack_ws_bytes"])
        assert math.isclose(c["time_s"], c["contract_s"] + c["pack_s"] / 8, rel_tol=1e-12)
    budget = sorted(c["total_bytes"] for c in cands)[len(cands) // 2]
    lim = host.rank(SPEC, EXT, N=[12, 14], g=[4, 7, 14], packs=("NONE", "A", "B", "AB"), reuse=8,
                    budget=budget)
    n_ok = sum(c["feasible"] for c in lim)
    assert 0 < n_ok < len(lim) and all(c["feasible"] for c in lim[:n_ok])
    assert all(c["infeasible"] == 2 and c["total_bytes"] > budget for c in lim[n_ok:])
    ties = host.rank(SPEC, EXT, N=14, g=[7, 14], order="TIES_BY_FOOTPRINT")
    tied = [c for c in ties if c["tie"]]
    assert ties[:len(tied)] == tied
    assert all(a["total_bytes"] <= b["total_bytes"] for a, b in zip(tied, tied[1:]))
    # an accuracy target makes the configurations that miss it infeasible
    acc = host._err_request("NORMWISE", 1e-13, 1.0, 1.0, 0.0, 0.0, "BOUND", 0.0)
    byacc = host.rank(SPEC, EXT, N=[10, 12, 14, 16], g=[2], accuracy=acc)
    assert {c["N"] for c in byacc if c["feasible"]} and all(
        (c["err_status"] == "MET") == c["feasible"] for c in byacc)


def test_rank_kernel_independent_fields_against_reference():
    """Same candidate set, statuses and exact footprints as the reference's ranking."""
    ref = ref_lib()
    rng = random.Random(5)
    for _ in range(25):
        e = dict(i=rng.choice([1, 3, 17, 200]), j=rng.choice([1, 5, 64, 300]), k=rng.choice([1, 2, 97, 1000]),
                 b=rng.choice([1, 2, 7]))
        spec = rng.choice(["bik,bkj->bij", "ik,kj->ij", "kib,jkb->ijb", "ik,kj->ji"])
        ext = {c: e[c] for c in set(spec) if c.isalpha()}
        kw = dict(N=[2, 9, 14, 20], g=[1, 5, 20], packs=("NONE", "A", "B", "AB"),
                  vec_modes=("GENERATE", "RESIDENT"), reuse=3)
        ours, theirs = host.rank(spec, ext, **kw), host.rank(spec, ext, lib=ref, **kw)
        key = lambda c: (c["N"], c["g"], c["vec_mode"], c["packs"])
        a, b = {key(c): c for c in ours}, {key(c): c for c in theirs}
        assert a.keys() == b.keys()
        for k_ in a:
            for f in ("status", "dispatch", "workspace_bytes", "plan_device_bytes", "pack_bytes",
                      "pack_ws_bytes", "total_bytes", "err_bound", "err_typical"):
                assert a[k_][f] == b[k_][f], (spec, ext, k_, f)
