"""libimmerdink_host.so: lowering, legality and exact sizes.

Checked against (a) the committed outputs of the reference's specification (tests/golden),
(b) the reference's own host library compiled from its sources (oracle/_ref, when present) on
seeded random descriptors, for every field that does not depend on the kernels, and (c) the
reference's published worked examples of the workspace formula."""
import ctypes as C
import os
import random

import pytest

import imd_oracle as orc
from golden_util import load
from immerdink_b200 import build, host

build.build_host()
LIB = host.load()
Z, MAN = load("tensor")
ZS, MANS = load("status")


def desc_tuple(d):
    return host.Desc(d["extent"], d["stride"], d["label"])


def test_exports_every_host_symbol():
    for name in host.HOST_SYMBOLS:
        assert hasattr(LIB.lib, name), name
    assert LIB.version == 13


@pytest.mark.parametrize("case", MAN, ids=[c["name"] for c in MAN])
def test_lowering_matches_reference_spec(case):
    ds = [desc_tuple(d) for d in case["desc"]]
    low = host.lowering(ds, N=case["N"], mode=case["mode"], rounding=case["rounding"])
    assert (low["m"], low["n"], low["k"], low["b"], bool(low["swapped"])) == (
        case["m"], case["n"], case["k"], case["b"], case["swapped"])
    kind = {"NOOP": "NOOP", "SCALE": "SCALE", "DIRECT": "DIRECT", "GEMM": "EMULATE"}[case["kind"]]
    if case["k"] == 0 and kind != "NOOP":
        kind = "SCALE"
    assert low["dispatch"] == kind
    assert low["status"] == "SUCCESS"


@pytest.mark.parametrize("case", MANS, ids=[c["name"] for c in MANS])
def test_status_matches_reference_spec(case):
    ds = [desc_tuple(d) for d in case["desc"]]
    low = host.lowering(ds, N=14, check=False)
    assert low["status"] == case["status"]


def test_worked_examples_of_the_workspace_formula():
    # north-star contraction, N = 14, g = 7 (reference README.md:32)
    spec, ext = "kjbc,kiac->abij", dict(a=200, b=200, c=200, i=40, j=40, k=40)
    assert host.workspace_size(spec, ext, N=14, g=7) == 1792432896
    # 8192^3, N = 14, g = 14 (reference docs/MEMORY_MODEL.md:95)
    assert host.workspace_size("ik,kj->ij", dict(i=8192, j=8192, k=8192), N=14) == 2819014912
    low = host.lowering(spec, ext, N=14, g=7)
    assert (low["m"], low["n"], low["k"], low["b"]) == (8000, 8000, 8000, 1)
    assert low["swapped"] == 1 and low["k_align"] == 64 and low["num_groups"] == 2


def test_monotone_footprint():
    spec, ext = "abcd,cdij->abij", dict(a=12, b=12, c=12, d=12, i=5, j=5)
    prev = 0
    for N in range(2, 21):
        cur = host.workspace_size(spec, ext, N=N, g=1)
        assert cur >= prev
        prev = cur
    tr = host.g_tradeoff(spec, ext, N=14)
    assert all(tr[g] <= tr[g + 1] for g in range(1, 14))


def test_rn_acceptance_is_last_and_only_in_plan_queries():
    # N = 2: T = 180; k = 180^2 gives kappa = 180 >= T
    spec, ext = "ik,kj->ij", dict(i=2, j=2, k=180 * 180)
    assert host.workspace_size(spec, ext, N=2) > 0
    with pytest.raises(host.ImmerdinkError) as e:
        host.plan_bytes(spec, ext, N=2)
    assert e.value.status == "NOT_SUPPORTED"
    assert host.plan_bytes(spec, ext, N=2, rounding="TRUNC")[0] == 0
    assert host.plan_bytes(spec, dict(i=2, j=2, k=179 * 179), N=2)[0] == 0
    assert host.lowering(spec, ext, N=2, check=False)["lowered"] == 1


def test_option_validation():
    spec, ext = "ik,kj->ij", dict(i=2, j=2, k=4)
    for bad in (dict(N=1), dict(N=21), dict(N=5, g=6), dict(N=5, g=-1)):
        with pytest.raises(host.ImmerdinkError) as e:
            host.workspace_size(spec, ext, **bad)
        assert e.value.status == "INVALID_VALUE"
    out = host.CLowering()
    out.struct_size = 100
    ds = [host.CDesc(d) for d in host.contraction(spec, ext)]
    assert LIB.lib.imd_lowering(ds[0].t, ds[1].t, ds[2].t, host.options(5), C.byref(out)) == 1


def test_struct_size_versions_write_only_what_fits():
    spec, ext = "ik,kj->ij", dict(i=20, j=30, k=200)
    ds = [host.CDesc(d) for d in host.contraction(spec, ext)]
    for size in (136, 152, 168, 176, 184, 192):
        out = host.CLowering()
        C.memset(C.byref(out), 0xEE, C.sizeof(out))
        out.struct_size = size
        if size >= 168:
            out.sm_count = 0
        assert LIB.lib.imd_lowering(ds[0].t, ds[1].t, ds[2].t, host.options(14), C.byref(out)) == 0
        raw = bytes(out)
        assert all(b == 0xEE for b in raw[size:])
        assert out.k == 200 and out.k_hat == 256


REF = orc.ref_host()


def random_descs(rng):
    labels = list(range(10, 17))
    ra, rb = rng.randint(0, 4), rng.randint(0, 4)
    la = [rng.choice(labels) for _ in range(ra)]
    lb = [rng.choice(labels) for _ in range(rb)]
    pool = sorted(set(la) | set(lb))
    lc = [x for x in pool if rng.random() < 0.6]
    if rng.random() < 0.1:
        lc.append(rng.choice(labels))
    rng.shuffle(lc)
    ext = {x: rng.choice((0, 1, 1, 2, 3, 4, 5, 7, 130)) if rng.random() < 0.9 else rng.choice((2**31, 2**20))
           for x in labels}
    out = []
    for lab in (la, lb, lc):
        e = [ext[x] for x in lab]
        if rng.random() < 0.05 and e:
            e[0] += 1
        order = list(range(len(lab)))
        rng.shuffle(order)
        st = [0] * len(lab)
        acc = 1
        for d in order:
            st[d] = acc * rng.choice((1, 1, 1, 2)) * rng.choice((1, 1, 1, -1))
            acc = abs(st[d]) * max(e[d], 1)
            if rng.random() < 0.03:
                st[d] = 0
        out.append(host.Desc(e, st, lab))
    return out


@pytest.mark.skipif(REF is None, reason="reference host library not built here")
def test_against_reference_host_library_on_random_descriptors():
    rng = random.Random(4)
    same = ("status", "lowered", "dispatch", "swapped", "num_moduli", "residue_group", "num_groups",
            "m", "n", "k", "b", "n_hat", "k_hat", "vec_entries", "kappa", "workspace_bytes",
            "plan_device_bytes", "k_align")
    seen = {}
    for it in range(3000):
        ds = random_descs(rng)
        N = rng.randint(2, 20)
        o = host.options(N, rng.randint(0, N), rng.choice(("RN", "TRUNC")),
                         rng.choice(("EMULATE", "EMULATE", "DIRECT")),
                         rng.choice(("GENERATE", "RESIDENT")))
        cd = [host.CDesc(d) for d in ds]
        mine, ref = host.CLowering(), host.CLowering()
        mine.struct_size = ref.struct_size = 192
        s1 = LIB.lib.imd_lowering(cd[0].t, cd[1].t, cd[2].t, o, C.byref(mine))
        s2 = REF.imd_lowering(C.byref(cd[0].t), C.byref(cd[1].t), C.byref(cd[2].t), C.byref(o),
                              C.byref(ref))
        assert s1 == s2, (it, ds, s1, s2)
        seen[s1] = seen.get(s1, 0) + 1
        for f in same:
            assert getattr(mine, f) == getattr(ref, f), (it, f, ds, getattr(mine, f), getattr(ref, f))
        # workspace size and layout
        b1, b2 = C.c_size_t(0), C.c_size_t(0)
        w1 = LIB.lib.imd_workspace_size(cd[0].t, cd[1].t, cd[2].t, o, C.byref(b1))
        w2 = REF.imd_workspace_size(C.byref(cd[0].t), C.byref(cd[1].t), C.byref(cd[2].t),
                                    C.byref(o), C.byref(b2))
        assert (w1, b1.value) == (w2, b2.value)
        if w1 == 0:
            r1, r2 = (host.CRegion * 8)(), (host.CRegion * 8)()
            LIB.lib.imd_workspace_layout(cd[0].t, cd[1].t, cd[2].t, o, r1, 8, None, None)
            REF.imd_workspace_layout(C.byref(cd[0].t), C.byref(cd[1].t), C.byref(cd[2].t),
                                     C.byref(o), r2, 8, None, None)
            assert [(r.offset, r.bytes) for r in r1] == [(r.offset, r.bytes) for r in r2]
    assert seen.get(0, 0) > 300 and seen.get(1, 0) > 50 and seen.get(2, 0) > 50, seen


@pytest.mark.skipif(REF is None, reason="reference host library not built here")
def test_error_estimates_against_reference_host_library():
    REF.imd_err_estimate.argtypes = LIB.lib.imd_err_estimate.argtypes
    rng = random.Random(5)
    for _ in range(400):
        N, k = rng.randint(2, 20), rng.choice((1, 2, 48, 8000, 14400, 16384, 10**6, 2**40))
        metric = rng.choice(list(host.ERR_METRICS))
        req = host._err_request(metric, rng.choice((0.0, 1e-15, 1e-10)), rng.uniform(1, 100),
                                rng.uniform(0.1, 10), rng.choice((0.0, 1.5, 40.0)),
                                rng.choice((0.0, 3.0)), rng.choice(("BOUND", "TYPICAL")),
                                rng.choice((0.0, 1e-6)))
        a, b = host.CErr(), host.CErr()
        a.struct_size = b.struct_size = 72
        args = (N, rng.randint(0, 1), rng.randint(0, 3), k, rng.choice((1, 10**6)))
        s1 = LIB.lib.imd_err_estimate(*args, C.byref(req), C.byref(a))
        s2 = REF.imd_err_estimate(*args, C.byref(req), C.byref(b))
        assert s1 == s2 == 0
        assert a.err_status == b.err_status
        for f in ("bound", "typical", "unit_bound", "unit_typical"):
            x, y = getattr(a, f), getattr(b, f)
            assert x == y or abs(x - y) <= 1e-12 * abs(y), (f, x, y)


def test_published_error_bounds():
    # normwise bounds quoted for the reference host library (N = 14)
    for k, want in ((48, 6.3e-16), (8000, 6.75e-15), (14400, 9.0e-15), (16384, 9.6e-15)):
        got = host.err_estimate(N=14, k=k)["bound"]
        assert abs(got - want) / want < 0.02, (k, got)
    assert abs(host.err_estimate(N=12, k=16384)["bound"] - 1.95e-12) / 1.95e-12 < 0.02
    assert abs(host.err_estimate(N=16, k=16384)["bound"] - 1.6e-16) / 1.6e-16 < 0.05


# ---------------------------------------------------------------------------- packed operands
def _pack_queries(lib_call_desc_for, lib_call_layout, lib_call_lowering, cd, o, ds, rng):
    """desc_for, layout and packed lowering through one library; returns a comparable record."""
    rec = []
    specs = []
    for operand in (0, 1):
        out = host.CPackDesc()
        out.struct_size = C.sizeof(host.CPackDesc)
        cap = max(len(ds[operand].label), 1)
        labels = (C.c_int32 * cap)()
        st = lib_call_desc_for(cd, o, operand, out, labels, cap)
        lists = None
        if st == 0:
            lists = tuple(tuple(ptr[i] for i in range(n)) for ptr, n in
                          ((out.contracted, out.num_contracted), (out.batch, out.num_batch),
                           (out.rows, out.num_rows)))
        rec.append(("desc_for", operand, st, lists))
        specs.append(lists)
    return rec, specs


def _layout_record(libcall, spec):
    cs = host.CPackSpec(spec)
    out = host.CPackLayout()
    out.struct_size = C.sizeof(host.CPackLayout)
    st = libcall(C.byref(cs.d), C.byref(out))
    fields = [getattr(out, f) for f in ("status", "format", "num_moduli", "rounding", "b", "r", "k",
                                        "k_hat", "kappa", "pack_bytes", "pack_ws_bytes", "key_digest")]
    regs = [(r.offset, r.bytes) for r in (out.sig, out.flag, out.res)]
    return st, fields, regs


@pytest.mark.skipif(REF is None, reason="reference host library not built here")
def test_packed_queries_against_reference_host_library():
    rng = random.Random(9)
    same = ("status", "lowered", "dispatch", "swapped", "num_moduli", "residue_group", "num_groups",
            "m", "n", "k", "b", "n_hat", "k_hat", "vec_entries", "kappa", "workspace_bytes",
            "plan_device_bytes", "k_align", "packed", "pack_mismatch")
    T, O = C.POINTER(host.CTensor), C.POINTER(host.COptions)
    for L in (LIB.lib, REF):
        L.imd_pack_desc_for.argtypes = [T, T, T, O, C.c_int32, C.POINTER(host.CPackDesc),
                                        C.POINTER(C.c_int32), C.c_int32]
        L.imd_pack_layout.argtypes = [C.POINTER(host.CPackDesc), C.POINTER(host.CPackLayout)]
        L.imd_lowering_packed.argtypes = [T, T, T, O, C.POINTER(host.CPacking), C.POINTER(host.CLowering)]
        L.imd_workspace_size_packed.argtypes = [T, T, T, O, C.POINTER(host.CPacking), C.POINTER(C.c_size_t)]
    statuses = {}
    checked = 0
    for it in range(1500):
        ds = random_descs(rng)
        N = rng.randint(2, 20)
        rounding = rng.choice(("RN", "TRUNC"))
        o = host.options(N, rng.randint(0, N), rounding, rng.choice(("EMULATE", "EMULATE", "DIRECT")))
        cd = [host.CDesc(d) for d in ds]
        specs = {}
        for name, L in (("mine", LIB.lib), ("ref", REF)):
            got = []
            for operand in (0, 1):
                out = host.CPackDesc()
                out.struct_size = C.sizeof(host.CPackDesc)
                cap = max(len(ds[operand].label), 1)
                labels = (C.c_int32 * cap)()
                st = L.imd_pack_desc_for(cd[0].t, cd[1].t, cd[2].t, o, operand, C.byref(out), labels, cap)
                lists = None
                if st == 0:
                    lists = tuple(tuple(ptr[i] for i in range(n)) for ptr, n in
                                  ((out.contracted, out.num_contracted), (out.batch, out.num_batch),
                                   (out.rows, out.num_rows)))
                got.append((st, lists))
            specs[name] = got
        assert specs["mine"] == specs["ref"], (it, ds, specs)
        if specs["mine"][0][0] != 0:
            continue
        # pack specs: the plan's own (GIVEN), AUTO variants, and deliberately wrong ones
        given = [host.PackSpec(ds[x], *specs["mine"][x][1], N, rounding, "GIVEN") for x in (0, 1)]
        variants = []
        for x in (0, 1):
            k, l, r = specs["mine"][x][1]
            variants.append([given[x],
                             host.PackSpec(ds[x], k, l, (), N, rounding, "AUTO"),
                             host.PackSpec(ds[x], k, l, (), max(2, (N + 1) % 21), rounding, "AUTO"),
                             host.PackSpec(ds[x], k, l, (), N, "TRUNC" if rounding == "RN" else "RN", "AUTO"),
                             host.PackSpec(host.Desc(ds[x].extent, [s * 2 for s in ds[x].stride], ds[x].label),
                                           k, l, (), N, rounding, "AUTO"),
                             host.PackSpec(ds[x], tuple(reversed(k)), l, r, N, rounding, "GIVEN")])
        for x in (0, 1):
            for ps in variants[x]:
                a = _layout_record(LIB.lib.imd_pack_layout, ps)
                b = _layout_record(REF.imd_pack_layout, ps)
                assert a == b, (it, ps, a, b)
        for trial in range(6):
            pa = rng.choice(variants[0] + [None])
            pb = rng.choice(variants[1] + [None])
            if pa is None and pb is None:
                continue
            cp, keep = host._packing((pa, pb))
            mine, ref = host.CLowering(), host.CLowering()
            mine.struct_size = ref.struct_size = 192
            s1 = LIB.lib.imd_lowering_packed(cd[0].t, cd[1].t, cd[2].t, o, C.byref(cp), C.byref(mine))
            s2 = REF.imd_lowering_packed(cd[0].t, cd[1].t, cd[2].t, o, C.byref(cp), C.byref(ref))
            assert s1 == s2, (it, ds, pa, pb, s1, s2, mine.pack_mismatch, ref.pack_mismatch)
            for f in same:
                assert getattr(mine, f) == getattr(ref, f), (it, f, pa, pb, getattr(mine, f), getattr(ref, f))
            b1, b2 = C.c_size_t(0), C.c_size_t(0)
            w1 = LIB.lib.imd_workspace_size_packed(cd[0].t, cd[1].t, cd[2].t, o, C.byref(cp), C.byref(b1))
            w2 = REF.imd_workspace_size_packed(cd[0].t, cd[1].t, cd[2].t, o, C.byref(cp), C.byref(b2))
            assert (w1, b1.value if w1 == 0 else 0) == (w2, b2.value if w2 == 0 else 0)
            statuses[(s1, mine.pack_mismatch)] = statuses.get((s1, mine.pack_mismatch), 0) + 1
            checked += 1
    assert checked > 1000 and statuses.get((0, 0), 0) > 100 and len(statuses) >= 5, statuses
