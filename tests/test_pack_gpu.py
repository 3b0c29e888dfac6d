"""Packed operands on the GPU through the C ABI: imd_pack's bytes and imd_contract_packed's results
against the reference's spec/oracle.py (tests/golden/pack.npz), packed == in-line at sizes that
reach the tensor-core kernels, and the documented argument checks."""
import numpy as np
import pytest

from golden_util import f64, load, same_bits, scalar

pytestmark = pytest.mark.gpu

Z, MAN = load("pack")
IDS = [c["name"] for c in MAN]


def host_descs(case):
    from immerdink_b200 import host
    return tuple(host.Desc(tuple(d["extent"]), tuple(d["stride"]), tuple(d["label"]))
                 for d in case["desc"])


def pack_spec_of(case, rec, ds):
    from immerdink_b200 import host
    return host.PackSpec(ds[rec["operand"]], tuple(rec["contracted"]), tuple(rec["batch"]),
                         tuple(rec["rows"]), case["N"], case["rounding"], rec["order"])


def pack_on_device(pk, X_dev, base):
    """imd_pack into a poisoned, guarded buffer; returns (buffer object, bytes as numpy)."""
    import torch
    import gpu_util as gu
    out = gu.Workspace(pk.pack_bytes)
    ws = gu.Workspace(pk.workspace_bytes)
    pk.pack_ptr(X_dev.data_ptr() + 8 * base, out.ptr if pk.pack_bytes else None, pk.pack_bytes,
                ws.ptr if pk.workspace_bytes else None, pk.workspace_bytes, 0)
    torch.cuda.synchronize()
    assert out.guards_intact() and ws.guards_intact()
    return out, out.region(0, pk.pack_bytes, np.uint8)


@pytest.mark.parametrize("case", MAN, ids=IDS)
def test_pack_bytes_and_packed_contraction_golden(case):
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    ds = host_descs(case)
    bases = [d["base"] for d in case["desc"]]
    dev = [gu.dev_f64(f64(Z[f"{case['key']}_{x}"])) for x in "ABC"]
    packs = {}
    for rec in case["packs"]:
        spec = pack_spec_of(case, rec, ds)
        if rec["status"] != "SUCCESS":
            with pytest.raises(imd.ImmerdinkError) as e:
                imd.Pack(spec)
            assert e.value.status == rec["status"]
            continue
        pk = imd.Pack(spec)
        assert pk.pack_bytes == rec["pack_bytes"]
        x = rec["operand"]
        buf, got = pack_on_device(pk, dev[x], bases[x])
        assert np.array_equal(got, Z[rec["tag"]]), "packed bytes differ from the reference's"
        packs[(x, rec["order"])] = (pk, buf)
    for run in case["runs"]:
        sel = [packs[(x, run["order"])] if x in run["which"] else None for x in (0, 1)]
        pk = tuple(None if s is None else s[0] for s in sel)
        if run["status"] == "PACK_MISMATCH":
            with pytest.raises(imd.PackMismatchError) as e:
                imd.Plan.from_descs(*ds, N=case["N"], rounding=case["rounding"], packs=pk)
            from immerdink_b200 import host
            assert e.value.reason == host.PACK_MISMATCH[run["reason"]]
            continue
        plan = imd.Plan.from_descs(*ds, N=case["N"], rounding=case["rounding"], packs=pk)
        Cd = gu.dev_f64(f64(Z[case["key"] + "_C"]))
        ws = gu.Workspace(plan.workspace_bytes)
        packed = tuple(None if s is None else s[1].arg() for s in sel)
        plan.contract_ptr(scalar(case["alpha"]), dev[0].data_ptr() + 8 * bases[0],
                          dev[1].data_ptr() + 8 * bases[1], scalar(case["beta"]),
                          Cd.data_ptr() + 8 * bases[2], ws.ptr if plan.workspace_bytes else None,
                          plan.workspace_bytes, 0, packed=packed)
        torch.cuda.synchronize()
        assert gu.lib().lib.imd_test_device_error() == 0
        assert ws.guards_intact()
        assert same_bits(gu.host_f64(Cd), f64(Z[run["tag"]])), (run["order"], run["which"])
        plan.close()


@pytest.mark.parametrize("N,rounding,variant", [(14, "RN", 0), (18, "RN", 1), (7, "TRUNC", 2),
                                                (14, "RN", "ref")])
def test_packed_equals_inline_at_tensor_core_sizes(N, rounding, variant):
    """GIVEN packs reproduce the in-line contraction bit for bit (m, n beyond one tile, several K
    blocks, batches, rows and columns that are no multiple of 16, non-finite entries)."""
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    b, m, n, k = 2, 300, 203, 333
    rng = np.random.default_rng(N)
    A = rng.standard_normal((b, m, k)) * np.exp2(rng.integers(-8, 8, (b, m, 1)))
    B = rng.standard_normal((b, k, n))
    A[1, 7, 5] = np.inf
    B[0, 3, 11] = np.nan
    dA, dB = gu.dev_f64(A).view(b, m, k), gu.dev_f64(B).view(b, k, n)
    L = gu.lib().lib
    L.imd_test_use_reference_gemm(1 if variant == "ref" else 0)
    L.imd_test_gemm_variant(0 if variant == "ref" else variant)
    try:
        spec = "bik,bkj->bij"
        C0 = torch.zeros((b, m, n), dtype=torch.float64, device="cuda")
        plan0 = imd.Plan(spec, dA, dB, C0, N=N, rounding=rounding)
        w0 = torch.empty(plan0.workspace_bytes, dtype=torch.uint8, device="cuda")
        plan0.contract(dA, dB, C0, workspace=w0)
        for which in ((0,), (1,), (0, 1)):
            pks, bufs = [None, None], [None, None]
            for x in which:
                pks[x] = imd.Pack(plan0.pack_spec(x))
                bufs[x] = imd.PackedBuffer(torch.empty(pks[x].pack_bytes, dtype=torch.uint8, device="cuda"))
                wp = torch.empty(pks[x].workspace_bytes, dtype=torch.uint8, device="cuda")
                pks[x].pack((dA, dB)[x], bufs[x], workspace=wp)
            plan = imd.Plan(spec, dA, dB, C0, N=N, rounding=rounding, packs=tuple(pks))
            assert plan.workspace_bytes < plan0.workspace_bytes
            C1 = torch.full((b, m, n), 7.0, dtype=torch.float64, device="cuda")
            w1 = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
            plan.contract(dA, dB, C1, workspace=w1, packed=tuple(bufs))
            torch.cuda.synchronize()
            assert L.imd_test_device_error() == 0
            assert same_bits(C1.cpu().numpy(), C0.cpu().numpy()), which
            # a second call on the same packed buffers (they are only read)
            plan.contract(dA, dB, C1, alpha=2.0, beta=0.0, workspace=w1, packed=tuple(bufs))
            plan0.contract(dA, dB, C0, alpha=2.0, workspace=w0)
            torch.cuda.synchronize()
            assert same_bits(C1.cpu().numpy(), C0.cpu().numpy())
            plan0.contract(dA, dB, C0, workspace=w0)
            plan.close()
    finally:
        L.imd_test_use_reference_gemm(0)
        L.imd_test_gemm_variant(0)


def small_packed_plan():
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    m, n, k = 8, 12, 40
    rng = np.random.default_rng(1)
    A = gu.dev_f64(rng.random((m, k))).view(m, k)
    B = gu.dev_f64(rng.random((k, n))).view(k, n)
    Cc = torch.zeros((m, n), dtype=torch.float64, device="cuda")
    spec = "ik,kj->ij"
    pk = imd.Pack(imd.pack_spec(spec, A, B, Cc, operand=0, N=14))
    buf = gu.Workspace(pk.pack_bytes)
    wp = gu.Workspace(pk.workspace_bytes)
    pk.pack_ptr(A.data_ptr(), buf.ptr, pk.pack_bytes, wp.ptr, pk.workspace_bytes)
    plan = imd.Plan(spec, A, B, Cc, N=14, packs=(pk, None))
    ws = gu.Workspace(plan.workspace_bytes)
    return plan, pk, buf, A, B, Cc, ws


def test_contract_packed_check_order():
    import torch
    import immerdink_b200 as imd
    plan, pk, buf, A, B, Cc, ws = small_packed_plan()
    a, b, c, w, nb = A.data_ptr(), B.data_ptr(), Cc.data_ptr(), ws.ptr, plan.workspace_bytes
    good = (buf.arg(), None)
    L = plan.lib.lib
    # imd_contract refuses a plan with a packed slot
    assert L.imd_contract(plan._h, 1.0, a, b, 0.0, c, w, nb, 0) == 8
    # 1. slots: a pack with another key; a packed buffer for the in-line slot (the front end
    # refuses that itself, so the C check is reached with a raw operand)
    other = imd.Pack(pk.spec.with_moduli(13))
    import ctypes as ct
    from immerdink_b200 import _capi
    opA = _capi.Operand(a, buf.ptr, pk.pack_bytes, other._h)
    opB = _capi.Operand(b, None, 0, None)
    assert L.imd_contract_packed(plan._h, 1.0, ct.byref(opA), ct.byref(opB), 0.0, c, w, nb, 0) == 8
    opA = _capi.Operand(a, buf.ptr, pk.pack_bytes, pk._h)
    opB = _capi.Operand(b, buf.ptr, pk.pack_bytes, None)
    assert L.imd_contract_packed(plan._h, 1.0, ct.byref(opA), ct.byref(opB), 0.0, c, w, nb, 0) == 8
    # a second handle of the same descriptor has the same key
    twin = imd.Pack(pk.spec)
    opA = _capi.Operand(a, buf.ptr, pk.pack_bytes, twin._h)
    opB = _capi.Operand(b, None, 0, None)
    assert L.imd_contract_packed(plan._h, 1.0, ct.byref(opA), ct.byref(opB), 0.0, c, w, nb, 0) == 0
    # 2. null pointers: data is always needed; the packed buffer when it is read
    with pytest.raises(imd.InvalidValueError):
        plan.contract_ptr(1.0, None, b, 0.0, c, w, nb, packed=good)
    with pytest.raises(imd.InvalidValueError):
        plan.contract_ptr(1.0, a, b, 0.0, c, w, nb, packed=(None, None))
    plan.contract_ptr(0.0, None, None, 0.0, c, w, nb, packed=(None, None))   # alpha = 0: not read
    # 4. aliasing before alignment and sizes: C against the packed buffer, the workspace too
    with pytest.raises(imd.AliasingError):
        plan.contract_ptr(1.0, a, b, 0.0, buf.ptr + 8, w, 0, packed=good)
    with pytest.raises(imd.AliasingError):
        plan.contract_ptr(1.0, a, b, 0.0, c, buf.ptr, nb, packed=good)
    # 5. alignment of the packed buffer; 6. sizes
    with pytest.raises(imd.MisalignedError):
        plan.contract_ptr(1.0, a, b, 0.0, c, w, 0, packed=((buf.ptr + 16, pk.pack_bytes), None))
    with pytest.raises(imd.InsufficientWorkspaceError):
        plan.contract_ptr(1.0, a, b, 0.0, c, w, nb - 1, packed=good)
    with pytest.raises(imd.InsufficientWorkspaceError):
        plan.contract_ptr(1.0, a, b, 0.0, c, w, nb, packed=((buf.ptr, pk.pack_bytes - 1), None))
    torch.cuda.synchronize()
    assert ws.guards_intact() and buf.guards_intact()


def test_pack_check_order_and_empty_pack():
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    from immerdink_b200 import host
    plan, pk, buf, A, B, Cc, ws = small_packed_plan()
    a = A.data_ptr()
    wp = gu.Workspace(pk.workspace_bytes)
    out = gu.Workspace(pk.pack_bytes)
    with pytest.raises(imd.InvalidValueError):
        pk.pack_ptr(None, out.ptr, pk.pack_bytes, wp.ptr, pk.workspace_bytes)
    with pytest.raises(imd.InvalidValueError):
        pk.pack_ptr(a, out.ptr, pk.pack_bytes, None, pk.workspace_bytes)
    with pytest.raises(imd.AliasingError):          # before alignment and sizes
        pk.pack_ptr(a, a + 8, 0, wp.ptr, 0)
    with pytest.raises(imd.AliasingError):
        pk.pack_ptr(a, out.ptr, pk.pack_bytes, out.ptr, pk.workspace_bytes)
    with pytest.raises(imd.MisalignedError):
        pk.pack_ptr(a, out.ptr + 8, 0, wp.ptr, 0)
    with pytest.raises(imd.InsufficientWorkspaceError):
        pk.pack_ptr(a, out.ptr, pk.pack_bytes - 1, wp.ptr, pk.workspace_bytes)
    with pytest.raises(imd.InsufficientWorkspaceError):
        pk.pack_ptr(a, out.ptr, pk.pack_bytes, wp.ptr, pk.workspace_bytes - 1)
    torch.cuda.synchronize()
    assert out.guards_intact() and (out.region(0, pk.pack_bytes, np.uint8) == gu.POISON).all()
    # an empty pack: 0 bytes, SUCCESS with null pointers
    i, h = ord("i"), ord("h")
    empty = imd.Pack(host.PackSpec(host.Desc((0, 5), (5, 1), (i, h)), (h,), (), (), 14, "RN", "AUTO"))
    assert (empty.pack_bytes, empty.workspace_bytes) == (0, 0)
    empty.pack_ptr(None, None, 0, None, 0)


def test_packed_buffer_record():
    import torch
    import immerdink_b200 as imd
    plan, pk, buf, A, B, Cc, ws = small_packed_plan()
    raw = torch.empty(pk.pack_bytes + 256, dtype=torch.uint8, device="cuda")
    pb = imd.PackedBuffer(raw)
    w = torch.empty(max(plan.workspace_bytes, 1), dtype=torch.uint8, device="cuda")
    with pytest.raises(imd.PackMismatchError, match="no pack recorded"):
        plan.contract(A, B, Cc, workspace=w, packed=(pb, None))
    other = imd.Pack(pk.spec.with_moduli(8))
    wp = torch.empty(max(pk.workspace_bytes, other.workspace_bytes), dtype=torch.uint8, device="cuda")
    other.pack(A, pb, workspace=wp)
    with pytest.raises(imd.PackMismatchError, match="N=8, plan expects N=14"):
        plan.contract(A, B, Cc, workspace=w, packed=(pb, None))
    pk.pack(A, pb, workspace=wp)
    assert pb.last_pack == pk.record
    plan.contract(A, B, Cc, workspace=w, packed=(pb, None))
    ref = torch.zeros_like(Cc)
    imd.contract("ik,kj->ij", A, B, ref, N=14,
                 workspace=torch.empty(imd.workspace_size("ik,kj->ij", A, B, ref, N=14),
                                       dtype=torch.uint8, device="cuda"))
    torch.cuda.synchronize()
    assert same_bits(Cc.cpu().numpy(), ref.cpu().numpy())
    # a closed pack stays usable by the plans made with it
    pk.close()
    plan.contract(A, B, Cc, workspace=w, packed=(pb, None))
    with pytest.raises(ValueError):
        imd.Plan("ik,kj->ij", A, B, Cc, N=14, packs=(pk, None))


@pytest.mark.parametrize("m,n,k,N,g", [(5, 20, 131500, 5, 2), (150, 40, 700, 7, 3), (16, 300, 97, 11, 4)])
def test_packed_with_residue_groups_and_k_chunks(m, n, k, N, g):
    """A packed buffer holds all N planes; a plan with g < N reads its group's planes at an offset,
    and k beyond one int32-safe chunk adds the second chunk into the product planes."""
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    rng = np.random.default_rng(k)
    A = gu.dev_f64(rng.uniform(-1, 1, (m, k))).view(m, k)
    B = gu.dev_f64(rng.uniform(-1, 1, (k, n))).view(k, n)
    spec = "ik,kj->ij"
    C0 = torch.zeros((m, n), dtype=torch.float64, device="cuda")
    plan0 = imd.Plan(spec, A, B, C0, N=N, g=g)
    w0 = torch.empty(plan0.workspace_bytes, dtype=torch.uint8, device="cuda")
    plan0.contract(A, B, C0, workspace=w0)
    for which in ((0,), (1,), (0, 1)):
        pks, bufs = [None, None], [None, None]
        for x in which:
            pks[x] = imd.Pack(plan0.pack_spec(x))
            bufs[x] = torch.empty(pks[x].pack_bytes, dtype=torch.uint8, device="cuda")
            pks[x].pack((A, B)[x], bufs[x],
                        workspace=torch.empty(pks[x].workspace_bytes, dtype=torch.uint8, device="cuda"))
        plan = imd.Plan(spec, A, B, C0, N=N, g=g, packs=tuple(pks))
        C1 = torch.full((m, n), -1.0, dtype=torch.float64, device="cuda")
        plan.contract(A, B, C1, workspace=torch.empty(max(plan.workspace_bytes, 1), dtype=torch.uint8, device="cuda"),
                      packed=tuple(bufs))
        torch.cuda.synchronize()
        assert gu.lib().lib.imd_test_device_error() == 0
        assert same_bits(C1.cpu().numpy(), C0.cpu().numpy()), which
    import imd_oracle as orc
    want = orc.gemm(A.cpu().numpy(), B.cpu().numpy().T.copy(), N)
    assert same_bits(C0.cpu().numpy(), want)


@pytest.mark.parametrize("b,rows,k,N,pieces", [(1, 96, 200, 14, 3), (2, 40, 97, 9, 2), (1, 1000, 64, 18, 4)])
def test_pack_scatter_assembles_a_slab_from_pieces(b, rows, k, N, pieces):
    """Pieces of a slab packed one by one (each into two destinations) give exactly the bytes of
    imd_pack of the whole slab."""
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    from immerdink_b200 import host
    rng = np.random.default_rng(rows)
    X = rng.standard_normal((b, rows, k)) * np.exp2(rng.integers(-30, 30, (b, rows, 1)))
    X[0, 3, 5] = np.nan
    dX = gu.dev_f64(X).view(b, rows, k)
    lab = tuple(ord(c) for c in "bik")
    whole = host.PackSpec(host.Desc((b, rows, k), (rows * k, k, 1), lab), (ord("k"),), (ord("b"),),
                          (ord("i"),), N, "RN", "GIVEN")
    pk = imd.Pack(whole)
    want, _ = pack_on_device_np(pk, dX)
    rp = rows // pieces
    piece = imd.Pack(host.PackSpec(host.Desc((b, rp, k), (rows * k, k, 1), lab), (ord("k"),), (ord("b"),),
                                   (ord("i"),), N, "RN", "GIVEN"))
    bufs = [gu.Workspace(pk.pack_bytes) for _ in range(2)]
    ws = gu.Workspace(piece.workspace_bytes)
    for x in range(pieces):
        order = (0, 1) if x % 2 == 0 else (1, 0)     # either buffer may be "the caller's own"
        piece.scatter_ptr(dX.data_ptr() + 8 * x * rp * k, rows, x * rp, [bufs[o].ptr for o in order],
                          pk.pack_bytes, ws.ptr, piece.workspace_bytes)
    torch.cuda.synchronize()
    for buf in bufs:
        assert buf.guards_intact()
        assert np.array_equal(buf.region(0, pk.pack_bytes, np.uint8), want)
    with pytest.raises(imd.InvalidValueError):
        piece.scatter_ptr(dX.data_ptr(), rows, rows - rp + 1, [bufs[0].ptr], pk.pack_bytes, ws.ptr,
                          piece.workspace_bytes)
    with pytest.raises(imd.InsufficientWorkspaceError):
        piece.scatter_ptr(dX.data_ptr(), rows, 0, [bufs[0].ptr], pk.pack_bytes - 1, ws.ptr,
                          piece.workspace_bytes)


def pack_on_device_np(pk, X_dev):
    buf, got = pack_on_device(pk, X_dev, 0)
    return got.copy(), buf


def test_contract_packed_in_two_parts():
    """Part 1 (emulated outputs, FP64 operands not read) then part 2 (native-path outputs) write
    exactly what the whole call writes; part 1 alone leaves the flagged outputs untouched."""
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    m, n, k, N = 70, 45, 130, 10
    rng = np.random.default_rng(8)
    A, B = rng.standard_normal((m, k)), rng.standard_normal((k, n))
    A[3, 7] = np.inf
    A[50, 0] = np.nan
    B[9, 44] = -np.inf
    dA, dB = gu.dev_f64(A).view(m, k), gu.dev_f64(B).view(k, n)
    spec = "ik,kj->ij"
    C0 = torch.full((m, n), 0.5, dtype=torch.float64, device="cuda")
    plan0 = imd.Plan(spec, dA, dB, C0, N=N)
    pks = [imd.Pack(plan0.pack_spec(x)) for x in (0, 1)]
    bufs = []
    for x, pk in enumerate(pks):
        bufs.append(torch.empty(pk.pack_bytes, dtype=torch.uint8, device="cuda"))
        pk.pack((dA, dB)[x], bufs[x], workspace=torch.empty(pk.workspace_bytes, dtype=torch.uint8, device="cuda"))
    plan = imd.Plan(spec, dA, dB, C0, N=N, packs=tuple(pks))
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    plan.contract(dA, dB, C0, alpha=1.5, beta=2.0, workspace=ws, packed=tuple(bufs))
    C1 = torch.full((m, n), 0.5, dtype=torch.float64, device="cuda")
    junk = torch.full_like(dA, 123.0), torch.full_like(dB, -7.0)       # part 1 must not read these
    plan.contract(junk[0], junk[1], C1, alpha=1.5, beta=2.0, workspace=ws, packed=tuple(bufs), part=1)
    torch.cuda.synchronize()
    got = C1.cpu().numpy()
    flagged = np.zeros((m, n), bool)
    flagged[[3, 50], :] = True
    flagged[:, 44] = True
    assert (got[flagged] == 0.5).all() and same_bits(got[~flagged], C0.cpu().numpy()[~flagged])
    plan.contract(dA, dB, C1, alpha=1.5, beta=2.0, workspace=ws, packed=tuple(bufs), part=2)
    torch.cuda.synchronize()
    assert same_bits(C1.cpu().numpy(), C0.cpu().numpy())
    # group by group, then the CRT, then the native path (N = 10, g = 4: three groups)
    planG = imd.Plan(spec, dA, dB, C0, N=N, g=4, packs=tuple(pks))
    wg = torch.empty(planG.workspace_bytes, dtype=torch.uint8, device="cuda")
    C2 = torch.full((m, n), 0.5, dtype=torch.float64, device="cuda")
    for part in (16, 17, 18, 3, 2):
        planG.contract(dA, dB, C2, alpha=1.5, beta=2.0, workspace=wg, packed=tuple(bufs), part=part)
    torch.cuda.synchronize()
    assert same_bits(C2.cpu().numpy(), C0.cpu().numpy())
    for bad in (4, 15, 19, 16 + 20):
        with pytest.raises(imd.InvalidValueError):
            planG.contract(dA, dB, C2, workspace=wg, packed=tuple(bufs), part=bad)
