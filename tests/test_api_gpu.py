"""imd_contract's argument checks in their documented order, and call-level invariants."""
import numpy as np
import pytest
import ctypes as C

pytestmark = pytest.mark.gpu


def setup_plan(m=8, n=12, k=40, N=14, **kw):
    import gpu_util as gu
    import immerdink_b200 as imd
    descs = gu.matrix_descs(m, n, k)
    plan = imd.Plan.from_descs(*descs, N=N, **kw)
    rng = np.random.default_rng(0)
    A, B, Cc = gu.dev_f64(rng.random((m, k))), gu.dev_f64(rng.random((n, k))), gu.dev_f64(np.zeros((m, n)))
    ws = gu.Workspace(plan.workspace_bytes)
    return plan, A, B, Cc, ws


def test_check_order():
    import immerdink_b200 as imd
    plan, A, B, Cc, ws = setup_plan()
    a, b, c, w, nb = A.data_ptr(), B.data_ptr(), Cc.data_ptr(), ws.ptr, plan.workspace_bytes
    with pytest.raises(imd.InvalidValueError):
        plan.contract_ptr(1.0, a, b, 0.0, None, w, nb)
    with pytest.raises(imd.InvalidValueError):
        plan.contract_ptr(1.0, None, b, 0.0, c, w, nb)
    with pytest.raises(imd.InvalidValueError):
        plan.contract_ptr(1.0, a, b, 0.0, c, None, nb)
    with pytest.raises(imd.AliasingError):          # aliasing before alignment and size
        plan.contract_ptr(1.0, a, b, 0.0, a + 4, w, 0)
    with pytest.raises(imd.AliasingError):
        plan.contract_ptr(1.0, a, b, 0.0, c, a, nb)
    with pytest.raises(imd.MisalignedError):        # alignment before size
        plan.contract_ptr(1.0, a, b, 0.0, c, w + 8, 0)
    with pytest.raises(imd.MisalignedError):
        plan.contract_ptr(1.0, a + 4, b, 0.0, c, w, nb)
    with pytest.raises(imd.InsufficientWorkspaceError):
        plan.contract_ptr(1.0, a, b, 0.0, c, w, nb - 1)
    plan.contract_ptr(0.0, None, None, 0.0, c, w, nb)   # alpha = 0: A, B may be NULL
    plan.contract_ptr(1.0, a, a, 0.0, c, w, nb) if A.numel() == B.numel() else None  # A may alias B


def test_beta_zero_never_reads_c_and_alpha_zero_never_reads_ab():
    import torch
    import gpu_util as gu
    plan, A, B, Cc, ws = setup_plan()
    Cc.fill_(float("nan"))
    plan.contract_ptr(1.0, A.data_ptr(), B.data_ptr(), 0.0, Cc.data_ptr(), ws.ptr, plan.workspace_bytes)
    torch.cuda.synchronize()
    assert not torch.isnan(Cc).any()
    Cc.fill_(3.0)
    plan.contract_ptr(0.0, None, None, 0.5, Cc.data_ptr(), ws.ptr, plan.workspace_bytes)
    torch.cuda.synchronize()
    assert bool((Cc == 1.5).all())


def test_python_front_end_arrays_and_cache():
    import torch
    import immerdink_b200 as imd
    import imd_oracle as orc
    rng = np.random.default_rng(3)
    A, B = rng.uniform(-1, 1, (6, 5, 9)), rng.uniform(-1, 1, (9, 7))
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.empty((7, 6, 5), dtype=torch.float64, device="cuda")
    nb = imd.workspace_size("ijk,kl->lij", dA, dB, dC, N=14)
    ws = torch.empty(nb + 256, dtype=torch.uint8, device="cuda")
    off = (-ws.data_ptr()) % 256
    cache = imd.PlanCache()
    for _ in range(2):
        imd.contract("ijk,kl->lij", dA, dB, dC, N=14, workspace=ws[off:off + nb], plan_cache=cache)
    assert len(cache) == 1
    torch.cuda.synchronize()
    descs = [orc.Desc(t.shape, [s for s in t.stride()], [ord(c) for c in lab])
             for t, lab in ((dA, "ijk"), (dB, "kl"), (dC, "lij"))]
    want = orc.contract_tensor(A.reshape(-1), B.reshape(-1), np.zeros(dC.numel()), *descs, 1.0, 0.0, 14)
    assert np.array_equal(dC.cpu().numpy().reshape(-1).view(np.uint64), want.view(np.uint64))
    # a non-contiguous view (strided A) through __cuda_array_interface__
    dA2 = torch.empty((6, 5, 18), dtype=torch.float64, device="cuda")[:, :, ::2]
    dA2.copy_(dA)
    imd.contract("ijk,kl->lij", dA2, dB, dC, N=14, workspace=ws[off:off + nb], plan_cache=cache)
    torch.cuda.synchronize()
    assert len(cache) == 2
    assert np.array_equal(dC.cpu().numpy().reshape(-1).view(np.uint64), want.view(np.uint64))
    with pytest.raises(TypeError):
        imd.contract("ijk,kl->lij", dA.float(), dB, dC, N=14, workspace=ws[off:off + nb])
    with pytest.raises(imd.InsufficientWorkspaceError):
        imd.contract("ijk,kl->lij", dA, dB, dC, N=14, workspace=ws[off:off + 256])


def test_graph_capture_and_replay():
    import torch
    plan, A, B, Cc, ws = setup_plan(m=40, n=50, k=300)
    s = torch.cuda.Stream()
    args = (1.0, A.data_ptr(), B.data_ptr(), 0.0, Cc.data_ptr(), ws.ptr, plan.workspace_bytes)
    with torch.cuda.stream(s):
        plan.contract_ptr(*args, s.cuda_stream)
        s.synchronize()
        ref = Cc.clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            plan.contract_ptr(*args, torch.cuda.current_stream().cuda_stream)
        for _ in range(2):
            Cc.zero_()
            g.replay()
            s.synchronize()
            assert torch.equal(Cc.view(torch.int64), ref.view(torch.int64))
