"""Small contractions (k <= 128, at most 256 tiles of 32 x 32 outputs) take one fused launch: its
results against the general kernel sequence and the CPU oracle, bit for bit, over the shapes,
moduli counts, rounding modes and data kinds that steer its branches; its shift and flag regions;
the lowering's launch count."""
import numpy as np
import pytest

import imd_oracle as orc
from golden_util import same_bits

pytestmark = pytest.mark.gpu


def _data(kind, rows, k, seed):
    rng = np.random.default_rng(seed)
    if kind == "uniform":
        return rng.uniform(-1, 1, (rows, k))
    if kind == "uniform01":
        return rng.uniform(0, 1, (rows, k))
    if kind == "wide":
        return rng.choice([-1.0, 1.0], (rows, k)) * np.ldexp(rng.uniform(1, 2, (rows, k)),
                                                              rng.integers(-30, 31, (rows, k)))
    if kind == "integers":
        return rng.integers(-5, 6, (rows, k)).astype(np.float64)
    if kind == "subnormal":
        return rng.choice([-1.0, 1.0], (rows, k)) * np.ldexp(rng.uniform(1, 2, (rows, k)),
                                                              rng.integers(-1074, -1040, (rows, k)))
    if kind == "flagged":
        x = rng.uniform(-1, 1, (rows, k))
        x[rng.integers(0, rows, max(rows // 8, 1)), rng.integers(0, k, max(rows // 8, 1))] = np.inf
        x[rng.integers(0, rows, max(rows // 9, 1)), rng.integers(0, k, max(rows // 9, 1))] = np.nan
        x[::5] *= 0.0
        return x
    raise ValueError(kind)


def _run(A, Bt, N, alpha, beta, Cin, rounding, small, exact_crt=False):
    import gpu_util as gu
    m, k = A.shape
    n = Bt.shape[0]
    L = gu.lib().lib
    L.imd_test_force_exact_crt(1 if exact_crt else 0)
    try:
        out = gu.run_descs(gu.matrix_descs(m, n, k), (A, Bt, Cin.copy()), (0, 0, 0), alpha, beta, N,
                           rounding=rounding, small=small)
    finally:
        L.imd_test_force_exact_crt(0)
    return out.reshape(m, n)


@pytest.mark.parametrize("m,n,k,N,rounding,kind,alpha,beta", [
    (40, 2048, 48, 14, "RN", "uniform01", 1.0, 0.0),     # the GEMM view of the first baseline configuration
    (1, 1, 2, 14, "RN", "uniform", 1.0, 0.0),
    (33, 65, 31, 14, "RN", "uniform", 1.0, 0.0),         # ragged tiles, k not a multiple of 32
    (100, 130, 128, 14, "RN", "wide", -1.5, 0.5),        # the longest rows the path takes
    (64, 64, 100, 20, "RN", "uniform", 1.0, 0.0),        # three-word integers, moduli in several passes
    (50, 70, 96, 17, "TRUNC", "wide", 1.0, 1.0),
    (31, 200, 64, 2, "RN", "uniform", 1.0, 0.0),
    (96, 96, 33, 7, "TRUNC", "uniform", 2.0, 0.0),
    (80, 120, 77, 14, "RN", "integers", 1.0, 0.0),       # exactly representable results: integer CRT
    (60, 60, 40, 12, "RN", "subnormal", 1.0, 0.0),
    (70, 90, 50, 14, "RN", "flagged", 1.0, 0.25),        # native path of non-finite rows and columns
    (128, 256, 128, 16, "RN", "uniform", 1.0, 0.0),      # 32 tiles
])
def test_fused_launch_equals_general_sequence_and_oracle(m, n, k, N, rounding, kind, alpha, beta):
    A = _data(kind, m, k, m * 7 + k)
    Bt = _data("uniform" if kind == "flagged" else kind, n, k, n * 5 + k)
    if kind == "flagged":
        Bt[3 % n, 1] = np.nan
    Cin = np.random.default_rng(3).uniform(-1, 1, (m, n))
    fused = _run(A, Bt, N, alpha, beta, Cin, rounding, small=True)
    general = _run(A, Bt, N, alpha, beta, Cin, rounding, small=False)
    assert np.array_equal(fused.view(np.uint64), general.view(np.uint64))
    want = orc.gemm(A, Bt, N, alpha=alpha, beta=beta, Cin=Cin, rounding=rounding)
    assert same_bits(fused, want)      # NaN payloads are not part of the contract
    forced = _run(A, Bt, N, alpha, beta, Cin, rounding, small=True, exact_crt=True)
    assert same_bits(forced, want)


def test_fused_launch_batched_and_strided():
    """Batches over the grid, C written through its own strides, operands gathered through theirs."""
    import torch
    import immerdink_b200 as imd
    import gpu_util as gu
    rng = np.random.default_rng(11)
    b, m, n, k = 5, 20, 30, 24
    A = rng.uniform(-1, 1, (k, b, m))            # K slowest: rows gathered with a large stride
    B = rng.uniform(-1, 1, (b, n, k))
    dA, dB = gu.dev_f64(A).view(k, b, m), gu.dev_f64(B).view(b, n, k)
    L = gu.lib().lib
    outs = []
    for small in (1, 0):
        L.imd_test_small_path(small)
        try:
            C = torch.full((m, b, n), 3.0, dtype=torch.float64, device="cuda")
            plan = imd.Plan("kbi,bjk->ibj", dA, dB, C, N=14)
            assert plan.lowering["fused"] == 1 and plan.lowering["kernel_launches"] == 2
            ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device="cuda")
            plan.contract(dA, dB, C, alpha=0.5, beta=2.0, workspace=ws)
            torch.cuda.synchronize()
            outs.append(C.cpu().numpy())
            plan.close()
        finally:
            L.imd_test_small_path(1)
    assert np.array_equal(outs[0].view(np.uint64), outs[1].view(np.uint64))
    for lam in range(b):
        want = orc.gemm(np.ascontiguousarray(A[:, lam, :].T), B[lam], 14, alpha=0.5, beta=2.0,
                        Cin=np.full((m, n), 3.0))
        assert np.array_equal(outs[0][:, lam, :].view(np.uint64), want.view(np.uint64))


def test_fused_launch_writes_shifts_and_flags():
    import gpu_util as gu
    rng = np.random.default_rng(2)
    m, n, k = 45, 100, 60
    A, Bt = _data("flagged", m, k, 1), _data("wide", n, k, 2)
    descs = gu.matrix_descs(m, n, k)
    import immerdink_b200 as imd
    import torch
    plan = imd.Plan.from_descs(*descs, N=14)
    dA, dB, dC = gu.dev_f64(A), gu.dev_f64(Bt), gu.dev_f64(np.zeros((m, n)))
    ws = gu.Workspace(plan.workspace_bytes)
    plan.contract_ptr(1.0, dA.data_ptr(), dB.data_ptr(), 0.0, dC.data_ptr(), ws.ptr, plan.workspace_bytes, 0)
    torch.cuda.synchronize()
    assert ws.guards_intact()
    lay = gu.layout_of(descs, 14)
    swapped = plan.lowering["swapped"]
    for X, rows, s_name, f_name in ((A, m, "sB" if swapped else "sA", "fB" if swapped else "fA"),
                                    (Bt, n, "sA" if swapped else "sB", "fA" if swapped else "fB")):
        want, want_fl = orc.scale(X, 14)
        sig = ws.region(lay[s_name][0], 2 * rows, np.int16)
        fl = ws.region(lay[f_name][0], rows, np.uint8)
        assert np.array_equal(sig, want) and np.array_equal(fl, want_fl)
    plan.close()


def test_lowering_counts_the_fused_launch():
    from immerdink_b200 import host
    import gpu_util as gu
    small = host.lowering(gu.matrix_descs(40, 2048, 48), N=14)
    assert small["fused"] == 1 and small["kernel_launches"] == 2
    resident = host.lowering(gu.matrix_descs(40, 2048, 48), N=14, vec_mode="RESIDENT")
    assert resident["kernel_launches"] == 1
    for m, n, k in ((40, 2048, 129), (4096, 4096, 48), (40, 2048, 1)):
        assert host.lowering(gu.matrix_descs(m, n, k), N=14)["fused"] == 0
