"""The shipped B200 calibration against live phase times (CUDA events of the library's phase
marks): whole calls within +-25 %, the GEMM phase within +-15 % on shapes the model was not
fitted on."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("b,m,n,k,N,g", [(1, 5000, 5000, 5000, 14, 7), (1, 3072, 6144, 7000, 16, 8),
                                         (3, 2048, 2048, 2500, 10, 5)])
def test_prediction_matches_measurement(b, m, n, k, N, g):
    import torch
    import immerdink_b200 as imd
    from immerdink_b200 import host
    spec = "bik,bkj->bij"
    A = torch.rand((b, m, k), dtype=torch.float64, device="cuda") * 2 - 1
    B = torch.rand((b, k, n), dtype=torch.float64, device="cuda") * 2 - 1
    Cd = torch.empty((b, m, n), dtype=torch.float64, device="cuda")
    plan = imd.Plan(spec, A, B, Cd, N=N, g=g)
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    L = imd.load_library().lib
    for _ in range(3):
        plan.contract(A, B, Cd, workspace=ws)
    steps = 5
    L.imd_prof_enable(64 * (steps + 1))
    torch.cuda.synchronize()
    for _ in range(steps):
        plan.contract(A, B, Cd, workspace=ws)
    torch.cuda.synchronize()
    ph = (C.c_float * 8)()
    L.imd_prof_read(ph, 8)
    L.imd_prof_enable(0)
    measured = sum(ph[1:5]) / steps * 1e-3
    pred = host.predict(spec, dict(b=b, i=m, j=n, k=k), N=N, g=g)
    assert pred["status"] == "SUCCESS"
    assert 0.75 < measured / pred["time_s"] < 1.25, (measured, pred["time_s"])
    gemm = next(q for q in pred["phases"] if q["phase"] == "K4 gemm")
    launch = next(q for q in pred["phases"] if q["phase"] == "call")["time_s"] / pred["kernel_launches"]
    assert 0.85 < (ph[3] / steps * 1e-3) / (gemm["time_s"] + gemm["launches"] * launch) < 1.15
