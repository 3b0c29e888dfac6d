"""imd_contract_builtin_ws: the entry point for callers that cannot allocate device memory (a
plugin inside a host application with a closed memory pool, a latency-critical step that must not
call into the driver's allocator). It must give the bits of imd_contract while using only the
library's fixed built-in workspace; called twice in a row because the array keeps the previous
call's contents. Collected last on purpose, so a run that stops at the first failure has already
run everything else."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call_builtin(lib, plan, alpha, A, B, beta, Cc, stream=0):
    f = lib.imd_contract_builtin_ws
    f.restype = C.c_int
    f.argtypes = [C.c_void_p, C.c_double, C.c_void_p, C.c_void_p, C.c_double, C.c_void_p, C.c_void_p]
    return f(plan._h, alpha, A.data_ptr(), B.data_ptr(), beta, Cc.data_ptr(), stream)


@pytest.mark.parametrize("m,n,k,N,alpha,beta", [(200, 300, 700, 14, 1.0, 0.0), (64, 80, 100, 16, -1.5, 0.5)])
def test_builtin_workspace_matches_imd_contract_twice(m, n, k, N, alpha, beta):
    import torch
    import gpu_util as gu
    import immerdink_b200 as imd
    lib = imd.load_library().lib
    rng = np.random.default_rng(m + n)
    A, Bt, C0 = rng.uniform(-1, 1, (m, k)), rng.uniform(-1, 1, (n, k)), rng.uniform(-1, 1, (m, n))
    descs = gu.matrix_descs(m, n, k)
    plan = imd.Plan.from_descs(*descs, N=N)
    assert plan.workspace_bytes <= (32 << 20)
    dA, dB = gu.dev_f64(A), gu.dev_f64(Bt)
    # the existing entry point, caller-owned workspace
    ws = gu.Workspace(plan.workspace_bytes)
    ref = gu.dev_f64(C0)
    plan.contract_ptr(alpha, dA.data_ptr(), dB.data_ptr(), beta, ref.data_ptr(), ws.ptr, plan.workspace_bytes)
    torch.cuda.synchronize()
    want = gu.host_f64(ref)
    for attempt in range(2):  # the second call meets the first call's leftovers in the array
        out = gu.dev_f64(C0)
        assert _call_builtin(lib, plan, alpha, dA, dB, beta, out) == 0
        torch.cuda.synchronize()
        got = gu.host_f64(out)
        assert np.array_equal(got.view(np.uint64), want.view(np.uint64)), attempt
    assert lib.imd_test_device_error() == 0
    plan.close()


def test_builtin_workspace_rejects_what_does_not_fit():
    import gpu_util as gu
    import immerdink_b200 as imd
    lib = imd.load_library().lib
    m = n = k = 2048
    plan = imd.Plan.from_descs(*gu.matrix_descs(m, n, k), N=14)
    assert plan.workspace_bytes > (32 << 20)
    dA, dB, dC = gu.dev_f64(np.zeros((m, k))), gu.dev_f64(np.zeros((n, k))), gu.dev_f64(np.full((m, n), 7.0))
    assert _call_builtin(lib, plan, 1.0, dA, dB, 0.0, dC) == 4  # IMD_STATUS_INSUFFICIENT_WORKSPACE
    assert bool((dC == 7.0).all())                              # a refused call touches nothing
    plan.close()
