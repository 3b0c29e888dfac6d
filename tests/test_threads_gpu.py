"""Concurrency and no-allocation properties of the C ABI on a GPU (after the reference's
tests/test_threads.cpp:1-16 and tests/alloc_shim.c:1-40 + tests/test_contract.py:391-407):

- eight host threads, one shared plan plus a plan of their own each, own streams, workspaces and
  outputs, all calling at once: every result equals the sequential one bit for bit;
- the number of kernels a call launches equals imd_lowering.kernel_launches: a CUDA graph capture
  of the call holds exactly that many nodes, all of them kernels;
- device memory in use does not change over a thousand calls (imd_contract allocates nothing).
"""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _problem(seed, m, n, k):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.rand((m, k), generator=g, device="cuda", dtype=torch.float64) * 2 - 1
    B = torch.rand((k, n), generator=g, device="cuda", dtype=torch.float64) * 2 - 1
    return A, B


def _ws(nbytes):
    import torch
    buf = torch.empty(nbytes + 256, dtype=torch.uint8, device="cuda")
    off = (-buf.data_ptr()) % 256
    return buf[off:off + nbytes]


def test_eight_threads_shared_and_own_plans():
    import torch
    import immerdink_b200 as imd
    T = 8
    A, B = _problem(1, 384, 300, 520)
    C = torch.empty((384, 300), dtype=torch.float64, device="cuda")
    shared = imd.Plan("ik,kj->ij", A, B, C, N=14, g=7)
    ws0 = _ws(shared.workspace_bytes)
    shared.contract(A, B, C, workspace=ws0)
    torch.cuda.synchronize()
    want_shared = C.clone()
    own = [_problem(10 + t, 130 + 17 * t, 96 + 8 * t, 200 + 64 * t) for t in range(T)]
    want_own = []
    for a, b in own:
        c = torch.empty((a.shape[0], b.shape[1]), dtype=torch.float64, device="cuda")
        with imd.Plan("ik,kj->ij", a, b, c, N=12, g=0) as p:
            p.contract(a, b, c, workspace=_ws(p.workspace_bytes))
        torch.cuda.synchronize()
        want_own.append(c)
    results, errors = [None] * T, []
    barrier = threading.Barrier(T)

    def work(t):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            a, b = own[t]
            c_sh = torch.empty_like(want_shared)
            c_own = torch.empty_like(want_own[t])
            ws_sh = _ws(shared.workspace_bytes)
            plan = imd.Plan("ik,kj->ij", a, b, c_own, N=12, g=0)   # plan creation in parallel too
            ws_own = _ws(plan.workspace_bytes)
            barrier.wait()
            for _ in range(20):
                shared.contract(A, B, c_sh, workspace=ws_sh, stream=stream)
                plan.contract(a, b, c_own, workspace=ws_own, stream=stream)
            stream.synchronize()
            plan.close()
            results[t] = (c_sh, c_own)
        except Exception as exc:  # surfaced below
            errors.append(repr(exc))

    threads = [threading.Thread(target=work, args=(t,)) for t in range(T)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    for t in range(T):
        assert torch.equal(results[t][0].view(torch.int64), want_shared.view(torch.int64))
        assert torch.equal(results[t][1].view(torch.int64), want_own[t].view(torch.int64))
    assert imd.load_library().device_error() == 0
    shared.close()


@pytest.mark.parametrize("spec,shape,N,g", [
    ("ik,kj->ij", dict(i=300, j=260, k=500), 14, 7),        # A fused, B needs its scale launch
    ("ik,jk->ij", dict(i=300, j=260, k=500), 14, 14),       # both fused, one group
    ("ik,kj->ij", dict(i=64, j=48, k=131500), 5, 2),        # two K chunks, three groups
    ("ik,kj->ij", dict(i=40, j=30, k=1), 14, 0),            # native path
    ("ijk,kl->lij", dict(i=64, j=32, k=48, l=40), 14, 0),   # small: the vectors and one fused launch
])
def test_kernel_launches_equal_the_lowering(spec, shape, N, g):
    """A stream capture of one imd_contract holds exactly kernel_launches kernel nodes."""
    import torch
    import immerdink_b200 as imd
    la, lb, lc = spec.replace("->", ",").split(",")
    A = torch.rand([shape[c] for c in la], device="cuda", dtype=torch.float64)
    B = torch.rand([shape[c] for c in lb], device="cuda", dtype=torch.float64)
    C = torch.zeros([shape[c] for c in lc], device="cuda", dtype=torch.float64)
    plan = imd.Plan(spec, A, B, C, N=N, g=g)
    ws = _ws(plan.workspace_bytes)
    plan.contract(A, B, C, workspace=ws)
    torch.cuda.synchronize()
    from cuda.bindings import runtime as rt
    graph = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.graph(graph):
        plan.contract(A, B, C, workspace=ws, stream=torch.cuda.current_stream())
    raw = rt.cudaGraph_t(graph.raw_cuda_graph())
    err, _, count = rt.cudaGraphGetNodes(raw, 0)
    assert int(err) == 0
    err, nodes, count = rt.cudaGraphGetNodes(raw, count)
    kinds = [rt.cudaGraphNodeGetType(n)[1] for n in nodes[:count]]
    kernels = sum(1 for k in kinds if k == rt.cudaGraphNodeType.cudaGraphNodeTypeKernel)
    assert len(kinds) == kernels, kinds     # a call is kernels only: no copies, no memsets
    assert kernels == plan.lowering["kernel_launches"], (kernels, plan.lowering["kernel_launches"])
    graph.instantiate()
    graph.replay()
    torch.cuda.synchronize()
    plan.close()


def test_a_thousand_calls_allocate_nothing():
    import torch
    import immerdink_b200 as imd
    A, B = _problem(3, 200, 180, 320)
    C = torch.empty((200, 180), dtype=torch.float64, device="cuda")
    plan = imd.Plan("ik,kj->ij", A, B, C, N=14, g=7)
    ws = _ws(plan.workspace_bytes)
    for _ in range(3):
        plan.contract(A, B, C, workspace=ws)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(1000):
        plan.contract(A, B, C, workspace=ws)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    plan.close()
