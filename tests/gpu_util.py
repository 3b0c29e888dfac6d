"""Helpers of the GPU parity tests: device buffers through torch (plumbing only), calls through
the C ABI of libimmerdink.so via the package's ctypes front end."""
import ctypes as C

import numpy as np
import torch

import immerdink_b200 as imd
from immerdink_b200 import host

POISON = 0xA5


def lib():
    return imd.load_library()


def dev_f64(arr):
    """float64 numpy array (any shape) -> flat CUDA tensor with the same bits."""
    a = np.ascontiguousarray(arr, np.float64).reshape(-1)
    t = torch.from_numpy(a.view(np.int64).copy()).cuda()
    return t.view(torch.float64)


def host_f64(t):
    return t.view(torch.int64).cpu().numpy().view(np.float64)


class Workspace:
    """A poisoned workspace with guard zones before and after the bytes the plan may write."""
    GUARD = 4096

    def __init__(self, nbytes):
        self.nbytes = nbytes
        self.buf = torch.full((nbytes + 2 * self.GUARD + 256,), POISON, dtype=torch.uint8, device="cuda")
        p = self.buf.data_ptr() + self.GUARD
        self.offset = self.GUARD + (-p) % 256
        self.ptr = self.buf.data_ptr() + self.offset

    def arg(self):
        return (self.ptr, self.nbytes)

    def region(self, off, nbytes, dtype):
        raw = self.buf[self.offset + off:self.offset + off + nbytes].cpu().numpy()
        return raw.view(dtype)

    def guards_intact(self):
        b = self.buf.cpu().numpy()
        return bool((b[:self.offset] == POISON).all() and (b[self.offset + self.nbytes:] == POISON).all())


def run_descs(descs, bufs, bases, alpha, beta, N, g=0, rounding="RN", mode="EMULATE",
              vec_mode="GENERATE", reference_gemm=False, want_ws=False, gemm_variant=0, small=None):
    """imd_plan_create + imd_contract on flat float64 buffers with raw descriptors. Returns the
    whole C buffer (numpy) and, optionally, (plan, workspace). small: False keeps small
    contractions on the general kernel sequence (always so when the workspace is wanted back:
    the one fused launch leaves no residue or product planes there); None / True: as in production."""
    L = lib()
    L.lib.imd_test_use_reference_gemm(1 if reference_gemm else 0)
    L.lib.imd_test_gemm_variant(gemm_variant)
    L.lib.imd_test_small_path(0 if (small is False or want_ws or reference_gemm or gemm_variant) else 1)
    try:
        plan = imd.Plan.from_descs(*descs, N=N, g=g, rounding=rounding, mode=mode, vec_mode=vec_mode)
        dA, dB, dC = (dev_f64(b) if b is not None else None for b in bufs)
        ws = Workspace(plan.workspace_bytes)
        ptr = [None if t is None else t.data_ptr() + 8 * base for t, base in zip((dA, dB, dC), bases)]
        plan.contract_ptr(alpha, ptr[0], ptr[1], beta, ptr[2], ws.ptr if plan.workspace_bytes else None,
                          plan.workspace_bytes, 0)
        torch.cuda.synchronize()
        err = L.lib.imd_test_device_error()
        assert err == 0, f"device error word {err:#x} (a bounded wait in a kernel gave up)"
        assert ws.guards_intact(), "bytes outside [ws, ws + workspace_size) were written"
        out = host_f64(dC)
    finally:
        L.lib.imd_test_use_reference_gemm(0)
        L.lib.imd_test_gemm_variant(0)
        L.lib.imd_test_small_path(1)
    if want_ws:
        return out, plan, ws
    plan.close()
    return out


def matrix_descs(m, n, k):
    """C[i][j] = sum_h A[i][h] Bt[j][h]: A m x k, Bt n x k, C m x n, all row-major (no role swap)."""
    i, j, h = ord("i"), ord("j"), ord("h")
    return (host.Desc((m, k), (k, 1), (i, h)), host.Desc((n, k), (k, 1), (j, h)),
            host.Desc((m, n), (n, 1), (i, j)))


def layout_of(descs, N, g=0, rounding="RN", mode="EMULATE"):
    return host.workspace_layout(descs, N=N, g=g, rounding=rounding, mode=mode)
