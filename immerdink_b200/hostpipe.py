"""Contractions whose operands live in (pinned) HOST memory: a slab pipeline over one GPU.

No counterpart in the reference, whose API takes device arrays only; a caller with host data
would copy A and B in, call imd_contract and copy C out, three steps that run one after the
other. Here the output is cut in slabs along one free label `split` of C, which is a label of
exactly one operand (the SLABBED operand); the other operand is SHARED by all slabs:

    copy stream     H2D shared | H2D slab 0 | H2D slab 1 | ...
    compute stream             | imd_pack(shared) | contract_packed(slab 0) | slab 1 | ...
    return stream                                 | D2H C slab 0 | D2H C slab 1 | ...

The shared operand is packed once (imd_pack) and every slab reads the packed buffer
(imd_contract_packed), so its shifts and residues are computed once, as in one undivided call.
Slabs are views of full-size device tensors (same strides, smaller extent along `split`), so ONE
plan serves all slabs with offset pointers and the results are bit-identical to the undivided
contraction: every output depends only on its own row of A and column of B.

Host <-> device slab copies are pitched 2-D DMA copies (cudaMemcpy2DAsync) straight from / to the
caller's pinned arrays. Device memory, streams and events come from torch (plumbing only); the
arithmetic is libimmerdink's.
"""
import math

from . import device as _dev


def _pitched(shape, pos, lo, hi):
    """(rows, width bytes, pitch bytes, offset bytes) of the slab [lo, hi) of mode `pos` of a dense
    row-major float64 tensor, as a pitched 2-D region."""
    inner = math.prod(shape[pos + 1:])
    return (math.prod(shape[:pos]), (hi - lo) * inner * 8, shape[pos] * inner * 8, lo * inner * 8)


class HostContraction:
    """`spec` with single-letter labels on dense row-major float64 operands of the given shapes.
    `split`: a label of C and of exactly one of A, B. Owns its device buffers (operands, packed
    buffer, workspaces: allocated here, once) and three streams. Call it with pinned host tensors
    (torch, `pin_memory()`); work is enqueued behind the current stream's work and the current
    stream waits for the result, so it composes with stream-ordered code and CUDA events."""

    def __init__(self, spec, shapeA, shapeB, shapeC, *, N, split, slabs=8, g=0, rounding="RN",
                 device=None, lib=None):
        import torch
        from cuda.bindings import runtime as rt
        self._torch, self._rt = torch, rt
        ins, out = spec.replace(" ", "").split("->")
        la, lb = ins.split(",")
        if split not in out or (split in la) == (split in lb):
            raise ValueError(f"split label {split!r} must be in C and in exactly one of A, B")
        self.spec, self.labels = spec, (la, lb, out)
        self.shapes = tuple(tuple(int(e) for e in s) for s in (shapeA, shapeB, shapeC))
        self.x = 0 if split in la else 1          # the slabbed operand; 1 - x is shared (packed)
        self.pos = (self.labels[self.x].index(split), out.index(split))
        if self.labels[self.x].count(split) != 1:
            raise ValueError("the split label may not repeat in its operand")
        extent = self.shapes[2][self.pos[1]]
        self.bounds = [(extent * s // slabs, extent * (s + 1) // slabs) for s in range(slabs)]
        widths = {hi - lo for lo, hi in self.bounds}
        if len(widths) != 1 or 0 in widths:
            raise ValueError(f"extent {extent} of {split!r} must divide into {slabs} equal slabs")
        self.width = widths.pop()
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = dev
        with torch.cuda.device(dev):
            self.d = [torch.empty(s, dtype=torch.float64, device=dev) for s in self.shapes]
            views = list(self.d)
            views[self.x] = self.d[self.x].narrow(self.pos[0], 0, self.width)
            views[2] = self.d[2].narrow(self.pos[1], 0, self.width)
            sh = 1 - self.x
            self.pack = _dev.Pack(_dev.pack_spec(spec, *views, operand=sh, N=N, g=g, rounding=rounding,
                                                 lib=lib), lib=lib)
            packs = [None, None]
            packs[sh] = self.pack
            self.plan = _dev.Plan(spec, *views, N=N, g=g, rounding=rounding, packs=tuple(packs), lib=lib)
            nbytes = lambda n: torch.empty(max(int(n), 1), dtype=torch.uint8, device=dev)
            self.packed = nbytes(self.pack.pack_bytes)
            self.pack_ws = nbytes(self.pack.workspace_bytes)
            self.ws = nbytes(self.plan.workspace_bytes)   # slabs run one after the other
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.device_bytes = (sum(t.numel() * 8 for t in self.d) + self.packed.numel() +
                             self.pack_ws.numel() + self.ws.numel())

    # -- pitched copies ---------------------------------------------------------------------
    def _copy2d(self, dst, src, region, to_device, stream):
        rows, width, pitch, off = region
        rt = self._rt
        kind = rt.cudaMemcpyKind.cudaMemcpyHostToDevice if to_device else rt.cudaMemcpyKind.cudaMemcpyDeviceToHost
        if rows == 0 or width == 0:
            return
        err, = rt.cudaMemcpy2DAsync(dst.data_ptr() + off, pitch, src.data_ptr() + off, pitch, width,
                                    rows, kind, stream.cuda_stream)
        if err != rt.cudaError_t.cudaSuccess:
            raise _dev.CudaError(f"cudaMemcpy2DAsync: {err}")

    def _check_host(self, t, shape, what):
        if tuple(t.shape) != shape or t.dtype != self._torch.float64 or not t.is_contiguous():
            raise ValueError(f"{what}: a contiguous float64 tensor of shape {shape} is needed")
        if not t.is_pinned():
            raise ValueError(f"{what} must be in pinned host memory (tensor.pin_memory())")

    # -- the call -----------------------------------------------------------------------------
    def __call__(self, hA, hB, hC, alpha=1.0, beta=0.0):
        """hC <- alpha hA.hB + beta hC. Returns hC; its contents are ready once the current stream
        reaches this point (synchronize it, or record an event on it, before reading hC)."""
        torch = self._torch
        h = (hA, hB, hC)
        for t, s, w in zip(h, self.shapes, "ABC"):
            self._check_host(t, s, w)
        x, sh = self.x, 1 - self.x
        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream()
            start = cur.record_event()
            for st in (self.s_in, self.s_run, self.s_out):
                st.wait_event(start)
            # shared operand in, then packed once
            with torch.cuda.stream(self.s_in):
                self.d[sh].copy_(h[sh], non_blocking=True)
                shared_in = self.s_in.record_event()
            self.s_run.wait_event(shared_in)
            self.pack.pack(self.d[sh], self.packed, workspace=self.pack_ws, stream=self.s_run)
            packed = [None, None]
            packed[sh] = self.packed
            for lo, hi in self.bounds:
                reg_x = _pitched(self.shapes[x], self.pos[0], lo, hi)
                reg_c = _pitched(self.shapes[2], self.pos[1], lo, hi)
                self._copy2d(self.d[x], h[x], reg_x, True, self.s_in)
                if beta != 0.0:
                    self._copy2d(self.d[2], hC, reg_c, True, self.s_in)
                self.s_run.wait_event(self.s_in.record_event())
                ops = [None, None]
                ops[x] = self.d[x].narrow(self.pos[0], lo, hi - lo)
                ops[sh] = self.d[sh]
                self.plan.contract(ops[0], ops[1], self.d[2].narrow(self.pos[1], lo, hi - lo),
                                   alpha=alpha, beta=beta, workspace=self.ws,
                                   stream=self.s_run, packed=tuple(packed))
                self.s_out.wait_event(self.s_run.record_event())
                self._copy2d(hC, self.d[2], reg_c, False, self.s_out)
            for st in (self.s_in, self.s_run, self.s_out):
                cur.wait_event(st.record_event())
        return hC

    def close(self):
        self.plan.close()
        self.pack.close()
