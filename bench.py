"""Benchmark of the emulated FP64 contraction path (imd_plan_create -> imd_contract).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line. Metric: FP64-equivalent TFLOPS = 2 b m n k / t (the reference's definition,
docs/BENCHMARKING.md:16) on 'kjbc,kiac->abij' with a=b=c=200, i=j=k=40 (GEMM view 8000^3), N = 14
moduli, residue group 7, alpha = 1, beta = 0, seeded synthetic uniform [-1, 1) operands.

  value  device-resident operands, CUDA events on the launching stream, max over ranks
  e2e    the same contraction with HOST operands through the package's host-operand pipeline
         (immerdink_b200.hostpipe): pinned host -> device copies of A and B and the device -> host
         copy of C inside the timed region, overlapped slab by slab with imd_contract_packed;
         `serial_ms` is the plain sequence copy in, imd_contract, copy out
  roofline      the tcgen05 int8 GEMM phase (algorithmic int8 ops 2 N b m n k over its measured time)
  cpu_baseline  the CPU oracle (oracle/, a port of the reference's specification) on a sampled block
  --impl reference  times that CPU oracle alone, all host threads (the reference has no other CPU
         implementation that can travel to the GPU box: its own is Python, spec/oracle.py)

With N > 1 ranks (torchrun) the output C is partitioned over its free modes a and b
(immerdink_b200.dist): every rank owns 1/N of A and of B, all-gathers the slabs of its tile over
NCCL inside its grid column / row, and computes the tile with its own plan; no collective follows.
A timed step is the WHOLE exchange + contraction of every rank (immerdink_b200.dist.RankContraction:
the all-gathers run on a side stream, A is packed while B's slab arrives); `value` is strong scaling
of the one contraction, max over ranks. `config` also gives the all-gathers alone and the
contraction with the slabs already gathered.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (spec, extents, N, g)
    "cc8000": ("kjbc,kiac->abij", dict(a=200, b=200, c=200, i=40, j=40, k=40), 14, 7),
    "cc4000": ("kjbc,kiac->abij", dict(a=100, b=100, c=100, i=40, j=40, k=40), 14, 7),
    "cc1000": ("kjbc,kiac->abij", dict(a=50, b=50, c=50, i=20, j=20, k=20), 14, 7),
}
GRID = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}  # ranks over (a, b)
RANK_GROUP = {2: 4, 4: 4, 8: 3}   # residue group of a rank's plan in the residue exchange, as measured
SEED = 20251125
MASK = (1 << 64) - 1


# ------------------------------------------------------------------ synthetic data (counter based)
def mix_np(idx, seed):
    """splitmix64 of (seed + flat index) -> uniform [-1, 1) float64; numpy, uint64 wraparound."""
    z = (idx.astype(np.uint64) + np.uint64(seed)) * np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    z = z ^ (z >> np.uint64(31))
    return (z >> np.uint64(11)).astype(np.float64) * (2.0 ** -52) - 1.0


def mix_torch(idx, seed):
    """The same function on the GPU: int64 arithmetic wraps like uint64; shifts made logical."""
    import torch

    def i64(v):
        v &= MASK
        return v - (1 << 64) if v >= (1 << 63) else v

    def shr(z, s):
        return (z >> s) & ((1 << (64 - s)) - 1)
    z = (idx + i64(seed)) * i64(0x9E3779B97F4A7C15)
    z = (z ^ shr(z, 30)) * i64(0xBF58476D1CE4E5B9)
    z = (z ^ shr(z, 27)) * i64(0x94D049BB133111EB)
    z = z ^ shr(z, 31)
    return shr(z, 11).to(torch.float64) * (2.0 ** -52) - 1.0


def slab_offsets_torch(extent, full_extent, start, device):
    """Flat offsets (in the FULL dense tensor) of the slab [start, start + extent) per mode."""
    import torch
    strides, acc = [], 1
    for e in reversed(full_extent):
        strides.append(acc)
        acc *= e
    strides = list(reversed(strides))
    off = torch.zeros((), dtype=torch.int64, device=device)
    for d, (e, s0, st) in enumerate(zip(extent, start, strides)):
        shape = [1] * len(extent)
        shape[d] = e
        off = off + (torch.arange(s0, s0 + e, dtype=torch.int64, device=device) * st).reshape(shape)
    return off


class Problem:
    """The contraction of one rank: its slab extents and where they sit in the full tensors."""

    def __init__(self, workload, rank, world):
        self.spec, self.ext, self.N, self.g = WORKLOADS[workload]
        self.labels = [s for s in self.spec.replace("->", ",").split(",")]
        pa, pb = GRID[world]
        ra, rb = rank // pb, rank % pb
        self.full = dict(self.ext)
        self.start = {c: 0 for c in self.ext}
        self.local = dict(self.ext)
        for lab, parts, r in (("a", pa, ra), ("b", pb, rb)):
            lo = self.ext[lab] * r // parts
            hi = self.ext[lab] * (r + 1) // parts
            self.start[lab], self.local[lab] = lo, hi - lo
        self.seeds = [SEED, SEED + 1]

    def shape(self, x, local=True):
        e = self.local if local else self.full
        return [e[c] for c in self.labels[x]]

    def flops_eq_full(self):
        e = self.full
        return 2.0 * math.prod(e[c] for c in set("".join(self.labels)))

    def device_operand(self, x, device):
        off = slab_offsets_torch(self.shape(x), self.shape(x, False),
                                 [self.start[c] for c in self.labels[x]], device)
        return mix_torch(off, self.seeds[x]).contiguous()


# ------------------------------------------------------------------ CPU oracle (baseline / reference arm)
def cpu_sample(prob, rows, cols, threads=None):
    """Time the CPU oracle on a rows x cols block of outputs (full k) of the FULL problem.
    Returns (seconds, flops_eq of the block, block result, row ids, col ids)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import imd_oracle as orc
    labels = prob.labels
    descs = []
    for x in range(3):
        ext = prob.shape(x, False)
        st, acc = [], 1
        for e in reversed(ext):
            st.append(acc)
            acc *= e
        descs.append(orc.Desc(ext, list(reversed(st)), [ord(c) for c in labels[x]]))
    view = orc.lower(*descs)
    rng = np.random.default_rng(5)
    ri = np.sort(rng.choice(view.m, size=min(rows, view.m), replace=False))
    cj = np.sort(rng.choice(view.n, size=min(cols, view.n), replace=False))
    seedA, seedB = (prob.seeds[1], prob.seeds[0]) if view.swapped else (prob.seeds[0], prob.seeds[1])
    offA = orc.vec(view, "A_row")[ri][:, None] + orc.vec(view, "A_k")[None, :]
    offB = orc.vec(view, "B_col")[cj][:, None] + orc.vec(view, "B_k")[None, :]
    Ab, Bb = mix_np(offA, seedA), mix_np(offB, seedB)
    t0 = time.perf_counter()
    out = orc.gemm(Ab, Bb, prob.N)
    dt = time.perf_counter() - t0
    coff = orc.vec(view, "C_row")[ri][:, None] + orc.vec(view, "C_col")[None, cj]
    return dt, 2.0 * len(ri) * len(cj) * view.k, out, coff


def cpu_threads():
    n = os.environ.get("OMP_NUM_THREADS")
    return int(n) if n else (os.cpu_count() or 1)


def run_reference(args, rank):
    """The reference arm: the CPU oracle port, all host threads, on bounded samples of the workload."""
    if rank != 0:
        return
    prob = Problem(args.workload, 0, 1)
    side = 384
    times = []
    for it in range(args.warmup + args.steps):
        dt, fl, _, _ = cpu_sample(prob, side, side)
        if it >= args.warmup:
            times.append(dt)
    t = float(np.mean(times))
    val = fl / t / 1e12
    line = dict(metric="fp64_equivalent_tflops", value=val, unit="TFLOPS-eq", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=t * 1e3, higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="int8xint8->int32 (FP64 emulation)",
                data="synthetic", impl="reference",
                config=dict(workload=f"{args.workload}: {prob.spec} {prob.ext} N={prob.N}",
                            note="CPU oracle port of the reference specification; each step is a "
                                 f"{side}x{side} output block with full k"),
                cpu_baseline=dict(value=val, unit="TFLOPS-eq", cores=cpu_threads(), kind="port",
                                  sample=f"{side}x{side} outputs x k, {args.steps} steps"),
                e2e=dict(value=val, unit="TFLOPS-eq", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ------------------------------------------------------------------ clocks
class ClockSampler(threading.Thread):
    """SM clock and throttle reasons of one GPU, sampled through NVML while the timed region runs."""

    def __init__(self, index, period=0.005):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag, self.max_mhz = index, [], False, None
        self.period = period
        self.error = None
        self.ready = threading.Event()     # NVML initialised (its first call takes a while)
        self.recording = False             # samples are kept only inside the timed region

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            self.ready.set()
            while not self.stop_flag:
                sample = (nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                          nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                if self.recording:
                    self.samples.append(sample)
                time.sleep(self.period)   # light: NVML calls take driver locks that submissions share
        except Exception as exc:  # NVML missing: report it, never fail the benchmark
            self.error = repr(exc)
        finally:
            self.ready.set()

    def begin(self):
        self.ready.wait(timeout=10)
        self.recording = True

    def summary(self):
        self.recording = False
        self.stop_flag = True
        self.join(timeout=2)
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=["unavailable: " + str(self.error)])
        sm = sorted(s[0] for s in self.samples)
        bits = 0
        for _, r in self.samples:
            bits |= r
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                 0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
                 0x10: "sync_boost", 0x100: "display_clock_setting"}
        return dict(sm_mhz=sm[len(sm) // 2], sm_min_mhz=sm[0], sm_max_mhz=self.max_mhz,
                    reasons=[n for b, n in names.items() if bits & b], samples=len(self.samples))


# ------------------------------------------------------------------ our arm
def run_ours(args, rank, world, local_rank):
    import ctypes as C

    import torch
    import torch.distributed as dist

    import immerdink_b200 as imd

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from immerdink_b200 import dist as idist
    prob = Problem(args.workload, 0, 1)          # the undivided contraction
    lib = imd.load_library()
    part = idist.Partition(prob.spec, prob.ext, world, rank, "a", "b")

    def synth(x, shape, start):
        labels = prob.labels[x]
        off = slab_offsets_torch(shape, prob.shape(x, False), [start.get(c, 0) for c in labels], dev)
        return mix_torch(off, prob.seeds[x]).contiguous()

    exchange = rankc = None
    if world == 1:
        A = synth(0, prob.shape(0), {})
        B = synth(1, prob.shape(1), {})
        Cd = torch.empty(prob.shape(2), dtype=torch.float64, device=dev)
        plan = imd.Plan(prob.spec, A, B, Cd, N=prob.N, g=prob.g)
        run_spec = prob.spec
    else:
        # every rank owns 1/world of A and of B; a step = exchange of the slabs + the rank's tile
        shard_a = synth(0, part.shard_shape(0), part.shard_start(0))
        shard_b = synth(1, part.shard_shape(1), part.shard_start(1))
        groups = idist.make_groups(world, dist)
        # the residue group is also the unit in which planes travel between ranks: smaller groups
        # start the first GEMM earlier (results do not depend on it)
        rank_g = args.group or (prob.g if args.exchange == "fp64" else RANK_GROUP.get(world, prob.g))
        store_push = {"auto": "auto", "none": None, "a": 0, "b": 1}[args.store_push]
        try:
            rankc = idist.RankContraction(part, N=prob.N, g=rank_g, dist=dist, groups=groups,
                                          exchange=args.exchange, push_streams=args.push_streams,
                                          sync=args.sync, store_push=store_push)
            ok = torch.ones(1, device=dev)
        except Exception as exc:   # e.g. CUDA IPC closed in this environment
            print(f"rank {rank}: residue exchange unavailable ({exc!r})", file=sys.stderr)
            rankc, ok = None, torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)   # all ranks take the same path
        if ok.item() == 0:
            if rankc is not None:
                rankc.close()
            rankc = idist.RankContraction(part, N=prob.N, g=rank_g, dist=dist, groups=groups,
                                          exchange="fp64")
        A, B, plan, run_spec = rankc.A, rankc.B, rankc.plan, rankc.spec
        Cd = torch.empty(rankc.tile_shape, dtype=torch.float64, device=dev)

        def exchange():
            idist.gather(part, shard_a, shard_b, A, B, groups, dist)
    ws = torch.empty(plan.workspace_bytes + 256, dtype=torch.uint8, device=dev)
    off = (-ws.data_ptr()) % 256
    wsv = ws[off:off + plan.workspace_bytes]
    stream = torch.cuda.current_stream()
    low = plan.lowering
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > L2 (126 MB)

    def step():
        if rankc is None:
            plan.contract(A, B, Cd, workspace=wsv, stream=stream)
        else:
            rankc(shard_a, shard_b, Cd)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # rank 0 reports its GPU's clocks; the other ranks do not poll (a step of several GPUs is many
    # short submissions, which NVML's locks delay)
    sampler = ClockSampler(local_rank, 0.005 if world == 1 else 0.010)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- device-resident timing with per-phase events
    # Per-phase events sit between the kernels of the timed steps on one GPU (five per step). With
    # more GPUs a step is many short launches that wait on other ranks, where the event records cost
    # a tenth of the step: there the phases come from a separate pass of the same steps just after.
    phases_in_timed_region = world == 1
    if phases_in_timed_region:
        lib.lib.imd_prof_enable(64 * (args.steps + 1))
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(args.steps)]
    barrier()
    if rank == 0:
        sampler.begin()
    host_ms = 0.0
    for s in range(args.steps):
        flush.fill_(s)  # evict the previous step's working set from L2 (outside the timed events)
        ev[s][0].record(stream)
        h0 = time.perf_counter()
        step()
        host_ms += (time.perf_counter() - h0) * 1e3 / args.steps   # enqueue only: nothing waits for the GPU
        ev[s][1].record(stream)
    barrier()
    clocks = sampler.summary() if rank == 0 else None
    ms = sum(a.elapsed_time(b) for a, b in ev) / args.steps
    phase_steps = args.steps
    if not phases_in_timed_region:
        phase_steps = min(args.steps, 5)
        lib.lib.imd_prof_enable(64 * (phase_steps + 1))
        for s in range(phase_steps):
            flush.fill_(s)
            step()
        barrier()
    phases = (C.c_float * 8)()
    lib.lib.imd_prof_read(phases, 8)
    lib.lib.imd_prof_enable(0)
    step_trace = None
    if rankc is not None and rankc.exchange == "residues":
        # one more step with an event at every stage (main and push stream), as a time line of rank 0
        flush.fill_(0)
        rankc.trace = []
        step()
        barrier()
        t0 = rankc.trace[0][1]
        step_trace = {label: round(t0.elapsed_time(e), 3) for label, e in rankc.trace[1:]}
        rankc.trace = None
    phase_ms = {name: phases[t] / phase_steps for t, name in
                ((1, "vectors+scale"), (2, "residues"), (3, "gemm"), (4, "crt"), (6, "pack"))}
    t_ms = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms_max = float(t_ms.item())

    # ---- end to end: pinned host operands in, host result out, through the public Python API
    srcA, srcB = (A, B) if world == 1 else (shard_a, shard_b)
    hA = torch.empty(srcA.shape, dtype=torch.float64).pin_memory()
    hB = torch.empty(srcB.shape, dtype=torch.float64).pin_memory()
    hC = torch.empty(Cd.shape, dtype=torch.float64).pin_memory()
    hA.copy_(srcA)
    hB.copy_(srcB)
    dA2, dB2 = (torch.empty_like(A), torch.empty_like(B)) if world == 1 else (shard_a, shard_b)
    inA, inB = (dA2, dB2) if world == 1 else (A, B)

    def e2e_step():
        dA2.copy_(hA, non_blocking=True)
        dB2.copy_(hB, non_blocking=True)
        if rankc is None:
            imd.contract(run_spec, inA, inB, Cd, N=prob.N, g=prob.g, workspace=wsv, stream=stream)
        else:
            rankc(dA2, dB2, Cd)
        hC.copy_(Cd, non_blocking=True)

    e2e_steps = max(2, min(args.steps, 5))

    def time_e2e(fn):
        fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            fn()
        e1.record(stream)
        barrier()
        return e0.elapsed_time(e1) / e2e_steps

    serial_ms = time_e2e(e2e_step)     # copy in, one call, copy out: one after the other
    e2e_ms, e2e_exact = serial_ms, None
    e2e_how = ("H2D A, B; one imd_contract; D2H C (in sequence)" if world == 1 else
               "per rank: H2D of its pieces of A and B; exchange + contraction (dist.RankContraction); D2H of its C tile")
    if world == 1:
        # the same host operands through the slab pipeline of the package: copies overlap the
        # contraction, the shared operand is packed once
        from immerdink_b200.hostpipe import HostContraction
        del dA2, dB2
        slabs = max(d for d in range(1, args.slabs + 1) if prob.ext["a"] % d == 0)
        pipe = HostContraction(prob.spec, prob.shape(0), prob.shape(1), prob.shape(2), N=prob.N,
                               g=prob.g, split="a", slabs=slabs)
        e2e_ms = time_e2e(lambda: pipe(hA, hB, hC))
        e2e_how = (f"immerdink_b200.hostpipe.HostContraction: C cut in {slabs} slabs along 'a'; "
                   "pitched H2D / D2H copies overlap imd_contract_packed per slab; the shared "
                   "operand (A) is packed once per step (imd_pack)")
        e2e_exact = bool(torch.equal(hC.view(torch.int64), Cd.cpu().view(torch.int64)))
        pipe.close()
        del pipe
    t_e2e = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    e2e_ms = float(t_e2e.item())
    exchange_ms = resident_ms = 0.0
    parity = None
    if world > 1:
        # every rank checks the outputs of one sampled block (CPU oracle, full k) that fall into its tile
        _, _, out, coff = cpu_sample(prob, 192, 192)
        labels_c = prob.labels[2]
        idx = np.unravel_index(coff.reshape(-1), prob.shape(2, False))
        local_shape = [part.local[c] for c in labels_c]
        inside, loc = np.ones(coff.size, dtype=bool), []
        for d, c in enumerate(labels_c):
            v = idx[d] - part.start.get(c, 0)
            inside &= (v >= 0) & (v < local_shape[d])
            loc.append(v)
        flat = np.ravel_multi_index([v[inside] for v in loc], local_shape)
        got = Cd.reshape(-1)[torch.from_numpy(flat).to(dev)].cpu().numpy()
        same = np.array_equal(got.view(np.uint64), out.reshape(-1)[inside].view(np.uint64))
        agree = torch.tensor([int(same)], dtype=torch.int64, device=dev)
        count = torch.tensor([int(inside.sum())], dtype=torch.int64, device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        dist.all_reduce(count, op=dist.ReduceOp.SUM)
        parity = dict(outputs=int(count.item()), bit_exact=bool(agree.item()),
                      how="each rank compares the sampled outputs inside its tile with the CPU oracle")
    if exchange is not None:
        def timed(fn, reps=5):
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            fn()
            barrier()
            x0.record(stream)
            for _ in range(reps):
                fn()
            x1.record(stream)
            barrier()
            t = torch.tensor([x0.elapsed_time(x1) / reps], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        exchange_ms = timed(exchange)            # the two all-gathers alone
        plain = imd.Plan(run_spec, A, B, Cd, N=prob.N, g=prob.g)
        wsp = torch.empty(plain.workspace_bytes, dtype=torch.uint8, device=dev)
        resident_ms = timed(lambda: plain.contract(A, B, Cd, workspace=wsp, stream=stream))
        plain.close()
    err = lib.lib.imd_test_device_error()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    flops = prob.flops_eq_full()
    # the int8 GEMM phase of this rank against the measured dense tensor peak
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    # dense int8 runs at twice the dense bf16 rate on this part; a call lasts milliseconds, so the
    # burst figure applies. The bare tensor pipe (back-to-back tcgen05.mma, no loads) is probed too.
    bf16 = peaks.get("bf16_tflops")
    peak_tops = 2.0 * bf16 if bf16 else 2.0 * 1590.0
    lib.lib.imd_prof_mma_peak.restype = C.c_double
    probe_tops = lib.lib.imd_prof_mma_peak(1) / 1e12
    # DRAM bytes (read + write) of ONE GEMM launch (one residue group), from single-pass ncu captures
    # of this command (dram__bytes_read.sum + dram__bytes_write.sum); None where not captured.
    gemm_traffic = {"cc8000": 2.95e9, "cc4000": 3.16e8}.get(args.workload) if world == 1 else None
    gemm_ops = 2.0 * prob.N * low["b"] * low["m"] * low["n"] * low["k"]
    achieved = gemm_ops / (phase_ms["gemm"] * 1e-3) / 1e12 if phase_ms["gemm"] > 0 else 0.0
    # kernels per step: the plan's launches; + the 4 of imd_pack (FP64 exchange: A goes through a pack);
    # residue exchange: 2 x 4 of imd_pack_scatter, per part call (one per residue group, CRT, native
    # path) the index vectors and the part's kernel, the flag waits and the conditional fetch
    launches_per_step = int(low["kernel_launches"])
    if rankc is not None and rankc.exchange == "fp64":
        launches_per_step += 4
    elif rankc is not None:
        n_groups = len(rankc.groups_of_planes)
        launches_per_step = 8 + 2 * (n_groups + 2) + (n_groups + 1 if rankc.sync == "flags" else 0) + 1
    line = dict(metric="fp64_equivalent_tflops", value=flops / (ms_max * 1e-3) / 1e12, unit="TFLOPS-eq",
                n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms_max,
                higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="int8xint8->int32 (FP64 emulation)", data="synthetic",
                config=dict(workload=f"{args.workload}: {prob.spec} {prob.ext} N={prob.N} g={prob.g} "
                                     "alpha=1 beta=0, uniform[-1,1)",
                            partition=(f"C modes (a,b) over {GRID[world]} ranks" + (
                                "" if world == 1 else
                                "; every step each rank packs its own pieces of A and B once (imd_pack_scatter), "
                                "copy engines push the residue planes into the other consumers' slab buffers "
                                "over NVLink group by group while the GEMM of the previous group runs (flag "
                                "words announce them; with three other consumers of one slab the other slab's "
                                "planes go by the pack kernel's own stores), and the tile is contracted from "
                                "the packed slabs; FP64 pieces are fetched from peers only when a row is "
                                "flagged for the native path" if rankc.exchange == "residues" else
                                "; every step all-gathers the FP64 slabs over NCCL (side stream), packs A "
                                "while B arrives and contracts the rank's tile")),
                            exchange_alone_ms=exchange_ms, contraction_slabs_resident_ms=resident_ms,
                            l2="256 MB buffer written between timed steps",
                            gemm_view=[low["m"], low["n"], low["k"], low["b"]]),
                e2e=dict(value=flops / (e2e_ms * 1e-3) / 1e12, unit="TFLOPS-eq",
                         h2d_bytes_per_step=(srcA.numel() + srcB.numel()) * 8 * world,
                         d2h_bytes_per_step=Cd.numel() * 8 * world, ms_per_step=e2e_ms,
                         how=e2e_how, serial_ms=serial_ms, equals_device_result=e2e_exact),
                gpu_launches=launches_per_step * args.steps * world,
                clocks=clocks,
                phases_ms=phase_ms,
                roofline=dict(bound="tensor", achieved=achieved, peak=peak_tops, unit="TOP/s (int8)",
                              frac=achieved / peak_tops, traffic=gemm_traffic,
                              peak_probe=probe_tops,
                              note=("peak = 2 x measured burst dense bf16 (of measured)" if bf16
                                    else "peak = 2 x 1590 TFLOP/s bf16 (of fallback)") +
                              "; peak_probe = back-to-back tcgen05.mma.kind::i8 on this GPU, no loads; achieved = "
                              "2 N b m n k int8 ops of the call / time of its GEMM launches; traffic = DRAM "
                              "bytes of one GEMM launch (algorithmic: both operands' planes once + product "
                              "planes once = 1.34e9 at cc8000)"),
                device_error=int(err))
    line["host_enqueue_ms_per_step"] = host_ms
    if step_trace is not None:
        line["step_trace_ms"] = step_trace
    line["phases_from"] = ("events inside the timed steps" if phases_in_timed_region else
                           f"a separate pass of {phase_steps} steps after the timed ones")
    if parity is not None:
        line["parity_sample"] = parity
    if world > 1 and rankc.exchange == "residues":
        line["config"]["exchange"] = dict(kind="residues", sync=rankc.sync, push_streams=len(rankc.push_streams),
                                          planes_by_pack_kernel_stores=(None if rankc.store_push is None
                                                                        else "AB"[rankc.store_push]),
                                          residue_group_per_rank=rank_g)
    elif world > 1:
        line["config"]["exchange"] = dict(kind="fp64", residue_group_per_rank=rank_g)
    if world == 1 and not args.no_cpu:
        # DGEMM on the same GPU, same GEMM view
        n = low["m"]
        x = torch.rand(n, low["k"], dtype=torch.float64, device=dev)
        y = torch.rand(low["k"], low["n"], dtype=torch.float64, device=dev)
        torch.matmul(x, y)
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        for _ in range(3):
            torch.matmul(x, y)
        d1.record()
        torch.cuda.synchronize()
        line["native_dgemm_tflops"] = 3 * 2.0 * n * low["k"] * low["n"] / (d0.elapsed_time(d1) * 1e-3) / 1e12
        del x, y
        # CPU oracle on a sampled block; the same block checks the GPU result bit for bit
        side = 64
        dt, _, _, _ = cpu_sample(prob, side, side)
        side = int(max(64, min(4096, side * math.sqrt(12.0 / max(dt, 1e-3)))))
        dt, fl, out, coff = cpu_sample(prob, side, side)
        got = Cd.reshape(-1)[torch.from_numpy(coff.reshape(-1)).to(dev)].cpu().numpy().reshape(out.shape)
        line["parity_sample"] = dict(outputs=int(out.size),
                                     bit_exact=bool(np.array_equal(got.view(np.uint64), out.view(np.uint64))))
        line["cpu_baseline"] = dict(value=fl / dt / 1e12, unit="TFLOPS-eq", cores=cpu_threads(), kind="port",
                                    sample=f"{side}x{side} outputs x k={low['k']} ({dt:.1f} s)")
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cc8000", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline and DGEMM legs")
    ap.add_argument("--slabs", type=int, default=8, help="slabs of the host-operand pipeline (e2e)")
    ap.add_argument("--exchange", default=None, choices=["residues", "fp64"],
                    help="multi-GPU exchange (default: residues)")
    ap.add_argument("--group", type=int, default=0,
                    help="residue group of the ranks' plans with more than one GPU (0 = as measured best)")
    ap.add_argument("--store-push", default="auto", choices=["auto", "none", "a", "b"],
                    help="residue exchange: operand whose planes the pack kernel stores into peers' buffers")
    ap.add_argument("--sync", default="flags", choices=["barrier", "flags"],
                    help="residue exchange: how consumers learn that planes have landed")
    ap.add_argument("--push-streams", type=int, default=1,
                    help="streams of the residue exchange's peer copies")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world not in GRID:
        raise SystemExit(f"unsupported number of ranks {world}")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
