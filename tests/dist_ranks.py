"""Rank program of tests/test_dist_multi_gpu.py (launched with torch.distributed.run, one process per
GPU): the partitioned contraction of immerdink_b200.dist on 2 or 4 GPUs against the single-GPU
call, bit for bit, for every way of exchanging the slabs. One rank's piece of A and another
rank's piece of B hold non-finite entries, so the native path reads FP64 pieces fetched from
peers; every variant runs two steps in a row (the second meets the first one's buffers and
flag words). Plain peer loads and stores only."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

import immerdink_b200 as imd  # noqa: E402
from immerdink_b200 import dist as idist  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    spec = "kjbc,kiac->abij"
    ext = dict(a=32, b=48, c=40, i=6, j=5, k=3)     # a, b divide by 2 and 4; piece rows multiples of 16
    rng = np.random.default_rng(3)
    A = rng.uniform(-1, 1, [ext[c] for c in "kjbc"])
    B = rng.uniform(-1, 1, [ext[c] for c in "kiac"])
    A[1, 2, 5, 7] = np.inf          # b = 5: in the piece of rank 0
    A[0, 0, 47, 3] = np.nan         # b = 47: in the last piece
    B[2, 3, 30, 9] = -np.inf        # a = 30: in a late piece
    dA, dB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
    full = torch.zeros([ext[c] for c in "abij"], dtype=torch.float64, device=dev)
    n = imd.workspace_size(spec, dA, dB, full, N=14, g=5)
    ws = torch.empty(n, dtype=torch.uint8, device=dev)
    imd.contract(spec, dA, dB, full, alpha=1.25, N=14, g=5, workspace=ws)
    torch.cuda.synchronize()

    failures = []
    variants = [dict(exchange="residues", push="kernel"), dict(exchange="residues", push="kernel", push_ctas=4),
                dict(exchange="residues", push="copy"), dict(exchange="residues", push="copy", store_push=0),
                dict(exchange="residues", push="kernel", store_push=1),
                dict(exchange="residues", push="copy", sync="barrier"), dict(exchange="fp64"),
                dict(exchange="pieces"), dict(exchange="pieces", carrier="nccl")]
    # the default grid with every variant; on 4 GPUs also the one-axis grids, where a slab has four
    # producers (three pieces arrive from other ranks, as on a 2 x 4 grid of 8 GPUs)
    runs = [(None, variants, (5, 14))]
    if world == 4:
        few = [dict(exchange="pieces"), dict(exchange="pieces", carrier="nccl"),
               dict(exchange="residues", push="copy"), dict(exchange=None)]
        runs += [((1, 4), few, (5,)), ((4, 1), few, (7,))]
    for grid, kinds, gs in runs:
        part = idist.Partition(spec, ext, world, rank, "a", "b", grid)
        sa, sb = part.shard_start(0), part.shard_start(1)
        ia = [slice(sa.get(c, 0), sa.get(c, 0) + e) for c, e in zip("kjbc", part.shard_shape(0))]
        ib = [slice(sb.get(c, 0), sb.get(c, 0) + e) for c, e in zip("kiac", part.shard_shape(1))]
        shard_a, shard_b = dA[tuple(ia)].contiguous(), dB[tuple(ib)].contiguous()
        tile = tuple(slice(part.start.get(c, 0), part.start.get(c, 0) + part.local[c]) for c in "abij")
        want = full[tile].contiguous()
        groups = idist.make_groups(world, dist, grid)
        for kw in kinds:
            for g in gs:
                rc = idist.RankContraction(part, N=14, g=g, dist=dist, groups=groups, **kw)
                C = torch.full(rc.tile_shape, 7.0, dtype=torch.float64, device=dev)
                for stepno in range(2):
                    C.fill_(7.0)
                    rc(shard_a, shard_b, C, alpha=1.25, beta=0.0)
                    torch.cuda.synchronize()
                    dist.barrier()
                    same = torch.equal(C.reshape(want.shape).view(torch.int64), want.view(torch.int64))
                    err = rc.device_error()
                    if not same or err:
                        failures.append((grid, kw, g, stepno, bool(same), int(err)))
                dist.barrier()
                rc.close()
    bad = torch.tensor([len(failures)], dtype=torch.int64, device=dev)
    dist.all_reduce(bad)
    if failures:
        print(f"rank {rank}: {failures}", file=sys.stderr)
    if rank == 0:
        print("DIST_OK" if int(bad.item()) == 0 else f"DIST_FAILED {int(bad.item())}")
    dist.destroy_process_group()
    sys.exit(0 if int(bad.item()) == 0 else 1)


if __name__ == "__main__":
    main()
