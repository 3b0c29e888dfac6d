"""Multi-rank partition of one contraction (immerdink_b200.dist) on CPU ranks over gloo: every rank
gathers its operand slabs, contracts its tile on the gathered buffers through the split-label
descriptors, and the tiles together equal the undivided result bit for bit. The CPU oracle stands
in for the device library here (host-side logic only)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SPEC = "kjbc,kiac->abij"
EXT = dict(a=8, b=8, c=5, i=2, j=3, k=2)


def _dense(labels, ext):
    st, acc = [], 1
    for c in reversed(labels):
        st.append(acc)
        acc *= ext[c]
    return [ext[c] for c in labels], list(reversed(st))


def _full_problem():
    rng = np.random.default_rng(11)
    A = rng.uniform(-1, 1, [EXT[c] for c in "kjbc"])
    B = rng.uniform(-1, 1, [EXT[c] for c in "kiac"])
    return A, B


def _worker(rank, world, port, out_dir, grid=None):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import imd_oracle as orc
    from immerdink_b200 import dist as idist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    part = idist.Partition(SPEC, EXT, world, rank, "a", "b", grid)
    A, B = _full_problem()
    # this rank's pieces
    sa = part.shard_start(0)["b"]
    sb = part.shard_start(1)["a"]
    shard_a = torch.from_numpy(np.ascontiguousarray(A[:, :, sa:sa + part.piece_b, :]))
    shard_b = torch.from_numpy(np.ascontiguousarray(B[:, :, sb:sb + part.piece_a, :]))
    out_a = torch.empty(part.gathered_shape(0), dtype=torch.float64)
    out_b = torch.empty(part.gathered_shape(1), dtype=torch.float64)
    groups = idist.make_groups(world, dist, grid)
    idist.gather(part, shard_a, shard_b, out_a, out_b, groups, dist)
    spec, la, lb, lc = part.plan_layouts()
    ins, outl = spec.split("->")
    labs = ins.split(",") + [outl]
    descs = [orc.Desc(l.shape, l.strides, [ord(c) for c in lab]) for l, lab in zip((la, lb, lc), labs)]
    tile = orc.contract_tensor(out_a.numpy().reshape(-1), out_b.numpy().reshape(-1),
                               np.zeros(int(np.prod(lc.shape))), descs[0], descs[1], descs[2],
                               1.0, 0.0, 14)
    np.save(os.path.join(out_dir, f"tile{rank}.npy"), tile.reshape(part.tile_shape()))
    np.save(os.path.join(out_dir, f"start{rank}.npy"), np.array([part.start["a"], part.start["b"]]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,grid", [(2, None), (4, None), (8, None), (4, (1, 4)), (4, (4, 1)), (2, (2, 1))])
def test_partition_tiles_equal_the_undivided_result(world, grid, tmp_path):
    """Default grids and one-axis splits (C cut along one label only, the other operand gathered whole)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import imd_oracle as orc
    port = 29500 + world + (os.getpid() % 1000) + (7 if grid else 0) + (grid[0] if grid else 0)
    mp.spawn(_worker, args=(world, port, str(tmp_path), grid), nprocs=world, join=True)
    A, B = _full_problem()
    descs = []
    for lab in ("kjbc", "kiac", "abij"):
        e, s = _dense(lab, EXT)
        descs.append(orc.Desc(e, s, [ord(c) for c in lab]))
    full = orc.contract_tensor(A.reshape(-1), B.reshape(-1), np.zeros(8 * 8 * 2 * 3), *descs, 1.0, 0.0, 14)
    full = full.reshape(8, 8, 2, 3)
    got = np.full_like(full, np.nan)
    for r in range(world):
        t = np.load(tmp_path / f"tile{r}.npy")
        a0, b0 = np.load(tmp_path / f"start{r}.npy")
        got[a0:a0 + t.shape[0], b0:b0 + t.shape[1]] = t
    assert np.array_equal(got.view(np.uint64), full.view(np.uint64))


def test_partition_rejects_labels_of_the_wrong_class():
    sys.path.insert(0, ROOT)
    from immerdink_b200.dist import Partition
    with pytest.raises(ValueError):
        Partition(SPEC, EXT, 2, 0, "k", "b")
    with pytest.raises(ValueError):
        Partition(SPEC, dict(EXT, a=7), 2, 0, "a", "b")
    with pytest.raises(ValueError):
        Partition(SPEC, EXT, 4, 0, "a", "b", (2, 4))          # 8 ranks' grid for a world of 4
    from immerdink_b200.dist import default_grid
    assert [default_grid(w) for w in (1, 2, 3, 4, 6, 7, 8, 12)] == [(1, 1), (1, 2), (1, 3), (2, 2), (2, 3),
                                                                  (1, 7), (2, 4), (3, 4)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_pieces_packed_separately_tile_the_slab_pack(world):
    """The residue exchange's data layout, on the CPU: the pack of every rank's piece (classes and
    orders of the slab's pack without the piece-index label) holds exactly the rows of the slab's
    pack at the piece's row offset; oracle packs, host-library layouts."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import imd_oracle as orc
    from immerdink_b200 import dist as idist, host
    A, B = _full_problem()
    full = (A, B)
    for rank in range(world):
        part = idist.Partition(SPEC, EXT, world, rank, "a", "b")
        spec, la, lb, lc = part.plan_layouts()
        ins, outl = spec.split("->")
        labs = ins.split(",") + [outl]
        descs = tuple(host.Desc(l.shape, l.strides, tuple(ord(c) for c in lab))
                      for l, lab in zip((la, lb, lc), labs))
        for x, (lab, n_pieces, pos, group) in enumerate(((part.lb, part.pieces_b, part.ra, part.column_group()),
                                                         (part.la, part.pieces_a, part.rb, part.row_group()))):
            slab_spec = host.pack_desc_for(descs, operand=x, N=14, g=7)
            piece_spec = idist.piece_pack_spec(part, x, slab_spec)
            assert piece_spec is not None
            sl, pl = host.pack_layout(slab_spec), host.pack_layout(piece_spec)
            assert sl["r"] == n_pieces * pl["r"] and (sl["k"], sl["k_hat"], sl["b"], sl["format"]) == (
                pl["k"], pl["k_hat"], pl["b"], pl["format"])
            # the slab as the group's ranks gather it, and its pack by the oracle
            axis = "kjbc".index(lab) if x == 0 else "kiac".index(lab)
            piece = part.piece_b if x == 0 else part.piece_a
            pieces = []
            for r in group:
                other = idist.Partition(SPEC, EXT, world, r, "a", "b")
                s0 = other.shard_start(x)[lab]
                pieces.append(np.ascontiguousarray(np.take(full[x], range(s0, s0 + piece), axis=axis)))
            slab = np.stack(pieces)
            sv = orc.pack_view(orc.Desc(list(slab_spec.tensor.extent), list(slab_spec.tensor.stride),
                                        list(slab_spec.tensor.label)), slab_spec.contracted,
                               slab_spec.batch, slab_spec.rows, "GIVEN", 14)
            want = orc.pack(slab.reshape(-1), 0, sv)
            pv = orc.pack_view(orc.Desc(list(piece_spec.tensor.extent), list(piece_spec.tensor.stride),
                                        list(piece_spec.tensor.label)), piece_spec.contracted,
                               piece_spec.batch, piece_spec.rows, "GIVEN", 14)
            got = orc.pack(pieces[pos].reshape(-1), 0, pv)
            R, rp, kh, b = sl["r"], pl["r"], sl["k_hat"], sl["b"]
            assert b == 1
            for l in range(14):
                w = want[sl["res"][0] + (l * R + pos * rp) * kh:sl["res"][0] + (l * R + (pos + 1) * rp) * kh]
                g_ = got[pl["res"][0] + l * rp * kh:pl["res"][0] + (l + 1) * rp * kh]
                assert np.array_equal(w, g_), (world, rank, x, l)
            assert np.array_equal(want[sl["sig"][0] + 2 * pos * rp:sl["sig"][0] + 2 * (pos + 1) * rp],
                                  got[pl["sig"][0]:pl["sig"][0] + 2 * rp])


def test_push_order_serves_every_consumer_from_one_producer_per_turn():
    from immerdink_b200.dist import push_order
    for sharers in (2, 3, 4, 8):
        turns = {}
        for own in range(sharers):
            peers = [p for p in range(sharers) if p != own]
            order = push_order(peers, own, sharers)
            assert sorted(order) == list(range(len(peers)))
            for t, j in enumerate(order):
                turns.setdefault(t, []).append(peers[j])
        for t, served in turns.items():
            assert sorted(served) == list(range(sharers)), (sharers, t, served)


def test_default_exchange_by_grid_and_arrival_order_of_pieces():
    """Residue planes up to four ranks, FP64 pieces once a slab has four producers (the default
    grid of 8 ranks, the one-axis grids of 4); a consumer waits for the pieces of the other
    producers in the order in which push_order makes them arrive."""
    from immerdink_b200.dist import Partition, default_exchange, push_order
    ext = dict(a=64, b=64, c=8, i=2, j=2, k=2)
    spec = "kjbc,kiac->abij"
    want = {(1, None): "fp64", (2, None): "residues", (4, None): "residues", (8, None): "pieces",
            (4, (1, 4)): "pieces", (4, (4, 1)): "pieces", (2, (2, 1)): "residues"}
    for (world, grid), name in want.items():
        assert default_exchange(Partition(spec, ext, world, 0, "a", "b", grid)) == name
    # consumer at position c of a slab with n producers: in turn t it is served by producer c - 1 - t
    for n in (2, 4):
        for c in range(n):
            arrival = [(c - 1 - t) % n for t in range(n - 1)]
            for turn, producer in enumerate(arrival):
                others = [q for q in range(n) if q != producer]
                served = [others[j] for j in push_order(others, producer, n)]
                assert served[turn] == c
