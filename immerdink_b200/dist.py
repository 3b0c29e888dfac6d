"""One contraction over several GPUs of one node: C's free modes are partitioned, one process per
GPU, one plan per rank. No counterpart in the reference (a single-GPU library); an addition above
the unchanged per-device C ABI.

Every output element depends only on its own row of A and column of B (the shifts are row and
column local), so a rank that owns the tile C[a-slab, b-slab, ...] needs the slab of B that carries
`a` and the slab of A that carries `b`, and no reduction follows: results are bit-identical to the
single-GPU call.

Ownership before the call: A is cut in `world` equal pieces along its label `lb` (a label of A and
C), B likewise along `la`; the pieces of a slab belong to exactly the ranks that consume it.
`gather` brings them together with one NCCL all-gather per operand inside the rank's grid column
(A) or row (B); `RankContraction` is the whole step of one rank: both gathers on a side stream,
operand A packed (`imd_pack`) as soon as its slab is complete and while B's slab is still arriving,
then `imd_contract_packed`. The pieces land
side by side in one buffer [pieces, ...piece shape]; instead of copying them into a dense slab the
plan describes that buffer directly by splitting the label in two (piece index, index inside the
piece), which the strided-tensor front end handles at no cost.
"""
from dataclasses import dataclass

GRID = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}


@dataclass
class Partition:
    """Rank `rank` of `world`: spec 'A,B->C' with single-letter labels, `la` = the label of B and C
    split over the grid rows, `lb` = the label of A and C split over the grid columns."""
    spec: str
    extents: dict
    world: int
    rank: int
    la: str
    lb: str

    def __post_init__(self):
        ins, out = self.spec.replace(" ", "").split("->")
        self.A, self.B = ins.split(",")
        self.C = out
        if not (self.la in self.B and self.la in self.C and self.la not in self.A):
            raise ValueError(f"label {self.la!r} must be in B and C only")
        if not (self.lb in self.A and self.lb in self.C and self.lb not in self.B):
            raise ValueError(f"label {self.lb!r} must be in A and C only")
        self.pa, self.pb = GRID[self.world]
        self.ra, self.rb = self.rank // self.pb, self.rank % self.pb
        for lab, parts in ((self.la, self.world), (self.lb, self.world)):
            if self.extents[lab] % parts:
                raise ValueError(f"extent of {lab!r} ({self.extents[lab]}) must divide by {parts}")
        # pieces: every operand is cut in `world` pieces along its split label
        self.piece_a = self.extents[self.la] // self.world   # piece of B along la
        self.piece_b = self.extents[self.lb] // self.world   # piece of A along lb
        # the rank's tile: grid row ra owns world/pa = pb consecutive la-pieces, column rb owns pa lb-pieces
        self.pieces_a = self.world // self.pa
        self.pieces_b = self.world // self.pb
        self.start = {self.la: self.ra * self.pieces_a * self.piece_a,
                      self.lb: self.rb * self.pieces_b * self.piece_b}
        self.local = dict(self.extents)
        self.local[self.la] = self.pieces_a * self.piece_a
        self.local[self.lb] = self.pieces_b * self.piece_b

    # ---- ownership: the pieces of a slab belong to exactly the ranks that consume it, so that one
    # all-gather inside the column (A) or row (B) group assembles it everywhere it is needed
    def column_group(self):
        """Ranks that share this rank's lb-slab of A, in piece order."""
        return [ra * self.pb + self.rb for ra in range(self.pa)]

    def row_group(self):
        """Ranks that share this rank's la-slab of B, in piece order."""
        return [self.ra * self.pb + rb for rb in range(self.pb)]

    def piece_index(self, operand):
        """Which piece (of `world`) of operand 0 (A, along lb) or 1 (B, along la) this rank owns."""
        return self.rb * self.pa + self.ra if operand == 0 else self.ra * self.pb + self.rb

    def shard_shape(self, operand):
        """Shape of the piece this rank owns of operand 0 (A) or 1 (B)."""
        labs, lab, piece = (self.A, self.lb, self.piece_b) if operand == 0 else (self.B, self.la, self.piece_a)
        return tuple(piece if c == lab else self.extents[c] for c in labs)

    def shard_start(self, operand):
        lab, piece = (self.lb, self.piece_b) if operand == 0 else (self.la, self.piece_a)
        return {lab: self.piece_index(operand) * piece}

    def gathered_shape(self, operand):
        n = self.pieces_b if operand == 0 else self.pieces_a
        return (n,) + self.shard_shape(operand)

    def tile_shape(self):
        return tuple(self.local[c] for c in self.C)

    def plan_layouts(self):
        """(spec, layoutA, layoutB, layoutC) of the rank's contraction on the gathered buffers: the
        split labels become two labels each (piece index X / Y outermost in the gathered operand)."""
        from .device import Layout
        X, Y = "X", "Y"   # piece indices of lb (in A) and la (in B)
        assert X not in self.spec and Y not in self.spec
        specA = X + self.A
        specB = Y + self.B
        specC = self.C.replace(self.la, Y + self.la).replace(self.lb, X + self.lb)
        shapeA, shapeB = self.gathered_shape(0), self.gathered_shape(1)
        shapeC = []
        for c in specC:
            shapeC.append(self.pieces_b if c == X else self.pieces_a if c == Y else
                          self.piece_a if c == self.la else self.piece_b if c == self.lb else
                          self.extents[c])
        return f"{specA},{specB}->{specC}", Layout(shapeA), Layout(shapeB), Layout(tuple(shapeC))


def make_groups(world, dist):
    """Process groups, created by every rank in the same order: one per grid column (the ranks that
    share a slab of A) and one per grid row (a slab of B). Returns ({rb: group}, {ra: group});
    a group of one rank is None."""
    pa, pb = GRID[world]
    cols, rows = {}, {}
    for rb in range(pb):
        ranks = [ra * pb + rb for ra in range(pa)]
        cols[rb] = dist.new_group(ranks) if len(ranks) > 1 else None
    for ra in range(pa):
        ranks = [ra * pb + rb for rb in range(pb)]
        rows[ra] = dist.new_group(ranks) if len(ranks) > 1 else None
    return cols, rows


def gather(part, shard_a, shard_b, out_a, out_b, groups, dist):
    """All-gather this rank's slabs: out_a [pa, ...piece of A] inside its grid column, out_b
    [pb, ...piece of B] inside its grid row. Pieces arrive in slab order."""
    cols, rows = groups
    for out, shard, grp in ((out_a, shard_a, cols[part.rb]), (out_b, shard_b, rows[part.ra])):
        if grp is None:
            out[0].copy_(shard)
        else:
            dist.all_gather_into_tensor(out.view(-1), shard.contiguous().view(-1), group=grp)


class RankContraction:
    """One rank's step of the partitioned contraction: exchange + compute, overlapped.

        side stream   all-gather A | all-gather B
        main stream                | imd_pack(A) ........ | imd_contract_packed(A packed, B in line)

    Owns the gathered buffers, the packed buffer and the workspaces (allocated here, once).
    `dist` is torch.distributed (initialised) and `groups` = make_groups(world, dist); with
    world = 1 the gathers are plain copies. Device memory and streams come from torch."""

    def __init__(self, part, *, N, g=0, rounding="RN", dist=None, groups=None, lib=None):
        import torch
        from . import device as _dev
        self._torch, self.part, self.dist = torch, part, dist
        self.groups = groups if groups is not None else ({part.rb: None}, {part.ra: None})
        dev = torch.device("cuda", torch.cuda.current_device())
        self.A = torch.empty(part.gathered_shape(0), dtype=torch.float64, device=dev)
        self.B = torch.empty(part.gathered_shape(1), dtype=torch.float64, device=dev)
        self.spec, _, _, lc = part.plan_layouts()
        self.tile_shape = lc.shape
        proto = torch.empty(lc.shape, dtype=torch.float64, device=dev)
        self.pack = _dev.Pack(_dev.pack_spec(self.spec, self.A, self.B, proto, operand=0, N=N, g=g,
                                             rounding=rounding, lib=lib), lib=lib)
        self.plan = _dev.Plan(self.spec, self.A, self.B, proto, N=N, g=g, rounding=rounding,
                              packs=(self.pack, None), lib=lib)
        del proto
        nbytes = lambda n: torch.empty(max(int(n), 1), dtype=torch.uint8, device=dev)
        self.packed, self.pack_ws = nbytes(self.pack.pack_bytes), nbytes(self.pack.workspace_bytes)
        self.ws = nbytes(self.plan.workspace_bytes)
        self.side = torch.cuda.Stream(dev)

    def _gather(self, out, shard, grp):
        if grp is None:
            out[0].copy_(shard, non_blocking=True)
        else:
            self.dist.all_gather_into_tensor(out.view(-1), shard.contiguous().view(-1), group=grp)

    def __call__(self, shard_a, shard_b, C, alpha=1.0, beta=0.0):
        """C (this rank's tile, shape `tile_shape`) <- alpha A.B + beta C from the rank's pieces of
        A and B; enqueued on the current stream (and a side stream that joins it)."""
        torch = self._torch
        main = torch.cuda.current_stream()
        cols, rows = self.groups
        self.side.wait_event(main.record_event())
        with torch.cuda.stream(self.side):
            self._gather(self.A, shard_a, cols[self.part.rb])
            a_in = self.side.record_event()
            self._gather(self.B, shard_b, rows[self.part.ra])
            b_in = self.side.record_event()
        main.wait_event(a_in)
        self.pack.pack(self.A, self.packed, workspace=self.pack_ws, stream=main)
        main.wait_event(b_in)
        return self.plan.contract(self.A, self.B, C, alpha=alpha, beta=beta, workspace=self.ws,
                                  stream=main, packed=(self.packed, None))

    def close(self):
        self.plan.close()
        self.pack.close()
