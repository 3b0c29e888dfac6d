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
(A) or row (B); `RankContraction` is the whole step of one rank (exchange + compute). The pieces land
side by side in one buffer [pieces, ...piece shape]; instead of copying them into a dense slab the
plan describes that buffer directly by splitting the label in two (piece index, index inside the
piece), which the strided-tensor front end handles at no cost.
"""
import math
from dataclasses import dataclass

GRID = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}     # default grids (rows along la, columns along lb)


def default_grid(world):
    """(pa, pb) with pa * pb = world: the table above, else the most square factorisation with
    pa <= pb (a prime world gives a one-axis split (1, world))."""
    if world in GRID:
        return GRID[world]
    pa = max(d for d in range(1, int(math.isqrt(world)) + 1) if world % d == 0)
    return pa, world // pa

_POSITIONS, _SLOTS = 8, 32      # flag words per operand: producers sharing a slab x (residue groups + FP64)


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
    grid: tuple = None   # (pa, pb), pa * pb = world; None = default_grid(world). (1, world) splits C
    #                      along lb only (every rank gathers all of B), (world, 1) along la only

    def __post_init__(self):
        ins, out = self.spec.replace(" ", "").split("->")
        self.A, self.B = ins.split(",")
        self.C = out
        if not (self.la in self.B and self.la in self.C and self.la not in self.A):
            raise ValueError(f"label {self.la!r} must be in B and C only")
        if not (self.lb in self.A and self.lb in self.C and self.lb not in self.B):
            raise ValueError(f"label {self.lb!r} must be in A and C only")
        self.pa, self.pb = self.grid if self.grid is not None else default_grid(self.world)
        if self.pa < 1 or self.pb < 1 or self.pa * self.pb != self.world:
            raise ValueError(f"grid {self.grid!r} does not have world = {self.world} ranks")
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


def make_groups(world, dist, grid=None):
    """Process groups, created by every rank in the same order: one per grid column (the ranks that
    share a slab of A) and one per grid row (a slab of B). Returns ({rb: group}, {ra: group});
    a group of one rank is None. `grid` as in Partition."""
    pa, pb = grid if grid is not None else default_grid(world)
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


def default_exchange(part):
    """The exchange RankContraction uses when none is named: residue planes group by group up to
    four ranks (measured: 3.53 ms on 2 and 2.00 ms on 4 B200 against 3.53 and 2.02 ms for the pieces);
    FP64 pieces once a slab has four producers: the planes of three other producers reach a
    consumer through one copy-engine stream at about 350 GB/s while the GEMM runs, which bounds
    the step (1.49 ms on 8 B200), whereas the pieces are 8 bytes per entry instead of 14, travel in
    a few large copies before any GEMM starts, and their quantisation at the consumer costs less
    than the difference (1.37 ms)."""
    if part.world == 1:
        return "fp64"
    return "pieces" if max(part.pa, part.pb) >= 4 else "residues"


def push_order(peer_positions, own_position, sharers):
    """Order (indices into `peer_positions`) in which the producer at `own_position` of a slab with
    `sharers` consumers serves the others: the one after itself first, then round. In turn t every
    producer serves the consumer t + 1 places after it, so no two producers serve one consumer at
    the same time."""
    return sorted(range(len(peer_positions)),
                  key=lambda j: (peer_positions[j] - own_position) % sharers)


def piece_pack_spec(part, x, slab_spec):
    """The GIVEN pack spec of a rank's piece of operand x (0 = A, 1 = B): the classes and orders of
    the slab's pack spec (`slab_spec`, of the gathered layout of Partition.plan_layouts) without the
    piece-index label, on the piece's own dense descriptor. The rows of piece p are then rows
    [p r, (p + 1) r) of the slab's packed layout. None when the piece index is not the slowest
    row mode of the slab (the rows of a piece would not be contiguous in the slab)."""
    from . import host
    piece_label = ord("X" if x == 0 else "Y")
    rows = list(slab_spec.rows)
    kept = [l for l, e in zip(slab_spec.tensor.label, slab_spec.tensor.extent) if e != 1]
    if piece_label in kept and [l for l in rows if l in kept][-1] != piece_label:
        return None
    if piece_label in slab_spec.contracted or piece_label in slab_spec.batch:
        return None
    shape = part.shard_shape(x)
    labels = tuple(ord(c) for c in (part.A if x == 0 else part.B))
    return host.PackSpec(host.Desc(shape, host.dense_strides(shape), labels),
                         tuple(slab_spec.contracted), tuple(slab_spec.batch),
                         tuple(l for l in rows if l != piece_label), slab_spec.N,
                         slab_spec.rounding, "GIVEN")


class RankContraction:
    """One rank's step of the partitioned contraction: exchange + compute, overlapped. Two ways to
    exchange (`exchange`):

    "residues" (the default with more than one rank): every rank quantises only ITS pieces of A
    and B, once, for all N moduli, and the pack kernels store the shifts, flags and int8 residue
    planes into its own packed slab buffers (`imd_pack_scatter`: the rows of a piece at their place
    in the slab); copy engines then push those rows into the packed slab buffers of the other
    consumers of the slab (peers' memory mapped through CUDA IPC, one contiguous peer copy per plane on a
    side stream: no SM is taken from the persistent GEMM), residue group by residue group, so the
    GEMM of one group runs while the planes of the next travel. No rank repeats another's
    quantisation. The operand whose slab has more consumers is packed first, so that its planes
    travel while the other is being packed. The FP64 values, which only the native path of
    non-finite rows reads, do not travel at all in the usual case: every rank stages its pieces in
    a buffer the others have mapped, and a consumer fetches them (imd_copy_if_flagged, peer loads)
    only if a row flag of its slabs is set:

        main   barrier | pack B | pack A | group 0 in, GEMM 0 | group 1 in, GEMM 1 | CRT | fetch if flagged, native path
        side           | push B group 0 | push A group 0, B group 1 ... | stage FP64 pieces |

    How a consumer learns that a group's planes have landed (`sync`): "barrier" = every rank waits
    for its own copies and the ranks meet in a tiny NCCL all-reduce per group; "flags" = after the
    copies to a consumer the producer's stream copies the step's number into a flag word in that
    consumer's memory, and the consumer's stream polls its flag words with a bounded wait
    (imd_wait_flags: a wait that runs out sets the device error word, the stream moves on); one
    all-reduce per step remains, before the slabs are overwritten.

    "pieces": the FP64 pieces themselves travel (8 bytes per entry instead of N), one contiguous
    peer copy per piece and consumer on the copy engines, announced by flag words; every consumer
    quantises the pieces of its slabs as they arrive (imd_pack_scatter on the rows of a piece: its
    own pieces first, while the others are on their way), then runs the whole contraction from
    the packed slabs in the plan's own residue groups. A rank repeats the quantisation of the
    other consumers of its slabs, but no GEMM launch waits for a transfer:

        main   barrier | pack own B, own A | piece in, pack | piece in, pack ... | GEMMs | CRT | native path
        side           | push own pieces to the other consumers |

    "fp64": the slabs are all-gathered as FP64 (NCCL, side stream), A is packed as soon as its
    slab is complete and while B's is still arriving, B is quantised in line.

    Owns its buffers (allocated here, once). `dist` is torch.distributed (initialised) and
    `groups` = make_groups(world, dist); with world = 1 nothing is exchanged. Device memory and
    streams come from torch; the buffers peers write into are cudaMalloc allocations opened by
    the peers through CUDA IPC (cuda-python)."""

    def __init__(self, part, *, N, g=0, rounding="RN", dist=None, groups=None, lib=None,
                 exchange=None, push_streams=1, sync="flags", store_push="auto", push="copy",
                 push_ctas=0, carrier="copy"):
        import torch
        from . import device as _dev
        self._torch, self.part, self.dist = torch, part, dist
        self.trace = None
        self.groups = groups if groups is not None else ({part.rb: None}, {part.ra: None})
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        self.spec, la_, lb_, lc = part.plan_layouts()
        self.tile_shape = lc.shape
        nbytes = lambda n: torch.empty(max(int(n), 1), dtype=torch.uint8, device=dev)
        self.side = torch.cuda.Stream(dev)
        # The default exchange by grid: see default_exchange().
        self.exchange = exchange or default_exchange(part)
        lays = (la_, lb_, lc)
        specs = [_dev.pack_spec(self.spec, *lays, operand=x, N=N, g=g, rounding=rounding, lib=lib)
                 for x in (0, 1)]
        if self.exchange not in ("residues", "pieces", "fp64"):
            raise ValueError("exchange must be 'residues', 'pieces' or 'fp64'")
        if self.exchange in ("residues", "pieces"):
            pieces = [piece_pack_spec(part, x, specs[x]) for x in (0, 1)]
            if any(p is None for p in pieces):
                self.exchange = "fp64"      # the piece index is not the slowest row mode
        if self.exchange == "fp64":
            self.A = torch.empty(part.gathered_shape(0), dtype=torch.float64, device=dev)
            self.B = torch.empty(part.gathered_shape(1), dtype=torch.float64, device=dev)
            self.pack = _dev.Pack(specs[0], lib=lib)
            self.plan = _dev.Plan(self.spec, *lays, N=N, g=g, rounding=rounding,
                                  packs=(self.pack, None), lib=lib)
            self.packed, self.pack_ws = nbytes(self.pack.pack_bytes), nbytes(self.pack.workspace_bytes)
        else:
            self.slab = [_dev.Pack(sp, lib=lib) for sp in specs]          # keys of the plan's slots
            self.piece = [_dev.Pack(sp, lib=lib) for sp in pieces]        # what this rank packs
            self.plan = _dev.Plan(self.spec, *lays, N=N, g=g, rounding=rounding,
                                  packs=tuple(self.slab), lib=lib)
            self.pack_ws = [nbytes(pk.workspace_bytes) for pk in self.piece]
            self.pack_ws2 = [nbytes(pk.workspace_bytes) for pk in self.piece]   # packs on the side stream
            self.gather_stream = torch.cuda.Stream(dev)
            self.slab_rows = [pk.layout["r"] for pk in self.slab]
            # this rank's piece inside each slab: its position in the group that shares the slab
            self.pos = (part.ra, part.rb)
            self.row0 = [self.pos[x] * self.piece[x].layout["r"] for x in (0, 1)]
            for x in (0, 1):
                n = part.pieces_b if x == 0 else part.pieces_a
                assert self.slab_rows[x] == n * self.piece[x].layout["r"], "pieces do not tile the slab"
            self._map_peers()
            # copies to different peers may go to different streams (copy engines); one by default
            self.push_streams = [torch.cuda.Stream(dev) for _ in range(max(1, int(push_streams)))]
            # store_push = the operand (0 = A, 1 = B) whose planes the pack kernel itself stores into the
            # other consumers' buffers (NVLink stores) instead of the copy engines, or None
            # push = "copy" (default): the planes travel by the copy engines, one cudaMemcpyAsync per
            # plane and flag; push = "kernel": by imd_push_ranges (a few CTAs, NVLink stores, one launch
            # per operand and residue group that also sets the consumers' flag words). Measured on 2 and
            # 4 GPUs: the copy kernel's stores stall the GEMM that runs beside it (0 - 40 % of its
            # normal progress), copy-engine transfers do not; more than one copy stream delays the
            # first group (2.09 ms with one stream, 2.44 with two, 2.70 with four at 4 GPUs)
            if push not in ("kernel", "copy"):
                raise ValueError("push must be 'kernel' or 'copy'")
            self.push, self.push_ctas = push, int(push_ctas)
            # carrier of the FP64 pieces in the piece exchange: "copy" = one peer copy per piece and
            # consumer on the copy engines, announced by flag words; "nccl" = one all-gather per
            # operand inside the group that shares its slab (side stream)
            if carrier not in ("copy", "nccl"):
                raise ValueError("carrier must be 'copy' or 'nccl'")
            self.carrier = carrier
            if push == "kernel" and sync != "flags":
                raise ValueError("push='kernel' announces by flag words: sync must be 'flags'")
            if store_push == "auto":   # one copy-engine stream carries about 350 GB/s in 8 MB copies: with
                # three other consumers of one slab, the other slab's planes go by stores
                store_push = None if (push == "kernel" or max(part.pa, part.pb) < 4) else \
                    (0 if part.pa < part.pb else 1)
            if store_push not in (None, 0, 1):
                raise ValueError("store_push must be 'auto', None, 0 or 1")
            self.store_push = store_push
            # every producer of a slab starts with the consumer after itself and goes round, so that
            # at any time a consumer receives from one producer (and not all producers send to the
            # first consumer at once)
            self.push_order = [push_order(self.peer_pos[x], self.pos[x],
                                          part.pieces_b if x == 0 else part.pieces_a) for x in (0, 1)]
            self.tick = torch.zeros(1, dtype=torch.int32, device=dev)
            if sync not in ("barrier", "flags"):
                raise ValueError("sync must be 'barrier' or 'flags'")
            self.sync = sync
            self.lib = self.slab[0].lib
            # flags: the value a producer copies into a consumer's flag word after its planes
            self.values = torch.arange(1 << 16, dtype=torch.int32, device=dev)
            self.step = 0
            # the device error word of the previous steps, mirrored into pinned host memory at the end
            # of every step (imd_device_error_peek): a bounded flag wait that gave up surfaces as an
            # exception from a later call instead of a silently wrong tile
            self._err_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            low = self.plan.lowering
            gg, NN = low["residue_group"], low["num_moduli"]
            self.groups_of_planes = [(l0, min(gg, NN - l0)) for l0 in range(0, NN, gg)]
            assert len(self.groups_of_planes) < _SLOTS, "one flag word per residue group and one for the FP64 pieces"
        self.ws = nbytes(self.plan.workspace_bytes)

    # -- set-up of the residue exchange ---------------------------------------------------------
    def _map_peers(self):
        """Allocates the buffers peers write into (per operand: the packed slab and the gathered
        FP64 slab; plain cudaMalloc allocations, so that an IPC handle names exactly the buffer)
        and opens the other consumers' buffers through CUDA IPC WITH THIS RANK'S DEVICE CURRENT:
        the mapping then belongs to this device's context and its kernels and copy engines may
        write through it (a mapping opened under the exporting device's index, as tensor sharing
        does, is not addressable from kernels of another device). Sets self.packed, self.A, self.B
        and, per operand, the destination pointers (own buffer first)."""
        from cuda.bindings import runtime as rt
        from ._arrays import DeviceArray
        torch, part = self._torch, self.part
        ok = rt.cudaError_t.cudaSuccess

        self._rt, self._owned, self._opened = rt, [], []
        failure = None
        shapes = [part.gathered_shape(0), part.gathered_shape(1)]
        sizes = [(pk.pack_bytes + 255) // 256 * 256 or 256 for pk in self.slab] + \
                [max(8 * math.prod(sh), 256) for sh in shapes] + [4 * 2 * _POSITIONS * _SLOTS]
        for n in sizes:
            err, ptr = rt.cudaMalloc(n)
            if err != ok:
                failure = f"cudaMalloc of a shared buffer of {n} bytes: {err}"
                break
            self._owned.append(int(ptr))
        if failure and part.world == 1:
            raise RuntimeError(failure)
        while len(self._owned) < 5:
            self._owned.append(0)           # placeholders: the ranks fail together below
        if not failure:
            err, = rt.cudaMemset(self._owned[4], 0, sizes[4])
            if err != ok:
                failure = f"cudaMemset of the flag words: {err}"
        self.packed = [(self._owned[x], sizes[x]) for x in (0, 1)]
        self.A = self.B = None
        if not failure:
            self.A, self.B = (torch.as_tensor(DeviceArray(self._owned[2 + x], shapes[x]), device=self.device)
                              for x in (0, 1))
        self.dests = [[self._owned[x]] for x in (0, 1)]          # packed slabs
        self.fp64_dests = [[self._owned[2 + x]] for x in (0, 1)]  # gathered FP64 slabs
        self.flags = self._owned[4]                              # [operand][producer position][slot] words
        self.flag_dests = [[], []]                               # the other consumers' flag words
        self.peer_pos = [[], []]                                 # their positions in the slab
        if part.world == 1:
            return
        # Every rank goes through both collectives whatever fails locally, and all ranks fail together.
        mine = []
        for ptr in self._owned:
            err, handle = (ok, None) if failure else rt.cudaIpcGetMemHandle(ptr)
            if failure:
                mine.append(b"")
            elif err != ok:
                failure = failure or f"cudaIpcGetMemHandle: {err}"
                mine.append(b"")
            else:
                mine.append(bytes(handle.reserved))
        everyone = [None] * part.world
        self.dist.all_gather_object(everyone, mine)
        sharers = (part.column_group(), part.row_group())     # ranks that consume the slab of A / B
        for x in (0, 1):
            for position, r in enumerate(sharers[x]):
                if r == part.rank or failure:
                    continue
                self.peer_pos[x].append(position)
                for which, out in ((x, self.dests[x]), (2 + x, self.fp64_dests[x]), (4, self.flag_dests[x])):
                    if len(everyone[r][which]) != 64:
                        failure = f"rank {r} exported no handle"
                        break
                    handle = rt.cudaIpcMemHandle_t()
                    handle.reserved = everyone[r][which]
                    err, ptr = rt.cudaIpcOpenMemHandle(handle, rt.cudaIpcMemLazyEnablePeerAccess)
                    if err != ok:
                        failure = f"cudaIpcOpenMemHandle of rank {r}'s buffer: {err}"
                        break
                    self._opened.append(int(ptr))
                    out.append(int(ptr))
        bad = torch.tensor([1 if failure else 0], dtype=torch.int32, device=self.device)
        self.dist.all_reduce(bad, op=self.dist.ReduceOp.MAX)
        if int(bad.item()):
            rt.cudaGetLastError()
            for ptr in self._opened:
                rt.cudaIpcCloseMemHandle(ptr)
            self.dist.barrier()
            for ptr in self._owned:
                if ptr:
                    rt.cudaFree(ptr)
            self._owned, self._opened = [], []
            self.A = self.B = None
            raise RuntimeError("residue exchange: peer buffers could not be mapped" +
                               (f" ({failure})" if failure else " (on another rank)"))

    def _mark(self, label, stream):
        """With `self.trace` a list: appends (label, timing event recorded on `stream`), to lay out
        one step on a time line afterwards."""
        if self.trace is not None:
            ev = self._torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            self.trace.append((label, ev))

    def _barrier(self):
        if self.part.world > 1:
            self.dist.all_reduce(self.tick)     # stream-ordered: no rank passes before all arrive

    def _gather(self, out, shard, grp):
        if grp is None:
            out[0].copy_(shard, non_blocking=True)
        else:
            self.dist.all_gather_into_tensor(out.view(-1), shard.contiguous().view(-1), group=grp)

    # -- the step ---------------------------------------------------------------------------------
    def __call__(self, shard_a, shard_b, C, alpha=1.0, beta=0.0):
        """C (this rank's tile, shape `tile_shape`) <- alpha A.B + beta C from the rank's pieces of
        A and B; enqueued on the current stream (and a side stream that joins it)."""
        torch = self._torch
        main = torch.cuda.current_stream()
        cols, rows = self.groups
        if self.exchange == "pieces":
            return self._step_pieces(shard_a, shard_b, C, alpha, beta)
        if self.exchange == "fp64":
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
        from .device import copy_if_flagged as _dev_copy_if, push_ranges as _dev_push, wait_flags as _dev_wait
        rt, s = self._rt, main.cuda_stream
        if int(self._err_host[0]) != 0:
            word = self.device_error()        # synchronises and clears
            self._err_host[0] = 0
            raise RuntimeError(f"residue exchange: device error word {word:#x} after an earlier step (bit 2: a "
                               "producer's planes did not arrive within the bounded wait); the tiles of that "
                               "step and of those enqueued since are not valid: repeat them")
        shards = (shard_a, shard_b)
        kind = rt.cudaMemcpyKind.cudaMemcpyDeviceToDevice
        # copies to different peers may go to different streams; all copies to one peer share one
        pushes = self.push_streams
        flags = self.sync == "flags" and self.part.world > 1
        self.step = self.step % 65535 + 1     # 1..65535: never the value of an untouched flag word
        tick = self.step

        turn = [0]

        def copy(j, dst, src, nbytes, on=None):
            """One peer copy. Copies go to the push streams in turn (whatever their destination),
            so that the fixed cost of one copy overlaps the transfer of another; `on` pins a stream."""
            st = pushes[(turn[0] if on is None else on) % len(pushes)]
            turn[0] += 1
            err, = rt.cudaMemcpyAsync(dst, src, nbytes, kind, st.cuda_stream)
            if err != rt.cudaError_t.cudaSuccess:
                raise RuntimeError(f"cudaMemcpyAsync to a peer: {err}")

        def join():
            """Stream 0 of the pushes waits for what the others hold so far."""
            for st in pushes[1:]:
                pushes[0].wait_event(st.record_event())

        def copy_rows(j, dst, src, off, rows, width, pitch):
            """`rows` runs of `width` bytes, `pitch` apart: contiguous copies (a few large runs;
            pitched copies between peers were several times slower)."""
            if rows == 0 or width == 0:
                return
            if width == pitch:
                rows, width = 1, rows * width
            for r in range(rows):
                copy(j, dst + off + r * pitch, src + off + r * pitch, width)

        def word(x, position, slot):          # offset of a flag word inside a rank's flag buffer
            return 4 * ((x * _POSITIONS + position) * _SLOTS + slot)

        def announce(x, j, slot):             # after the copies to consumer j of slab x: its flag word
            if flags:                         # on stream 0, which has joined the other push streams
                copy(j, self.flag_dests[x][j] + word(x, self.pos[x], slot),
                     self.values.data_ptr() + 4 * tick, 4, on=0)

        def await_(slot):                     # every other producer's copies of this slot have landed here
            ptrs = [self.flags + word(x, p, slot)
                    for x, n in ((0, self.part.pieces_b), (1, self.part.pieces_a))
                    for p in range(n) if p != self.pos[x]]
            _dev_wait(ptrs, tick, stream=s, lib=self.lib)

        self._mark("begin", main)
        self._barrier()                       # every rank is done with the previous step's slabs
        self._mark("all ranks in", main)
        # the operand whose slab has more consumers is packed first: its planes travel while the
        # other operand is being packed
        order = (1, 0) if self.part.pb > self.part.pa else (0, 1)
        packed_ev = [None, None]
        for x in order:                       # own pieces into the own slab buffers: shifts, flags, all planes
            if (tuple(shards[x].shape) != tuple(self.part.shard_shape(x)) or not shards[x].is_contiguous()
                    or shards[x].dtype != torch.float64):
                raise ValueError("the rank's pieces must be dense FP64 arrays of Partition.shard_shape")
            self.piece[x].scatter_ptr(shards[x].data_ptr(), self.slab_rows[x], self.row0[x],
                                      self.dests[x] if x == self.store_push else self.dests[x][:1],
                                      self.slab[x].pack_bytes,
                                      self.pack_ws[x].data_ptr(), self.pack_ws[x].numel(), s)
            packed_ev[x] = main.record_event()
            self._mark(f"packed {'AB'[x]}", main)
        # copy engines push the rows of the own pieces to the other consumers, group by group (the
        # first group of the operand packed first already while the other is being packed)
        arrived = []
        by_kernel = self.push == "kernel" and flags
        for gi, (l0, mods) in enumerate(self.groups_of_planes):
            for x in order:
                if not self.push_order[x]:    # nobody else consumes this slab
                    continue
                if gi == 0:
                    for st in pushes:
                        st.wait_event(packed_ev[x])
                lay, R, b = self.slab[x].layout, self.slab_rows[x], self.slab[x].layout["b"]
                rp, kh = self.piece[x].layout["r"], lay["k_hat"]
                own = self.dests[x][0]
                ranges, words = [], []        # push = "kernel": the operand's planes of the group in one launch
                for j in self.push_order[x]:
                    dst = self.dests[x][1 + j]
                    if x == self.store_push:  # the pack kernel has stored the planes there already
                        if by_kernel:
                            words.append(self.flag_dests[x][j] + word(x, self.pos[x], gi))
                        else:
                            announce(x, j, gi)
                        continue
                    if gi == 0:               # shifts and flags: a few KB, by the copy engine
                        copy_rows(j, dst, own, lay["sig"][0] + 2 * self.row0[x], b, 2 * rp, 2 * R)
                        copy_rows(j, dst, own, lay["flag"][0] + self.row0[x], b, rp, R)
                    if by_kernel:
                        off, width, pitch = lay["res"][0] + (l0 * b * R + self.row0[x]) * kh, rp * kh, R * kh
                        runs = [(off, mods * b * width)] if width == pitch else \
                               [(off + r * pitch, width) for r in range(mods * b)]
                        ranges += [(dst + o, own + o, n) for o, n in runs if n]
                        words.append(self.flag_dests[x][j] + word(x, self.pos[x], gi))
                    else:
                        copy_rows(j, dst, own, lay["res"][0] + (l0 * b * R + self.row0[x]) * kh, mods * b,
                                  rp * kh, R * kh)
                if not by_kernel and x != self.store_push:
                    join()                    # every plane of the group has left before a flag is set
                    for j in self.push_order[x]:
                        announce(x, j, gi)
                if by_kernel and (ranges or words):
                    for at in range(0, max(len(ranges), 1), 96):   # one launch unless there are more runs
                        last = at + 96 >= len(ranges)
                        _dev_push(ranges[at:at + 96], words if last else [], tick, ctas=self.push_ctas,
                                  stream=pushes[0].cuda_stream, lib=self.lib)
            arrived.append(None if flags else [st.record_event() for st in pushes])
            self._mark(f"pushed group {gi}", pushes[0])
        # FP64 pieces: only the native path of non-finite rows reads them. Every rank stages its
        # pieces in its own shared buffer (a local copy, behind the planes) and tells the other
        # consumers; a consumer fetches them only if a row flag of its slabs is set (below).
        piece_bytes = [shards[x].numel() * 8 for x in (0, 1)]
        for x in (0, 1):
            copy(0, self.fp64_dests[x][0] + self.pos[x] * piece_bytes[x], shards[x].data_ptr(), piece_bytes[x], on=0)
        for x in (0, 1):
            for j in range(len(self.flag_dests[x])):
                announce(x, j, _SLOTS - 1)
        fp64_in = [st.record_event() for st in pushes]
        self._mark("pushed fp64", pushes[0])
        packed = tuple(self.packed)
        if tuple(C.shape) != tuple(self.tile_shape) or not C.is_contiguous() or C.dtype != torch.float64:
            raise ValueError("C must be the rank's dense FP64 tile")
        ptrs = (self.A.data_ptr(), self.B.data_ptr(), C.data_ptr(), self.ws.data_ptr(), self.ws.numel())

        def run(part):                        # raw pointers: the C checks only, little host time per call
            self.plan.contract_ptr(alpha, ptrs[0], ptrs[1], beta, ptrs[2], ptrs[3], ptrs[4], s,
                                   packed=packed, part=part)
            return C
        for gi, evs in enumerate(arrived):
            if flags:
                await_(gi)                    # the other producers' planes of this group have landed here
            else:
                for ev in evs:
                    main.wait_event(ev)
                self._barrier()               # every rank's planes of this group have landed
            self._mark(f"group {gi} in", main)
            run(16 + gi)                      # GEMM of the group, while the next group's planes travel
            self._mark(f"gemm {gi}", main)
        run(3)                                # CRT of the emulated outputs
        self._mark("crt", main)
        for ev in fp64_in:                    # the own pushes are done before the next step repacks
            main.wait_event(ev)
        if flags:
            await_(_SLOTS - 1)
        else:
            self._barrier()                   # every rank's FP64 pieces have landed
        self._mark("fp64 staged", main)
        fetch = [(self.fp64_dests[x][0] + p * piece_bytes[x], self.fp64_dests[x][1 + j] + p * piece_bytes[x],
                  piece_bytes[x]) for x in (0, 1) for j, p in enumerate(self.peer_pos[x])]
        if fetch:                             # the others' FP64 pieces, only if a row of the slabs is flagged
            rows = [(self.dests[x][0] + self.slab[x].layout["flag"][0],
                     self.slab[x].layout["b"] * self.slab_rows[x]) for x in (0, 1)]
            _dev_copy_if(rows, fetch, stream=s, lib=self.lib)
        run(2)                                # native path of non-finite rows and columns
        if flags:
            st = self.lib.lib.imd_device_error_peek(self._err_host.data_ptr(), s)
            if st:
                raise RuntimeError(f"imd_device_error_peek: status {st}")
        self._mark("end", main)
        return C

    def _step_pieces(self, shard_a, shard_b, C, alpha, beta):
        """The step of the "pieces" exchange (see the class text)."""
        from .device import copy_if_flagged as _dev_copy_if, wait_flags as _dev_wait
        torch, rt = self._torch, self._rt
        main = torch.cuda.current_stream()
        s = main.cuda_stream
        if int(self._err_host[0]) != 0:
            word = self.device_error()        # synchronises and clears
            self._err_host[0] = 0
            raise RuntimeError(f"piece exchange: device error word {word:#x} after an earlier step (bit 2: a "
                               "producer's piece did not arrive within the bounded wait); the tiles of that "
                               "step and of those enqueued since are not valid: repeat them")
        shards = (shard_a, shard_b)
        for x in (0, 1):
            if (tuple(shards[x].shape) != tuple(self.part.shard_shape(x)) or not shards[x].is_contiguous()
                    or shards[x].dtype != torch.float64):
                raise ValueError("the rank's pieces must be dense FP64 arrays of Partition.shard_shape")
        if tuple(C.shape) != tuple(self.tile_shape) or not C.is_contiguous() or C.dtype != torch.float64:
            raise ValueError("C must be the rank's dense FP64 tile")
        kind = rt.cudaMemcpyKind.cudaMemcpyDeviceToDevice
        push = self.push_streams[0]
        self.step = self.step % 65535 + 1
        tick = self.step
        slot = _SLOTS - 1
        pieces_of = (self.part.pieces_b, self.part.pieces_a)     # pieces of the slab of A, of B
        piece_bytes = [shards[x].numel() * 8 for x in (0, 1)]

        def copy(dst, src, nbytes, st):
            err, = rt.cudaMemcpyAsync(dst, src, nbytes, kind, st.cuda_stream)
            if err != rt.cudaError_t.cudaSuccess:
                raise RuntimeError(f"cudaMemcpyAsync to a peer: {err}")

        def word(x, position):
            return 4 * ((x * _POSITIONS + position) * _SLOTS + slot)

        self._mark("begin", main)
        self._barrier()                       # every rank is done with the previous step's slabs
        self._mark("all ranks in", main)
        start = main.record_event()
        order = (1, 0) if self.part.pb > self.part.pa else (0, 1)
        gathered = [None, None]
        if self.carrier == "nccl" and self.part.world > 1:
            # one all-gather per operand inside the group that shares its slab, the larger group
            # first; the pieces land at their place in the gathered FP64 slabs (the own one too)
            cols, rows = self.groups
            grp = (cols[self.part.rb], rows[self.part.ra])
            slabs = (self.A, self.B)
            self.gather_stream.wait_event(start)
            with torch.cuda.stream(self.gather_stream):
                for x in order:
                    if grp[x] is None:
                        slabs[x][0].copy_(shards[x], non_blocking=True)
                    else:
                        self.dist.all_gather_into_tensor(slabs[x].view(-1), shards[x].view(-1), group=grp[x])
                    gathered[x] = self.gather_stream.record_event()
            sent = gathered[order[1]]
        else:
            for st in self.push_streams:
                st.wait_event(start)
            # the slab with more consumers first; every producer serves the consumer after itself
            # first; the copies go to the push streams in turn (a piece and its flag word on the same one)
            nth = 0
            for x in order:
                for j in self.push_order[x]:
                    st = self.push_streams[nth % len(self.push_streams)]
                    nth += 1
                    copy(self.fp64_dests[x][1 + j] + self.pos[x] * piece_bytes[x], shards[x].data_ptr(),
                         piece_bytes[x], st)
                    copy(self.flag_dests[x][j] + word(x, self.pos[x]), self.values.data_ptr() + 4 * tick, 4, st)
            for st in self.push_streams[1:]:
                push.wait_event(st.record_event())
            sent = push.record_event()
        self._mark("pushed", self.gather_stream if gathered[0] is not None else push)

        # The packs alternate between the main stream and a side stream: a pack of 1000 rows fills
        # the GPU for one wave and a third, two of them running side by side fill each other's tail
        lanes = [(main, s, self.pack_ws), (self.side, self.side.cuda_stream, self.pack_ws2)]
        self.side.wait_event(main.record_event())
        turn = [0]

        def pack(x, src, position, wait_for=None):
            stream, handle, wss = lanes[turn[0] % 2]
            turn[0] += 1
            if wait_for is not None and gathered[x] is not None:
                stream.wait_event(gathered[x])            # the operand's all-gather has completed
            elif wait_for is not None:
                _dev_wait([wait_for], tick, stream=handle, lib=self.lib)
            rp = self.piece[x].layout["r"]
            self.piece[x].scatter_ptr(src, self.slab_rows[x], position * rp, self.dests[x][:1],
                                      self.slab[x].pack_bytes, wss[x].data_ptr(), wss[x].numel(), handle)

        for x in order:                       # own pieces: nothing to wait for
            pack(x, shards[x].data_ptr(), self.pos[x])
        self._mark("packed own", main)
        for x in order:                       # the others in the order in which they arrive here
            n = pieces_of[x]
            for t in range(n - 1):
                position = (self.pos[x] - 1 - t) % n
                pack(x, self.fp64_dests[x][0] + position * piece_bytes[x], position,
                     wait_for=self.flags + word(x, position))
        main.wait_event(self.side.record_event())
        self._mark("packed all", main)
        # the own pieces at their place in the own FP64 slabs: only the native path of flagged rows
        # reads them, so they are copied only if a row flag of the slabs is set
        rows = [(self.dests[x][0] + self.slab[x].layout["flag"][0],
                 self.slab[x].layout["b"] * self.slab_rows[x]) for x in (0, 1)]
        own = [(self.fp64_dests[x][0] + self.pos[x] * piece_bytes[x], shards[x].data_ptr(), piece_bytes[x])
               for x in (0, 1)]
        if gathered[0] is None:
            _dev_copy_if(rows, own, stream=s, lib=self.lib)
        main.wait_event(sent)                 # the shards may change once the step's work is done
        self.plan.contract_ptr(alpha, self.A.data_ptr(), self.B.data_ptr(), beta, C.data_ptr(),
                               self.ws.data_ptr(), self.ws.numel(), s, packed=tuple(self.packed))
        st = self.lib.lib.imd_device_error_peek(self._err_host.data_ptr(), s)
        if st:
            raise RuntimeError(f"imd_device_error_peek: status {st}")
        self._mark("end", main)
        return C

    def device_error(self):
        """Reads and clears the device error word (synchronises the device): nonzero when a
        bounded wait gave up, e.g. bit 2 (4) when a producer's planes did not arrive within about
        a second; the step that saw it computed on incomplete slabs and must be repeated."""
        from .device import load_library
        lib = getattr(self, "lib", None) or load_library(None)
        return lib.device_error()

    def close(self):
        """Releases plans, packs and, with the residue exchange, the mappings and buffers (call it
        on every rank, once no step is in flight anywhere)."""
        self.plan.close()
        for pk in ([self.pack] if self.exchange == "fp64" else self.slab + self.piece):
            pk.close()
        if self.exchange in ("residues", "pieces") and getattr(self, "_owned", None):
            self._torch.cuda.synchronize()
            for ptr in self._opened:
                self._rt.cudaIpcCloseMemHandle(ptr)
            if self.part.world > 1:
                self.dist.barrier()         # nobody frees a buffer a peer still has mapped
            self.A = self.B = None
            for ptr in self._owned:
                self._rt.cudaFree(ptr)
            self._owned, self._opened = [], []
