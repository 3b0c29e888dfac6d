"""Seeded random contractions (random label sets, ranks, extents, memory orders, padding, negative
strides, diagonals, batches; random N, rounding, residue group, alpha, beta; a few non-finite
entries) through the C ABI against the CPU oracle's tensor front end, bit for bit; statuses of
illegal draws must agree too. A quarter of the legal emulated cases are also run through packs."""
import random

import numpy as np
import pytest

import imd_oracle as orc
from golden_util import same_bits

pytestmark = pytest.mark.gpu

LABELS = "abcdefgh"


def draw(seed):
    rng = random.Random(seed)
    names = list(LABELS)
    rng.shuffle(names)
    take = lambda n: [names.pop() for _ in range(n)]
    I, J, K, L = take(rng.randint(0, 2)), take(rng.randint(0, 2)), take(rng.randint(1, 2)), take(rng.randint(0, 1))
    la, lb, lc = I + K + L, J + K + L, I + J + L
    if rng.random() < 0.25 and names:
        (la if rng.random() < 0.5 else lb).append(names.pop())         # summed over one operand only
    for lst in (la, lb, lc):
        rng.shuffle(lst)
    if rng.random() < 0.15:
        la.insert(rng.randrange(len(la) + 1), rng.choice(la))          # a diagonal of A
    pool = sorted(set(la) | set(lb))
    ext = {x: rng.choice([1, 2, 3, 4, 5, 7, 17, 33]) for x in pool}
    tens = []
    for labels in (la, lb, lc):
        order = list(range(len(labels)))
        rng.shuffle(order)                       # memory order, slowest first
        stride, acc = [0] * len(labels), 1
        for pos in reversed(order):
            stride[pos] = acc
            acc *= ext[labels[pos]] * (rng.choice([1, 1, 1, 2]) if labels is not lc or True else 1)
        size = max(acc, 1)
        base = 0
        if labels is not lc:
            for pos in range(len(labels)):
                if rng.random() < 0.15:
                    base += stride[pos] * (ext[labels[pos]] - 1)
                    stride[pos] = -stride[pos]
        tens.append((labels, [ext[x] for x in labels], stride, size, base))
    N = rng.choice([2, 5, 8, 11, 14, 16, 17, 20])
    return dict(tens=tens, N=N, g=min(rng.choice([0, 1, 3, N]), N), rounding=rng.choice(["RN", "RN", "TRUNC"]),
                mode=rng.choice(["EMULATE"] * 5 + ["DIRECT"]),
                alpha=rng.choice([1.0, 1.0, -0.5, 0.0, 2.5]), beta=rng.choice([0.0, 0.0, 1.0, 0.3]),
                special=rng.random() < 0.3, seed=seed)


@pytest.mark.parametrize("seed", range(120))
def test_random_contraction(seed):
    import gpu_util as gu
    import immerdink_b200 as imd
    from immerdink_b200 import host
    c = draw(seed)
    rng = np.random.default_rng(seed)
    bufs = []
    for labels, extent, stride, size, base in c["tens"]:
        b = rng.standard_normal(size) * np.exp2(rng.integers(-12, 12, size))
        if c["special"] and labels is not c["tens"][2][0] and size > 3:
            b[rng.integers(0, size, 2)] = rng.choice([np.inf, -np.inf, np.nan, 0.0])
        bufs.append(b)
    hd = [host.Desc(tuple(e), tuple(s), tuple(ord(x) for x in l)) for l, e, s, _, _ in c["tens"]]
    od = [orc.Desc(e, s, [ord(x) for x in l]) for l, e, s, _, _ in c["tens"]]
    bases = [t[4] for t in c["tens"]]
    try:
        want = orc.contract_tensor(bufs[0], bufs[1], bufs[2], od[0], od[1], od[2], c["alpha"], c["beta"],
                                   c["N"], c["rounding"], c["mode"], bases[0], bases[1], bases[2])
        status = "SUCCESS"
    except orc.NotSupported:
        status = "NOT_SUPPORTED"
    except orc.InvalidValue:
        status = "INVALID_VALUE"
    if status != "SUCCESS":
        with pytest.raises(imd.ImmerdinkError) as e:
            imd.Plan.from_descs(*hd, N=c["N"], g=c["g"], rounding=c["rounding"], mode=c["mode"])
        assert e.value.status == status
        return
    out = gu.run_descs(hd, bufs, bases, c["alpha"], c["beta"], c["N"], g=c["g"], rounding=c["rounding"],
                       mode=c["mode"])
    assert same_bits(out, want), c
    low = host.lowering(tuple(hd), N=c["N"], g=c["g"], rounding=c["rounding"], mode=c["mode"])
    if seed % 4 or low["dispatch"] != "EMULATE":
        return
    # the same contraction through packs of both operands (GIVEN: bit-identical)
    import torch
    packs, packed, keep = [], [], []
    dev = [gu.dev_f64(b) for b in bufs]
    for x in (0, 1):
        spec = host.pack_desc_for(tuple(hd), operand=x, N=c["N"], g=c["g"], rounding=c["rounding"],
                                  mode=c["mode"])
        if host.pack_layout(spec, check=False)["status"] != "SUCCESS":
            return
        pk = imd.Pack(spec)
        buf, _ = _pack(pk, dev[x], bases[x])
        packs.append(pk)
        keep.append(buf)            # the packed buffer must outlive the call
        packed.append(buf.arg())
    specs = tuple(pk.spec for pk in packs)
    lw = host.lowering(tuple(hd), N=c["N"], g=c["g"], rounding=c["rounding"], mode=c["mode"],
                       packing=specs, check=False)
    if lw["status"] == "PACK_MISMATCH":     # e.g. a K label that only the partner operand has
        with pytest.raises(imd.PackMismatchError):
            imd.Plan.from_descs(*hd, N=c["N"], g=c["g"], rounding=c["rounding"], mode=c["mode"],
                                packs=tuple(packs))
        return
    plan = imd.Plan.from_descs(*hd, N=c["N"], g=c["g"], rounding=c["rounding"], mode=c["mode"],
                               packs=tuple(packs))
    ws = gu.Workspace(plan.workspace_bytes)
    plan.contract_ptr(c["alpha"], dev[0].data_ptr() + 8 * bases[0], dev[1].data_ptr() + 8 * bases[1],
                      c["beta"], dev[2].data_ptr() + 8 * bases[2],
                      ws.ptr if plan.workspace_bytes else None, plan.workspace_bytes, 0,
                      packed=tuple(packed))
    torch.cuda.synchronize()
    assert ws.guards_intact()
    assert same_bits(gu.host_f64(dev[2]), want), ("packed", c)
    assert all(b.guards_intact() for b in keep)


def _pack(pk, X_dev, base):
    import torch
    import gpu_util as gu
    out = gu.Workspace(pk.pack_bytes)
    ws = gu.Workspace(pk.workspace_bytes)
    pk.pack_ptr(X_dev.data_ptr() + 8 * base, out.ptr if pk.pack_bytes else None, pk.pack_bytes,
                ws.ptr if pk.workspace_bytes else None, pk.workspace_bytes, 0)
    torch.cuda.synchronize()
    assert out.guards_intact() and ws.guards_intact()
    return out, None
