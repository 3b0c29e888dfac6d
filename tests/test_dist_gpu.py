"""The rank-level step of the partitioned contraction on one GPU (world = 1: the gathers are
copies; the pack-while-gathering path and the split-label plan are the same as with more ranks)."""
import numpy as np
import pytest

from golden_util import same_bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("exchange", ["fp64", "residues", "pieces"])
def test_rank_contraction_world_1_equals_plain_call(exchange):
    import torch
    import immerdink_b200 as imd
    from immerdink_b200 import dist as idist
    spec = "kjbc,kiac->abij"
    e = dict(a=6, b=4, c=9, i=5, j=3, k=4)
    part = idist.Partition(spec, e, 1, 0, "a", "b")
    rng = np.random.default_rng(11)
    A = torch.from_numpy(rng.standard_normal(part.shard_shape(0))).cuda()
    B = torch.from_numpy(rng.standard_normal(part.shard_shape(1))).cuda()
    A[0, 1, 2, 3] = float("nan")
    rc = idist.RankContraction(part, N=14, g=7, exchange=exchange)
    assert rc.exchange == exchange
    C1 = torch.full(rc.tile_shape, 3.0, dtype=torch.float64, device="cuda")
    for _ in range(2):
        rc(A, B, C1, alpha=0.5, beta=0.0)
    C0 = torch.zeros(tuple(e[c] for c in "abij"), dtype=torch.float64, device="cuda")
    ws = torch.empty(imd.workspace_size(spec, A, B, C0, N=14, g=7), dtype=torch.uint8, device="cuda")
    imd.contract(spec, A, B, C0, alpha=0.5, N=14, g=7, workspace=ws)
    torch.cuda.synchronize()
    assert same_bits(C1.reshape(C0.shape).cpu().numpy(), C0.cpu().numpy())
    assert rc.device_error() == 0
    rc.close()


def test_wait_flags_passes_when_set_and_gives_up_when_not():
    """The bounded wait the residue exchange uses: flags that hold the expected value let the
    stream through; a flag nothing sets makes the wait run out, which sets bit 2 of the device
    error word and leaves the context usable."""
    import torch
    import immerdink_b200 as imd
    from immerdink_b200 import device
    lib = imd.load_library()
    lib.lib.imd_test_device_error()                       # clear
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[3] = 7
    flags[40] = 7
    base = flags.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    device.wait_flags([base + 4 * 3, base + 4 * 40], 7, stream=stream)
    device.wait_flags([], 7, stream=stream)               # nothing to wait for
    assert lib.lib.imd_test_device_error() == 0
    device.wait_flags([base + 4 * 3, base + 4 * 5], 7, max_polls=50, stream=stream)   # word 5 stays 0
    assert lib.lib.imd_test_device_error() == 4
    assert lib.lib.imd_test_device_error() == 0           # sticky until read, then clear
    assert int((flags + 1).sum().item()) == 64 + 14       # the context still works
    with pytest.raises(imd.InvalidValueError):
        device.wait_flags([base] * 33, 7, stream=stream)
    with pytest.raises(imd.MisalignedError):
        device.wait_flags([base + 2], 7, stream=stream)


def test_copy_if_flagged_copies_only_when_a_flag_byte_is_set():
    import torch
    import immerdink_b200 as imd
    from immerdink_b200 import device
    stream = torch.cuda.current_stream().cuda_stream
    flags = torch.zeros(5000, dtype=torch.uint8, device="cuda")
    src = torch.arange(3 * 1001, dtype=torch.float64, device="cuda")
    dst = torch.full_like(src, -1.0)
    n = 1001 * 8
    copies = [(dst.data_ptr() + i * n, src.data_ptr() + i * n, n) for i in (0, 2)]
    ranges = [(flags.data_ptr(), 1234), (flags.data_ptr() + 2000, 3000)]
    device.copy_if_flagged(ranges, copies, stream=stream)
    assert bool((dst == -1.0).all())                       # no flag: nothing is touched
    flags[1500] = 1                                        # outside both ranges
    device.copy_if_flagged(ranges, copies, stream=stream)
    assert bool((dst == -1.0).all())
    flags[4999] = 1                                        # last byte of the second range
    device.copy_if_flagged(ranges, copies, stream=stream)
    want = src.clone()
    want[1001:2002] = -1.0                                 # the piece that was not listed
    assert torch.equal(dst, want)
    device.copy_if_flagged(ranges, [], stream=stream)      # nothing to copy
    with pytest.raises(imd.MisalignedError):
        device.copy_if_flagged(ranges, [(dst.data_ptr() + 4, src.data_ptr(), 8)], stream=stream)
    with pytest.raises(imd.InvalidValueError):
        device.copy_if_flagged(ranges, copies * 9, stream=stream)


def test_push_ranges_copies_then_sets_the_flags():
    """imd_push_ranges on one GPU: every range arrives, the flag words hold the value afterwards,
    and a wait on those words gets through."""
    import torch
    import immerdink_b200 as imd
    from immerdink_b200 import device
    lib = imd.load_library()
    lib.device_error()
    src = torch.arange(5 << 20, dtype=torch.float64, device="cuda")
    dst = torch.zeros_like(src)
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    sizes = [16, 4096, (1 << 20) + 48, 7 << 20]     # bytes, 16-byte granular
    copies, at = [], 0
    for n in sizes:
        copies.append((dst.data_ptr() + at, src.data_ptr() + at, n))
        at += n + 64                                 # gaps stay untouched
    side = torch.cuda.Stream()
    words = [flags.data_ptr() + 4 * 2, flags.data_ptr() + 4 * 9]
    for ctas in (0, 1, 7):
        dst.zero_()
        flags.zero_()
        torch.cuda.synchronize()
        device.push_ranges(copies, words, 41 + ctas, ctas=ctas, stream=side.cuda_stream)
        side.synchronize()
        device.wait_flags(words, 41 + ctas, stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert lib.device_error() == 0
        assert flags.tolist().count(41 + ctas) == 2 and int(flags.sum().item()) == 2 * (41 + ctas)
        want = torch.zeros_like(src)
        at = 0
        for n in sizes:
            want[at // 8:(at + n) // 8] = src[at // 8:(at + n) // 8]
            at += n + 64
        assert torch.equal(dst, want), ctas
    device.push_ranges([], words, 5, stream=side.cuda_stream)     # flags only
    torch.cuda.synchronize()
    assert flags[2].item() == 5 and flags[9].item() == 5
    with pytest.raises(imd.MisalignedError):
        device.push_ranges([(dst.data_ptr() + 8, src.data_ptr(), 16)], [], 1, stream=side.cuda_stream)
    with pytest.raises(imd.InvalidValueError):
        device.push_ranges(copies * 25, [], 1, stream=side.cuda_stream)


def test_device_error_peek_mirrors_the_word_into_pinned_memory():
    import torch
    import immerdink_b200 as imd
    from immerdink_b200 import device
    lib = imd.load_library()
    lib.device_error()
    host_word = torch.zeros(1, dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.lib.imd_device_error_peek(host_word.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(host_word[0]) == 0
    device.wait_flags([flag.data_ptr()], 9, max_polls=20, stream=stream)   # nothing sets it
    assert lib.lib.imd_device_error_peek(host_word.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(host_word[0]) == 4                  # seen without clearing
    assert lib.device_error() == 4 and lib.device_error() == 0
