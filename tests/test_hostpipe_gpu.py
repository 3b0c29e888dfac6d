"""Host-resident operands through the slab pipeline: bit-identical to the undivided device call."""
import numpy as np
import pytest

from golden_util import same_bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("split,slabs,beta", [("a", 4, 0.0), ("b", 2, 0.5), ("a", 1, 0.0)])
def test_slab_pipeline_equals_one_call(split, slabs, beta):
    import torch
    import immerdink_b200 as imd
    from immerdink_b200.hostpipe import HostContraction
    spec = "kjbc,kiac->abij"
    e = dict(a=8, b=6, c=7, i=5, j=3, k=4)
    shp = [tuple(e[c] for c in lab) for lab in ("kjbc", "kiac", "abij")]
    rng = np.random.default_rng(3)
    hA, hB, hC = (torch.from_numpy(rng.standard_normal(s)).pin_memory() for s in shp)
    hA[1, 2, 3, 4] = float("inf")        # a flagged row takes the native path in both
    want_c = hC.clone()
    dA, dB, dC = hA.cuda(), hB.cuda(), hC.cuda()
    ws = torch.empty(imd.workspace_size(spec, dA, dB, dC, N=14), dtype=torch.uint8, device="cuda")
    imd.contract(spec, dA, dB, dC, alpha=1.5, beta=beta, N=14, workspace=ws)
    pipe = HostContraction(spec, *shp, N=14, split=split, slabs=slabs)
    for _ in range(2):                   # twice: buffers and streams are reused
        hC.copy_(want_c)
        pipe(hA, hB, hC, alpha=1.5, beta=beta)
        torch.cuda.current_stream().synchronize()
        assert same_bits(hC.numpy(), dC.cpu().numpy())
    pipe.close()


def test_rejects_bad_arguments():
    import torch
    from immerdink_b200.hostpipe import HostContraction
    with pytest.raises(ValueError):
        HostContraction("ik,kj->ij", (4, 5), (5, 6), (4, 6), N=14, split="k")
    with pytest.raises(ValueError):
        HostContraction("ik,kj->ij", (4, 5), (5, 6), (4, 6), N=14, split="i", slabs=3)
    pipe = HostContraction("ik,kj->ij", (4, 5), (5, 6), (4, 6), N=14, split="i", slabs=2)
    a, b, c = torch.zeros(4, 5, dtype=torch.float64), torch.zeros(5, 6, dtype=torch.float64).pin_memory(), \
        torch.zeros(4, 6, dtype=torch.float64).pin_memory()
    with pytest.raises(ValueError, match="pinned"):
        pipe(a, b, c)
