"""The reference's own, unmodified Python package (immerdink.Plan / contract / Pack over ctypes)
driving this repository's production libimmerdink.so through the environment variable it documents
(IMMERDINK_LIB): the drop-in claim where it matters, on a GPU. The package comes from the
reference tree when one is reachable, else from the unmodified copy that oracle/Makefile stages
under oracle/_ref/python; skipped when there is neither."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import imd_oracle as orc

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
_TREES = [os.environ.get("IMD_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference"),
          os.path.join(ROOT, "oracle", "_ref")]
REF_PY = next((os.path.join(t, "python") for t in _TREES
               if os.path.isdir(os.path.join(t, "python", "immerdink"))), "")
CUDA_LIB = os.path.join(ROOT, "immerdink_b200", "libimmerdink.so")

SCRIPT = r"""
import json, sys
import numpy as np, torch
sys.path.insert(0, %r)
import immerdink
from immerdink import _capi
spec, ext = "kjbc,kiac->abij", dict(a=12, b=10, c=16, i=5, j=6, k=4)
rng = np.random.default_rng(7)
A = torch.from_numpy(rng.uniform(-1, 1, [ext[c] for c in "kjbc"])).cuda()
B = torch.from_numpy(rng.uniform(-1, 1, [ext[c] for c in "kiac"])).cuda()
out = {"lib": _capi.load().path}
res = {}
for tag, g in (("g7", 7), ("g14", 0)):
    C = torch.full([ext[c] for c in "abij"], float("nan"), dtype=torch.float64, device="cuda")
    n = immerdink.workspace_size(spec, A, B, C, N=14, g=g)
    ws = torch.empty(n + 256, dtype=torch.uint8, device="cuda")
    off = (-ws.data_ptr()) %% 256
    immerdink.contract(spec, A, B, C, N=14, g=g, workspace=ws[off:off + n])
    torch.cuda.synchronize()
    res[tag] = C.cpu().numpy().view(np.uint64).reshape(-1).tolist()
# a plan object, alpha / beta, and a packed operand B
C0 = torch.from_numpy(rng.uniform(-1, 1, [ext[c] for c in "abij"])).cuda()
C = C0.clone()
plan = immerdink.Plan(spec, A, B, C, N=12, g=5)
ws = torch.empty(plan.workspace_bytes + 256, dtype=torch.uint8, device="cuda")
off = (-ws.data_ptr()) %% 256
plan.contract(A, B, C, alpha=1.5, beta=0.5, workspace=ws[off:off + plan.workspace_bytes])
torch.cuda.synchronize()
res["plan"] = C.cpu().numpy().view(np.uint64).reshape(-1).tolist()
pk = immerdink.Pack(plan.pack_spec(1))
pbuf = torch.empty(pk.pack_bytes + 256, dtype=torch.uint8, device="cuda")
po = (-pbuf.data_ptr()) %% 256
pws = torch.empty(pk.workspace_bytes + 256, dtype=torch.uint8, device="cuda")
pwo = (-pws.data_ptr()) %% 256
packed = immerdink.PackedBuffer(pbuf[po:po + pk.pack_bytes])
pk.pack(B, packed, workspace=pws[pwo:pwo + pk.workspace_bytes])
plan2 = immerdink.Plan(spec, A, B, C, N=12, g=5, packs=(None, pk))
C = C0.clone()
ws2 = torch.empty(plan2.workspace_bytes + 256, dtype=torch.uint8, device="cuda")
o2 = (-ws2.data_ptr()) %% 256
plan2.contract(A, B, C, alpha=1.5, beta=0.5, workspace=ws2[o2:o2 + plan2.workspace_bytes],
               packed=(None, packed))
torch.cuda.synchronize()
res["packed"] = C.cpu().numpy().view(np.uint64).reshape(-1).tolist()
out["A"] = A.cpu().numpy().reshape(-1).tolist()
out["B"] = B.cpu().numpy().reshape(-1).tolist()
out["C0"] = C0.cpu().numpy().reshape(-1).tolist()
out["res"] = res
print(json.dumps(out))
"""


@pytest.mark.skipif(not REF_PY, reason="reference Python package absent (no tree, nothing staged)")
def test_reference_package_runs_on_this_library():
    from immerdink_b200 import host
    env = dict(os.environ, IMMERDINK_LIB=CUDA_LIB)
    env.pop("IMMERDINK_LIB_DIR", None)
    r = subprocess.run([sys.executable, "-c", SCRIPT % REF_PY], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert os.path.samefile(out["lib"], CUDA_LIB)
    ext = dict(a=12, b=10, c=16, i=5, j=6, k=4)
    descs = host.contraction("kjbc,kiac->abij", ext)
    od = [orc.Desc(d.extent, d.stride, d.label) for d in descs]
    A, B, C0 = (np.array(out[x]) for x in ("A", "B", "C0"))
    want = orc.contract_tensor(A, B, np.zeros(C0.size), od[0], od[1], od[2], 1.0, 0.0, 14)
    for tag in ("g7", "g14"):
        assert np.array_equal(np.array(out["res"][tag], np.uint64), want.view(np.uint64)), tag
    want2 = orc.contract_tensor(A, B, C0.copy(), od[0], od[1], od[2], 1.5, 0.5, 12)
    for tag in ("plan", "packed"):
        assert np.array_equal(np.array(out["res"][tag], np.uint64), want2.view(np.uint64)), tag
