"""The reference's own, unmodified Python front end (host.py, planner.py, precision.py) running on
this repository's host library through its documented environment variable. Needs the reference
tree; skipped where it is absent."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference's package: its tree ($IMD_REFERENCE or a directory `reference` beside the repository),
# else the unmodified copy that oracle/Makefile stages under oracle/_ref/python
_TREES = [os.environ.get("IMD_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"),
          os.path.join(os.path.dirname(HERE), "oracle", "_ref")]
REF_PY = next((os.path.join(t, "python") for t in _TREES
               if os.path.isdir(os.path.join(t, "python", "immerdink"))), "")
HOST_LIB = os.path.join(os.path.dirname(HERE), "immerdink_b200", "libimmerdink_host.so")

SCRIPT = r"""
import json, sys
sys.path.insert(0, %r)
from immerdink import host, planner, precision
from immerdink.host import Accuracy
spec, ext = "kjbc,kiac->abij", dict(a=200, b=200, c=200, i=40, j=40, k=40)
out = {"lib": host.load().path, "ws": host.workspace_size(spec, ext, N=14, g=7)}
low = host.lowering(spec, ext, N=14, g=7)
out["view"] = [low.m, low.n, low.k, low.b, bool(low.swapped)]
p = host.predict(spec, ext, N=14, g=7)
out["predict"] = [p.status, p.time_s, [ph.name for ph in p.phases]]
r = host.rank(spec, ext, N=[12, 14], g=[7], packs=("NONE", "B"), reuse=4)
out["rank"] = [[c.num_moduli, c.packed, c.feasible] for c in r]
cal = host.Calibration.default()
out["calib_round_trip"] = host.Calibration.parse(cal.format()).format() == cal.format()
out["gpu"] = cal.meta["gpu"]
e = host.err_estimate(14, 8000)
out["err"] = e.bound
pl = planner.Planner()
pp = precision.PrecisionPlan(pl, {"ring": (spec, ext, 2)})
ph = pp.phase({"ring": Accuracy("NORMWISE", 1e-12)}, iterations=4)
out["phase"] = [ph.N["ring"], ph.status["ring"]]
ps = host.pack_desc_for(spec, ext, operand=1, N=14, g=7)
out["pack_bytes"] = host.pack_layout(ps).pack_bytes
print(json.dumps(out))
"""


@pytest.mark.skipif(not os.path.isdir(REF_PY), reason="reference tree absent")
def test_reference_python_front_end_on_this_host_library():
    env = dict(os.environ, IMMERDINK_HOST_LIB=HOST_LIB)
    r = subprocess.run([sys.executable, "-c", SCRIPT % REF_PY], env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["lib"] == HOST_LIB
    assert out["ws"] == 1792432896 and out["view"] == [8000, 8000, 8000, 1, True]
    assert out["predict"][0] == "SUCCESS" and 6.5e-3 < out["predict"][1] < 9e-3
    assert out["predict"][2][-3:] == ["K4 gemm", "K5 crt", "call"]
    assert len(out["rank"]) == 4 and all(c[2] for c in out["rank"])
    assert out["calib_round_trip"] and "B200" in out["gpu"]
    assert out["phase"] == [14, "MET"]
    from immerdink_b200 import host
    assert out["err"] == host.err_estimate(N=14, k=8000)["bound"]
    ps = host.pack_desc_for("kjbc,kiac->abij", dict(a=200, b=200, c=200, i=40, j=40, k=40), operand=1,
                            N=14, g=7)
    assert out["pack_bytes"] == host.pack_layout(ps)["pack_bytes"]
