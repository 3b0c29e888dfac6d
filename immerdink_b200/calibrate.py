"""Calibration of the performance model on the GPU at hand.

    python -m immerdink_b200.calibrate [--out FILE] [--quick]

Runs imd_contract, imd_pack and the degenerate paths on a set of shapes, measures every phase
with CUDA events on the launching stream (the library's phase marks, `imd_prof_*`), takes the
features x of each phase from `host.predict` (they do not depend on the calibration) and fits
one launch cost (call.launch, from the launch-bound shapes) and then the parameters of every
class by non-negative least squares on what is left of each phase; the prediction bands are the
10 % / 90 % quantiles of measured / predicted per class, widened by 3 %. Writes the calibration
text (format 2). The shipped calibration (csrc/host/perf_calib_b200.inc) is this script's output
on a B200. Needs torch (device memory only), numpy and scipy.
"""
import argparse
import ctypes as C
import datetime
import sys

import numpy as np


def shapes(quick):
    """(b, m, n, k, N, g) of the contractions measured."""
    out = []
    sizes = [(1, 256, 256, 512), (1, 1024, 1024, 1024), (1, 2048, 2048, 2048), (1, 4096, 4096, 4096),
             (1, 8000, 8000, 8000), (1, 8192, 1024, 4096), (1, 1024, 8192, 4096), (1, 4096, 4096, 512),
             (1, 512, 512, 16384), (4, 1024, 1024, 2048), (16, 512, 768, 1024), (1, 6000, 3000, 9000),
             (1, 128, 4096, 4096), (1, 96, 96, 96), (2, 3000, 3000, 3000)]
    if quick:
        sizes = sizes[:4]
    for s in sizes:
        for N, g in ((14, 7), (14, 14), (8, 8), (18, 6), (12, 4)):
            if quick and (N, g) != (14, 7):
                continue
            out.append(s + (N, g))
    return out


def measure(fn, L, tags, steps):
    import torch
    for _ in range(2):
        fn()
    L.imd_prof_enable(64 * (steps + 1))
    torch.cuda.synchronize()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    ph = (C.c_float * 8)()
    L.imd_prof_read(ph, 8)
    L.imd_prof_enable(0)
    return {t: ph[t] / steps * 1e6 for t in tags}   # ns


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args(argv)
    import torch
    from scipy.optimize import nnls

    import immerdink_b200 as imd
    from immerdink_b200 import host

    from . import build as _build
    lib = imd.load_library(_build.HOOKS_LIB)   # phase marks exist only in the instrumented library
    L = lib.lib
    dev = torch.device("cuda", torch.cuda.current_device())
    spec = "bik,bkj->bij"
    rows = {c: [] for c in ("scale", "res", "gemm", "crt", "direct", "beta", "pack", "kf")}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    # small contractions: one fused launch (phase tag 7)
    for (b, m, n, k) in ((1, 40, 2048, 48), (1, 96, 96, 96), (1, 256, 256, 64), (4, 128, 128, 32),
                         (1, 512, 512, 128), (1, 64, 64, 16), (1, 300, 200, 100), (16, 64, 96, 120)):
        A = torch.rand((b, m, k), dtype=torch.float64, device=dev) * 2 - 1
        B = torch.rand((b, k, n), dtype=torch.float64, device=dev) * 2 - 1
        Cd = torch.zeros((b, m, n), dtype=torch.float64, device=dev)
        for N in ((14,) if args.quick else (14, 8, 20)):
            pred = host.predict(spec, dict(b=b, i=m, j=n, k=k), N=N)
            ph = {p["phase"]: p for p in pred["phases"]}
            if "KF fused" not in ph:
                continue
            plan = imd.Plan(spec, A, B, Cd, N=N, lib=lib)
            ws = torch.empty(max(plan.workspace_bytes, 1), dtype=torch.uint8, device=dev)
            t = measure(lambda: (flush.fill_(1), plan.contract(A, B, Cd, workspace=ws)), L, (1, 7), args.steps)
            rows["kf"].append((t[7], [ph["KF fused"]["x"][2], ph["KF fused"]["x"][5]]))
            plan.close()
            print(f"measured fused b={b} m={m} n={n} k={k} N={N}: {t[7] / 1e3:.1f}us", file=sys.stderr)

    last = None
    for (b, m, n, k, N, g) in shapes(args.quick):
        if last != (b, m, n, k):
            A = torch.rand((b, m, k), dtype=torch.float64, device=dev) * 2 - 1
            B = torch.rand((b, k, n), dtype=torch.float64, device=dev) * 2 - 1
            Cd = torch.zeros((b, m, n), dtype=torch.float64, device=dev)
            last = (b, m, n, k)
        ext = dict(b=b, i=m, j=n, k=k)
        if host.lowering(spec, ext, N=N, g=g)["fused"]:
            continue                      # measured above
        plan = imd.Plan(spec, A, B, Cd, N=N, g=g, lib=lib)
        ws = torch.empty(max(plan.workspace_bytes, 1), dtype=torch.uint8, device=dev)

        def call():
            flush.fill_(1)
            plan.contract(A, B, Cd, workspace=ws)
        t = measure(call, L, (1, 2, 3, 4), args.steps)
        pred = host.predict(spec, ext, N=N, g=g)
        assert pred["status"] == "SUCCESS" and pred["dispatch"] == "EMULATE", pred["status"]
        ph = {p["phase"]: p for p in pred["phases"]}
        sc = [ph["K0 vec"], ph["KL A"], ph["KL B"]]
        rows["scale"].append((t[1], [float(sum(q["launches"] for q in sc)), sc[0]["x"][1],
                                     sc[1]["x"][2] + sc[2]["x"][2]]))
        rs = [ph["K2 pack A"], ph["K3 pack B"]]
        rows["res"].append((t[2], [rs[0]["x"][0] + rs[1]["x"][0], rs[0]["x"][2] + rs[1]["x"][2],
                                   rs[0]["x"][4] + rs[1]["x"][4], rs[0]["x"][3] + rs[1]["x"][3]]))
        rows["gemm"].append((t[3], [ph["K4 gemm"]["x"][0], ph["K4 gemm"]["x"][1]], ph["K4 gemm"]["x"][4],
                             ph["K4 gemm"]["launches"]))
        rows["crt"].append((t[4], [1.0, ph["K5 crt"]["x"][2]]))
        plan.close()
        if (N, g) == (14, 7):
            # imd_pack of A; DIRECT mode; the beta-only call
            pk = imd.Pack(imd.pack_spec(spec, A, B, Cd, operand=0, N=N, lib=lib), lib=lib)
            buf = torch.empty(max(pk.pack_bytes, 1), dtype=torch.uint8, device=dev)
            pw = torch.empty(max(pk.workspace_bytes, 1), dtype=torch.uint8, device=dev)
            tp = measure(lambda: (flush.fill_(1), pk.pack(A, buf, workspace=pw)), L, (6,), args.steps)
            pp = {p["phase"]: p for p in host.predict_pack(pk.spec)["phases"]}
            rows["pack"].append((tp[6], pp))
            pk.close()
            if m * n * k * b <= 2e10:
                pd = imd.Plan(spec, A, B, Cd, N=N, mode="DIRECT", lib=lib)
                wd = torch.empty(max(pd.workspace_bytes, 1), dtype=torch.uint8, device=dev)
                td = measure(lambda: (flush.fill_(1), pd.contract(A, B, Cd, workspace=wd)), L, (5,), args.steps)
                xd = {p["phase"]: p for p in host.predict(spec, ext, N=N, mode="DIRECT")["phases"]}
                rows["direct"].append((td[5], [2.0, xd["DIRECT"]["x"][2]], xd["DIRECT"]["x"][1]))
                tb = measure(lambda: (flush.fill_(1), pd.contract(A, B, Cd, alpha=0.0, beta=0.5, workspace=wd)),
                             L, (5,), args.steps)
                xb = {p["phase"]: p for p in host.predict(spec, ext, N=N, mode="DIRECT", alpha_zero=True,
                                                          beta=True)["phases"]}
                rows["beta"].append((tb[5], [2.0, xb["K5 beta-only"]["x"][1]]))
                pd.close()
        print(f"measured b={b} m={m} n={n} k={k} N={N} g={g}: " +
              " ".join(f"{v / 1e3:.1f}us" for v in t.values()), file=sys.stderr)

    # One launch cost for every kernel (call.launch), from the shapes small enough to be bound by
    # it; the class parameters are then fitted to what is left of each phase.
    tiny = [i for i, r in enumerate(rows["crt"]) if r[1][1] <= 14 * 1e5]
    per_launch = [(rows["scale"][i][0] + rows["res"][i][0] + rows["gemm"][i][0] + rows["crt"][i][0]) /
                  (rows["scale"][i][1][0] + rows["res"][i][1][0] + rows["gemm"][i][3] + 1) for i in tiny]
    launch = float(np.median(per_launch)) if per_launch else 5000.0

    def fit(y, X, launches):
        """Non-negative least squares on relative errors of what is left of each measurement once
        its launches are taken out; launch-dominated measurements carry no information here."""
        y = np.asarray(y, dtype=np.float64)
        rest = y - launch * np.asarray(launches, dtype=np.float64)
        keep = rest > np.maximum(0.3 * y, 5000.0)
        X = np.asarray(X, dtype=np.float64)[keep]
        rest = rest[keep]
        coef, _ = nnls(X / rest[:, None], np.ones_like(rest))
        return coef

    cal = host.calib_default()
    P = cal.param
    for i in range(96):
        P[i] = 0.0
    dram_ns = 1e9 / 6.5e12      # ns per DRAM byte at the measured copy bandwidth
    K0, KF, KL, PACK, K4, K5, DIRECT, BETA, CALL = 0, 6, 12, 18, 24, 48, 54, 60, 66
    P[CALL + 1] = launch
    if rows["kf"]:
        # the fused launch has a fixed cost of its own on top of a launch (its chain of dependent
        # cold loads: row offsets, rows, C)
        P[KF + 0], P[KF + 2], P[KF + 5] = fit([r[0] for r in rows["kf"]], [[1.0] + r[1] for r in rows["kf"]],
                                              [1] * len(rows["kf"]))
    n = len(rows["crt"])
    P[KL + 2] = fit([rows["scale"][i][0] for i in range(n)],
                    [[rows["scale"][i][1][2]] for i in range(n)], [rows["scale"][i][1][0] for i in range(n)])[0]
    # residues: the in-line launches and, with the scale part of the model taken out, imd_pack
    y = [rows["res"][i][0] for i in range(n)]
    X = [[rows["res"][i][1][1], rows["res"][i][1][2], rows["res"][i][1][3]] for i in range(n)]
    nl = [rows["res"][i][1][0] for i in range(n)]
    for tp, pp in rows["pack"]:
        y.append(tp - pp["pack KL"]["x"][2] * P[KL + 2])
        X.append([pp["K2 pack A"]["x"][2], pp["K2 pack A"]["x"][4], pp["K2 pack A"]["x"][3]])
        nl.append(2 + pp["pack KL"]["launches"] + 1)
    P[PACK + 2], P[PACK + 4], P[PACK + 3] = fit(y, X, nl)
    cg = fit([rows["gemm"][i][0] for i in range(n)], [rows["gemm"][i][1] for i in range(n)],
             [rows["gemm"][i][3] for i in range(n)])
    P[K4 + 0], P[K4 + 1], P[K4 + 4] = cg[0], cg[1], dram_ns
    P[K5 + 2] = fit([rows["crt"][i][0] for i in range(n)], [[rows["crt"][i][1][1]] for i in range(n)],
                    [1] * n)[0]
    if rows["direct"]:
        P[DIRECT + 2] = fit([r[0] for r in rows["direct"]], [[r[1][1]] for r in rows["direct"]],
                            [2] * len(rows["direct"]))[0]
        P[BETA + 1] = fit([r[0] for r in rows["beta"]], [[r[1][1]] for r in rows["beta"]],
                          [2] * len(rows["beta"]))[0]

    def model(i):
        sc = rows["scale"][i][1][0] * launch + rows["scale"][i][1][2] * P[KL + 2]
        rs = (rows["res"][i][1][0] * launch + rows["res"][i][1][1] * P[PACK + 2] + rows["res"][i][1][2] * P[PACK + 4] +
              rows["res"][i][1][3] * P[PACK + 3])
        gm = rows["gemm"][i][3] * launch + max(np.dot(rows["gemm"][i][1], [P[K4], P[K4 + 1]]),
                                               rows["gemm"][i][2] * dram_ns)
        cr = launch + rows["crt"][i][1][1] * P[K5 + 2]
        return sc, rs, gm, cr

    def band(r):
        r = np.asarray(r)
        lo, hi = np.quantile(r, 0.1) * 0.97, np.quantile(r, 0.9) * 1.03
        return min(lo, 1.0), max(hi, 1.0)
    names = host.class_names()
    for i in range(16):
        cal.band_class[i][0] = cal.band_class[i][1] = 1.0
    ratios = {"kl": [], "pack": [], "k4_128x256": [], "k5": []}
    tot = []
    for i in range(n):
        sc, rs, gm, cr = model(i)
        meas = (rows["scale"][i][0], rows["res"][i][0], rows["gemm"][i][0], rows["crt"][i][0])
        for key, m_, p_ in zip(ratios, meas, (sc, rs, gm, cr)):
            ratios[key].append(m_ / p_)
        tot.append(((sc + rs + gm + cr) * 1e-9, sum(meas) / (sc + rs + gm + cr)))
    ratios["k0"] = ratios["kl"]
    if rows["kf"]:
        ratios["kf"] = [r[0] / (launch + P[KF + 0] + r[1][0] * P[KF + 2] + r[1][1] * P[KF + 5])
                        for r in rows["kf"]]
        for r, q in zip(rows["kf"], ratios["kf"]):
            print(f"fused: measured {r[0] / 1e3:.1f} us, measured/predicted {q:.3f}", file=sys.stderr)
    if rows["direct"]:
        ratios["direct"] = [r[0] / (2 * launch + r[1][1] * P[DIRECT + 2]) for r in rows["direct"]]
        ratios["beta"] = [r[0] / (2 * launch + r[1][1] * P[BETA + 1]) for r in rows["beta"]]
    for cname, r in ratios.items():
        lo, hi = band(r)
        i = names.index(cname)
        cal.band_class[i][0], cal.band_class[i][1] = lo, hi
    for bi, (lo_t, hi_t) in enumerate(((0, 100e-6), (100e-6, 1e-3), (1e-3, 1e9))):
        r = [q for t, q in tot if lo_t <= t < hi_t] or [1.0]
        cal.band_call[bi][0], cal.band_call[bi][1] = band(r)
    cal.gpu = torch.cuda.get_device_name(dev).encode()[:63]
    cal.sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    cal.date = datetime.date.today().isoformat().encode()
    cal.notes = (f"{len(rows['crt'])} contractions, {len(rows['kf'])} fused, {len(rows['pack'])} packs; NNLS per class on "
                 "CUDA-event phase times, L2 flushed between calls").encode()[:127]
    text = host.calib_format(cal)
    host.calib_parse(text)      # must parse back
    for tp, pp in rows["pack"]:
        pr = ((3 + pp["pack KL"]["launches"]) * launch + pp["pack KL"]["x"][2] * P[KL + 2] +
              pp["K2 pack A"]["x"][2] * P[PACK + 2] + pp["K2 pack A"]["x"][4] * P[PACK + 4] +
              pp["K2 pack A"]["x"][3] * P[PACK + 3])
        print(f"pack: measured {tp / 1e3:.1f} us, model {pr / 1e3:.1f} us", file=sys.stderr)
    for (t, q) in tot:
        print(f"call: predicted {t * 1e3:.3f} ms, measured/predicted {q:.3f}", file=sys.stderr)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text)
    else:
        print(text)


if __name__ == "__main__":
    main()
