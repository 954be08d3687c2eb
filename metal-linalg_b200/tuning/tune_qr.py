#!/usr/bin/env python3
"""Measure the QR routing on this GPU (which kernel takes a shape and a batch) and write
up the result. It stands where the reference has tuning/tune_qr.py + tuning/sweep_qr.cpp:
the same questions (where does the grid-parallel QR overtake the block-per-matrix kernel,
how much does the rule lose against the best kernel per point, what is the noise floor),
asked of the B200 kernels through the library's own C ABI.

    python metal-linalg_b200/tuning/tune_qr.py --out metal-linalg_b200/tuning/results/<device>
    python metal-linalg_b200/tuning/tune_qr.py --from <dir>/results.json     # re-render the report only

Writes raw.csv (every timed run), results.json (the analysis) and report.md.

Method. The grid is balanced over square, tall, wide and near-square shapes (a square-heavy
grid cannot see where a crossover on min(M, N) fails). The order of the points is shuffled,
so that clock drift over the run does not line up with problem size. A timing is the median
of repeated calls (CUDA events on the launching stream, after two warm-up calls); two passes
over the whole grid give a run-to-run noise floor and are combined by their minimum
(interference only ever adds time). The rule that is fitted is the library's own,

    spread over the grid  iff  sqrt(M k) >= L sqrt(max(1, batch / F)),   k = min(M, N),

with L and F chosen on two thirds of the shapes and judged on the third that was held out.
Regret of a rule at a point = time of the kernel it picks / time of the faster kernel.
"""
import argparse
import csv
import json
import math
import os
import random
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

SQUARE = [96, 128, 192, 256, 320, 384, 448, 512, 640, 768, 896, 1024]
TALL = [(512, 64), (1024, 64), (640, 96), (1024, 128), (768, 192), (1024, 256), (1000, 500)]
WIDE = [(64, 512), (128, 1024), (384, 768), (256, 1024), (512, 2048), (500, 1000)]
NEAR = [(300, 256), (500, 400), (700, 600), (900, 1000), (1024, 900)]
BATCHES = [1, 2, 4, 8, 16, 32, 64, 128]
THIN = [(2048, 32), (4096, 64), (8192, 64), (8192, 128), (16384, 32)]       # tsqr against blocked
THIN_BATCHES = [1, 2, 4, 16]
MAX_ELEMENTS = 96 << 20          # batch * M * N of one point
LIBRARY_F = 3.0                  # the batch divisor in the library's rule (csrc/qr.cpp: qr_gpu_backend)


def shapes():
    out = [("square", n, n) for n in SQUARE]
    out += [("tall", m, n) for m, n in TALL] + [("wide", m, n) for m, n in WIDE] + [("near", m, n) for m, n in NEAR]
    return out


def time_kernel(torch, mlt, a, kernel, repeats):
    os.environ["QR_KERNEL"] = kernel
    try:
        if mlt.qr_kernel(a.shape[1], a.shape[2], a.shape[0]) != kernel:
            return None                        # the forced kernel does not take this shape
        for _ in range(2):
            mlt.qr(a)
        torch.cuda.synchronize()
        ts = []
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            mlt.qr(a)
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)
    finally:
        os.environ.pop("QR_KERNEL", None)


def sweep(out_dir, seed):
    import torch

    import metal_linalg_torch as mlt
    points = [(fam, m, n, b, ("mid", "blocked")) for fam, m, n in shapes() for b in BATCHES if b * m * n <= MAX_ELEMENTS]
    points += [("thin", m, n, b, ("tsqr", "blocked")) for m, n in THIN for b in THIN_BATCHES]
    rows = []
    rng = random.Random(seed)
    g = torch.Generator(device="cuda").manual_seed(seed)
    for pass_no in (1, 2):
        order = points[:]
        rng.shuffle(order)
        for fam, m, n, b, kernels in order:
            a = torch.randn(b, m, n, generator=g, device="cuda")
            for kernel in kernels:
                big = b * m * n > (8 << 20)
                ms = time_kernel(torch, mlt, a, kernel, 3 if big else 7)
                if ms is not None:
                    rows.append({"pass": pass_no, "family": fam, "rows": m, "cols": n, "batch": b, "kernel": kernel, "ms": ms})
            del a
    with open(os.path.join(out_dir, "raw.csv"), "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0]))
        w.writeheader()
        w.writerows(rows)
    ident = {"device": mlt.device_name(), "multiprocessors": mlt.gpu_core_count(), "policy_source": mlt.qr_policy_source(),
             "policy": mlt.qr_policy(), "torch": torch.__version__, "cuda": torch.version.cuda,
             "date": time.strftime("%Y-%m-%d")}
    return rows, ident


def analyse(rows, ident):
    # combine the passes: min per (point, kernel); noise = relative gap between the passes
    by = {}
    for r in rows:
        by.setdefault((r["family"], r["rows"], r["cols"], r["batch"], r["kernel"]), {})[r["pass"]] = r["ms"]
    noise = sorted(abs(v[1] - v[2]) / min(v[1], v[2]) for v in by.values() if 1 in v and 2 in v)
    t = {k: min(v.values()) for k, v in by.items()}
    pts = {}
    for (fam, m, n, b, kernel), ms in t.items():
        pts.setdefault((fam, m, n, b), {})[kernel] = ms
    pairs = {k: v for k, v in pts.items() if k[0] != "thin" and len(v) == 2}
    thin = {k: v for k, v in pts.items() if k[0] == "thin" and len(v) == 2}

    def spread(m, n, b, L, F):
        return m * min(m, n) >= L * L * max(1.0, b / F)

    def regrets(keys, L, F):
        out = []
        for k in keys:
            _, m, n, b = k
            v = pairs[k]
            pick = "blocked" if spread(m, n, b, L, F) else "mid"
            out.append(v[pick] / min(v.values()))
        return out

    def geo(xs):
        return math.exp(sum(math.log(x) for x in xs) / len(xs)) if xs else float("nan")

    # hold out every third shape of each family
    fam_shapes = {}
    for fam, m, n, _ in pairs:
        fam_shapes.setdefault(fam, set()).add((m, n))
    held = set()
    for fam, ss in fam_shapes.items():
        for i, s in enumerate(sorted(ss)):
            if i % 3 == 1:
                held.add((fam,) + s)
    train = [k for k in pairs if (k[0], k[1], k[2]) not in held]
    test = [k for k in pairs if (k[0], k[1], k[2]) in held]
    grid = [(L, F) for L in range(200, 621, 10) for F in (1.0, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0, 8.0)]
    fit = sorted((geo(regrets(train, L, F)), L, F) for L, F in grid)
    best_g = fit[0][0]
    band = [(L, F) for gg, L, F in fit if gg <= best_g * 1.005]
    # the curve is flat over a band (the grid has no shape between two neighbouring sizes): its argmin
    # is noise, so the fitted point is the middle of the tie, at the F most of the tie shares
    tie = [(L, F) for gg, L, F in fit if gg <= best_g * 1.0005]
    best_F = max({f for _, f in tie}, key=lambda f: sum(1 for _, g in tie if g == f))
    tie_L = sorted(L for L, f in tie if f == best_F)
    best_L = tie_L[len(tie_L) // 2]
    best_g = geo(regrets(train, best_L, best_F))
    cur = ident["policy"]
    cur_L = cur.get("gpu_large_min_k", 0)
    rules = {
        "fitted": (best_L, best_F),
        "library (gpu_large_min_k = %d, F = %g)" % (cur_L, LIBRARY_F): (cur_L, LIBRARY_F),
        "always the block-per-matrix kernel": (10 ** 9, 1.0),
        "always the grid-parallel QR": (0, 10 ** 9),
    }
    table = {}
    for name, (L, F) in rules.items():
        rt, rh = regrets(train, L, F), regrets(test, L, F)
        table[name] = {"L": L, "F": F, "train_geo": geo(rt), "train_max": max(rt), "held_geo": geo(rh), "held_max": max(rh),
                       "held_over_1.10": sum(x > 1.10 for x in rh), "held_points": len(rh)}
    worst = sorted(((v, k) for k, v in zip(test, regrets(test, best_L, best_F))), reverse=True)[:8]
    surface = [{"family": k[0], "rows": k[1], "cols": k[2], "batch": k[3], "mid_ms": v["mid"], "blocked_ms": v["blocked"]}
               for k, v in sorted(pairs.items())]
    thin_rows = [{"rows": k[1], "cols": k[2], "batch": k[3], "tsqr_ms": v["tsqr"], "blocked_ms": v["blocked"]}
                 for k, v in sorted(thin.items())]
    return {"identity": ident, "points": len(pairs), "train_points": len(train), "held_points": len(test),
            "held_shapes": sorted(held), "noise": {"median": noise[len(noise) // 2], "p90": noise[int(len(noise) * 0.9)],
                                                    "max": noise[-1], "pairs": len(noise)},
            "fit": {"L": best_L, "F": best_F, "train_geo": best_g, "band": band}, "rules": table,
            "worst_held": [{"regret": v, "family": k[0], "rows": k[1], "cols": k[2], "batch": k[3]} for v, k in worst],
            "surface": surface, "thin": thin_rows}


def report(res):
    i, nz, fit = res["identity"], res["noise"], res["fit"]
    L = ["# QR routing on %s (%d multiprocessors), %s" % (i["device"], i["multiprocessors"], i["date"]), "",
         "Made by `metal-linalg_b200/tuning/tune_qr.py` (torch %s, CUDA %s); raw timings in `raw.csv`, the analysis in"
         % (i["torch"], i["cuda"]), "`results.json`. Policy in force during the sweep: %s." % i["policy_source"], "",
         "## Grid and noise", "",
         "%d (shape, batch) points timed with both the block-per-matrix kernel (`mid`) and the grid-parallel QR (`blocked`),"
         % res["points"],
         "balanced over square, tall, wide and near-square shapes, batches 1-128, in shuffled order, two passes.",
         "Run-to-run noise (relative gap between the passes, %d kernel timings): median %.1f %%, 90th percentile %.1f %%, max %.1f %%."
         % (nz["pairs"], 100 * nz["median"], 100 * nz["p90"], 100 * nz["max"]),
         "A difference between rules below the 90th percentile is not a finding.", "",
         "## The rule", "",
         "`spread over the grid iff sqrt(M k) >= L sqrt(max(1, batch / F))`. Fitted on %d points (two thirds of the shapes):"
         % res["train_points"],
         "**L = %d, F = %g** (geometric-mean regret %.3f). Every (L, F) within 0.5 %% of that: L %d-%d, F %s."
         % (fit["L"], fit["F"], fit["train_geo"], min(b[0] for b in fit["band"]), max(b[0] for b in fit["band"]),
            ", ".join("%g" % f for f in sorted({b[1] for b in fit["band"]}))), "",
         "| rule | L | F | train geo-mean | train max | held-out geo-mean | held-out max | held-out points over 1.10 |",
         "|---|---|---|---|---|---|---|---|"]
    for name, r in res["rules"].items():
        L.append("| %s | %s | %s | %.3f | %.2f | %.3f | %.2f | %d of %d |"
                 % (name, r["L"] if r["L"] < 10 ** 8 else "inf", ("%g" % r["F"]) if r["F"] < 10 ** 8 else "inf",
                    r["train_geo"], r["train_max"], r["held_geo"], r["held_max"], r["held_over_1.10"], r["held_points"]))
    L += ["", "Held-out shapes: " + ", ".join("%dx%d" % (s[1], s[2]) for s in res["held_shapes"]) + ".", "",
          "Worst held-out points of the fitted rule:", "", "| regret | shape | batch |", "|---|---|---|"]
    L += ["| %.2f | %dx%d (%s) | %d |" % (w["regret"], w["rows"], w["cols"], w["family"], w["batch"]) for w in res["worst_held"]]
    L += ["", "## Decision surface (ms, minimum of the two passes)", "", "| shape | batch | mid | blocked | faster |", "|---|---|---|---|---|"]
    for s in res["surface"]:
        if s["batch"] in (1, 4, 16, 64):
            L.append("| %dx%d | %d | %.3f | %.3f | %s |" % (s["rows"], s["cols"], s["batch"], s["mid_ms"], s["blocked_ms"],
                                                           "mid" if s["mid_ms"] <= s["blocked_ms"] else "blocked"))
    L += ["", "## Tall thin matrices: the tree against the grid-parallel QR (ms)", "", "| shape | batch | tsqr | blocked | faster |",
          "|---|---|---|---|---|"]
    for s in res["thin"]:
        L.append("| %dx%d | %d | %.3f | %.3f | %s |" % (s["rows"], s["cols"], s["batch"], s["tsqr_ms"], s["blocked_ms"],
                                                       "tsqr" if s["tsqr_ms"] <= s["blocked_ms"] else "blocked"))
    return "\n".join(L) + "\n"


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="qr-tune-results")
    ap.add_argument("--from", dest="from_json", help="re-render report.md from an existing results.json")
    ap.add_argument("--seed", type=int, default=11)
    args = ap.parse_args()
    if args.from_json:
        res = json.load(open(args.from_json))
        out_dir = os.path.dirname(os.path.abspath(args.from_json))
    else:
        out_dir = args.out
        os.makedirs(out_dir, exist_ok=True)
        rows, ident = sweep(out_dir, args.seed)
        res = analyse(rows, ident)
        json.dump(res, open(os.path.join(out_dir, "results.json"), "w"), indent=1)
    open(os.path.join(out_dir, "report.md"), "w").write(report(res))
    print("wrote", os.path.join(out_dir, "report.md"))


if __name__ == "__main__":
    main()
