"""The routing analysis of metal-linalg_b200/tuning/tune_qr.py on synthetic timings (no GPU): the
fit recovers the constants of the model that made the timings, the held-out split is disjoint from
the training shapes, and the report renders."""
import importlib.util
import os

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("tune_qr", os.path.join(HERE, "..", "metal-linalg_b200", "tuning", "tune_qr.py"))
tune_qr = importlib.util.module_from_spec(spec)
spec.loader.exec_module(tune_qr)


def synthetic_rows(L=350.0, F=3.0):
    rows = []
    for fam, m, n in tune_qr.shapes():
        w2 = m * min(m, n)
        for b in tune_qr.BATCHES:
            blocked = 1.0 * max(1.0, b / F)                       # the grid-parallel QR: F matrices at a time
            mid = w2 / (L * L)                                    # the block-per-matrix kernel: flat in the batch
            for p, jitter in ((1, 1.00), (2, 1.02)):
                rows.append({"pass": p, "family": fam, "rows": m, "cols": n, "batch": b, "kernel": "mid", "ms": mid * jitter})
                rows.append({"pass": p, "family": fam, "rows": m, "cols": n, "batch": b, "kernel": "blocked", "ms": blocked * jitter})
    for m, n in tune_qr.THIN:
        for b in tune_qr.THIN_BATCHES:
            for p in (1, 2):
                rows.append({"pass": p, "family": "thin", "rows": m, "cols": n, "batch": b, "kernel": "tsqr", "ms": 1.0})
                rows.append({"pass": p, "family": "thin", "rows": m, "cols": n, "batch": b, "kernel": "blocked", "ms": 0.5 * b})
    return rows


def test_fit_recovers_the_model_and_report_renders():
    ident = {"device": "synthetic", "multiprocessors": 1, "policy_source": "test", "policy": {"gpu_large_min_k": 340},
             "torch": "-", "cuda": "-", "date": "2026-01-01"}
    res = tune_qr.analyse(synthetic_rows(), ident)
    assert res["points"] == res["train_points"] + res["held_points"] and res["held_points"] > 0
    assert abs(res["fit"]["L"] - 350) <= 40 and 2.0 <= res["fit"]["F"] <= 4.0
    assert res["fit"]["train_geo"] < 1.01
    fitted = res["rules"]["fitted"]
    assert fitted["held_geo"] < 1.02                                   # the rule carries over to shapes it has not seen
    assert res["rules"]["always the grid-parallel QR"]["held_geo"] > fitted["held_geo"]
    assert res["rules"]["always the block-per-matrix kernel"]["held_geo"] > fitted["held_geo"]
    assert 0.015 < res["noise"]["median"] < 0.025                      # the 2 % between the synthetic passes
    train_shapes = {(s["family"], s["rows"], s["cols"]) for s in res["surface"]} - {tuple(h) for h in res["held_shapes"]}
    assert not train_shapes & {tuple(h) for h in res["held_shapes"]}
    text = tune_qr.report(res)
    assert "## The rule" in text and "held-out" in text and "| 8192x128 | 16 |" in text
