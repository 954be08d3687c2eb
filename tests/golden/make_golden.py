"""Generates tests/golden/qr_golden.npz: outputs of the reference's own CPU QR
(src/qr_cpu.mm, compiled unchanged into oracle/_ref by oracle/Makefile) on small
seeded inputs. Run where the reference checkout exists:

    python tests/golden/make_golden.py

The inputs are regenerated from their seeds by the tests (workloads.generate and
the literals below), so only the reference's Q and R are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [os.path.join(ROOT, "oracle"), os.path.join(ROOT, "metal-linalg_b200")]

import harness  # noqa: E402
from metal_linalg_torch import workloads  # noqa: E402

# name -> (input, modes)
CASES = {
    # the two 3 x 2 matrices of the reference's C API test (tests/test_c_api.c:31)
    "capi_3x2": (np.array([1, 2, 3, 4, 5, 6, 2, 0, 0, 3, 1, 1], np.float32).reshape(2, 3, 2),
                 ("reduced", "complete", "r")),
    # the rank-2 3 x 3 example of the reference's documentation (docs/qr.md:77-88)
    "doc_3x3": (np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9]], np.float32).reshape(1, 3, 3), ("reduced",)),
    "c1_32x32": (lambda: workloads.generate("c1_32x32", batch=4).numpy(), ("reduced", "complete")),
    "c2_16x16_magnitudes": (lambda: workloads.generate("c2_16x16_magnitudes", batch=16).numpy(), ("reduced",)),
    "c3_256x256_rank224": (lambda: workloads.generate("c3_256x256_rank224", batch=1).numpy(), ("reduced",)),
    "c4_tall_512x64": (lambda: workloads.generate("c4_65536x64_tall", batch=1, rows=512).numpy(), ("reduced",)),
    "wide_5x8": (lambda: np.random.default_rng(7).standard_normal((3, 5, 8)).astype(np.float32),
                 ("reduced", "complete", "r")),
    "tall_9x4": (lambda: np.random.default_rng(8).standard_normal((3, 9, 4)).astype(np.float32),
                 ("reduced", "complete", "r")),
}


def case_input(name):
    a = CASES[name][0]
    return a() if callable(a) else a


def main():
    if harness.load_ref() is None:
        harness.build()
    if harness.load_ref() is None:
        raise SystemExit("oracle/_ref is not built: the reference checkout is needed")
    out = {}
    for name, (_, modes) in CASES.items():
        a = case_input(name)
        for mode in modes:
            q, r = harness.ref_qr(a, mode)
            if q is not None:
                out[f"{name}/{mode}/q"] = q
            out[f"{name}/{mode}/r"] = r
    path = os.path.join(HERE, "qr_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays,", harness.load_ref().ref_lapack_config().decode())


if __name__ == "__main__":
    main()
