"""Generates tests/golden/svd_golden.npz: singular values by LAPACK's sgesdd in float32, the routine the
reference's CPU SVD calls (src/svd.mm:807-874), from the OpenBLAS inside the scipy wheel, on small
seeded inputs, and the same in float64 (dgesdd):

    python tests/golden/make_svd_golden.py

The inputs are regenerated from their seeds by the tests (CASES below), so only the values are stored.
"""
import os

import numpy as np
import scipy.linalg

HERE = os.path.dirname(os.path.abspath(__file__))


def _graded(seed, m, n, lo):
    """A matrix with singular values 1 ... lo, log-spaced."""
    rng = np.random.default_rng(seed)
    k = min(m, n)
    u, _ = np.linalg.qr(rng.standard_normal((m, k)))
    v, _ = np.linalg.qr(rng.standard_normal((n, k)))
    return ((u * np.logspace(0, np.log10(lo), k)) @ v.T).astype(np.float32)[None]


# name -> input [batch, m, n]
CASES = {
    # the reference's C API case (tests/test_c_api.c:97-111): rows of norms 3 and 2
    "capi_2x3": lambda: np.array([3, 0, 0, 0, 0, 2], np.float32).reshape(1, 2, 3),
    "square_32": lambda: np.random.default_rng(21).standard_normal((6, 32, 32)).astype(np.float32),
    "square_16": lambda: np.random.default_rng(22).standard_normal((8, 16, 16)).astype(np.float32),
    "tall_800x12": lambda: np.random.default_rng(23).standard_normal((3, 800, 12)).astype(np.float32),
    "tall_5000x32": lambda: np.random.default_rng(24).standard_normal((2, 5000, 32)).astype(np.float32),
    "wide_7x300": lambda: np.random.default_rng(25).standard_normal((4, 7, 300)).astype(np.float32),
    "odd_19x5": lambda: np.random.default_rng(26).standard_normal((5, 19, 5)).astype(np.float32),
    "graded_80x24": lambda: _graded(27, 80, 24, 1e-5),
    "square_64": lambda: np.random.default_rng(30).standard_normal((3, 64, 64)).astype(np.float32),
    "tall_3000x100": lambda: np.random.default_rng(31).standard_normal((2, 3000, 100)).astype(np.float32),
    "wide_128x700": lambda: np.random.default_rng(32).standard_normal((2, 128, 700)).astype(np.float32),
    "graded_300x96": lambda: _graded(33, 300, 96, 1e-5),
    "rank5_200x48": lambda: (np.random.default_rng(34).standard_normal((2, 200, 5)).astype(np.float32)
                             @ np.random.default_rng(35).standard_normal((2, 5, 48)).astype(np.float32)),
    "rank3_40x8": lambda: (np.random.default_rng(28).standard_normal((2, 40, 3)).astype(np.float32)
                           @ np.random.default_rng(29).standard_normal((2, 3, 8)).astype(np.float32)),
}


def main():
    out = {}
    for name, make in CASES.items():
        a = make()
        out[f"{name}/s32"] = np.stack([scipy.linalg.svd(x, compute_uv=False, lapack_driver="gesdd") for x in a])
        out[f"{name}/s64"] = np.stack([scipy.linalg.svd(x.astype(np.float64), compute_uv=False, lapack_driver="gesdd")
                                       for x in a])
        assert out[f"{name}/s32"].dtype == np.float32
    path = os.path.join(HERE, "svd_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
