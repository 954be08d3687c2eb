"""Seeded random shapes, batches, modes and magnitudes through the default routing: reconstruction and orthogonality
in float64 on the GPU against 10 n eps (workloads.tolerance), R upper triangular and finite; for R alone, R^T R against
A^T A. Shapes are drawn around the routing's borders (192 to 511 rows with at most 64 columns, trees of several
levels, blocked matrices of two to twenty aggregates, wide matrices), where a kernel is entered with its smallest and
most ragged inputs."""
import os
import random
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(HERE, "..", "metal-linalg_b200"), os.path.join(HERE, "..")]

pytestmark = pytest.mark.gpu

EPS = 2.0 ** -23


def _draw(rng):
    kind = rng.choice(["tall64", "tall64", "talls", "blocked", "blocked", "mid", "wide", "tallbig"])
    if kind == "tall64":
        m, n, b = rng.randint(192, 6000), rng.randint(1, 64), rng.choice([1, 2, 3, 7, 33])
    elif kind == "talls":
        m, n, b = rng.randint(192, 511), rng.randint(1, 64), rng.choice([1, 5, 64, 300])
    elif kind == "tallbig":
        m, n, b = rng.randint(6000, 70000), rng.randint(1, 128), rng.choice([1, 2, 5])
    elif kind == "blocked":
        m, n, b = rng.randint(300, 3000), rng.randint(130, 2500), rng.choice([1, 1, 1, 2, 3])
    elif kind == "mid":
        m, n, b = rng.randint(33, 1024), rng.randint(33, 700), rng.choice([1, 4, 40])
    else:
        m, n, b = rng.randint(20, 600), rng.randint(601, 3000), rng.choice([1, 2, 9])
    if b * m * n > 40_000_000:
        b = max(1, 40_000_000 // (m * n))
    mode = rng.choice(["reduced", "reduced", "r", "complete"])
    if mode == "complete" and m > 2500:
        mode = "reduced"
    return kind, b, m, n, mode


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_shapes(seed):
    import metal_linalg_torch as mlt

    rng = random.Random(seed)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    failures = []
    for _ in range(30):
        kind, b, m, n, mode = _draw(rng)
        a = torch.randn(b, m, n, device="cuda", generator=gen)
        if rng.random() < 0.2:
            a *= 10.0 ** rng.uniform(-20, 20)
        if rng.random() < 0.15 and n > 4:
            a[:, :, n // 2] = a[:, :, n // 2 - 1] * 1.0001       # nearly dependent neighbours
        q, r = mlt.qr(a, mode)
        torch.cuda.synchronize()
        a64, r64 = a.double(), r.double()
        tol = 10 * n * EPS
        msg = []
        if not torch.isfinite(r).all():
            msg.append("R not finite")
        if (torch.tril(r, -1) != 0).any():
            msg.append("R not upper triangular")
        if mode != "r":
            q64 = q.double()
            recon = (torch.linalg.matrix_norm(a64 - q64 @ r64) / torch.linalg.matrix_norm(a64).clamp_min(1e-300)).max().item()
            eye = torch.eye(q.shape[-1], device="cuda", dtype=torch.float64)
            orth = torch.linalg.matrix_norm(q64.mT @ q64 - eye).max().item()
            if not recon <= tol:
                msg.append(f"reconstruction {recon:.2e} > {tol:.2e}")
            # a float32 Q of c columns is off by about 0.3 sqrt(c) eps from rounding its entries alone (the exact Q of
            # 1833 x 1, rounded: 1.5e-6), which passes 10 n eps for a complete Q of one or two columns
            floor = 0.5 * q.shape[-1] ** 0.5 * EPS
            if not orth <= max(tol, floor):
                msg.append(f"orthogonality {orth:.2e} > {max(tol, floor):.2e}")
        else:
            g = a64.mT @ a64
            d = (torch.linalg.matrix_norm(r64.mT @ r64 - g) / torch.linalg.matrix_norm(g).clamp_min(1e-300)).max().item()
            if not d <= 20 * n * EPS:
                msg.append(f"R^T R off A^T A by {d:.2e}")
        if msg:
            failures.append((kind, tuple(a.shape), mode, mlt.qr_kernel(m, n, b, mode), msg))
    assert not failures, failures
