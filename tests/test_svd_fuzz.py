"""Seeded random shapes, batches and magnitudes through the SVD's routing (min(M, N) <= 128): singular values against
torch.linalg.svdvals in float64 on the GPU within the reference's own bounds (tests/test_svd.cpp:41-43: 2e-5, here of
the largest singular value, growing as sqrt(K / 64) beyond 64 columns), and with vectors the reconstruction U diag(S) Vt. Shapes are drawn
around the borders of the QR kernels underneath (small, the trees of row blocks, wide matrices by their transpose)."""
import os
import random
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(HERE, "..", "metal-linalg_b200"), os.path.join(HERE, "..")]

pytestmark = pytest.mark.gpu


def _draw(rng):
    kind = rng.choice(["small", "tall", "wide", "mid", "talltall"])
    if kind == "small":
        m, n, b = rng.randint(1, 32), rng.randint(1, 32), rng.choice([1, 7, 300, 5000])
    elif kind == "tall":
        m, n, b = rng.randint(64, 4000), rng.randint(1, 128), rng.choice([1, 3, 40])
    elif kind == "talltall":
        m, n, b = rng.randint(4000, 70000), rng.randint(1, 64), rng.choice([1, 2])
    elif kind == "wide":
        m, n, b = rng.randint(1, 128), rng.randint(129, 3000), rng.choice([1, 3, 20])
    else:
        m, n, b = rng.randint(33, 128), rng.randint(33, 128), rng.choice([1, 9, 100])
    if b * m * n > 30_000_000:
        b = max(1, 30_000_000 // (m * n))
    return kind, b, m, n


@pytest.mark.parametrize("seed", [5, 6, 7])
def test_random_shapes(seed):
    import metal_linalg_torch as mlt

    rng = random.Random(seed)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    failures = []
    for _ in range(12):
        kind, b, m, n = _draw(rng)
        a = torch.randn(b, m, n, device="cuda", generator=gen)
        if rng.random() < 0.2:
            a *= 10.0 ** rng.uniform(-15, 15)
        vectors = rng.random() < 0.6
        if vectors:
            u, s, vt = mlt.svd(a)
        else:
            s = mlt.svdvals(a)
        torch.cuda.synchronize()
        a64 = a.double()
        ref = torch.linalg.svdvals(a64)
        bound = 2e-5 * max(1.0, (min(m, n) / 64) ** 0.5)
        msg = []
        err = ((s.double() - ref).abs() / ref[:, :1].clamp_min(1e-300)).max().item()
        if not err <= bound:
            msg.append(f"singular values off by {err:.2e} > {bound:.2e}")
        if vectors:
            back = (u.double() * s.double().unsqueeze(-2)) @ vt.double()
            rec = (torch.linalg.matrix_norm(a64 - back) / torch.linalg.matrix_norm(a64).clamp_min(1e-300)).max().item()
            if not rec <= bound:
                msg.append(f"reconstruction {rec:.2e} > {bound:.2e}")
        if msg:
            failures.append((kind, tuple(a.shape), "vectors" if vectors else "values", mlt.svd_backend(m, n, b), msg))
    assert not failures, failures
