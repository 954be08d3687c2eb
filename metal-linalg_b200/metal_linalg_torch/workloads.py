"""Seeded synthetic inputs for the five benchmark configurations of the QR path.

The reference benchmarks on synthetic N(0,1) matrices only (benchmarks/
benchmark_qr.cpp:52-60, tuning/sweep_qr.cpp:38-45); no dataset is involved. The
generators use torch's CPU generator so that the same seed gives the same
matrices on every machine. `batch` shrinks a configuration for tests (the
distribution and the seed stay).
"""
import math

import torch

CONFIGS = {
    # name: (default batch, rows, cols, modes, seed)
    "c1_32x32": (1024, 32, 32, ("reduced",), 0),
    "c2_16x16_magnitudes": (262144, 16, 16, ("reduced",), 1),
    "c3_256x256_rank224": (4096, 256, 256, ("reduced", "complete"), 2),
    "c4_65536x64_tall": (64, 65536, 64, ("reduced",), 3),
    "c5a_4096x4096": (1, 4096, 4096, ("reduced",), 4),
    "c5b_8192x8192": (8, 8192, 8192, ("reduced",), 4),
}


def qr_flops(m, n, mode="reduced"):
    """Algorithmic flops of one QR: sgeqrf 2mn^2 - 2n^3/3 (m >= n; by symmetry of
    the count for a wide matrix 2nm^2 - 2m^3/3) plus, unless R alone, sorgqr's
    4 m c k - 2 (m + c) k^2 + 4 k^3 / 3 for c columns of Q from k reflectors."""
    k = min(m, n)
    geqrf = 2.0 * max(m, n) * k * k - (2.0 / 3.0) * k ** 3
    if mode == "r":
        return geqrf
    c = m if mode == "complete" else k
    return geqrf + 4.0 * m * c * k - 2.0 * (m + c) * k * k + (4.0 / 3.0) * k ** 3


def qr_bytes(m, n, mode="reduced"):
    """Algorithmic bytes of one QR: A read once, Q and R written once."""
    k = min(m, n)
    qc = 0 if mode == "r" else (m if mode == "complete" else k)
    rr = m if mode == "complete" else k
    return 4 * (m * n + m * qc + rr * n)


def generate(name, batch=None, rows=None, device=None):
    """The input of configuration `name` as a float32 tensor [batch, M, N] (on the CPU unless
    `device` is given). `rows` shortens the tall configuration for tests. The random draws always
    come from the seeded CPU generator; `device` only says where the third configuration's float64
    orthogonal factors are formed (4096 pairs of 256 x 256 QRs take the host cores half a minute),
    so its matrices differ from the CPU-built ones in the last bits, not in distribution."""
    default_batch, m, n, _, seed = CONFIGS[name]
    b = default_batch if batch is None else batch
    if rows is not None:
        m = rows
    g = torch.Generator().manual_seed(seed)
    if name == "c1_32x32" or name == "c4_65536x64_tall":
        return torch.randn(b, m, n, generator=g, dtype=torch.float32)
    if name == "c2_16x16_magnitudes":
        a = torch.randn(b, m, n, generator=g, dtype=torch.float32)
        u = torch.rand(b, generator=g, dtype=torch.float64) * 67.0 - 30.0      # U(-30, 37)
        return (a.double() * torch.pow(torch.tensor(10.0, dtype=torch.float64), u)[:, None, None]).float()
    if name == "c3_256x256_rank224":
        # U diag(s) V^T, U and V the Q factors of N(0,1) matrices (float64), s log-spaced
        # from 1 to 1e-7 with the last 32 exactly zero
        where = torch.device(device) if device is not None else torch.device("cpu")
        u = torch.linalg.qr(torch.randn(b, m, m, generator=g, dtype=torch.float64).to(where))[0]
        v = torch.linalg.qr(torch.randn(b, n, n, generator=g, dtype=torch.float64).to(where))[0]
        k = min(m, n)
        s = torch.logspace(0.0, -7.0, k, dtype=torch.float64, device=where)
        s[k - max(1, k // 8):] = 0.0
        return ((u[:, :, :k] * s) @ v[:, :, :k].mT).float()
    if name in ("c5a_4096x4096", "c5b_8192x8192"):
        if name == "c5b_8192x8192":   # continues the stream after the 4096 x 4096 matrix
            torch.rand(4096 * 4096, generator=g, dtype=torch.float32)
        return torch.rand(b, m, n, generator=g, dtype=torch.float32) * 2.0 - 1.0
    raise KeyError(name)


def config2_scale(batch):
    """The 10^u factors of configuration 2, for tests that undo them."""
    g = torch.Generator().manual_seed(CONFIGS["c2_16x16_magnitudes"][4])
    torch.randn(batch, 16, 16, generator=g, dtype=torch.float32)
    u = torch.rand(batch, generator=g, dtype=torch.float64) * 67.0 - 30.0
    return torch.pow(torch.tensor(10.0, dtype=torch.float64), u)


def tolerance(n):
    """10 n eps with eps = 2^-23: the bound on ||A - QR||_F / ||A||_F and on ||Q^T Q - I||_F."""
    return 10.0 * n * math.ldexp(1.0, -23)
