"""Parity of the CUDA QR with the CPU oracle, through the C ABI, on a B200.

The checks restate the reference's own suites: tests/test_qr.cpp (edge shapes,
identity/zero/constant matrices, non-finite isolation, modes, magnitudes, nearly
dependent columns), tests/test_core.cpp:134-167,407-437 (buffers), tests/
test_c_api.c:29-81,201-206 (C API) and python-torch/tests/test_torch.py (the
binding), with the tolerances of the benchmark definition: ||A - QR||_F / ||A||_F
and ||Q^T Q - I||_F at most 10 n eps (eps = 2^-23), R within 1e-4 relative of
the oracle's after sign normalisation, R's strict lower triangle exactly zero.
"""
import os
import sys

import numpy as np
import pytest
import torch

import harness
import metal_linalg_torch as mlt
from metal_linalg_torch import _lib, workloads

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden  # noqa: E402

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qr_golden.npz"))


def gpu_qr(a, mode="reduced", kernel=None):
    """numpy in, numpy out, through the C ABI on device pointers (the torch binding)."""
    t = torch.as_tensor(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    if kernel:
        os.environ["QR_KERNEL"] = kernel
    try:
        q, r = mlt.qr(t, mode)
    finally:
        os.environ.pop("QR_KERNEL", None)
    torch.cuda.synchronize()
    return (q.cpu().numpy() if q.numel() else None), r.cpu().numpy()


def check(a, q, r, mode, r_ref=None, tol_scale=1.0):
    *lead, m, n = a.shape
    k = min(m, n)
    tol = workloads.tolerance(n) * tol_scale
    rr = m if mode == "complete" else k
    assert r.shape == (*lead, rr, n)
    assert np.isfinite(r).all()
    if rr > 1:
        assert np.abs(np.tril(r, -1)).max() == 0.0, "R is not exactly upper triangular"
    if mode == "complete" and m > k:
        assert np.abs(r[..., k:, :]).max() == 0.0, "rows below K are not exactly zero"
    if mode != "r":
        qc = m if mode == "complete" else k
        assert q.shape == (*lead, m, qc)
        recon, orth, _ = harness.metrics(a, q, r)
        assert recon.max() <= tol, f"reconstruction {recon.max():.3e} > {tol:.3e}"
        assert orth.max() <= tol, f"orthogonality {orth.max():.3e} > {tol:.3e}"
    if r_ref is not None:
        par = harness.r_parity(r, r_ref)
        assert par <= 1e-4, f"R differs from the oracle's by {par:.3e}"


# ---------------------------------------------------------------------------
# Shapes, modes, kernels
# ---------------------------------------------------------------------------

SMALL = [(1, 1), (1, 5), (5, 1), (2, 2), (3, 2), (2, 3), (7, 7), (8, 8), (9, 16), (16, 16), (16, 9), (17, 9),
         (31, 32), (32, 31), (32, 32), (32, 8), (8, 32), (20, 13), (13, 20)]
MID = [(33, 33), (40, 40), (64, 64), (64, 16), (16, 64), (100, 37), (37, 100), (96, 80), (128, 128), (129, 65),
       (65, 129), (200, 200), (256, 256), (300, 40), (520, 520), (600, 64), (1024, 16), (1000, 130), (64, 2048),
       (1024, 1024)]


@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
@pytest.mark.parametrize("shape", SMALL)
def test_small_kernel_shapes(shape, mode):
    m, n = shape
    rng = np.random.default_rng(m * 100 + n)
    a = rng.standard_normal((37, m, n)).astype(np.float32)     # 37: groups and warps only partly filled
    assert mlt.qr_kernel(m, n, 37, mode) == "small"
    q, r = gpu_qr(a, mode)
    _, r_ref = harness.oracle_qr(a, mode)
    check(a, q, r, mode, r_ref)


@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
@pytest.mark.parametrize("shape", MID)
def test_mid_kernel_shapes(shape, mode):
    m, n = shape
    if mode == "complete" and m * m > 1 << 21:
        batch = 1
    else:
        batch = 3
    rng = np.random.default_rng(m * 100 + n)
    a = rng.standard_normal((batch, m, n)).astype(np.float32)
    q, r = gpu_qr(a, mode, kernel="mid")
    _, r_ref = harness.oracle_qr(a, mode)
    check(a, q, r, mode, r_ref)


@pytest.mark.parametrize("stream", ["0", "2"])
@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
@pytest.mark.parametrize("n,batch", [(8, 60001), (16, 30001), (32, 9001), (32, 37), (16, 3), (8, 1)])
def test_small_square_streaming_and_direct(n, batch, mode, stream):
    """Square 8, 16 and 32: the kernel that streams matrices through shared memory by bulk copies
    (QR_SMALL_STREAM=2: wherever it can) and the one that loads and stores for itself (0), on batches
    that leave the last warp's unit part filled and give every persistent warp several units."""
    rng = np.random.default_rng(n + batch)
    a = rng.standard_normal((batch, n, n)).astype(np.float32)
    a[batch - 1] *= 1e-30
    good = np.ones(batch, bool)
    if batch > 2:
        a[batch // 2, n - 1, 0] = np.inf
        good[batch // 2] = False
    os.environ["QR_SMALL_STREAM"] = stream
    try:
        q, r = gpu_qr(a, mode)
    finally:
        os.environ.pop("QR_SMALL_STREAM", None)
    if batch > 2:
        assert np.isnan(r[batch // 2]).all() and (q is None or np.isnan(q[batch // 2]).all())
    _, r_ref = harness.oracle_qr(a[good], mode)
    check(a[good], None if q is None else q[good], r[good], mode, r_ref)


def test_small_square_off_a_16_byte_boundary():
    """The bulk copies need 16-byte boundaries: a tensor that starts 4 bytes off one takes the
    kernel that loads and stores for itself, with the same results."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((1000, 16, 16)).astype(np.float32)
    base = torch.empty(a.size + 1, dtype=torch.float32, device="cuda")
    t = base[1:].view(1000, 16, 16)
    t.copy_(torch.as_tensor(a))
    assert t.data_ptr() % 16 == 4
    q, r = mlt.qr(t)
    torch.cuda.synchronize()
    _, r_ref = harness.oracle_qr(a)
    check(a, q.cpu().numpy(), r.cpu().numpy(), "reduced", r_ref)


TALL = [(512, 32), (512, 64), (700, 50), (1000, 100), (1024, 128), (1024, 1), (1025, 8), (1500, 64), (2048, 64), (4096, 16), (5000, 33), (20000, 40), (17000, 24), (9000, 128), (70000, 5)]


@pytest.mark.parametrize("mode", ["reduced", "r"])
@pytest.mark.parametrize("shape", TALL)
def test_tsqr_shapes(shape, mode):
    """Tall thin matrices through the tree of row blocks (the reference's TSQR depth cases,
    tests/test_qr.cpp:364-367, among them)."""
    m, n = shape
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal((2, m, n)).astype(np.float32)
    assert mlt.qr_kernel(m, n, 64, mode) == "tsqr"             # a batch goes to the tree ...
    q, r = gpu_qr(a, mode, kernel="tsqr")
    _, r_ref = harness.oracle_qr(a, mode)
    check(a, q, r, mode, r_ref)


@pytest.mark.parametrize("mode", ["reduced", "r"])
@pytest.mark.parametrize("shape", [(513, 64), (520, 64), (1030, 64), (2050, 40), (2700, 48), (769, 3)])
def test_tsqr_short_last_blocks(shape, mode):
    """Row counts that leave a last block shorter than the matrix is wide, at the first level ((1030, 64): six rows
    over four blocks) and at the second ((2700, 48): eleven 48-row factors make 528 rows): the block before it
    gives up rows, so no block has fewer rows than columns."""
    m, n = shape
    rng = np.random.default_rng(3 * m + n)
    a = rng.standard_normal((3, m, n)).astype(np.float32)
    q, r = gpu_qr(a, mode, kernel="tsqr")
    _, r_ref = harness.oracle_qr(a, mode)
    check(a, q, r, mode, r_ref)


@pytest.mark.parametrize("mode", ["reduced", "r"])
@pytest.mark.parametrize("shape", [(256, 64), (192, 64), (200, 40), (255, 33), (384, 64), (500, 48), (300, 7), (257, 64), (511, 1)])
def test_tsqr_one_and_two_blocks(shape, mode):
    """With at most 64 columns a matrix of 192 to 511 rows goes to the tree of blocks kept as reflectors too: one block
    (no tree at all) up to 256 rows, two beyond (257 x 64: a second block of one row takes 63 from the first)."""
    m, n = shape
    assert mlt.qr_kernel(m, n, 64, mode) == "tsqr" and mlt.qr_kernel(m, n, 1, mode) == "tsqr"
    rng = np.random.default_rng(5 * m + n)
    a = rng.standard_normal((5, m, n)).astype(np.float32)
    a[3] *= 1e-20
    q, r = gpu_qr(a, mode)
    _, r_ref = harness.oracle_qr(a, mode)
    check(a, q, r, mode, r_ref)


@pytest.mark.parametrize("shape", [(512, 64), (5000, 33), (4096, 16)])
def test_tsqr_older_scheme_behind_its_switch(shape):
    """QR_TSQR_VT=0: blocks through the general block kernel with an explicit Q at every block (the scheme that
    stays for 65 to 128 columns), with the same results."""
    m, n = shape
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal((2, m, n)).astype(np.float32)
    os.environ["QR_TSQR_VT"] = "0"
    try:
        q, r = gpu_qr(a, "reduced", kernel="tsqr")
    finally:
        os.environ.pop("QR_TSQR_VT", None)
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


def test_tsqr_nearly_parallel_neighbours():
    """Column pairs that are nearly parallel below the diagonal make the two-column step fall back to two
    single steps (qr_tsqr_vt.cu, the same rule as qr_panel_cols.cuh); both sides of the rule in one matrix."""
    rng = np.random.default_rng(77)
    a = rng.standard_normal((4, 2048, 64)).astype(np.float32)
    a[:, :, 1] = a[:, :, 0] * 1.5 + 1e-2 * a[:, :, 1]          # pair (0, 1) of the first panel
    a[:, :, 41] = a[:, :, 40] - 1e-2 * a[:, :, 41]             # pair (40, 41) of the second
    a[:, :, 63] = a[:, :, 62] + 3e-2 * a[:, :, 63]
    q, r = gpu_qr(a, "reduced", kernel="tsqr")
    check(a, q, r, "reduced")
    _, r_ref = harness.oracle_qr(a)
    assert harness.r_parity(r, r_ref) <= 2e-3                  # columns 1e-2 apart: R's small entries carry the conditioning


def test_tsqr_nonfinite_and_constant():
    rng = np.random.default_rng(14)
    a = rng.standard_normal((4, 3000, 48)).astype(np.float32)
    a[1, 2999, 47] = np.nan
    a[2] = 2.5                                   # constant: rank one
    q, r = gpu_qr(a)
    assert np.isnan(q[1]).all() and np.isnan(r[1]).all()
    good = [0, 2, 3]
    check(a[good], q[good], r[good], "reduced")
    _, r_ref = harness.oracle_qr(a[[0, 3]])
    assert harness.r_parity(r[[0, 3]], r_ref) <= 1e-4


def test_config4_tall_shrunk_batch():
    a = workloads.generate("c4_65536x64_tall", batch=2).numpy()
    q, r = gpu_qr(a)
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


BLOCKED = [(40, 40), (100, 64), (64, 100), (200, 200), (300, 2000), (1025, 1025), (1500, 1200), (2000, 300),
           (1100, 130), (3000, 200)]


@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
@pytest.mark.parametrize("shape", BLOCKED)
def test_blocked_kernel_shapes(shape, mode):
    """The grid-parallel blocked QR, forced on shapes small enough for the CPU oracle."""
    m, n = shape
    if mode == "complete" and m > 2000:
        pytest.skip("a 3000 x 3000 Q on the CPU oracle takes too long")
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal((2, m, n)).astype(np.float32)
    q, r = gpu_qr(a, mode, kernel="blocked")
    _, r_ref = harness.oracle_qr(a, mode)
    check(a, q, r, mode, r_ref)


@pytest.mark.parametrize("switch", ["QR_TENSOR=0", "QR_NO_LOOKAHEAD=1", "QR_PANEL_TREE=1", "QR_BACKWARD_Q=1", "QR_PANEL_ROWS=1",
                                    "QR_NO_PDL=1", "QR_PANEL_CLUSTER=0", "QR_TC_SPLIT=0", "QR_PANEL_PAIRS=0", "QR_INNER_FUSED=0",
                                    "QR_PANEL_CLUSTER=8", "QR_LOOK_PANELS=0", "QR_PANEL_QUADS=0", "QR_PANEL_POST=0", "QR_TC_PAIR=0", "QR_TC_PAIR=1",
                                    "QR_TC_YZ_PAIR=1"])
def test_blocked_fallback_paths(switch):
    """The blocked QR's alternatives give the same factorisation: the FP32 FMA products instead of
    the tensor cores, one stream instead of look-ahead, the general tree for every panel, Q accumulated
    backward instead of forward, panels with a row per thread instead of a column per lane, ordinary
    launches instead of programmatic dependent ones (QR_NO_PDL is read once per process: it takes
    effect only when set before the first call), panels by the tree of row blocks instead of one
    cluster launch, tensor-core products that split their operands in every block instead of once,
    panel steps a column a reduction instead of two, the update inside the aggregate in two launches
    instead of one cluster launch, panel clusters of eight blocks of 512 rows instead of sixteen of 256, the wide products' blocks with one or two accumulators and one or two column tiles whatever the
    size, look-ahead by aggregates instead of by panels."""
    rng = np.random.default_rng(16)
    a = rng.standard_normal((1, 900, 900)).astype(np.float32)
    q0, r0 = gpu_qr(a, "reduced", kernel="blocked")
    name, value = switch.split("=")
    os.environ[name] = value
    try:
        q1, r1 = gpu_qr(a, "reduced", kernel="blocked")
    finally:
        os.environ.pop(name, None)
    check(a, q1, r1, "reduced")
    assert harness.r_parity(r1, r0) <= 1e-4
    _, r_ref = harness.oracle_qr(a)
    assert harness.r_parity(r1, r_ref) <= 1e-4


@pytest.mark.parametrize("switch", ["", "QR_PANEL_CLUSTER=8", "QR_PANEL_CLUSTER=0", "QR_PANEL_PAIRS=0", "QR_PANEL_QUADS=0",
                                    "QR_PANEL_POST=0"])
def test_blocked_panels_of_2049_to_4096_rows(switch):
    """Panels of 2049 to 4096 rows: a cluster of sixteen blocks of 256 rows (the default, with the published columns
    kept in registers between the products and the update, the sums of four columns posted to mbarriers), of eight
    blocks of 512 rows, the tree of row blocks, the cluster with a column a reduction, and the cluster's own barrier
    for the sums, all against the reference."""
    rng = np.random.default_rng(31)
    a = rng.standard_normal((1, 3000, 96)).astype(np.float32)
    if switch:
        name, value = switch.split("=")
        os.environ[name] = value
    try:
        q, r = gpu_qr(a, "reduced", kernel="blocked")
    finally:
        if switch:
            os.environ.pop(name, None)
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
@pytest.mark.parametrize("shape", [(3, 700, 700), (2, 1000, 420), (2, 400, 1100), (1, 1300, 130), (1, 640, 257)])
def test_blocked_look_ahead_by_panels(shape, mode):
    """The look-ahead that keeps the next aggregate's columns up to date panel by panel on a third stream (the default
    for one matrix of at most 4608 rows; QR_LOOK_PANELS=1 asks for it on a batch, whose matrices run on several sets of
    streams at once): shapes with two to six aggregates, a last aggregate narrower than 128, one and two columns of
    the aggregate after the next, wide and tall, against the look-ahead by aggregates and the reference."""
    b, m, n = shape
    rng = np.random.default_rng(b * 1000 + m + n)
    a = rng.standard_normal((b, m, n)).astype(np.float32)
    os.environ["QR_LOOK_PANELS"] = "0"
    try:
        q0, r0 = gpu_qr(a, mode, kernel="blocked")
        os.environ["QR_LOOK_PANELS"] = "1"
        q1, r1 = gpu_qr(a, mode, kernel="blocked")
    finally:
        os.environ.pop("QR_LOOK_PANELS", None)
    check(a, q1, r1, mode)
    assert harness.r_parity(r1, r0) <= 1e-4
    _, r_ref = harness.oracle_qr(a, mode)
    assert harness.r_parity(r1, r_ref) <= 1e-4


@pytest.mark.parametrize("shape", [(256, 256), (200, 64), (250, 300), (300, 96), (476, 64), (257, 40), (512, 512), (450, 500)])
def test_mid_panel_paths(shape):
    """The mid kernel's panels with a column per lane (the default: 32 rows a lane up to 256 rows, 64 rows a lane
    in the instantiation for matrices of 257 to 512 rows) and a thread per entry (QR_MID_ROWS=1; panels above
    512 rows always) give the same factorisation."""
    m, n = shape
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal((5, m, n)).astype(np.float32)
    a[3] = 1.5                                   # constant: rank one, every later reflector the identity
    q0, r0 = gpu_qr(a, "reduced", kernel="mid")
    os.environ["QR_MID_ROWS"] = "1"
    try:
        q1, r1 = gpu_qr(a, "reduced", kernel="mid")
    finally:
        os.environ.pop("QR_MID_ROWS", None)
    os.environ["QR_PANEL_PAIRS"] = "0"      # a column a reduction instead of two
    try:
        q2, r2 = gpu_qr(a, "reduced", kernel="mid")
    finally:
        os.environ.pop("QR_PANEL_PAIRS", None)
    check(a, q0, r0, "reduced")
    check(a, q1, r1, "reduced")
    check(a, q2, r2, "reduced")
    good = [0, 1, 2, 4]
    assert harness.r_parity(r0[good], r1[good]) <= 1e-4
    assert harness.r_parity(r0[good], r2[good]) <= 1e-4
    _, r_ref = harness.oracle_qr(a[good])
    assert harness.r_parity(r0[good], r_ref) <= 1e-4


def test_blocked_panels_taller_than_the_register_kernels():
    """More than 16384 rows: every panel goes through the general tree and reconstruct_kernel."""
    rng = np.random.default_rng(17)
    a = rng.standard_normal((1, 20000, 70)).astype(np.float32)
    q, r = gpu_qr(a, "reduced", kernel="blocked")
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


def test_blocked_special_matrices():
    m, n = 700, 500
    eye = np.eye(m, n, dtype=np.float32)
    rng = np.random.default_rng(15)
    low = (rng.standard_normal((m, 40)) @ rng.standard_normal((40, n))).astype(np.float32)      # rank 40
    bad = rng.standard_normal((m, n)).astype(np.float32)
    bad[5, 7] = np.inf
    a = np.stack([eye, np.zeros((m, n), np.float32), np.full((m, n), 3.25, np.float32), low, bad,
                  (rng.standard_normal((m, n)) * 1e-30).astype(np.float32),
                  (rng.standard_normal((m, n)) * 1e30).astype(np.float32)])
    q, r = gpu_qr(a, "reduced", kernel="blocked")
    assert np.isnan(q[4]).all() and np.isnan(r[4]).all()
    good = [0, 1, 2, 3, 5, 6]
    check(a[good], q[good], r[good], "reduced")
    assert np.abs(r[1]).max() == 0.0


def _gpu_float64_properties(a, q, r, unit=None):
    """Per-matrix reconstruction and orthogonality in float64 on the GPU, on the unit-scale problem
    (`unit`: per-matrix scale [batch, 1, 1], or None), for batches and matrices too large for the
    CPU oracle; R's strict lower triangle exactly zero. Returns (recon_max, orth_max)."""
    tol = workloads.tolerance(a.shape[-1])
    recon_max = orth_max = 0.0
    step = max(1, (1 << 27) // (a.shape[-2] * max(a.shape[-1], q.shape[-1])))      # about 1 GiB of float64 a slice
    for b0 in range(0, a.shape[0], step):
        sl = slice(b0, b0 + step)
        a64, q64, r64 = a[sl].double(), q[sl].double(), r[sl].double()
        if unit is not None:
            a64, r64 = a64 / unit[sl], r64 / unit[sl]
        recon = torch.linalg.matrix_norm(a64 - q64 @ r64) / torch.linalg.matrix_norm(a64)
        del a64, r64
        eye = torch.eye(q.shape[-1], device=a.device, dtype=torch.float64)
        orth = torch.linalg.matrix_norm(q64.mT @ q64 - eye)
        recon_max, orth_max = max(recon_max, recon.max().item()), max(orth_max, orth.max().item())
        del q64
    assert recon_max <= tol, f"reconstruction {recon_max:.3e} > {tol:.3e}"
    assert orth_max <= tol, f"orthogonality {orth_max:.3e} > {tol:.3e}"
    assert torch.count_nonzero(torch.tril(r, -1)).item() == 0
    return recon_max, orth_max


def _r_against_reference(a, r):
    """R against the reference's own CPU QR (src/qr_cpu.mm: LAPACK sgeqrf on all host cores) after sign
    normalisation; the plain-C restatement where that library was not built."""
    host = a.cpu().numpy()
    ref = harness.ref_qr(host, "r")
    r_ref = ref[1] if ref is not None else harness.oracle_qr(host, "r")[1]
    par = harness.r_parity(r.cpu().numpy(), r_ref)
    assert par <= 1e-4, f"R differs from the reference's by {par:.3e}"
    return par


def test_config5a_4096_square():
    a = workloads.generate("c5a_4096x4096").cuda()
    assert mlt.qr_kernel(4096, 4096, 1) == "blocked"
    q, r = mlt.qr(a)
    torch.cuda.synchronize()
    _gpu_float64_properties(a, q, r)
    _r_against_reference(a, r)


@pytest.mark.parametrize("tensor", ["1", "0"])
def test_config5b_8192_square(tensor):
    """One of configuration 5b's eight 8192 x 8192 matrices (the first of the seeded stream), on the
    default path (3xTF32 tensor-core products) and on the FP32 FMA fallback (QR_TENSOR=0): reconstruction
    and orthogonality of the whole 8192 x 8192 Q in float64 against 10 n eps, R against the reference's."""
    a = workloads.generate("c5b_8192x8192", batch=1).cuda()
    assert mlt.qr_kernel(8192, 8192, 1) == "blocked"
    os.environ["QR_TENSOR"] = tensor
    try:
        q, r = mlt.qr(a)
        torch.cuda.synchronize()
    finally:
        os.environ.pop("QR_TENSOR", None)
    recon, orth = _gpu_float64_properties(a, q, r)
    par = _r_against_reference(a, r)
    print(f"8192 x 8192, QR_TENSOR={tensor}: reconstruction {recon:.3e}, orthogonality {orth:.3e} "
          f"(bound {workloads.tolerance(8192):.3e}), R parity {par:.3e}")


@pytest.mark.parametrize("mode", ["reduced", "complete"])
def test_config3_full_batch_properties(mode):
    """All 4096 rank-224 matrices of configuration 3 (the seeded N(0,1) draws on the CPU, the float64
    orthogonal factors formed on the GPU): float64 properties of every matrix, R against the oracle on
    a sample across the batch."""
    a = workloads.generate("c3_256x256_rank224", device="cuda").cuda()
    assert a.shape == (4096, 256, 256) and mlt.qr_kernel(256, 256, 4096, mode) == "mid"
    q, r = mlt.qr(a, mode)
    torch.cuda.synchronize()
    _gpu_float64_properties(a, q, r)
    idx = np.arange(0, a.shape[0], 128)
    sample = a[idx].cpu().numpy()
    _, r_ref = harness.oracle_qr(sample, mode)
    assert harness.r_parity(r[idx].cpu().numpy(), r_ref) <= 1e-4


def test_config4_full_batch_properties():
    """All 64 matrices of 65536 x 64 of configuration 4."""
    a = workloads.generate("c4_65536x64_tall").cuda()
    assert mlt.qr_kernel(65536, 64, 64) == "tsqr"
    q, r = mlt.qr(a)
    torch.cuda.synchronize()
    _gpu_float64_properties(a, q, r)
    idx = [0, 63]
    _, r_ref = harness.oracle_qr(a[idx].cpu().numpy())
    assert harness.r_parity(r[idx].cpu().numpy(), r_ref) <= 1e-4


def test_mid_kernel_on_small_shapes_agrees_with_small_kernel():
    rng = np.random.default_rng(5)
    a = rng.standard_normal((50, 24, 18)).astype(np.float32)
    q1, r1 = gpu_qr(a, "reduced", kernel="small")
    q2, r2 = gpu_qr(a, "reduced", kernel="mid")
    assert np.abs(r1 - r2).max() <= 1e-5 * np.abs(r1).max()
    assert np.abs(q1 - q2).max() <= 1e-5


def test_large_batch_persistent_loop():
    """More matrices than resident thread blocks: every slot is reused many times."""
    rng = np.random.default_rng(11)
    a = rng.standard_normal((1500, 48, 40)).astype(np.float32)
    q, r = gpu_qr(a, "reduced")
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


# ---------------------------------------------------------------------------
# Golden vectors of the reference's own CPU path
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("name,mode", [(n, md) for n, (_, mds) in make_golden.CASES.items() for md in mds])
def test_against_reference_fixtures(name, mode):
    a = make_golden.case_input(name)
    q, r = gpu_qr(a, mode)
    check(a, q, r, mode, GOLDEN[f"{name}/{mode}/r"])
    if mode != "r" and name not in ("c3_256x256_rank224", "doc_3x3"):
        qn, _ = harness.sign_normalise(q, r)
        qr_, _ = harness.sign_normalise(GOLDEN[f"{name}/{mode}/q"], GOLDEN[f"{name}/{mode}/r"])
        k = min(a.shape[-2:])
        assert np.abs(qn[..., :k] - qr_[..., :k]).max() <= 1e-4


def test_lapack_signs_in_small_and_mid_kernels():
    """R's diagonal has LAPACK's signs (not just up to sign) where a matrix goes to a
    warp or a thread block (reference: docs/qr.md:457-470)."""
    rng = np.random.default_rng(2)
    for shape in [(20, 16, 16), (5, 80, 72)]:
        a = rng.standard_normal(shape).astype(np.float32)
        _, r = gpu_qr(a, "r")
        _, r_ref = harness.oracle_qr(a, "r")
        d, d_ref = np.diagonal(r, axis1=-2, axis2=-1), np.diagonal(r_ref, axis1=-2, axis2=-1)
        assert np.array_equal(np.sign(d), np.sign(d_ref))
        assert np.abs(r - r_ref).max() <= 1e-4 * np.abs(r_ref).max()


# ---------------------------------------------------------------------------
# Special matrices (tests/test_qr.cpp:252-281,372-400)
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(16, 16), (32, 20), (64, 64), (200, 100), (600, 64)])
def test_identity_zero_constant(shape):
    m, n = shape
    eye = np.zeros((m, n), np.float32)
    eye[np.arange(min(m, n)), np.arange(min(m, n))] = 1.0
    a = np.stack([eye, np.zeros((m, n), np.float32), np.full((m, n), 3.25, np.float32),
                  np.full((m, n), -1e-3, np.float32)])
    q, r = gpu_qr(a, "reduced")
    assert np.isfinite(q).all() and np.isfinite(r).all()
    recon, orth, low = harness.metrics(a, q, r)
    tol = workloads.tolerance(n)
    assert recon.max() <= tol and low.max() == 0.0
    # Q of the identity and of the constant matrices is orthonormal; the zero matrix's Q is I's columns
    assert orth.max() <= tol
    assert np.abs(r[1]).max() == 0.0


@pytest.mark.parametrize("shape", [(12, 12), (32, 32), (70, 50), (300, 64)])
@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
def test_nonfinite_isolation(shape, mode):
    m, n = shape
    rng = np.random.default_rng(9)
    a = rng.standard_normal((5, m, n)).astype(np.float32)
    a[1, m // 2, n // 3] = np.nan
    a[3, m - 1, n - 1] = -np.inf
    q, r = gpu_qr(a, mode)
    for b in (1, 3):
        assert np.isnan(r[b]).all()
        if q is not None:
            assert np.isnan(q[b]).all()
    good = [0, 2, 4]
    _, r_ref = harness.oracle_qr(a[good], mode)
    check(a[good], None if q is None else q[good], r[good], mode, r_ref)


@pytest.mark.parametrize("scale", [1e-3, 1e-5, 1e-20, 1e-30, 1e18, 1e30, 1e37])
@pytest.mark.parametrize("shape", [(16, 16), (32, 32), (100, 60)])
def test_magnitudes(shape, scale):
    """tests/test_qr.cpp:557-603: accuracy is that of the unit-scale problem."""
    m, n = shape
    rng = np.random.default_rng(4)
    unit = rng.standard_normal((4, m, n)).astype(np.float32)
    unit /= np.abs(unit).max() * 1.5
    a = (unit.astype(np.float64) * scale).astype(np.float32)
    q, r = gpu_qr(a)
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


def test_mixed_magnitudes_in_one_batch():
    rng = np.random.default_rng(6)
    unit = rng.standard_normal((6, 24, 24)).astype(np.float64)
    scales = np.array([1e-30, 1.0, 1e30, 1e-12, 1e37 / 8, 1e-38])
    a = (unit * scales[:, None, None]).astype(np.float32)
    q, r = gpu_qr(a)
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


@pytest.mark.parametrize("shape", [(32, 32), (128, 96)])
def test_nearly_dependent_columns(shape):
    """tests/test_qr.cpp:611-652: columns that differ by 1e-6 keep Q orthonormal."""
    m, n = shape
    rng = np.random.default_rng(8)
    base = rng.standard_normal((3, m, 1))
    a = (base + 1e-6 * rng.standard_normal((3, m, n))).astype(np.float32)
    q, r = gpu_qr(a)
    check(a, q, r, "reduced")


def test_modes_agree():
    """tests/test_qr.cpp:132-190: R alone equals the reduced R; the complete Q starts
    with the reduced Q; rows below K are exactly zero."""
    rng = np.random.default_rng(10)
    for shape in [(6, 20, 12), (4, 90, 50), (4, 12, 20)]:
        a = rng.standard_normal(shape).astype(np.float32)
        q, r = gpu_qr(a, "reduced")
        _, r1 = gpu_qr(a, "r")
        qc, rc = gpu_qr(a, "complete")
        k = min(shape[1:])
        assert np.abs(r1 - r).max() <= 1e-5 * np.abs(r).max()
        assert np.abs(qc[..., :k] - q).max() <= 1e-5
        assert np.abs(rc[..., :k, :] - r).max() <= 1e-5 * np.abs(r).max()


# ---------------------------------------------------------------------------
# The benchmark configurations (full size where a CPU check is affordable)
# ---------------------------------------------------------------------------

def test_config1_full():
    a = workloads.generate("c1_32x32").numpy()
    q, r = gpu_qr(a)
    _, r_ref = harness.oracle_qr(a)
    check(a, q, r, "reduced", r_ref)


def test_config2_full_magnitudes():
    a = workloads.generate("c2_16x16_magnitudes")
    t = a.cuda()
    q, r = mlt.qr(t)
    torch.cuda.synchronize()
    # properties on the GPU in float64, on the unit-scale problem, for the whole batch
    s = torch.as_tensor(harness.unit_scale(a.numpy()), device="cuda")
    a64, r64, q64 = t.double() / s, r.double() / s, q.double()
    tol = workloads.tolerance(16)
    recon = torch.linalg.matrix_norm(a64 - q64 @ r64) / torch.linalg.matrix_norm(a64)
    orth = torch.linalg.matrix_norm(q64.mT @ q64 - torch.eye(16, device="cuda", dtype=torch.float64))
    assert recon.max().item() <= tol and orth.max().item() <= tol
    assert torch.count_nonzero(torch.tril(r, -1)).item() == 0
    # R against the oracle on a sample across the batch
    idx = np.arange(0, a.shape[0], 64)
    sample = a.numpy()[idx]
    _, r_ref = harness.oracle_qr(sample)
    assert harness.r_parity(r[idx].cpu().numpy(), r_ref) <= 1e-4


@pytest.mark.parametrize("mode", ["reduced", "complete"])
def test_config3_rank_deficient(mode):
    a = workloads.generate("c3_256x256_rank224", batch=24).numpy()
    q, r = gpu_qr(a, mode)
    _, r_ref = harness.oracle_qr(a, mode)
    check(a, q, r, mode, r_ref)


# ---------------------------------------------------------------------------
# The C API on host and device pointers (tests/test_c_api.c of the reference)
# ---------------------------------------------------------------------------

def test_capi_host_pointers_known_answers():
    lib = _lib.lib
    a = np.array([1, 2, 3, 4, 5, 6, 2, 0, 0, 3, 1, 1], np.float32)
    q, r = np.zeros(12, np.float32), np.zeros(8, np.float32)
    assert lib.metal_linalg_qr(a.ctypes.data, 2, 3, 2, q.ctypes.data, r.ctypes.data) == _lib.OK, _lib.last_error()
    A, Q, R = a.reshape(2, 3, 2), q.reshape(2, 3, 2), r.reshape(2, 2, 2)
    assert R[0, 1, 0] == 0.0 and R[1, 1, 0] == 0.0
    assert np.allclose(Q @ R, A, rtol=1e-5, atol=1e-5)
    r_alone = np.zeros(8, np.float32)
    assert lib.metal_linalg_qr_with_mode(a.ctypes.data, 2, 3, 2, 1, None, r_alone.ctypes.data) == _lib.OK
    assert np.allclose(r_alone, r, rtol=1e-5, atol=1e-6)
    qc, rc = np.zeros(18, np.float32), np.zeros(12, np.float32)
    assert lib.metal_linalg_qr_with_mode(a.ctypes.data, 2, 3, 2, 2, qc.ctypes.data, rc.ctypes.data) == _lib.OK
    QC, RC = qc.reshape(2, 3, 3), rc.reshape(2, 3, 2)
    assert np.all(RC[:, 2, :] == 0.0)
    assert np.allclose(np.swapaxes(QC, -1, -2) @ QC, np.eye(3), atol=1e-5)
    assert np.allclose(QC @ RC, A, rtol=1e-5, atol=1e-5)
    assert np.allclose(QC[:, :, :2], Q, atol=1e-5)
    # an error, then a success (tests/test_c_api.c:201-206)
    assert lib.metal_linalg_qr(None, 1, 2, 2, q.ctypes.data, r.ctypes.data) == _lib.INVALID_ARGUMENT
    eye = np.eye(2, dtype=np.float32)
    assert lib.metal_linalg_qr(eye.ctypes.data, 1, 2, 2, q.ctypes.data, r.ctypes.data) == _lib.OK
    # an unaligned host pointer (tests/test_core.cpp:407-417)
    buf = np.zeros(1 + 5 * 7 * 3, np.float32)
    rng = np.random.default_rng(1)
    buf[1:] = rng.standard_normal(5 * 7 * 3).astype(np.float32)
    qq, rr = np.zeros(5 * 7 * 3, np.float32), np.zeros(5 * 3 * 3, np.float32)
    assert lib.metal_linalg_qr(buf.ctypes.data + 4, 5, 7, 3, qq.ctypes.data, rr.ctypes.data) == _lib.OK
    check(buf[1:].reshape(5, 7, 3), qq.reshape(5, 7, 3), rr.reshape(5, 3, 3), "reduced")


def test_capi_host_pointers_staged_in_chunks():
    """A host batch larger than one staging chunk: several chunks through both buffer sets."""
    rng = np.random.default_rng(12)
    a = rng.standard_normal((40000, 32, 32)).astype(np.float32)          # 160 MB in, 320 MB out
    q, r = np.empty_like(a), np.empty_like(a)
    assert _lib.lib.metal_linalg_qr(a.ctypes.data, a.shape[0], 32, 32, q.ctypes.data, r.ctypes.data) == _lib.OK
    idx = np.arange(0, a.shape[0], 997)
    _, r_ref = harness.oracle_qr(a[idx])
    check(a[idx], q[idx], r[idx], "reduced", r_ref)
    qd, rd = gpu_qr(a[-5:])
    assert np.array_equal(qd, q[-5:]) and np.array_equal(rd, r[-5:])


def test_capi_mixed_pointers_rejected():
    a = torch.randn(2, 8, 8, device="cuda")
    q = np.zeros((2, 8, 8), np.float32)
    r = torch.empty(2, 8, 8, device="cuda")
    status = _lib.lib.metal_linalg_qr(a.data_ptr(), 2, 8, 8, q.ctypes.data, r.data_ptr())
    assert status == _lib.INVALID_ARGUMENT and "device" in _lib.last_error()


def test_capi_device_pointers_on_a_side_stream():
    a = torch.randn(64, 32, 32, device="cuda")
    q, r = torch.empty_like(a), torch.empty_like(a)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    _lib.qr(a.data_ptr(), 64, 32, 32, q.data_ptr(), r.data_ptr(), "reduced", s.cuda_stream)
    assert _lib.lib.metal_linalg_stream() == s.cuda_stream
    assert _lib.lib.metal_linalg_synchronize() == _lib.OK
    _lib.lib.metal_linalg_set_stream(None)
    check(a.cpu().numpy(), q.cpu().numpy(), r.cpu().numpy(), "reduced")


def test_device_queries():
    assert "B200" in mlt.device_name()
    assert mlt.gpu_core_count() == 148
    assert mlt.qr_policy_source().startswith(("tuned:", "env:", "user"))
    assert mlt.calibration_status() == ""
    assert mlt.qr_kernel(32, 32, 1000) == "small" and mlt.qr_kernel(256, 256, 4096) == "mid"
    # the measured routing: one matrix is spread over the grid from sqrt(M k) of 240, a batch later
    assert mlt.qr_kernel(512, 512, 1) == "blocked" and mlt.qr_kernel(512, 512, 32) == "mid"
    assert mlt.qr_kernel(384, 384, 4) == "blocked" and mlt.qr_kernel(192, 192, 1) == "mid"
    assert mlt.qr_kernel(1024, 1024, 16) == "blocked" and mlt.qr_kernel(1024, 1024, 128) == "mid"
    assert mlt.qr_kernel(4096, 64, 1) == "blocked" and mlt.qr_kernel(4096, 64, 16) == "tsqr"
    assert mlt.qr_kernel(8192, 128, 4) == "blocked" and mlt.qr_kernel(8192, 128, 5) == "tsqr"
    assert mlt.qr_kernel(2048, 32, 2) == "tsqr" and mlt.qr_kernel(2048, 32, 1) == "tsqr" and mlt.qr_kernel(4096, 64, 2) == "tsqr"
    assert mlt.qr_kernel(1 << 20, 32, 1) == "tsqr" and mlt.qr_kernel(65536, 64, 64) == "tsqr"
    # tall thin matrices of 512 to 1024 rows go to the tree too, unless less than eight times as tall as wide
    assert mlt.qr_kernel(1024, 64, 16) == "tsqr" and mlt.qr_kernel(512, 32, 1) == "tsqr" and mlt.qr_kernel(640, 96, 16) == "mid"
    assert mlt.qr_kernel(1024, 128, 1) == "blocked" and mlt.qr_kernel(1024, 64, 16, "complete") == "mid"
    assert mlt.qr_kernel(128, 128, 1) == "mid" and mlt.qr_kernel(4096, 4096, 64) == "blocked"
    # at most 64 columns and at least 192 rows (three times the columns): the tree of blocks kept as reflectors, even as one block
    assert mlt.qr_kernel(256, 64, 1000) == "tsqr" and mlt.qr_kernel(200, 40, 8) == "tsqr" and mlt.qr_kernel(384, 64, 1) == "tsqr"
    assert mlt.qr_kernel(128, 64, 1000) == "mid" and mlt.qr_kernel(191, 40, 8) == "mid" and mlt.qr_kernel(256, 65, 8) == "mid"
    assert mlt.qr_kernel(256, 64, 8, "complete") == "mid"


# ---------------------------------------------------------------------------
# The torch binding (python-torch/tests/test_torch.py of the reference)
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("lead", [(), (3,), (2, 3)])
@pytest.mark.parametrize("shape", [(8, 8), (40, 24), (24, 40)])
def test_binding_shapes_and_lead_dims(lead, shape):
    a = torch.randn(*lead, *shape, device="cuda")
    q, r = mlt.qr(a)
    k = min(shape)
    assert q.shape == (*lead, shape[0], k) and r.shape == (*lead, k, shape[1])
    assert q.device == a.device and q.dtype == torch.float32
    assert torch.count_nonzero(torch.tril(r, -1)).item() == 0
    assert (q @ r - a).abs().max().item() < 2e-5 * max(1.0, a.abs().max().item()) * shape[1]
    res = mlt.qr(a)
    assert type(res).__name__ == "linalg_qr" and torch.equal(res.Q, q)


def test_binding_dtypes_and_views():
    a64 = torch.randn(4, 20, 20, device="cuda", dtype=torch.float64)
    q, r = mlt.qr(a64)
    assert q.dtype == torch.float32
    assert (q.double() @ r.double() - a64).abs().max().item() < 1e-4
    ai = torch.arange(12, device="cuda").reshape(3, 4) % 5
    q, r = mlt.qr(ai)
    assert (q @ r - ai.float()).abs().max().item() < 1e-5
    base = torch.randn(6, 30, 50, device="cuda")
    view = base[::2, :, ::2].mT                    # non-contiguous
    q, r = mlt.qr(view)
    assert (q @ r - view).abs().max().item() < 1e-4
    qh, rh = mlt.qr(base[0].cpu())                 # a CPU tensor is staged through the GPU
    assert qh.device.type == "cpu" and (qh @ rh - base[0].cpu()).abs().max().item() < 1e-4


def test_binding_outputs_usable_at_once_on_the_stream():
    a = torch.randn(256, 32, 32, device="cuda")
    q, r = mlt.qr(a)
    err = (q @ r - a).abs().max()                  # enqueued behind the QR on the same stream, no sync
    assert err.item() < 1e-4


@pytest.mark.parametrize("shape,mode", [((3, 10, 6), "reduced"), ((3, 6, 6), "complete"), ((2, 5, 9), "reduced"),
                                        ((3, 10, 6), "r")])
def test_binding_gradients_match_torch(shape, mode):
    torch.manual_seed(3)
    b, m, n = shape
    a = torch.randn(*shape, device="cuda", dtype=torch.float32)
    w0 = torch.randn(b, m, n, device="cuda", dtype=torch.float64)
    w1 = torch.randn(b, m, m, device="cuda", dtype=torch.float64)
    w2 = torch.randn(b, n, n, device="cuda", dtype=torch.float64)

    def loss(q, r):
        # invariant to the sign freedom of QR: R^T R, Q R and the projector Q Q^T
        out = ((r.mT @ r).double() * w2).sum()
        if mode != "r":
            out = out + ((q @ r).double() * w0).sum() + ((q @ q.mT).double() * w1).sum()
        return out

    x = a.clone().requires_grad_(True)
    q, r = mlt.qr(x, mode)
    loss(q, r).backward()
    y = a.double().clone().requires_grad_(True)
    q2, r2 = torch.linalg.qr(y, mode="reduced" if mode == "r" else mode)
    loss(q2, r2).backward()
    assert (x.grad.double() - y.grad).abs().max().item() <= 2e-4 * max(1.0, y.grad.abs().max().item())


def test_binding_opcheck_and_compile():
    a = torch.randn(3, 12, 8, device="cuda")
    torch.library.opcheck(torch.ops.metal_linalg.qr, (a, "reduced"),
                          test_utils=("test_schema", "test_faketensor"))

    @torch.compile(backend="aot_eager", fullgraph=True)
    def f(x):
        q, r = mlt.qr(x)
        return q @ r

    assert (f(a) - a).abs().max().item() < 1e-4


def test_binding_threads():
    import threading
    a = torch.randn(128, 32, 32, device="cuda")
    q0, r0 = mlt.qr(a)
    torch.cuda.synchronize()
    errors = []

    def work():
        try:
            for _ in range(5):
                q, r = mlt.qr(a)
                torch.cuda.synchronize()
                if not (torch.equal(q, q0) and torch.equal(r, r0)):
                    errors.append("mismatch")
        except Exception as e:   # pragma: no cover
            errors.append(repr(e))

    threads = [threading.Thread(target=work) for _ in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_interop_cuda_array_interface_and_dlpack():
    """The C ABI through __cuda_array_interface__ (caller's buffers, the arrays' stream) and DLPack."""
    rng = np.random.default_rng(23)
    a = rng.standard_normal((6, 40, 24)).astype(np.float32)
    t = torch.as_tensor(a).cuda()
    for mode in ("reduced", "complete", "r"):
        qs, rs = mlt.qr_shapes(t.shape, mode)
        q = None if qs is None else torch.empty(qs, device="cuda")
        r = torch.empty(rs, device="cuda")
        mlt.qr_into(t, q, r, mode=mode)
        torch.cuda.synchronize()
        _, r_ref = harness.oracle_qr(a, mode)
        check(a, None if q is None else q.cpu().numpy(), r.cpu().numpy(), mode, r_ref)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        q, r = torch.empty(6, 40, 24, device="cuda"), torch.empty(6, 24, 24, device="cuda")
        mlt.qr_into(t, q, r, stream=side.cuda_stream)
    side.synchronize()
    check(a, q.cpu().numpy(), r.cpu().numpy(), "reduced")
    _lib.lib.metal_linalg_set_stream(None)
    Q, R = mlt.qr_dlpack(t)
    torch.cuda.synchronize()
    check(a, Q.cpu().numpy(), R.cpu().numpy(), "reduced")


# ---------------------------------------------------------------------------
# Failures that surface, memory that can be given back, a second GPU in one process
# ---------------------------------------------------------------------------

def test_kernel_that_gives_up_surfaces_as_runtime_error():
    """A kernel that gives up on a bounded wait writes NaN, which alone cannot be told from a NaN in the
    input; metal_linalg_synchronize (device pointers) and the call's own status (host pointers) report
    it as RUNTIME_ERROR with the shape (reference: src/qr_householder.mm:372-377, src/c_api.cpp:17-35).
    The failure is injected on the host: the blocked QR starts with its give-up word already set, so
    its tensor-core products return at once. No GPU waits or faults."""
    lib = _lib.lib
    a = torch.randn(1, 600, 600, device="cuda")
    q0, r0 = gpu_qr(a.cpu().numpy(), kernel="blocked")
    assert lib.metal_linalg_synchronize() == _lib.OK
    lib.metal_linalg_inject_wait_failures(1)
    q, r = gpu_qr(a.cpu().numpy(), kernel="blocked")               # device pointers: the call itself cannot know yet
    assert np.isnan(q).all() and np.isnan(r).all()
    assert lib.metal_linalg_synchronize() == _lib.RUNTIME_ERROR
    message = _lib.last_error()
    assert "gave up" in message and "600 x 600" in message and "tensor-core" in message
    assert lib.metal_linalg_synchronize() == _lib.OK               # reported once
    q1, r1 = gpu_qr(a.cpu().numpy(), kernel="blocked")             # and the next call is sound
    assert np.array_equal(q1, q0) and np.array_equal(r1, r0)
    # host pointers: the call waits for its results, so its own status carries the failure
    host = a.cpu().numpy()
    hq, hr = np.zeros_like(host), np.zeros_like(host)
    os.environ["QR_KERNEL"] = "blocked"
    try:
        lib.metal_linalg_inject_wait_failures(1)
        status = lib.metal_linalg_qr(host.ctypes.data, 1, 600, 600, hq.ctypes.data, hr.ctypes.data)
        assert status == _lib.RUNTIME_ERROR and "gave up" in _lib.last_error()
        assert np.isnan(hq).all() and np.isnan(hr).all()
        assert lib.metal_linalg_qr(host.ctypes.data, 1, 600, 600, hq.ctypes.data, hr.ctypes.data) == _lib.OK
    finally:
        os.environ.pop("QR_KERNEL", None)
        lib.metal_linalg_inject_wait_failures(0)
    assert np.array_equal(hr, r0[0:1]) or harness.r_parity(hr, r0) <= 1e-6


def test_release_workspaces_gives_memory_back():
    a = torch.randn(1, 3000, 3000, device="cuda")
    q, r = mlt.qr(a)                                   # the blocked QR: a workspace of a few hundred MB
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    freed = _lib.release_workspaces()
    free_after, _ = torch.cuda.mem_get_info()
    assert freed >= 3000 * 3000 * 4 * 2
    assert free_after - free_before >= freed // 2      # the driver hands back whole blocks
    assert _lib.release_workspaces() == 0
    q2, r2 = mlt.qr(a)                                 # allocates again
    torch.cuda.synchronize()
    assert torch.equal(q2, q) and torch.equal(r2, r)


@pytest.mark.parametrize("shape", [(3, 1833, 1), (2, 3000, 2), (1, 2500, 15)])
def test_complete_q_of_a_few_columns(shape):
    """A complete Q of thousands of rows from one to a few columns. The bound on orthogonality, 10 n eps, is a few ulps
    here, and an m x m float32 matrix cannot keep it beyond about a thousand rows whatever the algorithm (the exact Q
    of 1833 x 1 rounded to float32: 1.5e-6 against 1.2e-6; the reference's CPU path: 1.5e-6): the kernels are held to
    the bound or to the reference's own figure on the same input plus a tenth, whichever is larger."""
    b, m, n = shape
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal((b, m, n)).astype(np.float32)
    q, r = gpu_qr(a, "complete")
    assert mlt.qr_kernel(m, n, b, "complete") == "blocked"
    q_ref, r_ref = harness.oracle_qr(a, "complete")
    tol = workloads.tolerance(n)
    eye = np.eye(m)
    for k in range(b):
        q64, ref64 = q[k].astype(np.float64), q_ref[k].astype(np.float64)
        orth, orth_ref = np.linalg.norm(q64.T @ q64 - eye), np.linalg.norm(ref64.T @ ref64 - eye)
        assert orth <= max(tol, 1.1 * orth_ref), (orth, orth_ref, tol)
        a64 = a[k].astype(np.float64)
        assert np.linalg.norm(a64 - q64 @ r[k].astype(np.float64)) / np.linalg.norm(a64) <= tol
    assert harness.r_parity(r, r_ref) <= 1e-4


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_second_gpu_in_one_process():
    """Every kernel family on cuda:1 after cuda:0 in ONE process (kernels that opt into more than 48 KB
    of shared memory do so per GPU): same bits as on cuda:0. `qr_sharded` is that path."""
    torch.manual_seed(31)
    cases = [(torch.randn(300, 32, 32), "reduced"), (torch.randn(100, 16, 16), "reduced"),
             (torch.randn(6, 256, 200), "complete"), (torch.randn(2, 5000, 64), "reduced"),
             (torch.randn(1, 1500, 1200), "reduced"), (torch.randn(1, 2100, 300), "r"),
             (torch.randn(4, 450, 300), "reduced"), (torch.randn(1, 3000, 160), "reduced")]
    for a, mode in cases:
        (q0, r0), (q1, r1) = mlt.qr_sharded([a.to("cuda:0"), a.to("cuda:1")], mode)
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        assert r1.device.index == 1
        assert torch.equal(r0.cpu(), r1.cpu()), (tuple(a.shape), mode)
        assert torch.equal(q0.cpu(), q1.cpu()), (tuple(a.shape), mode)
    a = torch.randn(8, 300, 12)
    u0, s0, v0 = mlt.svd(a.to("cuda:0"))
    u1, s1, v1 = mlt.svd(a.to("cuda:1"))
    assert torch.equal(s0.cpu(), s1.cpu()) and torch.equal(u0.cpu(), u1.cpu())
    big = torch.randn(4, 400, 128)                     # the block Jacobi and the wide left-vector kernel
    s0, s1 = mlt.svd(big.to("cuda:0")).S, mlt.svd(big.to("cuda:1")).S
    assert torch.equal(s0.cpu(), s1.cpu())


@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
@pytest.mark.parametrize("shape", [(128, 1024), (64, 2048), (48, 100), (33, 65), (200, 1000), (16, 64)])
def test_wide_by_leading_block(shape, mode):
    """A wide matrix is factored by its leading square block and R's other columns come from one product
    (the reference's CPU path: src/qr_cpu.mm:6-9,112-118): the same factorisation as the general kernels
    give on the whole matrix (QR_WIDE=0), and the oracle's R. A NaN right of the leading block still makes
    the whole matrix's outputs NaN."""
    m, n = shape
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal((5, m, n)).astype(np.float32)
    a[3, m - 1, n - 1] = np.nan
    a[4] *= 1e-30
    good = [0, 1, 2, 4]
    q, r = gpu_qr(a, mode)
    assert np.isnan(r[3]).all() and (q is None or np.isnan(q[3]).all())
    _, r_ref = harness.oracle_qr(a[good], mode)
    check(a[good], None if q is None else q[good], r[good], mode, r_ref)
    os.environ["QR_WIDE"] = "0"
    try:
        q0, r0 = gpu_qr(a, mode)
    finally:
        os.environ.pop("QR_WIDE", None)
    assert harness.r_parity(r[good], r0[good]) <= 1e-5


@pytest.mark.parametrize("kernel,shape", [("mid", (300, 96)), ("mid", (256, 64)), ("blocked", (1500, 160)), ("blocked", (3000, 64))])
def test_panel_pairs_with_nearly_parallel_columns(kernel, shape):
    """Panels take two columns a reduction and form the second reflector from sums taken before the first was
    applied; where a column is nearly parallel to the one before it that formula would lose digits, and the
    pair falls back to two ordinary steps. Columns that repeat, or differ by 1e-3 ... 1e-7, or vanish, exercise
    both sides of that decision: orthogonality, reconstruction and R against the oracle must hold as everywhere."""
    m, n = shape
    rng = np.random.default_rng(m * 3 + n)
    base = rng.standard_normal((m, n)).astype(np.float64)
    mats = []
    for eps in (0.0, 1e-7, 1e-5, 1e-3, 0.3):
        x = base.copy()
        x[:, 1::2] = x[:, 0::2][:, : x[:, 1::2].shape[1]] + eps * rng.standard_normal(x[:, 1::2].shape)   # odd columns ~ the even ones
        mats.append(x)
    x = base.copy()
    x[:, 5:9] = 0.0                                  # zero columns: identity reflectors inside pairs
    mats.append(x)
    a = np.stack(mats).astype(np.float32)
    q, r = gpu_qr(a, "reduced", kernel=kernel)
    check(a, q, r, "reduced")
    _, r_ref = harness.oracle_qr(a[[3, 4]])
    assert harness.r_parity(r[[4]], r_ref[[1]]) <= 1e-4          # well conditioned: the usual bound
    assert harness.r_parity(r[[3]], r_ref[[0]]) <= 2e-3          # column pairs 1e-3 apart: R is determined to about 1e3 eps


@pytest.mark.parametrize("shape", [(1500, 160), (3000, 64), (600, 96)])
def test_panel_quads_with_nearly_dependent_columns(shape):
    """The blocked QR's cluster panels take four columns a reduction: every step of a group is formed from sums taken
    before the group's first step, and a column whose tail the group's earlier steps have nearly removed leaves the
    group for single steps. Columns that copy an earlier column of their group (the third the first, the fourth the
    second, all four the same) to 0 ... 0.3, and zero columns inside a group, exercise the first, second and third
    step's guard."""
    m, n = shape
    rng = np.random.default_rng(m + 7 * n)
    base = rng.standard_normal((m, n)).astype(np.float64)
    mats = []
    for eps in (0.0, 1e-6, 1e-3, 0.3):
        for src, dst in ((0, 2), (1, 3), (0, 1)):
            x = base.copy()
            cols = x[:, dst::4].shape[1]
            x[:, dst::4] = x[:, src::4][:, :cols] + eps * rng.standard_normal((m, cols))
            mats.append(x)
        x = base.copy()
        for d in (1, 2, 3):
            cols = x[:, d::4].shape[1]
            x[:, d::4] = x[:, 0::4][:, :cols] + eps * rng.standard_normal((m, cols))
        mats.append(x)
    x = base.copy()
    x[:, 9:11] = 0.0
    x[:, 20:24] = 0.0
    mats.append(x)
    a = np.stack(mats).astype(np.float32)
    q, r = gpu_qr(a, "reduced", kernel="blocked")
    check(a, q, r, "reduced")
    well = [12, 13, 14, 15]                                      # the groups 0.3 apart: the usual bound on R
    _, r_ref = harness.oracle_qr(a[well])
    assert harness.r_parity(r[well], r_ref) <= 1e-4
    os.environ["QR_PANEL_QUADS"] = "0"
    try:
        q2, r2 = gpu_qr(a[well], "reduced", kernel="blocked")
    finally:
        os.environ.pop("QR_PANEL_QUADS", None)
    assert harness.r_parity(r[well], r2) <= 1e-4
