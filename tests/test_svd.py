"""The SVD that calls the QR (the QR-preconditioned Jacobi route): the CPU restatement pinned against the
reference's known-answer case and LAPACK's singular values, the C ABI's argument checks, the autograd formula
(all without a GPU), and the parity of the CUDA path with the restatement through the C ABI on a B200.

Tolerances are the reference's own (tests/test_svd.cpp:41-43,156-175): ||A - U S Vt||_F / ||A||_F <= 2e-5,
||U^T U - I||_F / sqrt(K) and the same for Vt <= 2e-5 max(1, sqrt(max(M, N) / 256)), |S - S_lapack| / ||A||_F <= 2e-5.
Beyond K = 64 the bounds on reconstruction and orthogonality grow as sqrt(K / 64): plain one-sided Jacobi in float32
applies about K rotations a sweep to every column of V, each entry's rounding error grows as sqrt(K sweeps) and the
Frobenius norm over K^2 entries, divided by sqrt(K), as sqrt(K) times that (the float32 restatement itself shows
2.2e-5 at K = 128; the reference sends such K to its block Jacobi backend, which is not built here).
"""
import os
import sys

import numpy as np
import pytest
import torch

import harness
import metal_linalg_torch as mlt
from metal_linalg_torch import _lib, _ops

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_svd_golden  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "svd_golden.npz"))
RECON_TOL = ORTHO_TOL = SVAL_TOL = 2e-5


def check_svd(a, u, s, vt, s_ref=None, slack=1.0):
    """`slack` scales the tolerances for matrices whose rounding exceeds them (graded over five decades), as the
    reference's own check does (tests/test_svd.cpp:94-98,173-175)."""
    a = np.asarray(a, np.float32)
    *lead, m, n = a.shape
    k = min(m, n)
    assert s.shape == (*lead, k)
    assert np.isfinite(s).all() and (s >= 0).all()
    assert (np.diff(s, axis=-1) <= 0).all(), "singular values are not descending"
    fro = np.linalg.norm(a.astype(np.float64), axis=(-2, -1))
    if s_ref is not None:
        err = np.abs(s.astype(np.float64) - s_ref).max(axis=-1) / np.maximum(fro, 1e-300)
        assert err.max() <= slack * SVAL_TOL, f"|S - S_lapack| / ||A|| = {err.max():.2e}"
    if u is None:
        return
    assert u.shape == (*lead, m, k) and vt.shape == (*lead, k, n)
    rec, ou, ov = harness.svd_metrics(a, u, s, vt)
    slack = slack * max(1.0, np.sqrt(k / 64.0))
    tol_o = slack * ORTHO_TOL * max(1.0, np.sqrt(max(m, n) / 256.0))
    assert rec.max() <= slack * RECON_TOL, f"reconstruction {rec.max():.2e}"
    assert (ou / np.sqrt(k)).max() <= tol_o, f"U orthogonality {(ou / np.sqrt(k)).max():.2e}"
    assert (ov / np.sqrt(k)).max() <= tol_o, f"Vt orthogonality {(ov / np.sqrt(k)).max():.2e}"


# ---------------------------------------------------------------------------
# Without a GPU: the restatement, the boundary, the gradient
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(make_svd_golden.CASES))
def test_oracle_matches_lapack_fixtures(name):
    a = make_svd_golden.CASES[name]()
    u, s, vt, info = harness.oracle_svd(a)
    check_svd(a, u, s, vt, s_ref=GOLDEN[f"{name}/s64"], slack=2.0 if name.startswith("graded") else 1.0)
    fro = np.linalg.norm(a.astype(np.float64), axis=(-2, -1))
    assert (np.abs(s - GOLDEN[f"{name}/s32"]).max(axis=-1) / fro).max() <= SVAL_TOL      # the reference's CPU path: sgesdd
    assert ((info >> 16) & 1).all(), "not converged"
    _, s_only, _, _ = harness.oracle_svd(a, vectors=False)
    assert np.array_equal(s_only, s)


def test_oracle_known_answer():
    """tests/test_c_api.c:97-111 of the reference: s = (3, 2), U S Vt = A, converged."""
    a = make_svd_golden.CASES["capi_2x3"]()
    u, s, vt, info = harness.oracle_svd(a)
    assert np.allclose(s, [[3.0, 2.0]], atol=1e-6)
    assert np.allclose((u * s[..., None, :]) @ vt, a, atol=1e-5)
    assert (info[0] >> 16) & 1 and (info[0] & 0xFFFF) >= 1


def test_oracle_rank_deficient_zero_and_nonfinite():
    a = make_svd_golden.CASES["rank3_40x8"]()
    u, s, vt, info = harness.oracle_svd(a)
    assert ((info >> 18) & 1).all() and ((info >> 16) & 1).all()
    assert (s[:, 3:] <= 1e-5 * s[:, :1]).all()
    a5 = make_svd_golden.CASES["rank5_200x48"]()
    u5, s5, vt5, info5 = harness.oracle_svd(a5)
    assert ((info5 >> 18) & 1).all() and (s5[:, 5:] <= 1e-5 * s5[:, :1]).all()
    check_svd(a5, u5, s5, vt5)
    check_svd(a, u, s, vt)                       # the null columns were completed to an orthonormal basis
    z = np.zeros((1, 6, 4), np.float32)
    u, s, vt, info = harness.oracle_svd(z)
    assert (s == 0).all() and (info[0] >> 18) & 1
    check_svd(z, u, s, vt)
    b = np.random.default_rng(3).standard_normal((3, 9, 5)).astype(np.float32)
    b[1, 2, 3] = np.nan
    u, s, vt, info = harness.oracle_svd(b)
    assert np.isnan(s[1]).all() and np.isnan(u[1]).all() and np.isnan(vt[1]).all() and (info[1] >> 17) & 1
    check_svd(b[[0, 2]], u[[0, 2]], s[[0, 2]], vt[[0, 2]])


@pytest.mark.parametrize("scale", [1e-30, 1e20, 1e37])
def test_oracle_scale_invariance(scale):
    a = np.random.default_rng(5).standard_normal((2, 60, 10)).astype(np.float32)
    _, s1, _, _ = harness.oracle_svd(a, vectors=False)
    big = (a.astype(np.float64) * scale / np.abs(a).max()).astype(np.float32)
    u, s, vt, info = harness.oracle_svd(big)
    ratio = float(np.float64(scale) / np.abs(a).max())
    assert np.allclose(s / ratio, s1, rtol=2e-5, atol=0)
    check_svd(big, u, s, vt)


def test_svd_argument_errors_need_no_gpu():
    lib = _lib.lib
    a = np.eye(2, dtype=np.float32)
    u, s = np.zeros(4, np.float32), np.zeros(2, np.float32)
    # tests/test_c_api.c:204 of the reference: u without vt
    assert lib.metal_linalg_svd(a.ctypes.data, 1, 2, 2, u.ctypes.data, s.ctypes.data, None, None) == _lib.INVALID_ARGUMENT
    assert "u and vt" in _lib.last_error()
    assert lib.metal_linalg_svd(None, 1, 2, 2, None, s.ctypes.data, None, None) == _lib.INVALID_ARGUMENT
    assert lib.metal_linalg_svd(a.ctypes.data, 1, 2, 2, None, None, None, None) == _lib.INVALID_ARGUMENT
    assert lib.metal_linalg_svd(None, 0, 2, 2, None, None, None, None) == _lib.OK          # an empty batch
    big = np.zeros((1, 130, 130), np.float32)
    sb = np.zeros(130, np.float32)
    assert lib.metal_linalg_svd(big.ctypes.data, 1, 130, 130, None, sb.ctypes.data, None, None) == _lib.INVALID_ARGUMENT
    assert "min(M, N)" in _lib.last_error()
    assert mlt.svd_backend(5000, 32) == "qr_jacobi" and mlt.svdvals_backend(32, 5000, 9) == "qr_jacobi"
    assert mlt.svd_backend(64, 33) == "qr_jacobi" and mlt.svd_backend(129, 4000) == "unavailable"
    with pytest.raises(NotImplementedError):
        mlt.svd(torch.zeros(2, 3, 3), full_matrices=True)
    with pytest.raises(ValueError):
        mlt.svd(torch.zeros(2, 140, 140))


@pytest.mark.parametrize("shape", [(3, 7, 4), (2, 4, 9), (2, 5, 5)])
def test_svd_grad_matches_torch(shape):
    """The autograd formula against torch.linalg.svd's on a loss that does not depend on the vectors' signs."""
    torch.manual_seed(0)
    a = torch.randn(*shape, dtype=torch.float64, requires_grad=True)
    U, S, Vh = torch.linalg.svd(a, full_matrices=False)
    G = torch.randn_like(a)
    w = torch.randn(shape[0], 1, S.shape[-1], dtype=torch.float64)
    gS = torch.randn_like(S)
    loss = (gS * S).sum() + (((U * w) @ Vh) * G).sum()
    (expected,) = torch.autograd.grad(loss, a)
    gU, gVh = (G @ Vh.mT) * w, (U * w).mT @ G
    mine = _ops.svd_grad(U.detach(), S.detach(), Vh.detach(), gU.detach(), gS, gVh.detach())
    assert (mine - expected).abs().max() < 1e-10
    only_s = _ops.svd_grad(U.detach(), S.detach(), Vh.detach(), None, gS, None)
    (expected_s,) = torch.autograd.grad((gS * torch.linalg.svdvals(a)).sum(), a)
    assert (only_s - expected_s).abs().max() < 1e-10


def test_fake_shapes():
    a = torch.empty(3, 2, 50, 7, device="meta")
    u, s, vt = torch.ops.metal_linalg.svd(a)
    assert u.shape == (3, 2, 50, 7) and s.shape == (3, 2, 7) and vt.shape == (3, 2, 7, 7)
    assert torch.ops.metal_linalg.svdvals(torch.empty(4, 5, 90, device="meta")).shape == (4, 5)


# ---------------------------------------------------------------------------
# On the GPU: parity with the restatement, through the C ABI
# ---------------------------------------------------------------------------

def gpu_svd(a, vectors=True):
    """numpy in, numpy out, through the C ABI on device pointers; info too."""
    t = torch.as_tensor(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    *lead, m, n = t.shape
    k = min(m, n)
    batch = int(np.prod(lead)) if lead else 1
    s = torch.empty(*lead, k, device="cuda")
    info = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda")
    u = torch.empty(*lead, m, k, device="cuda") if vectors else None
    vt = torch.empty(*lead, k, n, device="cuda") if vectors else None
    _lib.svd(t.data_ptr(), batch, m, n, u.data_ptr() if vectors else None, s.data_ptr(),
             vt.data_ptr() if vectors else None, info.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    out_info = info.cpu().numpy().astype(np.uint32).reshape(lead if lead else (1,))
    return (u.cpu().numpy() if vectors else None), s.cpu().numpy(), (vt.cpu().numpy() if vectors else None), out_info


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(make_svd_golden.CASES))
def test_gpu_matches_fixtures_and_oracle(name):
    a = make_svd_golden.CASES[name]()
    u, s, vt, info = gpu_svd(a)
    check_svd(a, u, s, vt, s_ref=GOLDEN[f"{name}/s64"], slack=2.0 if name.startswith("graded") else 1.0)
    _, s_o, _, info_o = harness.oracle_svd(a)
    fro = np.linalg.norm(a.astype(np.float64), axis=(-2, -1))
    assert (np.abs(s - s_o).max(axis=-1) / fro).max() <= SVAL_TOL
    assert ((info >> 16) & 1).all()
    assert np.array_equal(info >> 17, info_o >> 17)                     # non-finite and rank-deficient flags
    _, s_only, _, info_v = gpu_svd(a, vectors=False)
    assert (np.abs(s_only - s).max(axis=-1) / fro).max() <= 1e-6      # tests/test_svd.cpp:585 of the reference
    assert ((info_v >> 16) & 1).all()


SHAPES = [(1, 1), (1, 9), (9, 1), (2, 2), (3, 2), (2, 3), (4, 4), (5, 5), (8, 8), (9, 9), (16, 16), (17, 17), (31, 31),
          (32, 32), (33, 32), (32, 33), (100, 3), (3, 100), (257, 8), (1000, 16), (1025, 32), (20000, 20), (24, 3000),
          (70000, 32), (33, 33), (40, 64), (64, 64), (65, 65), (100, 100), (127, 127), (128, 128), (500, 33), (2000, 96),
          (128, 9000), (65536, 64)]


@pytest.mark.gpu
@pytest.mark.parametrize("shape", SHAPES)
def test_gpu_shapes(shape):
    m, n = shape
    batch = 3 if max(m, n) > 2000 else 37 if min(m, n) <= 32 else 5
    a = np.random.default_rng(m * 131 + n).standard_normal((batch, m, n)).astype(np.float32)
    u, s, vt, info = gpu_svd(a)
    s_ref = np.linalg.svd(a.astype(np.float64), compute_uv=False)
    check_svd(a, u, s, vt, s_ref=s_ref)
    assert ((info >> 16) & 1).all() and not ((info >> 17) & 3).any()
    _, s_only, _, _ = gpu_svd(a, vectors=False)
    check_svd(a, None, s_only, None, s_ref=s_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["rank3_40x8", "rank5_200x48"])
def test_gpu_rank_deficient_zero_nonfinite_and_isolation(name):
    a = make_svd_golden.CASES[name]()
    m, n = a.shape[-2:]
    a = np.concatenate([a, np.zeros((1, m, n), np.float32), np.random.default_rng(9).standard_normal((2, m, n)).astype(np.float32)])
    a[3, 5, 5] = np.inf
    u, s, vt, info = gpu_svd(a)
    assert ((info[[0, 1, 2]] >> 18) & 1).all() and not (info[4] >> 17) & 3
    assert (info[3] >> 17) & 1 and np.isnan(s[3]).all() and np.isnan(u[3]).all() and np.isnan(vt[3]).all()
    keep = [0, 1, 2, 4]
    check_svd(a[keep], u[keep], s[keep], vt[keep], s_ref=np.linalg.svd(a[keep].astype(np.float64), compute_uv=False))
    assert (s[2] == 0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("scale", [1e-30, 1e20, 1e37])
def test_gpu_magnitudes(scale):
    """tests/test_svd.cpp:327,589 of the reference: matrices scaled to the ends of float32's range."""
    a = np.random.default_rng(5).standard_normal((4, 800, 12)).astype(np.float32)
    big = (a.astype(np.float64) * scale / np.abs(a).max()).astype(np.float32)
    u, s, vt, info = gpu_svd(big)
    check_svd(big, u, s, vt, s_ref=np.linalg.svd(big.astype(np.float64), compute_uv=False))


@pytest.mark.gpu
def test_gpu_large_batch_and_binding():
    """A batch that fills the GPU, through the torch binding: result type, values against torch's own SVD,
    host tensors staged by the library, autograd through the custom operator."""
    torch.manual_seed(1)
    a = torch.randn(20000, 32, 16, device="cuda")
    out = mlt.svd(a)
    assert type(out).__name__ == "linalg_svd"
    U, S, Vh = out
    ref = torch.linalg.svdvals(a.double())
    assert ((S.double() - ref).abs().amax(-1) / torch.linalg.matrix_norm(a.double())).max() <= SVAL_TOL
    assert ((U * S.unsqueeze(-2)) @ Vh - a).norm() / a.norm() <= RECON_TOL
    assert (mlt.svdvals(a) - S).abs().max() <= 1e-5
    host = torch.randn(50, 300, 9)
    Uh, Sh, Vhh = mlt.svd(host)
    assert Uh.device.type == "cpu" and ((Uh * Sh.unsqueeze(-2)) @ Vhh - host).norm() / host.norm() <= RECON_TOL
    x = torch.randn(4, 30, 6, device="cuda", requires_grad=True)
    mlt.svdvals(x).sum().backward()                      # the nuclear norm: gradient U Vh
    Ux, _, Vx = torch.linalg.svd(x.detach().double(), full_matrices=False)
    assert (x.grad.double() - Ux @ Vx).abs().max() <= 1e-4


@pytest.mark.gpu
def test_gpu_qr_workspace_is_not_clobbered():
    """The SVD keeps its own scratch apart from the QR's: a QR between two SVDs on the same stream, and
    shapes that make the QR's workspace grow, leave the results intact."""
    rng = np.random.default_rng(11)
    a = rng.standard_normal((64, 3000, 24)).astype(np.float32)
    u0, s0, vt0, _ = gpu_svd(a)
    mlt.qr(torch.randn(2, 1500, 1500, device="cuda"))
    u1, s1, vt1, _ = gpu_svd(a)
    assert np.array_equal(s0, s1) and np.array_equal(u0, u1) and np.array_equal(vt0, vt1)
    check_svd(a, u1, s1, vt1, s_ref=np.linalg.svd(a.astype(np.float64), compute_uv=False))


@pytest.mark.gpu
def test_gpu_binding_opcheck_compile_and_threads():
    """The operators under torch.library.opcheck and torch.compile (full graph), and from several threads at once
    on their own streams (the library keeps stream and device per thread, the SVD's scratch per stream)."""
    import threading
    a = torch.randn(3, 40, 6, device="cuda")
    torch.library.opcheck(torch.ops.metal_linalg.svd, (a,), test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(torch.ops.metal_linalg.svdvals, (a,), test_utils=("test_schema", "test_faketensor"))

    @torch.compile(backend="aot_eager", fullgraph=True)
    def f(x):
        u, s, vh = mlt.svd(x)
        return (u * s.unsqueeze(-2)) @ vh, mlt.svdvals(x)

    rec, vals = f(a)
    assert (rec - a).abs().max().item() < 1e-4
    assert (vals.double() - torch.linalg.svdvals(a.double())).abs().max().item() < 1e-4

    b = torch.randn(512, 200, 24, device="cuda")
    ref = torch.linalg.svdvals(b.double())
    torch.cuda.synchronize()
    errors = []

    def work():
        try:
            with torch.cuda.stream(torch.cuda.Stream()):
                for _ in range(4):
                    s = mlt.svdvals(b)
                    u, s2, vh = mlt.svd(b)
                torch.cuda.current_stream().synchronize()
                if (s.double() - ref).abs().max().item() > 1e-3 or (s2 - s).abs().max().item() > 1e-4:
                    errors.append("values differ")
                if ((u * s2.unsqueeze(-2)) @ vh - b).norm().item() / b.norm().item() > RECON_TOL:
                    errors.append("reconstruction")
        except Exception as e:      # surfaced below
            errors.append(repr(e))

    threads = [threading.Thread(target=work) for _ in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
