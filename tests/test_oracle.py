"""The CPU oracle (oracle/qr_oracle.c) against the committed outputs of the
reference's own CPU QR (tests/golden/qr_golden.npz, made by make_golden.py) and,
where oracle/_ref was built, against that library directly. No GPU."""
import os
import sys

import numpy as np
import pytest

import harness
from metal_linalg_torch import workloads

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qr_golden.npz"))
CASES = [(name, mode) for name, (_, modes) in make_golden.CASES.items() for mode in modes]


@pytest.mark.parametrize("name,mode", CASES)
def test_oracle_matches_reference_fixtures(name, mode):
    a = make_golden.case_input(name)
    q, r = harness.oracle_qr(a, mode)
    r_ref = GOLDEN[f"{name}/{mode}/r"]
    assert r.shape == r_ref.shape
    # R to 1e-4 relative after sign normalisation (the same LAPACK signs, so also without it)
    assert harness.r_parity(r, r_ref) <= 1e-4
    n = a.shape[-1]
    if mode != "r":
        q_ref = GOLDEN[f"{name}/{mode}/q"]
        assert q.shape == q_ref.shape
        recon, orth, low = harness.metrics(a, q, r)
        tol = workloads.tolerance(n)
        assert recon.max() <= tol and orth.max() <= tol and low.max() == 0.0
        # the reference's own outputs meet the same bounds (the fixture is sound)
        recon, orth, low = harness.metrics(a, q_ref, r_ref)
        assert recon.max() <= tol and orth.max() <= tol and low.max() == 0.0
        if name not in ("c3_256x256_rank224", "doc_3x3"):   # full rank: Q is unique up to signs
            qn, _ = harness.sign_normalise(q, r)
            qrn, _ = harness.sign_normalise(q_ref, r_ref)
            k = min(a.shape[-2:])
            assert np.abs(qn[..., :k] - qrn[..., :k]).max() <= 1e-4


def test_capi_known_answers():
    """tests/test_c_api.c:29-81 of the reference: QR reproduces A, R upper triangular,
    R alone equals the reduced R, complete Q orthogonal with the reduced Q first."""
    a = make_golden.case_input("capi_3x2")
    q, r = harness.oracle_qr(a, "reduced")
    assert r[0, 1, 0] == 0.0 and r[1, 1, 0] == 0.0
    assert np.allclose(q @ r, a, rtol=1e-5, atol=1e-5)
    _, r_alone = harness.oracle_qr(a, "r")
    assert np.array_equal(r_alone, r)
    qc, rc = harness.oracle_qr(a, "complete")
    assert np.all(rc[:, 2, :] == 0.0)
    assert np.allclose(np.swapaxes(qc, -1, -2) @ qc, np.eye(3), atol=1e-5)
    assert np.allclose(qc[:, :, :2], q, atol=1e-5)
    # LAPACK's sign: the first diagonal entry is -||a_1||
    assert np.allclose(r[:, 0, 0], -np.linalg.norm(a[:, :, 0], axis=1), rtol=1e-6)


def test_doc_example_rank_two():
    """docs/qr.md:77-88 of the reference: [[1,2,3],[4,5,6],[7,8,9]] has rank 2, so R[2,2] ~ 0."""
    a = make_golden.case_input("doc_3x3")
    q, r = harness.oracle_qr(a)
    assert abs(r[0, 2, 2]) < 1e-5
    assert np.allclose(q @ r, a, atol=1e-5)
    assert np.allclose(np.abs(r[0, 0, 0]), np.sqrt(66.0), rtol=1e-6)


def test_nonfinite_matrix_is_isolated():
    """src/qr_cpu.mm:61-76: a NaN or an infinity gives NaN for that matrix alone."""
    rng = np.random.default_rng(1)
    a = rng.standard_normal((3, 6, 4)).astype(np.float32)
    a[1, 2, 3] = np.inf
    q, r = harness.oracle_qr(a, "complete")
    assert np.isnan(q[1]).all() and np.isnan(r[1]).all()
    assert np.isfinite(q[[0, 2]]).all() and np.isfinite(r[[0, 2]]).all()


@pytest.mark.skipif(harness.load_ref() is None, reason="oracle/_ref needs the reference checkout")
@pytest.mark.parametrize("shape", [(5, 1, 1), (4, 7, 7), (3, 33, 20), (2, 20, 33), (2, 130, 64), (1, 300, 300)])
@pytest.mark.parametrize("mode", ["reduced", "complete", "r"])
def test_oracle_matches_live_reference(shape, mode):
    rng = np.random.default_rng(shape[1] * 1000 + shape[2])
    a = rng.standard_normal(shape).astype(np.float32)
    q, r = harness.oracle_qr(a, mode)
    q_ref, r_ref = harness.ref_qr(a, mode)
    assert harness.r_parity(r, r_ref) <= 1e-4
    if q is not None:
        qn, _ = harness.sign_normalise(q, r)
        qrn, _ = harness.sign_normalise(q_ref, r_ref)
        k = min(shape[1:])
        assert np.abs(qn[..., :k] - qrn[..., :k]).max() <= 2e-4


def test_magnitudes_and_scale_invariance():
    """Scaling a matrix by a power of two scales R exactly and leaves Q alone."""
    rng = np.random.default_rng(3)
    a = rng.standard_normal((2, 12, 12)).astype(np.float32)
    q0, r0 = harness.oracle_qr(a)
    for e in (-100, -40, 60, 100):
        s = np.float32(2.0) ** e
        q, r = harness.oracle_qr(a * s)
        assert np.array_equal(q, q0)
        assert np.array_equal(r, r0 * s)
