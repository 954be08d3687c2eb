"""TEST INFRASTRUCTURE ONLY: ctypes loaders for the two CPU parity checkers and the
float64 checks the parity tests share. Imported by tests/, by the smoke check and
by the bench's CPU-baseline leg; never by the product package.

  oracle_qr(a, mode)     the plain-C restatement, oracle/libqr_oracle.so
  oracle_svd(a, vectors) the plain-C restatement of the QR-preconditioned Jacobi SVD, same library
  ref_qr(a, mode)        the reference's own src/qr_cpu.mm, oracle/_ref/libqr_cpu_ref.so
                         (None if that library was not built)

The checks restate the reference's own test metrics: tests/test_qr.cpp:76-111
(reconstruction, orthogonality, strict lower triangle), python-torch/tests/
test_torch.py:44-46,352-356 (rel = max|d| / max|ref| on R after removing the
sign freedom).
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
MODES = {"reduced": 0, "r": 1, "complete": 2}
EPS32 = 2.0 ** -23

_f32p = ctypes.POINTER(ctypes.c_float)


def build():
    """Compile the checkers (and oracle/_ref where the reference checkout exists)."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)


def _ptr(x):
    return x.ctypes.data_as(_f32p) if x is not None else None


def _shapes(a, mode):
    *lead, m, n = a.shape
    k = min(m, n)
    qc = {"reduced": k, "r": 0, "complete": m}[mode]
    rr = m if mode == "complete" else k
    return lead, m, n, qc, rr


_oracle = None
_ref = False


def _load_oracle():
    global _oracle
    if _oracle is None:
        path = os.path.join(HERE, "libqr_oracle.so")
        if not os.path.exists(path):
            build()
        lib = ctypes.CDLL(path)
        lib.oracle_qr.restype = ctypes.c_int
        lib.oracle_qr.argtypes = [_f32p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, _f32p, _f32p]
        _u32p = ctypes.POINTER(ctypes.c_uint32)
        lib.oracle_svd.restype = ctypes.c_int
        lib.oracle_svd.argtypes = [_f32p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, _f32p, _f32p, _f32p, _u32p]
        _oracle = lib
    return _oracle


def load_ref():
    """The reference's qr_cpu as a ctypes library, or None."""
    global _ref
    if _ref is False:
        path = os.path.join(HERE, "_ref", "libqr_cpu_ref.so")
        _ref = None
        if os.path.exists(path):
            try:
                lib = ctypes.CDLL(path)
                lib.ref_qr_cpu.restype = ctypes.c_int
                lib.ref_qr_cpu.argtypes = [_f32p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int,
                                           _f32p, _f32p, ctypes.c_uint]
                lib.ref_last_error.restype = ctypes.c_char_p
                lib.ref_lapack_config.restype = ctypes.c_char_p
                lib.ref_cpu_threads.restype = ctypes.c_uint
                _ref = lib
            except OSError:
                _ref = None
    return _ref


def _run(call, a, mode):
    a = np.ascontiguousarray(a, dtype=np.float32)
    lead, m, n, qc, rr = _shapes(a, mode)
    batch = int(np.prod(lead)) if lead else 1
    q = np.empty((*lead, m, qc), np.float32) if qc else None
    r = np.empty((*lead, rr, n), np.float32)
    call(_ptr(a), batch, m, n, MODES[mode], _ptr(q), _ptr(r))
    return q, r


def oracle_qr(a, mode="reduced"):
    lib = _load_oracle()

    def call(*args):
        if lib.oracle_qr(*args):
            raise MemoryError("oracle_qr")
    return _run(call, a, mode)


def oracle_svd(a, vectors=True):
    """(u, s, vt, info) of the thin SVD by the restatement; u and vt None without vectors."""
    lib = _load_oracle()
    a = np.ascontiguousarray(a, dtype=np.float32)
    *lead, m, n = a.shape
    k = min(m, n)
    batch = int(np.prod(lead)) if lead else 1
    s = np.empty((*lead, k), np.float32)
    info = np.zeros(tuple(lead) if lead else (1,), np.uint32)
    u = np.empty((*lead, m, k), np.float32) if vectors else None
    vt = np.empty((*lead, k, n), np.float32) if vectors else None
    if lib.oracle_svd(_ptr(a), batch, m, n, _ptr(u), _ptr(s), _ptr(vt),
                      info.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))):
        raise MemoryError("oracle_svd")
    return u, s, vt, info


def svd_metrics(a, u, s, vt):
    """Per matrix, in float64 on the unit-scale problem: ||A - U S Vt||_F / ||A||_F, ||U^T U - I||_F,
    ||Vt Vt^T - I||_F (the reference's checks: tests/test_svd.cpp reconstruction and orthogonality)."""
    a = np.asarray(a, np.float64)
    u, s, vt = np.asarray(u, np.float64), np.asarray(s, np.float64), np.asarray(vt, np.float64)
    scale = np.maximum(np.abs(a).max(axis=(-2, -1), keepdims=True), 1e-300)
    an = a / scale
    rec = np.linalg.norm(an - (u * (s / scale[..., 0])[..., None, :]) @ vt, axis=(-2, -1)) / \
        np.maximum(np.linalg.norm(an, axis=(-2, -1)), 1e-300)
    k = s.shape[-1]
    eye = np.eye(k)
    ou = np.linalg.norm(np.swapaxes(u, -1, -2) @ u - eye, axis=(-2, -1))
    ov = np.linalg.norm(vt @ np.swapaxes(vt, -1, -2) - eye, axis=(-2, -1))
    return rec, ou, ov


def ref_qr(a, mode="reduced", threads=0):
    lib = load_ref()
    if lib is None:
        return None

    def call(*args):
        if lib.ref_qr_cpu(*args, threads):
            raise RuntimeError(lib.ref_last_error().decode())
    return _run(call, a, mode)


# ---------------------------------------------------------------------------
# Checks, in float64
# ---------------------------------------------------------------------------

def unit_scale(a):
    """Per-matrix power of two 2^e with max|A| / 2^e in [0.5, 1) (1 for a zero matrix)."""
    amax = np.abs(a.astype(np.float64)).max(axis=(-2, -1))
    e = np.where(amax > 0, np.floor(np.log2(np.where(amax > 0, amax, 1.0))) + 1, 0.0)
    return np.exp2(e)[..., None, None]


def metrics(a, q, r):
    """Per matrix, on the unit-scale problem: ||A - QR||_F / ||A||_F, ||Q^T Q - I||_F,
    max |strict lower triangle of R| (exact)."""
    s = unit_scale(a)
    a64 = a.astype(np.float64) / s
    r64 = r.astype(np.float64) / s
    q64 = q.astype(np.float64)
    na = np.linalg.norm(a64, axis=(-2, -1))
    recon = np.linalg.norm(a64 - q64 @ r64, axis=(-2, -1)) / np.where(na > 0, na, 1.0)
    eye = np.eye(q.shape[-1])
    orth = np.linalg.norm(np.swapaxes(q64, -1, -2) @ q64 - eye, axis=(-2, -1))
    low = np.abs(np.tril(r, -1)).max(axis=(-2, -1)) if r.shape[-2] > 1 else np.zeros(r.shape[:-2])
    return recon, orth, low


def sign_normalise(q, r):
    """Flip column i of Q and row i of R wherever R[i, i] < 0."""
    k = min(r.shape[-2], r.shape[-1])
    d = np.diagonal(r, axis1=-2, axis2=-1)[..., :k]
    s = np.where(d < 0, -1.0, 1.0).astype(r.dtype)
    r2 = r.copy()
    r2[..., :k, :] *= s[..., :, None]
    q2 = None
    if q is not None and q.size:
        q2 = q.copy()
        q2[..., :, :k] *= s[..., None, :]
    return q2, r2


def r_parity(r, r_ref, a=None, tiny=1e-4):
    """max over matrices of max|R - R_ref| / max|R_ref| after sign normalisation. Rows
    whose diagonal is below `tiny` of the matrix's largest |R| (a rank-deficient tail,
    where the row's direction is arbitrary) are compared in magnitude of the diagonal
    only."""
    _, rn = sign_normalise(None, r)
    _, fn = sign_normalise(None, r_ref)
    rn = rn.astype(np.float64)
    fn = fn.astype(np.float64)
    top = np.abs(fn).max(axis=(-2, -1), keepdims=True)
    top = np.where(top > 0, top, 1.0)
    k = min(r.shape[-2], r.shape[-1])
    d = np.abs(np.diagonal(fn, axis1=-2, axis2=-1)[..., :k])
    solid = (d > tiny * top[..., 0]) .astype(np.float64)
    # a row is comparable only while every earlier pivot is solid too
    solid = np.cumprod(solid, axis=-1)
    mask = np.zeros(rn.shape)
    mask[..., :k, :] = solid[..., :, None]
    diff = np.abs(rn - fn) * mask
    dd = np.abs(np.abs(np.diagonal(rn, axis1=-2, axis2=-1)[..., :k]) - d) * (1 - solid)
    return max((diff / top).max(), (dd / top[..., 0]).max())
