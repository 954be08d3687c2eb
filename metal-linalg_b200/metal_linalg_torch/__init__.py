"""Batched float32 Householder QR on NVIDIA B200 for PyTorch, behind the API of
metal-linalg's torch binding.

ADAPTED COPY OF THE REFERENCE'S FILE, not written from scratch: `_prepare`, `_needs_grad`, `_TRACED`, `_result` and
`qr()` with its docstring are the reference's python-torch/metal_linalg_torch/__init__.py:45-115 (under half of this
file), kept so that a caller of the reference's binding finds the same functions with the same behaviour; "cuda" is
added to the devices served, and the helpers below `qr` are this build's.

    import torch
    import metal_linalg_torch as mlt

    Q, R = mlt.qr(a)                      # a: [..., M, N] on "cuda" (or "cpu": staged through the GPU)
    Q, R = mlt.qr(a, mode="complete")
    _, R = mlt.qr(a, mode="r")

`qr` takes the arguments of torch.linalg.qr and returns the same result type on
the input's device. It supports autograd (torch.linalg's formula) and
torch.compile: underneath it is the custom operator torch.ops.metal_linalg.qr.
Computation is in float32: other real dtypes are converted, results are float32.
Beside QR this build holds the SVD that calls it (`svd`, `svdvals`: the QR-preconditioned
Jacobi route, min(M, N) <= 128); the reference's other decompositions do not exist here.
"""
from collections import namedtuple

import torch

from . import _lib, _ops  # noqa: F401  (_ops registers torch.ops.metal_linalg.qr)
from ._build import version as __version__
from ._interop import qr_dlpack, qr_into, qr_shapes
from ._sharded import qr_sharded, shard_batch

__all__ = [
    "qr", "svd", "svdvals", "svd_backend", "svdvals_backend", "qr_sharded", "shard_batch", "qr_into", "qr_dlpack", "qr_shapes",
    "device_name", "gpu_core_count", "device_count", "cpu_threads", "set_cpu_threads",
    "cpu_only", "set_cpu_only", "CpuOnly",
    "qr_backend", "qr_kernel", "qr_policy", "set_qr_policy", "qr_policy_source",
    "calibration_status",
]

_DEVICES = ("cpu", "cuda", "meta")


def _prepare(A, name):
    """A as a float32 tensor [..., M, N] on a device the library serves."""
    if not isinstance(A, torch.Tensor):
        A = torch.as_tensor(A)
    if A.is_complex():
        raise TypeError(f"metal_linalg_torch.{name}: complex input is not supported (got {A.dtype}); "
                        f"the decompositions are real, in float32")
    if A.dim() < 2:
        raise ValueError(f"metal_linalg_torch.{name}: expected a tensor of shape [..., M, N], "
                         f"got shape {tuple(A.shape)}")
    if A.device.type not in _DEVICES:
        raise ValueError(f"metal_linalg_torch.{name}: tensors on {A.device} are not supported; "
                         f"use CUDA or the CPU")
    return A if A.dtype == torch.float32 else A.to(torch.float32)


def _needs_grad(a):
    return torch.is_grad_enabled() and a.requires_grad


_TRACED = {"linalg_qr": namedtuple("linalg_qr", ["Q", "R"]),
           "linalg_svd": namedtuple("linalg_svd", ["U", "S", "Vh"])}


def _result(kind, values):
    if torch.compiler.is_compiling():
        return _TRACED[kind](*values)
    return getattr(torch.return_types, kind)(values)


def qr(A, mode="reduced"):
    """QR of a batch of matrices, like ``torch.linalg.qr``: ``A = Q @ R``.

    ``A`` is ``[..., M, N]``. Returns ``(Q, R)``: ``Q`` ``[..., M, K]`` with
    orthonormal columns and ``R`` ``[..., K, N]`` upper triangular,
    ``K = min(M, N)``. ``mode`` as torch's: ``"reduced"`` (the default),
    ``"r"`` (``R`` alone, ``Q`` an empty tensor and never formed) or
    ``"complete"`` (``Q`` ``[..., M, M]`` square, ``R`` ``[..., M, N]`` with
    zero rows below ``K``).

    Unlike torch's, ``mode="r"`` is differentiable: when ``A`` requires grad,
    ``Q`` is computed for the gradient and dropped. As torch's,
    ``mode="complete"`` is not differentiable when ``M > N``.
    """
    a = _prepare(A, "qr")
    if mode not in ("reduced", "r", "complete"):
        raise ValueError(f"metal_linalg_torch.qr: mode must be 'reduced', 'r' or 'complete', got {mode!r}")
    if mode == "r" and _needs_grad(a):
        _, R = torch.ops.metal_linalg.qr(a)
        return _result("linalg_qr", (R.new_empty(0), R))
    Q, R = torch.ops.metal_linalg.qr(a, mode)
    return _result("linalg_qr", (Q, R))


def svd(A, full_matrices=False):
    """Thin SVD of a batch of matrices, like ``torch.linalg.svd(A, full_matrices=False)``:
    ``A = U @ diag(S) @ Vh`` with ``U`` ``[..., M, K]``, ``S`` ``[..., K]`` descending and ``Vh``
    ``[..., K, N]``, ``K = min(M, N)`` (reference: python-torch/metal_linalg_torch/__init__.py:144-160).
    ``full_matrices=True`` is refused, as by the reference. The route is A = Q R by this library's
    QR, then one-sided Jacobi on R: ``K <= 128`` (a larger K raises ValueError)."""
    if full_matrices:
        raise NotImplementedError("metal_linalg_torch.svd: full_matrices=True is not supported; the thin "
                                  "decomposition is what the library computes")
    a = _prepare(A, "svd")
    return _result("linalg_svd", torch.ops.metal_linalg.svd(a))


def svdvals(A):
    """The singular values alone, descending, like ``torch.linalg.svdvals``: the QR runs in mode "r",
    so Q is never formed."""
    a = _prepare(A, "svdvals")
    return torch.ops.metal_linalg.svdvals(a)


def svd_backend(m, n, batch=1):
    """"qr_jacobi", or "unavailable" for a shape `svd` refuses."""
    return _lib.lib.metal_linalg_svd_backend(m, n, batch).decode()


def svdvals_backend(m, n, batch=1):
    return _lib.lib.metal_linalg_svdvals_backend(m, n, batch).decode()


# ---------------------------------------------------------------------------
# Device and routing
# ---------------------------------------------------------------------------

def device_name():
    """The GPU's name, e.g. "NVIDIA B200" ("" without one)."""
    return (_lib.lib.metal_linalg_device_name() or b"").decode()


def gpu_core_count():
    """The GPU's multiprocessor count (0 without a GPU)."""
    return int(_lib.lib.metal_linalg_gpu_core_count())


def device_count():
    return int(_lib.lib.metal_linalg_device_count())


def cpu_threads():
    return int(_lib.lib.metal_linalg_cpu_threads())


def set_cpu_threads(n):
    _lib.lib.metal_linalg_set_cpu_threads(int(n))


def cpu_only():
    return bool(_lib.lib.metal_linalg_cpu_only())


def set_cpu_only(on=True):
    """The reference sends the calling thread's calls to its CPU paths while this
    is set. This build has no CPU path: while it is set, `qr` on this thread
    raises rather than run on the GPU unasked."""
    _lib.lib.metal_linalg_set_cpu_only(1 if on else 0)


class CpuOnly:
    """``with CpuOnly():`` sets `set_cpu_only` for the block, for this thread."""

    def __init__(self, on=True):
        self._on = on

    def __enter__(self):
        self._previous = cpu_only()
        set_cpu_only(self._on)
        return self

    def __exit__(self, *exc):
        set_cpu_only(self._previous)
        return False


def qr_backend(rows, cols, batch=1):
    """"unblocked" (a matrix to a warp or a thread block) or "streaming_reduced"
    (a matrix spread over the grid) under the policy in effect."""
    return _lib.lib.metal_linalg_qr_backend(rows, cols, batch).decode()


def qr_kernel(rows, cols, batch=1, mode="reduced"):
    """The kernel a call of that shape runs: "small", "mid", "tsqr" or "blocked"."""
    name = _lib.lib.metal_linalg_qr_kernel(rows, cols, batch, _lib.MODES[mode]).decode()
    if not name:
        raise RuntimeError(_lib.last_error())
    return name


_POLICY_FIELDS = [name for name, _ in _lib.QrPolicy._fields_]


def qr_policy():
    """The routing policy in effect, as a dict (fields as the reference's QrPolicy)."""
    p = _lib.lib.metal_linalg_qr_policy_get()
    return {name: int(getattr(p, name)) for name in _POLICY_FIELDS}


def set_qr_policy(**fields):
    """Replaces fields of the routing policy; it then reports its source as "user"."""
    p = _lib.lib.metal_linalg_qr_policy_get()
    for name, value in fields.items():
        if name not in _POLICY_FIELDS:
            raise ValueError(f"metal_linalg_torch.set_qr_policy: unknown field {name!r}")
        setattr(p, name, int(value))
    _lib.lib.metal_linalg_qr_policy_set(p)


def qr_policy_source():
    return _lib.lib.metal_linalg_qr_policy_source().decode()


def calibration_status():
    """"" if the routing table was measured on this GPU model, else a notice."""
    return (_lib.lib.metal_linalg_calibration_message(b"QR") or b"").decode()
