"""The QR for arrays of other libraries, on the same C ABI: anything that exposes
`__cuda_array_interface__` (CuPy, Numba, PyTorch, JAX through its DLPack capsule) or `__dlpack__`.

    q, r = mlt.qr_into(a, q, r, mode="reduced", stream=None)    # caller's buffers, no copies
    Q, R = mlt.qr_dlpack(x, mode="reduced")                      # torch tensors that share no memory with x's producer

`qr_into` hands the three device pointers to `metal_linalg_qr_with_mode` as they are: float32,
C-contiguous, one GPU, `a` of shape [..., M, N], `q` and `r` of the shapes the mode gives
(reference contract: include/metal_linalg/c_api.h:36-50). The work is enqueued on `stream` (a
cudaStream_t as an int; None: the stream named by the arrays' interface, else the default stream)
and the call does not wait for it.
"""
import math

from . import _lib

__all__ = ["qr_into", "qr_dlpack", "qr_shapes"]


def qr_shapes(shape, mode="reduced"):
    """The shapes of Q and R for an input of `shape` = (..., M, N) (Q: None for mode "r")."""
    if mode not in _lib.MODES:
        raise ValueError(f"mode must be one of {sorted(_lib.MODES)}, got {mode!r}")
    if len(shape) < 2:
        raise ValueError(f"expected a shape (..., M, N), got {tuple(shape)}")
    *lead, m, n = (int(s) for s in shape)
    k = min(m, n)
    q = None if mode == "r" else (*lead, m, m if mode == "complete" else k)
    r = (*lead, m if mode == "complete" else k, n)
    return q, r


def _describe(x, name, want_shape=None):
    """(pointer, shape, stream) of a float32 C-contiguous device array."""
    cai = getattr(x, "__cuda_array_interface__", None)
    if cai is None:
        raise TypeError(f"{name}: expected an object with __cuda_array_interface__, got {type(x).__name__}")
    if cai.get("typestr") not in ("<f4", "=f4", "|f4"):
        raise TypeError(f"{name}: expected float32 (typestr '<f4'), got {cai.get('typestr')!r}")
    shape = tuple(int(s) for s in cai["shape"])
    strides = cai.get("strides")
    if strides is not None:
        expect, acc = [], 4
        for s in reversed(shape):
            expect.append(acc)
            acc *= max(s, 1)
        if any(s > 1 and st != e for s, st, e in zip(shape, strides, reversed(expect))):
            raise ValueError(f"{name}: expected a C-contiguous array, got strides {tuple(strides)} for shape {shape}")
    if want_shape is not None and shape != tuple(want_shape):
        raise ValueError(f"{name}: expected shape {tuple(want_shape)}, got {shape}")
    ptr = int(cai["data"][0])
    if ptr == 0 and math.prod(shape) != 0:
        raise ValueError(f"{name}: null data pointer")
    return ptr, shape, cai.get("stream")


def qr_into(a, q, r, mode="reduced", stream=None):
    """A = Q R of the device array `a` into the caller's device arrays `q` (None for mode "r") and `r`.
    Returns (q, r). Raises TypeError / ValueError for arrays the C ABI cannot take as they are."""
    a_ptr, a_shape, a_stream = _describe(a, "a")
    q_shape, r_shape = qr_shapes(a_shape, mode)
    if (q is None) != (q_shape is None):
        raise ValueError("q must be None exactly when mode is 'r'")
    q_ptr = None if q is None else _describe(q, "q", q_shape)[0]
    r_ptr = _describe(r, "r", r_shape)[0]
    *lead, m, n = a_shape
    batch = math.prod(lead)
    if batch * m * n == 0:
        return q, r
    if stream is None:
        stream = a_stream if isinstance(a_stream, int) and a_stream > 2 else 0     # 1 and 2 name the default streams
    _lib.qr(a_ptr, batch, m, n, q_ptr, r_ptr, mode, stream)
    return q, r


def qr_dlpack(x, mode="reduced"):
    """A = Q R of any array that exports DLPack (`__dlpack__`), as torch tensors on its device."""
    import torch

    from . import qr
    return qr(torch.from_dlpack(x), mode=mode)
