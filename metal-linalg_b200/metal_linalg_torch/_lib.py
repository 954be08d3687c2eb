"""The C ABI through ctypes (reference: python-torch/metal_linalg_torch/_lib.py).

Only the QR, the SVD that calls it, and the device and policy entry points exist
in this build, and only they are bound. The library is lib/libmetal_linalg.so beside this package, or the
file METAL_LINALG_TORCH_LIBRARY names. Calls release the GIL (ctypes does); the
C side keeps the stream and the device per thread, so no lock is needed here.
"""
import ctypes
import os

from . import _build

OK, INVALID_ARGUMENT, RUNTIME_ERROR, OUT_OF_MEMORY = 0, 1, 2, 3
MODES = {"reduced": 0, "r": 1, "complete": 2}

_u32 = ctypes.c_uint32
_ptr = ctypes.c_void_p


class QrPolicy(ctypes.Structure):
    _fields_ = [(name, _u32) for name in (
        "m_crossover_small_batch", "m_crossover_large_batch", "batch_threshold", "gpu_max_k",
        "gpu_min_batch_times_k", "gpu_min_batch", "gpu_cores", "concurrent_matrices",
        "gpu_large_min_k", "gpu_large_max_batch", "gpu_min_k", "share_min_batch")]


def _path():
    return os.environ.get("METAL_LINALG_TORCH_LIBRARY") or _build.LIBRARY


def _load():
    path = _path()
    if not os.path.exists(path):
        raise ImportError(f"metal_linalg_torch: {path} is not built; run `python -c 'import __graft_entry__ as g; "
                          f"g.build()'` or `make -C {_build.ROOT}` (there is no fallback path)")
    lib = ctypes.CDLL(path)
    sig = {
        "metal_linalg_last_error": (ctypes.c_char_p, []),
        "metal_linalg_qr": (ctypes.c_int, [_ptr, _u32, _u32, _u32, _ptr, _ptr]),
        "metal_linalg_qr_with_mode": (ctypes.c_int, [_ptr, _u32, _u32, _u32, ctypes.c_int, _ptr, _ptr]),
        "metal_linalg_qr_no_alloc": (ctypes.c_int, [_ptr, _u32, _u32, _u32, ctypes.c_int, _ptr, _ptr]),
        "metal_linalg_qr_no_alloc_scratch_bytes": (ctypes.c_uint64, []),
        "metal_linalg_svd": (ctypes.c_int, [_ptr, _u32, _u32, _u32, _ptr, _ptr, _ptr, _ptr]),
        "metal_linalg_svd_backend": (ctypes.c_char_p, [_u32, _u32, _u32]),
        "metal_linalg_svdvals_backend": (ctypes.c_char_p, [_u32, _u32, _u32]),
        "metal_linalg_set_stream": (None, [_ptr]),
        "metal_linalg_stream": (_ptr, []),
        "metal_linalg_set_device": (ctypes.c_int, [ctypes.c_int]),
        "metal_linalg_device": (ctypes.c_int, []),
        "metal_linalg_device_count": (ctypes.c_int, []),
        "metal_linalg_synchronize": (ctypes.c_int, []),
        "metal_linalg_release_workspaces": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint64)]),
        "metal_linalg_inject_wait_failures": (None, [ctypes.c_int]),
        "metal_linalg_device_name": (ctypes.c_char_p, []),
        "metal_linalg_gpu_core_count": (_u32, []),
        "metal_linalg_set_calibration_notices": (None, [ctypes.c_int]),
        "metal_linalg_calibration_message": (ctypes.c_char_p, [ctypes.c_char_p]),
        "metal_linalg_set_cpu_threads": (None, [_u32]),
        "metal_linalg_cpu_threads": (_u32, []),
        "metal_linalg_set_cpu_only": (None, [ctypes.c_int]),
        "metal_linalg_cpu_only": (ctypes.c_int, []),
        "metal_linalg_qr_backend": (ctypes.c_char_p, [_u32, _u32, _u32]),
        "metal_linalg_qr_kernel": (ctypes.c_char_p, [_u32, _u32, _u32, ctypes.c_int]),
        "metal_linalg_qr_policy_get": (QrPolicy, []),
        "metal_linalg_qr_policy_set": (None, [ctypes.POINTER(QrPolicy)]),
        "metal_linalg_qr_policy_source": (ctypes.c_char_p, []),
    }
    for name, (restype, argtypes) in sig.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()
SYMBOLS = [n for n in dir(lib) if n.startswith("metal_linalg_")]


def last_error():
    return (lib.metal_linalg_last_error() or b"").decode()


def check(status):
    """A status as the exception the reference's binding raises for it."""
    if status == OK:
        return
    message = last_error()
    if status == INVALID_ARGUMENT:
        raise ValueError(message)
    if status == OUT_OF_MEMORY:
        raise MemoryError(message)
    raise RuntimeError(message)


def qr(a, batch, rows, cols, q, r, mode="reduced", stream=None):
    """metal_linalg_qr_with_mode on addresses (ints; None for NULL). `stream` is a
    cudaStream_t as an int for device pointers (None: leave this thread's as set)."""
    if stream is not None:
        lib.metal_linalg_set_stream(stream)
    check(lib.metal_linalg_qr_with_mode(a, batch, rows, cols, MODES[mode], q, r))


def synchronize():
    """Waits for this thread's stream; raises RuntimeError if a kernel gave up on a bounded wait."""
    check(lib.metal_linalg_synchronize())


def release_workspaces():
    """Frees the scratch memory the library keeps per (GPU, stream); returns the bytes freed."""
    freed = ctypes.c_uint64(0)
    check(lib.metal_linalg_release_workspaces(ctypes.byref(freed)))
    return freed.value


def svd(a, batch, rows, cols, u, s, vt, info=None, stream=None):
    """metal_linalg_svd on addresses (ints; None for NULL: u and vt both, for the values alone)."""
    if stream is not None:
        lib.metal_linalg_set_stream(stream)
    check(lib.metal_linalg_svd(a, batch, rows, cols, u, s, vt, info))
