"""The C-ABI library without a GPU: it loads, exports every function the header
declares, checks its arguments, keeps the policy, and fails loudly (never falls
back) when asked to compute with no GPU present."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import metal_linalg_torch as mlt
from metal_linalg_torch import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "metal_linalg", "c_api.h")
NO_GPU = not torch.cuda.is_available()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(metal_linalg_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_build.LIBRARY)
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in c_api.h but not exported"


def test_binding_binds_only_what_the_header_declares():
    for name in _lib.SYMBOLS:
        assert name in declared_functions()


def test_argument_errors_need_no_gpu():
    lib = _lib.lib
    q = np.zeros(4, np.float32)
    r = np.zeros(4, np.float32)
    qp, rp = q.ctypes.data, r.ctypes.data
    # tests/test_c_api.c:201-206 of the reference
    assert lib.metal_linalg_qr(None, 1, 2, 2, qp, rp) == _lib.INVALID_ARGUMENT
    assert len(_lib.last_error()) > 0
    assert lib.metal_linalg_qr(None, 0, 2, 2, None, None) == _lib.OK          # an empty batch needs no buffers
    a = np.eye(2, dtype=np.float32)
    assert lib.metal_linalg_qr_with_mode(a.ctypes.data, 1, 2, 2, 7, qp, rp) == _lib.INVALID_ARGUMENT
    assert lib.metal_linalg_qr_with_mode(a.ctypes.data, 1, 2, 2, 2, None, rp) == _lib.INVALID_ARGUMENT
    assert lib.metal_linalg_qr_with_mode(a.ctypes.data, 1, 2, 2, 1, None, None) == _lib.INVALID_ARGUMENT
    assert lib.metal_linalg_set_device(10 ** 6) == _lib.INVALID_ARGUMENT


@pytest.mark.skipif(not NO_GPU, reason="checks the behaviour on a machine without a GPU")
def test_no_gpu_fails_loudly():
    a = np.eye(4, dtype=np.float32)[None]
    q, r = np.zeros_like(a), np.zeros_like(a)
    status = _lib.lib.metal_linalg_qr(a.ctypes.data, 1, 4, 4, q.ctypes.data, r.ctypes.data)
    assert status == _lib.RUNTIME_ERROR
    assert "no CPU path" in _lib.last_error()
    assert not q.any() and not r.any()          # nothing was computed anywhere
    with pytest.raises(RuntimeError):
        mlt.qr(torch.eye(4))
    assert mlt.device_name() == "" and mlt.gpu_core_count() == 0


def test_complete_of_no_columns_is_identity_on_the_host():
    # tests/test_c_api.c:76-80 of the reference; needs no kernel
    qc = np.full(18, 7.0, np.float32)
    assert _lib.lib.metal_linalg_qr_with_mode(None, 2, 3, 0, 2, qc.ctypes.data, None) == _lib.OK
    assert np.array_equal(qc.reshape(2, 3, 3), np.stack([np.eye(3, dtype=np.float32)] * 2))


def test_policy_round_trip_and_routing():
    before = mlt.qr_policy()
    try:
        assert set(before) == {n for n, _ in _lib.QrPolicy._fields_}
        assert ctypes.sizeof(_lib.QrPolicy) == 12 * 4              # the reference's struct layout
        mlt.set_qr_policy(m_crossover_small_batch=100, m_crossover_large_batch=200, batch_threshold=8,
                          gpu_large_min_k=0)
        assert mlt.qr_policy_source() == "user"
        p = mlt.qr_policy()
        assert (p["m_crossover_small_batch"], p["m_crossover_large_batch"], p["batch_threshold"]) == (100, 200, 8)
        # k = min(M, N) against the crossover of the batch's side (reference: src/qr.mm:231-236)
        assert mlt.qr_backend(150, 150, 1) == "streaming_reduced"
        assert mlt.qr_backend(150, 150, 8) == "unblocked"
        assert mlt.qr_backend(4000, 99, 1) == "unblocked"
        assert mlt.qr_backend(99, 4000, 1) == "unblocked"
        assert mlt.qr_backend(250, 200, 1000) == "streaming_reduced"
        # the large clause on sqrt(M k) (reference: src/qr.mm:264-268)
        mlt.set_qr_policy(gpu_large_min_k=512, gpu_large_max_batch=4)
        assert mlt.qr_backend(8192, 64, 1) == "streaming_reduced"      # 8192 * 64 >= 512^2
        assert mlt.qr_backend(8192, 64, 5) == "unblocked"              # beyond gpu_large_max_batch
        assert mlt.qr_backend(4000, 64, 1) == "unblocked"
        mlt.set_qr_policy(gpu_large_min_k=512, gpu_large_max_batch=0)
        assert mlt.qr_backend(8192, 64, 6) == "streaming_reduced"      # 8192 * 64 >= 512^2 * 6 / 3
        assert mlt.qr_backend(8192, 64, 7) == "unblocked"              # the size grows with the batch
        # fields the GPU-only build carries without using are read back as set
        mlt.set_qr_policy(gpu_max_k=0, share_min_batch=5)
        assert mlt.qr_policy()["gpu_max_k"] == 0 and mlt.qr_policy()["share_min_batch"] == 5
        assert mlt.qr_backend(16, 16, 1) != "cpu"
        with pytest.raises(ValueError):
            mlt.set_qr_policy(no_such_field=1)
    finally:
        mlt.set_qr_policy(**{k: v for k, v in before.items() if k not in ("gpu_cores", "concurrent_matrices")})


def test_cpu_only_is_thread_local_and_refuses():
    import threading
    seen = {}
    with mlt.CpuOnly():
        assert mlt.cpu_only()
        t = threading.Thread(target=lambda: seen.setdefault("other", mlt.cpu_only()))
        t.start()
        t.join()
        with pytest.raises(RuntimeError, match="CPU"):
            mlt.qr(torch.eye(3))
    assert seen["other"] is False and not mlt.cpu_only()


def test_binding_rejects_and_shapes():
    # python-torch/tests/test_torch.py:269-281 of the reference
    with pytest.raises(TypeError):
        mlt.qr(torch.zeros(2, 2, dtype=torch.complex64))
    with pytest.raises(ValueError):
        mlt.qr(torch.zeros(3))
    with pytest.raises(ValueError):
        mlt.qr(torch.zeros(3, 3), mode="full")
    q, r = mlt.qr(torch.zeros(0, 5, 3))
    assert q.shape == (0, 5, 3) and r.shape == (0, 3, 3)
    q, r = mlt.qr(torch.zeros(2, 4, 0), mode="complete")
    assert torch.equal(q, torch.eye(4).expand(2, 4, 4)) and r.shape == (2, 4, 0)
    q, r = torch.ops.metal_linalg.qr(torch.zeros(2, 5, 3, device="meta"), "complete")
    assert q.shape == (2, 5, 5) and r.shape == (2, 5, 3) and q.dtype == torch.float32
    q, r = torch.ops.metal_linalg.qr(torch.zeros(2, 3, 5, device="meta"), "r")
    assert q.shape == (0,) and r.shape == (2, 3, 5)


def test_interop_shapes_and_argument_checks():
    """qr_into's checks need no GPU: shapes per mode, dtype, contiguity, missing interface."""
    assert mlt.qr_shapes((5, 7, 3)) == ((5, 7, 3), (5, 3, 3))
    assert mlt.qr_shapes((7, 3), "complete") == ((7, 7), (7, 3))
    assert mlt.qr_shapes((2, 2, 3, 7), "r") == (None, (2, 2, 3, 7))
    with pytest.raises(ValueError):
        mlt.qr_shapes((3,))
    with pytest.raises(ValueError):
        mlt.qr_shapes((3, 3), "full")

    class Fake:
        def __init__(self, shape, typestr="<f4", strides=None, ptr=4096):
            self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3,
                                             "strides": strides}

    with pytest.raises(TypeError, match="__cuda_array_interface__"):
        mlt.qr_into(torch.zeros(2, 2), Fake((2, 2)), Fake((2, 2)))
    with pytest.raises(TypeError, match="float32"):
        mlt.qr_into(Fake((4, 3), "<f8"), Fake((4, 3)), Fake((3, 3)))
    with pytest.raises(ValueError, match="C-contiguous"):
        mlt.qr_into(Fake((4, 3), strides=(4, 16)), Fake((4, 3)), Fake((3, 3)))
    with pytest.raises(ValueError, match="expected shape"):
        mlt.qr_into(Fake((4, 3)), Fake((4, 4)), Fake((3, 3)))
    with pytest.raises(ValueError, match="None exactly"):
        mlt.qr_into(Fake((4, 3)), Fake((4, 3)), Fake((3, 3)), mode="r")
    # an empty batch is a no-op and touches no pointer
    q, r = Fake((0, 4, 3), ptr=0), Fake((0, 3, 3), ptr=0)
    assert mlt.qr_into(Fake((0, 4, 3), ptr=0), q, r) == (q, r)
