"""metal_linalg_qr_no_alloc: the QR entry point for callers that cannot allocate
device memory at call time (a latency-bound request loop that cannot afford the
device-wide stall of a cudaFree, or a process whose memory pool already owns the
GPU, where a library's cudaMalloc may fail). It runs the block-per-matrix kernel
on a scratch array that is part of the library image.

Checked here, through the C ABI: its Q and R equal those of the ordinary entry
point, metal_linalg_qr_with_mode, on two calls in a row that reuse the shared
scratch array with different shapes, and sizes beyond its limits are refused
with a message. The file sorts last on purpose, so a run that stops at the first
failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from metal_linalg_torch import _lib

pytestmark = pytest.mark.gpu


def _both(a, mode):
    """(q, r) from the ordinary entry point and from the no-allocation one, device pointers."""
    b, m, n = a.shape
    k = min(m, n)
    qc = {"reduced": k, "complete": m, "r": 0}[mode]
    rr = m if mode == "complete" else k
    outs = []
    for entry in ("ordinary", "no_alloc"):
        q = torch.full((b, m, qc), 7.0, device="cuda") if qc else None
        r = torch.full((b, rr, n), 7.0, device="cuda")
        qp = q.data_ptr() if qc else None
        _lib.lib.metal_linalg_set_stream(torch.cuda.current_stream().cuda_stream)
        if entry == "ordinary":
            status = _lib.lib.metal_linalg_qr_with_mode(a.data_ptr(), b, m, n, _lib.MODES[mode], qp, r.data_ptr())
        else:
            status = _lib.lib.metal_linalg_qr_no_alloc(a.data_ptr(), b, m, n, _lib.MODES[mode], qp, r.data_ptr())
        assert status == _lib.OK, _lib.last_error()
        torch.cuda.synchronize()
        outs.append((q, r))
    return outs


def test_no_alloc_matches_ordinary_entry_point_twice_in_a_row():
    torch.manual_seed(21)
    # two calls back to back on the one shared scratch array: different shapes and modes, the
    # second with more matrices than the array has slots for at once
    first = torch.randn(300, 96, 80, device="cuda")
    second = torch.randn(40, 700, 520, device="cuda")
    for a, mode in ((first, "complete"), (second, "reduced")):
        (q0, r0), (q1, r1) = _both(a, mode)
        scale = r0.abs().max().item()
        assert (r1 - r0).abs().max().item() <= 1e-5 * scale
        assert (q1 - q0).abs().max().item() <= 1e-5
        assert torch.count_nonzero(torch.tril(r1, -1)).item() == 0
        # and it is a QR in its own right
        err = (q1.double() @ r1.double() - a.double()).abs().max().item()
        assert err <= 1e-4 * max(1.0, a.abs().max().item())


def test_no_alloc_limits_are_refused_with_a_message():
    lib = _lib.lib
    assert lib.metal_linalg_qr_no_alloc_scratch_bytes() == 32 << 20
    a = torch.zeros(1, 1025, 8, device="cuda")
    q, r = torch.zeros(1, 1025, 8, device="cuda"), torch.zeros(1, 8, 8, device="cuda")
    assert lib.metal_linalg_qr_no_alloc(a.data_ptr(), 1, 1025, 8, 0, q.data_ptr(), r.data_ptr()) == _lib.INVALID_ARGUMENT
    assert "1024 rows" in _lib.last_error()
    a = torch.zeros(1, 512, 20000, device="cuda")                 # 41 MB of scratch for one matrix
    q, r = torch.zeros(1, 512, 512, device="cuda"), torch.zeros(1, 512, 20000, device="cuda")
    assert lib.metal_linalg_qr_no_alloc(a.data_ptr(), 1, 512, 20000, 0, q.data_ptr(), r.data_ptr()) == _lib.INVALID_ARGUMENT
    assert "scratch" in _lib.last_error()
    host = np.zeros((1, 8, 8), np.float32)                        # host memory would need staging buffers
    assert lib.metal_linalg_qr_no_alloc(host.ctypes.data, 1, 8, 8, 0, host.ctypes.data, host.ctypes.data) == _lib.INVALID_ARGUMENT
    assert lib.metal_linalg_qr_no_alloc(None, 0, 8, 8, 0, None, None) == _lib.OK


def test_no_alloc_leaves_device_memory_alone():
    """What the entry point is for: a call changes the GPU's free memory by nothing, where the ordinary
    entry point, with no workspace left from earlier calls, has to allocate one."""
    lib = _lib.lib
    torch.manual_seed(22)
    a = torch.randn(64, 640, 384, device="cuda")
    q, r = torch.empty(64, 640, 384, device="cuda"), torch.empty(64, 384, 384, device="cuda")
    lib.metal_linalg_set_stream(torch.cuda.current_stream().cuda_stream)
    args = (a.data_ptr(), 64, 640, 384, _lib.MODES["reduced"], q.data_ptr(), r.data_ptr())
    assert lib.metal_linalg_qr_no_alloc(*args) == _lib.OK, _lib.last_error()      # the first call looks the array up
    torch.cuda.synchronize()
    _lib.release_workspaces()                                                      # nothing is kept from earlier tests
    free0, _ = torch.cuda.mem_get_info()
    assert lib.metal_linalg_qr_no_alloc(*args) == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"the call changed free device memory by {free0 - free1} bytes"
    assert lib.metal_linalg_qr_with_mode(*args) == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    free2, _ = torch.cuda.mem_get_info()
    assert free2 < free1, "the ordinary entry point was expected to allocate its workspace"
