"""The C++ entry point `qr_accelerated` (include/metal_linalg/qr.h) on a GPU: a C++ program built by
the package Makefile calls it for the three modes, a bad mode, batch shapes with several leading
dimensions and none, an empty batch, every real input type and a strided view, compares its results
with the C ABI's bit for bit and checks the properties the reference's dispatcher tests pin
(tests/test_qr.cpp:449-454 of the reference; the entry point's contract: src/mlx_api.cpp:37-71,122-149)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROGRAM = os.path.join(ROOT, "metal-linalg_b200", "build", "qr_accelerated_test")


def test_program_is_built():
    assert os.path.exists(PROGRAM), "the package Makefile builds it next to the library's objects"


@pytest.mark.gpu
def test_qr_accelerated_cpp_program():
    done = subprocess.run([PROGRAM], capture_output=True, text=True, timeout=600)
    print(done.stdout[-4000:])
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-1000:]
    assert " 0 failed" in done.stdout
