"""Test configuration: the `gpu` marker, import paths, shared helpers."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "metal-linalg_b200"), os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA B200 (run with -m gpu)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """The C-ABI library and the oracle are compiled before any test runs."""
    import __graft_entry__
    __graft_entry__.build()
