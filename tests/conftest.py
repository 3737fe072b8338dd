"""Shared test setup: import paths, the ``gpu`` marker, cached synthetic models."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "qwen3-0.6b-megakernel-rtx-5090_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """Path of the in-tree C-ABI library, compiled on demand (nvcc cross-compiles without a GPU)."""
    import build
    return build.build()


@pytest.fixture(scope="session")
def tiny_cfg():
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden
    return dict(make_golden.TINY)


@pytest.fixture(scope="session")
def full_cfg():
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden
    return dict(make_golden.FULL)
