import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "log-linear-attention_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(autouse=True)
def _read_status_words():
    """Every Mamba-2 driver call made by a test reads its workspace's status word and raises if a kernel gave
    up on a bounded wait (the drivers do not synchronise by default)."""
    from hattention_b200 import _lib
    old = _lib.CHECK_STATUS
    _lib.CHECK_STATUS = True
    yield
    _lib.CHECK_STATUS = old
