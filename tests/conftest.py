import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def native_lib():
    """The C-ABI library, built in-tree if stale.  No CPU fallback exists: a missing library
    is a failure, not a skip."""
    from edmir_b200 import _lib, build

    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture()
def cuda_clean():
    """GPU tests: fail if a kernel left a device-side status behind, and re-arm it."""
    import torch
    from edmir_b200 import linear

    assert torch.cuda.is_available(), "this test needs a CUDA device"
    linear.clear_status()
    yield
    st = linear.status()
    linear.clear_status()
    assert st[0] == 0, f"device-side wait timed out: {st[:8]}"
