"""Shared fixtures. GPU tests carry @pytest.mark.gpu and call through the C ABI."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(Path(__file__).resolve().parent)):
    if p not in sys.path:
        sys.path.insert(0, p)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def la():
    """The package (loads liblocal_cuda.so; builds it first if stale)."""
    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure)."""
    return entry.load_oracle()


@pytest.fixture(scope="session")
def ctx(la):
    c = la.CudaContext.new(0)
    yield c
    c.close()


@pytest.fixture(scope="session")
def kernels(la, ctx):
    k = la.Kernels.new(ctx)
    yield k
    k.close()
