"""pytest configuration: the `gpu` marker, package / oracle loaders and small fixtures."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built():
    """Library + oracle built once per session (no GPU needed to compile)."""
    entry.build()
    return True


@pytest.fixture(scope="session")
def pkg(built):
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle(built):
    return entry.load_oracle()


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"


@pytest.fixture(scope="session")
def device(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


@pytest.fixture()
def handle(pkg, device):
    from ops_sparse_b200 import api

    h = api.Handle()
    yield h
    h.close()
