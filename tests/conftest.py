"""pytest configuration: the `gpu` marker, import paths and build-on-demand.

CPU tests (`-m "not gpu"`) cover the oracle against the reference's fixtures
and CPU functions, the host-side logic and the C ABI's symbol table; GPU tests
(`-m gpu`) are the parity tests proper and call through the C ABI.
"""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Builds whatever is missing (incremental): the CUDA library, the C oracle and,
    where the reference tree is mounted, oracle/_ref/."""
    import __graft_entry__ as entry

    entry.build()


@pytest.fixture(scope="session")
def orc():
    from oracle import binding

    binding.lib()
    return binding


@pytest.fixture(scope="session")
def lib():
    from inferspore_b200 import capi

    return capi.load()


def has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.fixture(scope="session")
def cuda():
    if not has_gpu():
        pytest.skip("no CUDA device")
    import torch

    return torch.device("cuda:0")


@pytest.fixture()
def rng(request):
    import zlib

    return np.random.default_rng(zlib.crc32(request.node.nodeid.encode()))
