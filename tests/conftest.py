"""pytest configuration: the `gpu` marker and shared fixtures.

CPU tests (`-m "not gpu"`) cover the oracle against golden vectors, host logic, and that the
C-ABI library loads and exports every declared symbol. GPU tests (`-m gpu`) are the parity tests:
they call the CUDA engine through its C ABI and compare with the oracle.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box)")


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session")
def binding():
    from oracle import binding as b
    b.oracle_lib()
    return b


@pytest.fixture(scope="session")
def gpu_lib(pkg):
    """The CUDA library; fails loudly (no fallback) when it is missing or no GPU answers."""
    L = pkg.lib()
    assert L.g5b_device_count() > 0, "no CUDA device: GPU tests cannot run"
    return L
