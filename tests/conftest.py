"""pytest configuration: the `gpu` marker and shared fixtures.

CPU tests (`-m "not gpu"`) cover the oracle against the reference's pins and the
committed golden vectors, the host-side logic and the C-ABI library's exports.
GPU tests (`-m gpu`) are the parity tests proper and call the CUDA path through
the C ABI.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import orc
    return orc.Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle import orc
    if not orc.have_reference():
        pytest.skip("reference shim not built (oracle/_ref/libw4ref.so)")
    return orc.Reference()
