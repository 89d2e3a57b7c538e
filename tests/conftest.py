"""pytest configuration: registers the ``gpu`` marker and provides session fixtures.

``-m "not gpu"`` covers the oracle, the host logic and the C-ABI surface (no compute calls);
``-m gpu`` holds the parity tests proper, which call the CUDA library through its C-ABI and compare
with the CPU oracle.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    import oracle as _oracle
    _oracle.lib()
    return _oracle


@pytest.fixture(scope="session")
def gpu():
    """The loaded CUDA library, initialised on device 0.  Fails loudly when it is missing."""
    import simplang_b200 as sg
    sg.init(0)
    yield sg
    sg.sync()
