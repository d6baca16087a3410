import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import OracleExecutor
    return OracleExecutor()


@pytest.fixture(scope="session")
def cuda():
    """The CUDA device. No fallback: a missing library or GPU fails the test."""
    from anneal_b200 import build
    build.build()
    from anneal_b200.device import Device
    dev = Device(0)
    yield dev
    dev.close()


@pytest.fixture(autouse=True)
def fresh_graph():
    from anneal_b200 import realize
    realize.reset()
    yield
