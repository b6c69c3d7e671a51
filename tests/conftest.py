import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.load_port()


@pytest.fixture(scope="session")
def ref():
    """The reference compiled from its own headers, or None where it was never built."""
    import oracle
    return oracle.load_ref()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden")

    def load(name):
        return np.load(os.path.join(path, name + ".npz"))
    return load
