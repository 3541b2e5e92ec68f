import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.cpu_oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle.cpu_oracle import Reference
    if not Reference.available():
        pytest.skip("reference checker library not built on this machine")
    return Reference()


@pytest.fixture(scope="session")
def csr_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "csr_golden.npz"))


@pytest.fixture(scope="session")
def tensor3_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "tensor3_golden.npz"))
