import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    if not os.path.exists(os.path.join(orc.HERE, "libsager_oracle.so")):
        orc.build()
    return orc.Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU code, when oracle/_ref was built; else skip."""
    from oracle import oracle as orc
    try:
        return orc.Reference()
    except (FileNotFoundError, OSError):
        pytest.skip("oracle/_ref/libsager_ref.so not built (needs the reference tree)")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "ref_cpu_golden.npz")
    return dict(np.load(path))
