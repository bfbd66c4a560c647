import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def kats():
    import json
    with open(os.path.join(GOLDEN, "reference_kats.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def refout():
    return dict(np.load(os.path.join(GOLDEN, "ref_outputs.npz")))


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU code (oracle/_ref), or None where it has not been built."""
    from oracle import ref as r
    return r if r.available() else None


@pytest.fixture(scope="session")
def lib():
    from eddl_b200 import capi
    L = capi.lib()
    if L.device_count() < 1:
        pytest.fail("no CUDA device visible: GPU tests cannot run (there is no CPU fallback)")
    L.call("init", 0)
    return L
