"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA library through its C ABI;
everything else runs on CPU (oracle, host logic, symbol checks)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.build_oracle()
    return O


@pytest.fixture(scope="session")
def ctx():
    """One library context on cuda:0 for the whole session (fails loudly without a GPU)."""
    import runit_mac_b200 as R
    c = R.Context(int(os.environ.get("RUNIT_TEST_DEVICE", "0")))
    yield c
    c.close()


@pytest.fixture
def rng(request):
    # one deterministic stream per test name
    seed = abs(hash(request.node.name)) % (2 ** 31)
    return np.random.default_rng(1234 + (sum(map(ord, request.node.name)) % 100000))
