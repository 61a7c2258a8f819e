import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def qg():
    import crit_hub_b200

    return crit_hub_b200


@pytest.fixture(scope="session")
def handle(qg):
    """One library handle on cuda:0 for the whole GPU session."""
    h = qg.QGemv(device=0)
    yield h
    h.close()
