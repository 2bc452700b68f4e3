import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    return oracle.load("orc")


@pytest.fixture(scope="session")
def ref():
    from oracle import oracle
    if not oracle.available("ref"):
        pytest.skip("compiled reference (oracle/_ref) not present")
    return oracle.load("ref")
