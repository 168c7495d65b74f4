import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import zant_oracle
    zant_oracle.build()
    return zant_oracle


@pytest.fixture(scope="session")
def zb():
    """The product package (loaded from the hyphenated directory by __graft_entry__)."""
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="session")
def ctx(zb):
    c = zb.Context(0)
    yield c
    c.close()
