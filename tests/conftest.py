import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    from oracle.oracle import Ref
    if not Ref.available():
        pytest.skip("oracle/_ref/libfomoe_ref.so not built (reference tree absent)")
    return Ref()


@pytest.fixture(scope="session")
def fb():
    sys.path.insert(0, ROOT)
    import __graft_entry__
    __graft_entry__.build()
    import fomoe_b200
    fomoe_b200.lib()
    return fomoe_b200
