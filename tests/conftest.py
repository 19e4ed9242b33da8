import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle_port():
    import oracle
    if not os.path.exists(oracle.PORT_PATH):
        oracle.build()
    return oracle.Oracle("port")


@pytest.fixture(scope="session")
def oracle_ref():
    import oracle
    if not oracle.have_reference_build():
        pytest.skip("reference-linked oracle build not present on this machine")
    return oracle.Oracle("ref")
