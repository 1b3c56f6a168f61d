import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle import Reference
    ref = Reference()
    if not ref.available:
        pytest.skip("reference plain-backend build (oracle/_ref) not present on this machine")
    return ref


@pytest.fixture
def tuning():
    """Sets knobs of the library's launch plans for one test (nnf_set_tuning) and restores the built-in choices afterwards."""
    import nnforge_b200.capi as capi
    yield capi.set_tuning
    capi.set_tuning("reset", 0)
