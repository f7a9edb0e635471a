import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


def _gpu_available() -> bool:
    try:
        from spoc_b200 import Backend
        return Backend().Device.count() > 0
    except Exception:
        return False


@pytest.fixture(scope="session")
def backend():
    from spoc_b200 import Backend
    from spoc_b200.build import build_library
    build_library()
    b = Backend()
    b.Device.init()
    assert b.Device.count() > 0, "no sm_100 device visible: GPU tests must fail loudly, not fall back"
    return b


@pytest.fixture(scope="session")
def device(backend):
    d = backend.Device.get(0)
    backend.Device.set_current(d)
    return d


@pytest.fixture(scope="session")
def oracle():
    from tests import oracle_lib
    return oracle_lib.load()
