import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def oracle_lib():
    import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def psb():
    """The CUDA library binding; GPU tests fail loudly if it is not built or no sm_100 device exists."""
    from paraselect_b200 import api
    api.lib()
    assert api.device_count() > 0, "no sm_100 device: GPU tests must run on a B200"
    return api
