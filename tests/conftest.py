import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def kutacc_lib():
    """The C-ABI library, built on demand (nvcc cross-compiles without a GPU)."""
    from kutacc_b200 import api, build
    build.build()
    return api.lib()


@pytest.fixture(autouse=True)
def _clear_error_flag():
    """The library's error flag is sticky by design; tests must not leak it into each other."""
    yield
    from kutacc_b200 import api
    if api._lib is not None:
        api.clear_error()
