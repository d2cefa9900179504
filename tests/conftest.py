import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


@pytest.fixture(scope="session")
def backend():
    """The backend facade; builds the library on first use if it is missing."""
    from pjrtx_b200 import backend as be

    if not os.path.exists(be.LIB_PATH):
        import __graft_entry__

        __graft_entry__.build()
    return be.Backend()


@pytest.fixture(scope="session")
def gpu_backend(backend):
    if backend.lib.pjrtx_b200_device_count() < 1:
        pytest.fail("no CUDA device visible: GPU tests must run on a B200 (" + backend.lib.pjrtx_b200_last_error().decode() + ")")
    backend.enumerate_devices()
    return backend
