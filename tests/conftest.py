import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


@pytest.fixture(scope="session")
def oracle_engine():
    import oracle

    return oracle.engine()


@pytest.fixture(scope="session")
def gpu_engine():
    import rusttensor_b200

    return rusttensor_b200.engine()


@pytest.fixture(scope="session")
def capi(gpu_engine):
    """Raw C-ABI access on the same context the engine uses."""
    import rusttensor_b200

    return rusttensor_b200.CApi(ctx=rusttensor_b200.context_handle())
