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


@pytest.fixture(params=["tensor_cores", "fp32_kernels"])
def contraction_path(request, capi):
    """Runs a test once with the tcgen05 3xTF32 kernels and once with the exact FP32 kernels."""
    import ctypes

    capi.call("set_tensor_cores", ctypes.c_int(1 if request.param == "tensor_cores" else 0))
    yield request.param
    code = ctypes.c_int(0)
    capi.call("device_status", ctypes.byref(code))  # raises if a kernel gave up a bounded wait
    capi.call("set_tensor_cores", ctypes.c_int(1))
