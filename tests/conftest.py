import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _build_everything():
    from basalt_b200 import build as product_build
    product_build.build()
    from oracle import build as oracle_build
    return oracle_build.build()


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (oracle/liborc.so): the checker, never the thing under test."""
    lib = ctypes.CDLL(_build_everything())
    lib.orc_time_max_i32.restype = ctypes.c_double
    lib.orc_f16_to_f32.restype = ctypes.c_float
    lib.orc_f64_to_f16.restype = ctypes.c_uint16
    lib.orc_f64_to_f16.argtypes = [ctypes.c_double]
    return lib


@pytest.fixture(scope="session")
def ptx():
    _build_everything()
    import basalt_b200
    return basalt_b200.Ptx()


def vp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


@pytest.fixture(scope="session")
def gpu():
    """(driver, context) on device 0 through the C-ABI runtime."""
    _build_everything()
    import basalt_b200
    drv = basalt_b200.CudaDriver.load()
    assert drv.device_count() >= 1
    ctx = drv.create_context(0)
    yield ctx
    ctx.synchronize()
