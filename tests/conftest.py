"""Shared fixtures. `-m "not gpu"` tests need no GPU; `-m gpu` tests are the parity tests proper."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def oracle_lib():
    from kurumi_b200 import api, build
    if not os.path.exists(build.ORACLE_LIB):
        build.build_oracle()
    lib = api.Library(build.ORACLE_LIB)
    import ctypes as C
    lib.lib.ko_threefry2x32.restype = C.c_uint64
    lib.lib.ko_uniform_f32.restype = C.c_float
    lib.lib.ko_force_counted.restype = C.c_long
    return lib


@pytest.fixture(scope="session")
def cuda_lib():
    from kurumi_b200 import api, build
    if not os.path.exists(build.LIB):
        build.build_library()
    return api.Library(build.LIB)


@pytest.fixture(scope="session")
def cpu(oracle_lib):
    from kurumi_b200 import api
    return api.Backend(oracle_lib, 0)


@pytest.fixture(scope="session")
def cpu64(oracle_lib):
    from kurumi_b200 import api
    return api.Backend(oracle_lib, 64)


@pytest.fixture(scope="session")
def cpu_fused(oracle_lib):
    from kurumi_b200 import api
    return api.Backend(oracle_lib, 65)


@pytest.fixture(scope="session")
def gpu(cuda_lib):
    """The CUDA backend. Fails loudly (no skip, no fallback) when the device or library is missing."""
    from kurumi_b200 import api
    return api.CudaBackend(cuda_lib, 0)
