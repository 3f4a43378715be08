"""Shared fixtures. `-m "not gpu"` tests need no GPU; `-m gpu` tests are the parity tests proper."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    # The kernels are compiled at run time by whichever libnvrtc.so.12 the process holds first: the toolkit's, or the one
    # bundled with torch when torch was imported before the library (the benchmark does that). KURUMI_TEST_TORCH_FIRST=1
    # runs the suite in the second situation.
    if os.environ.get("KURUMI_TEST_TORCH_FIRST"):
        import torch  # noqa: F401


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


def pytest_terminal_summary(terminalreporter):
    """Achieved errors of the narrow-format parity checks (relative where the relative band applies, and in units of
    the row scale); also written to the file KURUMI_PARITY_LOG names, when it is set."""
    from tests import util
    if not util.PARITY_LOG:
        return
    terminalreporter.write_line("achieved parity errors (what: max rel err, max err / row scale)")
    lines = [f"  {what}: {rel:.3e}, {scaled:.3e}" for what, rel, scaled in util.PARITY_LOG]
    for ln in lines:
        terminalreporter.write_line(ln)
    path = os.environ.get("KURUMI_PARITY_LOG")
    if path:
        try:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            with open(path, "w") as f:
                f.write("\n".join(lines) + "\n")
        except OSError:
            pass
