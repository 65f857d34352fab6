import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (runs the CUDA kernels through the C ABI)")


@pytest.fixture(scope="session")
def gpu():
    """The package with a device context: a real one when a GPU is present, else the
    metadata-only mode (recording, validation and fusion plans work; eval does not)."""
    import applegpu_runtime_b200 as g
    from applegpu_runtime_b200 import _lib
    lib = _lib.load()
    if lib.applegpu_ffi_init():
        g.api._initialized = True
        g.has_device = True
    else:
        g.init_backend(dry_run=True)
        g.has_device = False
    return g


@pytest.fixture(scope="session")
def gpu_dev(gpu):
    if not gpu.has_device:
        pytest.fail("a test marked gpu ran without a CUDA device: the CUDA path is mandatory")
    from applegpu_runtime_b200 import _lib
    assert _lib.load().applegpu_eager_init()
    return gpu
