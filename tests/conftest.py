import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def built_library():
    """Path of libdcb200.so, building it first if a source is newer (nvcc cross-compiles without a GPU)."""
    from dotcompute_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def acc(built_library):
    """The accelerator all GPU tests share. Fails (never skips) if no B200 is present: GPU tests carry the gpu marker."""
    from dotcompute_b200 import CudaAccelerator
    a = CudaAccelerator.Default()
    yield a


@pytest.fixture(scope="session")
def c_oracle():
    import oracle
    return oracle.c_oracle()
