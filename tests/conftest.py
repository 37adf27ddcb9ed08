import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle_ops():
    from oracle.oracle import OracleTensorOperations
    return OracleTensorOperations(mode=1)


@pytest.fixture(scope="session")
def cuda_ops():
    """The CUDA backend on device 0.  Fails (never skips to a fallback) when the
    library or a device is missing."""
    from kten_b200.tensor_operations import CUDATensorOperations
    return CUDATensorOperations(0)


@pytest.fixture()
def gc_scope(cuda_ops):
    """One GC scope per test, like the OpenCL backend's test subclass
    (backend/kten-opencl/src/test/.../OpenCLTensorTests.kt:37-46)."""
    with cuda_ops.garbageCollector() as scope:
        yield scope
