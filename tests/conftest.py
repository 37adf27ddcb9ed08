import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# the tests choose the execution mode themselves: the process-wide default of the deferred mode must be the library's
os.environ.pop("KTEN_CUDA_LAZY", None)


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


@pytest.fixture()
def index_checks_at_call(cuda_ops):
    """The reference throws on an invalid index at the call (JVMRawTensor.kt:334-353); the library reads its index
    checks where the host next waits for the device unless `index_check_sync` is set.  Tests that expect the exception at
    the call switch it on."""
    from kten_b200 import _lib as L
    L.check(cuda_ops.lib.ktc_tune_set(b"index_check_sync", 1))
    yield
    L.check(cuda_ops.lib.ktc_tune_set(b"index_check_sync", 0))
