"""The C-ABI library loads on a machine without a GPU, exports exactly what
include/kten_cuda.h declares, and refuses to compute without a device."""
import ctypes as C
import os
import re
import subprocess

import pytest

from kten_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kten_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"KTC_API\s+[\w\s\*]+?\b(ktc_\w+)\s*\(", text)))


def exported_symbols():
    out = subprocess.run(["nm", "-D", "--defined-only", L.LIB_PATH], check=True, capture_output=True, text=True).stdout
    return sorted(line.split()[-1] for line in out.splitlines() if " T ktc_" in line)


def test_header_declares_every_bound_symbol():
    assert declared_symbols() == sorted(L._PROTOTYPES)


def test_library_exports_exactly_the_header():
    assert exported_symbols() == declared_symbols()


def test_every_symbol_resolves_through_ctypes():
    lib = L.load()
    for name in declared_symbols():
        assert getattr(lib, name) is not None


def test_header_compiles_as_c():
    # the boundary is plain C: no C++ and no CUDA types in the signatures
    r = subprocess.run(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", HEADER], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_no_silent_cpu_path_without_a_device():
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a CUDA device is present")
    lib = L.load()
    n = C.c_int(0)
    assert lib.ktc_init(C.byref(n)) == L.KTC_ECUDA
    assert b"no CPU path" in lib.ktc_last_error()
    h = C.c_uint64(0)
    assert lib.ktc_alloc(0, 16, C.byref(h)) == L.KTC_ESTATE       # not initialised
    from kten_b200.tensor_operations import CUDATensorOperations
    with pytest.raises(L.KtenCudaError):
        CUDATensorOperations(0)


def test_version_and_status_codes():
    lib = L.load()
    assert b"sm_100a" in lib.ktc_version()
    assert (L.KTC_EINVAL, L.KTC_ESTATE, L.KTC_ENOMEM, L.KTC_ECUDA, L.KTC_ECOMM, L.KTC_ETIMEOUT) == (-1, -2, -3, -4, -5, -6)
