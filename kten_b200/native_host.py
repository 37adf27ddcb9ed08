"""ctypes binding of libkten_host.so: the compiled host above the C ABI (kten_b200/csrc/host/kten_host.cpp).

kten's own host side is compiled code on a JVM; the Python mirror in this package spends about 0.2 ms of
interpreter time per training step.  libkten_host.so restates the raw tensor and the autograd caller of the
sharded benchmark step in C++, issuing the same C-ABI call sequence, so that the step can be timed with a
host as fast as the one the reference would bring."""
from __future__ import annotations

import ctypes as C
import os

from . import _lib as L

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkten_host.so")
_host = None


def load() -> C.CDLL:
    global _host
    if _host is None:
        L.load()                                             # libkten_cuda.so first: the host library links against it
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m kten_b200.build`")
        lib = C.CDLL(LIB_PATH)
        lib.kth_last_error.restype = C.c_char_p
        lib.kth_sharded_create.argtypes = [C.c_int, C.c_uint64, C.c_int64, C.c_int64, C.c_uint64, C.c_uint64, C.c_int, C.c_uint64, C.POINTER(C.c_void_p)]
        lib.kth_sharded_run.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_uint64)]
        lib.kth_sharded_destroy.argtypes = [C.c_void_p]
        _host = lib
    return _host


def _check(lib, status: int) -> None:
    if status != L.KTC_OK:
        raise RuntimeError(f"[{status}] {lib.kth_last_error().decode('utf-8', 'replace')}")


class NativeShardedStep:
    """loss = sum(sigmoid(x*w + b) pow 2) with backward for w and b, driven from C++.  x, w, b: raw tensors of
    the CUDA backend that the caller keeps alive; comm: the handle of a connected peer-memory communicator (0 in
    a world of one)."""

    def __init__(self, ops, x, w, b, lazy: bool, comm: int = 0):
        self.lib, self.ops = load(), ops
        self.handle = C.c_void_p(0)
        rows, cols = x.shape
        _check(self.lib, self.lib.kth_sharded_create(ops.device, x.storeReference, rows, cols, w.storeReference, b.storeReference,
                                                     1 if lazy else 0, comm, C.byref(self.handle)))

    def run(self, steps: int, results: bool = False):
        """`steps` steps back to back.  With `results`: the buffer handles of the last step's (loss, grad w, grad b),
        valid until the next call."""
        out = (C.c_uint64 * 3)() if results else None
        _check(self.lib, self.lib.kth_sharded_run(self.handle, steps, out))
        return [int(h) for h in out] if results else None

    def close(self) -> None:
        if self.handle:
            _check(self.lib, self.lib.kth_sharded_destroy(self.handle))
            self.handle = C.c_void_p(0)
