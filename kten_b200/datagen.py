"""Seeded synthetic inputs (host side) shared by the tests and the benchmark.

The generator is counter based -- element i of stream t under seed s depends on
(s, t, i) only -- so a shard [first, first + n) of a large tensor can be
generated on its own by the rank that owns it.  The definition is in
csrc/ktc_datagen.c; `uniform_numpy` restates the uniform path in numpy so the
compiled generator can be pinned from a test.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkten_datagen.so")
SRC = os.path.join(HERE, "csrc", "ktc_datagen.c")
_lib = None


def build(force: bool = False) -> str:
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(SRC):
        cc = shutil.which("gcc") or "gcc"
        subprocess.run([cc, "-O2", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", "-ffp-contract=off",
                        "-o", LIB_PATH, SRC, "-lm"], check=True, capture_output=True)
    return LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        l = C.CDLL(LIB_PATH)
        l.ktd_uniform.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_uint64, C.c_uint64, C.c_double, C.c_double]
        l.ktd_uniform.restype = None
        l.ktd_normal.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_uint64, C.c_uint64, C.c_double, C.c_double, C.c_double]
        l.ktd_normal.restype = None
        _lib = l
    return _lib


def _out(n: int, out):
    if out is None:
        return np.empty(n, dtype=np.float32)
    assert out.dtype == np.float32 and out.size >= n and out.flags.c_contiguous
    return out


def uniform(n: int, seed: int, lo: float, hi: float, stream: int = 0, first: int = 0, out=None) -> np.ndarray:
    """n floats ~ U(lo, hi): elements [first, first + n) of the stream."""
    a = _out(n, out)
    _load().ktd_uniform(a.ctypes.data, n, first, seed, stream, lo, hi)
    return a[:n] if out is not None else a


def normal(n: int, seed: int, mean: float = 0.0, sd: float = 1.0, stream: int = 0, first: int = 0,
           quantum: float = 0.0, out=None) -> np.ndarray:
    """n floats ~ N(mean, sd); quantum q > 0 rounds to multiples of 1/q."""
    a = _out(n, out)
    _load().ktd_normal(a.ctypes.data, n, first, seed, stream, mean, sd, quantum)
    return a[:n] if out is not None else a


def uniform_numpy(n: int, seed: int, lo: float, hi: float, stream: int = 0, first: int = 0) -> np.ndarray:
    """The uniform path restated in numpy (slow; for pinning the C generator)."""
    with np.errstate(over="ignore"):
        i = np.arange(first + 1, first + n + 1, dtype=np.uint64)
        z = (np.uint64(seed) ^ (np.uint64(stream) * np.uint64(0xD1B54A32D192ED03))) + i * np.uint64(0x9E3779B97F4A7C15)
        z ^= z >> np.uint64(30); z *= np.uint64(0xBF58476D1CE4E5B9)
        z ^= z >> np.uint64(27); z *= np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
    u = ((z >> np.uint64(40)).astype(np.float64) + 0.5) * (1.0 / 16777216.0)
    return (lo + (hi - lo) * u).astype(np.float32)
