"""Python face of the CPU oracle (libkten_oracle.so, built from kten_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline / reference legs of bench.py, never by the kten_b200 package.

Two layers:
  * thin numpy wrappers over the C functions (`binary`, `unary`, `aggregate`, ...);
  * `OracleRawTensor` / `OracleTensorOperations`, a CPU backend with the same
    RawTensor / TensorOperations methods as the CUDA backend, following
    kten-jvm (backend/kten-jvm/.../store/JVMRawTensor.kt and
    .../operations/AbstractJVMTensorOperations.kt) call for call, so that the
    autograd caller can be run on both and compared.

`mode`: 0 = jvm-faithful accumulation (float, axis order; sum() sequential
float), 1 = exact (double accumulators, one narrowing).  Reductions are judged
against mode 1; mode 0 is what kten-jvm itself would print.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import List, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkten_oracle.so")

PLUS, MINUS, TIMES, DIV, POW = range(5)
EXP, LOG, TANH, SIGMOID, RECIPROCAL, NEG = range(6)
SUM, MEAN, MAX, MIN, ARGMAX, ARGMIN = range(6)

_lib = None
p_f32 = C.POINTER(C.c_float)
p_i64 = C.POINTER(C.c_int64)


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "kten_oracle.cpp")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B" if force else "-s", "libkten_oracle.so"], check=True,
                       capture_output=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        l = C.CDLL(LIB_PATH)
        l.kto_common_shape.argtypes = [p_i64, C.c_int, p_i64, C.c_int, p_i64, C.POINTER(C.c_int)]
        l.kto_broadcast_to.argtypes = [p_f32, p_i64, C.c_int, p_i64, C.c_int, p_f32]
        l.kto_binary_same.argtypes = [C.c_int, p_f32, p_f32, p_f32, C.c_int64, C.c_int]
        l.kto_binary_bcast.argtypes = [C.c_int, p_f32, p_i64, C.c_int, p_f32, p_i64, C.c_int, p_f32]
        l.kto_binary_inplace.argtypes = [C.c_int, p_f32, p_f32, C.c_int64]
        l.kto_scalar.argtypes = [C.c_int, p_f32, C.c_float, C.c_int, p_f32, C.c_int64, C.c_int]
        l.kto_scalar_inplace.argtypes = [C.c_int, p_f32, C.c_float, C.c_int64]
        l.kto_unary.argtypes = [C.c_int, p_f32, p_f32, C.c_int64, C.c_int]
        l.kto_clamp.argtypes = [p_f32, C.c_float, C.c_float, p_f32, C.c_int64, C.c_int]
        l.kto_fill.argtypes = [p_f32, C.c_float, C.c_int64]
        l.kto_aggregate_axis.argtypes = [C.c_int, p_f32, C.c_int64, C.c_int64, C.c_int64, p_f32, C.c_int]
        l.kto_reduce_all.argtypes = [C.c_int, p_f32, C.c_int64, p_f32, C.c_int]
        l.kto_abs_sum.argtypes = [p_f32, C.c_int64]
        l.kto_abs_sum.restype = C.c_double
        l.kto_sum_to_shape.argtypes = [p_f32, p_i64, C.c_int, p_i64, C.c_int, p_f32, C.c_int]
        l.kto_num_threads.restype = C.c_int
        _lib = l
    return _lib


def _f(a: np.ndarray):
    return a.ctypes.data_as(p_f32)


def _s(shape: Sequence[int]):
    return (C.c_int64 * max(len(shape), 1))(*[int(d) for d in shape]), len(shape)


def _flat(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32).reshape(-1))


def _ok(rc: int, what: str):
    if rc != 0:
        raise ValueError(f"oracle: {what} rejected its arguments")


def volume(shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def common_shape(sa: Sequence[int], sb: Sequence[int]) -> List[int]:
    a, na = _s(sa)
    b, nb = _s(sb)
    out = (C.c_int64 * 16)()
    n = C.c_int(0)
    _ok(lib().kto_common_shape(a, na, b, nb, out, C.byref(n)), "common_shape")
    return [int(out[i]) for i in range(n.value)]


def broadcast_to(a, shape_a: Sequence[int], target: Sequence[int]) -> np.ndarray:
    a = _flat(a)
    out = np.empty(volume(target), dtype=np.float32)
    sa, na = _s(shape_a)
    st, nt = _s(target)
    _ok(lib().kto_broadcast_to(_f(a), sa, na, st, nt, _f(out)), "broadcast_to")
    return out


def binary(op: int, a, shape_a, b, shape_b):
    """elementwiseOpOnTensors: returns (flat result, common shape)."""
    a, b = _flat(a), _flat(b)
    cs = common_shape(shape_a, shape_b)
    out = np.empty(volume(cs), dtype=np.float32)
    sa, na = _s(shape_a)
    sb, nb = _s(shape_b)
    _ok(lib().kto_binary_bcast(op, _f(a), sa, na, _f(b), sb, nb, _f(out)), "binary")
    return out, cs


def binary_same(op: int, a, b, tuned: bool = False) -> np.ndarray:
    a, b = _flat(a), _flat(b)
    out = np.empty_like(a)
    lib().kto_binary_same(op, _f(a), _f(b), _f(out), a.size, int(tuned))
    return out


def binary_inplace(op: int, a: np.ndarray, b) -> None:
    b = _flat(b)
    lib().kto_binary_inplace(op, _f(a), _f(b), a.size)


def scalar(op: int, a, s: float, scalar_first: bool = False, tuned: bool = False) -> np.ndarray:
    a = _flat(a)
    out = np.empty_like(a)
    lib().kto_scalar(op, _f(a), C.c_float(s), int(scalar_first), _f(out), a.size, int(tuned))
    return out


def scalar_inplace(op: int, a: np.ndarray, s: float) -> None:
    lib().kto_scalar_inplace(op, _f(a), C.c_float(s), a.size)


def unary(op: int, a, tuned: bool = False) -> np.ndarray:
    a = _flat(a)
    out = np.empty_like(a)
    lib().kto_unary(op, _f(a), _f(out), a.size, int(tuned))
    return out


def clamp(a, lo: float, hi: float, tuned: bool = False) -> np.ndarray:
    a = _flat(a)
    out = np.empty_like(a)
    lib().kto_clamp(_f(a), C.c_float(lo), C.c_float(hi), _f(out), a.size, int(tuned))
    return out


def aggregate(op: int, a, outer: int, axis_len: int, inner: int, mode: int = 1) -> np.ndarray:
    a = _flat(a)
    assert a.size == outer * axis_len * inner
    out = np.empty(outer * inner, dtype=np.float32)
    _ok(lib().kto_aggregate_axis(op, _f(a), outer, axis_len, inner, _f(out), mode), "aggregate")
    return out


def reduce_all(op: int, a, mode: int = 1) -> np.float32:
    a = _flat(a)
    out = np.empty(1, dtype=np.float32)
    lib().kto_reduce_all(op, _f(a), a.size, _f(out), mode)
    return out[0]


def abs_sum(a) -> float:
    a = _flat(a)
    return float(lib().kto_abs_sum(_f(a), a.size))


def sum_to_shape(a, in_shape: Sequence[int], old_shape: Sequence[int], mode: int = 1) -> np.ndarray:
    a = _flat(a)
    out = np.empty(volume(old_shape), dtype=np.float32)
    si, ni = _s(in_shape)
    so, no = _s(old_shape)
    _ok(lib().kto_sum_to_shape(_f(a), si, ni, so, no, _f(out), mode), "sum_to_shape")
    return out


def num_threads() -> int:
    return int(lib().kto_num_threads())


def ulp_distance(a, b) -> np.ndarray:
    """Distance in units in the last place between float32 arrays (NaN == NaN -> 0,
    NaN vs number -> 2^32)."""
    a = np.asarray(a, dtype=np.float32).reshape(-1)
    b = np.asarray(b, dtype=np.float32).reshape(-1)
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7fffffff), ia)
    ib = np.where(ib < 0, -(ib & 0x7fffffff), ib)
    d = np.abs(ia - ib)
    na, nb = np.isnan(a), np.isnan(b)
    d = np.where(na & nb, 0, d)
    d = np.where(na ^ nb, 2 ** 32, d)
    return d


# ---------------------------------------------------------------------------
# CPU backend with the RawTensor / TensorOperations methods (kten-jvm restated)
# ---------------------------------------------------------------------------
def _normalize_axis(shape, axis):
    r = len(shape) + axis if axis < 0 else axis
    if r < 0 or r >= len(shape):
        raise ValueError(f"Cannot address axis: {axis} in tensor with dimensions: {len(shape)}")
    return r


class OracleRawTensor:
    def __init__(self, shape, data: np.ndarray, ops: "OracleTensorOperations"):
        self.shape = [int(d) for d in shape]
        self.data = data                      # flat float32, may be shared by shallow copies
        self.ops = ops

    @property
    def dimensions(self):
        return len(self.shape)

    def _wrap(self, data, shape=None):
        return OracleRawTensor(self.shape if shape is None else shape, data, self.ops)

    def toArray(self):
        return self.data.reshape(self.shape).copy()

    def getSingleValue(self, indexes):
        return float(self.data.reshape(self.shape)[tuple(indexes)])

    def _bin(self, op, other):
        if isinstance(other, OracleRawTensor):
            out, cs = binary(op, self.data, self.shape, other.data, other.shape)
            return self._wrap(out, cs)
        return self._wrap(scalar(op, self.data, float(other)))

    def _bin_assign(self, op, other):
        if isinstance(other, OracleRawTensor):
            if self.shape != other.shape:
                raise ValueError("Shapes does not match for inplace operation on tensors with shapes: "
                                 f"{self.shape} and {other.shape}.")
            binary_inplace(op, self.data, other.data)
        else:
            scalar_inplace(op, self.data, float(other))

    def plus(self, o): return self._bin(PLUS, o)
    def minus(self, o): return self._bin(MINUS, o)
    def times(self, o): return self._bin(TIMES, o)
    def div(self, o): return self._bin(DIV, o)
    def pow(self, o): return self._bin(POW, o)
    def plusAssign(self, o): self._bin_assign(PLUS, o)
    def timesAssign(self, o): self._bin_assign(TIMES, o)
    def divAssign(self, c): self._bin_assign(DIV, c)
    def unaryMinus(self): return self._wrap(unary(NEG, self.data))
    def reciprocal(self): return self._wrap(unary(RECIPROCAL, self.data))
    def log(self): return self._wrap(unary(LOG, self.data))
    def exp(self): return self._wrap(unary(EXP, self.data))
    def tanh(self): return self._wrap(unary(TANH, self.data))
    def sigmoid(self): return self._wrap(unary(SIGMOID, self.data))
    def clamp(self, min, max): return self._wrap(clamp(self.data, min, max))
    def gte(self, v): return self._wrap((self.data >= np.float32(v)).astype(np.float32))
    def lte(self, v): return self._wrap((self.data <= np.float32(v)).astype(np.float32))
    def gt(self, v): return self._wrap((self.data > np.float32(v)).astype(np.float32))
    def lt(self, v): return self._wrap((self.data < np.float32(v)).astype(np.float32))

    def broadcastTo(self, shape):
        shape = [int(d) for d in shape]
        if self.shape == shape:
            return self
        return self._wrap(broadcast_to(self.data, self.shape, shape), shape)

    def copy(self, shallow=False):
        return self._wrap(self.data if shallow else self.data.copy())

    def inplaceUnsqueeze(self, axis):
        n = len(self.shape)
        if axis != n:
            a = (0 if axis == -(n + 1) else _normalize_axis(self.shape, axis) + 1) if axis < 0 else _normalize_axis(self.shape, axis)
        else:
            a = axis
        s = list(self.shape)
        s.insert(a, 1)
        self.shape = s

    def inplaceFill(self, v):
        self.data[:] = np.float32(v)

    def _agg(self, op, axis, keep):
        a = _normalize_axis(self.shape, axis)
        outer, inner = volume(self.shape[:a]), volume(self.shape[a + 1:])
        out = aggregate(op, self.data, outer, self.shape[a], inner, self.ops.mode)
        res_shape = list(self.shape)
        res_shape[a] = 1
        if not keep and len(res_shape) > 1:
            del res_shape[a]
        return self._wrap(out, res_shape)

    def sum(self, axis=None, keepDimensions=False):
        if axis is None:
            return self._wrap(np.array([reduce_all(SUM, self.data, self.ops.mode)], dtype=np.float32), [1])
        return self._agg(SUM, axis, keepDimensions)

    def mean(self, axis=None, keepDimensions=False):
        if axis is None:
            return self._wrap(np.array([reduce_all(MEAN, self.data, self.ops.mode)], dtype=np.float32), [1])
        return self._agg(MEAN, axis, keepDimensions)

    def max(self, axis, keepDimensions=False): return self._agg(MAX, axis, keepDimensions)
    def min(self, axis, keepDimensions=False): return self._agg(MIN, axis, keepDimensions)
    def argMax(self, axis=0, keepDimensions=False): return self._agg(ARGMAX, axis, keepDimensions)
    def argMin(self, axis=0, keepDimensions=False): return self._agg(ARGMIN, axis, keepDimensions)

    def sumToShape(self, old_shape):
        return self._wrap(sum_to_shape(self.data, self.shape, old_shape, self.ops.mode), list(old_shape))

    def inplaceScatter(self, axis, index, src):
        # internalInplaceScatter (JVMRawTensor.kt:227-248) for index extent 1 along the axis
        a = _normalize_axis(self.shape, axis)
        outer, A, inner = volume(self.shape[:a]), self.shape[a], volume(self.shape[a + 1:])
        t = self.data.reshape(outer, A, inner)
        idx = index.data.reshape(outer, inner).astype(np.int64)
        if ((idx < 0) | (idx >= A)).any():
            raise ValueError(f"Scatter got invalid index, index value is out of bounds 0 and {A} at axis: {axis}")
        o, i = np.meshgrid(np.arange(outer), np.arange(inner), indexing="ij")
        t[o, idx, i] = src.data.reshape(outer, inner)


class _Scope:
    def __enter__(self): return self
    def __exit__(self, *exc): return False
    def close(self): pass


class OracleTensorOperations:
    """AbstractJVMTensorOperations restated: release / incrementRef / GC are no-ops
    (AbstractJVMTensorOperations.kt:73-92)."""

    platformKey = "ORACLE"

    def __init__(self, mode: int = 1):
        self.mode = mode

    def createRaw(self, shape, init=None):
        n = volume(shape)
        if init is None:
            data = np.zeros(n, dtype=np.float32)
        elif callable(init):
            data = np.fromiter((init(i) for i in range(n)), dtype=np.float32, count=n)
        else:
            data = _flat(init).copy()
        return OracleRawTensor(shape, data, self)

    def createRawFill(self, shape, constant):
        return OracleRawTensor(shape, np.full(volume(shape), constant, dtype=np.float32), self)

    def zerosLike(self, raw): return self.createRawFill(raw.shape, 0.0)
    def zeroOut(self, raw): raw.data[:] = 0.0
    def release(self, *raws): pass
    def incrementRef(self, raw): pass
    def markSurviveGC(self, raw): pass
    def markReleasableInGC(self, raw): pass
    def garbageCollector(self): return _Scope()

    def pow(self, constant, raw):
        return OracleRawTensor(raw.shape, scalar(POW, raw.data, float(constant), scalar_first=True), self)
