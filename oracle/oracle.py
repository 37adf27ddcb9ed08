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
float), 1 = exact (double accumulators, one narrowing).  Reductions are compared
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
(SINH, COSH, ABS, SIGN, SQRT, SIN, COS, TAN, ASIN, ACOS, ATAN, FLOOR, CEIL, ROUND, TRUNC, RSQRT) = range(6, 22)
LT, LTE, GT, GTE, EQ, NEQ = range(6)
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
        l.kto_compare_tensor.argtypes = [C.c_int, p_f32, p_f32, C.c_float, p_f32, C.c_int64]
        l.kto_compare_scalar.argtypes = [C.c_int, p_f32, C.c_float, C.c_float, p_f32, C.c_int64]
        l.kto_masked_fill.argtypes = [p_f32, p_i64, C.c_int, p_f32, p_i64, C.c_int, C.c_float, p_f32]
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


def binary(op: int, a, shape_a, b, shape_b, tuned: bool = False):
    """elementwiseOpOnTensors: returns (flat result, common shape).  `tuned`: the same values without the
    reference's materialised broadcast operands and on all host threads (host upper bound only)."""
    a, b = _flat(a), _flat(b)
    cs = common_shape(shape_a, shape_b)
    out = np.empty(volume(cs), dtype=np.float32)
    sa, na = _s(shape_a)
    sb, nb = _s(shape_b)
    fn = lib().kto_binary_bcast_tuned if tuned else lib().kto_binary_bcast
    _ok(fn(op, _f(a), sa, na, _f(b), sb, nb, _f(out)), "binary")
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


def compare(op: int, a, other, eps: float = 1e-7) -> np.ndarray:
    """lt/lte/gt/gte/eq/neq against a same-shape tensor or a constant (JVMRawTensor.kt:355-393)."""
    a = _flat(a)
    out = np.empty_like(a)
    if isinstance(other, np.ndarray):
        b = _flat(other)
        assert b.size == a.size
        lib().kto_compare_tensor(op, _f(a), _f(b), C.c_float(eps), _f(out), a.size)
    else:
        lib().kto_compare_scalar(op, _f(a), C.c_float(other), C.c_float(eps), _f(out), a.size)
    return out


def masked_fill(a, a_shape, mask, mask_shape, value: float) -> np.ndarray:
    a, mask = _flat(a), _flat(mask)
    out = np.empty_like(a)
    sa, na = _s(a_shape)
    sm, nm = _s(mask_shape)
    if lib().kto_masked_fill(_f(a), sa, na, _f(mask), sm, nm, C.c_float(value), _f(out)) != 0:
        raise ValueError(f"mask with shape {list(mask_shape)} cannot be broadcast to {list(a_shape)}")
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


def _SF():
    """The host shape algebra (a restatement of ShapeFunctions.kt) is shared with the backend's host side."""
    from kten_b200 import shape_functions
    return shape_functions


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
    # the remaining unary maps (JVMRawTensor.kt:401-435)
    def sinh(self): return self._wrap(unary(SINH, self.data))
    def cosh(self): return self._wrap(unary(COSH, self.data))
    def abs(self): return self._wrap(unary(ABS, self.data))
    def sign(self): return self._wrap(unary(SIGN, self.data))
    def sqrt(self): return self._wrap(unary(SQRT, self.data))
    def sin(self): return self._wrap(unary(SIN, self.data))
    def cos(self): return self._wrap(unary(COS, self.data))
    def tan(self): return self._wrap(unary(TAN, self.data))
    def asin(self): return self._wrap(unary(ASIN, self.data))
    def acos(self): return self._wrap(unary(ACOS, self.data))
    def atan(self): return self._wrap(unary(ATAN, self.data))
    def floor(self): return self._wrap(unary(FLOOR, self.data))
    def ceil(self): return self._wrap(unary(CEIL, self.data))
    def round(self): return self._wrap(unary(ROUND, self.data))
    def trunc(self): return self._wrap(unary(TRUNC, self.data))
    def rsqrt(self): return self._wrap(unary(RSQRT, self.data))

    def _cmp(self, op, other):
        # JVMRawTensor.kt:355-393: tensor compares need equal shapes (elementwiseOpOnCommonShapedTensors)
        if isinstance(other, OracleRawTensor):
            if self.shape != other.shape:
                raise ValueError(f"Tensor compare needs equal shapes, got {self.shape} and {other.shape}")
            return self._wrap(compare(op, self.data, other.data, self.ops.epsilon))
        return self._wrap(compare(op, self.data, float(other), self.ops.epsilon))

    def lt(self, o): return self._cmp(LT, o)
    def lte(self, o): return self._cmp(LTE, o)
    def gt(self, o): return self._cmp(GT, o)
    def gte(self, o): return self._cmp(GTE, o)
    def eq(self, o): return self._cmp(EQ, o)
    def neq(self, o): return self._cmp(NEQ, o)

    def maskedFill(self, mask, value):
        return self._wrap(masked_fill(self.data, self.shape, mask.data, mask.shape, value))

    def containsNan(self):
        return bool(np.isnan(self.data).any())                      # JVMRawTensor.kt:520-522

    # ---- slices, permutes, gather / scatter: index arithmetic restated with numpy ----------------
    def _nd(self):
        return self.data.reshape(self.shape)

    def view(self, shape):
        return self._wrap(self.data, _SF().reshape(self.shape, shape))    # JVM:264-268: same store

    def reshape(self, shape):
        return self._wrap(self.data.copy(), _SF().reshape(self.shape, shape))

    def inplaceReshape(self, shape):
        self.shape = _SF().reshape(self.shape, shape)

    def inplaceSqueeze(self, axis):
        s = list(self.shape)
        del s[_normalize_axis(self.shape, axis)]
        self.shape = s

    def squeeze(self, axis):
        res = self.copy()
        res.inplaceSqueeze(axis)
        return res

    def unsqueeze(self, axis):
        res = self.copy()
        res.inplaceUnsqueeze(axis)
        return res

    def get(self, index):
        """JVM:270-280: an IntArray addresses one contiguous store range, IntRanges a box."""
        SF = _SF()
        index = list(index)
        if all(isinstance(i, (int, np.integer)) for i in index):
            norm, res_shape = SF.normalized_indexed_shape(self.shape, index)
            return self._wrap(self._nd()[tuple(norm)].reshape(-1).copy(), res_shape)
        norm, res_shape = SF.normalized_indexed_shape_ranges(self.shape, index)
        return self._wrap(self._nd()[tuple(slice(f, l + 1) for f, l in norm)].reshape(-1).copy(), res_shape)

    def set(self, index, value):
        """JVM:282-315: the value is taken in store order; only its element count must match."""
        SF = _SF()
        index = list(index)
        if all(isinstance(i, (int, np.integer)) for i in index):
            sel = tuple(SF.normalize_index(self.shape, index))
        else:
            sel = tuple(slice(f, l + 1) for f, l in SF.normalize_index_ranges(self.shape, index))
        target = self._nd()
        box = target[sel]
        if isinstance(value, OracleRawTensor):
            if value.data.size != box.size:
                raise ValueError(f"Cannot set tensor with shape: {value.shape} to tensor with shape: {self.shape} at index: {index}")
            target[sel] = value.data.reshape(box.shape)
        else:
            target[sel] = np.float32(value)

    def narrow(self, axis, start, length):                          # JVM:468-482
        a = _normalize_axis(self.shape, axis)
        ranges = [(0, d - 1) for d in self.shape]
        ranges[a] = (start, start + length - 1)
        return self.get(ranges)

    def permute(self, axes):                                        # JVM:453-466: res dim i = this dim axes[i]
        new_shape = _SF().permute(self.shape, axes)
        return self._wrap(np.ascontiguousarray(np.transpose(self._nd(), axes)).reshape(-1), new_shape)

    def transpose(self, axis1, axis2):                              # JVM:437-451
        new_shape, a1, a2 = _SF().transpose_normalize_axes(self.shape, axis1, axis2)
        return self._wrap(np.ascontiguousarray(np.swapaxes(self._nd(), a1, a2)).reshape(-1), new_shape)

    def gather(self, axis, index):
        """JVM:334-353: res[c] = this[c with c[axis] = index[c]] for every position c of the index."""
        a = _normalize_axis(self.shape, axis)
        idx = index.data.reshape(index.shape).astype(np.int64)      # Float.toInt(): truncation
        if ((idx < 0) | (idx >= self.shape[a])).any():
            raise ValueError(f"Gather got invalid index, index value is out of bounds 0 and {self.shape[a]} at axis: {axis}")
        src = self._nd()[tuple(slice(0, d) if k != a else slice(None) for k, d in enumerate(index.shape))]
        return self._wrap(np.take_along_axis(src, idx, axis=a).reshape(-1).astype(np.float32), list(index.shape))

    def _scatter(self, axis, index, src, add):
        """internalInplaceScatter (JVM:227-247) / inplaceScatter(value) (JVM:317-332): sequential in the index
        position along the axis, so repeated indices resolve in that order."""
        const = not isinstance(src, OracleRawTensor)
        if const:
            a = _normalize_axis(self.shape, axis)
        else:
            a = _SF().normalized_axis_scatter(self.shape, axis, index.shape, src.shape)
        idx = index.data.reshape(index.shape).astype(np.int64)
        if ((idx < 0) | (idx >= self.shape[a])).any():
            raise ValueError(f"Scatter got invalid index, index value is out of bounds 0 and {self.shape[a]} at axis: {axis}")
        target = self._nd()
        other = [np.arange(d) for k, d in enumerate(index.shape) if k != a]
        grids = np.meshgrid(*other, indexing="ij") if other else []
        srcv = None if const else src.data.reshape(src.shape)
        for i in range(index.shape[a]):
            coords = list(grids)
            coords.insert(a, np.take(idx, i, axis=a))
            scoords = list(grids)
            scoords.insert(a, np.full_like(coords[a], i))
            if const:
                target[tuple(coords)] = np.float32(src)
            elif add:
                target[tuple(coords)] = target[tuple(coords)] + srcv[tuple(scoords)]
            else:
                target[tuple(coords)] = srcv[tuple(scoords)]

    def inplaceScatter(self, axis, index, src): self._scatter(axis, index, src, False)
    def inplaceScatterAdd(self, axis, index, src): self._scatter(axis, index, src, True)

    def scatter(self, axis, index, src):                            # AbstractRawTensor.kt:150-160
        res = self.copy()
        res.inplaceScatter(axis, index, src)
        return res

    def indexSelect(self, axis, index):                             # JVM:484-502
        a, res_shape = _SF().index_select_norm_axis_shape(self.shape, axis, index.shape)
        idx = index.data.astype(np.int64)
        if ((idx < 0) | (idx >= self.shape[a])).any():
            raise ValueError(f"Index select got invalid index, index value is out of bounds 0 and {self.shape[a]} at axis: {axis}")
        return self._wrap(np.ascontiguousarray(np.take(self._nd(), idx, axis=a)).reshape(-1), res_shape)

    def indexAdd(self, axis, index, src, alpha=1.0):                # JVM:504-518: k ascending, += src * alpha
        a = _SF().index_add_check_shapes_norm_axis(self.shape, axis, index.shape, src.shape)
        idx = index.data.astype(np.int64)
        if ((idx < 0) | (idx >= self.shape[a])).any():
            raise ValueError(f"Index Add got invalid index, index value is out of bounds 0 and {self.shape[a]} at axis: {axis}")
        target, srcv = self._nd(), src.data.reshape(src.shape)
        for k, j in enumerate(idx):
            sel_t = tuple(slice(None) if d != a else int(j) for d in range(len(self.shape)))
            sel_s = tuple(slice(None) if d != a else k for d in range(len(self.shape)))
            target[sel_t] = target[sel_t] + srcv[sel_s] * np.float32(alpha)

    def inplaceResize(self, *shape):                                # JVM:524-531
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        new = np.zeros(volume(shape), dtype=np.float32)
        keep = min(new.size, self.data.size)
        new[:keep] = self.data[:keep]
        self.data, self.shape = new, [int(d) for d in shape]

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
        self.epsilon = 1e-7                     # PlatformProvider.epsilon (PlatformProvider.kt:12)

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

    def batchNorm(self, axis, momentum, epsilon, training):
        return OracleBatchNorm(axis, momentum, epsilon, training, self)

    def upsample(self, upsampleType, scale):
        if upsampleType != "NEAREST":
            raise ValueError(f"unknown upsample type {upsampleType}")
        return OracleUpsample2DNearest(scale, self)

    def spatialPooling(self, kernel, padding, stride, dilation, options):
        return OracleSpatialPooling(kernel, padding, stride, dilation, options, self)

    def concat(self, axis, inputs):
        """AbstractJVMTensorOperations.kt:106-120: every input is set into its range of the result."""
        SF = _SF()
        res_shape = SF.concat_shapes([t.shape for t in inputs], axis)
        a = _normalize_axis(inputs[0].shape, axis)
        res = self.createRaw(res_shape)
        ranges = [(0, d - 1) for d in res_shape]
        last = 0
        for t in inputs:
            if t.shape[a] == 0:
                continue
            ranges[a] = (last, last + t.shape[a] - 1)
            res.set(ranges, t)
            last += t.shape[a]
        return res


# ---- nn operations that are reductions and broadcast maps (JVMBatchNorm.kt, JVMUpsample2DNearest.kt) ----------------
def _seq_sum(values: np.ndarray, mode: int) -> np.float32:
    """Sum in the order given: float32 sequential (mode 0, what the JVM loop does) or exact (mode 1: double)."""
    if values.size == 0:
        return np.float32(0.0)
    if mode == 0:
        return np.add.accumulate(values.astype(np.float32), dtype=np.float32)[-1]
    return np.float32(values.astype(np.float64).sum())


class OracleBatchNorm:
    """JVMBatchNorm.kt:9-167 restated: per index of `axis`, mean and inverse standard deviation over all other
    positions (two passes, float arithmetic per element), running statistics, scale and shift; the gradients of
    :88-165.  Sums follow the oracle's accumulation mode."""

    def __init__(self, axis, momentum, epsilon, training, ops):
        self.axis, self.training, self.ops = axis, training, ops
        self.momentum, self.epsilon = np.float32(momentum), np.float32(epsilon)

    def _split(self, shape):
        a = self.axis
        return volume(shape[:a]), shape[a], volume(shape[a + 1:])

    def calculateOutput(self, input, runningMean, runningVar, gamma, beta):
        outer, C, inner = self._split(input.shape)
        x = input.data.reshape(outer, C, inner)
        out = np.empty_like(x)
        cur_mean, cur_std = np.zeros(C, np.float32), np.zeros(C, np.float32)
        n = outer * inner
        one = np.float32(1.0)
        for c in range(C):
            xc = x[:, c, :].reshape(-1)                       # applyForAxis visits the positions in this order (:17-30)
            if self.training:
                mean = np.float32(_seq_sum(xc, self.ops.mode) / np.float32(n))
                cur_mean[c] = mean
                d = (xc - mean).astype(np.float32)
                ssq = _seq_sum((d * d).astype(np.float32), self.ops.mode)
                stdev = np.float32(0.0)
                if ssq != 0.0 or self.epsilon != 0.0:
                    stdev = np.float32(one / np.float32(np.sqrt(np.float32(np.float32(ssq / np.float32(n)) + self.epsilon))))
                cur_std[c] = stdev
                if runningMean is not None and runningVar is not None:
                    runningMean.data[c] = np.float32(self.momentum * mean) + np.float32(np.float32(one - self.momentum) * runningMean.data[c])
                    unbiased = np.float32(ssq / np.float32(n - 1))
                    runningVar.data[c] = np.float32(self.momentum * unbiased) + np.float32(np.float32(one - self.momentum) * runningVar.data[c])
            else:
                mean = runningMean.data[c]
                stdev = np.float32(one / np.float32(np.sqrt(np.float32(runningVar.data[c] + self.epsilon))))
            g = gamma.data[c] if gamma is not None else one
            b = beta.data[c] if beta is not None else np.float32(0.0)
            y = ((x[:, c, :] - mean).astype(np.float32) * stdev).astype(np.float32)
            out[:, c, :] = ((y * g).astype(np.float32) + b).astype(np.float32)
        mk = lambda v: OracleRawTensor([C], v, self.ops)
        return OracleRawTensor(list(input.shape), out.reshape(-1), self.ops), mk(cur_mean), mk(cur_std)

    def calculateGrads(self, input, runningMean, runningVar, currentMean, currentStd, gamma, gradOut, inRequiresGrad, gammaRequiresGrad, betaRequiresGrad):
        if not (inRequiresGrad or gammaRequiresGrad or betaRequiresGrad):
            return None, None, None
        outer, C, inner = self._split(input.shape)
        x = input.data.reshape(outer, C, inner)
        go = gradOut.data.reshape(outer, C, inner)
        n = outer * inner
        grad_in = np.empty_like(x) if inRequiresGrad else None
        grad_gamma = np.zeros(C, np.float32) if gammaRequiresGrad else None
        grad_beta = np.zeros(C, np.float32) if betaRequiresGrad else None
        for c in range(C):
            g = gamma.data[c] if gamma is not None else np.float32(1.0)
            if self.training:
                mean, stdev = currentMean.data[c], currentStd.data[c]
            else:
                mean = runningMean.data[c]
                stdev = np.float32(1.0 / np.sqrt(np.float64(np.float32(runningVar.data[c] + self.epsilon))))
            xc, gc = x[:, c, :].reshape(-1), go[:, c, :].reshape(-1)
            total = _seq_sum(gc, self.ops.mode)
            dot = _seq_sum(((xc - mean).astype(np.float32) * gc).astype(np.float32), self.ops.mode)
            if grad_in is not None:
                if self.training:
                    dps = np.float32(np.float32(np.float32(dot * stdev) * stdev) / np.float32(n))
                    gm = np.float32(total / np.float32(n))
                    base = ((x[:, c, :] - mean).astype(np.float32) * dps).astype(np.float32)
                    t = ((go[:, c, :] - gm).astype(np.float32) - base).astype(np.float32)
                    grad_in[:, c, :] = ((t * stdev).astype(np.float32) * g).astype(np.float32)
                else:
                    grad_in[:, c, :] = ((go[:, c, :] * stdev).astype(np.float32) * g).astype(np.float32)
            if grad_gamma is not None:
                grad_gamma[c] = np.float32(dot * stdev)
            if grad_beta is not None:
                grad_beta[c] = total
        wrap = lambda v, shape: None if v is None else OracleRawTensor(shape, v.reshape(-1), self.ops)
        return wrap(grad_in, list(input.shape)), wrap(grad_gamma, [C]), wrap(grad_beta, [C])


class OracleUpsample2DNearest:
    """JVMUpsample2DNearest.kt:9-79: every input pixel repeated scale x scale times; the gradient of an input pixel is
    the sum of its block, added in the loop order of :61-68."""

    def __init__(self, scale, ops):
        self.scale, self.ops = int(scale), ops

    @staticmethod
    def _check(shape):
        if len(shape) not in (3, 4):
            raise ValueError(f"2D Upsampling can only be applied to tensors with 3 or 4 dimensions, but got tensor with shape: {list(shape)}")

    def calculateOutputShape(self, shape):
        return list(shape[:-2]) + [shape[-2] * self.scale, shape[-1] * self.scale]

    def upsample(self, input):
        self._check(input.shape)
        s = self.scale
        x = input.data.reshape([-1] + list(input.shape[-2:]))
        out = np.repeat(np.repeat(x, s, axis=1), s, axis=2)
        return OracleRawTensor(self.calculateOutputShape(input.shape), np.ascontiguousarray(out).reshape(-1), self.ops)

    def calculateGrad(self, gradOut, inputShape):
        self._check(gradOut.shape)
        s = self.scale
        if len(inputShape) != len(gradOut.shape) or gradOut.shape[-2] % s or gradOut.shape[-1] % s \
                or [gradOut.shape[-2] // s, gradOut.shape[-1] // s] != list(inputShape[-2:]) or list(gradOut.shape[:-2]) != list(inputShape[:-2]):
            raise ValueError(f"2D Upsample output gradients shape: {list(gradOut.shape)} does not align with input tensor shape: {list(inputShape)} with scale: {s}")
        H, W = inputShape[-2], inputShape[-1]
        g = gradOut.data.reshape(-1, H, s, W, s)
        acc = np.zeros((g.shape[0], H, W), np.float32 if self.ops.mode == 0 else np.float64)
        for y in range(s):                                  # the column offset is the outer loop (:61-66)
            for xo in range(s):
                acc = (acc + g[:, :, xo, :, y]).astype(acc.dtype)
        return OracleRawTensor(list(inputShape), acc.astype(np.float32).reshape(-1), self.ops)


class OracleSpatialPooling:
    """JVMSpatialPoolingBase.kt:14-137 with JVMSpatialMaxPooling.kt:24-69 and JVMSpatialAvgPooling.kt:23-88: the loops of
    the reference over one plane, vectorised over the planes (every plane sees the same sequence of float operations
    as in the reference, so results are bit-identical to it).  `options` has the fields of PoolingOptions.kt:6-10."""

    def __init__(self, kernel, padding, stride, dilation, options, ops):
        self.kh, self.kw = int(kernel[0]), int(kernel[1])
        self.ph, self.pw = int(padding[0]), int(padding[1])
        self.sh, self.sw = int(stride[0]), int(stride[1])
        self.is_max = options.type == "MAX"
        self.dh, self.dw = (int(dilation[0]), int(dilation[1])) if self.is_max else (1, 1)
        self.useCeil, self.includePadding, self.ops = bool(options.useCeil), bool(options.includePadding), ops

    @staticmethod
    def size_on_floats(extent, dilation, kernel, padding, stride):       # PoolingOperation.kt:10-13
        f = np.float32
        return (f(extent) - (f(dilation) * (f(kernel) - f(1.0)) + f(1.0)) + f(2.0) * f(padding)) / f(stride) + f(1.0)

    def _geometry(self, input, gradOut=None, indices=None):
        if self.kh <= 0 or self.kw <= 0:
            raise ValueError("Kernel size should be greater than zero")
        if self.sh <= 0 or self.sw <= 0:
            raise ValueError("Stride should be greater than zero")
        if self.dh <= 0 or self.dw <= 0:
            raise ValueError("Dilation should be greater than zero")
        if len(input.shape) not in (3, 4):
            raise ValueError("Input must be 3D or 4D tensor")
        if self.ph > self.kh // 2 or self.pw > self.kw // 2:
            raise ValueError(f"Padding should be smaller than kernel size / 2, but got kernel: ({self.kh}, {self.kw}) and padding: ({self.ph}, {self.pw})")
        f = 1 if len(input.shape) == 4 else 0
        C_, H, W = input.shape[f], input.shape[f + 1], input.shape[f + 2]
        rnd = np.ceil if self.useCeil else np.floor
        OH = int(rnd(self.size_on_floats(H, self.dh, self.kh, self.ph, self.sh)))
        OW = int(rnd(self.size_on_floats(W, self.dw, self.kw, self.pw, self.sw)))
        if self.ph > 0 or self.pw > 0:
            if (OH - 1) * self.sh >= H + self.ph:
                OH -= 1
            if (OW - 1) * self.sw >= W + self.pw:
                OW -= 1
        if OH < 1 or OW < 1:
            raise ValueError(f"Calculated output size: {C_} x {OH} x {OW} is too small. Input size: {C_} x {H} x {W}")
        for t, what in ((gradOut, "gradient"), (indices, "indices")):
            if t is not None and (t.shape[f] != C_ or t.shape[f + 1] != OH or t.shape[f + 2] != OW):
                raise ValueError(f"Invalid {what} shape, {what} must have shape with (F x H x W) = {C_} x {OH} x {OW}, "
                                 f"but got {t.shape[f]} x {t.shape[f + 1]} x {t.shape[f + 2]}")
        return C_ * (input.shape[0] if f else 1), H, W, OH, OW, list(input.shape[:f + 1]) + [OH, OW]

    def _avg_window(self, i, j, H, W):
        h0, w0 = i * self.sh - self.ph, j * self.sw - self.pw
        h1, w1 = min(h0 + self.kh, H + self.ph), min(w0 + self.kw, W + self.pw)
        pool = (h1 - h0) * (w1 - w0)
        h0, w0, h1, w1 = max(h0, 0), max(w0, 0), min(h1, H), min(w1, W)
        return h0, h1, w0, w1, (pool if self.includePadding else (h1 - h0) * (w1 - w0))

    def updateOutput(self, input):
        P, H, W, OH, OW, out_shape = self._geometry(input)
        x = input.data.reshape(P, H, W)
        if self.is_max:
            best = np.full((P, OH, OW), -np.inf, np.float32)
            at = np.full((P, OH, OW), -1.0, np.float32)
            for i in range(OH):
                for j in range(OW):
                    h0, w0 = i * self.sh - self.ph, j * self.sw - self.pw
                    h1, w1 = min(h0 + (self.kh - 1) * self.dh + 1, H), min(w0 + (self.kw - 1) * self.dw + 1, W)
                    while h0 < 0:
                        h0 += self.dh
                    while w0 < 0:
                        w0 += self.dw
                    for y in range(h0, h1, self.dh):
                        for xx in range(w0, w1, self.dw):
                            v = x[:, y, xx]
                            win = v > best[:, i, j]                       # strict: NaN never wins, the first of equals stays
                            best[:, i, j] = np.where(win, v, best[:, i, j])
                            at[:, i, j] = np.where(win, np.float32(y * W + xx), at[:, i, j])
            return OracleRawTensor(out_shape, best.reshape(-1), self.ops), OracleRawTensor(out_shape, at.reshape(-1), self.ops)
        out = np.empty((P, OH, OW), np.float32)
        with np.errstate(divide="ignore", invalid="ignore"):
            for i in range(OH):
                for j in range(OW):
                    h0, h1, w0, w1, items = self._avg_window(i, j, H, W)
                    acc = np.zeros(P, np.float32)
                    for y in range(h0, h1):
                        for xx in range(w0, w1):
                            acc = acc + x[:, y, xx]                       # float32 + float32
                    out[:, i, j] = acc / np.float32(items)
        return OracleRawTensor(out_shape, out.reshape(-1), self.ops), None

    def calculateGradInput(self, input, gradOut, indices):
        P, H, W, OH, OW, _ = self._geometry(input, gradOut, indices)
        g = gradOut.data.reshape(P, OH, OW)
        gin = np.zeros((P, H * W), np.float32)
        planes = np.arange(P)
        if self.is_max:
            idx = indices.data.reshape(P, OH, OW).astype(np.int64)            # Float.toInt()
            for i in range(OH):
                for j in range(OW):
                    k = idx[:, i, j]
                    hit = k != -1
                    gin[planes[hit], k[hit]] = gin[planes[hit], k[hit]] + g[hit, i, j]
        else:
            gin3 = gin.reshape(P, H, W)
            with np.errstate(divide="ignore", invalid="ignore"):
                for i in range(OH):
                    for j in range(OW):
                        h0, h1, w0, w1, items = self._avg_window(i, j, H, W)
                        c = g[:, i, j] / np.float32(items)
                        for y in range(h0, h1):
                            for xx in range(w0, w1):
                                gin3[:, y, xx] = gin3[:, y, xx] + c
        return OracleRawTensor(list(input.shape), gin.reshape(-1), self.ops)
