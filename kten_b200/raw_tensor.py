"""CUDARawTensor -- the device-resident RawTensor of the kten-cuda backend.

Host-side mirror of the reference's backend SPI class
`AbstractRawTensor<STORE>` (kten-api/.../tensor/store/AbstractRawTensor.kt:5-248)
for the float32 hot path, with the method names, argument meaning and error
behaviour of the JVM implementation
(backend/kten-jvm/.../tensor/store/JVMRawTensor.kt).  The storage is a
reference-counted buffer handle of libkten_cuda.so; shapes stay on the host;
every operation is one call through the C ABI that enqueues kernels on the
device's stream.  Structure (two ref-counts, one for the tensor object and one
for the storage shared by shallow copies and views) follows
backend/kten-opencl/.../store/OCLRawTensor.kt:21-48, 252-263.

Exceptions: IllegalArgumentException -> ValueError, IllegalStateException ->
RuntimeError.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _lib as L
from . import shape_functions as SF


class CUDARawTensor:
    __slots__ = ("shape", "storeReference", "ops", "refCount", "mustSurviveGC", "_released")

    def __init__(self, shape: Sequence[int], store: int, ops: "CUDATensorOperations"):
        self.shape: List[int] = [int(d) for d in shape]
        self.storeReference: int = store          # ktc_buf handle (holds one reference)
        self.ops = ops
        self.refCount = 1
        self.mustSurviveGC = False
        self._released = False
        ops._instance_created(self)

    # ---- bookkeeping -------------------------------------------------------
    @property
    def dimensions(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        return SF.to_store_size(self.shape)

    def _buf(self) -> int:
        if self._released:
            raise RuntimeError("Raw tensor already released")   # OCLMemoryObject.kt:167-170
        return self.storeReference

    def incrementRef(self) -> None:
        self.refCount += 1

    def release(self) -> bool:
        """OCLRawTensor.release (OCLRawTensor.kt:37-48): drop one reference; at zero
        the storage reference goes back to the library (and the pool)."""
        if self._released:
            return False
        if not self.mustSurviveGC:
            self.refCount -= 1
        if self.refCount <= 0:
            L.check(self.ops.lib.ktc_release(self.storeReference))
            self._released = True
            return True
        return False

    def _new(self, shape: Sequence[int]) -> "CUDARawTensor":
        return self.ops.createRaw(list(shape))

    # ---- host reads ----------------------------------------------------------
    def toArray(self) -> np.ndarray:
        """Blocking device-to-host read of the whole tensor (toSerializableData,
        TensorOperations.kt:133)."""
        n = self.size
        out = np.empty(n, dtype=np.float32)
        if n:
            L.check(self.ops.lib.ktc_d2h(out.ctypes.data_as(C.c_void_p), self._buf(), 0, n, 1))
        return out.reshape(self.shape)

    def getSingleValue(self, indexes: Sequence[int]) -> float:
        """AbstractRawTensor.getSingleValue (ART:166): one element, blocking."""
        if len(indexes) != len(self.shape):
            raise ValueError(f"Cannot index tensor with shape: {self.shape} with index: {list(indexes)}")
        off = 0
        for i, (idx, ext) in enumerate(zip(indexes, self.shape)):
            j = ext + idx if idx < 0 else idx
            if j < 0 or j >= ext:
                raise ValueError(f"Index {idx} is out of bounds for dimension {i} with size {ext}")
            off = off * ext + j
        out = (C.c_float * 1)()
        L.check(self.ops.lib.ktc_d2h(out, self._buf(), off, 1, 1))
        return float(out[0])

    def containsNan(self) -> bool:
        return bool(np.isnan(self.toArray()).any())

    # ---- elementwise: tensor (op) tensor ------------------------------------------
    def _binary(self, op: int, other: "CUDARawTensor") -> "CUDARawTensor":
        """elementwiseOpOnTensors (JVMRawTensor.kt:81-87) without materialising the
        broadcast operand."""
        if self.shape == other.shape:
            res = self._new(self.shape)
            L.check(self.ops.lib.ktc_binary(op, res._buf(), self._buf(), other._buf(), self.size))
            return res
        common = SF.infer_implicit_broadcast_shape(self.shape, other.shape)
        res = self._new(common)
        sa, na = L.shape_array(self.shape)
        sb, nb = L.shape_array(other.shape)
        L.check(self.ops.lib.ktc_binary_bcast(op, res._buf(), self._buf(), sa, na, other._buf(), sb, nb))
        return res

    def _binary_assign(self, op: int, other: "CUDARawTensor") -> None:
        """inplaceElementwiseOpOnTensors (JVMRawTensor.kt:89-97)."""
        if self.shape != other.shape:
            raise ValueError("Shapes does not match for inplace operation on tensors with shapes: "
                             f"{self.shape} and {other.shape}.")
        L.check(self.ops.lib.ktc_binary_inplace(op, self._buf(), other._buf(), self.size))

    def _scalar(self, op: int, s: float, scalar_first: bool = False) -> "CUDARawTensor":
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_scalar(op, res._buf(), self._buf(), float(s), self.size, 1 if scalar_first else 0))
        return res

    def _scalar_assign(self, op: int, s: float) -> None:
        L.check(self.ops.lib.ktc_scalar_inplace(op, self._buf(), float(s), self.size))

    def _unary(self, op: int) -> "CUDARawTensor":
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_unary(op, res._buf(), self._buf(), self.size))
        return res

    def plus(self, other):
        return self._binary(L.PLUS, other) if isinstance(other, CUDARawTensor) else self._scalar(L.PLUS, other)

    def plusAssign(self, other) -> None:
        if isinstance(other, CUDARawTensor):
            self._binary_assign(L.PLUS, other)
        else:
            self._scalar_assign(L.PLUS, other)

    def minus(self, other):
        return self._binary(L.MINUS, other) if isinstance(other, CUDARawTensor) else self._scalar(L.MINUS, other)

    def unaryMinus(self):
        return self._unary(L.NEG)

    def times(self, other):
        return self._binary(L.TIMES, other) if isinstance(other, CUDARawTensor) else self._scalar(L.TIMES, other)

    def timesAssign(self, other) -> None:
        if isinstance(other, CUDARawTensor):
            self._binary_assign(L.TIMES, other)
        else:
            self._scalar_assign(L.TIMES, other)

    def div(self, other):
        return self._binary(L.DIV, other) if isinstance(other, CUDARawTensor) else self._scalar(L.DIV, other)

    def divAssign(self, constant: float) -> None:
        self._scalar_assign(L.DIV, constant)

    def pow(self, other):
        return self._binary(L.POW, other) if isinstance(other, CUDARawTensor) else self._scalar(L.POW, other)

    def reciprocal(self):
        return self._unary(L.RECIPROCAL)

    def log(self):
        return self._unary(L.LOG)

    def exp(self):
        return self._unary(L.EXP)

    def tanh(self):
        return self._unary(L.TANH)

    def sigmoid(self):
        return self._unary(L.SIGMOID)

    def clamp(self, min: float, max: float):
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_clamp(res._buf(), self._buf(), float(min), float(max), self.size))
        return res

    def _compare(self, op: int, value: float):
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_compare_scalar(op, res._buf(), self._buf(), float(value), self.size))
        return res

    def lt(self, value: float):
        return self._compare(L.LT, value)

    def lte(self, value: float):
        return self._compare(L.LTE, value)

    def gt(self, value: float):
        return self._compare(L.GT, value)

    def gte(self, value: float):
        return self._compare(L.GTE, value)

    # ---- broadcast / copies / shape-only ops -------------------------------------------
    def broadcastTo(self, shape: Sequence[int]) -> "CUDARawTensor":
        """JVMRawTensor.broadcastTo (JVMRawTensor.kt:51-73): same shape returns this."""
        shape = [int(d) for d in shape]
        if self.shape == shape:
            return self
        SF.infer_explicit_broadcast_shape(self.shape, shape)
        res = self._new(shape)
        so, no = L.shape_array(shape)
        sa, na = L.shape_array(self.shape)
        L.check(self.ops.lib.ktc_broadcast_to(res._buf(), so, no, self._buf(), sa, na))
        return res

    def copy(self, shallow: bool = False) -> "CUDARawTensor":
        """copy(shallow) (JVMRawTensor.kt:257-262; OCLRawTensor.kt:252-258): a shallow
        copy shares the storage (one more reference on the buffer)."""
        if shallow:
            L.check(self.ops.lib.ktc_retain(self._buf()))
            return CUDARawTensor(self.shape, self.storeReference, self.ops)
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_d2d(res._buf(), 0, self._buf(), 0, self.size))
        return res

    def view(self, shape: Sequence[int]) -> "CUDARawTensor":
        """view (JVMRawTensor.kt:264-268): same storage, new shape."""
        new_shape = SF.reshape(self.shape, shape)
        L.check(self.ops.lib.ktc_retain(self._buf()))
        return CUDARawTensor(new_shape, self.storeReference, self.ops)

    def reshape(self, shape: Sequence[int]) -> "CUDARawTensor":
        """reshape (ART:79-84): a deep copy with the new shape."""
        new_shape = SF.reshape(self.shape, shape)
        res = self.copy()
        res.shape = new_shape
        return res

    def inplaceReshape(self, shape: Sequence[int]) -> None:
        self.shape = SF.reshape(self.shape, shape)

    def inplaceSqueeze(self, axis: int) -> None:
        s = list(self.shape)
        del s[SF.normalize_axis(self.shape, axis)]
        self.shape = s

    def squeeze(self, axis: int):
        res = self.copy()
        res.inplaceSqueeze(axis)
        return res

    def inplaceUnsqueeze(self, axis: int) -> None:
        self.shape = SF.unsqueeze(self.shape, axis)

    def unsqueeze(self, axis: int):
        res = self.copy()
        res.inplaceUnsqueeze(axis)
        return res

    def inplaceFill(self, value: float) -> None:
        L.check(self.ops.lib.ktc_fill(self._buf(), 0, self.size, float(value)))

    # ---- reductions --------------------------------------------------------------
    def _aggregate(self, axis: int, keep_dimensions: bool, op: int) -> "CUDARawTensor":
        """aggregatingOpOverAxis (ART:92-108): the result is produced with the axis
        kept as extent 1 and the dimension dropped on the host afterwards."""
        a = SF.normalize_axis(self.shape, axis)
        res_shape = SF.aggregate_over(self.shape, a, True)
        outer, length, inner = SF.collapse_axis(self.shape, a)
        res = self._new(res_shape)
        L.check(self.ops.lib.ktc_reduce_axis(op, res._buf(), self._buf(), outer, length, inner))
        if not keep_dimensions and len(res_shape) > 1:
            del res_shape[a]
            res.shape = res_shape
        return res

    def sum(self, axis: Optional[int] = None, keepDimensions: bool = False):
        if axis is None:
            res = self._new([1])                     # sum() -> shape [1] (JVMRawTensor.kt:146-148)
            L.check(self.ops.lib.ktc_reduce_all(L.SUM, res._buf(), self._buf(), self.size))
            return res
        return self._aggregate(axis, keepDimensions, L.SUM)

    def mean(self, axis: Optional[int] = None, keepDimensions: bool = False):
        if axis is None:
            res = self._new([1])                     # mean() -> shape [1] (JVMRawTensor.kt:150-152)
            L.check(self.ops.lib.ktc_reduce_all(L.MEAN, res._buf(), self._buf(), self.size))
            return res
        return self._aggregate(axis, keepDimensions, L.MEAN)

    def max(self, axis: int, keepDimensions: bool = False):
        return self._aggregate(axis, keepDimensions, L.MAX)

    def min(self, axis: int, keepDimensions: bool = False):
        return self._aggregate(axis, keepDimensions, L.MIN)

    def argMax(self, axis: int = 0, keepDimensions: bool = False):
        return self._aggregate(axis, keepDimensions, L.ARGMAX)

    def argMin(self, axis: int = 0, keepDimensions: bool = False):
        return self._aggregate(axis, keepDimensions, L.ARGMIN)

    def maxWithIndices(self, axis: int, keepDimensions: bool = False, is_max: bool = True):
        """Value and index of max/min in one pass over the input (the merge the
        reference leaves as a TODO at AggregatingFunctions.kt:83-87)."""
        a = SF.normalize_axis(self.shape, axis)
        res_shape = SF.aggregate_over(self.shape, a, True)
        outer, length, inner = SF.collapse_axis(self.shape, a)
        val, idx = self._new(res_shape), self._new(res_shape)
        L.check(self.ops.lib.ktc_reduce_axis_validx(1 if is_max else 0, val._buf(), idx._buf(), self._buf(), outer, length, inner))
        if not keepDimensions and len(res_shape) > 1:
            s = list(res_shape)
            del s[a]
            val.shape, idx.shape = list(s), list(s)
        return val, idx

    def sumToShape(self, old_shape: Sequence[int]) -> "CUDARawTensor":
        """mayUnexpand in one call (autograd/functions/Utils.kt:14-41)."""
        old_shape = [int(d) for d in old_shape]
        res = self._new(old_shape)
        so, no = L.shape_array(old_shape)
        si, ni = L.shape_array(self.shape)
        L.check(self.ops.lib.ktc_sum_to_shape(res._buf(), so, no, self._buf(), si, ni))
        return res

    def inplaceScatter(self, axis: int, index: "CUDARawTensor", src: "CUDARawTensor") -> None:
        """inplaceScatter restricted to one index per position along `axis`
        (index/src extent 1 there): the Max/Min backward
        (AggregatingFunctions.kt:68-79; JVMRawTensor.kt:227-256)."""
        a = SF.normalize_axis(self.shape, axis)
        if len(index.shape) != len(self.shape) or len(src.shape) != len(self.shape):
            raise ValueError("Scatter expects tensors (target, index, source) to have the same dimensions, but got "
                             f"tensors with shapes: target: {self.shape}, index: {index.shape}, source: {src.shape}")
        if index.shape[a] != 1 or index.shape != src.shape:
            raise NotImplementedError("kten-cuda scatters one index per position along the axis (selection backward)")
        outer, length, inner = SF.collapse_axis(self.shape, a)
        L.check(self.ops.lib.ktc_scatter_axis(self._buf(), index._buf(), src._buf(), outer, length, inner))

    def __repr__(self) -> str:
        return f"CUDARawTensor(shape={self.shape}, buf=0x{self.storeReference:x}, refs={self.refCount})"
