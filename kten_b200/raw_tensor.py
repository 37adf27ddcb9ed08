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
from . import lazy
from . import shape_functions as SF


class _Cell:
    """Storage slot of one or more tensors: a buffer handle (one owned reference), or a cell of the
    library's expression recorder whose value is still pending, or both (the recorder cell then stands
    for the buffer when the tensor is an operand of a recorded call).  Shallow copies of a deferred
    tensor share the cell, so that they end up sharing storage exactly as in the reference; every other
    tensor has a cell of its own."""

    __slots__ = ("store", "lz", "lz_shape", "share", "rec", "__weakref__")

    def __init__(self, store, lz=None, lz_shape=None, rec=None):
        self.store, self.lz, self.lz_shape, self.share, self.rec = store, lz, lz_shape, 1, rec

    def __del__(self):
        # a tensor that was never released (an output its Function kept) still gives back its recorder cell, and
        # with it the operands its pending value holds, when the host object goes away
        if self.lz is not None and self.rec is not None:
            try:
                self.rec.free(self.lz)
            except Exception:
                pass


class CUDARawTensor:
    __slots__ = ("shape", "_cell", "ops", "refCount", "mustSurviveGC", "_released", "__weakref__")

    def __init__(self, shape: Sequence[int], store: Optional[int], ops: "CUDATensorOperations", lz=None, cell=None):
        self.shape: List[int] = [int(d) for d in shape]
        if cell is None:
            cell = _Cell(store, lz, list(self.shape) if lz is not None else None, ops._recorder)   # store: ktc_buf handle (one reference); None while deferred
        else:
            cell.share += 1
        self._cell = cell
        self.ops = ops
        self.refCount = 1
        self.mustSurviveGC = False
        self._released = False
        ops._instance_created(self)

    @property
    def _store(self) -> Optional[int]:
        return self._cell.store

    @_store.setter
    def _store(self, h) -> None:
        self._cell.store = h

    def _drop_recorded(self) -> None:
        """Forget the recorder cell (the tensor's value is about to be replaced by something the recorder does not see)."""
        cell = self._cell
        if cell.lz is not None:
            self.ops._recorder.free(cell.lz)
            cell.lz = cell.lz_shape = None

    # ---- bookkeeping -------------------------------------------------------
    @property
    def dimensions(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        return SF.to_store_size(self.shape)

    @property
    def isDeferred(self) -> bool:
        cell = self._cell
        return cell.store is None and cell.lz is not None and self.ops._recorder.is_pending(cell.lz)

    @property
    def storeReference(self) -> int:
        """The buffer handle; a deferred tensor is evaluated first."""
        return self._buf()

    def _buf(self) -> int:
        if self._released:
            raise RuntimeError("Raw tensor already released")   # OCLMemoryObject.kt:167-170
        cell = self._cell
        if cell.store is None:
            if cell.lz is None:
                raise RuntimeError("Raw tensor has no storage")
            cell.store = self.ops._recorder.buffer(cell.lz)     # evaluates the pending expression; one reference for this cell
        elif self.ops._pending_targets and cell.store in self.ops._pending_targets:
            self.ops._run_pending()                             # a `+= pending sum` update of this buffer is due
        return cell.store

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
            cell = self._cell
            cell.share -= 1
            if cell.share <= 0:
                if cell.store is not None:
                    L.check(self.ops.lib.ktc_release(cell.store))
                if cell.lz is not None:
                    self.ops._recorder.free(cell.lz)
                    cell.lz = None
            self._released = True
            return True
        return False

    def _new(self, shape: Sequence[int]) -> "CUDARawTensor":
        return self.ops.createRaw(list(shape))

    def _lz(self, apply_updates: bool = True) -> int:
        """This tensor as an operand of a recorded call: its recorder cell (a stored tensor gets one over its buffer).
        apply_updates = False leaves a recorded `+= pending sum` update of the buffer pending (the caller hands the
        cell to a recorder call that deals with it)."""
        if self._released:
            raise RuntimeError("Raw tensor already released")
        cell = self._cell
        if cell.store is None:
            return cell.lz
        if apply_updates and self.ops._pending_targets and cell.store in self.ops._pending_targets:
            self.ops._run_pending()
        if cell.lz is None or cell.lz_shape != self.shape:
            if cell.lz is not None:
                self.ops._recorder.free(cell.lz)
            cell.lz, cell.lz_shape = self.ops._recorder.leaf(cell.store, self.shape), list(self.shape)
        return cell.lz

    def _recorded(self, shape, lz: int) -> "CUDARawTensor":
        return CUDARawTensor(shape, None, self.ops, lz=lz)

    def _after_assign(self, state: int) -> None:
        """What an in-place call through the recorder left behind (ktc_lazy_assign_*)."""
        cell = self._cell
        if state == lazy.STATE_PENDING:
            if cell.store is not None:                          # the cell's value is pending now; its old buffer belongs to the recorder
                L.check(self.ops.lib.ktc_release(cell.store))
                cell.store = None
        elif state == lazy.STATE_UPDATE_RECORDED:
            self.ops._pending_targets.add(cell.store)
        # STATE_UPDATE_OF_ZEROED: the recorder gave the (pending) cell a buffer that receives 0 + sum; nothing to do here

    def _before_inplace_write(self) -> None:
        """Deferred tensors that read this buffer are evaluated before it changes."""
        if self._store is not None:
            self.ops._flush_dependents(self._store)

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
        """containsNan (JVMRawTensor.kt:520-522), evaluated on the device."""
        res = C.c_int(0)
        L.check(self.ops.lib.ktc_contains_nan(self._buf(), self.size, C.byref(res)))
        return bool(res.value)

    # ---- elementwise: tensor (op) tensor ------------------------------------------
    def _binary(self, op: int, other: "CUDARawTensor") -> "CUDARawTensor":
        """elementwiseOpOnTensors (JVMRawTensor.kt:81-87) without materialising the
        broadcast operand."""
        if self.ops.lazy:
            common = self.shape if self.shape == other.shape else SF.infer_implicit_broadcast_shape(self.shape, other.shape)
            return self._recorded(common, self.ops._recorder.binary(op, self._lz(), other._lz()))
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
        if self.ops.lazy:
            self._after_assign(self.ops._recorder.assign_binary(op, self._lz(), other._lz()))
            return
        self._before_inplace_write()
        L.check(self.ops.lib.ktc_binary_inplace(op, self._buf(), other._buf(), self.size))

    def _scalar(self, op: int, s: float, scalar_first: bool = False) -> "CUDARawTensor":
        if self.ops.lazy:
            return self._recorded(self.shape, self.ops._recorder.scalar(op, self._lz(), s, scalar_first))
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_scalar(op, res._buf(), self._buf(), float(s), self.size, 1 if scalar_first else 0))
        return res

    def _scalar_assign(self, op: int, s: float) -> None:
        if self.ops.lazy:
            self._after_assign(self.ops._recorder.assign_scalar(op, self._lz(), s))
            return
        self._before_inplace_write()
        L.check(self.ops.lib.ktc_scalar_inplace(op, self._buf(), float(s), self.size))

    def _unary(self, op: int) -> "CUDARawTensor":
        if self.ops.lazy and op in L.RECORDABLE_UNARY:          # the ops the fused expression kernels implement
            return self._recorded(self.shape, self.ops._recorder.unary(op, self._lz()))
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

    # the remaining unary maps (JVMRawTensor.kt:401-435)
    def sinh(self):
        return self._unary(L.SINH)

    def cosh(self):
        return self._unary(L.COSH)

    def abs(self):
        return self._unary(L.ABS)

    def sign(self):
        return self._unary(L.SIGN)

    def sqrt(self):
        return self._unary(L.SQRT)

    def sin(self):
        return self._unary(L.SIN)

    def cos(self):
        return self._unary(L.COS)

    def tan(self):
        return self._unary(L.TAN)

    def asin(self):
        return self._unary(L.ASIN)

    def acos(self):
        return self._unary(L.ACOS)

    def atan(self):
        return self._unary(L.ATAN)

    def floor(self):
        return self._unary(L.FLOOR)

    def ceil(self):
        return self._unary(L.CEIL)

    def round(self):
        return self._unary(L.ROUND)

    def trunc(self):
        return self._unary(L.TRUNC)

    def rsqrt(self):
        return self._unary(L.RSQRT)

    def clamp(self, min: float, max: float):
        if self.ops.lazy:
            return self._recorded(self.shape, self.ops._recorder.clamp(self._lz(), min, max))
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_clamp(res._buf(), self._buf(), float(min), float(max), self.size))
        return res

    def _compare(self, op: int, value: float):
        if self.ops.lazy:
            return self._recorded(self.shape, self.ops._recorder.compare_scalar(op, self._lz(), value))
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_compare_scalar(op, res._buf(), self._buf(), float(value), self.size))
        return res

    def _compare_any(self, op: int, other):
        """lt/lte/gt/gte/eq/neq with a constant (JVMRawTensor.kt:379-393) or with a tensor of the same
        shape (JVM:355-377: elementwiseOpOnCommonShapedTensors, no broadcasting)."""
        if isinstance(other, CUDARawTensor):
            if self.shape != other.shape:
                raise ValueError(f"Tensor compare needs equal shapes, got {self.shape} and {other.shape}")
            res = self._new(self.shape)
            L.check(self.ops.lib.ktc_compare_tensor(op, res._buf(), self._buf(), other._buf(), self.ops.epsilon, self.size))
            return res
        if op in (L.EQ, L.NEQ):
            res = self._new(self.shape)
            L.check(self.ops.lib.ktc_compare_scalar_eps(op, res._buf(), self._buf(), float(other), self.ops.epsilon, self.size))
            return res
        return self._compare(op, other)

    def lt(self, other):
        return self._compare_any(L.LT, other)

    def lte(self, other):
        return self._compare_any(L.LTE, other)

    def gt(self, other):
        return self._compare_any(L.GT, other)

    def gte(self, other):
        return self._compare_any(L.GTE, other)

    def eq(self, other):
        return self._compare_any(L.EQ, other)

    def neq(self, other):
        return self._compare_any(L.NEQ, other)

    def maskedFill(self, mask: "CUDARawTensor", value: float) -> "CUDARawTensor":
        """maskedFill (JVMRawTensor.kt:537-540): the mask is broadcast to this shape (never materialised)."""
        SF.infer_explicit_broadcast_shape(mask.shape, self.shape)
        res = self._new(self.shape)
        sa, na = L.shape_array(self.shape)
        sm, nm = L.shape_array(mask.shape)
        L.check(self.ops.lib.ktc_masked_fill(res._buf(), self._buf(), sa, na, mask._buf(), sm, nm, float(value)))
        return res

    # ---- broadcast / copies / shape-only ops -------------------------------------------
    def broadcastTo(self, shape: Sequence[int]) -> "CUDARawTensor":
        """JVMRawTensor.broadcastTo (JVMRawTensor.kt:51-73): same shape returns this."""
        shape = [int(d) for d in shape]
        if self.shape == shape:
            return self
        SF.infer_explicit_broadcast_shape(self.shape, shape)
        if self.ops.lazy:
            return self._recorded(shape, self.ops._recorder.broadcast_to(self._lz(), shape))
        res = self._new(shape)
        so, no = L.shape_array(shape)
        sa, na = L.shape_array(self.shape)
        L.check(self.ops.lib.ktc_broadcast_to(res._buf(), so, no, self._buf(), sa, na))
        return res

    def copy(self, shallow: bool = False) -> "CUDARawTensor":
        """copy(shallow) (JVMRawTensor.kt:257-262; OCLRawTensor.kt:252-258): a shallow
        copy shares the storage (one more reference on the buffer)."""
        if shallow:
            if self.isDeferred:                                 # aliases share the pending value, later its storage
                return CUDARawTensor(self.shape, None, self.ops, cell=self._cell)
            L.check(self.ops.lib.ktc_retain(self._buf()))
            return CUDARawTensor(self.shape, self._store, self.ops)
        if self.isDeferred:                                     # pending values are immutable: a deep copy can share one
            return self._recorded(self.shape, self.ops._recorder.broadcast_to(self._lz(), self.shape))
        res = self._new(self.shape)
        L.check(self.ops.lib.ktc_d2d(res._buf(), 0, self._buf(), 0, self.size))
        return res

    def view(self, shape: Sequence[int]) -> "CUDARawTensor":
        """view (JVMRawTensor.kt:264-268): same storage, new shape."""
        new_shape = SF.reshape(self.shape, shape)
        L.check(self.ops.lib.ktc_retain(self._buf()))
        return CUDARawTensor(new_shape, self._store, self.ops)

    def reshape(self, shape: Sequence[int]) -> "CUDARawTensor":
        """reshape (ART:79-84): a deep copy with the new shape."""
        new_shape = SF.reshape(self.shape, shape)
        res = self.copy()
        res._buf()                                              # a pending expression is tied to its shape
        res.shape = new_shape
        return res

    def inplaceReshape(self, shape: Sequence[int]) -> None:
        self._buf()                                             # a deferred expression is tied to its shape
        self.shape = SF.reshape(self.shape, shape)

    def inplaceSqueeze(self, axis: int) -> None:
        self._buf()
        s = list(self.shape)
        del s[SF.normalize_axis(self.shape, axis)]
        self.shape = s

    def squeeze(self, axis: int):
        res = self.copy()
        res.inplaceSqueeze(axis)
        return res

    def inplaceUnsqueeze(self, axis: int) -> None:
        self._buf()
        self.shape = SF.unsqueeze(self.shape, axis)

    def unsqueeze(self, axis: int):
        res = self.copy()
        res.inplaceUnsqueeze(axis)
        return res

    def inplaceFill(self, value: float) -> None:
        if self.ops.lazy and (self._cell.store is not None or self._cell.lz is not None):
            # recorded: a pending tensor, or a stored one whose buffer nobody else holds, becomes a pending constant
            # (zeroGrad before a backward pass costs no kernel and no traffic); others are filled at once
            self._after_assign(self.ops._recorder.assign_fill(self._lz(), value))
            return
        if self.isDeferred:                                     # the pending value is overwritten: just take storage
            self._drop_recorded()
            h = C.c_uint64(0)
            L.check(self.ops.lib.ktc_alloc(self.ops.device, self.size, C.byref(h)))
            self._store = h.value
        self._before_inplace_write()
        L.check(self.ops.lib.ktc_fill(self._buf(), 0, self.size, float(value)))

    # ---- reductions --------------------------------------------------------------
    def _aggregate(self, axis: int, keep_dimensions: bool, op: int) -> "CUDARawTensor":
        """aggregatingOpOverAxis (ART:92-108): the result is produced with the axis
        kept as extent 1 and the dimension dropped on the host afterwards."""
        a = SF.normalize_axis(self.shape, axis)
        res_shape = SF.aggregate_over(self.shape, a, True)
        outer, length, inner = SF.collapse_axis(self.shape, a)
        res = None
        if self.isDeferred and op == L.SUM and a == 0 and len(self.shape) >= 2:
            final = list(res_shape) if keep_dimensions else list(res_shape[1:])
            res = self._recorded(final, self.ops._recorder.sum(self._lz(), L.EXPR_SUM_ROWS, False, final))    # fused with the pending expression when possible
        elif self.isDeferred and op == L.SUM and a == len(self.shape) - 1 and len(self.shape) >= 2 and self.shape[a] > 1 and self.ops.deferSums:
            final = list(res_shape) if keep_dimensions else list(res_shape[:-1])
            res = self._recorded(final, self.ops._recorder.sum(self._lz(), L.EXPR_SUM_LAST, False, final))    # row sums: a pending sum over the last axis
        if res is None:
            res = self._new(res_shape)
            L.check(self.ops.lib.ktc_reduce_axis(op, res._buf(), self._buf(), outer, length, inner))
        res.shape = list(res_shape)
        if not keep_dimensions and len(res_shape) > 1:
            del res_shape[a]
            res.shape = res_shape
        return res

    def sum(self, axis: Optional[int] = None, keepDimensions: bool = False):
        if axis is None:
            if self.isDeferred:
                return self._recorded([1], self.ops._recorder.sum(self._lz(), L.EXPR_SUM_ALL, False, [1]))
            res = self._new([1])                     # sum() -> shape [1] (JVMRawTensor.kt:146-148)
            L.check(self.ops.lib.ktc_reduce_all(L.SUM, res._buf(), self._buf(), self.size))
            return res
        return self._aggregate(axis, keepDimensions, L.SUM)

    def mean(self, axis: Optional[int] = None, keepDimensions: bool = False):
        if axis is None:
            if self.isDeferred:
                return self._recorded([1], self.ops._recorder.sum(self._lz(), L.EXPR_SUM_ALL, True, [1]))
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

    def softmaxCrossEntropyForward(self, targets: "CUDARawTensor", lo: float, hi: float):
        """The forward of SoftmaxCrossEntropy (functions/nn/SoftmaxCrossEntropy.kt:40-59) on logits [rows, cols] in one
        pass: returns (softmax [rows, cols] -- the tensor the function saves for backward --, nll [rows]) with the bits of
        the eleven separate calls, or None where the one-pass kernel does not apply (the caller issues the calls)."""
        entry = getattr(self.ops.lib, "ktc_softmax_xent_forward", None)
        if entry is None or len(self.shape) != 2 or targets.size != self.shape[0]:
            return None
        rows, cols = self.shape
        if self.ops.lazy:
            # recorded: the kernel runs when the loss or the gradient is needed, and takes the recorded backward with it
            cells = self.ops._recorder.softmax_xent_forward(self._lz(), targets._lz(), lo, hi)
            if cells is not None:
                return self._recorded([rows, cols], cells[0]), self._recorded([rows], cells[1])
        softmax, nll = self._new([rows, cols]), self._new([rows])
        rc = entry(softmax._buf(), nll._buf(), self._buf(), targets._buf(), rows, cols, float(lo), float(hi))
        if rc == L.KTC_ENOTSUP:
            softmax.release(); nll.release()
            return None
        L.check(rc)
        return softmax, nll

    def softmaxCrossEntropyBackward(self, targets: "CUDARawTensor", rows: int):
        """The backward of SoftmaxCrossEntropy (functions/nn/SoftmaxCrossEntropy.kt:61-67) on the saved softmax (`self`):
        zerosLike, -1 scattered at the targets, `+= softmax`, `/= rows` as ONE program of ktc_expr_eval -- the same four
        operations with their own roundings, one pass instead of four.  None when the calls are recorded anyway (the
        recorder fuses them itself, and with the forward) or the program is declined: the caller issues the calls."""
        if self.ops.lazy or len(self.shape) != 2 or targets.size != self.shape[0] or self.shape[1] % 4:
            return None

        def ins(op, d=0, a=0, b=0, k=0):
            return op | d << 8 | a << 12 | b << 16 | k << 20

        # leaves: 0 the targets [rows, 1], 1 the softmax; immediates: 0f, -1f, rows
        code = [ins(L.X_CONST, 0, k=0), ins(L.X_LOAD, 1, k=0), ins(L.X_SCATC, 0, 0, 1, k=1), ins(L.X_LOAD, 1, k=1), ins(L.X_ADD, 0, 0, 1),
                ins(L.X_CONST, 1, k=2), ins(L.X_DIV, 0, 0, 1), ins(L.X_STORE, a=0, k=0)]
        n_rows, cols = self.shape
        grad = self._new([n_rows, cols])
        rc = self.ops.lib.ktc_expr_eval((C.c_uint32 * len(code))(*code), len(code), (C.c_float * 3)(0.0, -1.0, float(rows)), 3,
                                        (C.c_int64 * 2)(n_rows, cols), 2, (C.c_uint64 * 2)(targets._buf(), self._buf()),
                                        (C.c_int64 * 4)(n_rows, 1, n_rows, cols), 2, (C.c_uint64 * 1)(grad._buf()), 1, L.EXPR_STORE_ONLY, 0, 0)
        if rc == L.KTC_ENOTSUP:
            grad.release()
            return None
        L.check(rc)
        return grad

    def sumToShape(self, old_shape: Sequence[int]) -> "CUDARawTensor":
        """mayUnexpand in one call (autograd/functions/Utils.kt:14-41)."""
        old_shape = [int(d) for d in old_shape]
        res = self._new(old_shape)
        so, no = L.shape_array(old_shape)
        si, ni = L.shape_array(self.shape)
        L.check(self.ops.lib.ktc_sum_to_shape(res._buf(), so, no, self._buf(), si, ni))
        return res

    def inplaceScatter(self, axis: int, index: "CUDARawTensor", src) -> None:
        """inplaceScatter (JVMRawTensor.kt:227-251; with a constant: JVM:317-332).  One index per position
        along `axis` over the whole target -- the Max/Min backward (AggregatingFunctions.kt:68-79) -- takes a
        fully parallel kernel; every other form the general one."""
        if not isinstance(src, CUDARawTensor):
            a = SF.normalize_axis(self.shape, axis)
            if self.ops.lazy and a == len(self.shape) - 1 and list(index.shape) == self.shape[:-1] + [1] and self.shape[-1] > 1:
                # one index per row along the last axis (the `-1 at the target` of SoftmaxCrossEntropy.doBackward): recorded
                state = self.ops._recorder.assign_scatter_const(self._lz(), index._lz(), float(src))
                if state is not None:
                    self._after_assign(state)
                    return
            self._scatter_nd(L.SCATTER_CONST, axis, index, float(src))
            return
        a = SF.normalize_axis(self.shape, axis)
        if len(index.shape) != len(self.shape) or len(src.shape) != len(self.shape):
            raise ValueError("Scatter expects tensors (target, index, source) to have the same dimensions, but got "
                             f"tensors with shapes: target: {self.shape}, index: {index.shape}, source: {src.shape}")
        if index.shape[a] != 1 or index.shape != src.shape or index.shape[:a] + index.shape[a + 1:] != self.shape[:a] + self.shape[a + 1:]:
            self._scatter_nd(L.SCATTER_SET, axis, index, src)       # several positions along the axis / smaller index
            return
        outer, length, inner = SF.collapse_axis(self.shape, a)
        self._buf()
        self._before_inplace_write()
        L.check(self.ops.lib.ktc_scatter_axis(self._buf(), index._buf(), src._buf(), outer, length, inner))

    # ---- slices, permutes, gather / scatter (JVMRawTensor.kt:227-353, 437-518) -----------------
    def _box(self, ranges):
        """(offset, box shape) of a normalised range index; trailing dimensions are taken whole."""
        st = SF.strides_of(self.shape)
        off = sum(f * st[d] for d, (f, _) in enumerate(ranges))
        return off, [l - f + 1 for f, l in ranges] + list(self.shape[len(ranges):]), st

    def get(self, index) -> "CUDARawTensor":
        """get(IntArray) / get(Array<IntRange>) (JVM:270-280): a copy of the addressed sub-tensor.  `index` is a
        sequence of ints, or of ranges (see shape_functions.as_range)."""
        index = list(index)
        if all(isinstance(i, (int, np.integer)) for i in index):
            norm, res_shape = SF.normalized_indexed_shape(self.shape, index)
            sub = SF.to_store_size(self.shape[len(norm):])
            start = 0
            for d, i in enumerate(norm):
                start = start * self.shape[d] + i
            res = self._new(res_shape)
            L.check(self.ops.lib.ktc_d2d(res._buf(), 0, self._buf(), start * sub, sub))
            return res
        norm, res_shape = SF.normalized_indexed_shape_ranges(self.shape, index)
        off, box, st = self._box(norm)
        res = self._new(res_shape)
        pb, nb = L.shape_array(box)
        ps, _ = L.shape_array(st)
        pd, _ = L.shape_array(SF.strides_of(box))
        L.check(self.ops.lib.ktc_copy_strided(res._buf(), 0, pd, self._buf(), off, ps, pb, nb))
        return res

    def set(self, index, value) -> None:
        """set(index, tensor | constant) (JVM:282-315): the value tensor is taken in store order and only its
        element count has to match the addressed box."""
        index = list(index)
        if all(isinstance(i, (int, np.integer)) for i in index):
            norm = SF.normalize_index(self.shape, index)
            ranges = [(i, i) for i in norm]
        else:
            ranges = SF.normalize_index_ranges(self.shape, index)
        off, box, st = self._box(ranges)
        n = SF.to_store_size(box)
        self._buf()
        self._before_inplace_write()
        pb, nb = L.shape_array(box)
        ps, _ = L.shape_array(st)
        if isinstance(value, CUDARawTensor):
            if value.size != n:
                raise ValueError(f"Cannot set tensor with shape: {value.shape} to tensor with shape: {self.shape} at index: {index}")
            pv, _ = L.shape_array(SF.strides_of(box))
            L.check(self.ops.lib.ktc_copy_strided(self._buf(), off, ps, value._buf(), 0, pv, pb, nb))
        else:
            L.check(self.ops.lib.ktc_fill_strided(self._buf(), off, ps, pb, nb, float(value)))

    def narrow(self, axis: int, start: int, length: int) -> "CUDARawTensor":
        """narrow (JVM:468-482)."""
        a = SF.normalize_axis(self.shape, axis)
        ranges = [(0, d - 1) for d in self.shape]
        ranges[a] = (start, start + length - 1)
        return self.get(ranges)

    def permute(self, axes: Sequence[int]) -> "CUDARawTensor":
        """permute (JVM:453-466): result dimension i is this tensor's dimension axes[i]."""
        axes = [int(a) for a in axes]
        new_shape = SF.permute(self.shape, axes)
        st = SF.strides_of(self.shape)
        res = self._new(new_shape)
        pb, nb = L.shape_array(new_shape)
        ps, _ = L.shape_array([st[a] for a in axes])
        pd, _ = L.shape_array(SF.strides_of(new_shape))
        L.check(self.ops.lib.ktc_copy_strided(res._buf(), 0, pd, self._buf(), 0, ps, pb, nb))
        return res

    def transpose(self, axis1: int, axis2: int) -> "CUDARawTensor":
        """transpose (JVM:437-451)."""
        _, a1, a2 = SF.transpose_normalize_axes(self.shape, axis1, axis2)
        axes = list(range(len(self.shape)))
        axes[a1], axes[a2] = a2, a1
        return self.permute(axes)

    def gather(self, axis: int, index: "CUDARawTensor") -> "CUDARawTensor":
        """gather (JVM:334-353): the result has the index's shape."""
        a = SF.normalize_axis(self.shape, axis)
        if len(index.shape) != len(self.shape):
            raise ValueError(f"Gather expects the index to have the tensor's dimensions, got {index.shape} for {self.shape}")
        res = self._new(index.shape)
        pi, n = L.shape_array(self.shape)
        px, _ = L.shape_array(index.shape)
        L.check(self.ops.lib.ktc_gather_axis(res._buf(), self._buf(), pi, index._buf(), px, n, a))
        return res

    def _scatter_nd(self, mode: int, axis: int, index: "CUDARawTensor", src) -> None:
        if mode == L.SCATTER_CONST:
            a = SF.normalize_axis(self.shape, axis)
            if len(index.shape) != len(self.shape):
                raise ValueError(f"Scatter expects the index to have the target's dimensions, got {index.shape} for {self.shape}")
        else:
            a = SF.normalized_axis_scatter(self.shape, axis, index.shape, src.shape)
        self._buf()
        self._before_inplace_write()
        pt, n = L.shape_array(self.shape)
        px, _ = L.shape_array(index.shape)
        if mode == L.SCATTER_CONST:
            L.check(self.ops.lib.ktc_scatter_axis_nd(mode, self._buf(), pt, index._buf(), px, 0, None, n, a, float(src)))
        else:
            ps, _ = L.shape_array(src.shape)
            L.check(self.ops.lib.ktc_scatter_axis_nd(mode, self._buf(), pt, index._buf(), px, src._buf(), ps, n, a, 0.0))

    def inplaceScatterAdd(self, axis: int, index: "CUDARawTensor", src: "CUDARawTensor") -> None:
        """inplaceScatterAdd (JVM:253-255)."""
        self._scatter_nd(L.SCATTER_ADD, axis, index, src)

    def scatter(self, axis: int, index: "CUDARawTensor", src) -> "CUDARawTensor":
        """scatter (AbstractRawTensor.kt: copy, then the in-place form); src is a tensor or a constant."""
        res = self.copy()
        res.inplaceScatter(axis, index, src)
        return res

    def scatterAdd(self, axis: int, index: "CUDARawTensor", src: "CUDARawTensor") -> "CUDARawTensor":
        res = self.copy()
        res.inplaceScatterAdd(axis, index, src)
        return res

    def indexSelect(self, axis: int, index: "CUDARawTensor") -> "CUDARawTensor":
        """indexSelect (JVM:484-502)."""
        a, res_shape = SF.index_select_norm_axis_shape(self.shape, axis, index.shape)
        outer, length, inner = SF.collapse_axis(self.shape, a)
        res = self._new(res_shape)
        L.check(self.ops.lib.ktc_index_select(res._buf(), self._buf(), index._buf(), outer, length, index.shape[0], inner))
        return res

    def indexAdd(self, axis: int, index: "CUDARawTensor", src: "CUDARawTensor", alpha: float = 1.0) -> None:
        """indexAdd (JVM:504-518)."""
        a = SF.index_add_check_shapes_norm_axis(self.shape, axis, index.shape, src.shape)
        outer, length, inner = SF.collapse_axis(self.shape, a)
        self._buf()
        self._before_inplace_write()
        L.check(self.ops.lib.ktc_index_add(self._buf(), index._buf(), src._buf(), float(alpha), outer, length, index.shape[0], inner))

    def inplaceResize(self, *shape) -> None:
        """inplaceResize (JVM:524-531): the store is copied into one of the new size (zero-padded or cut)."""
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        new_shape = [int(d) for d in shape]
        n_new, n_old = SF.to_store_size(new_shape), self.size
        old = self._buf()
        h = C.c_uint64(0)
        L.check(self.ops.lib.ktc_alloc(self.ops.device, n_new, C.byref(h)))
        keep = min(n_new, n_old)
        if keep:
            L.check(self.ops.lib.ktc_d2d(h.value, 0, old, 0, keep))
        if n_new > keep:
            L.check(self.ops.lib.ktc_fill(h.value, keep, n_new - keep, 0.0))
        self._before_inplace_write()
        L.check(self.ops.lib.ktc_release(old))
        self._drop_recorded()
        self._store = h.value
        self.shape = new_shape

    def __repr__(self) -> str:
        where = "deferred" if self.isDeferred else f"buf=0x{(self._store or 0):x}"
        return f"CUDARawTensor(shape={self.shape}, {where}, refs={self.refCount})"
