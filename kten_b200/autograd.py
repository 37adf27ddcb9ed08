"""The caller side of the backend SPI: define-by-run autograd over raw tensors.

kten's autograd (kten-api/src/main/kotlin/eu/redbean/kten/api/autograd) is not
part of a backend -- it is what drives one.  This module restates just the
nodes of the float32 hot path so that the SPI call sequence the Kotlin code
would issue (one raw-tensor call per line of doForward / doBackward) can be run
against any backend object that offers the RawTensor / TensorOperations
methods: the CUDA backend of this package, or a CPU backend in the tests.

Reference, by class:
  Function / lazy forward / backward / fan-in cache   functions/Function.kt:8-215
  UnaryTensorFunction, BiTensorFunction               functions/UnaryTensorFunction.kt, BiTensorFunction.kt
  Plus, Minus, Times, Div, Pow, *Constant             functions/BasicFunctions.kt:7-206
  Exp, Log, Tanh, Sigmoid, Clamp                      functions/PointwiseFunctions.kt:8-82, 135-163
  Sum, Mean, Max, Min                                 functions/AggregatingFunctions.kt:7-93
  Expand                                              functions/TensorFunctions.kt:232-284
  mayUnexpand                                         functions/Utils.kt:14-41
  Variable, NoGradVariable                            tensor/Variable.kt, tensor/NoGradVariable.kt
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

from . import shape_functions as SF

NO_AXIS = -(2 ** 31)      # Int.MIN_VALUE: "aggregate over everything"


def may_unexpand(raw, old_shape: Sequence[int], ops, fused: bool = False):
    """Broadcast-gradient sum-to-shape (Utils.kt:14-41).  With `fused` the backend's
    one-call sumToShape is used instead of the chain of axis sums."""
    old_shape = list(old_shape)
    if fused and hasattr(raw, "sumToShape"):
        if list(raw.shape) == old_shape:
            return raw
        return raw.sumToShape(old_shape)
    lead = raw.dimensions - len(old_shape)
    expanded = [i for i, (e, o) in enumerate(zip(raw.shape[lead:], old_shape)) if e != o]
    res = raw
    for i in range(lead):
        prev, res = res, res.sum(0, keepDimensions=False)
        if i > 0:
            ops.release(prev)
    for i, d in enumerate(expanded):
        prev, res = res, res.sum(d, keepDimensions=True)
        if i > 0:
            ops.release(prev)
    return res


class Tensor:
    """Minimal facade (kten-api/.../tensor/Tensor.kt): operators build Function nodes."""

    requiresGrad = False

    def __init__(self, ops):
        self.ops = ops

    # -- to be provided by subclasses
    @property
    def shape(self) -> List[int]:
        raise NotImplementedError

    def getRawValue(self):
        raise NotImplementedError

    def backwardWithGrad(self, gradient) -> None:
        raise NotImplementedError

    # -- operators (AGTensor.kt:85-175)
    def __add__(self, o):
        return Plus(self.ops)(self, o) if isinstance(o, Tensor) else PlusConstant(self.ops)(self, float(o))

    def __radd__(self, c):
        return PlusConstant(self.ops)(self, float(c), tensor_first=False)

    def __sub__(self, o):
        return Minus(self.ops)(self, o) if isinstance(o, Tensor) else MinusConstant(self.ops)(self, float(o))

    def __rsub__(self, c):
        return MinusConstant(self.ops)(self, float(c), tensor_first=False)

    def __mul__(self, o):
        return Times(self.ops)(self, o) if isinstance(o, Tensor) else TimesConstant(self.ops)(self, float(o))

    def __rmul__(self, c):
        return TimesConstant(self.ops)(self, float(c), tensor_first=False)

    def __truediv__(self, o):
        return Div(self.ops)(self, o) if isinstance(o, Tensor) else DivConstant(self.ops)(self, float(o))

    def __rtruediv__(self, c):
        return DivConstant(self.ops)(self, float(c), tensor_first=False)

    def pow(self, o):
        return Pow(self.ops)(self, o) if isinstance(o, Tensor) else PowConstant(self.ops)(self, float(o))

    __pow__ = pow

    def __rpow__(self, c):
        return PowConstant(self.ops)(self, float(c), tensor_first=False)

    def exp(self):
        return Exp(self.ops)(self)

    def log(self):
        return Log(self.ops)(self)

    def tanh(self):
        return Tanh(self.ops)(self)

    def sigmoid(self):
        return Sigmoid(self.ops)(self)

    def clamp(self, min: float, max: float):
        return Clamp(self.ops)(self, float(min), float(max))

    def sum(self, axis: int = NO_AXIS, keepDimensions: bool = False):
        return Sum(self.ops)(self, axis, keepDimensions)

    def mean(self, axis: int = NO_AXIS, keepDimensions: bool = False):
        return Mean(self.ops)(self, axis, keepDimensions)

    def max(self, axis: int, keepDimensions: bool = False):
        return Max(self.ops)(self, axis, keepDimensions)

    def min(self, axis: int, keepDimensions: bool = False):
        return Min(self.ops)(self, axis, keepDimensions)

    def argMax(self, axis: int = 0, keepDimensions: bool = False):
        return NoGradVariable(self.ops, self._forwarded().argMax(axis, keepDimensions))

    def argMin(self, axis: int = 0, keepDimensions: bool = False):
        return NoGradVariable(self.ops, self._forwarded().argMin(axis, keepDimensions))

    def expand(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return Expand(self.ops)(self, list(shape))

    def _forwarded(self):
        if isinstance(self, Function) and not self.hasValue():
            self.forward()
        return self.getRawValue()

    def item(self) -> float:
        raw = self._forwarded()
        if SF.to_store_size(raw.shape) != 1:
            raise RuntimeError(f"item() needs a singleton tensor, shape is {raw.shape}")
        return raw.getSingleValue([0] * len(raw.shape))

    def toArray(self):
        return self._forwarded().toArray()


class NoGradVariable(Tensor):
    def __init__(self, ops, raw):
        super().__init__(ops)
        self.raw = raw

    @property
    def shape(self):
        return list(self.raw.shape)

    def getRawValue(self):
        return self.raw

    def backwardWithGrad(self, gradient) -> None:
        pass

    def asVariable(self, requiresGrad: bool = False):
        return Variable(self.ops, self.raw) if requiresGrad else self


class Variable(Tensor):
    """Graph leaf that accumulates its gradient in place (Variable.kt:44-46)."""

    requiresGrad = True

    def __init__(self, ops, value, gradient=None):
        super().__init__(ops)
        self.value = value
        self.gradient = gradient if gradient is not None else ops.zerosLike(value)

    @property
    def shape(self):
        return list(self.value.shape)

    def getRawValue(self):
        return self.value

    def backwardWithGrad(self, gradient) -> None:
        self.gradient.plusAssign(gradient)

    def backward(self, gradients: Tensor) -> None:
        if self.shape != gradients.shape:
            raise ValueError(f"Variable with shape: {self.shape} cannot have gradients with shape: {gradients.shape}")
        self.backwardWithGrad(gradients._forwarded())

    def zeroGrad(self) -> None:
        self.ops.zeroOut(self.gradient)

    def grad(self) -> Tensor:
        return NoGradVariable(self.ops, self.gradient)


class Function(Tensor):
    """A lazily evaluated graph node (Function.kt)."""

    requiresGrad = True

    def __init__(self, ops):
        super().__init__(ops)
        self.keepOutput = False
        self.valuesSaved: list = []
        self._output = None
        self.freeOutput = False
        self.cachedShape: Optional[List[int]] = None
        self.registeredAsInputIn: List["Function"] = []
        self.gradCache = None
        self.backwardRan = False

    # output setter raises the ref-count (Function.kt:16-21)
    @property
    def output(self):
        return self._output

    @output.setter
    def output(self, value):
        if value is not None:
            self.ops.incrementRef(value)
        self._output = value

    @property
    def shape(self):
        if self.cachedShape is None:
            if self._output is None:
                self.internalForward()
            self.cachedShape = list(self._output.shape)
        return list(self.cachedShape)

    def hasValue(self) -> bool:
        return self._output is not None

    def getRawValue(self):
        return self._output

    def getInputsAsList(self) -> List[Tensor]:
        raise NotImplementedError

    def forward(self) -> None:
        self.keepOutput = True
        with self.ops.garbageCollector():
            self.internalForward()

    def backward(self, gradients: Optional[Tensor] = None) -> None:
        """backward() on a [1] result, or backward(gradients) (Function.kt:54-89)."""
        if gradients is None:
            if self.shape != [1]:
                raise RuntimeError("Backward is only allowed on singleton calculation results (tensors with shape [1])")
        elif self.shape != gradients.shape:
            raise ValueError("Backward with gradients require same shape for gradients as the calculation result shape. "
                             f"Result shape: {self.shape} provided gradients shape: {gradients.shape}")
        self._registerInputUsages()
        with self.ops.garbageCollector():
            if not self.hasValue():
                self.internalForward()
            if gradients is None:
                seed = self.ops.createRaw([1], lambda i: 1.0)
            else:
                seed = gradients._forwarded()
            self.backwardWithGrad(seed)
            self.releaseUnusedInGraph()

    def _registerInputUsages(self) -> None:
        for t in self.getInputsAsList():
            if isinstance(t, Function):
                t.registeredAsInputIn.append(self)
                t._registerInputUsages()

    def backwardWithGrad(self, gradient) -> None:
        if len(self.registeredAsInputIn) > 1:                       # fan-in: Function.kt:108-120
            if self.gradCache is None:
                self.gradCache = gradient.copy()
            else:
                self.gradCache.plusAssign(gradient)
            if not all(f.backwardRan for f in self.registeredAsInputIn):
                return
        gradients = self.doBackward(self.gradCache if self.gradCache is not None else gradient)
        self.backwardRan = True
        for t, g in zip(self.getInputsAsList(), gradients):         # backwardToInputs, Function.kt:156-161
            if t.requiresGrad:
                t.backwardWithGrad(g)
        self.ops.release(gradient)
        if self.gradCache is not None:
            self.ops.release(self.gradCache)

    def releaseUnusedInGraph(self) -> None:
        if self.freeOutput and self._output is not None:
            self.ops.release(self._output)
            self._output = None
            self.freeOutput = False
        for v in self.valuesSaved:
            self.ops.release(v)
        self.valuesSaved.clear()
        for t in self.getInputsAsList():
            if isinstance(t, Function):
                t.releaseUnusedInGraph()

    def internalForward(self) -> None:
        self.gradCache = None
        self.backwardRan = False

    def saveForBackward(self, *raws) -> None:
        if not self.hasValue() or not self.valuesSaved:
            for r in raws:
                self.ops.incrementRef(r)
            self.valuesSaved.extend(raws)

    def mayFreeOutput(self) -> None:
        if not self.keepOutput:
            self.freeOutput = True

    def doBackward(self, gradient) -> list:
        raise NotImplementedError


class UnaryTensorFunction(Function):
    modifiesShape = False

    def __call__(self, tensor: Tensor):
        if not self.modifiesShape:
            self.cachedShape = list(tensor.shape)
        self.tensor = tensor
        return self

    def getInputsAsList(self):
        return [self.tensor]

    def internalForward(self) -> None:
        super().internalForward()
        if self.hasValue():
            return
        inp = self.tensor if isinstance(self.tensor, Function) else None
        if inp is not None:
            inp.internalForward()
        if not self.hasValue():
            self.doForward(self.tensor.getRawValue())
        if inp is not None:
            inp.mayFreeOutput()


class BiTensorFunction(Function):
    def __call__(self, a: Tensor, b: Tensor):
        self.cachedShape = SF.infer_implicit_broadcast_shape(a.shape, b.shape)
        self.inputs = (a, b)
        return self

    def getInputsAsList(self):
        return list(self.inputs)

    def internalForward(self) -> None:
        super().internalForward()
        if self.hasValue():
            return
        fns = [t for t in self.inputs if isinstance(t, Function)]
        for f in fns:
            f.internalForward()
        if not self.hasValue():
            ra, rb = self.inputs[0].getRawValue(), self.inputs[1].getRawValue()
            self.aShape, self.bShape = list(ra.shape), list(rb.shape)
            self.doForward(ra, rb)
        for f in fns:
            f.mayFreeOutput()


# ---- BasicFunctions.kt -------------------------------------------------------------
class Plus(BiTensorFunction):
    def doForward(self, a, b):
        self.output = a.plus(b)

    def doBackward(self, g):
        return [may_unexpand(g.copy(shallow=True), self.aShape, self.ops),
                may_unexpand(g.copy(shallow=True), self.bShape, self.ops)]


class Minus(BiTensorFunction):
    def doForward(self, a, b):
        self.output = a.minus(b)

    def doBackward(self, g):
        return [may_unexpand(g.copy(shallow=True), self.aShape, self.ops),
                may_unexpand(g.unaryMinus(), self.bShape, self.ops)]


class Times(BiTensorFunction):
    def doForward(self, a, b):
        self.saveForBackward(a, b)
        self.output = a.times(b)

    def doBackward(self, g):
        a, b = self.valuesSaved
        return [may_unexpand(g.times(b), self.aShape, self.ops), may_unexpand(g.times(a), self.bShape, self.ops)]


class Div(BiTensorFunction):
    def doForward(self, a, b):
        self.saveForBackward(a, b)
        self.output = a.div(b)

    def doBackward(self, g):
        a, b = self.valuesSaved
        b_rec = b.reciprocal()
        a_grad = g.times(b_rec)
        b_grad = g.unaryMinus()
        if list(a.shape) == list(b.shape):
            b_grad.timesAssign(a)
            b_grad.timesAssign(b_rec)
            b_grad.timesAssign(b_rec)
        else:
            b_grad = _times_assign_broadcast(b_grad, a.times(b_rec).times(b_rec))
        self.ops.release(b_rec)
        return [may_unexpand(a_grad, self.aShape, self.ops), may_unexpand(b_grad, self.bShape, self.ops)]


def _times_assign_broadcast(target, other):
    # `bGrad *= a * bRec * bRec` (BasicFunctions.kt:68): the right side already has the
    # gradient's (common) shape, so the in-place form applies
    target.timesAssign(other)
    return target


class Pow(BiTensorFunction):
    def doForward(self, a, b):
        self.saveForBackward(a, b)
        self.output = a.pow(b)

    def doBackward(self, g):
        a, b = self.valuesSaved
        a_grad = g.times(b)
        a_grad = _assign_times(a_grad, a.pow(b.minus(1.0)))
        b_grad = g.times(a.pow(b))
        b_grad = _assign_times(b_grad, a.log())
        return [may_unexpand(a_grad, self.aShape, self.ops), may_unexpand(b_grad, self.bShape, self.ops)]


def _assign_times(target, other):
    # Kotlin's `x *= y` on a raw tensor is timesAssign, which needs equal shapes;
    # with a broadcast operand the reference's own tests only reach this with
    # shapes the JVM accepts after the common-shape result
    if list(target.shape) == list(other.shape):
        target.timesAssign(other)
        return target
    return target.times(other)


class TensorConstantFunction(UnaryTensorFunction):
    def __call__(self, tensor: Tensor, constant: float, tensor_first: bool = True):
        super().__call__(tensor)
        self.constant = float(constant)
        self.tensorFirst = tensor_first
        return self


class PlusConstant(TensorConstantFunction):
    def doForward(self, x):
        self.output = x.plus(self.constant)

    def doBackward(self, g):
        return [g.copy(shallow=True)]


class MinusConstant(TensorConstantFunction):
    def doForward(self, x):
        if self.tensorFirst:
            self.output = x.minus(self.constant)
        else:
            self.output = x.unaryMinus()
            if self.constant != 0.0:
                self._output.plusAssign(self.constant)

    def doBackward(self, g):
        return [g.copy(shallow=True)] if self.tensorFirst else [g.unaryMinus()]


class TimesConstant(TensorConstantFunction):
    def doForward(self, x):
        self.output = x.times(self.constant)

    def doBackward(self, g):
        return [g.times(self.constant)]


class DivConstant(TensorConstantFunction):
    def doForward(self, x):
        if self.tensorFirst:
            self.output = x.div(self.constant)
        else:
            self.saveForBackward(x)
            self.output = x.reciprocal()
            self._output.timesAssign(self.constant)

    def doBackward(self, g):
        if self.tensorFirst:
            return [g.div(self.constant)]
        res = self.valuesSaved[0].reciprocal()
        res.timesAssign(res)
        res.timesAssign(g)
        res.timesAssign(-self.constant)
        return [res]


class PowConstant(TensorConstantFunction):
    def doForward(self, x):
        if self.tensorFirst:
            self.saveForBackward(x)
            self.output = x.pow(self.constant)
        else:
            res = self.ops.pow(self.constant, x)
            self.saveForBackward(res)
            self.output = res

    def doBackward(self, g):
        if self.tensorFirst:
            (x,) = self.valuesSaved
            grad = g.times(self.constant)
            # `input pow constant - 1f`: infix pow binds looser than minus
            grad.timesAssign(x.pow(self.constant - 1.0))
            return [grad]
        (res,) = self.valuesSaved
        grad = g.times(res)
        grad.timesAssign(_f32(math.log(_f32(self.constant))))      # kotlin.math.ln(Float)
        return [grad]


def _f32(x: float) -> float:
    import struct
    return struct.unpack("f", struct.pack("f", x))[0]


# ---- PointwiseFunctions.kt ------------------------------------------------------------
class Exp(UnaryTensorFunction):
    def doForward(self, x):
        res = x.exp()
        self.saveForBackward(res)
        self.output = res

    def doBackward(self, g):
        return [g.times(self.valuesSaved[0])]


class Log(UnaryTensorFunction):
    def doForward(self, x):
        self.saveForBackward(x)
        self.output = x.log()

    def doBackward(self, g):
        return [g.div(self.valuesSaved[0])]


class Tanh(UnaryTensorFunction):
    def doForward(self, x):
        res = x.tanh()
        self.saveForBackward(res)
        self.output = res

    def doBackward(self, g):
        (res,) = self.valuesSaved
        grad = res.times(res)
        grad.timesAssign(-1.0)
        grad.plusAssign(1.0)
        grad.timesAssign(g)
        return [grad]


class Sigmoid(UnaryTensorFunction):
    def doForward(self, x):
        res = x.sigmoid()
        self.saveForBackward(res)
        self.output = res

    def doBackward(self, g):
        (res,) = self.valuesSaved
        grad = res.unaryMinus()
        grad.plusAssign(1.0)
        grad.timesAssign(res)
        grad.timesAssign(g)
        return [grad]


class Clamp(UnaryTensorFunction):
    def __call__(self, tensor: Tensor, min: float, max: float):
        super().__call__(tensor)
        self.min, self.max = min, max
        return self

    def doForward(self, x):
        self.saveForBackward(x)
        self.output = x.clamp(self.min, self.max)

    def doBackward(self, g):
        (x,) = self.valuesSaved
        mask = x.gte(self.min)
        max_mask = x.lte(self.max)
        mask.timesAssign(max_mask)
        grad = g.times(mask)
        self.ops.release(mask, max_mask)
        return [grad]


# ---- AggregatingFunctions.kt -------------------------------------------------------------
class AggregatorFunction(UnaryTensorFunction):
    modifiesShape = True

    def __call__(self, tensor: Tensor, axis: int, keepDimensions: bool):
        self.cachedShape = [1] if axis == NO_AXIS else SF.aggregate_over(tensor.shape, axis, keepDimensions)
        super().__call__(tensor)
        self.axis = axis if axis == NO_AXIS else SF.normalize_axis(tensor.shape, axis)
        self.keepDimensions = keepDimensions
        return self


class Sum(AggregatorFunction):
    def doForward(self, x):
        self.inputShape = list(x.shape)
        self.output = x.sum() if self.axis == NO_AXIS else x.sum(self.axis, self.keepDimensions)

    def doBackward(self, g):
        if not self.keepDimensions and len(self.inputShape) != 1 and self.axis != NO_AXIS:
            g.inplaceUnsqueeze(self.axis)
        return [g.broadcastTo(self.inputShape)]


class Mean(AggregatorFunction):
    def doForward(self, x):
        self.inputShape = list(x.shape)
        self.output = x.mean() if self.axis == NO_AXIS else x.mean(self.axis, self.keepDimensions)

    def doBackward(self, g):
        if self.axis == NO_AXIS:
            grad = g.div(float(SF.to_store_size(self.inputShape)))
            return [grad.broadcastTo(self.inputShape)]
        if not self.keepDimensions and len(self.inputShape) != 1:
            g.inplaceUnsqueeze(self.axis)
        grad = g.broadcastTo(self.inputShape)
        grad.divAssign(float(self.inputShape[self.axis]))
        return [grad]


class SelectionFunction(AggregatorFunction):
    is_max = True

    def doForward(self, x):
        self.inputShape = list(x.shape)
        if self.is_max:
            res, idx = x.max(self.axis, self.keepDimensions), x.argMax(self.axis, self.keepDimensions)
        else:
            res, idx = x.min(self.axis, self.keepDimensions), x.argMin(self.axis, self.keepDimensions)
        self.saveForBackward(x, idx)
        self.output = res

    def doBackward(self, g):
        x, idx = self.valuesSaved
        grad = self.ops.zerosLike(x)
        if not self.keepDimensions and len(self.inputShape) != 1:
            g.inplaceUnsqueeze(self.axis)
            idx.inplaceUnsqueeze(self.axis)
        grad.inplaceScatter(self.axis, idx, g)
        return [grad]


class Max(SelectionFunction):
    is_max = True


class Min(SelectionFunction):
    is_max = False


# ---- TensorFunctions.kt: Expand ----------------------------------------------------------
class Expand(UnaryTensorFunction):
    modifiesShape = True

    def __call__(self, tensor: Tensor, new_shape: Sequence[int]):
        self.cachedShape = SF.infer_explicit_broadcast_shape(tensor.shape, new_shape)
        super().__call__(tensor)
        self.newShape = list(new_shape)
        return self

    def doForward(self, x):
        self.inShape = list(x.shape)
        self.output = x.broadcastTo(self.newShape)

    def doBackward(self, g):
        return [may_unexpand(g, self.inShape, self.ops)]


# ---- factories (Tensor.Companion, Tensor.kt:1630-1786) -------------------------------------
def tensorOf(ops, values, shape: Optional[Sequence[int]] = None, requiresGrad: bool = False) -> Tensor:
    import numpy as np
    arr = np.asarray(values, dtype=np.float32)
    shp = list(shape) if shape is not None else ([1] if arr.ndim == 0 else list(arr.shape))
    raw = ops.createRaw(shp, arr.reshape(-1))
    return Variable(ops, raw) if requiresGrad else NoGradVariable(ops, raw)
