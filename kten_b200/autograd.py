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
  Sinh ... Rsqrt, Floor/Ceil/Round/Sign/Trunc         functions/PointwiseFunctions.kt:84-133, 165-360
  Index, IndexSet*, Transpose, Reshape, Permute,
  IndexSelect, Concat, Copy, Squeeze, Unsqueeze,
  Gather, Scatter, MaskedFill                         functions/TensorFunctions.kt:33-586
  get / set redirection after an in-place set         tensor/AGTensor.kt:24-83
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
        self._inplaceSafeThis = None

    def inplaceSafe(self):
        """AGTensor.inplaceSafe (AGTensor.kt:24-35): after `t[index] = value` every later use of t goes
        through the function node that performed the set."""
        return self._inplaceSafeThis if self._inplaceSafeThis is not None else self

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

    def __neg__(self):
        return 0.0 - self                                        # Tensor.unaryMinus (Tensor.kt:553-555)

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

    def sinh(self): return Sinh(self.ops)(self.inplaceSafe())
    def cosh(self): return Cosh(self.ops)(self.inplaceSafe())
    def abs(self): return Abs(self.ops)(self.inplaceSafe())
    def sign(self): return Sign(self.ops)(self.inplaceSafe())
    def sqrt(self): return Sqrt(self.ops)(self.inplaceSafe())
    def sin(self): return Sin(self.ops)(self.inplaceSafe())
    def cos(self): return Cos(self.ops)(self.inplaceSafe())
    def tan(self): return Tan(self.ops)(self.inplaceSafe())
    def asin(self): return Asin(self.ops)(self.inplaceSafe())
    def acos(self): return Acos(self.ops)(self.inplaceSafe())
    def atan(self): return Atan(self.ops)(self.inplaceSafe())
    def reciprocal(self): return Reciprocal(self.ops)(self.inplaceSafe())
    def floor(self): return Floor(self.ops)(self.inplaceSafe())
    def ceil(self): return Ceil(self.ops)(self.inplaceSafe())
    def round(self): return Round(self.ops)(self.inplaceSafe())
    def trunc(self): return Trunc(self.ops)(self.inplaceSafe())
    def rsqrt(self): return Rsqrt(self.ops)(self.inplaceSafe())

    # -- indexing and data movement (AGTensor.kt:61-83; Tensor.kt)
    @staticmethod
    def _is_int_index(index) -> bool:
        return all(isinstance(i, int) for i in index)

    def __getitem__(self, index):
        index = list(index) if isinstance(index, (tuple, list)) else [index]
        return Index(self.ops)(self.inplaceSafe(), index)

    def __setitem__(self, index, value):
        index = list(index) if isinstance(index, (tuple, list)) else [index]
        me = self.inplaceSafe()
        if isinstance(value, Tensor):
            self._inplaceSafeThis = IndexSetTensor(self.ops)(me, index, value.inplaceSafe())
        else:
            self._inplaceSafeThis = IndexSetConstant(self.ops)(me, index, float(value))

    def transpose(self, axis1: int, axis2: int):
        return Transpose(self.ops)(self.inplaceSafe(), axis1, axis2)

    def permute(self, *axes):
        if len(axes) == 1 and isinstance(axes[0], (list, tuple)):
            axes = axes[0]
        return Permute(self.ops)(self.inplaceSafe(), list(axes))

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return Reshape(self.ops)(self.inplaceSafe(), list(shape))

    def view(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return Reshape(self.ops, viewMode=True)(self.inplaceSafe(), list(shape))

    def squeeze(self, axis: int):
        return Squeeze(self.ops)(self.inplaceSafe(), axis)

    def unsqueeze(self, axis: int):
        return Unsqueeze(self.ops)(self.inplaceSafe(), axis)

    def copy(self):
        return Copy(self.ops)(self.inplaceSafe())

    def gather(self, axis: int, index: "Tensor"):
        return Gather(self.ops)(self.inplaceSafe(), axis, index)

    def scatter(self, axis: int, index: "Tensor", source: "Tensor"):
        return Scatter(self.ops)(self.inplaceSafe(), axis, index, source.inplaceSafe())

    def indexSelect(self, axis: int, index: "Tensor"):
        return IndexSelect(self.ops)(self.inplaceSafe(), index, axis)

    def maskedFill(self, mask: "Tensor", value: float):
        return MaskedFill(self.ops)(self.inplaceSafe(), mask, float(value))

    def softmaxCrossEntropy(self, targets: "Tensor"):
        """Tensor.softmaxCrossEntropy (functions/nn/TensorExtensions.kt:252-255)."""
        res = SoftmaxCrossEntropy(self.ops)(self, targets)
        return res if self.requiresGrad else res.noGrad()

    def batchNorm(self, axis: int, runningMean: Optional["Tensor"], runningVar: Optional["Tensor"], training: bool = False,
                  momentum: float = 0.99, epsilon: float = 1e-3, gamma: Optional["Tensor"] = None, beta: Optional["Tensor"] = None):
        """Tensor.batchNorm (functions/nn/TensorExtensions.kt:234-245)."""
        res = BatchNormalizationFunction(axis, momentum, epsilon, training, self.ops)(self, runningMean, runningVar, gamma, beta)
        return res if self.requiresGrad else res.noGrad()

    def upsample2d(self, scale: int, upsampleType: str = "NEAREST"):
        """Tensor.upsample2d (functions/nn/TensorExtensions.kt:247-250)."""
        res = Upsample2DFunction(upsampleType, scale, self.ops)(self)
        return res if self.requiresGrad else res.noGrad()

    def _pooled(self, kernel, stride, padding, dilation, options, one_d: bool):
        function = Pooling2DOperation(self.ops, list(kernel), list(stride), list(padding), list(dilation), options)
        if not one_d:
            return function(self) if self.requiresGrad else function(self).noGrad()
        if len(self.shape) != 3:
            raise RuntimeError(f"1D pooling cannot be applied to tensor with shape: {self.shape} "
                               "only tensors with 3 dimensions allowed (batch x channels x elements)")
        inp = self.unsqueeze(3)
        return (function(inp) if self.requiresGrad else function(inp).noGrad()).squeeze(3)

    def maxPooling1d(self, kernel: int, stride: Optional[int] = None, padding: int = 0, dilation: int = 1, useCeil: bool = False):
        """Tensor.maxPooling1d (functions/nn/TensorExtensions.kt:158-175): 2-D pooling of [N, C, L, 1]."""
        from .nn import PoolingOptions, PoolingType
        stride = kernel if stride is None else stride
        return self._pooled((kernel, 1), (stride, 1), (padding, 0), (dilation, 1), PoolingOptions(PoolingType.MAX, useCeil), True)

    def maxPooling2d(self, kernel, stride=None, padding=(0, 0), dilation=(1, 1), useCeil: bool = False):
        """Tensor.maxPooling2d (TensorExtensions.kt:177-192)."""
        from .nn import PoolingOptions, PoolingType
        return self._pooled(kernel, kernel if stride is None else stride, padding, dilation, PoolingOptions(PoolingType.MAX, useCeil), False)

    def avgPooling1d(self, kernel: int, stride: Optional[int] = None, padding: int = 0, useCeil: bool = False, includePadding: bool = False):
        """Tensor.avgPooling1d (TensorExtensions.kt:194-215)."""
        from .nn import PoolingOptions, PoolingType
        stride = kernel if stride is None else stride
        return self._pooled((kernel, 1), (stride, 1), (padding, 0), (1, 1), PoolingOptions(PoolingType.AVG, useCeil, includePadding), True)

    def avgPooling2d(self, kernel, stride=None, padding=(0, 0), useCeil: bool = False, includePadding: bool = False):
        """Tensor.avgPooling2d (TensorExtensions.kt:217-232)."""
        from .nn import PoolingOptions, PoolingType
        return self._pooled(kernel, kernel if stride is None else stride, padding, (1, 1), PoolingOptions(PoolingType.AVG, useCeil, includePadding), False)

    def meanVariance(self, axis: int, keepDimensions: bool = False, unbiased: bool = True):
        """AGTensor.meanVariance (AGTensor.kt:454-461): the mean keeps the axis, as there."""
        tensor = self.inplaceSafe()
        mean = tensor.mean(axis, True)
        elements = tensor.shape[SF.normalize_axis(tensor.shape, axis)] - (1 if unbiased else 0)
        centred = tensor - mean
        return mean, (centred ** 2.0).sum(axis, keepDimensions) / float(elements)

    def expand(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return Expand(self.ops)(self, list(shape))

    def _forwarded(self):
        me = self.inplaceSafe()                                  # AGTensor.inplaceSafeForwarded (AGTensor.kt:52-59)
        if isinstance(me, Function) and not me.hasValue():
            me.forward()
        return me.getRawValue()

    def item(self) -> float:
        raw = self._forwarded()
        if SF.to_store_size(raw.shape) != 1:
            raise RuntimeError(f"item() needs a singleton tensor, shape is {raw.shape}")
        return raw.getSingleValue([0] * len(raw.shape))

    def toArray(self):
        return self._forwarded().toArray()

    def noGrad(self):
        return NoGradVariable(self.ops, self._forwarded())

    def asVariable(self, requiresGrad: bool = False):
        raw = self._forwarded()
        return Variable(self.ops, raw) if requiresGrad else NoGradVariable(self.ops, raw)


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

    def noGrad(self):
        return self

    # NoGradVariable.kt:42-64: indexing acts on the raw tensor at once
    def __getitem__(self, index):
        index = list(index) if isinstance(index, (tuple, list)) else [index]
        return NoGradVariable(self.ops, self.raw.get(index))

    def __setitem__(self, index, value):
        index = list(index) if isinstance(index, (tuple, list)) else [index]
        self.raw.set(index, value._forwarded() if isinstance(value, Tensor) else float(value))

    def expand(self, *shape):                      # NoGradVariable.kt:178
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return NoGradVariable(self.ops, self.raw.broadcastTo(list(shape)))

    def reshape(self, *shape):                     # NoGradVariable.kt:174
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return NoGradVariable(self.ops, self.raw.reshape(list(shape)))

    def view(self, *shape):                        # NoGradVariable.kt:176
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return NoGradVariable(self.ops, self.raw.view(list(shape)))


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
        tensor = tensor.inplaceSafe()
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
        a, b = a.inplaceSafe(), b.inplaceSafe()
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


# ---- PointwiseFunctions.kt: the remaining maps ------------------------------------------------
class _SavedInputUnary(UnaryTensorFunction):
    """doForward saves the input and applies `op`; doBackward is written per function."""
    op = ""

    def doForward(self, x):
        self.saveForBackward(x)
        self.output = getattr(x, self.op)()


class Sinh(_SavedInputUnary):                     # PointwiseFunctions.kt:84-99
    op = "sinh"

    def doBackward(self, g):
        grad = self.valuesSaved[0].cosh()
        grad.timesAssign(g)
        return [grad]


class Cosh(_SavedInputUnary):                     # :101-116
    op = "cosh"

    def doBackward(self, g):
        grad = self.valuesSaved[0].sinh()
        grad.timesAssign(g)
        return [grad]


class Abs(_SavedInputUnary):                      # :118-133
    op = "abs"

    def doBackward(self, g):
        grad = self.valuesSaved[0].sign()
        grad.timesAssign(g)
        return [grad]


class Sqrt(_SavedInputUnary):                     # :165-182
    op = "sqrt"

    def doBackward(self, g):
        grad = self.valuesSaved[0].pow(-0.5)
        grad.timesAssign(g)
        grad.divAssign(2.0)
        return [grad]


class Sin(_SavedInputUnary):                      # :184-199
    op = "sin"

    def doBackward(self, g):
        grad = self.valuesSaved[0].cos()
        grad.timesAssign(g)
        return [grad]


class Cos(_SavedInputUnary):                      # :201-217
    op = "cos"

    def doBackward(self, g):
        grad = self.valuesSaved[0].sin()
        grad.timesAssign(g)
        grad.timesAssign(-1.0)
        return [grad]


class Tan(_SavedInputUnary):                      # :219-236
    op = "tan"

    def doBackward(self, g):
        c = self.valuesSaved[0].cos()
        c2 = c.pow(2.0)
        grad = g.div(c2)
        self.ops.release(c, c2)
        return [grad]


class Asin(_SavedInputUnary):                     # :238-251
    op = "asin"

    def doBackward(self, g):
        x = self.valuesSaved[0]
        return [g.times(x.times(x).unaryMinus().plus(1.0).sqrt().reciprocal())]


class Acos(_SavedInputUnary):                     # :253-266
    op = "acos"

    def doBackward(self, g):
        x = self.valuesSaved[0]
        return [g.times(x.times(x).unaryMinus().plus(1.0).sqrt().reciprocal().unaryMinus())]


class Atan(_SavedInputUnary):                     # :268-281
    op = "atan"

    def doBackward(self, g):
        x = self.valuesSaved[0]
        return [g.times(x.times(x).plus(1.0).reciprocal())]


class Reciprocal(UnaryTensorFunction):            # :283-301
    def doForward(self, x):
        res = x.reciprocal()
        self.saveForBackward(res)
        self.output = res

    def doBackward(self, g):
        (res,) = self.valuesSaved
        sq = res.times(res)
        neg = sq.unaryMinus()
        grad = g.times(neg)
        self.ops.release(sq, neg)
        return [grad]


class ConstantGrad(UnaryTensorFunction):          # :303-320
    op = ""
    gradientValue = 0.0

    def doForward(self, x):
        self.inputShape = list(x.shape)
        self.output = getattr(x, self.op)()

    def doBackward(self, g):
        return [may_unexpand(g.times(self.gradientValue), self.inputShape, self.ops)]


class Floor(ConstantGrad):
    op = "floor"


class Ceil(ConstantGrad):
    op = "ceil"


class Round(ConstantGrad):
    op = "round"


class Sign(ConstantGrad):
    op = "sign"


class Trunc(ConstantGrad):
    op = "trunc"


class Rsqrt(UnaryTensorFunction):                 # :343-360
    def doForward(self, x):
        res = x.rsqrt()
        self.saveForBackward(res)
        self.output = res

    def doBackward(self, g):
        (res,) = self.valuesSaved
        gr = res.pow(3.0)
        gr.divAssign(-2.0)
        grad = g.times(gr)
        self.ops.release(gr)
        return [grad]


# ---- TensorFunctions.kt: indexing and data movement ---------------------------------------------
def _norm_index(shape, index):
    """(normalised index, indexed shape, is_int_index) -- normalizedIndexedShape, ShapeFunctions.kt:232-268."""
    if all(isinstance(i, int) for i in index):
        n, s = SF.normalized_indexed_shape(shape, index)
        return n, s, True
    n, s = SF.normalized_indexed_shape_ranges(shape, index)
    return n, s, False


class Index(UnaryTensorFunction):                 # TensorFunctions.kt:33-80
    modifiesShape = True

    def __call__(self, tensor: Tensor, index):
        self.index, self.cachedShape, _ = _norm_index(tensor.shape, index)
        return super().__call__(tensor)

    def doForward(self, x):
        self.inputShape = list(x.shape)
        self.output = x.get(self.index)

    def doBackward(self, g):
        grad = self.ops.createRawFill(self.inputShape, 0.0)
        grad.set(self.index, g)
        return [grad]


class IndexSetTensor(BiTensorFunction):           # :82-127
    def __call__(self, tensor: Tensor, index, value: Tensor):
        self.index, indexed_shape, _ = _norm_index(tensor.shape, index)
        self.valueShape = list(value.shape)
        if self.valueShape != indexed_shape:
            raise ValueError(f"Cannot set value with shape: {self.valueShape} at index: {list(index)} on tensor with shape: {tensor.shape}")
        self.inputs = (tensor.inplaceSafe(), value.inplaceSafe())
        self.cachedShape = list(tensor.shape)
        return self

    def doForward(self, a, b):
        self.ops.incrementRef(a)                  # the input is written in place and becomes the output
        a.set(self.index, b)
        self.output = a

    def doBackward(self, g):
        grad_input = g.copy()
        grad_input.set(self.index, 0.0)
        grad_value = g.get(self.index).view(self.valueShape)
        return [grad_input, grad_value]


class IndexSetConstant(UnaryTensorFunction):      # :129-170
    def __call__(self, tensor: Tensor, index, value: float):
        self.index, _, _ = _norm_index(tensor.shape, index)
        if len(self.index) != len(tensor.shape):
            raise ValueError(f"Cannot set value at index: {list(index)} on tensor with shape: {tensor.shape} "
                             "(All tensor dimensions must be indexed to set a constant value)")
        self.value = float(value)
        return super().__call__(tensor)

    def doForward(self, x):
        self.ops.incrementRef(x)
        x.set(self.index, self.value)
        self.output = x

    def doBackward(self, g):
        grad = g.copy()
        grad.set(self.index, 0.0)
        return [grad]


class Transpose(UnaryTensorFunction):             # :172-198
    modifiesShape = True

    def __call__(self, tensor: Tensor, axis1: int, axis2: int):
        self.cachedShape = SF.transpose_normalize_axes(tensor.shape, axis1, axis2)[0]
        self.axis1, self.axis2 = axis1, axis2
        return super().__call__(tensor)

    def doForward(self, x):
        self.output = x.transpose(self.axis1, self.axis2)

    def doBackward(self, g):
        return [g.transpose(self.axis1, self.axis2)]


class Reshape(UnaryTensorFunction):               # :200-231 (viewMode = View)
    modifiesShape = True

    def __init__(self, ops, viewMode: bool = False):
        super().__init__(ops)
        self.viewMode = viewMode

    def __call__(self, tensor: Tensor, new_shape):
        self.cachedShape = SF.reshape(tensor.shape, new_shape)
        self.newShape = list(new_shape)
        return super().__call__(tensor)

    def doForward(self, x):
        self.oldShape = list(x.shape)
        self.output = x.view(self.newShape) if self.viewMode else x.reshape(self.newShape)

    def doBackward(self, g):
        return [g.view(self.oldShape) if self.viewMode else g.reshape(self.oldShape)]


class Permute(UnaryTensorFunction):               # :286-314
    modifiesShape = True

    def __call__(self, tensor: Tensor, axes):
        self.cachedShape = SF.permute(tensor.shape, axes)
        self.axes = list(axes)
        return super().__call__(tensor)

    def doForward(self, x):
        self.reverse = [self.axes.index(i) for i in range(len(self.axes))]
        self.output = x.permute(self.axes)

    def doBackward(self, g):
        return [g.permute(self.reverse)]


class IndexSelect(UnaryTensorFunction):           # :316-348
    modifiesShape = True

    def __call__(self, tensor: Tensor, index: Tensor, axis: int):
        if index.requiresGrad:
            raise ValueError("Index select cannot differentiate the index. The index tensor passed to index select should "
                             "never require gradients.")
        self.axis, self.cachedShape = SF.index_select_norm_axis_shape(tensor.shape, axis, index.shape)
        self.originalShape = list(tensor.shape)
        self.index = index
        return super().__call__(tensor)

    def doForward(self, x):
        self.output = x.indexSelect(self.axis, self.index.getRawValue())

    def doBackward(self, g):
        grad = self.ops.createRawFill(self.originalShape, 0.0)
        grad.indexAdd(self.axis, self.index.getRawValue(), g)
        return [grad]


class AnyTensorFunction(Function):                # AnyTensorFunction.kt
    def getInputsAsList(self):
        return list(self.inputTensors)

    def internalForward(self) -> None:
        super().internalForward()
        if self.hasValue():
            return
        fns = [t for t in self.inputTensors if isinstance(t, Function)]
        for f in fns:
            f.internalForward()
        if not self.hasValue():
            self.doForward([t.getRawValue() for t in self.inputTensors])
        for f in fns:
            f.mayFreeOutput()


class Concat(AnyTensorFunction):                  # TensorFunctions.kt:350-375
    def __call__(self, axis: int, tensors):
        tensors = [t.inplaceSafe() for t in tensors]
        self.cachedShape = SF.concat_shapes([t.shape for t in tensors], axis)
        self.inputTensors = tensors
        self.axis = SF.normalize_axis(self.cachedShape, axis)
        return self

    def doForward(self, inputs):
        self.inputSizes = [r.shape[self.axis] for r in inputs]
        self.output = self.ops.concat(self.axis, inputs)

    def doBackward(self, g):
        grads, end = [], 0
        for size in self.inputSizes:
            end += size
            grads.append(g.narrow(self.axis, end - size, size))
        return grads


class Copy(UnaryTensorFunction):                  # :377-388
    def doForward(self, x):
        self.output = x.copy()

    def doBackward(self, g):
        return [g.copy(shallow=True)]


class Squeeze(UnaryTensorFunction):               # :390-416
    modifiesShape = True

    def __call__(self, tensor: Tensor, axis: int):
        self.cachedShape = SF.squeeze(tensor.shape, axis)
        self.axis = axis
        return super().__call__(tensor)

    def doForward(self, x):
        self.inputShape = list(x.shape)
        self.output = x.squeeze(self.axis)

    def doBackward(self, g):
        return [g.reshape(self.inputShape)]


class Unsqueeze(UnaryTensorFunction):             # :418-442
    modifiesShape = True

    def __call__(self, tensor: Tensor, axis: int):
        self.cachedShape = SF.unsqueeze(tensor.shape, axis)
        self.axis = axis
        return super().__call__(tensor)

    def doForward(self, x):
        self.output = x.unsqueeze(self.axis)

    def doBackward(self, g):
        return [g.squeeze(self.axis)]


class Gather(UnaryTensorFunction):                # :444-479
    modifiesShape = True

    def __call__(self, tensor: Tensor, axis: int, index: Tensor):
        if index.requiresGrad:
            raise ValueError("Gather cannot differentiate the index. The index tensor passed to gather should never require gradients.")
        self.cachedShape = list(index.shape)
        self.axis, self.index = axis, index
        return super().__call__(tensor)

    def doForward(self, x):
        self.inputShape = list(x.shape)
        idx = self.index.getRawValue()
        self.saveForBackward(idx)
        self.output = x.gather(self.axis, idx)

    def doBackward(self, g):
        grad = self.ops.createRawFill(self.inputShape, 0.0)
        grad.inplaceScatterAdd(self.axis, self.valuesSaved[0], g)
        return [grad]


class Scatter(BiTensorFunction):                  # :481-527
    def __call__(self, tensor: Tensor, axis: int, index: Tensor, source: Tensor):
        if index.requiresGrad:
            raise ValueError("Scatter cannot differentiate the index. The index tensor passed to scatter should never require gradients.")
        a, b = tensor.inplaceSafe(), source.inplaceSafe()
        self.inputs = (a, b)
        self.cachedShape = list(a.shape)
        self.axis, self.index = axis, index
        return self

    def doForward(self, t, source):
        idx = self.index.getRawValue()
        self.saveForBackward(idx)
        self.output = t.scatter(self.axis, idx, source)

    def doBackward(self, g):
        (idx,) = self.valuesSaved
        if list(idx.shape) != self.bShape:
            raise ValueError(f"Index shape: {idx.shape} is not compatible with source shape: {self.bShape}")
        grad_input = g.scatter(self.axis, idx, 0.0) if self.inputs[0].requiresGrad else None
        grad_source = g.gather(self.axis, idx) if self.inputs[1].requiresGrad else None
        return [grad_input, grad_source]


class MaskedFill(UnaryTensorFunction):            # :559-584
    def __call__(self, tensor: Tensor, mask: Tensor, value: float):
        if mask.requiresGrad:
            raise ValueError("Masked fill only accepts mask that doesn't require gradients")
        self.mask, self.value = mask.getRawValue(), float(value)
        return super().__call__(tensor)

    def doForward(self, x):
        self.output = x.maskedFill(self.mask, self.value)

    def doBackward(self, g):
        return [g.maskedFill(self.mask, 0.0)]


class SoftmaxCrossEntropy(UnaryTensorFunction):    # functions/nn/SoftmaxCrossEntropy.kt:10-81
    """Mean negative log-likelihood of integer class targets under softmax(logits), written as
    the reference writes it: a sequence of backend calls (row maximum, shifted exp, two
    normalisations, clamp to [epsilon, 1 - epsilon], log, gather at the targets, mean), so every
    backend rounds at the same places.  Backward is (softmax - onehot(targets)) / rows."""
    modifiesShape = True

    def __call__(self, logits: Tensor, targets: Tensor):
        super().__call__(logits)
        self.cachedShape = [1]
        if targets.requiresGrad:
            raise ValueError("SoftmaxCrossEntropy only accept targets that don't require gradients")
        if len(logits.shape) != 2:
            raise ValueError(f"SoftmaxCrossEntropy requires 2D logits, but got tensor with shape {logits.shape}")
        if len(targets.shape) != 1:
            raise ValueError(f"SoftmaxCrossEntropy requires 1D targets, but got tensor with shape {targets.shape}")
        if logits.shape[0] != targets.shape[0]:
            raise ValueError("Logits must have the same size at the first dimension as targets, "
                             f"but got tensors with shape: logits: {logits.shape}, targets: {targets.shape}")
        self.targets = targets.unsqueeze(-1)
        self.rows = targets.shape[0]
        return self

    def doForward(self, x):
        ops, eps = self.ops, self.ops.epsilon
        idx = self.targets._forwarded()
        fused = getattr(x, "softmaxCrossEntropyForward", None)
        if fused is not None:
            # a backend may offer the whole forward as one call with the results of the sequence below (the CUDA backend:
            # one pass over the logits); kten-api would test for the capability the same way
            res = fused(idx, eps, _f32(1.0 - _f32(eps)))
            if res is not None:
                softmax, nll = res
                self.saveForBackward(softmax)
                self.output = nll.mean()
                # both are this function's own: the saved reference keeps the softmax until backward has run, and once that is
                # dropped a backend that defers the forward knows that nobody reads the softmax again (it need not be written)
                ops.release(nll, softmax)
                return
        max_val = x.max(-1, keepDimensions=True)
        shifted = x.minus(max_val)
        exp_val = shifted.exp()
        exp_sum = exp_val.sum(-1, keepDimensions=True)
        softmax = exp_val.div(exp_sum)
        self.saveForBackward(softmax)
        softmax_sum = softmax.sum(-1, keepDimensions=True)
        softmax_norm = softmax.div(softmax_sum)
        clipped = softmax_norm.clamp(eps, _f32(1.0 - _f32(eps)))
        log_softmax = clipped.log()
        at_targets = log_softmax.gather(-1, idx)
        nll = at_targets.unaryMinus()
        self.output = nll.mean()
        ops.release(max_val, shifted, exp_val, exp_sum, softmax_sum, softmax_norm, clipped, log_softmax, at_targets, nll)

    def doBackward(self, g):
        fused = getattr(self.valuesSaved[0], "softmaxCrossEntropyBackward", None)
        if fused is not None:
            # the same capability test as in doForward: the four calls below as one pass, with their roundings
            res = fused(self.targets._forwarded(), self.rows)
            if res is not None:
                return [res]
        grad_in = self.ops.zerosLike(self.valuesSaved[0])
        grad_in.inplaceScatter(-1, self.targets._forwarded(), -1.0)
        grad_in.plusAssign(self.valuesSaved[0])
        grad_in.divAssign(float(self.rows))
        return [grad_in]


class BatchNormalizationFunction(Function):         # functions/nn/BatchNormalizationFunction.kt:12-157
    """Batch normalisation along `axis` through the backend's BatchNormOperation; the running statistics are
    variables without gradients that the forward pass updates in place."""

    def __init__(self, axis, momentum, epsilon, training, ops):
        super().__init__(ops)
        self.axis, self.momentum, self.epsilon, self.training = axis, momentum, epsilon, training

    def __call__(self, input: Tensor, runningMean, runningVar, gamma, beta):
        self.input = input.inplaceSafe()
        if runningMean is not None and runningVar is None:
            raise ValueError("Running mean and running var must be both set to non-null or both has to be null")
        if runningMean is None and runningVar is None and not self.training:
            raise ValueError("Running mean and running var must be non-null for inference mode")
        if runningMean is not None and (not isinstance(runningMean, NoGradVariable) or not isinstance(runningVar, NoGradVariable)):
            raise ValueError("Running mean and running var parameters for batch normalization must be variables requiring no gradients")
        self.runningMean, self.runningVar = runningMean, runningVar
        self.gamma = gamma.inplaceSafe() if gamma is not None else None
        self.beta = beta.inplaceSafe() if beta is not None else None
        norm_axis = SF.normalize_axis(input.shape, self.axis)
        self.keepOutput = True
        size = self.input.shape[norm_axis]
        if runningMean is not None:
            if len(runningMean.shape) != 1 or len(runningVar.shape) != 1 or runningMean.shape[0] != size or runningVar.shape[0] != size:
                raise ValueError(f"Running mean and running var parameters for batch normalization all must have shape: [{size}], "
                                 f"but got tensors with shapes: running mean: {runningMean.shape} running var: {runningVar.shape} ")
        for t in (self.gamma, self.beta):
            if t is not None and (len(t.shape) != 1 or t.shape[0] != size):
                raise ValueError(f"Gamma and beta parameters for batch normalization all must have shape: [{size}]")
        self.op = self.ops.batchNorm(norm_axis, self.momentum, self.epsilon, self.training)
        self.cachedShape = list(input.shape)
        return self

    def getInputsAsList(self):
        return [t for t in (self.input, self.gamma, self.beta) if t is not None]

    def internalForward(self) -> None:
        super().internalForward()
        if self.hasValue():
            return
        fns = [t for t in (self.input, self.runningMean, self.runningVar, self.gamma, self.beta) if isinstance(t, Function)]
        for f in fns:
            f.internalForward()
        if not self.hasValue():
            raw = lambda t: None if t is None else t.getRawValue()
            out, mean, std = self.op.calculateOutput(raw(self.input), raw(self.runningMean), raw(self.runningVar), raw(self.gamma), raw(self.beta))
            saved = [raw(self.input), mean, std]
            if self.runningMean is not None:
                saved += [raw(self.runningMean), raw(self.runningVar)]
            if self.gamma is not None:
                saved.append(raw(self.gamma))
            self.saveForBackward(*saved)
            self.output = out
        for f in fns:
            f.mayFreeOutput()

    def doBackward(self, gradient):
        saved = self.valuesSaved
        x, mean, std = saved[0], saved[1], saved[2]
        running = saved[3:5] if self.runningMean is not None else [None, None]
        gamma = saved[-1] if self.gamma is not None else None
        if list(gradient.shape) != list(x.shape):
            raise RuntimeError(f"Gradient shape mismatch, output grad shape: {gradient.shape} input shape: {x.shape}")
        gi, gg, gb = self.op.calculateGrads(x, running[0], running[1], mean, std, gamma, gradient, self.input.requiresGrad,
                                            bool(self.gamma is not None and self.gamma.requiresGrad),
                                            bool(self.beta is not None and self.beta.requiresGrad))
        grads = [gi]
        if self.gamma is not None:
            grads.append(gg)
        if self.beta is not None:
            grads.append(gb)
        return grads


class Upsample2DFunction(UnaryTensorFunction):       # functions/nn/Upsample2DFunction.kt:9-35
    modifiesShape = True

    def __init__(self, upsampleType, scale, ops):
        super().__init__(ops)
        self.op = ops.upsample(upsampleType, scale)

    def __call__(self, tensor: Tensor):
        self.inputShape = list(tensor.shape)
        self.op.checkDimensions(self.inputShape) if hasattr(self.op, "checkDimensions") else self.op._check(self.inputShape)
        self.cachedShape = self.op.calculateOutputShape(self.inputShape)
        return super().__call__(tensor)

    def doForward(self, x):
        self.output = self.op.upsample(x)

    def doBackward(self, gradient):
        return [self.op.calculateGrad(gradient, self.inputShape)]


class Pooling2DOperation(UnaryTensorFunction):       # functions/nn/PoolingFunctions.kt:11-88
    """2-D pooling through the backend's PoolingOperation; the input (and, for max pooling, the winners' positions) are
    saved for backward."""
    modifiesShape = True

    def __init__(self, ops, kernelSize, stride, padding, dilation, poolingOptions):
        super().__init__(ops)
        self.kernelSize, self.stride, self.padding, self.dilation, self.poolingOptions = kernelSize, stride, padding, dilation, poolingOptions

    def __call__(self, tensor: Tensor):
        if len(tensor.shape) not in (3, 4):
            raise ValueError(f"2D pooling requires input tensor with 3 or 4 dimensions, but got tensor with shape: {tensor.shape}")
        from .nn import pooled_size
        o = self.poolingOptions
        hw = [pooled_size(tensor.shape[-2], self.dilation[0], self.kernelSize[0], self.padding[0], self.stride[0], o.useCeil),
              pooled_size(tensor.shape[-1], self.dilation[1], self.kernelSize[1], self.padding[1], self.stride[1], o.useCeil)]
        self.cachedShape = list(tensor.shape[:-2]) + hw
        self.poolingOp = self.ops.spatialPooling(self.kernelSize, self.padding, self.stride, self.dilation, o)
        return super().__call__(tensor)

    def doForward(self, x):
        out, indices = self.poolingOp.updateOutput(x)
        if indices is not None:
            self.saveForBackward(x, indices)
        else:
            self.saveForBackward(x)
        self.output = out

    def doBackward(self, gradient):
        x = self.valuesSaved[0]
        indices = self.valuesSaved[1] if len(self.valuesSaved) == 2 else None
        return [self.poolingOp.calculateGradInput(x, gradient, indices)]


def oneHot(ops, targets: Tensor, classes: int) -> Tensor:
    """Tensor.oneHot (Tensor.kt:1712-1721): built on the host, element by element, then uploaded."""
    import numpy as np
    if len(targets.shape) != 1:
        raise ValueError(f"One hot encoding can only be applied to 1D tensors, but got tensor with shape: {targets.shape}")
    t = targets.toArray().astype(np.int64)
    hot = np.zeros((t.shape[0], classes), dtype=np.float32)
    ok = (t >= 0) & (t < classes)
    hot[np.nonzero(ok)[0], t[ok]] = 1.0
    return NoGradVariable(ops, ops.createRaw([t.shape[0], classes], hot.reshape(-1)))


def concat(tensors, axis: int = 0) -> Tensor:
    """Tensor.concat (Tensor.kt): along `axis`, default 0."""
    tensors = list(tensors)
    return Concat(tensors[0].ops)(axis, tensors)


# ---- factories (Tensor.Companion, Tensor.kt:1630-1786) -------------------------------------
def tensorOf(ops, values, shape: Optional[Sequence[int]] = None, requiresGrad: bool = False) -> Tensor:
    import numpy as np
    arr = np.asarray(values, dtype=np.float32)
    shp = list(shape) if shape is not None else ([1] if arr.ndim == 0 else list(arr.shape))
    raw = ops.createRaw(shp, arr.reshape(-1))
    return Variable(ops, raw) if requiresGrad else NoGradVariable(ops, raw)
