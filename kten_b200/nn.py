"""The nn operations of the TensorOperations SPI that are reductions and broadcast maps: batch normalisation
and nearest-neighbour upsampling (TensorOperations.kt:127-131; kten-jvm: JVMBatchNorm.kt, JVMUpsample2DNearest.kt).

Neither needs a kernel of its own.  Viewed as [outer, C * inner] -- `axis` of extent C in the middle -- the sums a
batch norm takes per channel are leading-axis sums of an elementwise expression followed by a small sum over
`inner`, and its output is a broadcast map with row vectors of C * inner floats.  With the calls below recorded
(ops.lazy) a training forward is three passes over the input (mean; centred squares; normalise -- the reference makes
the same three) and the backward two (both sums in ONE pass with two sinks; the gradient), each a generated kernel that
reads its operands once; run call by call they are the library's ordinary kernels.  Every per-element operation is
the reference's float operation in the reference's order, so given the same per-channel statistics the outputs are
bit-identical; the statistics themselves are sums (double accumulation, compared within the reduction tolerance).

Upsampling is a broadcast copy ([R, 1, W, 1] -> [R, s, W, s]) and its gradient a sum back to the small shape; with an
innermost extent of s (2, 3 ...) the general broadcast and reduction kernels fall to their element-wise forms, so the
library has two small kernels for it (ktc_nn.cu) and the composition remains as the form a backend without them uses.

Spatial pooling (TensorOperations.spatialPooling, TensorOperations.kt:127) is a window reduction with kernels of its own
(ktc_pool.cu); this file holds the host part of kten-jvm's JVMSpatialPoolingBase: the shape checks, the output extents
computed on floats, the result tensors."""
from __future__ import annotations

from typing import List, Optional, Sequence

from . import shape_functions as SF


def _volume(shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class _Recorded:
    """Runs the body with the calls recorded where the backend can (so that they fuse), and hands back stored
    tensors when the caller itself runs call by call."""

    def __init__(self, ops):
        self.ops, self.was = ops, getattr(ops, "lazy", False)

    def __enter__(self):
        if hasattr(self.ops, "lazy"):
            self.ops.lazy = True
        return self

    def __exit__(self, *exc):
        if hasattr(self.ops, "lazy"):
            self.ops.lazy = self.was
        return False

    def settle(self, *raws):
        if not self.was:
            for r in raws:
                if r is not None and hasattr(r, "_buf"):
                    r._buf()


class CUDABatchNorm:
    """BatchNormOperation over raw tensors of the CUDA backend (interface: BatchNormOperation.kt:5-44)."""

    def __init__(self, axis: int, momentum: float, epsilon: float, training: bool, ops):
        self.axis, self.momentum, self.epsilon, self.training, self.ops = int(axis), float(momentum), float(epsilon), bool(training), ops

    # ---- helpers ---------------------------------------------------------------------------------------------
    def _split(self, shape):
        a = self.axis
        return _volume(shape[:a]), int(shape[a]), _volume(shape[a + 1:])

    @staticmethod
    def _row(t, C, inner):
        """A [C] tensor as the row vector [1, C * inner] that broadcasts against [outer, C * inner]."""
        if inner == 1:
            return t.view([1, C])
        return t.view([C, 1]).broadcastTo([C, inner]).view([1, C * inner])

    @staticmethod
    def _channel_sums(t2d, C, inner):
        """Sum of a [outer, C * inner] tensor per channel: over the leading axis, then over `inner`."""
        s = t2d.sum(0)
        return s if inner == 1 else s.view([C, inner]).sum(1)

    # ---- forward ---------------------------------------------------------------------------------------------
    def calculateOutput(self, input, runningMean, runningVar, gamma, beta):
        outer, C, inner = self._split(input.shape)
        n = outer * inner
        with _Recorded(self.ops) as rec:
            x = input.view([outer, C * inner])
            if self.training:
                mean = self._channel_sums(x, C, inner).div(float(n))                    # sum / elementSize (JVMBatchNorm.kt:54)
                mean_row = self._row(mean, C, inner)
                d = x.minus(mean_row)
                ssq = self._channel_sums(d.times(d), C, inner)                          # :57-61
                var = ssq.div(float(n)).plus(self.epsilon)
                if self.epsilon == 0.0:
                    # the sum is zero and so is epsilon: 0f instead of 1f / 0f.  Where the sum is zero the root is taken of 1
                    # and the result multiplied by 0; elsewhere the two masks add 0f and multiply by 1f, which change nothing
                    stdev = var.plus(ssq.lte(0.0)).sqrt().reciprocal().times(ssq.gt(0.0))
                else:
                    stdev = var.sqrt().reciprocal()                                     # 1f / sqrt(sum / n + epsilon), :63-65
                if runningMean is not None and runningVar is not None:                  # :69-73
                    keep = _f32(_f32(1.0) - _f32(self.momentum))                        # (1f - momentum), a float subtraction
                    runningMean.timesAssign(keep)
                    runningMean.plusAssign(mean.times(self.momentum))
                    runningVar.timesAssign(keep)
                    runningVar.plusAssign(ssq.div(float(n - 1)).times(self.momentum))
            else:
                mean = runningMean
                stdev = runningVar.plus(self.epsilon).sqrt().reciprocal()               # :75-76
                mean_row = self._row(mean, C, inner)
            y = x.minus(mean_row).times(self._row(stdev, C, inner))                     # (x - mean) * stdev * g + b, :82-84
            if gamma is not None:
                y = y.times(self._row(gamma, C, inner))
            y = y.plus(self._row(beta, C, inner)) if beta is not None else y.plus(0.0)
            out = y.view(list(input.shape))
            if not self.training:                                                       # the reference leaves both untouched (zeros) here
                mean, stdev = self.ops.createRawFill([C], 0.0), self.ops.createRawFill([C], 0.0)
            rec.settle(out, mean, stdev, runningMean, runningVar)
        return out, mean, stdev

    # ---- backward --------------------------------------------------------------------------------------------
    def calculateGrads(self, input, runningMean, runningVar, currentMean, currentStd, gamma, gradOut,
                       inRequiresGrad: bool, gammaRequiresGrad: bool, betaRequiresGrad: bool):
        if not (inRequiresGrad or gammaRequiresGrad or betaRequiresGrad):
            return None, None, None
        outer, C, inner = self._split(input.shape)
        n = outer * inner
        with _Recorded(self.ops) as rec:
            x, go = input.view([outer, C * inner]), gradOut.view([outer, C * inner])
            if self.training:
                mean, stdev = currentMean, currentStd
            else:
                mean = runningMean
                # kten-jvm takes this one in double, (1.0 / sqrt((rv + eps).toDouble())).toFloat() (:117); rsqrt is 1f / sqrt(float):
                # two float roundings instead of one, at most one ulp apart in the inverse deviation
                stdev = runningVar.plus(self.epsilon).rsqrt()
            mean_row = self._row(mean, C, inner)
            d = x.minus(mean_row)
            # both sums are pending until the first is needed: one pass over x and gradOut with two sinks (a sum of a stored
            # tensor would run at once, so gradOut enters as the expression gradOut * 1f, which is gradOut bit for bit)
            s_go = go.times(1.0).sum(0)
            s_dot = d.times(go).sum(0)
            total = s_go if inner == 1 else s_go.view([C, inner]).sum(1)                # :120-123
            dot = s_dot if inner == 1 else s_dot.view([C, inner]).sum(1)                # :125-128
            grad_in = grad_gamma = grad_beta = None
            if inRequiresGrad:
                std_row = self._row(stdev, C, inner)
                if self.training:                                                       # :131-138
                    dps = dot.times(stdev).times(stdev).div(float(n))
                    gmean = total.div(float(n))
                    t = go.minus(self._row(gmean, C, inner)).minus(d.times(self._row(dps, C, inner))).times(std_row)
                else:                                                                   # :139-143
                    t = go.times(std_row)
                if gamma is not None:
                    t = t.times(self._row(gamma, C, inner))
                grad_in = t.view(list(input.shape))
            if gammaRequiresGrad:
                grad_gamma = dot.times(stdev)                                           # :147-149
            if betaRequiresGrad:
                grad_beta = total                                                       # :151-153
            rec.settle(grad_in, grad_gamma, grad_beta)
        return grad_in, grad_gamma, grad_beta


def _f32(v: float) -> float:
    import numpy as np
    return float(np.float32(v))


class CUDAUpsample2DNearest:
    """Upsample2DOperation (Upsample2DOperation.kt:5-44; kten-jvm: JVMUpsample2DNearest.kt:14-77)."""

    def __init__(self, scale: int, ops):
        self.scale, self.ops = int(scale), ops

    @staticmethod
    def checkDimensions(shape) -> None:
        if len(shape) not in (3, 4):
            raise ValueError(f"2D Upsampling can only be applied to tensors with 3 or 4 dimensions, but got tensor with shape: {list(shape)}")

    def calculateOutputShape(self, shape) -> List[int]:
        return list(shape[:-2]) + [shape[-2] * self.scale, shape[-1] * self.scale]

    def checkGradOutShape(self, grad_shape, input_shape) -> None:
        s = self.scale
        if len(input_shape) != len(grad_shape):
            raise ValueError(f"2D Upsample got gradient with different dimensions ({len(grad_shape)}) as the input tensor dimensions ({len(input_shape)})")
        if grad_shape[-2] % s != 0 or grad_shape[-1] % s != 0:
            raise ValueError(f"2D Upsample output gradients shape must be divisible by scale: {s} in the last two dimensions,"
                             f"but got gradient tensor with shape: {list(grad_shape)}")
        if grad_shape[-2] // s != input_shape[-2] or grad_shape[-1] // s != input_shape[-1] or list(grad_shape[:-2]) != list(input_shape[:-2]):
            raise ValueError(f"2D Upsample output gradients shape: {list(grad_shape)} does not align with input tensor shape: {list(input_shape)} "
                             f"with scale: {s}")

    def upsample(self, input):
        self.checkDimensions(input.shape)
        s = self.scale
        rows, W = _volume(input.shape[:-1]), int(input.shape[-1])
        entry = getattr(self.ops.lib, "ktc_upsample2d_nearest", None)
        if entry is not None:                                      # the library's kernel
            from . import _lib as L
            out = self.ops.createRaw(self.calculateOutputShape(input.shape))
            L.check(entry(out._buf(), input._buf(), rows, W, s))
            return out
        with _Recorded(self.ops) as rec:                           # a broadcast copy [rows, 1, W, 1] -> [rows, s, W, s]
            out = input.view([rows, 1, W, 1]).broadcastTo([rows, s, W, s]).view(self.calculateOutputShape(input.shape))
            rec.settle(out)
        return out

    def calculateGrad(self, gradOut, inputShape):
        self.checkDimensions(gradOut.shape)
        self.checkGradOutShape(gradOut.shape, inputShape)
        s = self.scale
        rows, W = _volume(inputShape[:-1]), int(inputShape[-1])
        entry = getattr(self.ops.lib, "ktc_upsample2d_nearest_grad", None)
        if entry is not None:
            from . import _lib as L
            res = self.ops.createRaw(list(inputShape))
            L.check(entry(res._buf(), gradOut._buf(), rows, W, s))
            return res
        return gradOut.view([rows, s, W, s]).sumToShape([rows, 1, W, 1]).view(list(inputShape))


class PoolingType:                                      # PoolingOptions.kt:3-5
    MAX, AVG = "MAX", "AVG"


class PoolingOptions:                                   # PoolingOptions.kt:6-10
    def __init__(self, type: str, useCeil: bool = False, includePadding: bool = False):
        self.type, self.useCeil, self.includePadding = type, bool(useCeil), bool(includePadding)


def pooled_size(extent: int, dilation: int, kernel: int, padding: int, stride: int, use_ceil: bool) -> int:
    """PoolingOperation.calculateSizeOnFloats (PoolingOperation.kt:10-13) in float arithmetic, then ceil or floor."""
    import numpy as np
    f = np.float32
    v = (f(extent) - (f(dilation) * (f(kernel) - f(1.0)) + f(1.0)) + f(2.0) * f(padding)) / f(stride) + f(1.0)
    return int(np.ceil(v)) if use_ceil else int(np.floor(v))


class CUDASpatialPooling:
    """PoolingOperation over raw tensors of the CUDA backend (interface: PoolingOperation.kt:5-15; host logic:
    JVMSpatialPoolingBase.kt:14-137; kernels: ktc_pool.cu).  [N, C, H, W] or [C, H, W] input; max pooling returns the
    positions of the winners inside their planes as a second tensor, average pooling none."""

    def __init__(self, kernel, padding, stride, dilation, options: PoolingOptions, ops):
        self.kh, self.kw = int(kernel[0]), int(kernel[1])
        self.ph, self.pw = int(padding[0]), int(padding[1])
        self.sh, self.sw = int(stride[0]), int(stride[1])
        self.is_max = options.type == PoolingType.MAX
        self.dh, self.dw = (int(dilation[0]), int(dilation[1])) if self.is_max else (1, 1)      # AbstractJVMTensorOperations: AVG ignores it
        self.useCeil, self.includePadding, self.ops = options.useCeil, options.includePadding, ops

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
            raise ValueError("Padding should be smaller than kernel size / 2, "
                             f"but got kernel: ({self.kh}, {self.kw}) and padding: ({self.ph}, {self.pw})")
        f = 1 if len(input.shape) == 4 else 0
        planes_c, H, W = input.shape[f], input.shape[f + 1], input.shape[f + 2]
        OH = pooled_size(H, self.dh, self.kh, self.ph, self.sh, self.useCeil)
        OW = pooled_size(W, self.dw, self.kw, self.pw, self.sw, self.useCeil)
        if self.ph > 0 or self.pw > 0:                      # a last window must start inside the plane or its left padding
            if (OH - 1) * self.sh >= H + self.ph:
                OH -= 1
            if (OW - 1) * self.sw >= W + self.pw:
                OW -= 1
        if OH < 1 or OW < 1:
            raise ValueError(f"Calculated output size: {planes_c} x {OH} x {OW} is too small. Input size: {planes_c} x {H} x {W}")
        for t, what in ((gradOut, "gradient"), (indices, "indices")):
            if t is not None and (t.shape[f] != planes_c or t.shape[f + 1] != OH or t.shape[f + 2] != OW):
                raise ValueError(f"Invalid {what} shape, {what} must have shape with (F x H x W) = {planes_c} x {OH} x {OW}, "
                                 f"but got {t.shape[f]} x {t.shape[f + 1]} x {t.shape[f + 2]}")
        planes = planes_c * (input.shape[0] if f else 1)
        import ctypes as C
        geom = (C.c_int * 12)(H, W, OH, OW, self.kh, self.kw, self.ph, self.pw, self.sh, self.sw, self.dh, self.dw)
        return planes, list(input.shape[:f + 1]) + [OH, OW], geom

    def updateOutput(self, input):
        from . import _lib as L
        planes, out_shape, geom = self._geometry(input)
        out = self.ops.createRaw(out_shape)
        if self.is_max:
            indices = self.ops.createRaw(out_shape)
            L.check(self.ops.lib.ktc_pool2d_max(out._buf(), indices._buf(), input._buf(), planes, geom))
            return out, indices
        L.check(self.ops.lib.ktc_pool2d_avg(out._buf(), input._buf(), planes, geom, 1 if self.includePadding else 0))
        return out, None

    def calculateGradInput(self, input, gradOut, indices):
        from . import _lib as L
        planes, _, geom = self._geometry(input, gradOut, indices)
        grad_in = self.ops.createRaw(list(input.shape))
        if self.is_max:
            L.check(self.ops.lib.ktc_pool2d_max_grad(grad_in._buf(), gradOut._buf(), indices._buf(), planes, geom))
        else:
            L.check(self.ops.lib.ktc_pool2d_avg_grad(grad_in._buf(), gradOut._buf(), planes, geom, 1 if self.includePadding else 0))
        return grad_in
