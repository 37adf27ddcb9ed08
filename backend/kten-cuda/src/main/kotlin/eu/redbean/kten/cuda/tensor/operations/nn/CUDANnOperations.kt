package eu.redbean.kten.cuda.tensor.operations.nn

import eu.redbean.kten.api.autograd.utils.toStoreSize
import eu.redbean.kten.api.tensor.operations.nn.BatchNormOperation
import eu.redbean.kten.api.tensor.operations.nn.Upsample2DOperation
import eu.redbean.kten.cuda.tensor.operations.CUDATensorOperations
import eu.redbean.kten.cuda.tensor.platform.KtcNative
import eu.redbean.kten.cuda.tensor.platform.KtcNative.check
import eu.redbean.kten.cuda.tensor.store.CUDARawTensor

/**
 * Batch normalisation and nearest-neighbour upsampling as compositions of raw-tensor calls (the mirror of
 * kten_b200/nn.py).  Neither needs a kernel of its own: viewed as [outer, C * inner] the per-channel sums of a batch
 * norm are leading-axis sums of an elementwise expression followed by a small sum over `inner`, its output a
 * broadcast map with row vectors of C * inner floats.  The calls are recorded (ops.lazy) while an operation runs, so a
 * training forward is three passes over the input and the backward two; every per-element operation is kten-jvm's
 * float operation in kten-jvm's order (JVMBatchNorm.kt:32-165).  Not compiled: no JDK on this box.
 */
private inline fun <T> CUDATensorOperations.recorded(body: () -> T): T {
    val was = lazy
    lazy = true
    try {
        return body()
    } finally {
        lazy = was
    }
}

class CUDABatchNorm(
    val axis: Int,
    val momentum: Float,
    val epsilon: Float,
    val training: Boolean,
    val ops: CUDATensorOperations
) : BatchNormOperation<CUDARawTensor> {

    private fun split(shape: List<Int>) = Triple(shape.take(axis).toStoreSize(), shape[axis], shape.drop(axis + 1).toStoreSize())

    /** A [C] tensor as the row vector [1, C * inner] that broadcasts against [outer, C * inner]. */
    private fun row(t: CUDARawTensor, c: Int, inner: Int): CUDARawTensor =
        if (inner == 1) t.view(listOf(1, c)) else t.view(listOf(c, 1)).broadcastTo(listOf(c, inner)).view(listOf(1, c * inner))

    private fun channelSums(t: CUDARawTensor, c: Int, inner: Int): CUDARawTensor {
        val s = t.sum(0, false) as CUDARawTensor
        return if (inner == 1) s else s.view(listOf(c, inner)).sum(1, false) as CUDARawTensor
    }

    override fun calculateOutput(
        input: CUDARawTensor, runningMean: CUDARawTensor?, runningVar: CUDARawTensor?, gamma: CUDARawTensor?, beta: CUDARawTensor?
    ): BatchNormOperation.BatchNormOutputs<CUDARawTensor> = ops.recorded {
        val (outer, c, inner) = split(input.shape)
        val n = outer * inner
        val x = input.view(listOf(outer, c * inner))
        var mean: CUDARawTensor
        var stdev: CUDARawTensor
        if (training) {
            mean = channelSums(x, c, inner).div(n.toFloat()) as CUDARawTensor
            val d = x.minus(row(mean, c, inner)) as CUDARawTensor
            val ssq = channelSums(d.times(d) as CUDARawTensor, c, inner)
            val variance = ssq.div(n.toFloat()).plus(epsilon) as CUDARawTensor
            stdev = if (epsilon == 0f)          // sum == 0 and epsilon == 0: 0f instead of 1f / 0f (JVMBatchNorm.kt:63-65)
                (variance.plus(ssq.lte(0f)).sqrt().reciprocal() as CUDARawTensor).times(ssq.gt(0f)) as CUDARawTensor
            else variance.sqrt().reciprocal() as CUDARawTensor
            if (runningMean != null && runningVar != null) {
                val keep = 1f - momentum
                runningMean.timesAssign(keep)
                runningMean.plusAssign(mean.times(momentum))
                runningVar.timesAssign(keep)
                runningVar.plusAssign(ssq.div((n - 1).toFloat()).times(momentum))
            }
        } else {
            mean = runningMean!!
            stdev = runningVar!!.plus(epsilon).sqrt().reciprocal() as CUDARawTensor
        }
        var y = x.minus(row(mean, c, inner)).times(row(stdev, c, inner)) as CUDARawTensor
        if (gamma != null) y = y.times(row(gamma, c, inner)) as CUDARawTensor
        y = (if (beta != null) y.plus(row(beta, c, inner)) else y.plus(0f)) as CUDARawTensor
        if (!training) {                        // kten-jvm leaves both untouched (zeros) in inference mode
            mean = ops.createRawFill(listOf(c), 0f)
            stdev = ops.createRawFill(listOf(c), 0f)
        }
        BatchNormOperation.BatchNormOutputs(y.view(input.shape), mean, stdev)
    }

    override fun calculateGrads(
        input: CUDARawTensor, runningMean: CUDARawTensor?, runningVar: CUDARawTensor?, currentMean: CUDARawTensor, currentStd: CUDARawTensor,
        gamma: CUDARawTensor?, gradOut: CUDARawTensor, inRequiresGrad: Boolean, gammaRequiresGrad: Boolean, betaRequiresGrad: Boolean
    ): BatchNormOperation.BatchNormGrads<CUDARawTensor> {
        if (!inRequiresGrad && !gammaRequiresGrad && !betaRequiresGrad) return BatchNormOperation.BatchNormGrads(null, null, null)
        return ops.recorded {
            val (outer, c, inner) = split(input.shape)
            val n = outer * inner
            val x = input.view(listOf(outer, c * inner))
            val go = gradOut.view(listOf(outer, c * inner))
            val mean = if (training) currentMean else runningMean!!
            // kten-jvm takes the inference-mode deviation in double (JVMBatchNorm.kt:117); rsqrt is 1f / sqrt(float): at most one ulp apart
            val stdev = if (training) currentStd else runningVar!!.plus(epsilon).rsqrt() as CUDARawTensor
            val d = x.minus(row(mean, c, inner)) as CUDARawTensor
            // both sums stay pending until the first is needed: one pass over x and gradOut with two sinks (a sum of a stored
            // tensor would run at once, so gradOut enters as the expression gradOut * 1f, which is gradOut bit for bit)
            val sGo = go.times(1f).sum(0, false) as CUDARawTensor
            val sDot = d.times(go).sum(0, false) as CUDARawTensor
            val total = if (inner == 1) sGo else sGo.view(listOf(c, inner)).sum(1, false) as CUDARawTensor
            val dot = if (inner == 1) sDot else sDot.view(listOf(c, inner)).sum(1, false) as CUDARawTensor
            var gradIn: CUDARawTensor? = null
            if (inRequiresGrad) {
                val stdRow = row(stdev, c, inner)
                var t = if (training) {
                    val dps = dot.times(stdev).times(stdev).div(n.toFloat()) as CUDARawTensor
                    val gradMean = total.div(n.toFloat()) as CUDARawTensor
                    go.minus(row(gradMean, c, inner)).minus(d.times(row(dps, c, inner))).times(stdRow) as CUDARawTensor
                } else go.times(stdRow) as CUDARawTensor
                if (gamma != null) t = t.times(row(gamma, c, inner)) as CUDARawTensor
                gradIn = t.view(input.shape)
            }
            BatchNormOperation.BatchNormGrads(gradIn, if (gammaRequiresGrad) dot.times(stdev) as CUDARawTensor else null, if (betaRequiresGrad) total else null)
        }
    }
}

class CUDAUpsample2DNearest(override val scale: Int, val ops: CUDATensorOperations) : Upsample2DOperation<CUDARawTensor> {

    override fun upsample(input: CUDARawTensor): CUDARawTensor {
        checkDimensions(input.shape)
        val rows = input.shape.dropLast(1).toStoreSize().toLong()
        val out = ops.createRaw(calculateOutputShape(input.shape))
        check(KtcNative.upsample2dNearest.invokeExact(out.handle, input.handle, rows, input.shape.last().toLong(), scale) as Int)
        return out
    }

    override fun calculateGrad(gradOut: CUDARawTensor, inputShape: List<Int>): CUDARawTensor {
        checkDimensions(gradOut.shape)
        checkGradOutShape(gradOut.shape, inputShape)
        val rows = inputShape.dropLast(1).toStoreSize().toLong()
        val gradIn = ops.createRaw(inputShape)
        check(KtcNative.upsample2dNearestGrad.invokeExact(gradIn.handle, gradOut.handle, rows, inputShape.last().toLong(), scale) as Int)
        return gradIn
    }
}

/**
 * Spatial pooling (TensorOperations.spatialPooling; interface: PoolingOperation.kt:5-15): the host part of kten-jvm's
 * JVMSpatialPoolingBase.kt:14-137 -- shape checks, output extents on floats, result tensors -- over the library's window
 * kernels (ktc_pool2d_*), which keep kten-jvm's arithmetic and order to the bit.  The mirror of kten_b200/nn.py.
 * Not compiled: no JDK on this box.
 */
class CUDASpatialPooling(
    kernel: List<Int>, padding: List<Int>, stride: List<Int>, dilation: List<Int>,
    val options: eu.redbean.kten.api.tensor.operations.nn.PoolingOptions,
    val ops: CUDATensorOperations
) : eu.redbean.kten.api.tensor.operations.nn.PoolingOperation<CUDARawTensor> {

    private val kh = kernel[0]; private val kw = kernel[1]
    private val ph = padding[0]; private val pw = padding[1]
    private val sh = stride[0]; private val sw = stride[1]
    private val dh = dilation[0]; private val dw = dilation[1]
    private val isMax = options.type == eu.redbean.kten.api.tensor.operations.nn.PoolingType.MAX

    private class Geometry(val planes: Long, val outShape: List<Int>, val values: IntArray)

    private fun pooled(extent: Int, dilation: Int, kernel: Int, padding: Int, stride: Int): Int {
        val v = eu.redbean.kten.api.tensor.operations.nn.PoolingOperation.calculateSizeOnFloats(
            extent.toFloat(), dilation.toFloat(), kernel.toFloat(), padding.toFloat(), stride.toFloat())
        return if (options.useCeil) kotlin.math.ceil(v).toInt() else kotlin.math.floor(v).toInt()
    }

    private fun geometry(input: CUDARawTensor, gradOut: CUDARawTensor?, indices: CUDARawTensor?): Geometry {
        if (kh <= 0 || kw <= 0) throw IllegalArgumentException("Kernel size should be greater than zero")
        if (sh <= 0 || sw <= 0) throw IllegalArgumentException("Stride should be greater than zero")
        if (dh <= 0 || dw <= 0) throw IllegalArgumentException("Dilation should be greater than zero")
        if (input.dimensions !in listOf(3, 4)) throw IllegalArgumentException("Input must be 3D or 4D tensor")
        if (ph > kh / 2 || pw > kw / 2)
            throw IllegalArgumentException("Padding should be smaller than kernel size / 2, but got kernel: ($kh, $kw) and padding: ($ph, $pw)")
        val f = if (input.dimensions == 4) 1 else 0
        val c = input.shape[f]; val h = input.shape[f + 1]; val w = input.shape[f + 2]
        var oh = pooled(h, dh, kh, ph, sh)
        var ow = pooled(w, dw, kw, pw, sw)
        if (ph > 0 || pw > 0) {                               // a last window must not start in the right / bottom padding
            if ((oh - 1) * sh >= h + ph) oh--
            if ((ow - 1) * sw >= w + pw) ow--
        }
        if (oh < 1 || ow < 1)
            throw IllegalArgumentException("Calculated output size: $c x $oh x $ow is too small. Input size: $c x $h x $w")
        for ((t, what) in listOf(gradOut to "gradient", indices to "indices")) {
            if (t != null && (t.shape[f] != c || t.shape[f + 1] != oh || t.shape[f + 2] != ow))
                throw IllegalArgumentException("Invalid $what shape, $what must have shape with (F x H x W) = $c x $oh x $ow, " +
                        "but got ${t.shape[f]} x ${t.shape[f + 1]} x ${t.shape[f + 2]}")
        }
        val planes = c.toLong() * (if (f == 1) input.shape[0] else 1)
        return Geometry(planes, input.shape.take(f + 1) + listOf(oh, ow), intArrayOf(h, w, oh, ow, kh, kw, ph, pw, sh, sw, dh, dw))
    }

    private fun <T> withGeom(g: Geometry, call: (java.lang.foreign.MemorySegment) -> T): T =
        java.lang.foreign.Arena.ofConfined().use { arena -> call(arena.allocateFrom(java.lang.foreign.ValueLayout.JAVA_INT, *g.values)) }

    override fun updateOutput(input: CUDARawTensor): eu.redbean.kten.api.tensor.operations.nn.PoolingResult<CUDARawTensor> {
        val g = geometry(input, null, null)
        val out = ops.createRaw(g.outShape)
        if (isMax) {
            val indices = ops.createRaw(g.outShape)
            withGeom(g) { check(KtcNative.pool2dMax.invokeExact(out.handle, indices.handle, input.handle, g.planes, it) as Int) }
            return eu.redbean.kten.api.tensor.operations.nn.PoolingResult(out, indices)
        }
        withGeom(g) { check(KtcNative.pool2dAvg.invokeExact(out.handle, input.handle, g.planes, it, if (options.includePadding) 1 else 0) as Int) }
        return eu.redbean.kten.api.tensor.operations.nn.PoolingResult(out, null)
    }

    override fun calculateGradInput(input: CUDARawTensor, gradOut: CUDARawTensor, indices: CUDARawTensor?): CUDARawTensor {
        val g = geometry(input, gradOut, indices)
        val gradIn = ops.createRaw(input.shape)
        if (isMax)
            withGeom(g) { check(KtcNative.pool2dMaxGrad.invokeExact(gradIn.handle, gradOut.handle, indices!!.handle, g.planes, it) as Int) }
        else
            withGeom(g) { check(KtcNative.pool2dAvgGrad.invokeExact(gradIn.handle, gradOut.handle, g.planes, it, if (options.includePadding) 1 else 0) as Int) }
        return gradIn
    }
}
