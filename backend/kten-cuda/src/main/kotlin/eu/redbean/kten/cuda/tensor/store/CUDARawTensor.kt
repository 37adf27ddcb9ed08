package eu.redbean.kten.cuda.tensor.store

import eu.redbean.kten.api.autograd.utils.inferExplicitBroadcastShape
import eu.redbean.kten.api.autograd.utils.normalizeAxis
import eu.redbean.kten.api.autograd.utils.reshape
import eu.redbean.kten.api.autograd.utils.toStoreSize
import eu.redbean.kten.api.tensor.store.AbstractRawTensor
import eu.redbean.kten.api.tensor.store.AggregatingOperation
import eu.redbean.kten.cuda.tensor.operations.CUDATensorOperations
import eu.redbean.kten.cuda.tensor.platform.KtcNative
import eu.redbean.kten.cuda.tensor.platform.KtcNative.check
import java.lang.foreign.Arena
import java.lang.foreign.ValueLayout.JAVA_FLOAT

/** Device storage: one reference-counted buffer handle of libkten_cuda.so. */
class CUDABuffer(val handle: Long, val size: Int)

/**
 * RawTensor of the kten-cuda backend: shape on the JVM heap, data in HBM.  Every operation of the
 * float32 hot path is one call through the C ABI; operations outside that path are not provided by
 * the native library yet and throw UnsupportedOperationException.
 */
class CUDARawTensor(
    shape: List<Int>,
    store: CUDABuffer,
    private val ops: CUDATensorOperations
) : AbstractRawTensor<CUDABuffer>(shape, store) {

    internal var refCount = 1
    internal var mustSurviveGC = false
    private var released = false

    init {
        ops.instanceCreated(this)
    }

    private val handle: Long
        get() {
            if (released) throw IllegalStateException("Raw tensor already released")
            return storeReference.handle
        }

    private val volume: Long get() = shape.toStoreSize().toLong()

    internal fun release(): Boolean {
        if (released) return false
        if (!mustSurviveGC) refCount--
        if (refCount <= 0) {
            check(KtcNative.release.invokeExact(storeReference.handle) as Int)
            released = true
            return true
        }
        return false
    }

    // ---- elementwise -------------------------------------------------------------------------------
    private fun binary(op: Int, other: AbstractRawTensor<CUDABuffer>): CUDARawTensor {
        other as CUDARawTensor
        if (shape == other.shape) {
            val res = ops.createRaw(shape)
            check(KtcNative.binary.invokeExact(op, res.handle, handle, other.handle, volume) as Int)
            return res
        }
        val res = ops.createRaw(calculateCommonShapeWith(other))
        Arena.ofConfined().use { arena ->
            check(KtcNative.binaryBcast.invokeExact(op, res.handle, handle, KtcNative.shape(arena, shape), shape.size,
                                                    other.handle, KtcNative.shape(arena, other.shape), other.shape.size) as Int)
        }
        return res
    }

    private fun binaryAssign(op: Int, other: AbstractRawTensor<CUDABuffer>) {
        if (shape != other.shape)
            throw IllegalArgumentException("Shapes does not match for inplace operation on tensors with shapes: $shape and ${other.shape}.")
        check(KtcNative.binaryInplace.invokeExact(op, handle, (other as CUDARawTensor).handle, volume) as Int)
    }

    internal fun scalar(op: Int, constant: Float, scalarFirst: Boolean = false): CUDARawTensor {
        val res = ops.createRaw(shape)
        check(KtcNative.scalar.invokeExact(op, res.handle, handle, constant, volume, if (scalarFirst) 1 else 0) as Int)
        return res
    }

    private fun scalarAssign(op: Int, constant: Float) =
        check(KtcNative.scalarInplace.invokeExact(op, handle, constant, volume) as Int)

    private fun unary(op: Int): CUDARawTensor {
        val res = ops.createRaw(shape)
        check(KtcNative.unary.invokeExact(op, res.handle, handle, volume) as Int)
        return res
    }

    private fun compare(op: Int, value: Float): CUDARawTensor {
        val res = ops.createRaw(shape)
        check(KtcNative.compareScalar.invokeExact(op, res.handle, handle, value, volume) as Int)
        return res
    }

    override fun plus(other: AbstractRawTensor<CUDABuffer>) = binary(KtcNative.PLUS, other)
    override fun plus(constant: Float) = scalar(KtcNative.PLUS, constant)
    override fun plusAssign(other: AbstractRawTensor<CUDABuffer>) = binaryAssign(KtcNative.PLUS, other)
    override fun plusAssign(constant: Float) = scalarAssign(KtcNative.PLUS, constant)
    override fun minus(other: AbstractRawTensor<CUDABuffer>) = binary(KtcNative.MINUS, other)
    override fun minus(constant: Float) = scalar(KtcNative.MINUS, constant)
    override fun unaryMinus() = unary(KtcNative.NEG)
    override fun times(other: AbstractRawTensor<CUDABuffer>) = binary(KtcNative.TIMES, other)
    override fun timesAssign(other: AbstractRawTensor<CUDABuffer>) = binaryAssign(KtcNative.TIMES, other)
    override fun times(constant: Float) = scalar(KtcNative.TIMES, constant)
    override fun timesAssign(constant: Float) = scalarAssign(KtcNative.TIMES, constant)
    override fun div(other: AbstractRawTensor<CUDABuffer>) = binary(KtcNative.DIV, other)
    override fun div(constant: Float) = scalar(KtcNative.DIV, constant)
    override fun divAssign(constant: Float) = scalarAssign(KtcNative.DIV, constant)
    override fun pow(other: AbstractRawTensor<CUDABuffer>) = binary(KtcNative.POW, other)
    override fun pow(constant: Float) = scalar(KtcNative.POW, constant)
    override fun reciprocal() = unary(KtcNative.RECIPROCAL)
    override fun log() = unary(KtcNative.LOG)
    override fun exp() = unary(KtcNative.EXP)
    override fun tanh() = unary(KtcNative.TANH)
    override fun sigmoid() = unary(KtcNative.SIGMOID)

    override fun clamp(min: Float, max: Float): CUDARawTensor {
        val res = ops.createRaw(shape)
        check(KtcNative.clamp.invokeExact(res.handle, handle, min, max, volume) as Int)
        return res
    }

    override fun lt(value: Float) = compare(KtcNative.LT, value)
    override fun lte(value: Float) = compare(KtcNative.LTE, value)
    override fun gt(value: Float) = compare(KtcNative.GT, value)
    override fun gte(value: Float) = compare(KtcNative.GTE, value)

    // ---- reductions --------------------------------------------------------------------------------
    override fun aggregateOverAxis(axis: Int, resShape: List<Int>, aggregatingOperation: AggregatingOperation): CUDARawTensor {
        val outer = shape.take(axis).toStoreSize().toLong()
        val inner = shape.drop(axis + 1).toStoreSize().toLong()
        val op = when (aggregatingOperation) {
            AggregatingOperation.SUM -> KtcNative.SUM
            AggregatingOperation.MEAN -> KtcNative.MEAN
            AggregatingOperation.MAX -> KtcNative.MAX
            AggregatingOperation.MIN -> KtcNative.MIN
            AggregatingOperation.ARG_MAX -> KtcNative.ARGMAX
            AggregatingOperation.ARG_MIN -> KtcNative.ARGMIN
        }
        val res = ops.createRaw(resShape)
        check(KtcNative.reduceAxis.invokeExact(op, res.handle, handle, outer, shape[axis].toLong(), inner) as Int)
        return res
    }

    override fun sum(): CUDARawTensor = ops.createRaw(listOf(1)).also {
        check(KtcNative.reduceAll.invokeExact(KtcNative.SUM, it.handle, handle, volume) as Int)
    }

    override fun mean(): CUDARawTensor = ops.createRaw(listOf(1)).also {
        check(KtcNative.reduceAll.invokeExact(KtcNative.MEAN, it.handle, handle, volume) as Int)
    }

    override fun inplaceScatter(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: AbstractRawTensor<CUDABuffer>) {
        val a = shape.normalizeAxis(axis)
        if (index.shape[a] != 1 || index.shape != src.shape)
            throw UnsupportedOperationException("kten-cuda scatters one index per position along the axis (selection backward)")
        val outer = shape.take(a).toStoreSize().toLong()
        val inner = shape.drop(a + 1).toStoreSize().toLong()
        check(KtcNative.scatterAxis.invokeExact(handle, (index as CUDARawTensor).handle, (src as CUDARawTensor).handle,
                                                outer, shape[a].toLong(), inner) as Int)
    }

    // ---- broadcast, copies, host access ------------------------------------------------------------------
    override fun broadcastTo(shape: List<Int>): CUDARawTensor {
        if (this.shape == shape) return this
        this.shape.inferExplicitBroadcastShape(shape)
        val res = ops.createRaw(shape)
        Arena.ofConfined().use { arena ->
            check(KtcNative.broadcastTo.invokeExact(res.handle, KtcNative.shape(arena, shape), shape.size,
                                                    handle, KtcNative.shape(arena, this.shape), this.shape.size) as Int)
        }
        return res
    }

    override fun copy(shallow: Boolean): CUDARawTensor {
        if (shallow) {
            check(KtcNative.retain.invokeExact(handle) as Int)
            return CUDARawTensor(shape, storeReference, ops)
        }
        val res = ops.createRaw(shape)
        check(KtcNative.d2d.invokeExact(res.handle, 0L, handle, 0L, volume) as Int)
        return res
    }

    override fun view(shape: List<Int>): CUDARawTensor {
        check(KtcNative.retain.invokeExact(handle) as Int)
        return CUDARawTensor(this.shape.reshape(shape), storeReference, ops)
    }

    override fun getSingleValue(indexes: List<Int>): Float {
        val offset = shape.foldIndexed(0L) { i, acc, extent -> acc * extent + indexes[i] }
        Arena.ofConfined().use { arena ->
            val host = arena.allocate(JAVA_FLOAT)
            check(KtcNative.d2h.invokeExact(host, handle, offset, 1L, 1) as Int)
            return host.get(JAVA_FLOAT, 0)
        }
    }

    fun toFloatArray(): FloatArray {
        val n = volume
        Arena.ofConfined().use { arena ->
            val host = arena.allocate(JAVA_FLOAT, maxOf(1L, n))
            if (n > 0) check(KtcNative.d2h.invokeExact(host, handle, 0L, n, 1) as Int)
            return host.toArray(JAVA_FLOAT).copyOf(n.toInt())
        }
    }

    override fun inplaceFill(value: Float) = check(KtcNative.fill.invokeExact(handle, 0L, volume, value) as Int)

    override fun containsNan(): Boolean = toFloatArray().any { it.isNaN() }

    // ---- outside the float32 hot path: not provided by libkten_cuda.so yet -------------------------------
    private fun notOnHotPath(name: String): Nothing =
        throw UnsupportedOperationException("$name is not part of the kten-cuda hot path yet")

    override fun get(index: IntArray): AbstractRawTensor<CUDABuffer> = notOnHotPath("get")
    override fun get(index: Array<out IntRange>): AbstractRawTensor<CUDABuffer> = notOnHotPath("get")
    override fun set(index: IntArray, value: AbstractRawTensor<CUDABuffer>) = notOnHotPath("set")
    override fun set(index: Array<out IntRange>, value: AbstractRawTensor<CUDABuffer>) = notOnHotPath("set")
    override fun set(index: IntArray, value: Float) = notOnHotPath("set")
    override fun set(index: Array<out IntRange>, value: Float) = notOnHotPath("set")
    override fun inplaceScatterAdd(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: AbstractRawTensor<CUDABuffer>) = notOnHotPath("inplaceScatterAdd")
    override fun inplaceScatter(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: Float) = notOnHotPath("inplaceScatter(constant)")
    override fun gather(axis: Int, index: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("gather")
    override fun lt(tensor: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("lt(tensor)")
    override fun lte(tensor: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("lte(tensor)")
    override fun gt(tensor: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("gt(tensor)")
    override fun gte(tensor: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("gte(tensor)")
    override fun eq(tensor: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("eq(tensor)")
    override fun neq(tensor: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("neq(tensor)")
    override fun eq(value: Float): AbstractRawTensor<CUDABuffer> = notOnHotPath("eq")
    override fun neq(value: Float): AbstractRawTensor<CUDABuffer> = notOnHotPath("neq")
    override fun sinh(): AbstractRawTensor<CUDABuffer> = notOnHotPath("sinh")
    override fun cosh(): AbstractRawTensor<CUDABuffer> = notOnHotPath("cosh")
    override fun abs(): AbstractRawTensor<CUDABuffer> = notOnHotPath("abs")
    override fun sign(): AbstractRawTensor<CUDABuffer> = notOnHotPath("sign")
    override fun sqrt(): AbstractRawTensor<CUDABuffer> = notOnHotPath("sqrt")
    override fun sin(): AbstractRawTensor<CUDABuffer> = notOnHotPath("sin")
    override fun cos(): AbstractRawTensor<CUDABuffer> = notOnHotPath("cos")
    override fun tan(): AbstractRawTensor<CUDABuffer> = notOnHotPath("tan")
    override fun asin(): AbstractRawTensor<CUDABuffer> = notOnHotPath("asin")
    override fun acos(): AbstractRawTensor<CUDABuffer> = notOnHotPath("acos")
    override fun atan(): AbstractRawTensor<CUDABuffer> = notOnHotPath("atan")
    override fun floor(): AbstractRawTensor<CUDABuffer> = notOnHotPath("floor")
    override fun ceil(): AbstractRawTensor<CUDABuffer> = notOnHotPath("ceil")
    override fun round(): AbstractRawTensor<CUDABuffer> = notOnHotPath("round")
    override fun trunc(): AbstractRawTensor<CUDABuffer> = notOnHotPath("trunc")
    override fun rsqrt(): AbstractRawTensor<CUDABuffer> = notOnHotPath("rsqrt")
    override fun transpose(axis1: Int, axis2: Int): AbstractRawTensor<CUDABuffer> = notOnHotPath("transpose")
    override fun permute(axes: List<Int>): AbstractRawTensor<CUDABuffer> = notOnHotPath("permute")
    override fun narrow(axis: Int, start: Int, length: Int): AbstractRawTensor<CUDABuffer> = notOnHotPath("narrow")
    override fun dot(vector: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("dot")
    override fun indexSelect(axis: Int, index: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> = notOnHotPath("indexSelect")
    override fun indexAdd(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: AbstractRawTensor<CUDABuffer>, alpha: Float) = notOnHotPath("indexAdd")
    override fun inplaceResize(vararg shape: Int) = notOnHotPath("inplaceResize")
    override fun maskedFill(mask: AbstractRawTensor<CUDABuffer>, value: Float): AbstractRawTensor<CUDABuffer> = notOnHotPath("maskedFill")
}
