package eu.redbean.kten.cuda.tensor.operations

import eu.redbean.kten.api.autograd.tensor.NoGradVariable
import eu.redbean.kten.api.autograd.tensor.Variable
import eu.redbean.kten.api.autograd.utils.concatShapes
import eu.redbean.kten.api.autograd.utils.normalizeAxis
import eu.redbean.kten.api.autograd.utils.toStoreSize
import eu.redbean.kten.api.tensor.Tensor
import eu.redbean.kten.api.tensor.operations.TensorOperations
import eu.redbean.kten.api.tensor.operations.TensorOperationsGarbageCollector
import eu.redbean.kten.api.tensor.operations.nn.BatchNormOperation
import eu.redbean.kten.api.tensor.operations.nn.ConvolutionOperation
import eu.redbean.kten.api.tensor.operations.nn.PoolingOperation
import eu.redbean.kten.api.tensor.operations.nn.PoolingOptions
import eu.redbean.kten.api.tensor.operations.nn.Upsample2DOperation
import eu.redbean.kten.api.tensor.operations.nn.UpsampleType
import eu.redbean.kten.api.tensor.serialization.CommonSerializableTensorDescriptor
import eu.redbean.kten.api.tensor.serialization.SerializableTensorData
import eu.redbean.kten.api.tensor.store.AbstractRawTensor
import eu.redbean.kten.api.tensor.operations.nn.PoolingType
import eu.redbean.kten.cuda.tensor.operations.nn.CUDABatchNorm
import eu.redbean.kten.cuda.tensor.operations.nn.CUDASpatialPooling
import eu.redbean.kten.cuda.tensor.operations.nn.CUDAUpsample2DNearest
import eu.redbean.kten.cuda.tensor.platform.KtcNative
import eu.redbean.kten.cuda.tensor.platform.KtcNative.check
import eu.redbean.kten.cuda.tensor.store.CUDABuffer
import eu.redbean.kten.cuda.tensor.store.CUDARawTensor
import java.lang.foreign.Arena
import java.lang.foreign.ValueLayout.JAVA_FLOAT
import java.lang.foreign.ValueLayout.JAVA_LONG
import java.util.Random

/**
 * TensorOperations of one CUDA device.  Reference counting and the scoped garbage collector follow
 * the OpenCL backend (OCLTensorOperations.kt:72-94): raw tensors created while a scope is open are
 * released when it closes unless their reference count was raised or they were marked to survive.
 */
class CUDATensorOperations(override val platformKey: String, val device: Int) : TensorOperations<CUDARawTensor> {

    private val collector = ThreadLocal<MutableList<CUDARawTensor>?>()

    /**
     * Deferred mode: elementwise calls and sums on raw tensors are recorded by the library's expression recorder
     * (ktc_lazy_*) instead of running at once; the recorder fuses them into one kernel per iteration space when a
     * value is needed.  Results equal the call-by-call results bit for bit (sums: up to summation order).
     */
    var lazy = System.getenv("KTEN_CUDA_LAZY") == "1"      // the process-wide default (off: every call runs at once, like kten-jvm)
    var deferSums = true
        set(value) { field = value; setRecorderOption("defer_sums", if (value) 1 else 0) }

    /** buffers with a recorded `+= pending sum` update; may hold stale entries (the recorder runs updates on its own too) */
    internal val pendingTargets = HashSet<Long>()

    internal fun runPending() {
        pendingTargets.clear()
        check(KtcNative.lazyRunPending.invokeExact() as Int)
    }

    /** before `handle` is written by a call the recorder does not see */
    internal fun flush(handle: Long) {
        pendingTargets.remove(handle)
        check(KtcNative.lazyFlush.invokeExact(handle) as Int)
    }

    fun setRecorderOption(name: String, value: Int) = Arena.ofConfined().use { arena ->
        check(KtcNative.lazyOption.invokeExact(arena.allocateFrom(name), value) as Int)
    }

    /** Sum raw tensors over the ranks of a peer-memory communicator, in place; pending work runs first and takes the exchange along. */
    fun allreduceSum(comm: Long, tensors: List<CUDARawTensor>) = Arena.ofConfined().use { arena ->
        val cells = arena.allocate(JAVA_LONG, tensors.size.toLong())
        tensors.forEachIndexed { i, t -> cells.setAtIndex(JAVA_LONG, i.toLong(), t.cell(applyUpdates = false)) }
        check(KtcNative.lazyAllreduce.invokeExact(comm, cells, tensors.size) as Int)
        pendingTargets.clear()
    }

    internal fun instanceCreated(raw: CUDARawTensor) {
        collector.get()?.add(raw)
    }

    override fun garbageCollector(): TensorOperationsGarbageCollector {
        if (collector.get() != null) return TensorOperationsGarbageCollector { }        // nested scopes are no-ops
        collector.set(mutableListOf())
        return TensorOperationsGarbageCollector {
            val created = collector.get()
            collector.set(null)
            created?.forEach { it.release() }
        }
    }

    override fun createRaw(shape: List<Int>): CUDARawTensor {
        Arena.ofConfined().use { arena ->
            val out = arena.allocate(JAVA_LONG)
            check(KtcNative.alloc.invokeExact(device, shape.toStoreSize().toLong(), out) as Int)
            return CUDARawTensor(shape, CUDABuffer(out.get(JAVA_LONG, 0), shape.toStoreSize()), this)
        }
    }

    override fun createRaw(shape: List<Int>, init: (Int) -> Float): CUDARawTensor {
        val raw = createRaw(shape)
        upload(raw, FloatArray(shape.toStoreSize(), init))
        return raw
    }

    override fun createRawFill(shape: List<Int>, constant: Float): CUDARawTensor {
        if (!lazy) return createRaw(shape).also { it.inplaceFill(constant) }
        // a pending constant: no buffer and no fill until somebody needs one
        val cell = Arena.ofConfined().use { arena ->
            KtcNative.cell { out -> KtcNative.lazyFull.invokeExact(device, KtcNative.shape(arena, shape), shape.size, constant, out) as Int }
        }
        return CUDARawTensor(shape, CUDABuffer(0L, shape.toStoreSize()).also { it.lz = cell; it.lzShape = shape }, this)
    }

    internal fun upload(raw: CUDARawTensor, data: FloatArray) {
        if (data.isEmpty()) return
        Arena.ofConfined().use { arena ->
            val host = arena.allocateFrom(JAVA_FLOAT, *data)
            check(KtcNative.h2d.invokeExact(raw.bufferForWrite(), 0L, host, data.size.toLong(), 1) as Int)
        }
    }

    override fun create(shape: List<Int>, requiresGrad: Boolean, init: (Int) -> Float): Tensor = wrap(createRaw(shape, init), requiresGrad)

    override fun createRandom(shape: List<Int>, requiresGrad: Boolean): Tensor {
        val rnd = Random()
        return wrap(createRaw(shape) { rnd.nextGaussian().toFloat() }, requiresGrad)
    }

    override fun createBernoulli(shape: List<Int>, rate: Float, requiresGrad: Boolean): Tensor {
        val rnd = Random()
        return wrap(createRaw(shape) { if (rnd.nextFloat() < rate) 1.0f else 0.0f }, requiresGrad)
    }

    @Suppress("UNCHECKED_CAST")
    private fun wrap(raw: CUDARawTensor, requiresGrad: Boolean): Tensor {
        val ops = this as TensorOperations<AbstractRawTensor<Any>>
        return if (requiresGrad) Variable(ops, raw as AbstractRawTensor<Any>) else NoGradVariable(ops, raw as AbstractRawTensor<Any>)
    }

    override fun release(vararg rawTensors: AbstractRawTensor<Any>) = rawTensors.forEach { (it as AbstractRawTensor<*> as CUDARawTensor).release() }
    override fun incrementRef(rawTensor: CUDARawTensor) { rawTensor.refCount++ }
    override fun markSurviveGC(rawTensor: AbstractRawTensor<Any>) { (rawTensor as AbstractRawTensor<*> as CUDARawTensor).mustSurviveGC = true }
    override fun markReleasableInGC(rawTensor: AbstractRawTensor<Any>) { (rawTensor as AbstractRawTensor<*> as CUDARawTensor).mustSurviveGC = false }
    override fun zerosLike(rawTensor: CUDARawTensor): CUDARawTensor = createRawFill(rawTensor.shape, 0.0f)
    override fun zeroOut(rawTensor: CUDARawTensor) = rawTensor.inplaceFill(0.0f)
    override fun pow(constant: Float, rawTensor: CUDARawTensor): CUDARawTensor = rawTensor.scalar(KtcNative.POW, constant, scalarFirst = true)

    override fun toSerializableData(rawTensor: CUDARawTensor) = SerializableTensorData(rawTensor.shape, rawTensor.toFloatArray())

    override fun fromCommonSerializable(commonDescriptor: CommonSerializableTensorDescriptor): Tensor {
        val data = commonDescriptor.data
        val value = createRaw(data.shape) { data.data[it] }
        val grad = commonDescriptor.gradientData
        @Suppress("UNCHECKED_CAST")
        val ops = this as TensorOperations<AbstractRawTensor<Any>>
        @Suppress("UNCHECKED_CAST")
        return if (grad != null) Variable(ops, value as AbstractRawTensor<Any>, createRaw(grad.shape) { grad.data[it] } as AbstractRawTensor<Any>)
        else NoGradVariable(ops, value as AbstractRawTensor<Any>)
    }

    // ---- dense contractions and nn layers are outside the float32 hot path this library covers -----------
    private fun unsupported(name: String): Nothing = throw UnsupportedOperationException("$name is not provided by kten-cuda")

    // AbstractJVMTensorOperations.kt:106-120: every input is set into its range of the result
    override fun concat(axis: Int, inputs: List<CUDARawTensor>): CUDARawTensor {
        val shapes = inputs.map { it.shape }
        val resShape = concatShapes(shapes, axis)
        val normAxis = shapes[0].normalizeAxis(axis)
        val ranges = resShape.map { 0 until it }.toTypedArray()
        val res = createRaw(resShape)
        var last = 0
        for (input in inputs) {
            ranges[normAxis] = last until (last + input.shape[normAxis])
            res[ranges] = input
            last += input.shape[normAxis]
        }
        return res
    }
    override fun gemm(addMatrix: CUDARawTensor, matrix1: CUDARawTensor, matrix2: CUDARawTensor, alpha: Float, beta: Float,
                      transposeFirst: Boolean, transposeSecond: Boolean): CUDARawTensor = unsupported("gemm")
    override fun gemv(addVector: CUDARawTensor, matrix: CUDARawTensor, vector: CUDARawTensor, alpha: Float, beta: Float,
                      transposeMatrix: Boolean): CUDARawTensor = unsupported("gemv")
    override fun gemmBatched(addTensor: CUDARawTensor, tensor1: CUDARawTensor, tensor2: CUDARawTensor, alpha: Float, beta: Float,
                             transposeFirst: Boolean, transposeSecond: Boolean): CUDARawTensor = unsupported("gemmBatched")
    override fun ger(vector1: CUDARawTensor, vector2: CUDARawTensor, matrix: CUDARawTensor, alpha: Float): CUDARawTensor = unsupported("ger")
    override fun spatialConvolution(kernel: List<Int>, padding: List<Int>, stride: List<Int>, dilation: List<Int>): ConvolutionOperation<CUDARawTensor> = unsupported("spatialConvolution")
    override fun spatialConvolutionTranspose(kernel: List<Int>, padding: List<Int>, stride: List<Int>, dilation: List<Int>,
                                             outputPadding: List<Int>): ConvolutionOperation<CUDARawTensor> = unsupported("spatialConvolutionTranspose")
    override fun volumetricConvolution(kernel: List<Int>, padding: List<Int>, stride: List<Int>, dilation: List<Int>): ConvolutionOperation<CUDARawTensor> = unsupported("volumetricConvolution")
    override fun volumetricConvolutionTranspose(kernel: List<Int>, padding: List<Int>, stride: List<Int>, dilation: List<Int>,
                                                outputPadding: List<Int>): ConvolutionOperation<CUDARawTensor> = unsupported("volumetricConvolutionTranspose")
    override fun spatialPooling(kernel: List<Int>, padding: List<Int>, stride: List<Int>, dilation: List<Int>,
                                options: PoolingOptions): PoolingOperation<CUDARawTensor> =
        CUDASpatialPooling(kernel, padding, stride, if (options.type == PoolingType.MAX) dilation else listOf(1, 1), options, this)
    // reductions and broadcast maps: built from raw-tensor calls on the path's kernels (operations/nn/CUDANnOperations.kt)
    override fun batchNorm(axis: Int, momentum: Float, epsilon: Float, training: Boolean): BatchNormOperation<CUDARawTensor> =
        CUDABatchNorm(axis, momentum, epsilon, training, this)
    override fun upsample(upsampleType: UpsampleType, scale: Int): Upsample2DOperation<CUDARawTensor> = when (upsampleType) {
        UpsampleType.NEAREST -> CUDAUpsample2DNearest(scale, this)
    }
}
