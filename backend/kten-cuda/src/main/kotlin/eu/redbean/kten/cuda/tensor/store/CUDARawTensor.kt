package eu.redbean.kten.cuda.tensor.store

import eu.redbean.kten.api.autograd.utils.indexAddCheckShapesNormAxis
import eu.redbean.kten.api.autograd.utils.indexSelectNormAxisShape
import eu.redbean.kten.api.autograd.utils.inferExplicitBroadcastShape
import eu.redbean.kten.api.autograd.utils.normalizeAxis
import eu.redbean.kten.api.autograd.utils.normalizeIndex
import eu.redbean.kten.api.autograd.utils.normalizedAxisScatter
import eu.redbean.kten.api.autograd.utils.normalizedIndexedShape
import eu.redbean.kten.api.autograd.utils.permute
import eu.redbean.kten.api.autograd.utils.reshape
import eu.redbean.kten.api.autograd.utils.toStoreSize
import eu.redbean.kten.api.autograd.utils.transposeNormalizeAxes
import eu.redbean.kten.api.tensor.platform.PlatformProvider
import eu.redbean.kten.api.tensor.store.AbstractRawTensor
import eu.redbean.kten.api.tensor.store.AggregatingOperation
import eu.redbean.kten.cuda.tensor.operations.CUDATensorOperations
import eu.redbean.kten.cuda.tensor.platform.KtcNative
import eu.redbean.kten.cuda.tensor.platform.KtcNative.check
import java.lang.foreign.Arena
import java.lang.foreign.MemorySegment
import java.lang.foreign.ValueLayout.JAVA_FLOAT
import java.lang.foreign.ValueLayout.JAVA_INT
import java.lang.foreign.ValueLayout.JAVA_LONG

/**
 * Storage slot of one or more raw tensors: a reference-counted buffer handle of libkten_cuda.so (one owned reference),
 * or a cell of the library's expression recorder whose value is still pending, or both (the recorder cell then stands
 * for the buffer when the tensor is an operand of a recorded call).  Shallow copies of a pending tensor share the slot,
 * so that they end up sharing storage exactly as in the other backends; every other tensor has a slot of its own.
 */
class CUDABuffer(var handle: Long, val size: Int) {
    var lz = 0L                          // recorder cell, 0: none
    var lzShape: List<Int>? = null
    var share = 1
}

/**
 * RawTensor of the kten-cuda backend: shape on the JVM heap, data in HBM.  Every operation of the
 * float32 hot path is one call through the C ABI -- run at once, or, with `ops.lazy`, recorded by the
 * library's expression recorder and run fused when a value is needed; operations outside that path are not
 * provided by the native library yet and throw UnsupportedOperationException.
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

    /** The buffer handle; a pending value is computed first, a recorded `+= pending sum` update of the buffer applied. */
    internal val handle: Long
        get() {
            if (released) throw IllegalStateException("Raw tensor already released")
            val slot = storeReference
            if (slot.handle == 0L) {
                slot.handle = KtcNative.cell { out -> KtcNative.lazyBuffer.invokeExact(slot.lz, out) as Int }     // one reference for this slot
            } else if (ops.pendingTargets.isNotEmpty() && slot.handle in ops.pendingTargets) ops.runPending()
            return slot.handle
        }

    /** The handle of a buffer that is about to be written by a call the recorder does not see. */
    internal fun bufferForWrite(): Long {
        val h = handle
        ops.flush(h)
        return h
    }

    /** This tensor as an operand of a recorded call: its recorder cell (a stored tensor gets one over its buffer). */
    internal fun cell(applyUpdates: Boolean = true): Long {
        if (released) throw IllegalStateException("Raw tensor already released")
        val slot = storeReference
        if (slot.handle == 0L) return slot.lz
        if (applyUpdates && ops.pendingTargets.isNotEmpty() && slot.handle in ops.pendingTargets) ops.runPending()
        if (slot.lz == 0L || slot.lzShape != shape) {
            if (slot.lz != 0L) check(KtcNative.lazyFree.invokeExact(slot.lz) as Int)
            slot.lz = Arena.ofConfined().use { arena ->
                KtcNative.cell { out -> KtcNative.lazyLeaf.invokeExact(slot.handle, KtcNative.shape(arena, shape), shape.size, out) as Int }
            }
            slot.lzShape = shape
        }
        return slot.lz
    }

    private val isDeferred: Boolean
        get() {
            val slot = storeReference
            if (slot.handle != 0L || slot.lz == 0L) return false
            return Arena.ofConfined().use { arena ->
                val pending = arena.allocate(JAVA_INT)
                check(KtcNative.lazyInfo.invokeExact(slot.lz, pending, MemorySegment.NULL, MemorySegment.NULL, MemorySegment.NULL) as Int)
                pending.get(JAVA_INT, 0) != 0
            }
        }

    /**
     * SoftmaxCrossEntropy.doForward (SoftmaxCrossEntropy.kt:40-59) in one pass over the logits: the saved softmax and the
     * per-row negative log-likelihood with the bits of the call sequence; null when rows of this length are not handled,
     * and the caller issues the calls as written.
     */
    fun softmaxCrossEntropyForward(targets: CUDARawTensor, lo: Float, hi: Float): Pair<CUDARawTensor, CUDARawTensor>? {
        if (shape.size != 2) return null
        if (ops.lazy) {
            // recorded: the kernel runs when the loss or the gradient is needed and takes the recorded backward with it -- the
            // saved softmax is then written only if a tensor still holds it (ktc_lazy_softmax_xent_forward)
            val cells = Arena.ofConfined().use { arena ->
                val sm = arena.allocate(JAVA_LONG); val nl = arena.allocate(JAVA_LONG)
                val status = KtcNative.lazySoftmaxXentForward.invokeExact(cell(), targets.cell(), lo, hi, sm, nl) as Int
                if (status == KtcNative.ENOTSUP) null else { check(status); sm.get(JAVA_LONG, 0) to nl.get(JAVA_LONG, 0) }
            }
            if (cells != null) return recorded(shape, cells.first) to recorded(listOf(shape[0], 1), cells.second)
        }
        val softmax = ops.createRaw(shape)
        val nll = ops.createRaw(listOf(shape[0], 1))
        val status = KtcNative.softmaxXentForward.invokeExact(softmax.handle, nll.handle, handle, targets.handle,
                                                              shape[0].toLong(), shape[1].toLong(), lo, hi) as Int
        if (status == KtcNative.ENOTSUP) { ops.release(softmax, nll); return null }
        check(status)
        return softmax to nll
    }

    /**
     * SoftmaxCrossEntropy.doBackward (SoftmaxCrossEntropy.kt:61-67) on the saved softmax (`this`) as one program of
     * ktc_expr_eval: zerosLike, -1 scattered at the targets, `+= softmax`, `/= rows` -- the same four operations with
     * their own roundings, one pass instead of four.  null when the calls are recorded anyway (the recorder fuses them
     * itself, and with the forward) or the program is declined: the caller issues the calls.
     */
    fun softmaxCrossEntropyBackward(targets: CUDARawTensor, rows: Int): CUDARawTensor? {
        if (ops.lazy || shape.size != 2 || shape[1] % 4 != 0) return null
        fun ins(op: Int, d: Int = 0, a: Int = 0, b: Int = 0, k: Int = 0) = op or (d shl 8) or (a shl 12) or (b shl 16) or (k shl 20)
        // leaves: 0 the targets [rows, 1], 1 the softmax; immediates: 0f, -1f, rows
        val code = intArrayOf(ins(KtcNative.X_CONST, 0, k = 0), ins(KtcNative.X_LOAD, 1, k = 0), ins(KtcNative.X_SCATC, 0, 0, 1, k = 1),
                              ins(KtcNative.X_LOAD, 1, k = 1), ins(KtcNative.X_ADD, 0, 0, 1), ins(KtcNative.X_CONST, 1, k = 2),
                              ins(KtcNative.X_DIV, 0, 0, 1), ins(KtcNative.X_STORE, a = 0, k = 0))
        val grad = ops.createRaw(shape)
        val status = Arena.ofConfined().use { arena ->
            KtcNative.exprEval.invokeExact(arena.allocateFrom(JAVA_INT, *code), code.size,
                arena.allocateFrom(java.lang.foreign.ValueLayout.JAVA_FLOAT, 0f, -1f, rows.toFloat()), 3,
                arena.allocateFrom(JAVA_LONG, shape[0].toLong(), shape[1].toLong()), 2,
                arena.allocateFrom(JAVA_LONG, targets.handle, handle),
                arena.allocateFrom(JAVA_LONG, shape[0].toLong(), 1L, shape[0].toLong(), shape[1].toLong()), 2,
                arena.allocateFrom(JAVA_LONG, grad.handle), 1, 0 /* KTC_EXPR_STORE_ONLY */, 0L, 0) as Int
        }
        if (status == KtcNative.ENOTSUP) { ops.release(grad); return null }
        check(status)
        return grad
    }

    internal fun recorded(shape: List<Int>, cell: Long): CUDARawTensor =
        CUDARawTensor(shape, CUDABuffer(0L, shape.toStoreSize()).also { it.lz = cell; it.lzShape = shape }, ops)

    /** What an in-place call through the recorder left behind (ktc_lazy_assign_*). */
    private fun afterAssign(state: Int) {
        val slot = storeReference
        when (state) {
            KtcNative.ASSIGN_PENDING -> if (slot.handle != 0L) {       // the value is pending now; the old buffer belongs to the recorder
                check(KtcNative.release.invokeExact(slot.handle) as Int)
                slot.handle = 0L
            }
            KtcNative.ASSIGN_UPDATE_RECORDED -> ops.pendingTargets.add(slot.handle)
            // ASSIGN_UPDATE_OF_ZEROED: the recorder gave the (pending, all-zero) cell a buffer that receives 0f + sum; nothing to do here
        }
    }

    private fun assignState(call: (MemorySegment) -> Int): Int = Arena.ofConfined().use { arena ->
        val state = arena.allocate(JAVA_INT)
        check(call(state))
        state.get(JAVA_INT, 0)
    }

    private val volume: Long get() = shape.toStoreSize().toLong()

    internal fun release(): Boolean {
        if (released) return false
        if (!mustSurviveGC) refCount--
        if (refCount <= 0) {
            val slot = storeReference
            if (--slot.share <= 0) {
                if (slot.handle != 0L) check(KtcNative.release.invokeExact(slot.handle) as Int)
                if (slot.lz != 0L) { check(KtcNative.lazyFree.invokeExact(slot.lz) as Int); slot.lz = 0L }
            }
            released = true
            return true
        }
        return false
    }

    // ---- elementwise -------------------------------------------------------------------------------
    private fun binary(op: Int, other: AbstractRawTensor<CUDABuffer>): CUDARawTensor {
        other as CUDARawTensor
        if (ops.lazy) {
            val common = if (shape == other.shape) shape else calculateCommonShapeWith(other)
            return recorded(common, KtcNative.cell { out -> KtcNative.lazyBinary.invokeExact(op, cell(), other.cell(), out) as Int })
        }
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
        other as CUDARawTensor
        if (ops.lazy) {
            afterAssign(assignState { state -> KtcNative.lazyAssignBinary.invokeExact(op, cell(), other.cell(), state) as Int })
            return
        }
        check(KtcNative.binaryInplace.invokeExact(op, bufferForWrite(), other.handle, volume) as Int)
    }

    internal fun scalar(op: Int, constant: Float, scalarFirst: Boolean = false): CUDARawTensor {
        if (ops.lazy)
            return recorded(shape, KtcNative.cell { out -> KtcNative.lazyScalar.invokeExact(op, cell(), constant, if (scalarFirst) 1 else 0, out) as Int })
        val res = ops.createRaw(shape)
        check(KtcNative.scalar.invokeExact(op, res.handle, handle, constant, volume, if (scalarFirst) 1 else 0) as Int)
        return res
    }

    private fun scalarAssign(op: Int, constant: Float) {
        if (ops.lazy) {
            afterAssign(assignState { state -> KtcNative.lazyAssignScalar.invokeExact(op, cell(), constant, state) as Int })
            return
        }
        check(KtcNative.scalarInplace.invokeExact(op, bufferForWrite(), constant, volume) as Int)
    }

    private fun unary(op: Int): CUDARawTensor {
        if (ops.lazy && (op <= KtcNative.NEG || op == KtcNative.SQRT || op == KtcNative.RSQRT || op == KtcNative.ABS))   // the maps that are expression instructions
            return recorded(shape, KtcNative.cell { out -> KtcNative.lazyUnary.invokeExact(op, cell(), out) as Int })
        val res = ops.createRaw(shape)
        check(KtcNative.unary.invokeExact(op, res.handle, handle, volume) as Int)
        return res
    }

    private fun compare(op: Int, value: Float): CUDARawTensor {
        if (ops.lazy) return recorded(shape, KtcNative.cell { out -> KtcNative.lazyCompareScalar.invokeExact(op, cell(), value, out) as Int })
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
        if (ops.lazy) return recorded(shape, KtcNative.cell { out -> KtcNative.lazyClamp.invokeExact(cell(), min, max, out) as Int })
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
        // sums of a pending value over the leading or the innermost axis join its expression (resShape keeps the axis as 1)
        if (op == KtcNative.SUM && shape.size >= 2 && isDeferred) {
            val kind = if (axis == 0) KtcNative.EXPR_SUM_ROWS else if (axis == shape.size - 1 && shape[axis] > 1 && ops.deferSums) KtcNative.EXPR_SUM_LAST else 0
            if (kind != 0) return recordedSum(kind, false, resShape)
        }
        val res = ops.createRaw(resShape)
        check(KtcNative.reduceAxis.invokeExact(op, res.handle, handle, outer, shape[axis].toLong(), inner) as Int)
        return res
    }

    private fun recordedSum(kind: Int, mean: Boolean, resShape: List<Int>): CUDARawTensor = Arena.ofConfined().use { arena ->
        recorded(resShape, KtcNative.cell { out ->
            KtcNative.lazySum.invokeExact(cell(), kind, if (mean) 1 else 0, KtcNative.shape(arena, resShape), resShape.size, out) as Int
        })
    }

    override fun sum(): CUDARawTensor {
        if (isDeferred) return recordedSum(KtcNative.EXPR_SUM_ALL, false, listOf(1))
        return ops.createRaw(listOf(1)).also { check(KtcNative.reduceAll.invokeExact(KtcNative.SUM, it.handle, handle, volume) as Int) }
    }

    override fun mean(): CUDARawTensor {
        if (isDeferred) return recordedSum(KtcNative.EXPR_SUM_ALL, true, listOf(1))
        return ops.createRaw(listOf(1)).also { check(KtcNative.reduceAll.invokeExact(KtcNative.MEAN, it.handle, handle, volume) as Int) }
    }

    // one index per position along the axis over the whole target (Max / Min backward): fully parallel kernel;
    // every other form: the general kernel, sequential along the axis like JVMRawTensor.kt:227-247
    override fun inplaceScatter(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: AbstractRawTensor<CUDABuffer>) {
        val a = shape.normalizedAxisScatter(axis, index.shape, src.shape)
        val offAxis = { s: List<Int> -> s.filterIndexed { i, _ -> i != a } }
        if (index.shape[a] == 1 && index.shape == src.shape && offAxis(index.shape) == offAxis(shape)) {
            val outer = shape.take(a).toStoreSize().toLong()
            val inner = shape.drop(a + 1).toStoreSize().toLong()
            check(KtcNative.scatterAxis.invokeExact(bufferForWrite(), (index as CUDARawTensor).handle, (src as CUDARawTensor).handle,
                                                    outer, shape[a].toLong(), inner) as Int)
        } else scatterNd(KtcNative.SCATTER_SET, a, index as CUDARawTensor, src as CUDARawTensor, 0f)
    }

    override fun inplaceScatterAdd(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: AbstractRawTensor<CUDABuffer>) =
        scatterNd(KtcNative.SCATTER_ADD, shape.normalizedAxisScatter(axis, index.shape, src.shape), index as CUDARawTensor, src as CUDARawTensor, 0f)

    override fun inplaceScatter(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: Float) {
        val a = shape.normalizeAxis(axis)
        if (ops.lazy && a == shape.size - 1 && shape[a] > 1 && index.shape == shape.dropLast(1) + 1) {
            // one index per row along the last axis (the -1 at the target of SoftmaxCrossEntropy.doBackward): an expression instruction
            var state = -1
            val status = Arena.ofConfined().use { arena ->
                val out = arena.allocate(JAVA_INT)
                (KtcNative.lazyAssignScatterConst.invokeExact(cell(), (index as CUDARawTensor).cell(), src, out) as Int).also { state = out.get(JAVA_INT, 0) }
            }
            if (status == 0) { afterAssign(state); return }
            if (status != KtcNative.ENOTSUP) check(status)
        }
        scatterNd(KtcNative.SCATTER_CONST, a, index as CUDARawTensor, null, src)
    }

    private fun scatterNd(mode: Int, axis: Int, index: CUDARawTensor, src: CUDARawTensor?, constant: Float) {
        Arena.ofConfined().use { arena ->
            check(KtcNative.scatterAxisNd.invokeExact(mode, bufferForWrite(), KtcNative.shape(arena, shape), index.handle, KtcNative.shape(arena, index.shape),
                                                      src?.handle ?: 0L, if (src == null) MemorySegment.NULL else KtcNative.shape(arena, src.shape),
                                                      shape.size, axis, constant) as Int)
        }
    }

    // ---- broadcast, copies, host access ------------------------------------------------------------------
    override fun broadcastTo(shape: List<Int>): CUDARawTensor {
        if (this.shape == shape) return this
        this.shape.inferExplicitBroadcastShape(shape)
        if (ops.lazy) return Arena.ofConfined().use { arena ->
            recorded(shape, KtcNative.cell { out -> KtcNative.lazyBroadcastTo.invokeExact(cell(), KtcNative.shape(arena, shape), shape.size, out) as Int })
        }
        val res = ops.createRaw(shape)
        Arena.ofConfined().use { arena ->
            check(KtcNative.broadcastTo.invokeExact(res.handle, KtcNative.shape(arena, shape), shape.size,
                                                    handle, KtcNative.shape(arena, this.shape), this.shape.size) as Int)
        }
        return res
    }

    override fun copy(shallow: Boolean): CUDARawTensor {
        if (shallow) {
            if (isDeferred) {                                    // aliases share the pending value, later its storage
                storeReference.share++
                return CUDARawTensor(shape, storeReference, ops)
            }
            check(KtcNative.retain.invokeExact(handle) as Int)
            return CUDARawTensor(shape, CUDABuffer(storeReference.handle, storeReference.size), ops)
        }
        if (isDeferred) return Arena.ofConfined().use { arena ->   // pending values are immutable: a deep copy can share one
            recorded(shape, KtcNative.cell { out -> KtcNative.lazyBroadcastTo.invokeExact(cell(), KtcNative.shape(arena, shape), shape.size, out) as Int })
        }
        val res = ops.createRaw(shape)
        check(KtcNative.d2d.invokeExact(res.handle, 0L, handle, 0L, volume) as Int)
        return res
    }

    override fun view(shape: List<Int>): CUDARawTensor {
        check(KtcNative.retain.invokeExact(handle) as Int)
        return CUDARawTensor(this.shape.reshape(shape), CUDABuffer(storeReference.handle, storeReference.size), ops)
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

    override fun inplaceFill(value: Float) {
        val slot = storeReference
        if (ops.lazy && (slot.handle != 0L || slot.lz != 0L)) {
            // recorded: a pending tensor, or a stored one whose buffer nobody else holds, becomes a pending constant
            // (zeroing a gradient before a backward pass costs no kernel and no traffic); others are filled at once
            afterAssign(assignState { state -> KtcNative.lazyAssignFill.invokeExact(cell(), value, state) as Int })
            return
        }
        if (slot.handle == 0L) {                                 // a pending value is overwritten: just take storage
            if (slot.lz != 0L) { check(KtcNative.lazyFree.invokeExact(slot.lz) as Int); slot.lz = 0L }
            slot.handle = KtcNative.cell { out -> KtcNative.alloc.invokeExact(ops.device, volume, out) as Int }
        }
        check(KtcNative.fill.invokeExact(bufferForWrite(), 0L, volume, value) as Int)
    }

    override fun containsNan(): Boolean = Arena.ofConfined().use { arena ->
        val res = arena.allocate(JAVA_INT)
        check(KtcNative.containsNan.invokeExact(handle, volume, res) as Int)
        res.get(JAVA_INT, 0) != 0
    }

    // ---- the remaining maps and compares (JVMRawTensor.kt:355-435) ---------------------------------------
    override fun sinh() = unary(KtcNative.SINH)
    override fun cosh() = unary(KtcNative.COSH)
    override fun abs() = unary(KtcNative.ABS)
    override fun sign() = unary(KtcNative.SIGN)
    override fun sqrt() = unary(KtcNative.SQRT)
    override fun sin() = unary(KtcNative.SIN)
    override fun cos() = unary(KtcNative.COS)
    override fun tan() = unary(KtcNative.TAN)
    override fun asin() = unary(KtcNative.ASIN)
    override fun acos() = unary(KtcNative.ACOS)
    override fun atan() = unary(KtcNative.ATAN)
    override fun floor() = unary(KtcNative.FLOOR)
    override fun ceil() = unary(KtcNative.CEIL)
    override fun round() = unary(KtcNative.ROUND)
    override fun trunc() = unary(KtcNative.TRUNC)
    override fun rsqrt() = unary(KtcNative.RSQRT)

    private fun compareTensor(op: Int, tensor: AbstractRawTensor<CUDABuffer>): CUDARawTensor {
        if (shape != tensor.shape)                               // kten-jvm's tensor compares do not broadcast
            throw IllegalArgumentException("Tensor compare needs equal shapes, got $shape and ${tensor.shape}")
        val res = ops.createRaw(shape)
        check(KtcNative.compareTensor.invokeExact(op, res.handle, handle, (tensor as CUDARawTensor).handle, PlatformProvider.epsilon, volume) as Int)
        return res
    }

    private fun compareEps(op: Int, value: Float): CUDARawTensor {
        val res = ops.createRaw(shape)
        check(KtcNative.compareScalarEps.invokeExact(op, res.handle, handle, value, PlatformProvider.epsilon, volume) as Int)
        return res
    }

    override fun lt(tensor: AbstractRawTensor<CUDABuffer>) = compareTensor(KtcNative.LT, tensor)
    override fun lte(tensor: AbstractRawTensor<CUDABuffer>) = compareTensor(KtcNative.LTE, tensor)
    override fun gt(tensor: AbstractRawTensor<CUDABuffer>) = compareTensor(KtcNative.GT, tensor)
    override fun gte(tensor: AbstractRawTensor<CUDABuffer>) = compareTensor(KtcNative.GTE, tensor)
    override fun eq(tensor: AbstractRawTensor<CUDABuffer>) = compareTensor(KtcNative.EQ, tensor)
    override fun neq(tensor: AbstractRawTensor<CUDABuffer>) = compareTensor(KtcNative.NEQ, tensor)
    override fun eq(value: Float) = compareEps(KtcNative.EQ, value)
    override fun neq(value: Float) = compareEps(KtcNative.NEQ, value)

    override fun maskedFill(mask: AbstractRawTensor<CUDABuffer>, value: Float): CUDARawTensor {
        mask.shape.inferExplicitBroadcastShape(shape)
        val res = ops.createRaw(shape)
        Arena.ofConfined().use { arena ->
            check(KtcNative.maskedFill.invokeExact(res.handle, handle, KtcNative.shape(arena, shape), shape.size,
                                                   (mask as CUDARawTensor).handle, KtcNative.shape(arena, mask.shape), mask.shape.size, value) as Int)
        }
        return res
    }

    // ---- slices, permutes, gather / index ops (JVMRawTensor.kt:270-353, 437-518) -----------------------------
    private fun strides(s: List<Int>): List<Int> = s.indices.map { s.drop(it + 1).toStoreSize() }

    /** offset, box shape and this tensor's strides for a normalised range index (trailing dimensions whole) */
    private fun box(ranges: List<IntRange>): Triple<Long, List<Int>, List<Int>> {
        val st = strides(shape)
        val offset = ranges.foldIndexed(0L) { d, acc, r -> acc + r.first.toLong() * st[d] }
        return Triple(offset, ranges.map { it.last - it.first + 1 } + shape.drop(ranges.size), st)
    }

    private fun copyBox(dst: CUDARawTensor, dstOffset: Long, dstStrides: List<Int>, src: CUDARawTensor, srcOffset: Long, srcStrides: List<Int>, box: List<Int>) =
        Arena.ofConfined().use { arena ->
            check(KtcNative.copyStrided.invokeExact(dst.handle, dstOffset, KtcNative.shape(arena, dstStrides), src.handle, srcOffset,
                                                    KtcNative.shape(arena, srcStrides), KtcNative.shape(arena, box), box.size) as Int)
        }

    override fun get(index: IntArray): CUDARawTensor {
        val (norm, resShape) = shape.normalizedIndexedShape(index)
        val sub = shape.drop(norm.size).toStoreSize().toLong()
        val start = norm.foldIndexed(0L) { d, acc, i -> acc * shape[d] + i }
        val res = ops.createRaw(resShape)
        check(KtcNative.d2d.invokeExact(res.handle, 0L, handle, start * sub, sub) as Int)
        return res
    }

    override fun get(index: Array<out IntRange>): CUDARawTensor {
        val (norm, resShape) = shape.normalizedIndexedShape(index)
        val (offset, boxShape, st) = box(norm.toList())
        val res = ops.createRaw(resShape)
        copyBox(res, 0L, strides(boxShape), this, offset, st, boxShape)
        return res
    }

    private fun setBox(ranges: List<IntRange>, value: CUDARawTensor?, constant: Float, indexForMessage: List<*>) {
        val (offset, boxShape, st) = box(ranges)
        if (value != null) {
            if (value.volume != boxShape.toStoreSize().toLong())
                throw IllegalArgumentException("Cannot set tensor with shape: ${value.shape} to tensor with shape: $shape at index: $indexForMessage")
            ops.flush(handle)
            copyBox(this, offset, st, value, 0L, strides(boxShape), boxShape)
        } else Arena.ofConfined().use { arena ->
            check(KtcNative.fillStrided.invokeExact(bufferForWrite(), offset, KtcNative.shape(arena, st), KtcNative.shape(arena, boxShape), boxShape.size, constant) as Int)
        }
    }

    override fun set(index: IntArray, value: AbstractRawTensor<CUDABuffer>) =
        setBox(shape.normalizeIndex(index).map { it..it }, value as CUDARawTensor, 0f, index.toList())
    override fun set(index: Array<out IntRange>, value: AbstractRawTensor<CUDABuffer>) =
        setBox(shape.normalizeIndex(index).toList(), value as CUDARawTensor, 0f, index.toList())
    override fun set(index: IntArray, value: Float) = setBox(shape.normalizeIndex(index).map { it..it }, null, value, index.toList())
    override fun set(index: Array<out IntRange>, value: Float) = setBox(shape.normalizeIndex(index).toList(), null, value, index.toList())

    override fun narrow(axis: Int, start: Int, length: Int): CUDARawTensor {
        val ranges = shape.map { 0 until it }.toTypedArray()
        ranges[shape.normalizeAxis(axis)] = start until (start + length)
        return get(ranges)
    }

    override fun permute(axes: List<Int>): CUDARawTensor {
        val newShape = shape.permute(axes)
        val st = strides(shape)
        val res = ops.createRaw(newShape)
        copyBox(res, 0L, strides(newShape), this, 0L, axes.map { st[it] }, newShape)     // result dimension i = this dimension axes[i]
        return res
    }

    override fun transpose(axis1: Int, axis2: Int): CUDARawTensor {
        val (_, a1, a2) = shape.transposeNormalizeAxes(axis1, axis2)
        return permute(shape.indices.map { if (it == a1) a2 else if (it == a2) a1 else it })
    }

    override fun gather(axis: Int, index: AbstractRawTensor<CUDABuffer>): CUDARawTensor {
        val res = ops.createRaw(index.shape)
        Arena.ofConfined().use { arena ->
            check(KtcNative.gatherAxis.invokeExact(res.handle, handle, KtcNative.shape(arena, shape), (index as CUDARawTensor).handle,
                                                   KtcNative.shape(arena, index.shape), shape.size, shape.normalizeAxis(axis)) as Int)
        }
        return res
    }

    override fun indexSelect(axis: Int, index: AbstractRawTensor<CUDABuffer>): CUDARawTensor {
        val (a, resShape) = shape.indexSelectNormAxisShape(axis, index.shape)
        val res = ops.createRaw(resShape)
        check(KtcNative.indexSelect.invokeExact(res.handle, handle, (index as CUDARawTensor).handle, shape.take(a).toStoreSize().toLong(),
                                                shape[a].toLong(), index.shape[0].toLong(), shape.drop(a + 1).toStoreSize().toLong()) as Int)
        return res
    }

    override fun indexAdd(axis: Int, index: AbstractRawTensor<CUDABuffer>, src: AbstractRawTensor<CUDABuffer>, alpha: Float) {
        val a = shape.indexAddCheckShapesNormAxis(axis, index.shape, src.shape)
        check(KtcNative.indexAdd.invokeExact(bufferForWrite(), (index as CUDARawTensor).handle, (src as CUDARawTensor).handle, alpha,
                                             shape.take(a).toStoreSize().toLong(), shape[a].toLong(), index.shape[0].toLong(),
                                             shape.drop(a + 1).toStoreSize().toLong()) as Int)
    }

    // ---- BLAS: not provided by libkten_cuda.so ---------------------------------------------------------------
    override fun dot(vector: AbstractRawTensor<CUDABuffer>): AbstractRawTensor<CUDABuffer> =
        throw UnsupportedOperationException("dot is a BLAS operation; kten-cuda does not provide BLAS yet")

    override fun inplaceResize(vararg shape: Int) =
        throw UnsupportedOperationException("inplaceResize swaps the store object; bind it where CUDABuffer is made replaceable")
}
