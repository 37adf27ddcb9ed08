package eu.redbean.kten.cuda.tensor.platform

import java.lang.foreign.Arena
import java.lang.foreign.FunctionDescriptor
import java.lang.foreign.Linker
import java.lang.foreign.MemoryLayout
import java.lang.foreign.MemorySegment
import java.lang.foreign.SymbolLookup
import java.lang.foreign.ValueLayout.ADDRESS
import java.lang.foreign.ValueLayout.JAVA_FLOAT
import java.lang.foreign.ValueLayout.JAVA_INT
import java.lang.foreign.ValueLayout.JAVA_LONG
import java.lang.invoke.MethodHandle
import java.nio.file.Path

/**
 * Downcall handles for libkten_cuda.so (include/kten_cuda.h), one per entry point, plus the
 * status-to-exception mapping.  The library path comes from the system property
 * `kten.cuda.library` (default: `libkten_cuda.so` on java.library.path).
 */
internal object KtcNative {

    const val PLUS = 0; const val MINUS = 1; const val TIMES = 2; const val DIV = 3; const val POW = 4
    const val EXP = 0; const val LOG = 1; const val TANH = 2; const val SIGMOID = 3; const val RECIPROCAL = 4; const val NEG = 5
    const val SUM = 0; const val MEAN = 1; const val MAX = 2; const val MIN = 3; const val ARGMAX = 4; const val ARGMIN = 5
    const val SINH = 6; const val COSH = 7; const val ABS = 8; const val SIGN = 9; const val SQRT = 10; const val SIN = 11
    const val COS = 12; const val TAN = 13; const val ASIN = 14; const val ACOS = 15; const val ATAN = 16; const val FLOOR = 17
    const val CEIL = 18; const val ROUND = 19; const val TRUNC = 20; const val RSQRT = 21
    const val LT = 0; const val LTE = 1; const val GT = 2; const val GTE = 3; const val EQ = 4; const val NEQ = 5
    const val SCATTER_SET = 0; const val SCATTER_ADD = 1; const val SCATTER_CONST = 2

    private val linker: Linker = Linker.nativeLinker()
    private val lookup: SymbolLookup = System.getProperty("kten.cuda.library")
        ?.let { SymbolLookup.libraryLookup(Path.of(it), Arena.global()) }
        ?: SymbolLookup.libraryLookup(System.mapLibraryName("kten_cuda"), Arena.global())

    private fun handle(name: String, result: MemoryLayout?, vararg args: MemoryLayout): MethodHandle {
        val symbol = lookup.find(name).orElseThrow { UnsatisfiedLinkError("libkten_cuda.so does not export $name") }
        val descriptor = if (result == null) FunctionDescriptor.ofVoid(*args) else FunctionDescriptor.of(result, *args)
        return linker.downcallHandle(symbol, descriptor)
    }

    val init = handle("ktc_init", JAVA_INT, ADDRESS)
    val lastError = handle("ktc_last_error", ADDRESS)
    val deviceInfo = handle("ktc_device_info", JAVA_INT, JAVA_INT, ADDRESS, JAVA_LONG, ADDRESS, ADDRESS)
    val alloc = handle("ktc_alloc", JAVA_INT, JAVA_INT, JAVA_LONG, ADDRESS)
    val retain = handle("ktc_retain", JAVA_INT, JAVA_LONG)
    val release = handle("ktc_release", JAVA_INT, JAVA_LONG)
    val poolStats = handle("ktc_pool_stats", JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS)
    val poolLimit = handle("ktc_pool_limit", JAVA_INT, JAVA_INT, JAVA_LONG)
    val h2d = handle("ktc_h2d", JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_LONG, JAVA_INT)
    val d2h = handle("ktc_d2h", JAVA_INT, ADDRESS, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_INT)
    val d2d = handle("ktc_d2d", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    val fill = handle("ktc_fill", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_FLOAT)
    val sync = handle("ktc_sync", JAVA_INT, JAVA_INT)
    val binary = handle("ktc_binary", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    val binaryBcast = handle("ktc_binary_bcast", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT)
    val binaryInplace = handle("ktc_binary_inplace", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    val scalar = handle("ktc_scalar", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_LONG, JAVA_INT)
    val scalarInplace = handle("ktc_scalar_inplace", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_FLOAT, JAVA_LONG)
    val unary = handle("ktc_unary", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    val clamp = handle("ktc_clamp", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_FLOAT, JAVA_LONG)
    val compareScalar = handle("ktc_compare_scalar", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_LONG)
    val broadcastTo = handle("ktc_broadcast_to", JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT)
    val reduceAxis = handle("ktc_reduce_axis", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    val reduceAll = handle("ktc_reduce_all", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    val scatterAxis = handle("ktc_scatter_axis", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    val compareScalarEps = handle("ktc_compare_scalar_eps", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_FLOAT, JAVA_LONG)
    val compareTensor = handle("ktc_compare_tensor", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_LONG)
    val maskedFill = handle("ktc_masked_fill", JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_FLOAT)
    val containsNan = handle("ktc_contains_nan", JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS)
    val copyStrided = handle("ktc_copy_strided", JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_LONG, JAVA_LONG, ADDRESS, ADDRESS, JAVA_INT)
    val fillStrided = handle("ktc_fill_strided", JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, ADDRESS, JAVA_INT, JAVA_FLOAT)
    val gatherAxis = handle("ktc_gather_axis", JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_INT)
    val scatterAxisNd = handle("ktc_scatter_axis_nd", JAVA_INT, JAVA_INT, JAVA_LONG, ADDRESS, JAVA_LONG, ADDRESS, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_INT, JAVA_FLOAT)
    val indexSelect = handle("ktc_index_select", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG)
    // sum of a few small tensors across the GPUs of one box, one kernel per rank over peer memory
    val p2pCreate = handle("ktc_p2p_create", JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS)
    val p2pConnect = handle("ktc_p2p_connect", JAVA_INT, JAVA_LONG, ADDRESS)
    val p2pAllreduceSum = handle("ktc_p2p_allreduce_sum", JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS, JAVA_INT)
    val p2pStatus = handle("ktc_p2p_status", JAVA_INT, JAVA_LONG, ADDRESS)
    val p2pDestroy = handle("ktc_p2p_destroy", JAVA_INT, JAVA_LONG)
    // fused expression programs (optional: a binder that defers elementwise calls and sums submits them here)
    val exprEval = handle("ktc_expr_eval", JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, JAVA_INT,
        ADDRESS, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_INT)
    val exprEvalMulti = handle("ktc_expr_eval_multi", JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, JAVA_INT,
        ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_INT)
    val exprEvalMultiFused = handle("ktc_expr_eval_multi_fused", JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, JAVA_INT,
        ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, JAVA_LONG, ADDRESS, ADDRESS, JAVA_INT)
    // SoftmaxCrossEntropy.doForward in one pass: (softmax, nll, logits, targets, rows, cols, lo, hi); KTC_ENOTSUP (-4): issue the calls instead
    val softmaxXentForward = handle("ktc_softmax_xent_forward", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_FLOAT)
    // nearest-neighbour upsampling and its gradient: (out, in, P, W, scale) with P = the product of all dimensions but the last
    val upsample2dNearest = handle("ktc_upsample2d_nearest", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_INT)
    val upsample2dNearestGrad = handle("ktc_upsample2d_nearest_grad", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_INT)
    // spatial pooling: (out, indices, in, planes, geom), (grad_in, grad_out, indices, planes, geom), (out, in, planes, geom, include_padding),
    // (grad_in, grad_out, planes, geom, include_padding); geom = {H, W, OH, OW, kH, kW, pH, pW, sH, sW, dH, dW} as twelve ints
    val pool2dMax = handle("ktc_pool2d_max", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, ADDRESS)
    val pool2dMaxGrad = handle("ktc_pool2d_max_grad", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, ADDRESS)
    val pool2dAvg = handle("ktc_pool2d_avg", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_INT)
    val pool2dAvgGrad = handle("ktc_pool2d_avg_grad", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_INT)
    // instruction codes of ktc_expr_eval programs used by the binding itself (enum in kten_cuda.h: op | dst << 8 | a << 12 | b << 16 | k << 20)
    const val X_LOAD = 1; const val X_CONST = 2; const val X_ADD = 3; const val X_DIV = 6; const val X_STORE = 20; const val X_SCATC = 22
    const val ENOTSUP = -4
    // the deferred-expression recorder: elementwise calls and sums are recorded below the C ABI and run fused when a value is needed
    const val EXPR_SUM_ALL = 1; const val EXPR_SUM_ROWS = 2; const val EXPR_SUM_LAST = 4
    const val ASSIGN_WRITTEN = 0; const val ASSIGN_PENDING = 1; const val ASSIGN_UPDATE_RECORDED = 2; const val ASSIGN_UPDATE_OF_ZEROED = 3
    val lazyLeaf = handle("ktc_lazy_leaf", JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, ADDRESS)
    val lazyFree = handle("ktc_lazy_free", JAVA_INT, JAVA_LONG)
    val lazyUnary = handle("ktc_lazy_unary", JAVA_INT, JAVA_INT, JAVA_LONG, ADDRESS)
    val lazyBinary = handle("ktc_lazy_binary", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS)
    val lazyScalar = handle("ktc_lazy_scalar", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_FLOAT, JAVA_INT, ADDRESS)
    val lazyClamp = handle("ktc_lazy_clamp", JAVA_INT, JAVA_LONG, JAVA_FLOAT, JAVA_FLOAT, ADDRESS)
    val lazyCompareScalar = handle("ktc_lazy_compare_scalar", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_FLOAT, ADDRESS)
    val lazyBroadcastTo = handle("ktc_lazy_broadcast_to", JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, ADDRESS)
    val lazyAssignBinary = handle("ktc_lazy_assign_binary", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS)
    val lazyAssignScalar = handle("ktc_lazy_assign_scalar", JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_FLOAT, ADDRESS)
    val lazyFull = handle("ktc_lazy_full", JAVA_INT, JAVA_INT, ADDRESS, JAVA_INT, JAVA_FLOAT, ADDRESS)
    val lazyAssignFill = handle("ktc_lazy_assign_fill", JAVA_INT, JAVA_LONG, JAVA_FLOAT, ADDRESS)
    val lazyAssignScatterConst = handle("ktc_lazy_assign_scatter_const", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, ADDRESS)
    // the forward of SoftmaxCrossEntropy, recorded: (logits cell, targets cell, lo, hi, &softmax cell, &nll cell); ENOTSUP: issue the calls
    val lazySoftmaxXentForward = handle("ktc_lazy_softmax_xent_forward", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_FLOAT, ADDRESS, ADDRESS)
    val lazySum = handle("ktc_lazy_sum", JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS)
    val lazyBuffer = handle("ktc_lazy_buffer", JAVA_INT, JAVA_LONG, ADDRESS)
    val lazyInfo = handle("ktc_lazy_info", JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS, ADDRESS, ADDRESS)
    val lazyFlush = handle("ktc_lazy_flush", JAVA_INT, JAVA_LONG)
    val lazyRunPending = handle("ktc_lazy_run_pending", JAVA_INT)
    val lazyAllreduce = handle("ktc_lazy_allreduce", JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT)
    val lazyOption = handle("ktc_lazy_option", JAVA_INT, ADDRESS, JAVA_INT)
    val lazyStats = handle("ktc_lazy_stats", JAVA_INT, ADDRESS)
    val refcount = handle("ktc_refcount", JAVA_INT, JAVA_LONG, ADDRESS)
    val indexAdd = handle("ktc_index_add", JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG)

    /** KTC_EINVAL -> IllegalArgumentException, KTC_ESTATE -> IllegalStateException, KTC_ENOMEM -> OutOfMemoryError. */
    fun check(status: Int) {
        if (status == 0) return
        val message = (lastError.invokeExact() as MemorySegment).reinterpret(1024).getString(0)
        when (status) {
            -1 -> throw IllegalArgumentException(message)
            -2 -> throw IllegalStateException(message)
            -3 -> throw OutOfMemoryError(message)
            else -> throw RuntimeException("kten-cuda [$status]: $message")
        }
    }

    /** Calls a recorder entry point whose last argument is the result cell and returns that cell. */
    fun cell(call: (MemorySegment) -> Int): Long = Arena.ofConfined().use { arena ->
        val out = arena.allocate(JAVA_LONG)
        check(call(out))
        out.get(JAVA_LONG, 0)
    }

    fun shape(arena: Arena, shape: List<Int>): MemorySegment {
        val seg = arena.allocate(JAVA_LONG, maxOf(1, shape.size).toLong())
        shape.forEachIndexed { i, d -> seg.setAtIndex(JAVA_LONG, i.toLong(), d.toLong()) }
        return seg
    }
}
