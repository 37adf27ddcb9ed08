/* kten_cuda.h -- C ABI of libkten_cuda.so, the sm_100a compute backend for the
 * KTen tensor library's float32 hot path (broadcast elementwise ops, axis and
 * full reductions, and the broadcast-gradient sum-to-shape reduction).
 *
 * This is the surface a `backend/kten-cuda` module binds (JNI `external fun`
 * or Java FFM downcall handles) to implement the reference's backend SPI:
 *   ART  = kten-api/src/main/kotlin/eu/redbean/kten/api/tensor/store/AbstractRawTensor.kt
 *   TOPS = kten-api/src/main/kotlin/eu/redbean/kten/api/tensor/operations/TensorOperations.kt
 *   JVM  = backend/kten-jvm/src/main/kotlin/eu/redbean/kten/jvm/tensor/store/JVMRawTensor.kt
 *   OCLM = backend/kten-opencl/src/main/kotlin/eu/redbean/kten/opencl/tensor/store/OCLMemoryObject.kt
 *   OCLE = backend/kten-opencl/src/main/kotlin/eu/redbean/kten/opencl/tensor/platform/OCLEnvironment.kt
 *   OCLK = backend/kten-opencl/src/main/kotlin/eu/redbean/kten/opencl/tensor/platform/kernels/OCLKernels.kt
 * Each entry point names the reference interface it stands in for.
 *
 * Conventions
 *  - Every function returns 0 (KTC_OK) or a negative KTC_E* status; the text
 *    of the last failure on the calling thread is ktc_last_error().
 *  - Buffers are opaque 64-bit handles to device-resident float32 storage,
 *    reference counted (a handle starts at 1).  Shapes live on the caller's
 *    side exactly as AbstractRawTensor keeps them on the JVM heap (ART:5-23);
 *    calls that need them take `const int64_t*` + ndim (ndim <= KTC_MAX_DIMS).
 *  - All compute calls enqueue on the owning device's single in-order stream
 *    (the role of the one in-order command queue at OCLE:291-299) and return
 *    without waiting; host reads (ktc_d2h, ktc_get) wait for that stream.
 *  - There is no CPU fallback: without a usable CUDA device ktc_init fails.
 */
#ifndef KTEN_CUDA_H
#define KTEN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KTC_API __attribute__((visibility("default")))
#else
#define KTC_API
#endif

#define KTC_MAX_DIMS 10   /* same limit as the OpenCL backend's shape arrays (OCLKernelConstant.kt:4) */

typedef uint64_t ktc_buf;   /* device buffer handle; 0 is never valid */
typedef uint64_t ktc_comm;  /* communicator handle */

/* status codes */
enum {
    KTC_OK        = 0,
    KTC_EINVAL    = -1,  /* bad argument / shape mismatch  -> IllegalArgumentException */
    KTC_ESTATE    = -2,  /* released handle, not initialised -> IllegalStateException (OCLM:167-170) */
    KTC_ENOMEM    = -3,  /* pool limit or device allocation failure */
    KTC_ECUDA     = -4,  /* CUDA runtime error */
    KTC_ECOMM     = -5,  /* collective library error */
    KTC_ETIMEOUT  = -6,  /* a bounded device-side wait ran out */
    KTC_ENOTSUP   = -7
};

/* elementwise binary ops: JVM:110-140, kernels.cl calc_by_elwise_op (kernels.cl:79-94) */
enum { KTC_PLUS = 0, KTC_MINUS = 1, KTC_TIMES = 2, KTC_DIV = 3, KTC_POW = 4 };
/* unary maps: JVM:122,142,144,395-435, kernels.cl tensor_mapping_op (kernels.cl:132-156) */
enum { KTC_EXP = 0, KTC_LOG = 1, KTC_TANH = 2, KTC_SIGMOID = 3, KTC_RECIPROCAL = 4, KTC_NEG = 5,
       KTC_SINH = 6, KTC_COSH = 7, KTC_ABS = 8, KTC_SIGN = 9, KTC_SQRT = 10, KTC_SIN = 11, KTC_COS = 12, KTC_TAN = 13,
       KTC_ASIN = 14, KTC_ACOS = 15, KTC_ATAN = 16, KTC_FLOOR = 17, KTC_CEIL = 18, KTC_ROUND = 19, KTC_TRUNC = 20,
       KTC_RSQRT = 21 };
/* aggregations: kten-api/.../tensor/store/AggregatingOperation.kt:3-4 */
enum { KTC_SUM = 0, KTC_MEAN = 1, KTC_MAX = 2, KTC_MIN = 3, KTC_ARGMAX = 4, KTC_ARGMIN = 5 };
/* compares (JVM:355-393); lt..gte are used by Clamp.doBackward (PointwiseFunctions.kt:154-162) */
enum { KTC_LT = 0, KTC_LTE = 1, KTC_GT = 2, KTC_GTE = 3, KTC_EQ = 4, KTC_NEQ = 5 };

/* ---- lifecycle / devices ------------------------------------------------
 * Stands in for OCLPlatformInitializer device enumeration
 * (OCLPlatformInitializer.kt:20-41) and the lazily created per-device
 * environment (OCLE:20-28). */
KTC_API int ktc_init(int* n_devices);
KTC_API int ktc_shutdown(void);
KTC_API int ktc_device_info(int dev, char* name, size_t name_len, int64_t* total_mem_bytes, int* sm_count);
KTC_API const char* ktc_last_error(void);
KTC_API const char* ktc_version(void);

/* ---- storage --------------------------------------------------------------
 * ktc_alloc: createRaw(shape) (TOPS:16; OCLM lazy cl_mem + reuse pool OCLE:98-107,191-200).
 * ktc_retain / ktc_release: incrementRef / release (TOPS:22-28; OCLM:108-145).
 * ktc_wrap: adopt caller-owned device memory (not pooled, never freed here).
 * ktc_view: a handle on a sub-range of a buffer (the slices of get / narrow, JVM:270-275, and the chunks
 *           of a pipelined upload); it keeps the parent alive.
 * ktc_pool_limit: PlatformProvider.memoryUsageScaleHint (PlatformProvider.kt:12-40, OCLE:53-54).
 * ktc_pool_stats: PlatformMetricsProvider.getMetrics (PlatformMetricsProvider.kt:3-6, OCLE:89-96). */
KTC_API int ktc_alloc(int dev, int64_t n_floats, ktc_buf* out);
KTC_API int ktc_wrap(int dev, void* device_ptr, int64_t n_floats, ktc_buf* out);
KTC_API int ktc_view(ktc_buf buf, int64_t off, int64_t n_floats, ktc_buf* out);   /* sub-range handle; holds a reference on `buf` */
KTC_API int ktc_retain(ktc_buf buf);
KTC_API int ktc_release(ktc_buf buf);
KTC_API int ktc_refcount(ktc_buf buf, int* count);
KTC_API int ktc_buf_info(ktc_buf buf, int* dev, int64_t* n_floats, void** device_ptr);
KTC_API int ktc_pool_stats(int dev, int64_t* live_bytes, int64_t* cached_bytes, int64_t* n_alloc_calls, int64_t* n_pool_hits);
KTC_API int ktc_pool_trim(int dev);
KTC_API int ktc_pool_limit(int dev, int64_t max_bytes);   /* <= 0: no limit */

/* pinned host staging memory for createRaw(shape, init) uploads (TOPS:11; OCLM:209-231) */
KTC_API int ktc_host_alloc(int64_t n_floats, float** out);
KTC_API int ktc_host_free(float* p);

/* ---- transfers -------------------------------------------------------------
 * h2d: createRaw(shape, init) / fromCommonSerializable (TOPS:11,135; OCLM:209-231).
 * d2h: toSerializableData, getSingleValue, item() (TOPS:133; OCLM:189-207, 357-361).
 * d2d: copy(shallow=false) (JVM:257-262; CLBlastScopy at OCLM:242).
 * fill: createRawFill / zerosLike / zeroOut / inplaceFill (TOPS:18-26; kernels.cl:73-76).
 * Copy modes of h2d / d2h:
 *   KTC_COPY_ASYNC    enqueue on the compute stream and return (the host range must stay valid, and
 *                     pinned for a truly asynchronous copy, until ktc_sync);
 *   KTC_COPY_SYNC     the same, then wait for the compute stream;
 *   KTC_COPY_OVERLAP  run on a dedicated upload / download stream, ordered after the compute work
 *                     queued so far and before the compute work queued afterwards (safe without
 *                     further thought, but a download then holds back the following upload);
 *   KTC_COPY_OVERLAP_UNFENCED  the pipelining form.  An upload does not wait for queued compute work
 *                     (the caller guarantees nothing queued still reads the destination); later
 *                     compute work waits for it.  A download waits for the compute work queued so
 *                     far, but later compute work does NOT wait for it: before queuing work that
 *                     overwrites the source, call ktc_copy_fence.  Uploads, kernels and downloads of
 *                     neighbouring chunks then overlap (full-duplex copy engines).
 * ktc_sync waits for the copy streams too; ktc_copy_fence orders both ways without a host wait:
 * compute work queued afterwards waits for every overlapped copy issued so far, and overlapped
 * copies issued afterwards wait for the compute work queued so far. */
enum { KTC_COPY_ASYNC = 0, KTC_COPY_SYNC = 1, KTC_COPY_OVERLAP = 2, KTC_COPY_OVERLAP_UNFENCED = 3 };
KTC_API int ktc_h2d(ktc_buf dst, int64_t dst_off, const float* src, int64_t n, int mode);
KTC_API int ktc_d2h(float* dst, ktc_buf src, int64_t src_off, int64_t n, int mode);
KTC_API int ktc_d2d(ktc_buf dst, int64_t dst_off, ktc_buf src, int64_t src_off, int64_t n);
KTC_API int ktc_fill(ktc_buf buf, int64_t off, int64_t n, float value);
KTC_API int ktc_sync(int dev);
KTC_API int ktc_copy_fence(int dev);

/* ---- elementwise -----------------------------------------------------------
 * ktc_binary:         elementwiseOpOnCommonShapedTensors (JVM:75-79), kernels.cl:96-99.
 * ktc_binary_bcast:   elementwiseOpOnTensors (JVM:81-87) WITHOUT materialising
 *                     the broadcast operand (replaces broadcast_to_shape,
 *                     kernels.cl:44-70, + OCLRawTensor.kt:107-114).  Shapes are
 *                     right-aligned; a non-singleton mismatch is KTC_EINVAL
 *                     (ShapeFunctions.kt:168-185).  `out` holds the common volume.
 * ktc_binary_inplace: inplaceElementwiseOpOnTensors (JVM:89-97): a = a op b, equal sizes.
 * ktc_scalar:         mapElementsCopy with a constant (JVM:112-140) and
 *                     TensorOperations.pow(constant, raw) (TOPS:39) via scalar_first.
 * ktc_scalar_inplace: inplaceMapElements (JVM:105-108,116,130,136).
 * ktc_unary:          JVM:122,142,144,395-399.   ktc_clamp: JVM:409-411.
 * ktc_compare_scalar: lt/lte/gt/gte(value) -> 1.0f / 0.0f (JVM:377-383). */
KTC_API int ktc_binary(int op, ktc_buf out, ktc_buf a, ktc_buf b, int64_t n);
KTC_API int ktc_binary_bcast(int op, ktc_buf out,
                             ktc_buf a, const int64_t* a_shape, int a_ndim,
                             ktc_buf b, const int64_t* b_shape, int b_ndim);
KTC_API int ktc_binary_inplace(int op, ktc_buf a, ktc_buf b, int64_t n);
KTC_API int ktc_scalar(int op, ktc_buf out, ktc_buf a, float s, int64_t n, int scalar_first);
KTC_API int ktc_scalar_inplace(int op, ktc_buf a, float s, int64_t n);
KTC_API int ktc_unary(int op, ktc_buf out, ktc_buf a, int64_t n);
KTC_API int ktc_clamp(ktc_buf out, ktc_buf a, float lo, float hi, int64_t n);
KTC_API int ktc_compare_scalar(int op, ktc_buf out, ktc_buf a, float value, int64_t n);
/* ktc_compare_scalar_eps: eq / neq (value) as |x - value| < epsilon (JVM:387-393; epsilon is
 *                         PlatformProvider.epsilon, 1e-7f by default, PlatformProvider.kt:12).
 * ktc_compare_tensor:     lt/lte/gt/gte/eq/neq (tensor), equal shapes -> 1.0f / 0.0f (JVM:355-377;
 *                         kten-jvm does not broadcast tensor compares).
 * ktc_masked_fill:        maskedFill (JVM:537-540): out = mask == 1f ? value : a, the mask broadcast
 *                         to a's shape without being materialised.
 * ktc_contains_nan:       containsNan (JVM:520-522) evaluated on the device; *result = 0 / 1.  Waits. */
KTC_API int ktc_compare_scalar_eps(int op, ktc_buf out, ktc_buf a, float value, float epsilon, int64_t n);
KTC_API int ktc_compare_tensor(int op, ktc_buf out, ktc_buf a, ktc_buf b, float epsilon, int64_t n);
KTC_API int ktc_masked_fill(ktc_buf out, ktc_buf a, const int64_t* a_shape, int a_ndim,
                            ktc_buf mask, const int64_t* mask_shape, int mask_ndim, float value);
KTC_API int ktc_contains_nan(ktc_buf a, int64_t n, int* result);

/* broadcastTo for callers that really need the expanded tensor
 * (Sum/Mean/Expand backward: AggregatingFunctions.kt:19-25,40-53; JVM:51-73). */
KTC_API int ktc_broadcast_to(ktc_buf out, const int64_t* out_shape, int out_ndim,
                             ktc_buf a, const int64_t* a_shape, int a_ndim);

/* ---- reductions ------------------------------------------------------------
 * ktc_reduce_axis: aggregateOverAxis (JVM:154-225; kernels.cl:198-260) on the
 *   collapsed view [outer, axis_len, inner]; out holds outer*inner floats
 *   (index results are float32, JVM:180).
 * ktc_reduce_axis_validx: value and index in one pass (what
 *   AggregatingFunctions.kt:83-87 asks for in its TODO).
 * ktc_reduce_all: sum() / mean() to one float (JVM:146-152; OCLK:336-415).
 * ktc_sum_to_shape: mayUnexpand (Utils.kt:14-41) and Expand.doBackward
 *   (TensorFunctions.kt:262-283): out has old_shape's volume. */
KTC_API int ktc_reduce_axis(int op, ktc_buf out, ktc_buf in, int64_t outer, int64_t axis_len, int64_t inner);
KTC_API int ktc_reduce_axis_validx(int is_max, ktc_buf out_val, ktc_buf out_idx, ktc_buf in,
                                   int64_t outer, int64_t axis_len, int64_t inner);
KTC_API int ktc_reduce_all(int op, ktc_buf out, ktc_buf in, int64_t n);
KTC_API int ktc_sum_to_shape(ktc_buf out, const int64_t* old_shape, int old_ndim,
                             ktc_buf in, const int64_t* in_shape, int in_ndim);

/* The forward of SoftmaxCrossEntropy (kten-api/.../functions/nn/SoftmaxCrossEntropy.kt:40-59) in one pass over the
 * logits [rows, cols]: row maximum, exp of the shifted row, its sum, the quotients -- written to `softmax`, the tensor
 * the function saves for backward --, their sum, and -log(clamp(softmax[target] / that sum, lo, hi)) per row into
 * `nll` [rows]; the mean over the rows is ktc_reduce_all(KTC_MEAN) on nll.  Every operation is the reference's, in its
 * order, and the two row sums accumulate exactly as ktc_reduce_axis does, so both outputs carry the bits of the
 * eleven separate calls.  targets [rows]: class indices as floats (truncated like Float.toInt); an index outside
 * [0, cols) is recorded like an invalid gather index and gives a NaN row.  KTC_ENOTSUP (cols > 12288 or <= 64, cols not
 * a multiple of 4, unaligned rows): issue the separate calls. */
KTC_API int ktc_softmax_xent_forward(ktc_buf softmax, ktc_buf nll, ktc_buf logits, ktc_buf targets, int64_t rows, int64_t cols, float lo, float hi);

/* The same forward with an elementwise program (the encoding of ktc_expr_eval) as its epilogue: leaf `soft_leaf` of the
 * program is the row's softmax while it is still in registers.  A consumer of the saved tensor -- the function's backward,
 * (softmax with -1 at the target) / rows, SoftmaxCrossEntropy.kt:61-67, and the accumulation into the Variable's gradient,
 * Variable.kt:44-46 -- then runs in the pass that reads the logits, and `softmax` may be 0: the saved tensor is not written.
 * The other leaves are [rows | 1, cols | 1] tensors (leaf_shapes: two extents per leaf; the entry of soft_leaf is ignored),
 * STORE k writes stores[k], [rows, cols]; ACC is not allowed.  Each instruction is the reference operation of the
 * stand-alone call with its own rounding, so nll and the stored tensors carry the bits of ktc_softmax_xent_forward
 * followed by ktc_expr_eval on the stored softmax.  The kernel is generated at run time; KTC_ENOTSUP (rows the one-pass
 * kernel does not take, no run-time compiler): run the two separately.  ktc_lazy_softmax_xent_forward records the forward
 * and makes this call when the recorded consumer is evaluated. */
KTC_API int ktc_softmax_xent_forward_expr(ktc_buf softmax, ktc_buf nll, ktc_buf logits, ktc_buf targets, int64_t rows, int64_t cols, float lo, float hi,
                                          const uint32_t* code, int n_code, const float* imm, int n_imm,
                                          const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves, int soft_leaf,
                                          const ktc_buf* stores, int n_stores);

/* Nearest-neighbour upsampling of the last two dimensions by `scale` and its gradient (TensorOperations.upsample,
 * TensorOperations.kt:131; Upsample2DOperation.kt:5-44; kten-jvm: JVMUpsample2DNearest.kt:14-77).  P is the product of
 * all dimensions but the last (N * C * H): in [P, W] -> out [P, scale, W * scale]; grad_out [P, scale, W * scale] ->
 * grad_in [P, W], every position the sum of its scale x scale block, added in float from 0f in the reference's loop
 * order (JVMUpsample2DNearest.kt:61-68): bit-identical to kten-jvm. */
KTC_API int ktc_upsample2d_nearest(ktc_buf out, ktc_buf in, int64_t P, int64_t W, int scale);
KTC_API int ktc_upsample2d_nearest_grad(ktc_buf grad_in, ktc_buf grad_out, int64_t P, int64_t W, int scale);

/* Spatial (2-D) pooling and its gradient (TensorOperations.spatialPooling, TensorOperations.kt:127; PoolingOperation.kt:
 * 5-15; kten-jvm: JVMSpatialMaxPooling.kt:24-69, JVMSpatialAvgPooling.kt:23-88; 1-D pooling is the same with a trailing
 * extent of 1).  planes = N * C; in and grad_in are [planes, H, W], out / indices / grad_out [planes, OH, OW].
 * geom: {H, W, OH, OW, kernelH, kernelW, paddingH, paddingW, strideH, strideW, dilationH, dilationW}; the caller computes
 * OH and OW as the reference does (on floats, ceil or floor, minus a last window that would start in the padding:
 * JVMSpatialPoolingBase.kt:27-77).  Max: strict `>` from -infinity in window order, so NaN never wins and the first of
 * equals stays; indices are positions inside the plane (y * W + x) as floats, -1 where no value won.  Average: a float sum
 * in row-major order divided by the items in the window (include_padding: by the window clipped to the padded extent).
 * Gradients: every input position adds the contributions of the outputs that reach it, in output order, in float --
 * the additions the reference's sequential scatter performs, so results are bit-identical and run-to-run stable. */
KTC_API int ktc_pool2d_max(ktc_buf out, ktc_buf indices, ktc_buf in, int64_t planes, const int* geom);
KTC_API int ktc_pool2d_max_grad(ktc_buf grad_in, ktc_buf grad_out, ktc_buf indices, int64_t planes, const int* geom);
KTC_API int ktc_pool2d_avg(ktc_buf out, ktc_buf in, int64_t planes, const int* geom, int include_padding);
KTC_API int ktc_pool2d_avg_grad(ktc_buf grad_in, ktc_buf grad_out, int64_t planes, const int* geom, int include_padding);

/* Full sum / mean that obtains no memory, for callers that must not allocate
 * while they run: loops whose free device memory is already committed to
 * another allocator, latency-bound sections that cannot take the device-wide
 * synchronisation of cudaMalloc, code running while someone else holds the
 * allocator.  This entry point has no counterpart in the reference.
 * Same result contract as ktc_reduce_all (op is KTC_SUM or KTC_MEAN, `out`
 * receives one float); the per-CTA partials live in a fixed
 * KTC_NOALLOC_SCRATCH_BYTES array inside the library image on every GPU that
 * loads it.  n may not exceed KTC_NOALLOC_MAX_ELEMS (KTC_EINVAL otherwise).
 * All calls on a device share that array.  A call is two launches on the
 * device's one compute stream, issued under a per-device lock, so calls from
 * several host threads of this process do not interleave; anything else that
 * could make two calls overlap on the GPU is the caller's to prevent.  The first call
 * on a device resolves the array's device address; make it before any stream
 * capture begins. */
#define KTC_NOALLOC_SCRATCH_BYTES 16384
#define KTC_NOALLOC_MAX_ELEMS ((int64_t)1 << 30)
KTC_API int ktc_reduce_all_noalloc(int op, ktc_buf out, ktc_buf in, int64_t n);

/* ---- fused elementwise chains (no single counterpart in the reference) ---------------------
 * kten's autograd issues one raw-tensor call per line of doForward / doBackward
 * (BasicFunctions.kt, PointwiseFunctions.kt), each a full pass over memory.  A backend may
 * defer elementwise calls and submit the accumulated chain here: a program for a small
 * register machine (registers hold 4 neighbouring elements) whose instructions are exactly the
 * operations above -- the same arithmetic, rounded per operation, so the fused result equals
 * the chain of separate calls bit for bit.  Instruction word: op | dst << 8 | a << 12 | b << 16 |
 * k << 20 (k: leaf / store / immediate index).  `shape` is the iteration space; leaf_shapes holds
 * n_leaves rows of `ndim` right-aligned extents (1 where the leaf is broadcast; nothing is
 * materialised).  Sinks: STORE_ONLY (results leave through STORE instructions into full-size
 * buffers), SUM_ALL (ACC values summed, or averaged with mean != 0, into sink_out[0]: sum() /
 * mean(), JVM:146-152), SUM_ROWS (ACC values summed over all but the innermost dimension into
 * sink_out[shape[ndim-1]]: the leading-axis sum of mayUnexpand, Utils.kt:14-41).
 * KTC_ENOTSUP means "not fusable" (more than 3 collapsed dimensions, innermost extent not a
 * multiple of 4, unaligned rows): issue the separate calls instead. */
#define KTC_EXPR_MAX_INSTR 32
#define KTC_EXPR_MAX_IMM 16
#define KTC_EXPR_MAX_LEAVES 8
#define KTC_EXPR_MAX_STORES 3
#define KTC_EXPR_REGS 8
#define KTC_EXPR_MAX_SINKS 4
enum { KTC_X_LOAD = 1, KTC_X_CONST, KTC_X_ADD, KTC_X_SUB, KTC_X_MUL, KTC_X_DIV, KTC_X_POW, KTC_X_NEG, KTC_X_RCP,
       KTC_X_SQUARE, KTC_X_EXP, KTC_X_LOG, KTC_X_TANH, KTC_X_SIGMOID, KTC_X_CLAMP, KTC_X_CMP_LT, KTC_X_CMP_LTE,
       KTC_X_CMP_GT, KTC_X_CMP_GTE, KTC_X_STORE, KTC_X_ACC,
       KTC_X_SCATC,     /* d = (column == (int)b) ? imm[k] : a -- inplaceScatter(-1, index, constant) with one index per row (JVM:317-332):
                           b is the row's index broadcast over the columns; an index outside the row is recorded, nothing is written */
       KTC_X_SQRT, KTC_X_RSQRT, KTC_X_ABS };   /* sqrt (JVM:413), 1f / sqrt (JVM:435), abs (JVM:405): the chains of optimisers and normalisations */
enum { KTC_EXPR_STORE_ONLY = 0, KTC_EXPR_SUM_ALL = 1, KTC_EXPR_SUM_ROWS = 2, KTC_EXPR_MULTI = 3, KTC_EXPR_SUM_LAST = 4 };
KTC_API int ktc_expr_eval(const uint32_t* code, int n_code, const float* imm, int n_imm,
                          const int64_t* shape, int ndim,
                          const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                          const ktc_buf* stores, int n_stores,
                          int sink, ktc_buf sink_out, int mean);

/* Several sums of one pass: the loss and both broadcast gradients of a training step share their
 * operands (Mean.doForward, AggregatingFunctions.kt; the mayUnexpand sums of Plus / Times backward,
 * BasicFunctions.kt:12-55), so a backend that defers the sums as well can read those operands once.
 * Same program encoding; an ACC instruction's k field names the sink (0 .. n_sinks-1, at most
 * KTC_EXPR_MAX_SINKS), sink j is of kind sink_kinds[j] (KTC_EXPR_SUM_ALL, KTC_EXPR_SUM_ROWS or
 * KTC_EXPR_SUM_LAST, with means[j] != 0 dividing a SUM_ALL by the element count) and writes
 * sink_outs[j].  SUM_LAST sums over the innermost dimension of `shape` -- sum(-1), the row sums of a
 * softmax (SoftmaxCrossEntropy.kt:44,49) -- into one float per row (all leading dimensions
 * flattened); ktc_expr_eval accepts it as a single sink as well.  The iteration
 * space is partitioned as for a single SUM_ROWS sink, and every sink accumulates as its single-sink
 * call does (float runs folded into doubles, fixed combination order): SUM_ROWS results equal those
 * of separate ktc_expr_eval calls bit for bit, a SUM_ALL result is the same sum taken over a
 * possibly different partition (equal within the reduction tolerance, exact on exactly summable
 * data).  Runs only as a
 * generated kernel (see below): KTC_ENOTSUP also when the iteration space is below
 * `expr_jit_min_elems` or NVRTC is missing -- issue the single-sink calls instead. */
KTC_API int ktc_expr_eval_multi(const uint32_t* code, int n_code, const float* imm, int n_imm,
                                const int64_t* shape, int ndim,
                                const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                                const ktc_buf* stores, int n_stores,
                                const int* sink_kinds, const ktc_buf* sink_outs, const int* means, int n_sinks);

/* ktc_expr_eval_multi with the rest of a training step folded into its second pass (one kernel combines the partial
 * sums of all sinks): add_to[j] != 0 adds sink j's result into that tensor as well -- add_mode[j] = 1: target = target +
 * result, the float addition of Variable.backwardWithGrad's plusAssign (Variable.kt:44-46); add_mode[j] = 2: target =
 * 0f + result, the same call on a gradient that was just zeroed (its old contents are not read) -- and comm != 0 sums the n_x tensors
 * x_bufs (x_counts floats each; typically the sink outputs and the tensors added to) over the ranks of a peer-memory
 * communicator, in place, when the last block of that kernel has finished: the exchange of ktc_p2p_allreduce_sum,
 * without a launch of its own.  add_to / add_mode may be null; comm 0 ignores x_*. */
KTC_API int ktc_expr_eval_multi_fused(const uint32_t* code, int n_code, const float* imm, int n_imm,
                                      const int64_t* shape, int ndim,
                                      const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                                      const ktc_buf* stores, int n_stores,
                                      const int* sink_kinds, const ktc_buf* sink_outs, const int* means, int n_sinks,
                                      const ktc_buf* add_to, const int* add_mode, uint64_t comm, const ktc_buf* x_bufs, const int64_t* x_counts, int n_x);

/* For iteration spaces of at least `expr_jit_min_elems` elements (tunable, default 2^20; tunable
 * `expr_jit` = 0 turns it off) ktc_expr_eval does not interpret the program: it generates CUDA
 * source for it -- straight-line code over hardware registers built from the library's own
 * per-operation arithmetic, so results stay bit-identical --, compiles it once with NVRTC for
 * sm_100a and caches the kernel by program, as kten-opencl builds its kernels from source at
 * start-up (OCLKernels.kt).  Without NVRTC the interpreter kernel runs.
 * Shape of the generated code (tunables, part of the cache key; `expr_jit_multi_*` for programs
 * with several sums): `expr_jit_rows` rows per thread and batch (4), `expr_jit_min_blocks` resident
 * CTAs per SM asked of the compiler (none; 3 for several sums), `expr_jit_smem_acc` the double
 * accumulators of the sums live in shared memory (off; on for several sums, whose nine accumulators
 * would otherwise cost 18 registers).  None of them changes a result bit.
 * ktc_expr_stats fills out6 with: kernels compiled, launches of generated kernels, launches of the
 * interpreter kernel, failed compilations, microseconds spent compiling, NVRTC present (1 / 0 /
 * -1 = not tried yet).  ktc_expr_jit_log copies the log of the last failed compilation. */
KTC_API int ktc_expr_stats(int64_t* out6);
KTC_API int ktc_expr_jit_log(char* buf, int len);

/* ---- deferred-expression recorder (no counterpart in the reference; it absorbs the reference's call
 * sequence) ------------------------------------------------------------------------------------------
 * kten's Function nodes call the backend once per line of doForward / doBackward (Function.kt:54-68,
 * 108-141; BasicFunctions.kt:37-45, 182-204; PointwiseFunctions.kt:66-81; Utils.kt:14-41;
 * Variable.kt:44-46).  A binding may pass its elementwise calls to this recorder instead of running
 * them: each call returns a CELL -- the storage slot of one raw tensor -- whose value is a pending
 * expression until somebody needs it; the recorder then compiles the expression DAG into a program for
 * ktc_expr_eval / ktc_expr_eval_multi (programs are cached by DAG structure and re-bound to the step's
 * fresh operands), or falls back to the separate calls above where the kernel declines.  Results equal
 * the call-by-call results bit for bit; fused sums differ only in summation order.
 *   ktc_lazy_leaf            a cell over a stored buffer (retains it): how stored tensors enter expressions.
 *   ktc_lazy_unary/binary/scalar/clamp/compare_scalar/broadcast_to
 *                            record one operation; the result cell is pending (op codes as for ktc_unary,
 *                            KTC_EXP..KTC_NEG only, ktc_binary, ktc_compare_scalar KTC_LT..KTC_GTE; shapes
 *                            broadcast as in ktc_binary_bcast; broadcast_to with the operand's own shape
 *                            is a deep copy that is not made yet).
 *   ktc_lazy_assign_binary/scalar   target = target op other, in place (inplaceElementwiseOpOnTensors,
 *                            JVM:89-97, 105-108).  *state: 0 the target's buffer was written; 1 the
 *                            target cell is pending now -- a caller that holds a reference on its old
 *                            buffer drops it; 2 the call was `stored += pending sum` and is remembered as
 *                            an update of the buffer, applied when the pending sums run (ktc_lazy_buffer,
 *                            ktc_lazy_flush and every recorder call that reads the buffer apply it first).
 *                            The caller is expected to hold exactly one reference of its own on a stored
 *                            target's buffer; the recorder reads "nobody else holds it" off the count.
 *                            3: the call was `zeroed pending cell += pending sum`: the cell owns a new buffer that
 *                            receives 0f + sum when the pending sums run (fetch it with ktc_lazy_buffer when needed).
 *   ktc_lazy_full            a cell whose pending value is `value` everywhere (createRawFill, zerosLike): no buffer, no fill kernel
 *                            until somebody needs one; constants fold into the programs that use them.
 *   ktc_lazy_assign_fill     inplaceFill on a cell: a pending cell, or a stored one whose buffer nobody else holds, becomes
 *                            that pending constant (*state = 1); another stored cell is filled at once (*state = 0).
 *   ktc_lazy_assign_scatter_const   inplaceScatter(-1, index, constant) with one index per row (the `-1 at the target`
 *                            of SoftmaxCrossEntropy.doBackward, SoftmaxCrossEntropy.kt:61-67), recorded as an expression
 *                            instruction; index: a cell of the target's shape with last extent 1.  KTC_ENOTSUP for other
 *                            index shapes: use ktc_scatter_axis_nd on the buffers.
 *   ktc_lazy_softmax_xent_forward   the forward of SoftmaxCrossEntropy (SoftmaxCrossEntropy.kt:40-59), recorded: *softmax
 *                            is the tensor the function saves for backward, *nll the loss per row; nothing runs until one
 *                            of them is needed.  An elementwise expression of the softmax's shape recorded meanwhile (the
 *                            function's backward, the accumulation into the Variable's gradient) is then evaluated inside
 *                            the forward's kernel (ktc_softmax_xent_forward_expr) and the softmax is written only if a
 *                            tensor still holds it: logits in, gradient out.  KTC_ENOTSUP for rows the one-pass kernel
 *                            does not take.
 *   ktc_lazy_sum             sum() / mean() (KTC_EXPR_SUM_ALL), sum over axis 0 (KTC_EXPR_SUM_ROWS) or over
 *                            the innermost axis (KTC_EXPR_SUM_LAST) of a cell; with option defer_sums the
 *                            sum of a pending cell is pending too, and pending sums over one iteration
 *                            space run as ONE pass with several sinks.
 *   ktc_lazy_buffer          the buffer holding the cell's value, computed if pending; adds one reference
 *                            for the caller.
 *   ktc_lazy_flush           to be called before `buf` is written by any call that is not recorded here:
 *                            pending expressions that read it are evaluated first.
 *   ktc_lazy_free            drops the cell (values other expressions still need stay alive).
 *   ktc_lazy_option          recompute_limit (2), store_cost (8), defer_sums (1), defer_inplace (1).
 *   ktc_lazy_allreduce       sums the values of up to 8 cells over the ranks of a peer-memory communicator, in
 *                            place (ktc_p2p_allreduce_sum on their buffers, after whatever is pending).  When
 *                            all the pending work is one pass with several sums whose updates it applies --
 *                            loss, gradients and their accumulation in a training step -- the exchange runs
 *                            inside that pass's second-pass kernel (ktc_expr_eval_multi_fused).
 *   ktc_lazy_stats           out10: programs run, expressions run as separate calls, passes with several
 *                            sums, sums pending now, program-cache hits, programs compiled, live nodes,
 *                            live cells, `+= sum` updates applied by a second-pass kernel, all-reduces
 *                            performed by a second-pass kernel.
 * All calls are serialised by one lock; cells of different devices must not meet in one expression. */
typedef uint64_t ktc_lazy_cell;
KTC_API int ktc_lazy_leaf(ktc_buf buf, const int64_t* shape, int ndim, ktc_lazy_cell* out);
KTC_API int ktc_lazy_free(ktc_lazy_cell cell);
KTC_API int ktc_lazy_unary(int op, ktc_lazy_cell a, ktc_lazy_cell* out);
KTC_API int ktc_lazy_binary(int op, ktc_lazy_cell a, ktc_lazy_cell b, ktc_lazy_cell* out);
KTC_API int ktc_lazy_scalar(int op, ktc_lazy_cell a, float s, int scalar_first, ktc_lazy_cell* out);
KTC_API int ktc_lazy_clamp(ktc_lazy_cell a, float lo, float hi, ktc_lazy_cell* out);
KTC_API int ktc_lazy_compare_scalar(int op, ktc_lazy_cell a, float value, ktc_lazy_cell* out);
KTC_API int ktc_lazy_broadcast_to(ktc_lazy_cell a, const int64_t* shape, int ndim, ktc_lazy_cell* out);
KTC_API int ktc_lazy_assign_binary(int op, ktc_lazy_cell target, ktc_lazy_cell other, int* state);
KTC_API int ktc_lazy_assign_scalar(int op, ktc_lazy_cell target, float s, int* state);
KTC_API int ktc_lazy_full(int dev, const int64_t* shape, int ndim, float value, ktc_lazy_cell* out);
KTC_API int ktc_lazy_assign_fill(ktc_lazy_cell target, float value, int* state);
KTC_API int ktc_lazy_assign_scatter_const(ktc_lazy_cell target, ktc_lazy_cell index, float value, int* state);
KTC_API int ktc_lazy_softmax_xent_forward(ktc_lazy_cell logits, ktc_lazy_cell targets, float lo, float hi, ktc_lazy_cell* softmax, ktc_lazy_cell* nll);
KTC_API int ktc_lazy_sum(ktc_lazy_cell a, int kind, int mean, const int64_t* res_shape, int res_ndim, ktc_lazy_cell* out);
KTC_API int ktc_lazy_buffer(ktc_lazy_cell cell, ktc_buf* out);
KTC_API int ktc_lazy_info(ktc_lazy_cell cell, int* pending, int* is_sum, int64_t* shape, int* ndim);
KTC_API int ktc_lazy_flush(ktc_buf buf);
KTC_API int ktc_lazy_run_pending(void);
KTC_API int ktc_lazy_option(const char* name, int value);
KTC_API int ktc_lazy_allreduce(uint64_t comm, const ktc_lazy_cell* cells, int n);
KTC_API int ktc_lazy_stats(int64_t* out10);

/* ---- slices, permutes, gather / scatter -----------------------------------------
 * ktc_copy_strided:  dst[dst_offset + i.dst_strides] = src[src_offset + i.src_strides] for every i in the
 *                    box `shape`; strides in elements, >= 0.  With a contiguous dst this is get(ranges)
 *                    (JVM:276-280), narrow (JVM:468-482), transpose / permute (JVM:437-466; the source
 *                    strides permuted); with a contiguous src it is set(ranges, tensor) (JVM:291-304)
 *                    and the pieces of TensorOperations.concat.  Transposes go through a shared-memory
 *                    tile so that both sides are accessed in whole lines.
 * ktc_fill_strided:  set(index / ranges, value) (JVM:306-315).
 * ktc_gather_axis:   gather (JVM:334-353): out[c] = in[c with c[axis] = index[c]], out and index of
 *                    shape index_shape (<= in_shape off the axis), all of `ndim` dimensions.
 * ktc_scatter_axis_nd: inplaceScatter / inplaceScatterAdd / inplaceScatter(value) (JVM:227-255, 317-332;
 *                    shape rules ShapeFunctions.kt:346-371): for every index position c, in the order
 *                    of the position along the axis, target[c with c[axis] = index[c]] = / += src[c] /
 *                    = constant.  Repeated indices resolve as in the reference's sequential loop.
 * ktc_index_select:  indexSelect (JVM:484-502) on the [outer, axis_len, inner] view, 1-D index.
 * ktc_index_add:     indexAdd (JVM:504-518): target[o, index[k], n] += src[o, k, n] * alpha, k ascending.
 * An index outside [0, extent) returns KTC_EINVAL (the reference throws IllegalArgumentException);
 * these five calls wait for the device in order to report it. */
enum { KTC_SCATTER_SET = 0, KTC_SCATTER_ADD = 1, KTC_SCATTER_CONST = 2 };
KTC_API int ktc_copy_strided(ktc_buf dst, int64_t dst_offset, const int64_t* dst_strides,
                             ktc_buf src, int64_t src_offset, const int64_t* src_strides,
                             const int64_t* shape, int ndim);
KTC_API int ktc_fill_strided(ktc_buf dst, int64_t dst_offset, const int64_t* dst_strides,
                             const int64_t* shape, int ndim, float value);
KTC_API int ktc_gather_axis(ktc_buf out, ktc_buf in, const int64_t* in_shape,
                            ktc_buf index, const int64_t* index_shape, int ndim, int axis);
KTC_API int ktc_scatter_axis_nd(int mode, ktc_buf target, const int64_t* target_shape,
                                ktc_buf index, const int64_t* index_shape,
                                ktc_buf src, const int64_t* src_shape, int ndim, int axis, float constant);
KTC_API int ktc_index_select(ktc_buf out, ktc_buf in, ktc_buf index,
                             int64_t outer, int64_t axis_len, int64_t n_index, int64_t inner);
KTC_API int ktc_index_add(ktc_buf target, ktc_buf index, ktc_buf src, float alpha,
                          int64_t outer, int64_t axis_len, int64_t n_index, int64_t inner);

/* inplaceScatter along an axis with one index per [outer, inner] position:
 * the Max/Min backward (AggregatingFunctions.kt:68-79; JVM:227-256,
 * kernels.cl:521-546).  target is [outer, axis_len, inner]; index and src are
 * [outer, 1, inner].  An index outside [0, axis_len) is reported as
 * KTC_EINVAL after the stream drains (the JVM throws, JVM:236-237). */
KTC_API int ktc_scatter_axis(ktc_buf target, ktc_buf index, ktc_buf src,
                             int64_t outer, int64_t axis_len, int64_t inner);

/* ---- multi-GPU (no counterpart in the reference, which is single-device) ----
 * One process per GPU.  Rank 0 creates the id, every rank joins with it, and
 * partial reductions / weight gradients are summed in place across ranks. */
#define KTC_COMM_ID_BYTES 128
KTC_API int ktc_comm_unique_id(unsigned char id[KTC_COMM_ID_BYTES]);
KTC_API int ktc_comm_init_rank(int dev, int n_ranks, int rank, const unsigned char id[KTC_COMM_ID_BYTES], ktc_comm* out);
KTC_API int ktc_allreduce_sum(ktc_comm comm, ktc_buf buf, int64_t off, int64_t n);
KTC_API int ktc_comm_destroy(ktc_comm comm);

/* ---- all-reduce through peer memory (one process per GPU, one kernel per call) -------------
 * No counterpart in the reference (a kten tensor lives on one platform, Tensor.kt:143).  The sum of a
 * few small tensors -- the loss partial and the broadcast-gradient results of the sharded path --
 * across the GPUs of one box, without a collective library: each rank owns a mailbox in device
 * memory that every peer maps through a CUDA IPC handle; ONE kernel per rank stores the values into
 * every peer's mailbox (ordinary peer stores over NVLink), waits -- for a bounded time -- until all
 * ranks have done so, and adds the mailbox slots in rank order, in place.  All ranks perform the
 * same additions in the same order: results are identical on every rank and from run to run.
 *   ktc_p2p_create   allocates this rank's mailbox and returns its 64-byte IPC handle; the caller
 *                    gathers the handles of all ranks (any host channel) ...
 *   ktc_p2p_connect  ... and passes them, rank-major, n_ranks * 64 bytes.  A host barrier must
 *                    separate connect from the first all-reduce, and the last all-reduce from destroy.
 *   ktc_p2p_allreduce_sum  enqueues the kernel on the device's compute stream: up to
 *                    KTC_P2P_MAX_TENSORS tensors, KTC_P2P_MAX_FLOATS floats in total per call.  Every
 *                    rank must make the same sequence of calls.
 *   ktc_p2p_status   waits for the stream; *status = KTC_OK, or KTC_ETIMEOUT if a rank failed to
 *                    arrive within the limit (tunable p2p_wait_ms, default 10000): the kernel then
 *                    returned without summing, the context stays usable, the communicator does not
 *                    (destroy it).
 * ktc_test_p2p_connect_self wires every peer slot to this rank's own mailbox, so that the absent ranks
 * never arrive: the time-out path on a single GPU, without a second process. */
#define KTC_P2P_HANDLE_BYTES 64
#define KTC_P2P_MAX_RANKS 16
#define KTC_P2P_MAX_FLOATS 16384
#define KTC_P2P_MAX_TENSORS 8
typedef uint64_t ktc_p2p;
KTC_API int ktc_p2p_create(int dev, int n_ranks, int rank, ktc_p2p* out, unsigned char handle_out[KTC_P2P_HANDLE_BYTES]);
KTC_API int ktc_p2p_connect(ktc_p2p p, const unsigned char* all_handles);
KTC_API int ktc_p2p_allreduce_sum(ktc_p2p p, const ktc_buf* bufs, const int64_t* counts, int n_bufs);
KTC_API int ktc_p2p_status(ktc_p2p p, int* status);
KTC_API int ktc_p2p_destroy(ktc_p2p p);
KTC_API int ktc_test_p2p_connect_self(ktc_p2p p);

/* ---- measurement -----------------------------------------------------------
 * CUDA events recorded on the device's compute stream; launch counter. */
KTC_API int ktc_timer_start(int dev);
KTC_API int ktc_timer_stop(int dev, float* elapsed_ms);   /* waits for the stop event */
KTC_API int64_t ktc_launch_count(void);                    /* kernels launched by this library so far */
KTC_API int ktc_flush_l2(int dev);                         /* overwrites a scratch buffer larger than L2 */
KTC_API int ktc_tune_set(const char* key, int value);      /* launch-shape tunables (tile sizes, CTAs per SM); also env KTC_<KEY> */

/* ---- test hooks (host-side failure injection; nothing here faults a GPU) ---- */
KTC_API int ktc_test_inject_comm_error(int n_calls);        /* next n collective calls report KTC_ECOMM */
KTC_API int ktc_test_bounded_wait(int dev, int64_t limit_ns, int* status);   /* waits on a flag nothing sets */
/* Generates and compiles (NVRTC, no device needed) the kernel for an expression program: the
 * build check for run-time generated code.  leaf_inner[l] != 0: leaf l varies along the innermost
 * axis; leaf_fixed[l] != 0: it does not depend on the row.  rank3: three collapsed dimensions.
 * KTC_ENOTSUP when NVRTC is not installed. */
KTC_API int ktc_test_expr_compile(const uint32_t* code, int n_code, int n_leaves, const int* leaf_inner, const int* leaf_fixed,
                                  int rank3, int sink, int64_t* cubin_bytes, double* compile_ms);
/* The same for the softmax row kernel with an epilogue program (ktc_softmax_xent_forward_expr) on rows of `cols` columns. */
KTC_API int ktc_test_softmax_expr_compile(const uint32_t* code, int n_code, int n_leaves, const int* leaf_inner, const int* leaf_fixed,
                                          int soft_leaf, int cols, int64_t* cubin_bytes, double* compile_ms);
/* The same for a program with several sums (ktc_expr_eval_multi). */
KTC_API int ktc_test_expr_compile_multi(const uint32_t* code, int n_code, int n_leaves, const int* leaf_inner, const int* leaf_fixed,
                                        int rank3, const int* sink_kinds, int n_sinks, int64_t* cubin_bytes, double* compile_ms);

#ifdef __cplusplus
}
#endif
#endif /* KTEN_CUDA_H */
