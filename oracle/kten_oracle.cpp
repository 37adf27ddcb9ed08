// kten_oracle.cpp -- CPU restatement of kten-jvm's float32 hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
// compared against (tests, the smoke check and the CPU-baseline leg of the
// benchmark).  Nothing in the shipped library calls it and it is never a
// fallback for a missing GPU.
//
// Parity status: the reference (Kotlin 1.4.21 / JDK 12) cannot be compiled or
// run where this is built, so the restatement is pinned against the literal
// vectors of the reference's own test-suite
// (kten-testing/src/main/kotlin/eu/redbean/kten/tensor/tests/TensorTestsBase.kt),
// which hold transcendental results only to 1e-4 absolute.  At the ulp level
// parity is UNPINNED by reference outputs: java.lang.Math is restated through
// glibc's double-precision libm (both < 1 ulp in double, so the narrowed
// float agrees except for rare double-rounding ties).
//
// Every function cites the reference lines it follows; paths are relative to
// the reference project root, with
//   JVM = backend/kten-jvm/src/main/kotlin/eu/redbean/kten/jvm/tensor/store/JVMRawTensor.kt
//   ART = kten-api/src/main/kotlin/eu/redbean/kten/api/tensor/store/AbstractRawTensor.kt
//   SHF = kten-api/src/main/kotlin/eu/redbean/kten/api/autograd/utils/ShapeFunctions.kt
//
// Threading mirrors the reference: out-of-place maps are single-threaded
// (JVM:75-79, 99-103 build a FloatArray with a sequential initialiser), while
// in-place maps, axis aggregation and zeroOut use IntStream.parallel()
// (JVM:95, 106, 219) -- restated as OpenMP "parallel for".  A `tuned` flag
// additionally parallelises the out-of-place maps to report the host's fair
// upper bound.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define KTO_API extern "C" __attribute__((visibility("default")))

enum { KTO_OK = 0, KTO_EINVAL = -1 };

// op codes shared with include/kten_cuda.h
enum { OP_PLUS = 0, OP_MINUS = 1, OP_TIMES = 2, OP_DIV = 3, OP_POW = 4 };
enum { U_EXP = 0, U_LOG = 1, U_TANH = 2, U_SIGMOID = 3, U_RECIPROCAL = 4, U_NEG = 5,
       U_SINH = 6, U_COSH = 7, U_ABS = 8, U_SIGN = 9, U_SQRT = 10, U_SIN = 11, U_COS = 12, U_TAN = 13,
       U_ASIN = 14, U_ACOS = 15, U_ATAN = 16, U_FLOOR = 17, U_CEIL = 18, U_ROUND = 19, U_TRUNC = 20, U_RSQRT = 21 };
enum { C_LT = 0, C_LTE = 1, C_GT = 2, C_GTE = 3, C_EQ = 4, C_NEQ = 5 };
enum { R_SUM = 0, R_MEAN = 1, R_MAX = 2, R_MIN = 3, R_ARGMAX = 4, R_ARGMIN = 5 };

// ---------------------------------------------------------------------------
// java.lang.Math restatements
// ---------------------------------------------------------------------------

// Math.pow(double,double): C99 pow with the two cases where Java differs
// (second argument NaN -> NaN even for base 1; |base| == 1 with an infinite
// exponent -> NaN).  kotlin.math Float.pow widens, calls Math.pow, narrows
// (JVM:138,140).
static inline double java_pow(double x, double y) {
    if (y == 0.0) return 1.0;
    if (std::isnan(y)) return std::numeric_limits<double>::quiet_NaN();
    if (std::isnan(x)) return std::numeric_limits<double>::quiet_NaN();
    if (std::isinf(y) && std::fabs(x) == 1.0) return std::numeric_limits<double>::quiet_NaN();
    return std::pow(x, y);
}

// Math.max / Math.min (float,float): NaN-propagating, -0 < +0
// (used by JVM:159-160 for MAX/MIN and JVM:409-411 for clamp).
static inline float java_max(float a, float b) {
    if (a != a) return a;
    if (a == 0.0f && b == 0.0f) {
        uint32_t ia, ib; std::memcpy(&ia, &a, 4); std::memcpy(&ib, &b, 4);
        uint32_t r = ia & ib; float f; std::memcpy(&f, &r, 4); return f;   // +0 unless both -0
    }
    return (a >= b) ? a : b;   // b NaN -> comparison false -> b
}
static inline float java_min(float a, float b) {
    if (a != a) return a;
    if (a == 0.0f && b == 0.0f) {
        uint32_t ia, ib; std::memcpy(&ia, &a, 4); std::memcpy(&ib, &b, 4);
        uint32_t r = ia | ib; float f; std::memcpy(&f, &r, 4); return f;   // -0 if either is -0
    }
    return (a <= b) ? a : b;
}

static inline float bin_op(int op, float a, float b) {
    switch (op) {
    case OP_PLUS:  return a + b;                                   // JVM:110
    case OP_MINUS: return a - b;                                   // JVM:118
    case OP_TIMES: return a * b;                                   // JVM:124
    case OP_DIV:   return a / b;                                   // JVM:132
    default:       return (float)java_pow((double)a, (double)b);  // JVM:138
    }
}

static inline float un_op(int op, float x) {
    switch (op) {
    case U_EXP:   return (float)std::exp((double)x);               // JVM:395
    case U_LOG:   return (float)std::log((double)x);               // JVM:144
    case U_TANH:  return (float)std::tanh((double)x);              // JVM:397
    case U_SIGMOID: {                                              // JVM:399
        float e = (float)std::exp((double)(-1.0f * x));
        return 1.0f / (1.0f + e);
    }
    case U_RECIPROCAL: return 1.0f / x;                            // JVM:142
    case U_NEG:   return -x;                                       // JVM:122
    // kotlin.math.f(Float) = Math.f(x.toDouble()).toFloat() for the functions below
    case U_SINH:  return (float)std::sinh((double)x);              // JVM:401
    case U_COSH:  return (float)std::cosh((double)x);              // JVM:403
    case U_ABS:   return std::fabs(x);                             // JVM:405
    case U_SIGN:  return (x != x || x == 0.0f) ? x : (x > 0.0f ? 1.0f : -1.0f);   // JVM:407, Math.signum
    case U_SQRT:  return (float)std::sqrt((double)x);              // JVM:413
    case U_SIN:   return (float)std::sin((double)x);               // JVM:415
    case U_COS:   return (float)std::cos((double)x);               // JVM:417
    case U_TAN:   return (float)std::tan((double)x);               // JVM:419
    case U_ASIN:  return (float)std::asin((double)x);              // JVM:421
    case U_ACOS:  return (float)std::acos((double)x);              // JVM:423
    case U_ATAN:  return (float)std::atan((double)x);              // JVM:425
    case U_FLOOR: return (float)std::floor((double)x);             // JVM:427
    case U_CEIL:  return (float)std::ceil((double)x);              // JVM:429
    case U_ROUND: {                                                // JVM:431: Math.round(float).toFloat()
        if (x != x) return 0.0f;                                   // (int) NaN == 0
        double r = std::floor((double)x + 0.5);                    // exact in double; ties go up
        if (r >= 2147483647.0) return (float)2147483647;           // saturates at the Int range
        if (r <= -2147483648.0) return (float)(-2147483647 - 1);
        return (float)(int32_t)r;                                  // through an Int: never -0
    }
    case U_TRUNC: return (x != x || std::isinf(x)) ? x : (x > 0.0f ? (float)std::floor((double)x) : (float)std::ceil((double)x));  // JVM:433, kotlin.math.truncate
    default:      return 1.0f / (float)std::sqrt((double)x);       // JVM:435: 1f / sqrt(x)
    }
}

static inline float cmp_op(int op, float a, float b, float eps) {   // JVM:355-393
    switch (op) {
    case C_LT:  return a < b ? 1.0f : 0.0f;
    case C_LTE: return a <= b ? 1.0f : 0.0f;
    case C_GT:  return a > b ? 1.0f : 0.0f;
    case C_GTE: return a >= b ? 1.0f : 0.0f;
    case C_EQ:  return std::fabs(a - b) < eps ? 1.0f : 0.0f;
    default:    return std::fabs(a - b) < eps ? 0.0f : 1.0f;
    }
}

// ---------------------------------------------------------------------------
// shape algebra
// ---------------------------------------------------------------------------

// Right-aligned NumPy-style common shape; a non-singleton mismatch is an error
// (ART:170-192 builds the shape, SHF:168-185 / 187-201 reject mismatches).
KTO_API int kto_common_shape(const int64_t* sa, int na, const int64_t* sb, int nb,
                             int64_t* out, int* nout) {
    int n = na > nb ? na : nb;
    for (int i = 0; i < n; ++i) {
        int ia = i - (n - na), ib = i - (n - nb);
        int64_t da = ia >= 0 ? sa[ia] : 1, db = ib >= 0 ? sb[ib] : 1;
        if (!(da == db || da == 1 || db == 1)) return KTO_EINVAL;
        out[i] = da > db ? da : db;
    }
    *nout = n;
    return KTO_OK;
}

static int64_t volume(const int64_t* s, int n) {
    int64_t v = 1; for (int i = 0; i < n; ++i) v *= s[i]; return v;
}

// JVMRawTensor.broadcastTo (JVM:51-73): materialise `src` at `tshape`; every
// target index is taken modulo the (left-padded) source extent.
KTO_API int kto_broadcast_to(const float* src, const int64_t* sshape, int sn,
                             const int64_t* tshape, int tn, float* dst) {
    if (sn > tn) return KTO_EINVAL;                                 // SHF:188-189
    int64_t padded[16], sstride[16];
    if (tn > 16) return KTO_EINVAL;
    for (int i = 0; i < tn; ++i) {
        int is = i - (tn - sn);
        padded[i] = is >= 0 ? sshape[is] : 1;
        if (!(padded[i] == tshape[i] || padded[i] == 1)) return KTO_EINVAL;  // SHF:193-199
    }
    int64_t st = 1;
    for (int i = tn - 1; i >= 0; --i) { sstride[i] = st; st *= padded[i]; }
    int64_t total = volume(tshape, tn);
    for (int64_t e = 0; e < total; ++e) {
        int64_t rem = e, off = 0;
        for (int d = tn - 1; d >= 0; --d) {
            int64_t idx = rem % tshape[d]; rem /= tshape[d];
            off += (idx % padded[d]) * sstride[d];
        }
        dst[e] = src[off];
    }
    return KTO_OK;
}

// ---------------------------------------------------------------------------
// elementwise
// ---------------------------------------------------------------------------

// elementwiseOpOnCommonShapedTensors (JVM:75-79): sequential map.  `tuned`
// != 0 parallelises it (not what the reference does; host upper bound only).
KTO_API int kto_binary_same(int op, const float* a, const float* b, float* out,
                            int64_t n, int tuned) {
    if (tuned) {
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) out[i] = bin_op(op, a[i], b[i]);
    } else {
        for (int64_t i = 0; i < n; ++i) out[i] = bin_op(op, a[i], b[i]);
    }
    return KTO_OK;
}

// elementwiseOpOnTensors (JVM:81-87): both operands are materialised at the
// common shape, then mapped.  `out` must hold the common volume.
KTO_API int kto_binary_bcast(int op, const float* a, const int64_t* ashape, int an,
                             const float* b, const int64_t* bshape, int bn, float* out) {
    int64_t cs[16]; int cn;
    if (an > 16 || bn > 16) return KTO_EINVAL;
    if (kto_common_shape(ashape, an, bshape, bn, cs, &cn) != KTO_OK) return KTO_EINVAL;
    int64_t total = volume(cs, cn);
    bool a_same = (an == cn) && std::memcmp(ashape, cs, sizeof(int64_t) * cn) == 0;
    bool b_same = (bn == cn) && std::memcmp(bshape, cs, sizeof(int64_t) * cn) == 0;
    std::vector<float> ta, tb;
    const float* pa = a; const float* pb = b;
    if (!a_same) { ta.resize(total); kto_broadcast_to(a, ashape, an, cs, cn, ta.data()); pa = ta.data(); }
    if (!b_same) { tb.resize(total); kto_broadcast_to(b, bshape, bn, cs, cn, tb.data()); pb = tb.data(); }
    return kto_binary_same(op, pa, pb, out, total, 0);
}

// The same values without materialising anything and on all host threads: not what the reference does,
// the host's upper bound only (the "tuned" CPU figure of the benchmark).  Rows of the innermost dimension
// are spread over the threads; operand offsets follow broadcast strides (0 where an extent is 1).
KTO_API int kto_binary_bcast_tuned(int op, const float* a, const int64_t* ashape, int an,
                                   const float* b, const int64_t* bshape, int bn, float* out) {
    int64_t cs[16]; int cn;
    if (an > 16 || bn > 16) return KTO_EINVAL;
    if (kto_common_shape(ashape, an, bshape, bn, cs, &cn) != KTO_OK) return KTO_EINVAL;
    int64_t sa[16], sb[16], st_a = 1, st_b = 1;
    for (int i = cn - 1; i >= 0; --i) {
        const int ia = i - (cn - an), ib = i - (cn - bn);
        const int64_t da = ia >= 0 ? ashape[ia] : 1, db = ib >= 0 ? bshape[ib] : 1;
        sa[i] = (da == 1 && cs[i] != 1) ? 0 : st_a; st_a *= da;
        sb[i] = (db == 1 && cs[i] != 1) ? 0 : st_b; st_b *= db;
    }
    const int64_t inner = cn ? cs[cn - 1] : 1;
    const int64_t rows = volume(cs, cn) / (inner ? inner : 1);
    const int64_t ia_step = cn ? sa[cn - 1] : 0, ib_step = cn ? sb[cn - 1] : 0;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        int64_t rem = r, oa = 0, ob = 0;
        for (int d = cn - 2; d >= 0; --d) { const int64_t idx = rem % cs[d]; rem /= cs[d]; oa += idx * sa[d]; ob += idx * sb[d]; }
        float* o = out + r * inner;
        for (int64_t i = 0; i < inner; ++i) o[i] = bin_op(op, a[oa + i * ia_step], b[ob + i * ib_step]);
    }
    return KTO_OK;
}

// inplaceElementwiseOpOnTensors (JVM:89-97): equal shapes only (checked by
// the caller), parallel stream.
KTO_API int kto_binary_inplace(int op, float* a, const float* b, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) a[i] = bin_op(op, a[i], b[i]);
    return KTO_OK;
}

// mapElementsCopy with a constant (JVM:99-103, 112-140) and
// TensorOperations.pow(constant, raw)
// (backend/kten-jvm/.../operations/AbstractJVMTensorOperations.kt:94-96).
KTO_API int kto_scalar(int op, const float* a, float s, int scalar_first, float* out,
                       int64_t n, int tuned) {
    if (tuned) {
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) out[i] = scalar_first ? bin_op(op, s, a[i]) : bin_op(op, a[i], s);
    } else {
        for (int64_t i = 0; i < n; ++i) out[i] = scalar_first ? bin_op(op, s, a[i]) : bin_op(op, a[i], s);
    }
    return KTO_OK;
}

// inplaceMapElements with a constant (JVM:105-108, 116, 130, 136): parallel.
KTO_API int kto_scalar_inplace(int op, float* a, float s, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) a[i] = bin_op(op, a[i], s);
    return KTO_OK;
}

// unary maps (JVM:122, 142, 144, 395-399): sequential.
KTO_API int kto_unary(int op, const float* a, float* out, int64_t n, int tuned) {
    if (tuned) {
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) out[i] = un_op(op, a[i]);
    } else {
        for (int64_t i = 0; i < n; ++i) out[i] = un_op(op, a[i]);
    }
    return KTO_OK;
}

// tensor (cmp) tensor on equal shapes and tensor (cmp) constant (JVM:355-393): 1.0f / 0.0f.
KTO_API int kto_compare_tensor(int op, const float* a, const float* b, float eps, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = cmp_op(op, a[i], b[i], eps);
    return KTO_OK;
}
KTO_API int kto_compare_scalar(int op, const float* a, float v, float eps, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = cmp_op(op, a[i], v, eps);
    return KTO_OK;
}

// maskedFill (JVM:537-540): the mask is broadcast to the tensor's shape, then
// out = (mask == 1f) ? value : this.
KTO_API int kto_masked_fill(const float* a, const int64_t* ashape, int an, const float* mask, const int64_t* mshape, int mn,
                            float value, float* out) {
    int64_t n = 1;
    for (int i = 0; i < an; ++i) n *= ashape[i];
    std::vector<float> m((size_t)n);
    if (kto_broadcast_to(mask, mshape, mn, ashape, an, m.data()) != KTO_OK) return KTO_EINVAL;
    for (int64_t i = 0; i < n; ++i) out[i] = (m[(size_t)i] == 1.0f) ? value : a[i];
    return KTO_OK;
}

// clamp (JVM:409-411): Math.min(Math.max(x, lo), hi).
KTO_API int kto_clamp(const float* a, float lo, float hi, float* out, int64_t n, int tuned) {
    if (tuned) {
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) out[i] = java_min(java_max(a[i], lo), hi);
    } else {
        for (int64_t i = 0; i < n; ++i) out[i] = java_min(java_max(a[i], lo), hi);
    }
    return KTO_OK;
}

// fill (FloatArray.fill / createRaw(shape){c}) and zeroOut
// (AbstractJVMTensorOperations.kt:85-88, parallel).
KTO_API int kto_fill(float* a, float v, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) a[i] = v;
    return KTO_OK;
}

// ---------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------

// aggregateOverAxis (JVM:211-225) with mapAggregatingOp (JVM:154-209) on the
// collapsed view [outer, axis_len, inner]: parallel over the outputs, serial
// in axis order inside.  mode 0 = jvm-faithful (float accumulator, axis
// order); mode 1 = exact (double accumulator, one narrowing) for SUM/MEAN.
// Index results are float32 (JVM:180).
KTO_API int kto_aggregate_axis(int op, const float* in, int64_t outer, int64_t A,
                               int64_t inner, float* out, int mode) {
    if (outer < 0 || A < 0 || inner < 0) return KTO_EINVAL;
    const int64_t nout = outer * inner;
    #pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < nout; ++o) {
        const int64_t io = o / inner, ii = o % inner;
        const float* p = in + io * A * inner + ii;
        float r;
        switch (op) {
        case R_ARGMAX: case R_ARGMIN: {                            // JVM:166-184
            float best = (op == R_ARGMAX) ? -INFINITY : INFINITY;
            float idx = 0.0f;
            for (int64_t j = 0; j < A; ++j) {
                float v = p[j * inner];
                if ((op == R_ARGMAX && v > best) || (op == R_ARGMIN && v < best)) { best = v; idx = (float)j; }
            }
            r = idx; break;
        }
        case R_MEAN: case R_SUM: {                                 // JVM:185-192, 193-207
            if (mode == 0) {
                float acc = 0.0f;
                for (int64_t j = 0; j < A; ++j) acc += p[j * inner];
                r = (op == R_MEAN) ? acc / (float)A : acc;
            } else {
                double acc = 0.0;
                for (int64_t j = 0; j < A; ++j) acc += (double)p[j * inner];
                r = (op == R_MEAN) ? (float)(acc / (double)A) : (float)acc;
            }
            break;
        }
        case R_MAX: {
            float acc = -INFINITY;
            for (int64_t j = 0; j < A; ++j) acc = java_max(acc, p[j * inner]);
            r = acc; break;
        }
        default: {
            float acc = INFINITY;
            for (int64_t j = 0; j < A; ++j) acc = java_min(acc, p[j * inner]);
            r = acc; break;
        }
        }
        out[o] = r;
    }
    return KTO_OK;
}

// sum() (JVM:146-148, FloatArray.sum = sequential float) and mean()
// (JVM:150-152, FloatArray.average = sequential double then narrowed).
// mode 0 = jvm-faithful, mode 1 = exact (double accumulate).
KTO_API int kto_reduce_all(int op, const float* in, int64_t n, float* out, int mode) {
    if (op == R_SUM && mode == 0) {
        float acc = 0.0f;
        for (int64_t i = 0; i < n; ++i) acc += in[i];
        *out = acc;
        return KTO_OK;
    }
    double acc = 0.0;
    for (int64_t i = 0; i < n; ++i) acc += (double)in[i];
    if (op == R_MEAN) *out = (float)(acc / (double)n);   // average(): NaN when n == 0
    else *out = (float)acc;
    return KTO_OK;
}

// Sum of |x| in double: the scale the reduction tolerance is relative to.
KTO_API double kto_abs_sum(const float* in, int64_t n) {
    double acc = 0.0;
    #pragma omp parallel for reduction(+:acc) schedule(static)
    for (int64_t i = 0; i < n; ++i) acc += std::fabs((double)in[i]);
    return acc;
}

// mayUnexpand (kten-api/.../autograd/functions/Utils.kt:14-41): reduce `in`
// (shape in_shape) to old_shape: one sum(0) per prepended dimension, then
// sum(d, keepDims) for every remaining dimension whose extent differs.
// Done here in one sweep with a double accumulator per output (mode 1) or by
// literally chaining the axis sums in the reference's order (mode 0).
KTO_API int kto_sum_to_shape(const float* in, const int64_t* in_shape, int in_n,
                             const int64_t* old_shape, int old_n, float* out, int mode) {
    if (old_n > in_n || in_n > 16) return KTO_EINVAL;
    const int lead = in_n - old_n;
    for (int i = 0; i < old_n; ++i)
        if (!(old_shape[i] == in_shape[lead + i] || old_shape[i] == 1)) return KTO_EINVAL;
    if (mode == 0) {
        std::vector<float> cur(in, in + volume(in_shape, in_n));
        std::vector<int64_t> shp(in_shape, in_shape + in_n);
        for (int i = 0; i < lead; ++i) {                            // Utils.kt:24-30
            int64_t A = shp[0], inner = 1;
            for (size_t d = 1; d < shp.size(); ++d) inner *= shp[d];
            std::vector<float> nxt(inner);
            kto_aggregate_axis(R_SUM, cur.data(), 1, A, inner, nxt.data(), 0);
            cur.swap(nxt);
            if (shp.size() > 1) shp.erase(shp.begin()); else shp[0] = 1;
        }
        for (int d = 0; d < old_n; ++d) {                           // Utils.kt:32-38
            if (shp[d] == old_shape[d]) continue;
            int64_t outer = 1, inner = 1, A = shp[d];
            for (int k = 0; k < d; ++k) outer *= shp[k];
            for (size_t k = d + 1; k < shp.size(); ++k) inner *= shp[k];
            std::vector<float> nxt(outer * inner);
            kto_aggregate_axis(R_SUM, cur.data(), outer, A, inner, nxt.data(), 0);
            cur.swap(nxt);
            shp[d] = 1;
        }
        std::memcpy(out, cur.data(), cur.size() * sizeof(float));
        return KTO_OK;
    }
    bool any_reduced = lead > 0;
    for (int i = 0; i < old_n; ++i) any_reduced |= (old_shape[i] != in_shape[lead + i]);
    if (!any_reduced) {                                             // no sum is issued: the tensor itself comes back
        std::memcpy(out, in, volume(in_shape, in_n) * sizeof(float));
        return KTO_OK;
    }
    int64_t ostride[16]; int64_t st = 1;
    for (int i = in_n - 1; i >= 0; --i) {
        int io = i - lead;
        int64_t ext = io >= 0 ? old_shape[io] : 1;
        ostride[i] = (ext == 1) ? 0 : st;
        st *= ext;
    }
    const int64_t nout = volume(old_shape, old_n);
    std::vector<double> acc(nout, 0.0);
    const int64_t total = volume(in_shape, in_n);
    for (int64_t e = 0; e < total; ++e) {
        int64_t rem = e, off = 0;
        for (int d = in_n - 1; d >= 0; --d) { off += (rem % in_shape[d]) * ostride[d]; rem /= in_shape[d]; }
        acc[off] += (double)in[e];
    }
    for (int64_t i = 0; i < nout; ++i) out[i] = (float)acc[i];
    return KTO_OK;
}

KTO_API int kto_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
