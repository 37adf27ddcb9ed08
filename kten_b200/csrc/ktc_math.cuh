// ktc_math.cuh -- per-element arithmetic of the kten float32 hot path.
//
// The target semantics are kten-jvm's (backend/kten-jvm/.../store/JVMRawTensor.kt):
//   + - * /            IEEE-754 binary32, round-to-nearest-even, denormals kept
//                      (JVM:110-136).  This translation unit is compiled with
//                      -fmad=false so a fused multiply-add is emitted only where
//                      fmaf() is written out.
//   pow/exp/log/tanh   java.lang.Math on the widened double, narrowed once
//                      (JVM:138-144, 395-397): effectively the correctly
//                      rounded float.
//   sigmoid            e = (float)exp((double)(-1f*x)); 1f / (1f + e)  (JVM:399)
//   max/min/clamp      Math.max/min: NaN-propagating, -0 < +0 (JVM:159-160, 409-411)
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>

#include "../../include/kten_cuda.h"
#include "ktc_fastmath_d.h"

namespace ktc {

// ---- Math.max / Math.min -------------------------------------------------------
__device__ __forceinline__ float jmax(float a, float b) {
    if (a != a) return a;
    if (a == 0.0f && b == 0.0f) return __int_as_float(__float_as_int(a) & __float_as_int(b));
    return (a >= b) ? a : b;
}
__device__ __forceinline__ float jmin(float a, float b) {
    if (a != a) return a;
    if (a == 0.0f && b == 0.0f) return __int_as_float(__float_as_int(a) | __float_as_int(b));
    return (a <= b) ? a : b;
}

// ---- transcendental functions -----------------------------------------------------
// kten-jvm evaluates these on the widened double and narrows once.  exp, sigmoid and pow do the same
// with a short table-driven double evaluation (ktc_fastmath_d.h): the value before narrowing is within
// 2^-41 of the true one, so the result is the reference's float except for about one argument in 10^7
// (one ulp there; sigmoid at most two).  pow arguments outside that routine's domain -- zero, negative,
// subnormal or non-finite base, non-finite exponent, results far outside the float range -- take the
// double-precision library routine below, which also carries Math.pow's special cases.  It is kept out
// of line: it is rarely taken, and inlining it into every unrolled element blows up the kernel.
//
// Math.pow differs from C99 pow in two corners: a NaN exponent gives NaN even for base 1, and
// |base| == 1 with an infinite exponent gives NaN.
static __device__ __noinline__ float pow_ref(float x, float y) {
    if (y == 0.0f) return 1.0f;
    if (y != y || x != x) return CUDART_NAN_F;
    if (isinf(y) && fabsf(x) == 1.0f) return CUDART_NAN_F;
    return (float)pow((double)x, (double)y);
}

__device__ __forceinline__ float exp_f(float x) { return kd_expf(x); }
__device__ __forceinline__ float pow_f(float x, float y) {
    bool ok;
    const float r = kd_pow(x, y, &ok);
    return ok ? r : pow_ref(x, y);
}
// log and tanh: CUDA's logf (max error 1 ulp) and tanhf (2 ulp) stay within the
// 2-ulp bar against the correctly rounded value kten-jvm returns.
__device__ __forceinline__ float log_f(float x)  { return logf(x); }
__device__ __forceinline__ float tanh_f(float x) { return tanhf(x); }

template <int OP> struct BinOp;
template <> struct BinOp<KTC_PLUS>  { __device__ __forceinline__ float operator()(float a, float b) const { return __fadd_rn(a, b); } };
template <> struct BinOp<KTC_MINUS> { __device__ __forceinline__ float operator()(float a, float b) const { return __fsub_rn(a, b); } };
template <> struct BinOp<KTC_TIMES> { __device__ __forceinline__ float operator()(float a, float b) const { return __fmul_rn(a, b); } };
template <> struct BinOp<KTC_DIV>   { __device__ __forceinline__ float operator()(float a, float b) const { return __fdiv_rn(a, b); } };
template <> struct BinOp<KTC_POW>   { __device__ __forceinline__ float operator()(float a, float b) const { return pow_f(a, b); } };

template <int OP> struct UnOp;
template <> struct UnOp<KTC_EXP>  { __device__ __forceinline__ float operator()(float x) const { return exp_f(x); } };
template <> struct UnOp<KTC_LOG>  { __device__ __forceinline__ float operator()(float x) const { return log_f(x); } };
template <> struct UnOp<KTC_TANH> { __device__ __forceinline__ float operator()(float x) const { return tanh_f(x); } };
// sigmoid = 1f / (1f + exp(-1f * x)) with the reference's own two IEEE operations after the exp
// (JVMRawTensor.kt:399); e is Math.exp's narrowed value (see kd_sigmoid).
template <> struct UnOp<KTC_SIGMOID> { __device__ __forceinline__ float operator()(float x) const { return kd_sigmoid(x); } };
template <> struct UnOp<KTC_RECIPROCAL> { __device__ __forceinline__ float operator()(float x) const { return __frcp_rn(x); } };
template <> struct UnOp<KTC_NEG>  { __device__ __forceinline__ float operator()(float x) const { return -x; } };

// tensor (op) constant and constant (op) tensor
template <int OP> struct ScalarRight { float s; __device__ __forceinline__ float operator()(float a) const { return BinOp<OP>()(a, s); } };
template <int OP> struct ScalarLeft  { float s; __device__ __forceinline__ float operator()(float a) const { return BinOp<OP>()(s, a); } };
// x pow 2 is exactly x*x: the double product of two widened floats has at most
// 48 significant bits, so Math.pow's result narrows to the float product.
struct Square { __device__ __forceinline__ float operator()(float a) const { return __fmul_rn(a, a); } };
struct Identity { __device__ __forceinline__ float operator()(float a) const { return a; } };

// ---- float4 forms picked by the map kernels, the interpreter and the generated kernels ---------------------
// Same values as the scalar functors; the rare slow paths (IEEE reciprocal for a subnormal sigmoid, the
// library pow) are tested once per float4 instead of once per element, which keeps the common path free of
// branches and reconvergence points.
static __device__ __noinline__ float4 exp4_any(float4 a) {
    return make_float4(kd_expf(a.x), kd_expf(a.y), kd_expf(a.z), kd_expf(a.w));
}
__device__ __forceinline__ float4 apply1(const UnOp<KTC_EXP>&, float4 a) {
    const float m = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w)));
    if (m <= KD_EXP_PLAIN_RANGE)                       // no clamp needed (a NaN passes and comes out as NaN)
        return make_float4(kd_expf_in_range(a.x), kd_expf_in_range(a.y), kd_expf_in_range(a.z), kd_expf_in_range(a.w));
    return exp4_any(a);
}
static __device__ __noinline__ float4 sigmoid4_any(float4 a) {
    return make_float4(kd_sigmoid(a.x), kd_sigmoid(a.y), kd_sigmoid(a.z), kd_sigmoid(a.w));
}
__device__ __forceinline__ float4 apply1(const UnOp<KTC_SIGMOID>&, float4 a) {
    // arguments within +-80 (a NaN passes: it comes out as NaN either way) need neither clamp nor denominator test
    const float m = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w)));
    if (m <= KD_SIGMOID_PLAIN_RANGE)
        return make_float4(kd_sigmoid_in_range(a.x), kd_sigmoid_in_range(a.y), kd_sigmoid_in_range(a.z), kd_sigmoid_in_range(a.w));
    return sigmoid4_any(a);
}
__device__ __forceinline__ float4 pow4(float4 a, float4 b) {
    bool k0, k1, k2, k3;
    float4 o;
    o.x = kd_pow(a.x, b.x, &k0); o.y = kd_pow(a.y, b.y, &k1); o.z = kd_pow(a.z, b.z, &k2); o.w = kd_pow(a.w, b.w, &k3);
    if (!(k0 && k1 && k2 && k3)) {
        if (!k0) o.x = pow_ref(a.x, b.x);
        if (!k1) o.y = pow_ref(a.y, b.y);
        if (!k2) o.z = pow_ref(a.z, b.z);
        if (!k3) o.w = pow_ref(a.w, b.w);
    }
    return o;
}
__device__ __forceinline__ float4 apply2(const BinOp<KTC_POW>&, float4 a, float4 b) { return pow4(a, b); }
__device__ __forceinline__ float4 apply1(const ScalarRight<KTC_POW>& f, float4 a) { return pow4(a, make_float4(f.s, f.s, f.s, f.s)); }
__device__ __forceinline__ float4 apply1(const ScalarLeft<KTC_POW>& f, float4 a) { return pow4(make_float4(f.s, f.s, f.s, f.s), a); }

// x / b for a divisor shared by many dividends (a row scalar of a broadcast division, the row sum of a softmax), with
// r = kd_row_reciprocal(b): kd_div_by_reciprocal where its window holds -- tested once per float4 -- and IEEE division elsewhere
static __device__ __noinline__ float4 div_ieee4(float4 x, float b) {
    return make_float4(__fdiv_rn(x.x, b), __fdiv_rn(x.y, b), __fdiv_rn(x.z, b), __fdiv_rn(x.w, b));
}
__device__ __forceinline__ float4 div_by_row(float4 x, float b, float r) {
    const uint32_t in_window = kd_div_window(x.x) & kd_div_window(x.y) & kd_div_window(x.z) & kd_div_window(x.w);
    if (in_window == 0u || r == 0.f) return div_ieee4(x, b);
    return make_float4(kd_div_by_reciprocal(x.x, b, r), kd_div_by_reciprocal(x.y, b, r), kd_div_by_reciprocal(x.z, b, r), kd_div_by_reciprocal(x.w, b, r));
}

// the same with the window test done by the caller (in_window: every dividend of x is known to lie in kd_div_window's
// range -- e.g. exp of an argument above -43); both forms give the IEEE quotient wherever they apply
__device__ __forceinline__ float4 div_by_row_known(float4 x, float b, float r, bool in_window) {
    if (!in_window || r == 0.f) return div_ieee4(x, b);
    return make_float4(kd_div_by_reciprocal(x.x, b, r), kd_div_by_reciprocal(x.y, b, r), kd_div_by_reciprocal(x.z, b, r), kd_div_by_reciprocal(x.w, b, r));
}
// x / b for a divisor that is the same for a whole kernel (a constant of a recorded expression): r = kd_row_reciprocal(b),
// pow2 = kd_is_pow2_divisor(b).  A power of two (a batch size, usually) is one multiplication by its exact reciprocal.
__device__ __forceinline__ float4 div_by_const(float4 x, float b, float r, bool pow2) {
    if (pow2) return make_float4(__fmul_rn(x.x, r), __fmul_rn(x.y, r), __fmul_rn(x.z, r), __fmul_rn(x.w, r));
    return div_by_row(x, b, r);
}

struct ClampOp { float lo, hi; __device__ __forceinline__ float operator()(float x) const { return jmin(jmax(x, lo), hi); } };

template <int OP> struct CompareOp {
    float v;
    __device__ __forceinline__ float operator()(float x) const {
        bool r = (OP == KTC_LT) ? (x < v) : (OP == KTC_LTE) ? (x <= v) : (OP == KTC_GT) ? (x > v) : (x >= v);
        return r ? 1.0f : 0.0f;
    }
};

}  // namespace ktc
