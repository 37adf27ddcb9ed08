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
// Reference path: evaluate in double and narrow once, exactly as the JVM does.
__device__ __forceinline__ float exp_ref(float x)  { return (float)exp((double)x); }
__device__ __forceinline__ float log_ref(float x)  { return (float)log((double)x); }
__device__ __forceinline__ float tanh_ref(float x) { return (float)tanh((double)x); }

// Math.pow differs from C99 pow in two corners: a NaN exponent gives NaN even
// for base 1, and |base| == 1 with an infinite exponent gives NaN.
__device__ __forceinline__ float pow_ref(float x, float y) {
    if (y == 0.0f) return 1.0f;
    if (y != y || x != x) return CUDART_NAN_F;
    if (isinf(y) && fabsf(x) == 1.0f) return CUDART_NAN_F;
    return (float)pow((double)x, (double)y);
}

// exp(x) to well under one ulp in float arithmetic only.
// x = n*ln2 + r with a two-part ln2 (r carried as hi + lo), exp(r) by a
// degree-9 Taylor polynomial, and the final 1 + r + t summed with an exact
// two-sum so that only one rounding of size ulp/2 remains.  Arguments whose
// result would leave the normal range take the double path.
__device__ __forceinline__ float exp_fast(float x) {
    if (!(fabsf(x) <= 87.0f)) return exp_ref(x);          // also NaN
    const float n = rintf(x * 1.44269504088896341f);
    // ln2 = LN2_HI + LN2_LO, LN2_HI has 11 trailing zero bits so n*LN2_HI is exact for |n| < 2^11
    const float LN2_HI = 0.693145751953125f;               // 0x1.62e400p-1
    const float LN2_LO = 1.42860682030941723212e-6f;       // ln2 - LN2_HI
    const float r_hi = fmaf(n, -LN2_HI, x);                // exact
    const float nl = n * LN2_LO;
    const float nl_err = fmaf(n, LN2_LO, -nl);             // exact product error
    const float r = r_hi - nl;
    const float r_lo = ((r_hi - r) - nl) - nl_err;         // r_hi - n*LN2_LO = r + r_lo
    // q(r) = sum_{k=2..9} r^(k-2)/k!
    float q = 2.7557319223985893e-6f;                      // 1/9!
    q = fmaf(q, r, 2.4801587301587302e-5f);
    q = fmaf(q, r, 1.9841269841269841e-4f);
    q = fmaf(q, r, 1.3888888888888889e-3f);
    q = fmaf(q, r, 8.3333333333333333e-3f);
    q = fmaf(q, r, 4.1666666666666664e-2f);
    q = fmaf(q, r, 1.6666666666666666e-1f);
    q = fmaf(q, r, 0.5f);
    const float t = fmaf(r * r, q, fmaf(r, r_lo, r_lo));   // r^2 q + r_lo (1 + r)
    const float hi = 1.0f + r;
    const float err = (1.0f - hi) + r;                     // exact: |1| >= |r|
    const float s = hi + (err + t);
    return s * __int_as_float(((int)n + 127) << 23);       // exact scaling, result normal
}

template <int OP> struct BinOp;
template <> struct BinOp<KTC_PLUS>  { __device__ __forceinline__ float operator()(float a, float b) const { return __fadd_rn(a, b); } };
template <> struct BinOp<KTC_MINUS> { __device__ __forceinline__ float operator()(float a, float b) const { return __fsub_rn(a, b); } };
template <> struct BinOp<KTC_TIMES> { __device__ __forceinline__ float operator()(float a, float b) const { return __fmul_rn(a, b); } };
template <> struct BinOp<KTC_DIV>   { __device__ __forceinline__ float operator()(float a, float b) const { return __fdiv_rn(a, b); } };
template <> struct BinOp<KTC_POW>   { __device__ __forceinline__ float operator()(float a, float b) const { return pow_ref(a, b); } };

template <int OP> struct UnOp;
template <> struct UnOp<KTC_EXP>  { __device__ __forceinline__ float operator()(float x) const { return exp_ref(x); } };
template <> struct UnOp<KTC_LOG>  { __device__ __forceinline__ float operator()(float x) const { return log_ref(x); } };
template <> struct UnOp<KTC_TANH> { __device__ __forceinline__ float operator()(float x) const { return tanh_ref(x); } };
template <> struct UnOp<KTC_SIGMOID> {
    __device__ __forceinline__ float operator()(float x) const {
        const float e = exp_ref(__fmul_rn(-1.0f, x));
        return __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
    }
};
template <> struct UnOp<KTC_RECIPROCAL> { __device__ __forceinline__ float operator()(float x) const { return __fdiv_rn(1.0f, x); } };
template <> struct UnOp<KTC_NEG>  { __device__ __forceinline__ float operator()(float x) const { return -x; } };

// tensor (op) constant and constant (op) tensor
template <int OP> struct ScalarRight { float s; __device__ __forceinline__ float operator()(float a) const { return BinOp<OP>()(a, s); } };
template <int OP> struct ScalarLeft  { float s; __device__ __forceinline__ float operator()(float a) const { return BinOp<OP>()(s, a); } };
// x pow 2 is exactly x*x: the double product of two widened floats has at most
// 48 significant bits, so Math.pow's result narrows to the float product.
struct Square { __device__ __forceinline__ float operator()(float a) const { return __fmul_rn(a, a); } };
struct Identity { __device__ __forceinline__ float operator()(float a) const { return a; } };

struct ClampOp { float lo, hi; __device__ __forceinline__ float operator()(float x) const { return jmin(jmax(x, lo), hi); } };

template <int OP> struct CompareOp {
    float v;
    __device__ __forceinline__ float operator()(float x) const {
        bool r = (OP == KTC_LT) ? (x < v) : (OP == KTC_LTE) ? (x <= v) : (OP == KTC_GT) ? (x > v) : (x >= v);
        return r ? 1.0f : 0.0f;
    }
};

}  // namespace ktc
