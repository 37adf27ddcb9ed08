// ktc_math_more.cuh -- the remaining unary maps and the tensor compares of the raw-tensor SPI.
//
// Semantics are kten-jvm's (backend/kten-jvm/.../store/JVMRawTensor.kt):
//   sinh cosh sin cos tan asin acos atan   java.lang.Math on the widened double, narrowed once
//                                          (JVM:401-403, 415-425): effectively the correctly rounded float.
//                                          CUDA's float functions are used where their documented error is
//                                          at most 2 ulp (cosh 2, sin 1, cos 1, asin 2, acos 2, atan 1); tan (4)
//                                          and sinh (3) are evaluated in double like the reference.
//   abs sign sqrt floor ceil trunc rsqrt   exact IEEE operations (JVM:405-407, 413, 427-429, 433-435);
//                                          sqrt of the widened double narrows to the correctly rounded float sqrt;
//                                          rsqrt is 1f / sqrt(x), two roundings (JVM:435)
//   round                                  Math.round(float).toFloat() (JVM:431): ties towards +infinity, NaN -> 0,
//                                          saturation at the Int range, never -0
//   eq / neq                               |a - b| < epsilon in float (JVM:371-377, 387-393)
#pragma once

#include "ktc_math.cuh"

namespace ktc {

__device__ __forceinline__ float java_round(float x) {
    if (x != x) return 0.0f;
    if (x >= 2147483648.0f) return 2147483648.0f;          // Int.MAX_VALUE.toFloat()
    if (x <= -2147483648.0f) return -2147483648.0f;
    float r = floorf(x);
    if (__fsub_rn(x, r) >= 0.5f) r = __fadd_rn(r, 1.0f);    // x - floor(x) is exact
    return __fadd_rn(r, 0.0f);                              // -0 -> +0: the result went through an Int
}

__device__ __forceinline__ float java_signum(float x) {
    if (x != x || x == 0.0f) return x;                      // NaN and +-0 are returned unchanged
    return x > 0.0f ? 1.0f : -1.0f;
}

template <> struct UnOp<KTC_SINH>  { __device__ __forceinline__ float operator()(float x) const { return (float)sinh((double)x); } };
template <> struct UnOp<KTC_COSH>  { __device__ __forceinline__ float operator()(float x) const { return coshf(x); } };
template <> struct UnOp<KTC_ABS>   { __device__ __forceinline__ float operator()(float x) const { return fabsf(x); } };
template <> struct UnOp<KTC_SIGN>  { __device__ __forceinline__ float operator()(float x) const { return java_signum(x); } };
template <> struct UnOp<KTC_SQRT>  { __device__ __forceinline__ float operator()(float x) const { return __fsqrt_rn(x); } };
template <> struct UnOp<KTC_SIN>   { __device__ __forceinline__ float operator()(float x) const { return sinf(x); } };
template <> struct UnOp<KTC_COS>   { __device__ __forceinline__ float operator()(float x) const { return cosf(x); } };
template <> struct UnOp<KTC_TAN>   { __device__ __forceinline__ float operator()(float x) const { return (float)tan((double)x); } };
template <> struct UnOp<KTC_ASIN>  { __device__ __forceinline__ float operator()(float x) const { return asinf(x); } };
template <> struct UnOp<KTC_ACOS>  { __device__ __forceinline__ float operator()(float x) const { return acosf(x); } };
template <> struct UnOp<KTC_ATAN>  { __device__ __forceinline__ float operator()(float x) const { return atanf(x); } };
template <> struct UnOp<KTC_FLOOR> { __device__ __forceinline__ float operator()(float x) const { return floorf(x); } };
template <> struct UnOp<KTC_CEIL>  { __device__ __forceinline__ float operator()(float x) const { return ceilf(x); } };
template <> struct UnOp<KTC_ROUND> { __device__ __forceinline__ float operator()(float x) const { return java_round(x); } };
template <> struct UnOp<KTC_TRUNC> { __device__ __forceinline__ float operator()(float x) const { return truncf(x); } };
template <> struct UnOp<KTC_RSQRT> { __device__ __forceinline__ float operator()(float x) const { return __fdiv_rn(1.0f, __fsqrt_rn(x)); } };

// eq / neq against a constant
template <bool NEQ> struct EqScalar {
    float v, eps;
    __device__ __forceinline__ float operator()(float x) const {
        const bool same = fabsf(__fsub_rn(x, v)) < eps;
        return (same != NEQ) ? 1.0f : 0.0f;
    }
};

// tensor (cmp) tensor -> 1.0f / 0.0f
template <int OP> struct CompareT {
    float eps;
    __device__ __forceinline__ float operator()(float a, float b) const {
        bool r;
        if (OP == KTC_LT) r = a < b;
        else if (OP == KTC_LTE) r = a <= b;
        else if (OP == KTC_GT) r = a > b;
        else if (OP == KTC_GTE) r = a >= b;
        else { const bool same = fabsf(__fsub_rn(a, b)) < eps; r = (OP == KTC_EQ) ? same : !same; }
        return r ? 1.0f : 0.0f;
    }
};

// maskedFill (JVM:537-540): where the mask is exactly 1f the value, else the element
struct MaskedFill {
    float value;
    __device__ __forceinline__ float operator()(float x, float m) const { return m == 1.0f ? value : x; }
};

}  // namespace ktc
