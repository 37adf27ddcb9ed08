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
#include "ktc_fastmath.h"
#include "ktc_fastmath2.cuh"

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
// Reference path: evaluate in double and narrow once, exactly as the JVM does.  Kept out
// of line: these are the rarely taken slow paths of the float-only functions below, and
// inlining them into every unrolled element blows up the instruction footprint.
static __device__ __noinline__ float exp_ref(float x)  { return (float)exp((double)x); }
__device__ __forceinline__ float log_ref(float x)  { return (float)log((double)x); }
__device__ __forceinline__ float tanh_ref(float x) { return (float)tanh((double)x); }

// Math.pow differs from C99 pow in two corners: a NaN exponent gives NaN even
// for base 1, and |base| == 1 with an infinite exponent gives NaN.
static __device__ __noinline__ float pow_ref(float x, float y) {
    if (y == 0.0f) return 1.0f;
    if (y != y || x != x) return CUDART_NAN_F;
    if (isinf(y) && fabsf(x) == 1.0f) return CUDART_NAN_F;
    return (float)pow((double)x, (double)y);
}

// Fast paths (ktc_fastmath.h): float-only exp and pow, about 0.5-0.6 ulp, verified on
// the host against the double libm; arguments outside their domain (results that
// leave the normal range, zero / negative / non-finite operands) take the double path,
// which also carries Math.pow's special cases.
__device__ __forceinline__ float exp_f(float x) {
    float r;
    return kf_exp(x, &r) ? r : exp_ref(x);
}
// correctly rounded exp for the sigmoid composite: e is then bit-identical to the
// JVM's (float)Math.exp, and the two IEEE operations that follow reproduce it exactly
__device__ __forceinline__ float exp_cr(float x) {
    float r;
    return kf_exp_cr(x, &r) ? r : exp_ref(x);
}
__device__ __forceinline__ float pow_f(float x, float y) {
    if (y == 0.0f) return 1.0f;
    float r;
    return kf_pow(x, y, &r) ? r : pow_ref(x, y);
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
// sigmoid = 1f / (1f + exp(-1f * x)) with the reference's own two IEEE operations after the exp.  A one-ulp
// slip in e = exp(-x) can move the result by up to 3 ulp (1 + e rounds away a bit of e, and the reciprocal can
// double a relative error when its mantissa wraps), so e is always the CORRECTLY ROUNDED exp: the result is
// then the reference's, bit for bit, for every argument, and does not depend on which kernel evaluates it.
template <> struct UnOp<KTC_SIGMOID> {
    __device__ __forceinline__ float operator()(float x) const {
        const float e = exp_cr(__fmul_rn(-1.0f, x));
        return __frcp_rn(__fadd_rn(1.0f, e));        // 1f / (1f + e): the IEEE reciprocal is the IEEE quotient
    }
};
template <> struct UnOp<KTC_RECIPROCAL> { __device__ __forceinline__ float operator()(float x) const { return __frcp_rn(x); } };
template <> struct UnOp<KTC_NEG>  { __device__ __forceinline__ float operator()(float x) const { return -x; } };

// tensor (op) constant and constant (op) tensor
template <int OP> struct ScalarRight { float s; __device__ __forceinline__ float operator()(float a) const { return BinOp<OP>()(a, s); } };
template <int OP> struct ScalarLeft  { float s; __device__ __forceinline__ float operator()(float a) const { return BinOp<OP>()(s, a); } };
// x pow 2 is exactly x*x: the double product of two widened floats has at most
// 48 significant bits, so Math.pow's result narrows to the float product.
struct Square { __device__ __forceinline__ float operator()(float a) const { return __fmul_rn(a, a); } };
struct Identity { __device__ __forceinline__ float operator()(float a) const { return a; } };

// ---- two elements per instruction (ktc_fastmath2.cuh); each lane equals the scalar function above ----------
__device__ __forceinline__ void exp_f_pair(float x0, float x1, float& o0, float& o1) {
    const f2 r = kf2_exp(make_float2(x0, x1));
    o0 = kf_exp_in_domain(x0) ? r.x : exp_ref(x0);
    o1 = kf_exp_in_domain(x1) ? r.y : exp_ref(x1);
}
__device__ __forceinline__ void exp_cr_pair(float x0, float x1, float& o0, float& o1) {
    bool ok0, ok1;
    const f2 r = kf2_exp_cr(make_float2(x0, x1), &ok0, &ok1);
    o0 = ok0 ? r.x : exp_ref(x0);
    o1 = ok1 ? r.y : exp_ref(x1);
}
__device__ __forceinline__ void pow_f_pair(float x0, float x1, float y0, float y1, float& o0, float& o1) {
    bool ok0, ok1;
    const f2 r = kf2_pow(make_float2(x0, x1), make_float2(y0, y1), &ok0, &ok1);
    o0 = (y0 == 0.0f) ? 1.0f : (ok0 ? r.x : pow_ref(x0, y0));
    o1 = (y1 == 0.0f) ? 1.0f : (ok1 ? r.y : pow_ref(x1, y1));
}
__device__ __forceinline__ void sigmoid_pair(float x0, float x1, float& o0, float& o1) {
    const f2 a = mul2(make_float2(x0, x1), F2(-1.0f));
    float e0, e1;
    exp_cr_pair(a.x, a.y, e0, e1);
    const f2 d = add2(F2(1.0f), make_float2(e0, e1));
    o0 = __frcp_rn(d.x); o1 = __frcp_rn(d.y);
}
// float4 forms picked by the map kernels (overloads of the generic per-element application)
__device__ __forceinline__ float4 apply1(const UnOp<KTC_EXP>&, float4 a) {
    float4 o; exp_f_pair(a.x, a.y, o.x, o.y); exp_f_pair(a.z, a.w, o.z, o.w); return o;
}
__device__ __forceinline__ float4 apply1(const UnOp<KTC_SIGMOID>&, float4 a) {
    float4 o; sigmoid_pair(a.x, a.y, o.x, o.y); sigmoid_pair(a.z, a.w, o.z, o.w); return o;
}
__device__ __forceinline__ float4 apply2(const BinOp<KTC_POW>&, float4 a, float4 b) {
    float4 o; pow_f_pair(a.x, a.y, b.x, b.y, o.x, o.y); pow_f_pair(a.z, a.w, b.z, b.w, o.z, o.w); return o;
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
