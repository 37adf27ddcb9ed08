// ktc_fastmath2.cuh -- the float-only exp / pow / correctly-rounded exp of ktc_fastmath.h, two
// arguments at a time, on Blackwell's packed single-precision instructions.
//
// sm_100 adds IEEE round-to-nearest add, mul and fma on float2 operands (__fadd2_rn, __fmul2_rn,
// __ffma2_rn): one instruction rounds both lanes exactly as the scalar instruction would.  The
// transcendental kernels of this library are bound by instruction issue, not by memory (pow: 88
// thread-instructions per element), and more than half of those instructions are the float-float
// arithmetic below, so evaluating two elements per instruction removes about a third of the issue
// slots.  Every function here mirrors its scalar original operation by operation -- same
// constants, same order, same fused multiply-adds -- so each lane produces the bits the scalar
// code produces (tests/test_gpu_parity.py compares the two on the device), and the accuracy
// bounds verified on the host for ktc_fastmath.h carry over unchanged.  Integer steps (exponent
// extraction, table index, scaling by a power of two) and the domain checks stay per lane.
#pragma once

#include <cuda_runtime.h>

#include "ktc_fastmath.h"

namespace ktc {

typedef float2 f2;

__device__ __forceinline__ f2 F2(float a) { return make_float2(a, a); }
__device__ __forceinline__ f2 mul2(f2 a, f2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ f2 add2(f2 a, f2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) { return __ffma2_rn(a, b, c); }
// a - b: b * -1 is exact, so the fused form rounds a - b once, like the scalar subtraction
__device__ __forceinline__ f2 sub2(f2 a, f2 b) { return __ffma2_rn(b, F2(-1.0f), a); }
__device__ __forceinline__ f2 neg2(f2 a) { return __fmul2_rn(a, F2(-1.0f)); }          // exact

// kf_exp_core, two lanes
__device__ __forceinline__ f2 kf2_exp_core(f2 r, f2 rl) {
    f2 q = F2(2.7557319223985893e-6f);
    q = fma2(q, r, F2(2.4801587301587302e-5f));
    q = fma2(q, r, F2(1.9841269841269841e-4f));
    q = fma2(q, r, F2(1.3888888888888889e-3f));
    q = fma2(q, r, F2(8.3333333333333333e-3f));
    q = fma2(q, r, F2(4.1666666666666664e-2f));
    q = fma2(q, r, F2(1.6666666666666666e-1f));
    q = fma2(q, r, F2(0.5f));
    const f2 t = fma2(mul2(r, r), q, fma2(r, rl, rl));
    const f2 hi = add2(F2(1.0f), r);
    const f2 err = add2(sub2(F2(1.0f), hi), r);
    return add2(hi, add2(err, t));
}

__device__ __forceinline__ f2 kf2_pow2_from_magic(f2 v_plus_magic) {
    return make_float2(kf_pow2_from_magic(v_plus_magic.x), kf_pow2_from_magic(v_plus_magic.y));
}

// kf_exp on two arguments; the result of a lane is meaningful only if that lane's argument is in
// the fast domain (|x| <= 87): the caller checks kf2_exp_ok per lane
__device__ __forceinline__ bool kf_exp_in_domain(float x) { return fabsf(x) <= 87.0f; }

__device__ __forceinline__ f2 kf2_exp(f2 x) {
    const f2 v = fma2(x, F2(1.44269504088896341f), F2(KF_MAGIC));
    const f2 n = sub2(v, F2(KF_MAGIC));
    const f2 rh = fma2(n, F2(-0.693145751953125f), x);
    const f2 nl = mul2(n, F2(1.42860682030941723212e-6f));
    const f2 r = sub2(rh, nl);
    const f2 rl = sub2(sub2(rh, r), nl);
    return mul2(kf2_exp_core(r, rl), kf2_pow2_from_magic(v));
}

// kf_exp_cr on two arguments.  ok0 / ok1: the lane's result is the correctly rounded exp (argument in
// the domain and the rounding test passed); otherwise the caller takes the double path for that lane.
__device__ __forceinline__ f2 kf2_exp_cr(f2 x, bool* ok0, bool* ok1) {
    const f2 v = fma2(x, F2(92.33248138427734f), F2(KF_MAGIC));
    const f2 kf = sub2(v, F2(KF_MAGIC));
    const int32_t k0 = __float_as_int(v.x) - KF_MAGIC_BITS, k1 = __float_as_int(v.y) - KF_MAGIC_BITS;
    const f2 r1 = fma2(kf, F2(-0.0108184814453125f), x);
    const f2 p2 = mul2(kf, F2(1.1943250683543738e-05f));
    const f2 p2e = fma2(kf, F2(1.1943250683543738e-05f), neg2(p2));
    const f2 r = sub2(r1, p2);
    const f2 bb = sub2(r, r1);
    const f2 e1 = add2(sub2(r1, sub2(r, bb)), sub2(neg2(p2), bb));
    const f2 rl = fma2(kf, F2(-2.5310171168115014e-13f), sub2(e1, p2e));
    const int32_t j0 = k0 & 63, j1 = k1 & 63;
    const float2 row0 = __ldg(reinterpret_cast<const float2*>(&kf_exp2_tab[j0][0]));     // (high, low) of 2^(j/64)
    const float2 row1 = __ldg(reinterpret_cast<const float2*>(&kf_exp2_tab[j1][0]));
    const f2 th = make_float2(row0.x, row1.x), tl = make_float2(row0.y, row1.y);
    f2 q = fma2(r, F2(4.1666666666666664e-2f), F2(1.6666666666666666e-1f));
    q = fma2(r, q, F2(0.5f));
    const f2 e = fma2(mul2(r, r), q, fma2(r, rl, rl));
    const f2 m = mul2(th, r);
    const f2 me = fma2(th, r, neg2(m));
    const f2 s = add2(th, m);
    const f2 se = add2(sub2(th, s), m);
    const f2 low = add2(add2(se, me), fma2(th, e, fma2(tl, r, tl)));
    const f2 res = add2(s, low);
    const f2 rho = add2(sub2(s, res), low);
    const float u0 = __int_as_float((__float_as_int(res.x) & 0x7f800000) - (23 << 23));
    const float u1 = __int_as_float((__float_as_int(res.y) & 0x7f800000) - (23 << 23));
    *ok0 = fabsf(x.x) <= 87.0f && !(fabsf(fabsf(rho.x) - 0.5f * u0) < u0 * 2.44140625e-4f);
    *ok1 = fabsf(x.y) <= 87.0f && !(fabsf(fabsf(rho.y) - 0.5f * u1) < u1 * 2.44140625e-4f);
    return mul2(res, make_float2(__int_as_float(((k0 >> 6) + 127) << 23), __int_as_float(((k1 >> 6) + 127) << 23)));
}

// kf_log2_ff on two arguments (both positive normal floats, or the lane's result is ignored)
__device__ __forceinline__ void kf2_log2_ff(f2 x, f2* zh, f2* zl) {
    const int32_t ix0 = __float_as_int(x.x), ix1 = __float_as_int(x.y);
    const int32_t t0 = ix0 - 0x3f3504f3, t1 = ix1 - 0x3f3504f3;
    const int32_t e0 = t0 >> 23, e1 = t1 >> 23;
    const int32_t j0 = (t0 >> 17) & 63, j1 = (t1 >> 17) & 63;
    const f2 m = make_float2(__int_as_float(ix0 - e0 * 0x00800000), __int_as_float(ix1 - e1 * 0x00800000));
    // one 128-bit load per lane fetches the whole table row (inv, thi, tlo, pad)
    const float4 row0 = __ldg(reinterpret_cast<const float4*>(&kf_log2_tab[j0][0]));
    const float4 row1 = __ldg(reinterpret_cast<const float4*>(&kf_log2_tab[j1][0]));
    const f2 inv = make_float2(row0.x, row1.x), thi = make_float2(row0.y, row1.y), tlo = make_float2(row0.z, row1.z);
    const f2 p = mul2(m, inv);
    const f2 rl = fma2(m, inv, neg2(p));
    const f2 rh = sub2(p, F2(1.0f));
    f2 q = fma2(rh, F2(-1.6666666666666666e-1f), F2(0.2f));
    q = fma2(rh, q, F2(-0.25f));
    q = fma2(rh, q, F2(3.3333333333333331e-1f));
    q = fma2(rh, q, F2(-0.5f));
    const f2 w = fma2(mul2(rh, rh), q, fma2(neg2(rh), rl, rl));
    const f2 C_HI = F2(1.44269502162933349609375f), C_LO = F2(1.9259629911266175e-8f);
    const f2 mh = mul2(rh, C_HI);
    const f2 ml = fma2(rh, C_HI, neg2(mh));
    const f2 low = add2(add2(ml, tlo), fma2(w, C_HI, mul2(rh, C_LO)));
    const f2 ef = make_float2(__int_as_float(KF_MAGIC_BITS + e0) - KF_MAGIC, __int_as_float(KF_MAGIC_BITS + e1) - KF_MAGIC);
    const f2 a = add2(ef, thi);
    const f2 s = add2(a, mh);
    const f2 se = add2(sub2(a, s), mh);
    *zh = s; *zl = add2(se, low);
}

// kf_pow on two argument pairs.  ok0 / ok1: the lane is inside the fast domain (positive normal base,
// |y * log2 x| < 125); the caller handles y == 0 and the other lanes through the double path.
__device__ __forceinline__ f2 kf2_pow(f2 x, f2 y, bool* ok0, bool* ok1) {
    const int32_t ix0 = __float_as_int(x.x), ix1 = __float_as_int(x.y);
    f2 zh, zl;
    kf2_log2_ff(x, &zh, &zl);
    const f2 ph = mul2(zh, y);
    *ok0 = (ix0 >= 0x00800000 && ix0 < 0x7f800000) && (fabsf(ph.x) < 125.0f);
    *ok1 = (ix1 >= 0x00800000 && ix1 < 0x7f800000) && (fabsf(ph.y) < 125.0f);
    const f2 pl = add2(fma2(zh, y, neg2(ph)), mul2(zl, y));
    const f2 v = add2(ph, F2(KF_MAGIC));
    const f2 n = sub2(v, F2(KF_MAGIC));
    const f2 rh = sub2(ph, n);
    const f2 LN2_HI = F2(0.693147182464599609375f), LN2_LO = F2(-1.904654323148236017e-9f);
    const f2 th = mul2(rh, LN2_HI);
    const f2 tl = add2(fma2(rh, LN2_HI, neg2(th)), add2(mul2(rh, LN2_LO), mul2(pl, LN2_HI)));
    const f2 r = add2(th, tl);
    const f2 bb = sub2(r, th);
    const f2 rl = add2(sub2(th, sub2(r, bb)), sub2(tl, bb));
    return mul2(kf2_exp_core(r, rl), kf2_pow2_from_magic(v));
}

}  // namespace ktc
