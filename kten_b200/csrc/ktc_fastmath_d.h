// ktc_fastmath_d.h -- exp, sigmoid and pow of float arguments through a short stretch of double
// arithmetic, written so that the SAME source compiles for the device (nvcc / NVRTC) and for the
// host (g++ -ffp-contract=off): only IEEE-754 add / mul / fma in binary64 and binary32, the
// float <-> double conversions, integer operations and bit casts are used, so host and device
// produce identical bits and the accuracy is measured on a CPU against a multi-precision value.
//
// Why double, and why so little of it: kten-jvm evaluates Math.exp / Math.pow on the widened
// double and narrows once (JVMRawTensor.kt:138-140, 395, 399).  A full double libm routine
// costs 4-5x the HBM time of the kernel; float-float arithmetic reaches the correctly rounded
// float only with ~50 instructions per element and a rounding test.  B200 issues a double fma
// at half the float rate, so a table-driven reduction plus a degree-5 polynomial in double
// (9 double operations for exp, 18 for pow) gives a value within 2^-42 of the true one (2^-45
// on average) -- the narrowing then returns the float the double libm's result narrows to
// except for fewer than one argument in a million (measured on the host, bit for bit) -- at
// roughly two thirds of the issue slots of the float-float versions.
//
// Tables are small on purpose: the 16 doubles of 2^(j/16) are one 128-byte line, so a warp's
// lookups are served in one pass of the L1 pipeline; the 64-entry table is used only where one
// double operation less is worth three more passes.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define KD_FN __device__ __forceinline__
#define KD_TABLE static __device__ const
#define KD_ALIGN(n) __align__(n)
#else
#include <math.h>
#define KD_FN static inline
#define KD_TABLE static const
#define KD_ALIGN(n) __attribute__((aligned(n)))
#endif

namespace ktc {

// 2^(j/16), j = 0..15, with the high word lowered by j << 16 (gen_fastmath_d_tables.py): adding k << 16 to the high
// word of entry k & 15 gives 2^(k/16) -- the index bits of k cancel against the bias and k >> 4 lands in the exponent
// field -- with one integer multiply-add instead of a mask, a shift and an add.
KD_TABLE KD_ALIGN(128) double kd_exp2_tab[16] = {
    0x1.0000000000000p+0, 0x1.fb5586cf9890fp-1, 0x1.f72b83c7d517bp-1, 0x1.f387a6e756238p-1,
    0x1.f06fe0a31b715p-1, 0x1.edea64c123422p-1, 0x1.ebfdad5362a27p-1, 0x1.eab07dd485429p-1,
    0x1.ea09e667f3bcdp-1, 0x1.ea11473eb0187p-1, 0x1.eace5422aa0dbp-1, 0x1.ec49182a3f090p-1,
    0x1.ee89f995ad3adp-1, 0x1.f199bdd85529cp-1, 0x1.f5818dcfba487p-1, 0x1.fa4afa2a490dap-1
};

// 2^(j/64), j = 0..63, high word lowered by j << 14: four cache lines.  sigmoid reduces to |z| <= ln2/128 with it, where a degree-4 polynomial
// truncates below 2^-44.5 (kd_exp_wide); exp and pow keep the 16-entry table.
KD_TABLE KD_ALIGN(128) double kd_exp2_tab64[64] = {
    0x1.0000000000000p+0, 0x1.fec9a3e778061p-1, 0x1.fd9b0d3158574p-1, 0x1.fc74518759bc8p-1,
    0x1.fb5586cf9890fp-1, 0x1.fa3ec32d3d1a2p-1, 0x1.f9301d0125b51p-1, 0x1.f829aaea92de0p-1,
    0x1.f72b83c7d517bp-1, 0x1.f635beb6fcb75p-1, 0x1.f54873168b9aap-1, 0x1.f463b88628cd6p-1,
    0x1.f387a6e756238p-1, 0x1.f2b4565e27cddp-1, 0x1.f1e9df51fdee1p-1, 0x1.f1285a6e4030bp-1,
    0x1.f06fe0a31b715p-1, 0x1.efc08b26416ffp-1, 0x1.ef1a7373aa9cbp-1, 0x1.ee7db34e59ff7p-1,
    0x1.edea64c123422p-1, 0x1.ed60a21f72e2ap-1, 0x1.ece086061892dp-1, 0x1.ec6a2b5c13cd0p-1,
    0x1.ebfdad5362a27p-1, 0x1.eb9b2769d2ca7p-1, 0x1.eb42b569d4f82p-1, 0x1.eaf4736b527dap-1,
    0x1.eab07dd485429p-1, 0x1.ea76f15ad2148p-1, 0x1.ea47eb03a5585p-1, 0x1.ea23882552225p-1,
    0x1.ea09e667f3bcdp-1, 0x1.e9fb23c651a2fp-1, 0x1.e9f75e8ec5f74p-1, 0x1.e9feb564267c9p-1,
    0x1.ea11473eb0187p-1, 0x1.ea2f336cf4e62p-1, 0x1.ea589994cce13p-1, 0x1.ea8d99b4492edp-1,
    0x1.eace5422aa0dbp-1, 0x1.eb1ae99157736p-1, 0x1.eb737b0cdc5e5p-1, 0x1.ebd829fde4e50p-1,
    0x1.ec49182a3f090p-1, 0x1.ecc667b5de565p-1, 0x1.ed503b23e255dp-1, 0x1.ede6b5579fdbfp-1,
    0x1.ee89f995ad3adp-1, 0x1.ef3a2b84f15fbp-1, 0x1.eff76f2fb5e47p-1, 0x1.f0c1e904bc1d2p-1,
    0x1.f199bdd85529cp-1, 0x1.f27f12e57d14bp-1, 0x1.f3720dcef9069p-1, 0x1.f472d4a07897cp-1,
    0x1.f5818dcfba487p-1, 0x1.f69e603db3285p-1, 0x1.f7c97337b9b5fp-1, 0x1.f902ee78b3ff6p-1,
    0x1.fa4afa2a490dap-1, 0x1.fba1bee615a27p-1, 0x1.fd0765b6e4540p-1, 0x1.fe7c1819e90d8p-1
};

// For the 32 equal slices (in bit-pattern space) of [sqrt(1/2), sqrt(2)): inv = 1/centre rounded to 13
// significant bits -- stored as the high word of the double, whose low word is zero -- and -log2(inv).
// mantissa * inv - 1 is exact in double and below 2^-6 in magnitude; the slice holding 1.0 has inv = 1 and
// logarithm 0, which keeps the relative accuracy of log2(x) for x near 1.  The two tables are 128 and 256
// bytes: a warp's 32 lookups touch three cache lines (64 rows of 16 bytes made the L1 data pipe the bound
// of pow, 84 % busy).
KD_TABLE KD_ALIGN(128) int32_t kd_log2_inv_hi[32] = {
    0x3ff66100, 0x3ff5e700, 0x3ff57100, 0x3ff50100, 0x3ff49500, 0x3ff42d00, 0x3ff3c900, 0x3ff36900,
    0x3ff30d00, 0x3ff2b400, 0x3ff25e00, 0x3ff20b00, 0x3ff1bb00, 0x3ff16e00, 0x3ff12300, 0x3ff0db00,
    0x3ff09500, 0x3ff05100, 0x3ff00000, 0x3fef4300, 0x3fee5600, 0x3fed7700, 0x3feca400, 0x3febdc00,
    0x3feb1f00, 0x3fea6c00, 0x3fe9c200, 0x3fe92000, 0x3fe88600, 0x3fe7f300, 0x3fe76700, 0x3fe6e100
};
KD_TABLE KD_ALIGN(128) double kd_log2_lc[32] = {
    -0x1.efaf6c3d98561p-2, -0x1.cfe2bb985617dp-2, -0x1.b076a714ac256p-2, -0x1.9202002050725p-2,
    -0x1.740871deb8e15p-2, -0x1.5694f733077e4p-2, -0x1.39b2e9355671ap-2, -0x1.1d6df91c8071fp-2,
    -0x1.01d228cf4071ap-2, -0x1.cd398e83e815fp-3, -0x1.97ac270c8f462p-3, -0x1.630d19b62f7b9p-3,
    -0x1.2f6ddde311e73p-3, -0x1.f9c0b5c56ba69p-4, -0x1.9594f001c4a9ap-4, -0x1.33cb147ba548ep-4,
    -0x1.a649bfe7f2265p-5, -0x1.cedf14019136ep-6, 0x0.0p+0, 0x1.13dd2fde5e190p-5,
    0x1.3b927f71b18e0p-4, 0x1.e7bd967ba24c6p-4, 0x1.47b2c2f8cb155p-3, 0x1.9969e5729c466p-3,
    0x1.e8c4c318315acp-3, 0x1.1af8a01977729p-2, 0x1.409347a934e48p-2, 0x1.6552b49986277p-2,
    0x1.891fe20affb86p-2, 0x1.ac20a720617f0p-2, 0x1.ce40c0591c530p-2, 0x1.efabce08e9f28p-2
};

// Polynomial and reduction constants.  On the device they live in constant memory and are named by
// index, so that every double operation takes its constant straight from the constant bank (written
// as literals, each use costs two extra instructions that build the 64-bit value in registers --
// measured: 15 of 41 instructions per sigmoid).
#define KD_C_16_LN2    0   /* 16 / ln 2 */
#define KD_C_LN2_16    1   /* -(ln 2) / 16 */
#define KD_C_E5        2   /* 1/120 */
#define KD_C_E4        3   /* 1/24 */
#define KD_C_E3        4   /* 1/6 */
#define KD_C_L5        5   /* log2(e) * (-1/6) */
#define KD_C_L4        6   /* log2(e) / 5 */
#define KD_C_L3        7   /* log2(e) * (-1/4) */
#define KD_C_L2        8   /* log2(e) / 3 */
#define KD_C_L1        9   /* log2(e) * (-1/2) */
#define KD_C_L0       10   /* log2(e) */
#define KD_C_P5       11   /* (ln 2)^5 / 120 */
#define KD_C_P4       12   /* (ln 2)^4 / 24 */
#define KD_C_P3       13   /* (ln 2)^3 / 6 */
#define KD_C_P2       14   /* (ln 2)^2 / 2 */
#define KD_C_P1       15   /* ln 2 */
#define KD_C_MAGIC    16   /* 2^52 + 2^51: adding it leaves the nearest integer in the low word */
#define KD_C_64_LN2   17   /* 64 / ln 2 */
#define KD_C_LN2_64   18   /* -(ln 2) / 64 */
#define KD_C_COUNT    19
#define KD_CONST_VALUES { \
    23.083120654223414, -0.043321698784996581, 8.3333333333333332e-3, 4.1666666666666664e-2, 1.6666666666666666e-1, \
    -2.404491734814939e-1, 2.8853900817779266e-1, -3.6067376022224085e-1, 4.808983469629878e-1, -7.213475204444817e-1, \
    1.4426950408889634, 1.3333558146428443e-3, 9.618129107628477e-3, 5.550410866482158e-2, 2.4022650695910072e-1, \
    6.9314718055994531e-1, 6755399441055744.0, 92.332482616893656, -0.010830424696249145 }
#if defined(__CUDACC__)
static __constant__ double kd_consts[KD_C_COUNT] = KD_CONST_VALUES;
#else
static const double kd_consts[KD_C_COUNT] = KD_CONST_VALUES;
#endif
#define KD_K(i) (kd_consts[i])

#if defined(__CUDA_ARCH__)
#define KD_LO32(d) __double2loint(d)
#define KD_HI32(d) __double2hiint(d)
#define KD_MAKE(hi, lo) __hiloint2double(hi, lo)
#define KD_F2I(x) __float_as_int(x)
#define KD_I2F(x) __int_as_float(x)
#define KD_EXP2_TAB(j) __ldg(&kd_exp2_tab[j])
#define KD_EXP2_TAB64(j) __ldg(&kd_exp2_tab64[j])
#else
KD_FN int32_t kd_lo32(double d) { int64_t i; memcpy(&i, &d, 8); return (int32_t)(uint32_t)(uint64_t)i; }
KD_FN int32_t kd_hi32(double d) { int64_t i; memcpy(&i, &d, 8); return (int32_t)((uint64_t)i >> 32); }
KD_FN double kd_make(int32_t hi, int32_t lo) { uint64_t u = ((uint64_t)(uint32_t)hi << 32) | (uint32_t)lo; double d; memcpy(&d, &u, 8); return d; }
KD_FN int32_t kd_f2i(float f) { int32_t i; memcpy(&i, &f, 4); return i; }
KD_FN float kd_i2f(int32_t i) { float f; memcpy(&f, &i, 4); return f; }
#define KD_LO32(d) kd_lo32(d)
#define KD_HI32(d) kd_hi32(d)
#define KD_MAKE(hi, lo) kd_make(hi, lo)
#define KD_F2I(x) kd_f2i(x)
#define KD_I2F(x) kd_i2f(x)
#define KD_EXP2_TAB(j) (kd_exp2_tab[j])
#define KD_EXP2_TAB64(j) (kd_exp2_tab64[j])
#endif

// 2^(k/16) for |k| < 2^14 (the result stays far inside the double range): see the bias of kd_exp2_tab.
KD_FN double kd_scaled_tab(int32_t k) {
    const double t = KD_EXP2_TAB(k & 15);
    return KD_MAKE((int32_t)((uint32_t)KD_HI32(t) + ((uint32_t)k << 16)), KD_LO32(t));
}

// exp(t) for |t| <= 700 with the 16-entry table: t = k ln2/16 + z, |z| <= ln2/32, degree 5; relative error below
// 2^-42 (truncation 2^-42.7 at the edge of the reduced range, 2^-45 on average).  The plain exp kernel is bound by
// memory, and the one cache line of this table leaves the L1 pipe to the data stream.
KD_FN double kd_exp(double t) {
    const double v = fma(t, KD_K(KD_C_16_LN2), KD_K(KD_C_MAGIC));
    const double kd = v - KD_K(KD_C_MAGIC);                            // nearest integer to t * 16 / ln2
    const double z = fma(kd, KD_K(KD_C_LN2_16), t);                    // t - k * ln2/16
    double p = fma(z, KD_K(KD_C_E5), KD_K(KD_C_E4));
    p = fma(p, z, KD_K(KD_C_E3));
    p = fma(p, z, 0.5);
    p = fma(p, z, 1.0);
    p = fma(p, z, 1.0);
    return kd_scaled_tab(KD_LO32(v)) * p;
}

// The same with the 64-entry table: |z| <= ln2/128, degree 4, truncation below 2^-44.5 at the edge.  One double
// operation fewer for three more cache lines per warp lookup: the choice where instruction issue is the bound
// (sigmoid, and the fused training-step kernels built on it: measured 2 % faster, plain exp 3 % slower).
KD_FN double kd_exp_wide(double t) {
    const double v = fma(t, KD_K(KD_C_64_LN2), KD_K(KD_C_MAGIC));
    const double kd = v - KD_K(KD_C_MAGIC);                            // nearest integer to t * 64 / ln2
    const double z = fma(kd, KD_K(KD_C_LN2_64), t);                    // t - k * ln2/64
    double p = fma(z, KD_K(KD_C_E4), KD_K(KD_C_E3));
    p = fma(p, z, 0.5);
    p = fma(p, z, 1.0);
    p = fma(p, z, 1.0);
    const int32_t k = KD_LO32(v);
    const double s = KD_EXP2_TAB64(k & 63);
    return KD_MAKE((int32_t)((uint32_t)KD_HI32(s) + ((uint32_t)k << 14)), KD_LO32(s)) * p;
}

// Math.max / Math.min-style clamps that keep a NaN argument
#if defined(__CUDA_ARCH__)
KD_FN float kd_max_nan(float a, float b) { float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
KD_FN float kd_min_nan(float a, float b) { float r; asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
#else
KD_FN float kd_max_nan(float a, float b) { return (a != a) ? a : (a > b ? a : b); }
KD_FN float kd_min_nan(float a, float b) { return (a != a) ? a : (a < b ? a : b); }
#endif

// 1f / d for 1 <= d < 4e37: the hardware's approximate reciprocal plus one Newton step whose residual is
// exact (fma) is the IEEE quotient for every such d (compared with the IEEE reciprocal for all 2^23 * 125
// of them on the device).  Larger d (subnormal quotients) and infinity need the IEEE routine; a NaN
// passes through either.
#define KD_RCP_FAST_LIMIT 4.0e37f
KD_FN float kd_rcp_fast(float d) {
#if defined(__CUDA_ARCH__)
    float y0;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y0) : "f"(d));
    const float r = fmaf(-d, y0, 1.0f);
    return fmaf(y0, r, y0);
#else
    return 1.0f / d;
#endif
}
KD_FN float kd_rcp_ieee(float d) {
#if defined(__CUDA_ARCH__)
    return __frcp_rn(d);
#else
    return 1.0f / d;
#endif
}

// x / b for a divisor that many dividends share (the b[1,J,1] operand of a broadcast division).  IEEE division costs
// about ten instructions per element; with r = RN(1/b) computed once, q = RN(x r), e = x - q b (exact in one fma) and
// RN(q + e r) is the correctly rounded quotient -- Markstein's theorem for a correctly rounded reciprocal, checked on the
// host for every mantissa of x against thousands of divisors -- in three instructions.  It holds while nothing over- or
// underflows: divisors in [2^-60, 2^60] (kd_row_reciprocal returns 0 for the others) and dividends in [2^-63, 2^64), i.e.
// an exponent field in [64, 192): adding 64 to the field sets its top bit exactly then (a zero dividend would lose its
// sign in the fast form; NaN and infinity are out of the window too).  Everything else takes the IEEE division.
KD_FN float kd_row_reciprocal(float b) {
    const float ab = b < 0.0f ? -b : b;
    return (ab >= 0x1p-60f && ab <= 0x1p60f) ? kd_rcp_ieee(b) : 0.0f;
}
KD_FN uint32_t kd_div_window(float x) { return ((uint32_t)KD_F2I(x) + 0x20000000u) & 0x40000000u; }
KD_FN float kd_div_by_reciprocal(float x, float b, float r) {
    const float q = x * r;
    return fmaf(fmaf(-q, b, x), r, q);
}

// A divisor that is a power of two inside kd_row_reciprocal's range: x / b and x * (1 / b) are then roundings of the same
// real number (the reciprocal is exact), for every x -- zeros keep their sign, subnormal quotients round alike, infinities
// and NaN pass -- so one multiplication is the IEEE quotient and no window test is needed.
KD_FN bool kd_is_pow2_divisor(float b) {
    const uint32_t bits = (uint32_t)KD_F2I(b) & 0x7fffffffu;
    return (bits & 0x007fffffu) == 0u && bits >= (67u << 23) && bits <= (187u << 23);      // 2^-60 .. 2^60
}

// kten-jvm's sigmoid: e = (float)Math.exp((double)(-1f * x)); 1f / (1f + e)   (JVMRawTensor.kt:399).
// x is clamped to [-89, 30] first: beyond 30 the sum 1f + e is 1f exactly, below -88.73 e is +infinity
// (exp(89) narrows to infinity as Math.exp's value does), so the clamp does not change any result.
// kd_sigmoid_den returns the denominator 1f + e; the quotient is kd_rcp_fast where the denominator is
// below KD_RCP_FAST_LIMIT and the IEEE reciprocal otherwise -- the same bits either way where both apply.
KD_FN float kd_sigmoid_den(float x) {
    const float xc = kd_max_nan(kd_min_nan(x, 30.0f), -89.0f);
    const float e = (float)kd_exp_wide(-(double)xc);
    return 1.0f + e;
}
KD_FN float kd_sigmoid(float x) {
    const float d = kd_sigmoid_den(x);
    return (d < KD_RCP_FAST_LIMIT) ? kd_rcp_fast(d) : kd_rcp_ieee(d);
}

// The same value for |x| <= KD_SIGMOID_PLAIN_RANGE (and NaN for NaN) without the two clamps and without the test of
// the denominator: exp(80) < 4e37.  The vector forms test the range once per four elements.
#define KD_SIGMOID_PLAIN_RANGE 80.0f
KD_FN float kd_sigmoid_in_range(float x) {
    return kd_rcp_fast(1.0f + (float)kd_exp_wide(-(double)x));
}

// float exp with Math.exp's narrowing: the argument is clamped to [-104, 89] (exp(-104) narrows to 0,
// exp(89) to +infinity, as the unclamped values do)
KD_FN float kd_expf(float x) {
    const float xc = kd_max_nan(kd_min_nan(x, 89.0f), -104.0f);
    return (float)kd_exp((double)xc);
}
// the same value for |x| <= 104 (and NaN for NaN) without the clamps; the vector forms test the range once per four elements
#define KD_EXP_PLAIN_RANGE 104.0f
KD_FN float kd_expf_in_range(float x) { return (float)kd_exp((double)x); }

// log2 of the float with bit pattern ix (a positive normal float), relative error below 2^-38
KD_FN double kd_log2(int32_t ix) {
    const int32_t t = ix - 0x3f3504f3;
    const int32_t e = t >> 23;
    const int32_t j = (t >> 18) & 31;
    const double m = (double)KD_I2F(ix - (e << 23));                   // [sqrt(1/2), sqrt(2))
#if defined(__CUDA_ARCH__)
    const double inv = KD_MAKE(__ldg(&kd_log2_inv_hi[j]), 0), lc = __ldg(&kd_log2_lc[j]);
#else
    const double inv = KD_MAKE(kd_log2_inv_hi[j], 0), lc = kd_log2_lc[j];
#endif
    const double r = fma(m, inv, -1.0);                                // exact, |r| < 2^-6
    // log2(1 + r) = r * log2(e) * (1 - r/2 + r^2/3 - r^3/4 + r^4/5 - r^5/6); the first dropped term is below
    // 2^-38 of the logarithm, i.e. below 2^-8 ulp of x^y even where |y log2 x| reaches 128
    double q = fma(r, KD_K(KD_C_L5), KD_K(KD_C_L4));
    q = fma(q, r, KD_K(KD_C_L3));
    q = fma(q, r, KD_K(KD_C_L2));
    q = fma(q, r, KD_K(KD_C_L1));
    q = fma(q, r, KD_K(KD_C_L0));
    return fma(q, r, (double)e + lc);
}

// x^y = Math.pow's value narrowed as the JVM narrows it (the double carries results below the float range,
// so subnormal and overflowing results round as (float)Math.pow does).  *ok is true for a positive normal
// x with |y * log2 x| < 160 (y == 0 gives exactly 1, as Math.pow does); for every other argument pair -- zero,
// negative, subnormal, infinite or NaN base, non-finite y, results far outside the float range -- the returned value is
// meaningless (but computing it is harmless) and the caller takes the double-precision routine that holds
// Java's special cases.
KD_FN float kd_pow(float x, float y, bool* ok) {
    const int32_t ix = KD_F2I(x);
    const double p = kd_log2(ix) * (double)y;
    *ok = ((uint32_t)(ix - 0x00800000) < 0x7f000000u) && ((uint32_t)(KD_HI32(p) & 0x7fffffff) < 0x40640000u);
    const double v = fma(p, 16.0, KD_K(KD_C_MAGIC));
    const double kd = v - KD_K(KD_C_MAGIC);
    const double z = fma(kd, -0.0625, p);                             // p - k/16 exactly, |z| <= 1/32
    double s = fma(z, KD_K(KD_C_P5), KD_K(KD_C_P4));                   // 2^z = 1 + z ln2 + (z ln2)^2 / 2 + ...
    s = fma(s, z, KD_K(KD_C_P3));
    s = fma(s, z, KD_K(KD_C_P2));
    s = fma(s, z, KD_K(KD_C_P1));
    s = fma(s, z, 1.0);
    return (float)(kd_scaled_tab(KD_LO32(v)) * s);
}

}  // namespace ktc
