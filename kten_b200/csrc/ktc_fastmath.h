// ktc_fastmath.h -- exp and pow in float arithmetic only, accurate to well under
// one ulp, written so that the SAME source compiles for the device (nvcc,
// -fmad=false) and for the host (g++, -ffp-contract=off).  Only IEEE-754
// binary32 + - * / fma, integer operations and bit casts are used, so host and
// device produce identical bits and the accuracy can be verified exhaustively on
// a CPU against a double-precision libm.
//
// Why not double: kten-jvm evaluates Math.exp / Math.pow on the widened double
// and narrows once (JVMRawTensor.kt:138-140, 395, 399), i.e. it returns the
// correctly rounded float in all but rare ties.  Doing the same on the GPU costs
// 4-5x the HBM time of the kernel (FP64 issue rate); CUDA's expf/powf are fast
// but documented at 2 and 4 ulp.  Float-float ("double-single") arithmetic on
// the critical terms keeps the error at about 0.5-0.6 ulp at float speed.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define KF_FN __host__ __device__ __forceinline__
#else
#include <math.h>
#define KF_FN static inline
#endif

#if defined(__CUDACC__)
#define KF_TABLE static __device__ const
#else
#define KF_TABLE static const
#endif
#if defined(__CUDACC__)
#define KF_ALIGN16 __align__(16)
#else
#define KF_ALIGN16 __attribute__((aligned(16)))
#endif
#if defined(__CUDA_ARCH__)
#define KF_TAB(t, j, c) __ldg(&(t)[j][c])
#else
#define KF_TAB(t, j, c) ((t)[j][c])
#endif

#if defined(__CUDA_ARCH__)
#define KF_RCP(x) __frcp_rn(x)
#define KF_F2I(x) __float_as_int(x)
#define KF_I2F(x) __int_as_float(x)
#else
#define KF_RCP(x) (1.0f / (x))
KF_FN int32_t kf_f2i(float f) { int32_t i; memcpy(&i, &f, 4); return i; }
KF_FN float kf_i2f(int32_t i) { float f; memcpy(&f, &i, 4); return f; }
#define KF_F2I(x) kf_f2i(x)
#define KF_I2F(x) kf_i2f(x)
#endif

namespace ktc {

// exp(rh + rl) for |rh| <= ~0.36, |rl| << |rh|: 1 + rh + t, with t = the tail of
// the Taylor series plus rl*(1+rh), summed so that a single rounding of half an
// ulp dominates the error.
KF_FN float kf_exp_core(float r, float rl) {
    // q(r) = sum_{k=2..9} r^(k-2) / k!
    float q = 2.7557319223985893e-6f;
    q = fmaf(q, r, 2.4801587301587302e-5f);
    q = fmaf(q, r, 1.9841269841269841e-4f);
    q = fmaf(q, r, 1.3888888888888889e-3f);
    q = fmaf(q, r, 8.3333333333333333e-3f);
    q = fmaf(q, r, 4.1666666666666664e-2f);
    q = fmaf(q, r, 1.6666666666666666e-1f);
    q = fmaf(q, r, 0.5f);
    const float t = fmaf(r * r, q, fmaf(r, rl, rl));
    const float hi = 1.0f + r;
    const float err = (1.0f - hi) + r;            // exact (|1| >= |r|)
    return hi + (err + t);
}

// Round-to-integer without the (slow) conversion instructions: adding 1.5 * 2^23
// leaves the nearest integer in the low mantissa bits; the same bits, shifted
// into the exponent field, build 2^n.
#define KF_MAGIC 12582912.0f            /* 0x4B400000 */
#define KF_MAGIC_BITS 0x4B400000

// 2^n (-126 <= n <= 127) from the bits of (n + KF_MAGIC)
KF_FN float kf_pow2_from_magic(float v_plus_magic) {
    return KF_I2F((int32_t)((uint32_t)KF_F2I(v_plus_magic) << 23) + 0x3f800000);
}

// exp(x), fast path for |x| <= 87 (result normal); returns false when the
// caller must use the double-precision path (huge / tiny / NaN arguments).
// Error below 1 ulp (about 1 % of the results are one ulp off the correctly
// rounded value).
KF_FN bool kf_exp(float x, float* out) {
    if (!(fabsf(x) <= 87.0f)) return false;
    const float v = fmaf(x, 1.44269504088896341f, KF_MAGIC);
    const float n = v - KF_MAGIC;                       // nearest integer to x * log2(e)
    const float LN2_HI = 0.693145751953125f;            // 0x1.62e400p-1: 13 significant bits, n*LN2_HI is exact
    const float LN2_LO = 1.42860682030941723212e-6f;    // ln2 - LN2_HI
    const float rh = fmaf(n, -LN2_HI, x);               // exact
    const float nl = n * LN2_LO;
    const float r = rh - nl;
    const float rl = (rh - r) - nl;                     // rounding error of the subtraction (both are tiny when |rh| < |nl|)
    *out = kf_exp_core(r, rl) * kf_pow2_from_magic(v);
    return true;
}

// 2^(j/64), j = 0..63, as high + low floats
KF_TABLE KF_ALIGN16 float kf_exp2_tab[64][2] = {   /* rows are read with one 64-bit load by the packed variant */
    {1.000000000e+00f, 0.000000000e+00f},
    {1.010889292e+00f, -5.711605411e-09f},
    {1.021897197e+00f, -4.811559862e-08f},
    {1.033024907e+00f, -2.809089317e-08f},
    {1.044273734e+00f, 4.833470157e-08f},
    {1.055645227e+00f, -4.907169426e-08f},
    {1.067140460e+00f, -5.933751979e-08f},
    {1.078760743e+00f, 5.461594554e-08f},
    {1.090507746e+00f, -1.307753994e-08f},
    {1.102382541e+00f, 4.260501996e-08f},
    {1.114386797e+00f, -5.435540018e-08f},
    {1.126521587e+00f, 3.123641434e-08f},
    {1.138788581e+00f, 5.386222313e-08f},
    {1.151189208e+00f, 2.192228266e-08f},
    {1.163724899e+00f, -4.051441493e-08f},
    {1.176396966e+00f, 2.566975077e-08f},
    {1.189207077e+00f, 3.797635273e-08f},
    {1.202156782e+00f, -5.069756526e-08f},
    {1.215247393e+00f, -3.267394888e-08f},
    {1.228480577e+00f, -4.136200360e-08f},
    {1.241857767e+00f, 4.496838102e-08f},
    {1.255380750e+00f, 7.322237483e-09f},
    {1.269050956e+00f, 1.419333318e-09f},
    {1.282870054e+00f, -3.816621685e-08f},
    {1.296839595e+00f, -4.018999533e-08f},
    {1.310961246e+00f, -3.496571566e-08f},
    {1.325236678e+00f, -3.496373324e-08f},
    {1.339667559e+00f, -3.461673970e-08f},
    {1.354255557e+00f, -1.012334927e-08f},
    {1.369002461e+00f, -3.845881835e-08f},
    {1.383909941e+00f, -5.875577358e-08f},
    {1.398979664e+00f, 8.689434061e-09f},
    {1.414213538e+00f, 2.420323497e-08f},
    {1.429613352e+00f, -1.342992917e-08f},
    {1.445180774e+00f, 3.324199938e-08f},
    {1.460917830e+00f, -3.628657552e-08f},
    {1.476826191e+00f, -4.500898854e-08f},
    {1.492907763e+00f, -3.423620143e-08f},
    {1.509164453e+00f, -2.495937323e-08f},
    {1.525598168e+00f, -1.762856883e-08f},
    {1.542210817e+00f, 8.070904833e-09f},
    {1.559004426e+00f, -2.576466507e-08f},
    {1.575980902e+00f, -5.661025426e-08f},
    {1.593142152e+00f, -4.903136785e-10f},
    {1.610490322e+00f, 9.836217174e-09f},
    {1.628027439e+00f, -1.726008314e-08f},
    {1.645755529e+00f, -5.124972091e-08f},
    {1.663676620e+00f, -3.920298752e-08f},
    {1.681792855e+00f, -2.475532668e-08f},
    {1.700106382e+00f, -2.865147231e-08f},
    {1.718619347e+00f, -4.849617596e-08f},
    {1.737333894e+00f, -5.850223417e-08f},
    {1.756252170e+00f, -9.235770371e-09f},
    {1.775376439e+00f, 5.343197884e-08f},
    {1.794709086e+00f, -1.141504491e-08f},
    {1.814252138e+00f, 3.736258236e-08f},
    {1.834008098e+00f, -1.123927795e-08f},
    {1.853979111e+00f, 1.436561181e-08f},
    {1.874167681e+00f, -4.663005626e-08f},
    {1.894575953e+00f, 2.810338451e-08f},
    {1.915206552e+00f, 9.845328108e-09f},
    {1.936061740e+00f, 5.357072297e-08f},
    {1.957144141e+00f, -1.702180441e-08f},
    {1.978456020e+00f, 6.032726318e-09f}
};

// exp(x), correctly rounded, for |x| <= 87; declines (returns false) about once in
// 2000 arguments, when its internal result is too close to a rounding boundary.
// x = k * ln2/64 + r with |r| <= ln2/128, exp(x) = 2^(k >> 6) * T[k & 63] * exp(r).
// Because |r| < 2^-7, every term that is only known to float accuracy is below
// 2^-13 of the result, i.e. its rounding error is below 2^-37; the terms that
// are larger (T, T*r) are carried as exact float pairs.  Used where the exp
// feeds further IEEE operations whose result must match the reference bit for
// bit (sigmoid), so that a one-ulp slip here is not amplified downstream.
KF_FN bool kf_exp_cr(float x, float* out) {
    if (!(fabsf(x) <= 87.0f)) return false;
    const float v = fmaf(x, 92.33248138427734f, KF_MAGIC);          // 64 / ln2
    const float kf = v - KF_MAGIC;
    const int32_t k = KF_F2I(v) - KF_MAGIC_BITS;                    // the same integer, exactly
    const float C1 = 0.0108184814453125f;                           // ln2/64 = C1 + C2 + C3; C1 has 10 significant bits
    const float C2 = 1.1943250683543738e-05f;
    const float C3 = 2.5310171168115014e-13f;
    const float r1 = fmaf(kf, -C1, x);                              // exact
    const float p2 = kf * C2;
    const float p2e = fmaf(kf, C2, -p2);                            // kf*C2 = p2 + p2e exactly
    const float r = r1 - p2;
    const float bb = r - r1;
    const float e1 = (r1 - (r - bb)) + (-p2 - bb);                  // two-sum: r1 - p2 = r + e1 exactly
    const float rl = fmaf(kf, -C3, e1 - p2e);
    const int32_t j = k & 63;
    const float th = KF_TAB(kf_exp2_tab, j, 0), tl = KF_TAB(kf_exp2_tab, j, 1);
    // e = exp(r) - 1 - r  (+ rl): |e| < 2^-14
    float q = fmaf(r, 4.1666666666666664e-2f, 1.6666666666666666e-1f);
    q = fmaf(r, q, 0.5f);
    const float e = fmaf(r * r, q, fmaf(r, rl, rl));          // exp(r + rl) - 1 - r, to first order in rl
    // T * (1 + r + e) = th + th*r + [tl*(1 + r) + th*e]
    const float m = th * r;
    const float me = fmaf(th, r, -m);                               // exact product error
    const float s = th + m;
    const float se = (th - s) + m;                                  // exact (|th| >= |m|)
    const float low = (se + me) + fmaf(th, e, fmaf(tl, r, tl));
    const float res = s + low;
    // Rounding test: s + low is within 2^-14 ulp of exp(x) (largest deviation seen over
    // 4e8 arguments: 4.8e-5 ulp).  If it lies within 2^-12 ulp of the midpoint between two
    // floats the rounding could go either way -- decline and let the caller use double.
    const float rho = (s - res) + low;                              // exact (|s| >= |low|)
    const float u = KF_I2F((KF_F2I(res) & 0x7f800000) - (23 << 23));   // ulp(res)
    if (fabsf(fabsf(rho) - 0.5f * u) < u * 2.44140625e-4f) return false;
    // scale by 2^(k >> 6)
    *out = res * KF_I2F(((k >> 6) + 127) << 23);
    return true;
}

// For the 64 equal slices (in bit-pattern space) of [sqrt(1/2), sqrt(2)): a float
// approximation inv of 1/centre, and -log2(inv) split into a part with 16 fractional
// bits (so that adding the exponent is exact) and a remainder.  The slice that contains
// 1.0 has inv = 1 and log 0, which keeps full relative accuracy for arguments near 1.
KF_TABLE KF_ALIGN16 float kf_log2_tab[64][4] = {   /* rows are read with one 128-bit load by the packed variant */
    {1.406444073e+00f, -4.920501709e-01f, -2.014097618e-06f, 0.0f},
    {1.391158223e+00f, -4.762878418e-01f, 1.327901259e-06f, 0.0f},
    {1.376201153e+00f, -4.606933594e-01f, 2.002024303e-06f, 0.0f},
    {1.361562133e+00f, -4.452667236e-01f, 3.904535788e-06f, 0.0f},
    {1.347231388e+00f, -4.299926758e-01f, -4.980352514e-06f, 0.0f},
    {1.333199143e+00f, -4.148864746e-01f, -5.821009381e-06f, 0.0f},
    {1.319456220e+00f, -3.999481201e-01f, 4.638121482e-06f, 0.0f},
    {1.305993676e+00f, -3.851470947e-01f, -8.164320775e-07f, 0.0f},
    {1.292803168e+00f, -3.704986572e-01f, -3.981619557e-06f, 0.0f},
    {1.279876351e+00f, -3.560028076e-01f, -1.630810061e-06f, 0.0f},
    {1.267205477e+00f, -3.416442871e-01f, -6.188647149e-06f, 0.0f},
    {1.254783034e+00f, -3.274383545e-01f, 4.264629183e-07f, 0.0f},
    {1.242601871e+00f, -3.133697510e-01f, 5.618730484e-06f, 0.0f},
    {1.230654836e+00f, -2.994232178e-01f, -2.965130307e-06f, 0.0f},
    {1.218935490e+00f, -2.856292725e-01f, 7.496968919e-06f, 0.0f},
    {1.207437158e+00f, -2.719421387e-01f, -5.965723631e-06f, 0.0f},
    {1.196153641e+00f, -2.584075928e-01f, 4.883414931e-06f, 0.0f},
    {1.185079217e+00f, -2.449798584e-01f, -3.641308467e-06f, 0.0f},
    {1.174207807e+00f, -2.316894531e-01f, 1.699700533e-06f, 0.0f},
    {1.163534164e+00f, -2.185211182e-01f, 7.545471362e-06f, 0.0f},
    {1.153052807e+00f, -2.054595947e-01f, 1.008499908e-06f, 0.0f},
    {1.142758608e+00f, -1.925201416e-01f, -5.445261309e-07f, 0.0f},
    {1.132646561e+00f, -1.797027588e-01f, 5.016535397e-06f, 0.0f},
    {1.122711897e+00f, -1.669921875e-01f, 4.427387921e-06f, 0.0f},
    {1.112949967e+00f, -1.543884277e-01f, -3.101126822e-07f, 0.0f},
    {1.103356361e+00f, -1.418914795e-01f, -7.347497558e-06f, 0.0f},
    {1.093926787e+00f, -1.295166016e-01f, 4.146417325e-07f, 0.0f},
    {1.084656954e+00f, -1.172332764e-01f, -5.554975814e-06f, 0.0f},
    {1.075542927e+00f, -1.050720215e-01f, 6.915106496e-06f, 0.0f},
    {1.066580772e+00f, -9.298706055e-02f, -6.164886145e-06f, 0.0f},
    {1.057766795e+00f, -8.102416992e-02f, 2.577019586e-06f, 0.0f},
    {1.049097180e+00f, -6.915283203e-02f, 4.507653557e-06f, 0.0f},
    {1.040568709e+00f, -5.737304688e-02f, 8.166411476e-07f, 0.0f},
    {1.032177687e+00f, -4.568481445e-02f, -6.533868600e-06f, 0.0f},
    {1.023920894e+00f, -3.410339355e-02f, -8.660022104e-07f, 0.0f},
    {1.015795112e+00f, -2.261352539e-02f, 4.089034974e-06f, 0.0f},
    {1.007797360e+00f, -1.119995117e-02f, -5.631608019e-06f, 0.0f},
    {1.000000000e+00f, 0.000000000e+00f, 0.000000000e+00f, 0.0f},
    {9.844690561e-01f, 2.258300781e-02f, -7.729166782e-07f, 0.0f},
    {9.695550203e-01f, 4.460144043e-02f, 3.883708359e-06f, 0.0f},
    {9.550861120e-01f, 6.629943848e-02f, -2.158190000e-06f, 0.0f},
    {9.410427213e-01f, 8.766174316e-02f, 6.132098406e-06f, 0.0f},
    {9.274063706e-01f, 1.087188721e-01f, 7.585754247e-06f, 0.0f},
    {9.141595364e-01f, 1.294860840e-01f, -3.951134204e-06f, 0.0f},
    {9.012857676e-01f, 1.499481201e-01f, -4.634119250e-06f, 0.0f},
    {8.887696266e-01f, 1.701202393e-01f, -1.658355359e-06f, 0.0f},
    {8.765962720e-01f, 1.900177002e-01f, -2.148657813e-06f, 0.0f},
    {8.647519350e-01f, 2.096405029e-01f, 1.255120992e-06f, 0.0f},
    {8.532233834e-01f, 2.290039062e-01f, 6.839393905e-07f, 0.0f},
    {8.419982195e-01f, 2.481079102e-01f, 3.002194262e-06f, 0.0f},
    {8.310645223e-01f, 2.669677734e-01f, -1.679887731e-07f, 0.0f},
    {8.204112053e-01f, 2.855834961e-01f, -2.597690809e-06f, 0.0f},
    {8.100274801e-01f, 3.039550781e-01f, 2.164606940e-06f, 0.0f},
    {7.999033928e-01f, 3.220977783e-01f, 4.545512638e-06f, 0.0f},
    {7.900292277e-01f, 3.400268555e-01f, -4.788461410e-06f, 0.0f},
    {7.803958654e-01f, 3.577270508e-01f, -5.090421382e-06f, 0.0f},
    {7.709946036e-01f, 3.752136230e-01f, -6.290585134e-06f, 0.0f},
    {7.618171573e-01f, 3.924865723e-01f, -3.257308208e-06f, 0.0f},
    {7.528555989e-01f, 4.095611572e-01f, -6.238404694e-06f, 0.0f},
    {7.441024184e-01f, 4.264221191e-01f, 4.767879545e-06f, 0.0f},
    {7.355504632e-01f, 4.430999756e-01f, 3.796841838e-06f, 0.0f},
    {7.271928787e-01f, 4.595947266e-01f, -4.703207651e-06f, 0.0f},
    {7.190230489e-01f, 4.758911133e-01f, -1.036580898e-06f, 0.0f},
    {7.110347748e-01f, 4.920043945e-01f, 3.580488737e-06f, 0.0f}
};

// log2(x) = zh + zl for a positive normal float x; error about 2^-38 absolute, and
// about 2^-33 relative when x is close to 1.  x = 2^e * m, m in [sqrt(1/2), sqrt(2));
// r = m * inv - 1 is formed exactly as a float pair (|r| < 2^-6.9), ln(1 + r) needs
// only a short polynomial, and everything larger than 2^-14 is carried exactly.
KF_FN void kf_log2_ff(float x, float* zh, float* zl) {
    const int32_t ix = KF_F2I(x);
    const int32_t t = ix - 0x3f3504f3;
    const int32_t e = t >> 23;
    const int32_t j = (t >> 17) & 63;
    const float m = KF_I2F(ix - e * 0x00800000);
    const float inv = KF_TAB(kf_log2_tab, j, 0), thi = KF_TAB(kf_log2_tab, j, 1), tlo = KF_TAB(kf_log2_tab, j, 2);
    const float p = m * inv;
    const float rl = fmaf(m, inv, -p);                  // exact product error
    const float rh = p - 1.0f;                          // exact
    // ln(1 + rh + rl) - rh = rl * (1 - rh) + rh^2 * (-1/2 + rh/3 - rh^2/4 + rh^3/5 - rh^4/6)
    float q = fmaf(rh, -1.6666666666666666e-1f, 0.2f);
    q = fmaf(rh, q, -0.25f);
    q = fmaf(rh, q, 3.3333333333333331e-1f);
    q = fmaf(rh, q, -0.5f);
    const float w = fmaf(rh * rh, q, fmaf(-rh, rl, rl));
    // times log2(e) = C_HI + C_LO
    const float C_HI = 1.44269502162933349609375f, C_LO = 1.9259629911266175e-8f;
    const float mh = rh * C_HI;
    const float ml = fmaf(rh, C_HI, -mh);               // exact
    const float low = (ml + tlo) + fmaf(w, C_HI, rh * C_LO);
    // exponent + table value (exact), then the head of the product
    const float a = (KF_I2F(KF_MAGIC_BITS + e) - KF_MAGIC) + thi;
    const float s = a + mh;
    const float se = (a - s) + mh;                      // exact: |a| >= |mh|, or a == 0
    *zh = s; *zl = se + low;
}

// x^y, fast path for positive normal x, finite y, result comfortably inside the
// normal range; returns false when the caller must take the double path
// (zero / negative / subnormal / infinite / NaN base, non-finite exponent,
// results near overflow or underflow).  y == 0 must be handled by the caller.
KF_FN bool kf_pow(float x, float y, float* out) {
    const int32_t ix = KF_F2I(x);
    if (!(ix >= 0x00800000 && ix < 0x7f800000)) return false;
    float zh, zl;
    kf_log2_ff(x, &zh, &zl);
    const float ph = zh * y;
    if (!(fabsf(ph) < 125.0f)) return false;            // also rejects NaN / infinite y
    const float pl = fmaf(zh, y, -ph) + zl * y;
    const float v = ph + KF_MAGIC;
    const float n = v - KF_MAGIC;                       // nearest integer to ph
    const float rh = ph - n;                            // exact
    // (rh + pl) * ln2 in float-float
    const float LN2_HI = 0.693147182464599609375f, LN2_LO = -1.904654323148236017e-9f;
    const float th = rh * LN2_HI;
    const float tl = fmaf(rh, LN2_HI, -th) + (rh * LN2_LO + pl * LN2_HI);
    // renormalise so the low part is below half an ulp of the high part (two-sum)
    const float r = th + tl;
    const float bb = r - th;
    const float rl = (th - (r - bb)) + (tl - bb);
    *out = kf_exp_core(r, rl) * kf_pow2_from_magic(v);
    return true;
}

}  // namespace ktc
