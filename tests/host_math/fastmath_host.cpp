// Host build of kten_b200/csrc/ktc_fastmath_d.h for accuracy checks on a CPU (test
// infrastructure).  The header uses only IEEE float / double add, mul, fma, the
// conversions between them and integer operations, so what is measured here is bit
// for bit what the GPU computes.
#include <cmath>
#include <cstdint>
#include <cstring>
#include "../../kten_b200/csrc/ktc_fastmath_d.h"

static inline int64_t ord(float f) { int32_t i; std::memcpy(&i, &f, 4); return i < 0 ? -(int64_t)(i & 0x7fffffff) : i; }

extern "C" {

void kfh_exp(const float* x, float* out, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = ktc::kd_expf(x[i]);
}

void kfh_sigmoid(const float* x, float* out, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = ktc::kd_sigmoid(x[i]);
}

// out[i] = x[i] ^ y[i] where the routine accepts the pair (ok[i] = 1)
void kfh_pow(const float* x, const float* y, float* out, unsigned char* ok, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) { bool k; out[i] = ktc::kd_pow(x[i], y[i], &k); ok[i] = k ? 1 : 0; }
}

// Every `stride`-th float bit pattern (all of them: both signs, subnormals, infinities, NaNs) through
// exp (fn = 0) or sigmoid (fn = 1; fn = 2: its form for |x| <= 80 against the full form; fn = 3: likewise exp for |x| <= 104), against the double libm narrowed as kten-jvm narrows it
// (JVMRawTensor.kt:395, 399).  counts[k] = inputs at ulp distance k (3 = ">= 3"); a NaN on one side only
// counts as ">= 3".  Returns the largest distance.
int64_t kfh_sweep(int fn, uint32_t stride, int64_t* counts) {
    int64_t worst = 0, c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    const int64_t steps = (1LL << 32) / stride;
    #pragma omp parallel for schedule(static) reduction(max:worst) reduction(+:c0,c1,c2,c3)
    for (int64_t k = 0; k < steps; ++k) {
        const uint32_t b = (uint32_t)(k * stride);
        float x; std::memcpy(&x, &b, 4);
        float got, want;
        if (fn == 0) { got = ktc::kd_expf(x); want = (float)std::exp((double)x); }
        else if (fn == 3) {                          // exp without clamps against the full form, inside its range (NaN included)
            if (x == x && !(std::fabs(x) <= KD_EXP_PLAIN_RANGE)) continue;
            got = ktc::kd_expf_in_range(x); want = ktc::kd_expf(x);
        }
        else if (fn == 2) {                          // the form without clamps against the full one, inside its range (NaN included)
            if (x == x && !(std::fabs(x) <= KD_SIGMOID_PLAIN_RANGE)) continue;
            got = ktc::kd_sigmoid_in_range(x); want = ktc::kd_sigmoid(x);
        }
        else { got = ktc::kd_sigmoid(x); const float e = (float)std::exp((double)(-1.0f * x)); want = 1.0f / (1.0f + e); }
        int64_t d;
        if (want != want || got != got) d = (want != want && got != got) ? 0 : 99;
        else { d = ord(got) - ord(want); if (d < 0) d = -d; }
        if (d > worst) worst = d;
        if (d == 0) ++c0; else if (d == 1) ++c1; else if (d == 2) ++c2; else ++c3;
    }
    counts[0] = c0; counts[1] = c1; counts[2] = c2; counts[3] = c3;
    return worst;
}

// x / b through the reciprocal of a shared divisor (kd_div_by_reciprocal) against the IEEE quotient.
// mode 0: for `n` divisors (the first 64 with the mantissas nearest to all-ones and to 1.0, the rest seeded) every one of
// the 2^23 dividend mantissas, which covers the divisor completely: the algorithm is invariant under scaling by powers
// of two inside its window.  mode 1: n seeded pairs whose exponents span the whole window of both operands, signs mixed.
// Returns the number of quotients that differ in any bit.
int64_t kfh_div(int mode, int64_t n) {
    int64_t bad = 0;
    if (mode == 0) {
        #pragma omp parallel for schedule(dynamic) reduction(+:bad)
        for (int64_t k = 0; k < n; ++k) {
            uint64_t s = 4242 + (uint64_t)k * 0x9E3779B97F4A7C15ull;
            s ^= s >> 29; s *= 0xBF58476D1CE4E5B9ull; s ^= s >> 32;
            uint32_t m = (uint32_t)(s & 0x7fffff);
            if (k < 32) m = 0x7fffff - (uint32_t)k; else if (k < 64) m = (uint32_t)(k - 32);
            const uint32_t bb = m | (127u << 23);
            float b; std::memcpy(&b, &bb, 4);
            const float r = ktc::kd_row_reciprocal(b);
            for (uint32_t xm = 0; xm < (1u << 23); ++xm) {
                const uint32_t xb = xm | (127u << 23);
                float x; std::memcpy(&x, &xb, 4);
                const float got = ktc::kd_div_by_reciprocal(x, b, r), want = x / b;
                if (std::memcmp(&got, &want, 4) != 0) ++bad;
            }
        }
    } else {
        #pragma omp parallel for schedule(static) reduction(+:bad)
        for (int64_t i = 0; i < n; ++i) {
            uint64_t z = 77 + (uint64_t)i * 0x9E3779B97F4A7C15ull;
            z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
            uint64_t w = z * 0xD6E8FEB86659FD93ull; w ^= w >> 32;
            const uint32_t xb = (uint32_t)(z & 0x807fffffu) | ((uint32_t)(64 + (z >> 40) % 128) << 23);     // the whole dividend window
            const uint32_t bb = (uint32_t)(w & 0x807fffffu) | ((uint32_t)(67 + (w >> 40) % 120) << 23);     // 2^-60 .. 2^60 (exclusive)
            float x, b; std::memcpy(&x, &xb, 4); std::memcpy(&b, &bb, 4);
            const float r = ktc::kd_row_reciprocal(b);
            if (r == 0.0f || ktc::kd_div_window(x) == 0u) { ++bad; continue; }     // both are inside by construction
            const float got = ktc::kd_div_by_reciprocal(x, b, r), want = x / b;
            if (std::memcmp(&got, &want, 4) != 0) ++bad;
        }
    }
    return bad;
}

// Division by a power of two as a multiplication by its reciprocal: every divisor kd_is_pow2_divisor accepts against n seeded
// dividends over ALL bit patterns (zeros, subnormals, infinities, NaN included) plus the edges; returns the mismatches.
// NaN results count as equal when both are NaN.
int64_t kfh_div_pow2(int64_t n) {
    int64_t bad = 0;
    for (int e = -62; e <= 62; ++e) {
        for (int sign = 0; sign < 2; ++sign) {
            const float b = std::ldexp(sign ? -1.0f : 1.0f, e);
            const bool ok = ktc::kd_is_pow2_divisor(b);
            if (ok != (e >= -60 && e <= 60)) { ++bad; continue; }
            if (!ok) continue;
            const float r = ktc::kd_row_reciprocal(b);
            #pragma omp parallel for schedule(static) reduction(+:bad)
            for (int64_t i = 0; i < n; ++i) {
                uint64_t z = 99 + (uint64_t)(i + 1) * 0x9E3779B97F4A7C15ull + (uint64_t)(e + 100) * 0xD6E8FEB86659FD93ull;
                z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
                uint32_t xb = (uint32_t)z;
                if (i < 8) { const uint32_t edge[8] = {0u, 0x80000000u, 1u, 0x007fffffu, 0x00800000u, 0x7f7fffffu, 0x7f800000u, 0x7fc00000u}; xb = edge[i]; }
                float x; std::memcpy(&x, &xb, 4);
                const float got = x * r, want = x / b;
                if (got != got && want != want) continue;
                if (std::memcmp(&got, &want, 4) != 0) ++bad;
            }
        }
    }
    const float no[6] = {3.0f, 0.75f, 0.0f, 1.5f, 0x1p61f, 0x1p-61f};
    for (float b : no) if (ktc::kd_is_pow2_divisor(b)) ++bad;
    float inf = INFINITY, nan = NAN;
    if (ktc::kd_is_pow2_divisor(inf) || ktc::kd_is_pow2_divisor(nan)) ++bad;
    return bad;
}

// 1 where the fast form may be used for this pair (what the kernel tests), else 0
int kfh_div_accepts(float x, float b) { return (ktc::kd_row_reciprocal(b) != 0.0f && ktc::kd_div_window(x) != 0u) ? 1 : 0; }

}  // extern "C"
