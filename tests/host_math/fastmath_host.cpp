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
// exp (fn = 0) or sigmoid (fn = 1), against the double libm narrowed as kten-jvm narrows it
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

}  // extern "C"
