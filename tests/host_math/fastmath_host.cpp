// Host build of kten_b200/csrc/ktc_fastmath.h for accuracy checks on a CPU (test
// infrastructure).  The header uses only IEEE float operations, so what is
// measured here is bit for bit what the GPU computes.
#include <cmath>
#include <cstdint>
#include <cstring>
#include "../../kten_b200/csrc/ktc_fastmath.h"

extern "C" {

// out[i] = exp(x[i]); ok[i] = 1 when the fast path took it
void kfh_exp(const float* x, float* out, unsigned char* ok, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) { float r = 0.f; ok[i] = ktc::kf_exp(x[i], &r) ? 1 : 0; out[i] = r; }
}

void kfh_pow(const float* x, const float* y, float* out, unsigned char* ok, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) { float r = 0.f; ok[i] = ktc::kf_pow(x[i], y[i], &r) ? 1 : 0; out[i] = r; }
}

static inline int64_t ord(float f) { int32_t i; std::memcpy(&i, &f, 4); return i < 0 ? -(int64_t)(i & 0x7fffffff) : i; }

// Sweep every `stride`-th float bit pattern in [lo_bits, hi_bits] through kf_exp
// and compare with the narrowed double exp: returns the largest ulp distance,
// counts[k] = number of inputs at distance k (k = 0..3, 3 = ">= 3").
int64_t kfh_exp_sweep(uint32_t lo_bits, uint32_t hi_bits, uint32_t stride, int64_t* counts, int64_t* n_fast) {
    int64_t worst = 0, c0 = 0, c1 = 0, c2 = 0, c3 = 0, nf = 0;
    const int64_t steps = ((int64_t)hi_bits - lo_bits) / stride + 1;
    #pragma omp parallel for schedule(static) reduction(max:worst) reduction(+:c0,c1,c2,c3,nf)
    for (int64_t k = 0; k < steps; ++k) {
        uint32_t b = lo_bits + (uint32_t)(k * stride);
        float x; std::memcpy(&x, &b, 4);
        float r;
        if (!ktc::kf_exp(x, &r)) continue;
        ++nf;
        const float want = (float)std::exp((double)x);
        int64_t d = ord(r) - ord(want); if (d < 0) d = -d;
        if (d > worst) worst = d;
        if (d == 0) ++c0; else if (d == 1) ++c1; else if (d == 2) ++c2; else ++c3;
    }
    counts[0] = c0; counts[1] = c1; counts[2] = c2; counts[3] = c3; *n_fast = nf;
    return worst;
}

}  // extern "C"

extern "C" void kfh_log2(const float* x, float* zh, float* zl, int64_t n) {
    for (int64_t i = 0; i < n; ++i) ktc::kf_log2_ff(x[i], &zh[i], &zl[i]);
}

extern "C" void kfh_exp_cr(const float* x, float* out, unsigned char* ok, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) { float r = 0.f; ok[i] = ktc::kf_exp_cr(x[i], &r) ? 1 : 0; out[i] = r; }
}

// sigmoid exactly as the device functor composes it: e = exp(-1f * x) through the
// accurate path (double exp where that path declines), then 1f / (1f + e)
extern "C" void kfh_sigmoid(const float* x, float* out, int64_t n) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float a = -1.0f * x[i];
        float e;
        if (!ktc::kf_exp_cr(a, &e)) e = (float)std::exp((double)a);
        out[i] = 1.0f / (1.0f + e);
    }
}
