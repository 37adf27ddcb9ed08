/* ktc_datagen.c -- seeded synthetic inputs for tests and benchmarks (host only).
 *
 * The reference cannot seed its random tensors (kten-jvm draws from the global
 * unseeded Random, backend/kten-jvm/.../operations/AbstractJVMTensorOperations.kt:41-61),
 * and names no dataset, so "seed s" is defined here: a counter-based generator,
 * element i of stream t under seed s is a pure function of (s, t, i):
 *
 *   z   = mix(s ^ (t * 0xD1B54A32D192ED03) + (i + 1) * 0x9E3779B97F4A7C15)   (splitmix64 finaliser)
 *   k1  = z >> 40            (24 bits)        u1 = (k1 + 0.5) / 2^24  in (0,1)
 *   k2  = (z >> 16) & 0xFFFFFF                u2 = (k2 + 0.5) / 2^24
 *   uniform(lo,hi) = (float)(lo + (hi - lo) * u1)                       (double arithmetic, one narrowing)
 *   normal(m,sd)   = (float)(m + sd * sqrt(-2 ln u1) * cos(2 pi u2))    (Box-Muller in double)
 *   quantised normal = rint(normal * q) / q   (q = 16 gives multiples of 1/16, so ties occur)
 */
#include <math.h>
#include <stdint.h>

#define KTD_API __attribute__((visibility("default")))

static inline uint64_t ktd_mix(uint64_t seed, uint64_t stream, uint64_t i) {
    uint64_t z = (seed ^ (stream * 0xD1B54A32D192ED03ULL)) + (i + 1) * 0x9E3779B97F4A7C15ULL;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ULL;
    z ^= z >> 27; z *= 0x94D049BB133111EBULL;
    z ^= z >> 31;
    return z;
}

KTD_API void ktd_uniform(float* out, int64_t n, int64_t first, uint64_t seed, uint64_t stream, double lo, double hi) {
    #pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        const uint64_t z = ktd_mix(seed, stream, (uint64_t)(first + j));
        const double u = ((double)(z >> 40) + 0.5) * (1.0 / 16777216.0);
        out[j] = (float)(lo + (hi - lo) * u);
    }
}

KTD_API void ktd_normal(float* out, int64_t n, int64_t first, uint64_t seed, uint64_t stream, double mean, double sd, double quantum) {
    #pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        const uint64_t z = ktd_mix(seed, stream, (uint64_t)(first + j));
        const double u1 = ((double)(z >> 40) + 0.5) * (1.0 / 16777216.0);
        const double u2 = ((double)((z >> 16) & 0xFFFFFFULL) + 0.5) * (1.0 / 16777216.0);
        double v = mean + sd * sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
        if (quantum > 0.0) v = rint(v * quantum) / quantum;
        out[j] = (float)v;
    }
}
