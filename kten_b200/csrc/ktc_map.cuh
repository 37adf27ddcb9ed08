// ktc_map.cuh -- contiguous elementwise maps shared by the elementwise translation units.
//
// HBM-bandwidth kernels: every thread moves 128-bit vectors, issues all the loads of its
// tile before the first use, reads with the streaming hint (ld.global.cs: each element is
// used once) and writes with st.global.cs.
//   map1 : out[i] = f(a[i])          map2 : out[i] = f(a[i], b[i])   (also in place)
#pragma once

#include "ktc_internal.hpp"
#include "ktc_math.cuh"

namespace ktc {

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

template <class F> __device__ __forceinline__ float4 apply1(const F& f, float4 a) {
    return make_float4(f(a.x), f(a.y), f(a.z), f(a.w));
}
template <class F> __device__ __forceinline__ float4 apply2(const F& f, float4 a, float4 b) {
    return make_float4(f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w));
}

// ---- contiguous maps ---------------------------------------------------------
// One tile of kMapThreads * U float4 per CTA, CTAs in address order.  Each thread forms
// its base pointers once; the U accesses are then fixed offsets from them.  n4 is the
// number of whole float4; the (< 4 element) remainder and unaligned buffers go through
// the scalar kernels below.
constexpr int kMapThreads = 256;

template <int U, class F>
__global__ void __launch_bounds__(kMapThreads) k_map1_vec(const float4* a, float4* out, int64_t n4, F f) {     // out may be a (in-place forms): no __restrict__
    const int64_t base = (int64_t)blockIdx.x * (kMapThreads * U) + threadIdx.x;
    const float4* pa = a + base;
    float4* po = out + base;
    if (base - threadIdx.x + kMapThreads * U <= n4) {              // whole tile: every load before the first use, no guards
        float4 va[U];
        #pragma unroll
        for (int u = 0; u < U; ++u) va[u] = ld_stream(pa + u * kMapThreads);
        #pragma unroll
        for (int u = 0; u < U; ++u) st_stream(po + u * kMapThreads, apply1(f, va[u]));
    } else {
        for (int64_t i = base; i < n4; i += kMapThreads) st_stream(out + i, apply1(f, ld_stream(a + i)));
    }
}

// MINB: resident CTAs per SM the register allocation must allow.  pow's double arithmetic wants about 66
// registers, two over the step from 4 to 3 resident CTAs; capped at 64 it runs a tenth faster.
template <class F> struct MapMinBlocks { static constexpr int value = 1; };
template <> struct MapMinBlocks<BinOp<KTC_POW>> { static constexpr int value = 4; };

template <int U, class F>
__global__ void __launch_bounds__(kMapThreads, MapMinBlocks<F>::value) k_map2_vec(const float4* a, const float4* b, float4* out, int64_t n4, F f) {     // out may be a
    const int64_t base = (int64_t)blockIdx.x * (kMapThreads * U) + threadIdx.x;
    const float4* pa = a + base;
    const float4* pb = b + base;
    float4* po = out + base;
    if (base - threadIdx.x + kMapThreads * U <= n4) {
        float4 va[U], vb[U];
        #pragma unroll
        for (int u = 0; u < U; ++u) { va[u] = ld_stream(pa + u * kMapThreads); vb[u] = ld_stream(pb + u * kMapThreads); }
        #pragma unroll
        for (int u = 0; u < U; ++u) st_stream(po + u * kMapThreads, apply2(f, va[u], vb[u]));
    } else {
        for (int64_t i = base; i < n4; i += kMapThreads) st_stream(out + i, apply2(f, ld_stream(a + i), ld_stream(b + i)));
    }
}

// the in-place forms call these with out == a: no __restrict__, no read-only loads
template <class F>
__global__ void k_map1_scalar(const float* a, float* out, int64_t n, F f) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = f(a[i]);
}
template <class F>
__global__ void k_map2_scalar(const float* a, const float* b, float* out, int64_t n, F f) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = f(a[i], b[i]);
}

static inline int grid_for(Device* d, int64_t items, int64_t per_block, int max_blocks_per_sm) {
    int64_t need = (items + per_block - 1) / per_block;
    int64_t cap = (int64_t)d->sm_count * max_blocks_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

static inline int finish_launch(const char* what, int launches = 1) {
    count_launch(launches);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

static inline int64_t map_tiles(int64_t n4, int U) { return (n4 + (int64_t)kMapThreads * U - 1) / ((int64_t)kMapThreads * U); }

template <class F>
static int run_map1(Device* d, float* out, const float* a, int64_t n, F f) {
    if (n <= 0) return KTC_OK;
    if (aligned16(out) && aligned16(a) && n >= 4) {
        const int64_t n4 = n / 4;
        const int U = tune("map_unroll", 4);
        if (map_tiles(n4, 2) > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
        int launches = 1;
        if (U == 8)      k_map1_vec<8, F><<<(int)map_tiles(n4, 8), kMapThreads, 0, d->stream>>>((const float4*)a, (float4*)out, n4, f);
        else if (U == 2) k_map1_vec<2, F><<<(int)map_tiles(n4, 2), kMapThreads, 0, d->stream>>>((const float4*)a, (float4*)out, n4, f);
        else             k_map1_vec<4, F><<<(int)map_tiles(n4, 4), kMapThreads, 0, d->stream>>>((const float4*)a, (float4*)out, n4, f);
        if (n & 3) { k_map1_scalar<F><<<1, 32, 0, d->stream>>>(a + n4 * 4, out + n4 * 4, n & 3, f); ++launches; }
        return finish_launch("map1", launches);
    }
    k_map1_scalar<F><<<grid_for(d, n, 256, 16), 256, 0, d->stream>>>(a, out, n, f);
    return finish_launch("map1(scalar)");
}

template <class F>
static int run_map2(Device* d, float* out, const float* a, const float* b, int64_t n, F f) {
    if (n <= 0) return KTC_OK;
    if (aligned16(out) && aligned16(a) && aligned16(b) && n >= 4) {
        const int64_t n4 = n / 4;
        const int U = tune("map_unroll", 4);
        if (map_tiles(n4, 2) > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
        int launches = 1;
        if (U == 8)      k_map2_vec<8, F><<<(int)map_tiles(n4, 8), kMapThreads, 0, d->stream>>>((const float4*)a, (const float4*)b, (float4*)out, n4, f);
        else if (U == 2) k_map2_vec<2, F><<<(int)map_tiles(n4, 2), kMapThreads, 0, d->stream>>>((const float4*)a, (const float4*)b, (float4*)out, n4, f);
        else             k_map2_vec<4, F><<<(int)map_tiles(n4, 4), kMapThreads, 0, d->stream>>>((const float4*)a, (const float4*)b, (float4*)out, n4, f);
        if (n & 3) { k_map2_scalar<F><<<1, 32, 0, d->stream>>>(a + n4 * 4, b + n4 * 4, out + n4 * 4, n & 3, f); ++launches; }
        return finish_launch("map2", launches);
    }
    k_map2_scalar<F><<<grid_for(d, n, 256, 16), 256, 0, d->stream>>>(a, b, out, n, f);
    return finish_launch("map2(scalar)");
}

}  // namespace ktc
