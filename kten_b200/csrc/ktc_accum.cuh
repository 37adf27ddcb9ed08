// ktc_accum.cuh -- accumulators and second-pass kernels shared by the reduction kernels
// (ktc_reduce.cu) and the fused expression kernel (ktc_expr.cu).
#pragma once

#include "ktc_internal.hpp"
#include "ktc_math.cuh"

namespace ktc {

// Math.max / Math.min in one instruction: NaN if either operand is NaN, +0 > -0
__device__ __forceinline__ float max_nan(float a, float b) { float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ float min_nan(float a, float b) { float r; asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }

// ---- accumulators ---------------------------------------------------------------
// A thread feeds its accumulator in batches: begin(); add(v, j) for at most 32
// values in increasing j; end().  `Partial` is what a split first pass stores
// per (segment, output).
constexpr int kNoIndex = 0x7fffffff;

struct SumAcc {
    typedef double Partial;
    float run; double acc;
    __device__ __forceinline__ void init() { run = 0.f; acc = 0.0; }
    __device__ __forceinline__ void begin() { run = 0.f; }
    __device__ __forceinline__ void add(float v, int) { run = __fadd_rn(run, v); }
    __device__ __forceinline__ void add4(float4 v, int) { run = __fadd_rn(run, __fadd_rn(__fadd_rn(v.x, v.y), __fadd_rn(v.z, v.w))); }
    __device__ __forceinline__ void end() { acc += (double)run; run = 0.f; }
    __device__ __forceinline__ void merge_partial(double p) { acc += p; }
    __device__ __forceinline__ void merge(SumAcc& o) { acc += o.acc; }
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) { acc += __shfl_xor_sync(mask, acc, off); }
    __device__ __forceinline__ double partial() { return acc; }
};

template <bool IS_MAX> struct ExtAcc {
    typedef float Partial;
    float v;
    __device__ __forceinline__ static float op(float a, float b) { return IS_MAX ? max_nan(a, b) : min_nan(a, b); }
    __device__ __forceinline__ void init() { v = IS_MAX ? -CUDART_INF_F : CUDART_INF_F; }
    __device__ __forceinline__ void begin() {}
    __device__ __forceinline__ void add(float x, int) { v = op(v, x); }
    __device__ __forceinline__ void add4(float4 x, int) { v = op(v, op(op(x.x, x.y), op(x.z, x.w))); }
    __device__ __forceinline__ void end() {}
    __device__ __forceinline__ void merge_partial(float p) { v = op(v, p); }
    __device__ __forceinline__ void merge(ExtAcc& o) { v = op(v, o.v); }
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) { v = op(v, __shfl_xor_sync(mask, v, off)); }
    __device__ __forceinline__ float partial() { return v; }
};

struct ArgPair { float v; int i; };

template <bool IS_MAX> struct ArgAcc {
    typedef ArgPair Partial;
    float v; int i;
    // "no candidate yet" is (-inf / +inf, kNoIndex); index 0 is substituted at the very end
    __device__ __forceinline__ void init() { v = IS_MAX ? -CUDART_INF_F : CUDART_INF_F; i = kNoIndex; }
    __device__ __forceinline__ void begin() {}
    // a thread sees its indices in increasing order, so the strict compare of the
    // reference loop is enough: NaN and the initial value never win, the first of equals stays
    __device__ __forceinline__ void add(float x, int j) { if (IS_MAX ? (x > v) : (x < v)) { v = x; i = j; } }
    __device__ __forceinline__ void add4(float4 x, int j) { add(x.x, j); add(x.y, j + 1); add(x.z, j + 2); add(x.w, j + 3); }
    __device__ __forceinline__ void end() {}
    // candidates from another thread / segment: larger value wins, equal values -> lower index
    __device__ __forceinline__ void take(float x, int j) {
        if (j != kNoIndex && ((IS_MAX ? (x > v) : (x < v)) || (x == v && j < i))) { v = x; i = j; }
    }
    __device__ __forceinline__ void merge_partial(ArgPair p) { take(p.v, p.i); }
    __device__ __forceinline__ void merge(ArgAcc& o) { take(o.v, o.i); }
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) {
        const float ov = __shfl_xor_sync(mask, v, off);
        const int oi = __shfl_xor_sync(mask, i, off);
        take(ov, oi);
    }
    __device__ __forceinline__ ArgPair partial() { ArgPair p; p.v = v; p.i = i; return p; }
};

// value + index in one pass: the value follows Math.max/min (NaN propagates), the index the strict-compare rule
struct ValIdxPair { float e; float v; int i; };
template <bool M> struct ValIdxAcc {
    typedef ValIdxPair Partial;
    ExtAcc<M> e; ArgAcc<M> a;
    __device__ __forceinline__ void init() { e.init(); a.init(); }
    __device__ __forceinline__ void begin() {}
    __device__ __forceinline__ void add(float x, int j) { e.add(x, j); a.add(x, j); }
    __device__ __forceinline__ void add4(float4 x, int j) { e.add4(x, j); a.add4(x, j); }
    __device__ __forceinline__ void end() {}
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) { e.shfl_merge(mask, off); a.shfl_merge(mask, off); }
    __device__ __forceinline__ void merge_partial(ValIdxPair p) { e.merge_partial(p.e); a.take(p.v, p.i); }
    __device__ __forceinline__ void merge(ValIdxAcc& o) { e.merge(o.e); a.merge(o.a); }
    __device__ __forceinline__ ValIdxPair partial() { ValIdxPair p; p.e = e.v; p.v = a.v; p.i = a.i; return p; }
};

// final store: OUT_KIND 0 = value, 1 = mean (sum / count), 2 = index, 3 = value + index
template <int OUT_KIND, class Acc> struct Finish;
template <> struct Finish<0, SumAcc> { static __device__ __forceinline__ void put(SumAcc& a, float* out, float*, int64_t o, int64_t) { out[o] = (float)a.acc; } };
template <> struct Finish<1, SumAcc> { static __device__ __forceinline__ void put(SumAcc& a, float* out, float*, int64_t o, int64_t A) { out[o] = (float)(a.acc / (double)A); } };
template <bool M> struct Finish<0, ExtAcc<M>> { static __device__ __forceinline__ void put(ExtAcc<M>& a, float* out, float*, int64_t o, int64_t) { out[o] = a.v; } };
template <bool M> struct Finish<2, ArgAcc<M>> {
    static __device__ __forceinline__ void put(ArgAcc<M>& a, float* out, float*, int64_t o, int64_t) { out[o] = (a.i != kNoIndex) ? (float)a.i : 0.0f; }
};
template <bool M> struct Finish<3, ValIdxAcc<M>> {
    static __device__ __forceinline__ void put(ValIdxAcc<M>& a, float* out, float* out_idx, int64_t o, int64_t) {
        out[o] = a.e.v;
        out_idx[o] = (a.a.i != kNoIndex) ? (float)a.a.i : 0.0f;
    }
};

// ---- second pass: combine S partials per output in segment order --------------------
// One warp per output when there are many segments, one thread per output when few
// (coalesced across outputs).
template <int OUT_KIND, class Acc>
__global__ void __launch_bounds__(256) k_combine_warp(const typename Acc::Partial* __restrict__ part, float* __restrict__ out,
                                                      float* __restrict__ out_idx, int64_t n_out, int S, int64_t A) {
    const int64_t o = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (o >= n_out) return;
    Acc acc; acc.init();
    for (int s = lane; s < S; s += 32) acc.merge_partial(part[(int64_t)s * n_out + o]);
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
    if (lane == 0) Finish<OUT_KIND, Acc>::put(acc, out, out_idx, o, A);
}

template <int OUT_KIND, class Acc>
__global__ void __launch_bounds__(256) k_combine_thread(const typename Acc::Partial* __restrict__ part, float* __restrict__ out,
                                                        float* __restrict__ out_idx, int64_t n_out, int S, int64_t A) {
    const int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= n_out) return;
    Acc acc; acc.init();
    for (int s = 0; s < S; ++s) acc.merge_partial(part[(int64_t)s * n_out + o]);
    Finish<OUT_KIND, Acc>::put(acc, out, out_idx, o, A);
}

// few outputs, many segments: one CTA per output, threads stride over the segments,
// then shuffles inside each warp and a fixed-order pass over the warp leaders
template <int OUT_KIND, class Acc>
__global__ void __launch_bounds__(512) k_combine_block(const typename Acc::Partial* __restrict__ part, float* __restrict__ out,
                                                       float* __restrict__ out_idx, int64_t n_out, int S, int64_t A) {
    __shared__ Acc sm[16];
    const int64_t o = blockIdx.x;
    Acc acc; acc.init();
    for (int s = threadIdx.x; s < S; s += blockDim.x) acc.merge_partial(part[(int64_t)s * n_out + o]);
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) sm[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        Acc r = sm[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) { Acc other = sm[w]; r.merge(other); }
        Finish<OUT_KIND, Acc>::put(r, out, out_idx, o, A);
    }
}


}  // namespace ktc
