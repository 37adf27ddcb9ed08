// ktc_reduce.cu -- axis reductions, full reductions, sum-to-shape, scatter (sm_100a).
//
// Every reduction works on the collapsed view [outer, A, inner] of a contiguous
// float32 tensor (aggregateOverAxis, JVMRawTensor.kt:154-225).  Three read-only
// streaming kernels cover the shapes, each usable as a single pass or as the
// first pass of a split reduction (the axis cut into S segments, partials in
// scratch memory, combined by a small second kernel in a fixed order, so the
// result does not depend on scheduling and is bit-stable from run to run):
//
//   rows_small : inner == 1, short rows: G lanes (1..32) per row, shuffle tree
//   rows_block : inner == 1, long rows : one CTA per (row, segment), float4 loads,
//                several independent loads in flight per thread, block tree
//   cols       : inner  > 1           : a CTA owns TX (x4) adjacent columns and a
//                segment of the axis, threads stride over the axis (every
//                warp-level load is one contiguous row piece), tree over TY
//
// Accumulation.  SUM/MEAN: each thread sums at most CHUNK values in float, then
// folds that partial into a double accumulator; all cross-thread and
// cross-segment combining is done in double and narrowed once.  The result is
// therefore within a few float ulps of the exact sum for any length, which is
// the tolerance reductions are held to (kten-jvm's own float-sequential sum()
// stalls at 2^24-scale totals and cannot serve as the target).  MAX/MIN follow
// Math.max/min (NaN-propagating, -0 < +0).  ARGMAX/ARGMIN use strict compares
// from -inf/+inf, so a NaN is never selected, ties resolve to the lowest index
// and an all -inf (or all-NaN) row yields index 0 (JVMRawTensor.kt:166-184);
// indices are returned as float32.
#include "ktc_internal.hpp"
#include "ktc_math.cuh"

namespace ktc {

static inline int finish_launch(const char* what, int launches = 1) {
    count_launch(launches);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

// ---- accumulators ---------------------------------------------------------------
// One accumulator type per operation family; `Partial` is what a split first
// pass stores per (segment, output).
struct SumAcc {
    typedef double Partial;
    float run; int cnt; double acc;
    static constexpr int CHUNK = 32;
    __device__ __forceinline__ void init() { run = 0.f; cnt = 0; acc = 0.0; }
    __device__ __forceinline__ void add(float v, int64_t) {
        run = __fadd_rn(run, v);
        if (++cnt == CHUNK) { acc += (double)run; run = 0.f; cnt = 0; }
    }
    __device__ __forceinline__ void flush() { acc += (double)run; run = 0.f; cnt = 0; }
    __device__ __forceinline__ void merge_partial(double p) { acc += p; }
    __device__ __forceinline__ void merge(SumAcc& o) { flush(); acc += o.partial(); }
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) { flush(); acc += __shfl_xor_sync(mask, acc, off); }
    __device__ __forceinline__ double partial() { flush(); return acc; }
};

template <bool IS_MAX> struct ExtAcc {
    typedef float Partial;
    float v;
    __device__ __forceinline__ void init() { v = IS_MAX ? -CUDART_INF_F : CUDART_INF_F; }
    __device__ __forceinline__ void add(float x, int64_t) { v = IS_MAX ? jmax(v, x) : jmin(v, x); }
    __device__ __forceinline__ void merge_partial(float p) { v = IS_MAX ? jmax(v, p) : jmin(v, p); }
    __device__ __forceinline__ void merge(ExtAcc& o) { merge_partial(o.v); }
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) {
        const float o = __shfl_xor_sync(mask, v, off);
        v = IS_MAX ? jmax(v, o) : jmin(v, o);
    }
    __device__ __forceinline__ float partial() { return v; }
};

struct ArgPair { float v; int64_t i; };

template <bool IS_MAX> struct ArgAcc {
    typedef ArgPair Partial;
    float v; int64_t i;
    // "no candidate yet" is (-inf / +inf, index 2^62); index 0 is substituted at the very end
    __device__ __forceinline__ void init() { v = IS_MAX ? -CUDART_INF_F : CUDART_INF_F; i = (int64_t)1 << 62; }
    __device__ __forceinline__ void take(float x, int64_t j) {
        const bool better = IS_MAX ? (x > v) : (x < v);
        if (better || (x == v && j < i)) { v = x; i = j; }
    }
    __device__ __forceinline__ void add(float x, int64_t j) {
        // strict compare against the running best: NaN and the initial value never win
        const bool cand = IS_MAX ? (x > -CUDART_INF_F) : (x < CUDART_INF_F);
        if (cand) take(x, j);
    }
    __device__ __forceinline__ void merge_partial(ArgPair p) { if (p.i < ((int64_t)1 << 62)) take(p.v, p.i); }
    __device__ __forceinline__ void merge(ArgAcc& o) { merge_partial(o.partial()); }
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) {
        const float ov = __shfl_xor_sync(mask, v, off);
        const long long oi = __shfl_xor_sync(mask, (long long)i, off);
        if (oi < ((long long)1 << 62)) take(ov, (int64_t)oi);
    }
    __device__ __forceinline__ ArgPair partial() { ArgPair p; p.v = v; p.i = i; return p; }
};

// final store: OUT_KIND 0 = value, 1 = mean (sum / count), 2 = index, 3 = value + index
template <int OUT_KIND, class Acc> struct Finish;
template <> struct Finish<0, SumAcc> { static __device__ __forceinline__ void put(SumAcc& a, float* out, float*, int64_t o, int64_t) { out[o] = (float)a.partial(); } };
template <> struct Finish<1, SumAcc> { static __device__ __forceinline__ void put(SumAcc& a, float* out, float*, int64_t o, int64_t A) { out[o] = (float)(a.partial() / (double)A); } };
template <bool M> struct Finish<0, ExtAcc<M>> { static __device__ __forceinline__ void put(ExtAcc<M>& a, float* out, float*, int64_t o, int64_t) { out[o] = a.v; } };
template <bool M> struct Finish<2, ArgAcc<M>> {
    static __device__ __forceinline__ void put(ArgAcc<M>& a, float* out, float*, int64_t o, int64_t) {
        out[o] = (a.i < ((int64_t)1 << 62)) ? (float)a.i : 0.0f;
    }
};
// value + index: the value follows Math.max/min (so NaN propagates), computed by a second accumulator
template <bool M> struct ValIdxAcc {
    typedef ArgPair Partial;   // unused: the fused kernel is never split
    ExtAcc<M> e; ArgAcc<M> a;
    __device__ __forceinline__ void init() { e.init(); a.init(); }
    __device__ __forceinline__ void add(float x, int64_t j) { e.add(x, j); a.add(x, j); }
    __device__ __forceinline__ void shfl_merge(unsigned mask, int off) { e.shfl_merge(mask, off); a.shfl_merge(mask, off); }
    __device__ __forceinline__ void merge_partial(ArgPair) {}
    __device__ __forceinline__ void merge(ValIdxAcc& o) { e.merge(o.e); a.merge(o.a); }
    __device__ __forceinline__ ArgPair partial() { return a.partial(); }
};
template <bool M> struct Finish<3, ValIdxAcc<M>> {
    static __device__ __forceinline__ void put(ValIdxAcc<M>& a, float* out, float* out_idx, int64_t o, int64_t) {
        out[o] = a.e.v;
        out_idx[o] = (a.a.i < ((int64_t)1 << 62)) ? (float)a.a.i : 0.0f;
    }
};

// block-level tree: every warp reduces with shuffles, warp leaders publish to
// shared memory, warp 0 combines them in warp order.
template <class Acc>
__device__ __forceinline__ void block_reduce(Acc& a, Acc* sm) {
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) a.shfl_merge(0xffffffffu, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) sm[warp] = a;
    __syncthreads();
    if (warp == 0) {
        Acc b; b.init();
        if (lane < nwarps) b = sm[lane];
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) b.shfl_merge(0xffffffffu, off);
        a = b;
    }
}

// ---- rows_small: inner == 1, G lanes per row --------------------------------------
template <int G, int OUT_KIND, class Acc>
__global__ void __launch_bounds__(256) k_rows_small(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ out_idx,
                                                    int64_t outer, int64_t A) {
    const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
    const int lane_in_group = threadIdx.x & (G - 1);
    // all lanes of a warp run the same number of iterations so the shuffles stay converged
    const int64_t rows_per_sweep = nthreads / G;
    const int64_t sweeps = (outer + rows_per_sweep - 1) / rows_per_sweep;
    for (int64_t s = 0; s < sweeps; ++s) {
        const int64_t row = s * rows_per_sweep + gthread / G;
        Acc acc; acc.init();
        if (row < outer) {
            const float* p = in + row * A;
            for (int64_t j = lane_in_group; j < A; j += G) acc.add(__ldg(p + j), j);
        }
        #pragma unroll
        for (int off = G >> 1; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
        if (row < outer && lane_in_group == 0) Finish<OUT_KIND, Acc>::put(acc, out, out_idx, row, A);
    }
}

// ---- rows_block: inner == 1, one CTA per (row, segment) ------------------------------
// A % 4 == 0 and 16-byte aligned rows are required for the float4 path (VEC=4);
// VEC=1 is the scalar variant.  When S > 1 the CTA writes a Partial to
// part[seg * outer + row] instead of the final value.
template <int VEC, int OUT_KIND, bool SPLIT, class Acc>
__global__ void __launch_bounds__(512) k_rows_block(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ out_idx,
                                                    typename Acc::Partial* __restrict__ part,
                                                    int64_t outer, int64_t A, int S, int64_t seg_len) {
    __shared__ Acc sm[32];
    const int64_t n_items = outer * S;
    for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int64_t row = item / S; const int seg = (int)(item - row * S);
        const int64_t j0 = (int64_t)seg * seg_len;
        const int64_t j1 = min(A, j0 + seg_len);
        const float* p = in + row * A;
        Acc acc; acc.init();
        if (VEC == 4) {
            constexpr int U = 4;
            const float4* p4 = reinterpret_cast<const float4*>(p);
            const int64_t q0 = j0 >> 2, q1 = j1 >> 2;          // seg_len is a multiple of 4
            for (int64_t q = q0 + threadIdx.x; q < q1; q += (int64_t)blockDim.x * U) {
                float4 v[U];
                #pragma unroll
                for (int u = 0; u < U; ++u) { const int64_t k = q + (int64_t)u * blockDim.x; if (k < q1) v[u] = __ldcs(p4 + k); }
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int64_t k = q + (int64_t)u * blockDim.x;
                    if (k < q1) { const int64_t j = k << 2; acc.add(v[u].x, j); acc.add(v[u].y, j + 1); acc.add(v[u].z, j + 2); acc.add(v[u].w, j + 3); }
                }
            }
        } else {
            for (int64_t j = j0 + threadIdx.x; j < j1; j += blockDim.x) acc.add(__ldg(p + j), j);
        }
        block_reduce(acc, sm);
        if (threadIdx.x == 0) {
            if (SPLIT) part[(int64_t)seg * outer + row] = acc.partial();
            else Finish<OUT_KIND, Acc>::put(acc, out, out_idx, row, A);
        }
    }
}

// ---- cols: inner > 1 ------------------------------------------------------------
// blockDim = (TX, TY).  A CTA owns columns [c0, c0 + TX*VEC) of one `outer`
// slice and axis rows [j0, j1); thread (tx, ty) walks rows j0+ty, j0+ty+TY, ...
template <int VEC, int OUT_KIND, bool SPLIT, class Acc>
__global__ void __launch_bounds__(256) k_cols(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ out_idx,
                                              typename Acc::Partial* __restrict__ part,
                                              int64_t outer, int64_t A, int64_t inner, int S, int64_t seg_len, int64_t col_tiles) {
    extern __shared__ __align__(16) unsigned char sm_raw[];
    Acc* sm = reinterpret_cast<Acc*>(sm_raw);               // [TY][TX*VEC]
    const int TX = blockDim.x, TY = blockDim.y;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t n_items = outer * col_tiles * S;
    for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int seg = (int)(item % S);
        const int64_t rest = item / S;
        const int64_t ct = rest % col_tiles, o = rest / col_tiles;
        const int64_t c = ct * (int64_t)TX * VEC + (int64_t)tx * VEC;
        const int64_t j0 = (int64_t)seg * seg_len, j1 = min(A, j0 + seg_len);
        Acc acc[VEC];
        #pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k].init();
        if (c < inner) {
            const float* p = in + o * A * inner + c;
            constexpr int U = 4;
            for (int64_t j = j0 + ty; j < j1; j += (int64_t)TY * U) {
                if (VEC == 4) {
                    float4 v[U];
                    #pragma unroll
                    for (int u = 0; u < U; ++u) { const int64_t jj = j + (int64_t)u * TY; if (jj < j1) v[u] = __ldcs(reinterpret_cast<const float4*>(p + jj * inner)); }
                    #pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int64_t jj = j + (int64_t)u * TY;
                        if (jj < j1) { acc[0].add(v[u].x, jj); acc[1 % VEC].add(v[u].y, jj); acc[2 % VEC].add(v[u].z, jj); acc[3 % VEC].add(v[u].w, jj); }
                    }
                } else {
                    float v[U];
                    #pragma unroll
                    for (int u = 0; u < U; ++u) { const int64_t jj = j + (int64_t)u * TY; if (jj < j1) v[u] = __ldg(p + jj * inner); }
                    #pragma unroll
                    for (int u = 0; u < U; ++u) { const int64_t jj = j + (int64_t)u * TY; if (jj < j1) acc[0].add(v[u], jj); }
                }
            }
        }
        // tree over ty in shared memory (fixed order)
        __syncthreads();
        #pragma unroll
        for (int k = 0; k < VEC; ++k) sm[(ty * TX + tx) * VEC + k] = acc[k];
        __syncthreads();
        if (ty == 0 && c < inner) {
            #pragma unroll
            for (int k = 0; k < VEC; ++k) {
                Acc r = sm[tx * VEC + k];
                for (int y = 1; y < TY; ++y) {
                    Acc other = sm[(y * TX + tx) * VEC + k];
                    r.merge(other);
                }
                const int64_t oidx = o * inner + c + k;
                if (SPLIT) part[(int64_t)seg * (outer * inner) + oidx] = r.partial();
                else Finish<OUT_KIND, Acc>::put(r, out, out_idx, oidx, A);
            }
        }
    }
}

// ---- second pass: combine S partials per output in segment order --------------------
template <int OUT_KIND, class Acc>
__global__ void k_combine(const typename Acc::Partial* __restrict__ part, float* __restrict__ out, float* __restrict__ out_idx,
                          int64_t n_out, int S, int64_t A) {
    // one warp per output; lanes stride over the segments, then a shuffle tree
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t o = warp; o < n_out; o += nwarps) {
        Acc acc; acc.init();
        for (int s = lane; s < S; s += 32) acc.merge_partial(part[(int64_t)s * n_out + o]);
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
        if (lane == 0) Finish<OUT_KIND, Acc>::put(acc, out, out_idx, o, A);
    }
}

// ---- host side ------------------------------------------------------------------
struct Plan {
    int kind;          // 0 rows_small, 1 rows_block, 2 cols
    int G;             // rows_small lanes per row
    int vec;           // 1 or 4
    int S;             // segments
    int64_t seg_len;
    int tx, ty; int64_t col_tiles;
    int grid;
};

static Plan make_plan(Device* d, const float* in, int64_t outer, int64_t A, int64_t inner, bool allow_split) {
    Plan p{}; p.S = 1; p.seg_len = A; p.vec = 1; p.G = 1;
    const int64_t target_ctas = (int64_t)d->sm_count * tune("reduce_ctas_per_sm", 8);
    if (inner == 1) {
        const bool vec_ok = (A % 4 == 0) && aligned16(in);
        const int64_t small_limit = tune("reduce_rows_small_max", 512);
        if (A <= small_limit || (A < 4096 && !vec_ok && outer >= 2048)) {
            p.kind = 0;
            int g = 1; while (g < 32 && g * 4 < A) g <<= 1;      // about four elements per lane, at most a warp
            p.G = g;
            const int64_t threads_needed = outer * g;
            int64_t blocks = (threads_needed + 255) / 256;
            const int64_t cap = (int64_t)d->sm_count * 16;
            p.grid = (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
            return p;
        }
        p.kind = 1; p.vec = vec_ok ? 4 : 1;
        if (allow_split && outer < target_ctas) {
            int64_t S = (target_ctas + outer - 1) / outer;
            const int64_t min_seg = 8192;                        // floats per segment worth a CTA
            const int64_t max_S = (A + min_seg - 1) / min_seg;
            if (S > max_S) S = max_S;
            if (S > 1) {
                int64_t seg = (A + S - 1) / S; seg = (seg + 3) & ~(int64_t)3;
                p.S = (int)((A + seg - 1) / seg); p.seg_len = seg;
            }
        }
        const int64_t items = outer * p.S;
        p.grid = (int)(items < target_ctas * 4 ? items : target_ctas * 4);
        if (p.grid < 1) p.grid = 1;
        return p;
    }
    p.kind = 2;
    const bool vec_ok = (inner % 4 == 0) && aligned16(in);
    p.vec = vec_ok ? 4 : 1;
    const int64_t lanes_needed = (inner + p.vec - 1) / p.vec;
    int tx = 1; while (tx < 32 && tx < lanes_needed) tx <<= 1;
    p.tx = tx; p.ty = 256 / tx;
    if ((int64_t)p.ty > A) { int ty = 1; while (ty < A) ty <<= 1; p.ty = ty < 1 ? 1 : ty; }
    p.col_tiles = (lanes_needed + tx - 1) / tx;
    const int64_t base_items = outer * p.col_tiles;
    if (allow_split && base_items < target_ctas) {
        int64_t S = (target_ctas + base_items - 1) / base_items;
        const int64_t min_seg = (int64_t)p.ty * 16;
        const int64_t max_S = (A + min_seg - 1) / min_seg;
        if (S > max_S) S = max_S;
        if (S > 1) { const int64_t seg = (A + S - 1) / S; p.S = (int)((A + seg - 1) / seg); p.seg_len = seg; }
    }
    const int64_t items = base_items * p.S;
    p.grid = (int)(items < target_ctas * 4 ? items : target_ctas * 4);
    if (p.grid < 1) p.grid = 1;
    return p;
}

template <int OUT_KIND, class Acc>
static int run_reduce(Device* d, float* out, float* out_idx, const float* in, int64_t outer, int64_t A, int64_t inner,
                      bool allow_split) {
    const int64_t n_out = outer * inner;
    if (n_out == 0) return KTC_OK;
    const Plan p = make_plan(d, in, outer, A, inner, allow_split);
    typedef typename Acc::Partial Partial;
    Scratch scratch; Partial* part = nullptr;
    if (p.S > 1) {
        const int64_t floats = ((int64_t)sizeof(Partial) * p.S * n_out + 3) / 4;
        KTC_TRY(scratch.get(d, floats));
        part = reinterpret_cast<Partial*>(scratch.ptr);
    }
    if (p.kind == 0) {
#define KTC_RS(GG) case GG: k_rows_small<GG, OUT_KIND, Acc><<<p.grid, 256, 0, d->stream>>>(in, out, out_idx, outer, A); break;
        switch (p.G) { KTC_RS(1) KTC_RS(2) KTC_RS(4) KTC_RS(8) KTC_RS(16) KTC_RS(32) }
#undef KTC_RS
        return finish_launch("rows_small");
    }
    if (p.kind == 1) {
        const int threads = tune("reduce_block_threads", 256);
        if (p.S > 1) {
            if (p.vec == 4) k_rows_block<4, OUT_KIND, true, Acc><<<p.grid, threads, 0, d->stream>>>(in, out, out_idx, part, outer, A, p.S, p.seg_len);
            else            k_rows_block<1, OUT_KIND, true, Acc><<<p.grid, threads, 0, d->stream>>>(in, out, out_idx, part, outer, A, p.S, p.seg_len);
        } else {
            if (p.vec == 4) k_rows_block<4, OUT_KIND, false, Acc><<<p.grid, threads, 0, d->stream>>>(in, out, out_idx, part, outer, A, 1, A);
            else            k_rows_block<1, OUT_KIND, false, Acc><<<p.grid, threads, 0, d->stream>>>(in, out, out_idx, part, outer, A, 1, A);
        }
    } else {
        const dim3 block(p.tx, p.ty);
        const size_t smem = sizeof(Acc) * (size_t)p.tx * p.ty * p.vec;
        if (p.S > 1) {
            if (p.vec == 4) k_cols<4, OUT_KIND, true, Acc><<<p.grid, block, smem, d->stream>>>(in, out, out_idx, part, outer, A, inner, p.S, p.seg_len, p.col_tiles);
            else            k_cols<1, OUT_KIND, true, Acc><<<p.grid, block, smem, d->stream>>>(in, out, out_idx, part, outer, A, inner, p.S, p.seg_len, p.col_tiles);
        } else {
            if (p.vec == 4) k_cols<4, OUT_KIND, false, Acc><<<p.grid, block, smem, d->stream>>>(in, out, out_idx, part, outer, A, inner, 1, A, p.col_tiles);
            else            k_cols<1, OUT_KIND, false, Acc><<<p.grid, block, smem, d->stream>>>(in, out, out_idx, part, outer, A, inner, 1, A, p.col_tiles);
        }
    }
    KTC_TRY(finish_launch(p.kind == 1 ? "rows_block" : "cols"));
    if (p.S > 1) {
        const int64_t warps = n_out;
        int64_t blocks = (warps * 32 + 255) / 256;
        const int64_t cap = (int64_t)d->sm_count * 8;
        if (blocks > cap) blocks = cap;
        k_combine<OUT_KIND, Acc><<<(int)blocks, 256, 0, d->stream>>>(part, out, out_idx, n_out, p.S, A);
        KTC_TRY(finish_launch("combine"));
    }
    return KTC_OK;
}

// op: KTC_SUM..KTC_ARGMIN, or 100 / 101 for fused (value, index) of max / min
int launch_reduce_axis(Device* d, int op, float* out, float* out_idx, const float* in,
                       int64_t outer, int64_t A, int64_t inner) {
    switch (op) {
    case KTC_SUM:    return run_reduce<0, SumAcc>(d, out, nullptr, in, outer, A, inner, true);
    case KTC_MEAN:   return run_reduce<1, SumAcc>(d, out, nullptr, in, outer, A, inner, true);
    case KTC_MAX:    return run_reduce<0, ExtAcc<true>>(d, out, nullptr, in, outer, A, inner, true);
    case KTC_MIN:    return run_reduce<0, ExtAcc<false>>(d, out, nullptr, in, outer, A, inner, true);
    case KTC_ARGMAX: return run_reduce<2, ArgAcc<true>>(d, out, nullptr, in, outer, A, inner, true);
    case KTC_ARGMIN: return run_reduce<2, ArgAcc<false>>(d, out, nullptr, in, outer, A, inner, true);
    case 100:        return run_reduce<3, ValIdxAcc<true>>(d, out, out_idx, in, outer, A, inner, false);
    case 101:        return run_reduce<3, ValIdxAcc<false>>(d, out, out_idx, in, outer, A, inner, false);
    }
    return fail(KTC_EINVAL, "unknown aggregating op %d", op);
}

// ---- scatter along an axis (Max/Min backward) -----------------------------------------
__global__ void k_scatter_axis(float* __restrict__ target, const float* __restrict__ index, const float* __restrict__ src,
                               int64_t outer, int64_t A, int64_t inner, int* err) {
    const int64_t n = outer * inner;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = e / inner, i = e - o * inner;
        const int idx = (int)index[e];                      // Float.toInt(): truncation
        if (idx < 0 || idx >= A) { *err = 1; continue; }    // recorded, never dereferenced
        target[(o * A + idx) * inner + i] = src[e];
    }
}

int launch_scatter_axis(Device* d, float* target, const float* index, const float* src,
                        int64_t outer, int64_t A, int64_t inner) {
    const int64_t n = outer * inner;
    if (n == 0) return KTC_OK;
    int64_t blocks = (n + 255) / 256; const int64_t cap = (int64_t)d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    k_scatter_axis<<<(int)blocks, 256, 0, d->stream>>>(target, index, src, outer, A, inner, d->err_flag);
    KTC_TRY(finish_launch("scatter_axis"));
    int h = 0;
    KTC_CUDA(cudaMemcpyAsync(&h, d->err_flag, sizeof(int), cudaMemcpyDeviceToHost, d->stream));
    KTC_CUDA(cudaStreamSynchronize(d->stream));
    if (h != 0) {
        KTC_CUDA(cudaMemsetAsync(d->err_flag, 0, sizeof(int), d->stream));
        return fail(KTC_EINVAL, "Scatter got invalid index, an index value is out of bounds 0 and %lld", (long long)A);
    }
    return KTC_OK;
}

}  // namespace ktc
