// ktc_reduce.cu -- axis reductions, full reductions, scatter (sm_100a).
//
// Every reduction works on the collapsed view [outer, A, inner] of a contiguous
// float32 tensor (aggregateOverAxis, JVMRawTensor.kt:154-225).  Three read-only
// streaming kernels cover the shapes.  Each can run as a single pass or as the
// first pass of a split reduction: the axis is cut into S segments, every
// segment leaves one partial in scratch memory, and a small second kernel
// combines the S partials of each output in a fixed order, so results do not
// depend on scheduling and are bit-stable from run to run.
//
//   rows_small : inner == 1, short rows : G lanes (1..32) per row, shuffle tree
//   rows_warp  : inner == 1, long rows  : one WARP per (row, segment) of at most
//                32 KB; 128-bit loads, eight independent requests in flight per
//                lane, shuffle tree, no shared memory and no block barrier
//   cols_warp  : inner  > 1            : one warp per (slice, segment, column tile);
//                each lane owns up to four adjacent columns and walks the axis, every
//                warp-level load is a contiguous row piece; no shared memory
//
// Work items are small (tens of KB) and launched in address order, one per
// warp / CTA, so that the set of items in flight at any time covers one
// contiguous region of memory: DRAM sees a single forward stream instead of
// a thousand interleaved ones.
//
// Accumulation.  SUM/MEAN: every batch of loads (at most 32 values per thread)
// is added in float and folded into a double accumulator; all cross-thread and
// cross-segment combining is done in double and narrowed once.  The result is
// within a few float ulps of the exact sum for any length, which is the
// tolerance reductions are held to (kten-jvm's own float-sequential sum() stalls
// at 2^24-scale totals and cannot serve as the target).  MAX/MIN follow Math.max
// / Math.min (NaN-propagating, -0 < +0: the max.NaN / min.NaN instructions).
// ARGMAX/ARGMIN use strict compares from -inf/+inf, so a NaN is never selected,
// ties resolve to the lowest index and an all -inf (or all-NaN) row yields index
// 0 (JVMRawTensor.kt:166-184); indices are returned as float32.
#include "ktc_accum.cuh"

namespace ktc {

static inline int finish_launch(const char* what, int launches = 1) {
    count_launch(launches);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

// ---- rows_small: inner == 1, G lanes per row --------------------------------------
template <int G, int OUT_KIND, class Acc>
__global__ void __launch_bounds__(256) k_rows_small(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ out_idx,
                                                    int64_t outer, int64_t A) {
    const int lane_in_group = threadIdx.x & (G - 1);
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;     // whole groups share a row; a warp never splits a group
    Acc acc; acc.init();
    if (row < outer) {
        const float* p = in + row * A;
        constexpr int U = 8;
        int64_t j = lane_in_group;
        for (; j + (int64_t)G * (U - 1) < A; j += (int64_t)G * U) {      // full batches: all loads first, no guards
            float v[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) v[u] = __ldg(p + j + (int64_t)u * G);
            acc.begin();
            #pragma unroll
            for (int u = 0; u < U; ++u) acc.add(v[u], (int)(j + (int64_t)u * G));
            acc.end();
        }
        acc.begin();
        for (; j < A; j += G) acc.add(__ldg(p + j), (int)j);              // at most U - 1 values
        acc.end();
    }
    #pragma unroll
    for (int off = G >> 1; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
    if (row < outer && lane_in_group == 0) Finish<OUT_KIND, Acc>::put(acc, out, out_idx, row, A);
}

// ---- rows_warp: inner == 1, one warp per (row, segment) ------------------------------
// Item w = row * S + seg covers in[row*A + seg*seg_len ... ) -- items are in address
// order.  VEC = 4 needs A % 4 == 0, seg_len % 4 == 0 and a 16-byte aligned base;
// VEC = 1 is the scalar variant.  MODE 0: final value per row (S == 1).  MODE 1: one
// Partial per segment at part[seg * outer + row].  MODE 2 (S % 8 == 0): the eight
// warps of a CTA hold consecutive segments of one row and leave ONE Partial, combined
// in warp order, at part[(seg / 8) * outer + row].
template <int VEC, int OUT_KIND, int MODE, class Acc>
__global__ void __launch_bounds__(256) k_rows_warp(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ out_idx,
                                                   typename Acc::Partial* __restrict__ part,
                                                   int64_t outer, int64_t A, int S, int64_t seg_len) {
    __shared__ Acc sm[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t item = (int64_t)blockIdx.x * 8 + warp;
    if (MODE != 2 && item >= outer * S) return;          // whole warps leave together (MODE 2 grids are exact)
    const int64_t row = item / S; const int seg = (int)(item - row * S);
    const int64_t j0 = (int64_t)seg * seg_len;
    const int64_t j1 = min(A, j0 + seg_len);
    const float* p = in + row * A;
    Acc acc; acc.init();
    constexpr int U = 8;
    if (VEC == 4) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
        const int64_t q1 = j1 >> 2;
        int64_t q = (j0 >> 2) + lane;
        for (; q + 32 * (U - 1) < q1; q += 32 * U) {                       // full batches: all loads first, no guards
            float4 v[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) v[u] = __ldcs(p4 + q + 32 * u);
            acc.begin();
            #pragma unroll
            for (int u = 0; u < U; ++u) acc.add4(v[u], (int)((q + 32 * u) << 2));
            acc.end();
        }
        acc.begin();
        for (; q < q1; q += 32) acc.add4(__ldcs(p4 + q), (int)(q << 2));   // at most U - 1 vectors
        acc.end();
    } else {
        int64_t j = j0 + lane;
        for (; j + 32 * (U - 1) < j1; j += 32 * U) {
            float v[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) v[u] = __ldg(p + j + 32 * u);
            acc.begin();
            #pragma unroll
            for (int u = 0; u < U; ++u) acc.add(v[u], (int)(j + 32 * u));
            acc.end();
        }
        acc.begin();
        for (; j < j1; j += 32) acc.add(__ldg(p + j), (int)j);
        acc.end();
    }
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
    if (MODE == 2) {
        if (lane == 0) sm[warp] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            Acc r = sm[0];
            #pragma unroll
            for (int w = 1; w < 8; ++w) { Acc other = sm[w]; r.merge(other); }
            part[(int64_t)(seg >> 3) * outer + row] = r.partial();
        }
    } else if (lane == 0) {
        if (MODE == 1) part[(int64_t)seg * outer + row] = acc.partial();
        else Finish<OUT_KIND, Acc>::put(acc, out, out_idx, row, A);
    }
}

// ---- cols: inner > 1, one warp per (o, segment, column tile) --------------------------
// A warp owns TX*VEC adjacent columns (TX lanes, a power of two) and the rows
// [j0, j1) of the axis; when TX < 32 the other lanes take different rows (TYW = 32/TX
// rows at a time).  Every lane accumulates its own columns over its rows -- each
// warp-level load is TYW contiguous row pieces -- and the TYW row groups are merged
// with shuffles at the end: no shared memory, no barrier.  Items are ordered with the
// column tile fastest, then the segment, then o, i.e. in address order.
// MODE 0: final values (S == 1).  MODE 1: one Partial per segment.  MODE 2 (S % 8 == 0):
// the eight warps of a CTA take eight consecutive segments of the same column tile and
// leave ONE Partial per column, combined in warp order, at part[(seg / 8) * n_out + o].
// The kernel is bound by the number of loads in flight.  Measured on the middle-axis sum of [512, 4096, 128]: one batch
// of 8 float4 per lane at five CTAs per SM (48 registers) 6200 GB/s; two batches in flight per lane -- the next one
// requested before the current one is added -- at two CTAs per SM (120 registers) 6840 GB/s, level with the maximum,
// whose begin / end are empty so that the compiler overlaps its batches by itself.  Few warps with many requests each
// beat many warps with few.
template <class Acc> struct ColsPipelined { static constexpr bool value = false; };
template <> struct ColsPipelined<SumAcc> { static constexpr bool value = true; };

template <int VEC, int OUT_KIND, int MODE, class Acc, int PIPE = 0>
__global__ void __launch_bounds__(256, PIPE == 0 ? 1 : 2) k_cols_warp(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ out_idx,
                                                   typename Acc::Partial* __restrict__ part,
                                                   int64_t outer, int64_t A, int64_t inner, int S, int64_t seg_len,
                                                   int64_t col_tiles, int TX) {
    __shared__ Acc sm[MODE == 2 ? 8 * 32 * VEC : 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t ct, o; int seg;
    if (MODE == 2) {
        ct = blockIdx.x % col_tiles;
        const int64_t rest = blockIdx.x / col_tiles;
        const int SG = S >> 3;
        seg = (int)(rest % SG) * 8 + warp;
        o = rest / SG;
    } else {
        const int64_t item = (int64_t)blockIdx.x * 8 + warp;
        if (item >= outer * S * col_tiles) return;       // whole warps leave together
        ct = item % col_tiles;
        const int64_t rest = item / col_tiles;
        seg = (int)(rest % S);
        o = rest / S;
    }
    const int tx = lane & (TX - 1), tyw = lane / TX, TYW = 32 / TX;
    const int64_t c = (ct * TX + tx) * VEC;
    const int64_t j0 = (int64_t)seg * seg_len, j1 = min(A, j0 + seg_len);
    Acc acc[VEC];
    #pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k].init();
    if (c < inner) {
        const float* p = in + o * A * inner + c;
        constexpr int U = 8;
        const int64_t step = (int64_t)TYW * inner;            // floats between this lane's consecutive rows
        int64_t j = j0 + tyw;
        const float* pj = p + j * inner;
        if (VEC == 4 && PIPE != 0) {
            // Two batches of U loads in flight per lane: the next batch is requested before the current one is added, so a
            // warp keeps 16 float4 outstanding without waiting in between.  Same order of additions as below for full
            // groups: float runs of 4 batches (32 values), folded into the doubles.
            const int64_t bstep = (int64_t)TYW * U;
            const int64_t nb = (j + (int64_t)TYW * (U - 1) < j1) ? (j1 - 1 - j - (int64_t)TYW * (U - 1)) / bstep + 1 : 0;
            float4 va[U], vb[U];
            const float* q = pj;                               // the next row to request: one running address, no table of offsets
            if (nb > 0) {
                #pragma unroll
                for (int u = 0; u < U; ++u, q += step) va[u] = __ldcs(reinterpret_cast<const float4*>(q));
            }
            int64_t b = 0;
            for (; b + 1 < nb; b += 2) {
                #pragma unroll
                for (int u = 0; u < U; ++u, q += step) vb[u] = __ldcs(reinterpret_cast<const float4*>(q));
                if ((b & 3) == 0) {
                    #pragma unroll
                    for (int k = 0; k < VEC; ++k) acc[k].begin();
                }
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int jj = (int)(j + (int64_t)u * TYW);
                    acc[0].add(va[u].x, jj); acc[1 % VEC].add(va[u].y, jj); acc[2 % VEC].add(va[u].z, jj); acc[3 % VEC].add(va[u].w, jj);
                }
                if (b + 2 < nb) {
                    #pragma unroll
                    for (int u = 0; u < U; ++u, q += step) va[u] = __ldcs(reinterpret_cast<const float4*>(q));
                }
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int jj = (int)(j + bstep + (int64_t)u * TYW);
                    acc[0].add(vb[u].x, jj); acc[1 % VEC].add(vb[u].y, jj); acc[2 % VEC].add(vb[u].z, jj); acc[3 % VEC].add(vb[u].w, jj);
                }
                if ((b & 3) == 2) {
                    #pragma unroll
                    for (int k = 0; k < VEC; ++k) acc[k].end();
                }
                j += 2 * bstep;
            }
            if (b < nb) {                                      // an odd batch is left in va
                if ((b & 3) == 0) {
                    #pragma unroll
                    for (int k = 0; k < VEC; ++k) acc[k].begin();
                }
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int jj = (int)(j + (int64_t)u * TYW);
                    acc[0].add(va[u].x, jj); acc[1 % VEC].add(va[u].y, jj); acc[2 % VEC].add(va[u].z, jj); acc[3 % VEC].add(va[u].w, jj);
                }
                j += bstep;
            }
            pj = q;                                            // q has passed exactly the nb full batches
            // the open run, if any, takes the remaining rows too
            if (nb == 0 || (nb & 3) == 0) {
                #pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k].begin();
            }
            for (; j < j1; j += TYW, pj += step) {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(pj));
                acc[0].add(v.x, (int)j); acc[1 % VEC].add(v.y, (int)j); acc[2 % VEC].add(v.z, (int)j); acc[3 % VEC].add(v.w, (int)j);
            }
            #pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k].end();
        } else if (VEC == 4) {
            // four batches per fold into the double accumulators (32 values per float run)
            for (; j + (int64_t)TYW * (4 * U - 1) < j1;) {
                #pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k].begin();
                #pragma unroll 1
                for (int b = 0; b < 4; ++b, j += (int64_t)TYW * U, pj += step * U) {
                    float4 v[U];
                    #pragma unroll
                    for (int u = 0; u < U; ++u) v[u] = __ldcs(reinterpret_cast<const float4*>(pj + step * u));
                    #pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int jj = (int)(j + (int64_t)u * TYW);
                        acc[0].add(v[u].x, jj); acc[1 % VEC].add(v[u].y, jj); acc[2 % VEC].add(v[u].z, jj); acc[3 % VEC].add(v[u].w, jj);
                    }
                }
                #pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k].end();
            }
            for (; j + (int64_t)TYW * (U - 1) < j1; j += (int64_t)TYW * U, pj += step * U) {   // full batches, no guards
                float4 v[U];
                #pragma unroll
                for (int u = 0; u < U; ++u) v[u] = __ldcs(reinterpret_cast<const float4*>(pj + step * u));
                #pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k].begin();
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int jj = (int)(j + (int64_t)u * TYW);
                    acc[0].add(v[u].x, jj); acc[1 % VEC].add(v[u].y, jj); acc[2 % VEC].add(v[u].z, jj); acc[3 % VEC].add(v[u].w, jj);
                }
                #pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k].end();
            }
            #pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k].begin();
            for (; j < j1; j += TYW, pj += step) {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(pj));
                acc[0].add(v.x, (int)j); acc[1 % VEC].add(v.y, (int)j); acc[2 % VEC].add(v.z, (int)j); acc[3 % VEC].add(v.w, (int)j);
            }
            #pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k].end();
        } else {
            for (; j + (int64_t)TYW * (U - 1) < j1; j += (int64_t)TYW * U, pj += step * U) {
                float v[U];
                #pragma unroll
                for (int u = 0; u < U; ++u) v[u] = __ldg(pj + step * u);
                acc[0].begin();
                #pragma unroll
                for (int u = 0; u < U; ++u) acc[0].add(v[u], (int)(j + (int64_t)u * TYW));
                acc[0].end();
            }
            acc[0].begin();
            for (; j < j1; j += TYW, pj += step) acc[0].add(__ldg(pj), (int)j);
            acc[0].end();
        }
    }
    for (int off = TX; off < 32; off <<= 1) {            // merge the row groups (all lanes take part)
        #pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k].shfl_merge(0xffffffffu, off);
    }
    if (MODE == 2) {
        #pragma unroll
        for (int k = 0; k < VEC; ++k) sm[(warp * 32 + lane) * VEC + k] = acc[k];
        __syncthreads();
        if (warp == 0 && tyw == 0 && c < inner) {
            #pragma unroll
            for (int k = 0; k < VEC; ++k) {
                Acc r = sm[lane * VEC + k];
                #pragma unroll
                for (int w = 1; w < 8; ++w) { Acc other = sm[(w * 32 + lane) * VEC + k]; r.merge(other); }
                part[(int64_t)(seg >> 3) * (outer * inner) + o * inner + c + k] = r.partial();
            }
        }
    } else if (tyw == 0 && c < inner) {
        #pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const int64_t oidx = o * inner + c + k;
            if (MODE == 1) part[(int64_t)seg * (outer * inner) + oidx] = acc[k].partial();
            else Finish<OUT_KIND, Acc>::put(acc[k], out, out_idx, oidx, A);
        }
    }
}

// ---- host side ------------------------------------------------------------------
struct Plan {
    int kind;          // 0 rows_small, 1 rows_warp, 2 cols_warp
    int G;             // rows_small lanes per row
    int vec;           // 1 or 4
    int S;             // segments of the axis
    int S_out;         // partials per output the first pass leaves (S, or S/8 with the CTA pre-combine)
    int64_t seg_len;
    int tx; int64_t col_tiles;
    int64_t grid;
};

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

static Plan make_plan(Device* d, const float* in, int64_t outer, int64_t A, int64_t inner, int partial_bytes) {
    Plan p{}; p.S = 1; p.S_out = 1; p.seg_len = A; p.vec = 1; p.G = 1;
    if (inner == 1) {
        const bool vec_ok = (A % 4 == 0) && aligned16(in);
        if (A <= tune("reduce_rows_small_max", 64)) {
            p.kind = 0;
            int g = 1; while (g < 32 && g * 4 < A) g <<= 1;      // about four elements per lane
            p.G = g;
            p.grid = ceil_div(outer * g, 256);
            return p;
        }
        p.kind = 1; p.vec = vec_ok ? 4 : 1;
        int64_t seg = tune("reduce_seg_floats", 8192);            // 32 KB per warp
        seg = (seg + 3) & ~(int64_t)3;
        if (A > seg + seg / 2) {
            p.S = (int)ceil_div(A, seg); p.seg_len = seg;
            if (p.S >= 16) {                                       // eight segments per CTA, one partial per CTA
                p.S = (p.S + 7) & ~7;                              // (trailing segments may be empty)
                p.S_out = p.S / 8;
            } else p.S_out = p.S;
        }
        p.grid = ceil_div(outer * p.S, 8);                        // 8 warps per CTA
        return p;
    }
    p.kind = 2;
    const bool vec_ok = (inner % 4 == 0) && aligned16(in);   // every row start is then 16-byte aligned
    p.vec = vec_ok ? 4 : 1;
    const int64_t lanes_needed = ceil_div(inner, p.vec);
    int tx = 1; while (tx < 32 && tx < lanes_needed) tx <<= 1;
    p.tx = tx;
    p.col_tiles = ceil_div(lanes_needed, tx);
    // a warp streams about reduce_cols_item_kb; the partial traffic must stay under ~3 % of the input
    const int64_t row_bytes = (int64_t)tx * p.vec * 4;
    int64_t seg = tune("reduce_cols_item_kb", 32) * 1024 / row_bytes;
    const int64_t min_seg = (int64_t)partial_bytes * 8;           // S * partial_bytes <= A * 4 / 32
    if (seg < min_seg) seg = min_seg;
    if (A > seg + seg / 2) { p.S = (int)ceil_div(A, seg); p.seg_len = seg; }
    p.S_out = p.S;
    if (p.S >= 16) {                                              // eight segments per CTA, one partial per CTA and column
        p.S = (p.S + 7) & ~7;
        p.S_out = p.S / 8;
        p.grid = outer * p.S_out * p.col_tiles;
    } else p.grid = ceil_div(outer * p.S * p.col_tiles, 8);
    return p;
}

template <int OUT_KIND, class Acc>
static int run_reduce(Device* d, float* out, float* out_idx, const float* in, int64_t outer, int64_t A, int64_t inner) {
    const int64_t n_out = outer * inner;
    if (n_out == 0) return KTC_OK;
    typedef typename Acc::Partial Partial;
    const Plan p = make_plan(d, in, outer, A, inner, (int)sizeof(Partial));
    if (p.grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "reduction needs %lld CTAs", (long long)p.grid);
    Scratch scratch; Partial* part = nullptr;
    if (p.S > 1) {
        const int64_t floats = ((int64_t)sizeof(Partial) * p.S_out * n_out + 3) / 4;
        KTC_TRY(scratch.get(d, floats));
        part = reinterpret_cast<Partial*>(scratch.ptr);
    }
    const int grid = (int)(p.grid < 1 ? 1 : p.grid);
    if (p.kind == 0) {
#define KTC_RS(GG) case GG: k_rows_small<GG, OUT_KIND, Acc><<<grid, 256, 0, d->stream>>>(in, out, out_idx, outer, A); break;
        switch (p.G) { KTC_RS(1) KTC_RS(2) KTC_RS(4) KTC_RS(8) KTC_RS(16) KTC_RS(32) }
#undef KTC_RS
        return finish_launch("rows_small");
    }
    if (p.kind == 1) {
        const int mode = p.S == 1 ? 0 : (p.S_out == p.S ? 1 : 2);
#define KTC_RW(V, M) k_rows_warp<V, OUT_KIND, M, Acc><<<grid, 256, 0, d->stream>>>(in, out, out_idx, part, outer, A, p.S, p.seg_len)
        if (p.vec == 4) { if (mode == 0) KTC_RW(4, 0); else if (mode == 1) KTC_RW(4, 1); else KTC_RW(4, 2); }
        else            { if (mode == 0) KTC_RW(1, 0); else if (mode == 1) KTC_RW(1, 1); else KTC_RW(1, 2); }
#undef KTC_RW
    } else {
        const int mode = p.S == 1 ? 0 : (p.S_out == p.S ? 1 : 2);
#define KTC_CW(V, M) k_cols_warp<V, OUT_KIND, M, Acc><<<grid, 256, 0, d->stream>>>(in, out, out_idx, part, outer, A, inner, p.S, p.seg_len, p.col_tiles, p.tx)
#define KTC_CWP(M, P) k_cols_warp<4, OUT_KIND, M, Acc, P><<<grid, 256, 0, d->stream>>>(in, out, out_idx, part, outer, A, inner, p.S, p.seg_len, p.col_tiles, p.tx)
        constexpr int kPipe = ColsPipelined<Acc>::value ? 1 : 0;
        if (p.vec == 4 && kPipe == 1 && tune("cols_sum_pipe", 1) == 1) { if (mode == 0) KTC_CWP(0, kPipe); else if (mode == 1) KTC_CWP(1, kPipe); else KTC_CWP(2, kPipe); }
        else if (p.vec == 4) { if (mode == 0) KTC_CW(4, 0); else if (mode == 1) KTC_CW(4, 1); else KTC_CW(4, 2); }
        else            { if (mode == 0) KTC_CW(1, 0); else if (mode == 1) KTC_CW(1, 1); else KTC_CW(1, 2); }
#undef KTC_CW
#undef KTC_CWP
    }
    KTC_TRY(finish_launch(p.kind == 1 ? "rows_warp" : "cols_warp"));
    if (p.S > 1) {
        const int S2 = p.S_out;
        if (S2 >= 1024 && n_out <= 64) {
            k_combine_block<OUT_KIND, Acc><<<(int)n_out, 512, 0, d->stream>>>(part, out, out_idx, n_out, S2, A);
        } else if (S2 >= 64 || n_out < 4096) {
            const int64_t blocks = ceil_div(n_out * 32, 256);
            if (blocks > 0x7fffffffLL) return fail(KTC_ENOTSUP, "combine needs %lld CTAs", (long long)blocks);
            k_combine_warp<OUT_KIND, Acc><<<(int)blocks, 256, 0, d->stream>>>(part, out, out_idx, n_out, S2, A);
        } else {
            k_combine_thread<OUT_KIND, Acc><<<(int)ceil_div(n_out, 256), 256, 0, d->stream>>>(part, out, out_idx, n_out, S2, A);
        }
        KTC_TRY(finish_launch("combine"));
    }
    return KTC_OK;
}

// op: KTC_SUM..KTC_ARGMIN, or 100 / 101 for fused (value, index) of max / min
int launch_reduce_axis(Device* d, int op, float* out, float* out_idx, const float* in,
                       int64_t outer, int64_t A, int64_t inner) {
    if ((op == KTC_ARGMAX || op == KTC_ARGMIN || op >= 100) && A >= (int64_t)kNoIndex)
        return fail(KTC_EINVAL, "index reductions support an axis of at most 2^31 - 2 elements (the reference indexes with Int)");
    switch (op) {
    case KTC_SUM:    return run_reduce<0, SumAcc>(d, out, nullptr, in, outer, A, inner);
    case KTC_MEAN:   return run_reduce<1, SumAcc>(d, out, nullptr, in, outer, A, inner);
    case KTC_MAX:    return run_reduce<0, ExtAcc<true>>(d, out, nullptr, in, outer, A, inner);
    case KTC_MIN:    return run_reduce<0, ExtAcc<false>>(d, out, nullptr, in, outer, A, inner);
    case KTC_ARGMAX: return run_reduce<2, ArgAcc<true>>(d, out, nullptr, in, outer, A, inner);
    case KTC_ARGMIN: return run_reduce<2, ArgAcc<false>>(d, out, nullptr, in, outer, A, inner);
    case 100:        return run_reduce<3, ValIdxAcc<true>>(d, out, out_idx, in, outer, A, inner);
    case 101:        return run_reduce<3, ValIdxAcc<false>>(d, out, out_idx, in, outer, A, inner);
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
    k_scatter_axis<<<(int)blocks, 256, 0, d->stream>>>(target, index, src, outer, A, inner, d->idx_err);
    KTC_TRY(finish_launch("scatter_axis"));
    return take_index_error(d, "Scatter", A, 1);       // read where the host next waits for the stream (or at once: index_check_sync)
}

}  // namespace ktc
