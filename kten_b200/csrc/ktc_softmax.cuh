// ktc_softmax.cuh -- one row of SoftmaxCrossEntropy's forward, held in registers by one warp.
//
// kten-api's SoftmaxCrossEntropy.doForward (functions/nn/SoftmaxCrossEntropy.kt:40-59) is eleven raw-tensor
// calls: row maximum, shifted exp, row sum, divide, row sum of the quotients, divide, clamp, log, gather at the
// targets, negate, mean.  sx_rows performs the same operations in the same order with the same roundings:
//
//   m   = max_j x[j]                        Math.max semantics (NaN propagates), as ktc_reduce_axis(MAX)
//   e_j = (float)exp((double)(x[j] - m))    the library's exp (ktc_math.cuh)
//   S   = sum_j e_j                         accumulated exactly as ktc_reduce_axis(SUM) accumulates a row of this
//                                           length: per lane float runs of 8 vectors folded into a double, lanes
//                                           combined by a xor-shuffle tree in double, one rounding to float
//   p_j = e_j / S                           the IEEE quotient (through the row's reciprocal where that gives it): the
//                                           tensor the function saves for backward
//   S2  = sum_j p_j                         same accumulation
//   nll = -log(clamp(p_t / S2, lo, hi))     only at the target column t of the row -- the reference computes the
//                                           second normalisation, the clamp and the log for every column and then
//                                           gathers one; the picked value is the same
//
// The quotients p_j are written to `softmax` when the caller wants them in memory, and handed, vector by vector, to
// an epilogue: the stand-alone kernel (ktc_softmax.cu) passes none, a kernel generated at run time (ktc_jit.cu,
// whose source embeds this file) passes the elementwise program that consumes the softmax -- the backward of the
// function -- so that the saved tensor never crosses HBM.
// A target outside [0, cols) is recorded in the device's index-error word and that row's nll is NaN; nothing is
// read out of bounds.
#pragma once

#include "ktc_accum.cuh"

namespace ktc {

constexpr int kSxMaxVec = 16;             // float4 per lane: rows of up to 2048 columns
constexpr float kSxWindowArg = -43.0f;    // exp of anything above is >= 2^-62.1, inside kd_div_window's dividend range [2^-63, 2^64)

struct SxArgs {
    const float* logits; const float* targets;
    float* softmax;                       // nullptr: the quotients are not written
    float* nll;
    int64_t rows; int cols;
    float lo, hi;                         // the clamp bounds
    int* err;                             // device word set when a target lies outside its row
};

// the row sum of ktc_reduce_axis(SUM) for a row whose vectors v[u] sit at float4 index lane + 32 u (u < n_l)
__device__ __forceinline__ float sx_row_sum(const float4 (&v)[kSxMaxVec], int n_l) {
    SumAcc acc; acc.init();
    const int full = n_l >> 3;
    #pragma unroll
    for (int b = 0; b < kSxMaxVec / 8; ++b) {
        if (b < full) {
            acc.begin();
            #pragma unroll
            for (int k = 0; k < 8; ++k) acc.add4(v[b * 8 + k], 0);
            acc.end();
        }
    }
    acc.begin();
    #pragma unroll
    for (int u = 0; u < kSxMaxVec; ++u) if (u >= full * 8 && u < n_l) acc.add4(v[u], 0);
    acc.end();
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
    return (float)acc.acc;
}

struct SxNoEpilogue {
    __device__ __forceinline__ void begin(int64_t) {}
    __device__ __forceinline__ void operator()(int64_t, int, const float4&) const {}
};

// One warp per row, eight rows per CTA of 256 threads.  NV > 0: every lane owns exactly NV vectors (cols == 128 NV)
// and the guards below fold away; NV == 0: any row length.  The epilogue: begin(row) once -- whatever it needs per row --,
// then epi(row, column of the vector's first element, p) for every vector of quotients.
template <int NV, class Epi>
__device__ __forceinline__ void sx_rows(const SxArgs& a, Epi& epi) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= a.rows) return;                                     // whole warps leave together
    epi.begin(row);
    const int cols = a.cols;
    const int q1 = cols >> 2;
    const int n_l = NV > 0 ? NV : (q1 > lane ? (q1 - lane + 31) >> 5 : 0);        // vectors of this lane
    const float4* px = reinterpret_cast<const float4*>(a.logits + row * cols);
    float4 v[kSxMaxVec];
    #pragma unroll
    for (int u = 0; u < kSxMaxVec; ++u) if (u < n_l) v[u] = __ldcs(px + lane + 32 * u);
    // row maximum
    ExtAcc<true> mx; mx.init();
    #pragma unroll
    for (int u = 0; u < kSxMaxVec; ++u) if (u < n_l) mx.add4(v[u], 0);
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx.shfl_merge(0xffffffffu, off);
    const float m = mx.v;
    // exp(x - max); an argument above kSxWindowArg gives a dividend inside the window of the division by the row's reciprocal
    // (exp(-43) > 2^-63; a NaN fails the comparison): tested here on the argument, one comparison per element
    unsigned in_window = 0u;
    #pragma unroll
    for (int u = 0; u < kSxMaxVec; ++u) {
        if (u < n_l) {
            const float4 s = make_float4(__fsub_rn(v[u].x, m), __fsub_rn(v[u].y, m), __fsub_rn(v[u].z, m), __fsub_rn(v[u].w, m));
            if (s.x >= kSxWindowArg && s.y >= kSxWindowArg && s.z >= kSxWindowArg && s.w >= kSxWindowArg) in_window |= 1u << u;
            v[u] = apply1(UnOp<KTC_EXP>(), s);
        }
    }
    const float S = sx_row_sum(v, n_l);
    const float rS = kd_row_reciprocal(S);                         // the IEEE quotients through the row's reciprocal (ktc_math.cuh)
    const bool keep = a.softmax != nullptr;
    float4* ps = keep ? reinterpret_cast<float4*>(a.softmax + row * cols) : nullptr;
    #pragma unroll
    for (int u = 0; u < kSxMaxVec; ++u) {
        if (u < n_l) {
            v[u] = div_by_row_known(v[u], S, rS, (in_window >> u) & 1u);
            if (keep) __stcs(ps + lane + 32 * u, v[u]);
            epi(row, (lane + 32 * u) * 4, v[u]);
        }
    }
    const float S2 = sx_row_sum(v, n_l);
    // the target column: its owner has it in a register
    const float tf = a.targets[row];
    const int t = (int)tf;                                          // Float.toInt(): truncation
    const bool ok = tf == tf && t >= 0 && t < cols;
    float picked = 0.f;
    if (ok) {
        const int q = t >> 2, owner = q & 31, u_t = q >> 5, c = t & 3;
        float mine = 0.f;
        #pragma unroll
        for (int u = 0; u < kSxMaxVec; ++u)
            if (u == u_t) mine = c == 0 ? v[u].x : c == 1 ? v[u].y : c == 2 ? v[u].z : v[u].w;
        picked = __shfl_sync(0xffffffffu, mine, owner);
    }
    if (lane == 0) {
        if (ok) {
            const float p = __fdiv_rn(picked, S2);
            a.nll[row] = -log_f(jmin(jmax(p, a.lo), a.hi));
        } else {
            *a.err = 1;
            a.nll[row] = CUDART_NAN_F;
        }
    }
}

// Rows of exactly 2048 columns with TWO warps per row (four rows per CTA of 256 threads): each lane then holds 8 vectors
// instead of 16, the kernel needs half the registers, and twice as many warps are resident to hide the latency of the
// loads and of the exp chain.  The bits do not change: warp h of the pair owns the vectors lane + 32 (8 h + u), u < 8 --
// exactly the h-th float run of the one-warp form -- so a lane's double is (0.0 + run_0) + run_1 as before (the second run
// arrives through shared memory), and both warps then walk the same xor-shuffle tree; the maximum is associative.
template <class Epi>
__device__ __forceinline__ void sx_rows_pair(const SxArgs& a, Epi& epi) {
    __shared__ float sh_max[8];
    __shared__ double sh_run[2][8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, half = warp & 1, pr = warp >> 1;
    const int64_t row = (int64_t)blockIdx.x * 4 + pr;
    if (row >= a.rows) return;                                     // both warps of a pair leave together
    epi.begin(row);
    constexpr int cols = 2048;
    const int first = lane + 256 * half;                           // float4 index of this lane's first vector
    const float4* px = reinterpret_cast<const float4*>(a.logits + row * cols) + first;
    float4 v[8];
    #pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcs(px + 32 * u);
    auto pair_barrier = [&]() { asm volatile("bar.sync %0, 64;" :: "r"(pr + 1) : "memory"); };
    ExtAcc<true> mx; mx.init();
    #pragma unroll
    for (int u = 0; u < 8; ++u) mx.add4(v[u], 0);
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx.shfl_merge(0xffffffffu, off);
    if (lane == 0) sh_max[warp] = mx.v;
    pair_barrier();
    const float m = max_nan(sh_max[2 * pr], sh_max[2 * pr + 1]);
    unsigned in_window = 0u;
    #pragma unroll
    for (int u = 0; u < 8; ++u) {
        const float4 s = make_float4(__fsub_rn(v[u].x, m), __fsub_rn(v[u].y, m), __fsub_rn(v[u].z, m), __fsub_rn(v[u].w, m));
        if (s.x >= kSxWindowArg && s.y >= kSxWindowArg && s.z >= kSxWindowArg && s.w >= kSxWindowArg) in_window |= 1u << u;
        v[u] = apply1(UnOp<KTC_EXP>(), s);
    }
    // the row sum: this warp's float run, folded with the partner's in the order run_0, run_1
    auto row_sum = [&](int which) -> float {
        SumAcc acc; acc.init();
        acc.begin();
        #pragma unroll
        for (int u = 0; u < 8; ++u) acc.add4(v[u], 0);
        sh_run[which][warp][lane] = (double)acc.run;
        pair_barrier();
        acc.acc = 0.0;
        acc.acc += sh_run[which][2 * pr][lane];
        acc.acc += sh_run[which][2 * pr + 1][lane];
        acc.acc += 0.0;                                            // the empty tail run of the one-warp form
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc.shfl_merge(0xffffffffu, off);
        return (float)acc.acc;
    };
    const float S = row_sum(0);
    const float rS = kd_row_reciprocal(S);
    const bool keep = a.softmax != nullptr;
    float4* ps = keep ? reinterpret_cast<float4*>(a.softmax + row * cols) + first : nullptr;
    #pragma unroll
    for (int u = 0; u < 8; ++u) {
        v[u] = div_by_row_known(v[u], S, rS, (in_window >> u) & 1u);
        if (keep) __stcs(ps + 32 * u, v[u]);
        epi(row, (first + 32 * u) * 4, v[u]);
    }
    const float S2 = row_sum(1);
    const float tf = a.targets[row];
    const int t = (int)tf;                                          // Float.toInt(): truncation
    const bool ok = tf == tf && t >= 0 && t < cols;
    if (ok) {
        const int q = t >> 2, owner = q & 31, u_all = q >> 5, c = t & 3;
        if ((u_all >> 3) != half) return;                           // the other warp of the pair holds the target column
        const int u_t = u_all & 7;
        float mine = 0.f;
        #pragma unroll
        for (int u = 0; u < 8; ++u)
            if (u == u_t) mine = c == 0 ? v[u].x : c == 1 ? v[u].y : c == 2 ? v[u].z : v[u].w;
        const float picked = __shfl_sync(0xffffffffu, mine, owner);
        if (lane == 0) a.nll[row] = -log_f(jmin(jmax(__fdiv_rn(picked, S2), a.lo), a.hi));
    } else if (half == 0 && lane == 0) {
        *a.err = 1;
        a.nll[row] = CUDART_NAN_F;
    }
}

// Rows of more than 2048 columns (up to kSxMaxColsCta): ONE CTA per row, one warp for every 1024 columns (up to twelve),
// eight vectors per lane.  ktc_reduce_axis(SUM) gives such a row to a single warp (up to 12288 columns with its default
// segment length): lane l adds its vectors l + 32 u in runs of eight -- float runs, each folded into the lane's double in
// order, the remainder as a last shorter run -- and the lanes are combined by the xor-shuffle tree.  Here warp w owns
// u in [8 w, 8 w + 8), i.e. run w of every lane; the run sums go through shared memory and every warp folds all of its
// lane's runs in order (a run beyond the row is 0f: adding it changes nothing) and then walks the tree: the same
// operations in the same order, so the same bits.  The maximum is associative.  This is sx_rows_pair for any number of
// warps, with the CTA's barrier in place of the pair's.
constexpr int kSxMaxColsCta = 12288;
constexpr int kSxMaxWarpsCta = kSxMaxColsCta / 1024;
__host__ __device__ inline int sx_cta_warps(int cols) { return (cols + 1023) / 1024; }
// FULL: the row is a multiple of 1024 columns, every lane of every warp owns exactly eight vectors and the guards fold away
template <bool FULL, class Epi>
__device__ __forceinline__ void sx_rows_cta(const SxArgs& a, Epi& epi) {
    __shared__ float sh_max[kSxMaxWarpsCta];
    __shared__ float sh_run[2][kSxMaxWarpsCta][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int64_t row = blockIdx.x;                                 // grid == rows
    epi.begin(row);
    const int cols = a.cols;
    const int q1 = cols >> 2;
    const int n_row = q1 > lane ? (q1 - lane + 31) >> 5 : 0;        // this lane's vectors in the one-warp form
    const int n_l = FULL ? 8 : min(max(n_row - 8 * warp, 0), 8);   // ... of which this warp holds [8 warp, 8 warp + n_l)
    const int first = lane + 256 * warp;                           // float4 index of the first
    const float4* px = reinterpret_cast<const float4*>(a.logits + row * cols) + first;
    float4 v[8];
    #pragma unroll
    for (int u = 0; u < 8; ++u) if (u < n_l) v[u] = __ldcs(px + 32 * u);
    ExtAcc<true> mx; mx.init();
    #pragma unroll
    for (int u = 0; u < 8; ++u) if (u < n_l) mx.add4(v[u], 0);
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx.shfl_merge(0xffffffffu, off);
    if (lane == 0) sh_max[warp] = mx.v;
    __syncthreads();
    float m = sh_max[0];
    for (int w = 1; w < n_warps; ++w) m = max_nan(m, sh_max[w]);
    unsigned in_window = 0u;
    #pragma unroll
    for (int u = 0; u < 8; ++u) {
        if (u < n_l) {
            const float4 s = make_float4(__fsub_rn(v[u].x, m), __fsub_rn(v[u].y, m), __fsub_rn(v[u].z, m), __fsub_rn(v[u].w, m));
            if (s.x >= kSxWindowArg && s.y >= kSxWindowArg && s.z >= kSxWindowArg && s.w >= kSxWindowArg) in_window |= 1u << u;
            v[u] = apply1(UnOp<KTC_EXP>(), s);
        }
    }
    auto row_sum = [&](int which) -> float {
        SumAcc acc; acc.init();
        acc.begin();
        #pragma unroll
        for (int u = 0; u < 8; ++u) if (u < n_l) acc.add4(v[u], 0);
        sh_run[which][warp][lane] = acc.run;
        __syncthreads();
        double d = 0.0;
        for (int r = 0; r < n_warps; ++r) d += (double)sh_run[which][r][lane];
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        return (float)d;
    };
    const float S = row_sum(0);
    const float rS = kd_row_reciprocal(S);
    const bool keep = a.softmax != nullptr;
    float4* ps = keep ? reinterpret_cast<float4*>(a.softmax + row * cols) + first : nullptr;
    #pragma unroll
    for (int u = 0; u < 8; ++u) {
        if (u < n_l) {
            v[u] = div_by_row_known(v[u], S, rS, (in_window >> u) & 1u);
            if (keep) __stcs(ps + 32 * u, v[u]);
            epi(row, (first + 32 * u) * 4, v[u]);
        }
    }
    const float S2 = row_sum(1);
    const float tf = a.targets[row];
    const int t = (int)tf;                                          // Float.toInt(): truncation
    const bool ok = tf == tf && t >= 0 && t < cols;
    if (ok) {
        const int q = t >> 2, owner = q & 31, u_all = q >> 5, c = t & 3;
        if ((u_all >> 3) != warp) return;                           // another warp holds the target column
        const int u_t = u_all & 7;
        float mine = 0.f;
        #pragma unroll
        for (int u = 0; u < 8; ++u)
            if (u == u_t) mine = c == 0 ? v[u].x : c == 1 ? v[u].y : c == 2 ? v[u].z : v[u].w;
        const float picked = __shfl_sync(0xffffffffu, mine, owner);
        if (lane == 0) a.nll[row] = -log_f(jmin(jmax(__fdiv_rn(picked, S2), a.lo), a.hi));
    } else if (warp == 0 && lane == 0) {
        *a.err = 1;
        a.nll[row] = CUDART_NAN_F;
    }
}

}  // namespace ktc
