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

struct SxNoEpilogue { __device__ __forceinline__ void operator()(int64_t, int, const float4&) const {} };

// One warp per row, eight rows per CTA of 256 threads.  NV > 0: every lane owns exactly NV vectors (cols == 128 NV)
// and the guards below fold away; NV == 0: any row length.  epi(row, column of the vector's first element, p).
template <int NV, class Epi>
__device__ __forceinline__ void sx_rows(const SxArgs& a, const Epi& epi) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= a.rows) return;                                     // whole warps leave together
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
    // exp(x - max)
    #pragma unroll
    for (int u = 0; u < kSxMaxVec; ++u) {
        if (u < n_l) {
            const float4 s = make_float4(__fsub_rn(v[u].x, m), __fsub_rn(v[u].y, m), __fsub_rn(v[u].z, m), __fsub_rn(v[u].w, m));
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
            v[u] = div_by_row(v[u], S, rS);
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

}  // namespace ktc
