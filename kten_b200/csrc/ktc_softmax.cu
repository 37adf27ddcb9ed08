// ktc_softmax.cu -- the forward of SoftmaxCrossEntropy in one pass over the logits.
//
// kten-api's SoftmaxCrossEntropy.doForward (functions/nn/SoftmaxCrossEntropy.kt:40-59) is eleven raw-tensor
// calls: row maximum, shifted exp, row sum, divide, row sum of the quotients, divide, clamp, log, gather at the
// targets, negate, mean.  Call by call the logits' volume crosses HBM about fourteen times.  Here one warp owns a
// row, keeps it in registers, and performs the same operations in the same order with the same roundings:
//
//   m   = max_j x[j]                        Math.max semantics (NaN propagates), as ktc_reduce_axis(MAX)
//   e_j = (float)exp((double)(x[j] - m))    the library's exp (ktc_math.cuh)
//   S   = sum_j e_j                         accumulated exactly as ktc_reduce_axis(SUM) accumulates a row of this
//                                           length: per lane float runs of 8 vectors folded into a double, lanes
//                                           combined by a xor-shuffle tree in double, one rounding to float
//   p_j = e_j / S                           the IEEE quotient (through the row's reciprocal where that gives it); written out:
//                                           the tensor saved for backward
//   S2  = sum_j p_j                         same accumulation
//   nll = -log(clamp(p_t / S2, lo, hi))     only at the target column t of the row -- the reference computes the
//                                           second normalisation, the clamp and the log for every column and then
//                                           gathers one; the picked value is the same
//
// so `softmax` and `nll` carry the bits the call-by-call sequence produces on this library (tests compare them), and
// the mean over the rows is left to ktc_reduce_all.  Traffic: the logits read once, the softmax written once.
// A target outside [0, cols) is recorded in the device's index-error word and that row's nll is NaN; nothing is
// read out of bounds.
#include "ktc_accum.cuh"

namespace ktc {

constexpr int kSxMaxVec = 16;             // float4 per lane: rows of up to 2048 columns

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

// NV > 0: every lane owns exactly NV vectors (cols == 128 NV) and the guards below fold away; NV == 0: any row length
// MINB: resident CTAs per SM the register allocation must allow (the row of 2048 columns alone is 64 registers per lane)
template <int NV, int MINB>
__global__ void __launch_bounds__(256, MINB) k_softmax_xent_forward(const float* __restrict__ logits, const float* __restrict__ targets,
                                                              float* __restrict__ softmax, float* __restrict__ nll,
                                                              int64_t rows, int cols, float lo, float hi, int* err) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;                                       // whole warps leave together
    const int q1 = cols >> 2;
    const int n_l = NV > 0 ? NV : (q1 > lane ? (q1 - lane + 31) >> 5 : 0);        // vectors of this lane
    const float4* px = reinterpret_cast<const float4*>(logits + row * cols);
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
    float4* ps = reinterpret_cast<float4*>(softmax + row * cols);
    #pragma unroll
    for (int u = 0; u < kSxMaxVec; ++u) {
        if (u < n_l) {
            v[u] = div_by_row(v[u], S, rS);
            __stcs(ps + lane + 32 * u, v[u]);
        }
    }
    const float S2 = sx_row_sum(v, n_l);
    // the target column: its owner has it in a register
    const float tf = targets[row];
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
            nll[row] = -log_f(jmin(jmax(p, lo), hi));
        } else {
            *err = 1;
            nll[row] = CUDART_NAN_F;
        }
    }
}

int launch_softmax_xent_forward(Device* d, float* softmax, float* nll, const float* logits, const float* targets,
                                int64_t rows, int64_t cols, float lo, float hi) {
    if (rows == 0) return KTC_OK;
    const int64_t grid = (rows + 7) / 8;
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
#define KTC_SX(NV, MINB) k_softmax_xent_forward<NV, MINB><<<(int)grid, 256, 0, d->stream>>>(logits, targets, softmax, nll, rows, (int)cols, lo, hi, d->idx_err)
    if (cols == 2048) { if (tune("softmax_min_blocks", 2) == 3) KTC_SX(16, 3); else KTC_SX(16, 2); }
    else if (cols == 1024) KTC_SX(8, 3); else if (cols == 512) KTC_SX(4, 4); else KTC_SX(0, 2);
#undef KTC_SX
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of softmax_xent_forward failed: %s", cudaGetErrorString(e));
    return take_index_error(d, "SoftmaxCrossEntropy target", cols, 1);
}

}  // namespace ktc

using namespace ktc;

// softmax [rows, cols] and nll [rows] of logits [rows, cols] against targets [rows] (class indices as floats);
// lo / hi: the clamp bounds, PlatformProvider.epsilon and 1 - epsilon.  KTC_ENOTSUP (cols > 2048, cols not a
// multiple of 4, unaligned rows): run the reference's call sequence instead.
extern "C" int ktc_softmax_xent_forward(ktc_buf softmax, ktc_buf nll, ktc_buf logits, ktc_buf targets, int64_t rows, int64_t cols, float lo, float hi) {
    if (rows < 0 || cols < 1) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: bad shape [%lld, %lld]", (long long)rows, (long long)cols);
    Buf bs, bn, bl, bt;
    KTC_TRY(resolve(softmax, &bs)); KTC_TRY(resolve(nll, &bn)); KTC_TRY(resolve(logits, &bl)); KTC_TRY(resolve(targets, &bt));
    if (bs.dev != bl.dev || bn.dev != bl.dev || bt.dev != bl.dev) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: buffers live on different devices");
    if (bl.n < rows * cols || bs.n < rows * cols || bn.n < rows || bt.n < rows) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: a buffer is too small for [%lld, %lld]", (long long)rows, (long long)cols);
    if (bs.ptr == bl.ptr) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: softmax aliases logits");
    if (cols > kSxMaxVec * 128 || cols <= tune("reduce_rows_small_max", 64) || (cols & 3) || !aligned16(bl.ptr) || !aligned16(bs.ptr))
        return fail(KTC_ENOTSUP, "ktc_softmax_xent_forward: rows of %lld columns are not handled in one pass (more than 64 and at most %d, a multiple of 4, 16-byte aligned)",
                    (long long)cols, kSxMaxVec * 128);
    Device* d = device(bl.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    return launch_softmax_xent_forward(d, bs.ptr, bn.ptr, bl.ptr, bt.ptr, rows, cols, lo, hi);
}
