// ktc_softmax.cu -- the forward of SoftmaxCrossEntropy in one pass over the logits (the row arithmetic: ktc_softmax.cuh).
//
// Call by call the eleven calls of SoftmaxCrossEntropy.doForward (functions/nn/SoftmaxCrossEntropy.kt:40-59) move the
// logits' volume through HBM about fourteen times; here the logits are read once and the softmax written once (one warp
// per row up to 2048 columns -- two for exactly 2048 --, one CTA per row up to 12288), and
// `softmax` and `nll` carry the bits the call-by-call sequence produces on this library (tests compare them).  The mean
// over the rows is left to ktc_reduce_all.
#include "ktc_softmax.cuh"

namespace ktc {

// MINB: resident CTAs per SM the register allocation must allow (the row of 2048 columns alone is 64 registers per lane)
template <int NV, int MINB>
__global__ void __launch_bounds__(256, MINB) k_softmax_xent_forward(const __grid_constant__ SxArgs a) {
    SxNoEpilogue none;
    sx_rows<NV>(a, none);
}

template <int MINB>
__global__ void __launch_bounds__(256, MINB) k_softmax_xent_forward_pair(const __grid_constant__ SxArgs a) {
    SxNoEpilogue none;
    sx_rows_pair(a, none);
}

template <bool FULL>
__global__ void __launch_bounds__(32 * kSxMaxWarpsCta, 2) k_softmax_xent_forward_cta(const __grid_constant__ SxArgs a) {
    SxNoEpilogue none;
    sx_rows_cta<FULL>(a, none);
}

// Row lengths the one-pass kernels take: what ktc_reduce_axis(SUM) gives to ONE warp per row (whose accumulation they
// reproduce), in float4 steps.
bool softmax_row_length_ok(int64_t cols) {
    const int64_t seg = (tune("reduce_seg_floats", 8192) + 3) & ~(int64_t)3;
    return cols > tune("reduce_rows_small_max", 64) && cols <= kSxMaxColsCta && cols <= seg + seg / 2 && (cols & 3) == 0;
}

// rows that get one CTA (sx_rows_cta) instead of one warp: beyond what a warp's registers hold, and rows of fewer than 1024
// columns without a kernel specialised on their length (a CTA of one warp with eight vectors per lane: measured 0.71 ms
// against 1.04 ms for 2^28 logits in rows of 768, forward + backward; between 1024 and 2048 columns the two are level)
bool softmax_row_takes_cta(int64_t cols) {
    if (cols > kSxMaxVec * 128) return true;
    return cols < 1024 && cols != 512 && tune("softmax_cta_short_rows", 1);
}

int launch_softmax_xent_forward(Device* d, float* softmax, float* nll, const float* logits, const float* targets,
                                int64_t rows, int64_t cols, float lo, float hi) {
    if (rows == 0) return KTC_OK;
    const int64_t grid = (rows + 7) / 8;
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    const SxArgs a{logits, targets, softmax, nll, rows, (int)cols, lo, hi, d->idx_err};
#define KTC_SX(NV, MINB) k_softmax_xent_forward<NV, MINB><<<(int)grid, 256, 0, d->stream>>>(a)
    if (softmax_row_takes_cta(cols)) {                             // one CTA per row
        if (rows > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
        if (cols % 1024 == 0) k_softmax_xent_forward_cta<true><<<(unsigned)rows, 32 * sx_cta_warps((int)cols), 0, d->stream>>>(a);
        else k_softmax_xent_forward_cta<false><<<(unsigned)rows, 32 * sx_cta_warps((int)cols), 0, d->stream>>>(a);
    }
    else if (cols == 2048 && tune("softmax_pair", 1)) {                 // two warps per row: half the registers, twice the warps in flight
        const int64_t grid4 = (rows + 3) / 4;
        if (grid4 > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
        if (tune("softmax_pair_min_blocks", 4) == 3) k_softmax_xent_forward_pair<3><<<(int)grid4, 256, 0, d->stream>>>(a);
        else k_softmax_xent_forward_pair<4><<<(int)grid4, 256, 0, d->stream>>>(a);
    }
    else if (cols == 2048) { if (tune("softmax_min_blocks", 2) == 3) KTC_SX(16, 3); else KTC_SX(16, 2); }
    else if (cols == 1024) KTC_SX(8, 3); else if (cols == 512) KTC_SX(4, 4); else KTC_SX(0, 2);
#undef KTC_SX
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of softmax_xent_forward failed: %s", cudaGetErrorString(e));
    return take_index_error(d, "SoftmaxCrossEntropy target", cols, 1);
}

}  // namespace ktc

using namespace ktc;

// softmax [rows, cols] (0: not wanted in memory) and nll [rows] of logits [rows, cols] against targets [rows] (class
// indices as floats); lo / hi: the clamp bounds, PlatformProvider.epsilon and 1 - epsilon.  KTC_ENOTSUP (cols > 2048, cols not a
// multiple of 4, unaligned rows): run the reference's call sequence instead.
extern "C" int ktc_softmax_xent_forward(ktc_buf softmax, ktc_buf nll, ktc_buf logits, ktc_buf targets, int64_t rows, int64_t cols, float lo, float hi) {
    if (rows < 0 || cols < 1) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: bad shape [%lld, %lld]", (long long)rows, (long long)cols);
    Buf bs{}, bn, bl, bt;
    if (softmax) KTC_TRY(resolve(softmax, &bs));
    KTC_TRY(resolve(nll, &bn)); KTC_TRY(resolve(logits, &bl)); KTC_TRY(resolve(targets, &bt));
    if ((softmax && bs.dev != bl.dev) || bn.dev != bl.dev || bt.dev != bl.dev) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: buffers live on different devices");
    if (bl.n < rows * cols || (softmax && bs.n < rows * cols) || bn.n < rows || bt.n < rows) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: a buffer is too small for [%lld, %lld]", (long long)rows, (long long)cols);
    if (softmax && bs.ptr == bl.ptr) return fail(KTC_EINVAL, "ktc_softmax_xent_forward: softmax aliases logits");
    if (!softmax_row_length_ok(cols) || !aligned16(bl.ptr) || (softmax && !aligned16(bs.ptr)))
        return fail(KTC_ENOTSUP, "ktc_softmax_xent_forward: rows of %lld columns are not handled in one pass (more than 64 and at most %d, a multiple of 4, 16-byte aligned)",
                    (long long)cols, kSxMaxColsCta);
    Device* d = device(bl.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    return launch_softmax_xent_forward(d, bs.ptr, bn.ptr, bl.ptr, bt.ptr, rows, cols, lo, hi);
}
