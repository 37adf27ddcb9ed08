// ktc_nn.cu -- nearest-neighbour upsampling (TensorOperations.upsample, TensorOperations.kt:131; kten-jvm:
// JVMUpsample2DNearest.kt:14-77) as two streaming kernels.
//
// With P = the product of all dimensions but the last (N * C * H) the input is [P, W] and the output [P, s, W * s]:
// every input row becomes s identical output rows in which every value is repeated s times.  Forward: a thread builds
// one float4 of the expanded row from the (at most four) input values under it and stores it to the s output rows --
// the input is read once, through L1, and the output, s * s times as large, is written once with 128-bit stores.
// Gradient: an input position receives the sum of its s x s block, added in float from 0f in the reference's order (column
// offset in the outer loop, row offset in the inner one, JVMUpsample2DNearest.kt:61-68): the reference's own additions, so
// the result is bit-identical to kten-jvm's; a thread produces four neighbouring positions from s rows of
// 4 * s contiguous floats (128-bit loads for scales 2 to 4).  Shapes whose rows do not split into float4 take one-element-per-thread forms of the same loops.
#include "ktc_internal.hpp"

namespace ktc {

namespace {

// S > 0: the scale is S (2, 3 or 4) at compile time, so the divisions below are shifts or multiplications; S == 0: any scale
template <bool VEC, int S>
__global__ void __launch_bounds__(256) k_upsample_nearest(const float* __restrict__ in, float* __restrict__ out, int64_t P, int64_t W, int s_arg) {
    const int s = S > 0 ? S : s_arg;
    const int64_t OW = W * s;
    if (VEC) {
        const int64_t q = OW >> 2;                                       // float4 per expanded row
        const int64_t total = P * q;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t p = i / q, ox = (i - p * q) << 2;
            const float* row = in + p * W;
            float4 v;
            v.x = __ldg(row + ox / s); v.y = __ldg(row + (ox + 1) / s); v.z = __ldg(row + (ox + 2) / s); v.w = __ldg(row + (ox + 3) / s);
            float* o = out + p * s * OW + ox;
            for (int dy = 0; dy < s; ++dy) __stcs(reinterpret_cast<float4*>(o + dy * OW), v);
        }
    } else {
        const int64_t total = P * s * OW;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t orow = i / OW, ox = i - orow * OW;
            out[i] = __ldg(in + (orow / s) * W + ox / s);
        }
    }
}

// S > 0: rows split into float4 and the scale is S (2, 3 or 4): the s rows of 4 * S contiguous floats under four
// neighbouring input positions are fetched with 128-bit loads, all before the first use.  S == 0: any shape, one position per thread.
template <int S>
__global__ void __launch_bounds__(256) k_upsample_nearest_grad(const float* __restrict__ gout, float* __restrict__ gin, int64_t P, int64_t W, int s) {
    const int64_t OW = W * s;
    if (S > 0) {
        const int64_t q = W >> 2;
        const int64_t total = P * q;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t p = i / q, w = (i - p * q) << 2;
            const float* base = gout + p * S * OW + w * S;                // the block rows of this input row, at the first of four positions
            float v[S > 0 ? S : 1][4 * (S > 0 ? S : 1)];
            #pragma unroll
            for (int x = 0; x < S; ++x) {
                #pragma unroll
                for (int j = 0; j < S; ++j) {
                    const float4 t = __ldcs(reinterpret_cast<const float4*>(base + x * OW) + j);
                    v[x][4 * j] = t.x; v[x][4 * j + 1] = t.y; v[x][4 * j + 2] = t.z; v[x][4 * j + 3] = t.w;
                }
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            #pragma unroll
            for (int y = 0; y < S; ++y) {                                 // column offset: the reference's outer loop
                #pragma unroll
                for (int x = 0; x < S; ++x) {                             // row offset
                    #pragma unroll
                    for (int k = 0; k < 4; ++k) acc[k] = __fadd_rn(acc[k], v[x][k * S + y]);
                }
            }
            __stcs(reinterpret_cast<float4*>(gin + p * W + w), make_float4(acc[0], acc[1], acc[2], acc[3]));
        }
    } else {
        const int64_t total = P * W;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t p = i / W, w = i - p * W;
            const float* base = gout + p * s * OW + w * s;
            float acc = 0.f;
            for (int y = 0; y < s; ++y)
                for (int x = 0; x < s; ++x) acc = __fadd_rn(acc, __ldg(base + x * OW + y));
            gin[i] = acc;
        }
    }
}

int check_args(const char* what, ktc_buf big, ktc_buf small, int64_t P, int64_t W, int s, Buf* bb, Buf* bs) {
    if (P < 0 || W < 0 || s < 1) return fail(KTC_EINVAL, "%s: bad extents (P = %lld, W = %lld, scale = %d)", what, (long long)P, (long long)W, s);
    KTC_TRY(resolve(big, bb)); KTC_TRY(resolve(small, bs));
    if (bb->dev != bs->dev) return fail(KTC_EINVAL, "%s: buffers live on different devices", what);
    if (bs->n < P * W || bb->n < P * W * s * s) return fail(KTC_EINVAL, "%s: a buffer is too small for [%lld, %lld] at scale %d", what, (long long)P, (long long)W, s);
    if (bb->ptr == bs->ptr) return fail(KTC_EINVAL, "%s: the two tensors alias", what);
    return KTC_OK;
}

int grid_of(Device* d, int64_t items) {
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = (int64_t)d->sm_count * 32;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

int finish(const char* what) {
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

}  // namespace

}  // namespace ktc

using namespace ktc;

// out[P, scale, W * scale] from in[P, W] (P = the product of all dimensions but the last: N * C * H)
extern "C" int ktc_upsample2d_nearest(ktc_buf out, ktc_buf in, int64_t P, int64_t W, int scale) {
    Buf bo, bi;
    KTC_TRY(check_args("ktc_upsample2d_nearest", out, in, P, W, scale, &bo, &bi));
    if (P * W == 0) return KTC_OK;
    Device* d = device(bi.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    const bool vec = ((W * scale) & 3) == 0 && aligned16(bo.ptr);
    const int g4 = grid_of(d, P * (W * scale / 4));
    if (vec && scale == 2)      k_upsample_nearest<true, 2><<<g4, 256, 0, d->stream>>>(bi.ptr, bo.ptr, P, W, scale);
    else if (vec && scale == 3) k_upsample_nearest<true, 3><<<g4, 256, 0, d->stream>>>(bi.ptr, bo.ptr, P, W, scale);
    else if (vec && scale == 4) k_upsample_nearest<true, 4><<<g4, 256, 0, d->stream>>>(bi.ptr, bo.ptr, P, W, scale);
    else if (vec)               k_upsample_nearest<true, 0><<<g4, 256, 0, d->stream>>>(bi.ptr, bo.ptr, P, W, scale);
    else                        k_upsample_nearest<false, 0><<<grid_of(d, P * W * scale * scale), 256, 0, d->stream>>>(bi.ptr, bo.ptr, P, W, scale);
    return finish("upsample2d_nearest");
}

// grad_in[P, W] from grad_out[P, scale, W * scale]: every position receives the sum of its scale x scale block
extern "C" int ktc_upsample2d_nearest_grad(ktc_buf grad_in, ktc_buf grad_out, int64_t P, int64_t W, int scale) {
    Buf bo, bi;
    KTC_TRY(check_args("ktc_upsample2d_nearest_grad", grad_out, grad_in, P, W, scale, &bo, &bi));
    if (P * W == 0) return KTC_OK;
    Device* d = device(bi.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    const bool vec = (W & 3) == 0 && aligned16(bi.ptr) && aligned16(bo.ptr) && scale >= 2 && scale <= 4;
    const int g4 = grid_of(d, P * (W / 4));
    if (vec && scale == 2)      k_upsample_nearest_grad<2><<<g4, 256, 0, d->stream>>>(bo.ptr, bi.ptr, P, W, scale);
    else if (vec && scale == 3) k_upsample_nearest_grad<3><<<g4, 256, 0, d->stream>>>(bo.ptr, bi.ptr, P, W, scale);
    else if (vec && scale == 4) k_upsample_nearest_grad<4><<<g4, 256, 0, d->stream>>>(bo.ptr, bi.ptr, P, W, scale);
    else                        k_upsample_nearest_grad<0><<<grid_of(d, P * W), 256, 0, d->stream>>>(bo.ptr, bi.ptr, P, W, scale);
    return finish("upsample2d_nearest_grad");
}
