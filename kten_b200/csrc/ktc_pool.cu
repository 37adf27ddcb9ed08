// ktc_pool.cu -- spatial (2-D) max and average pooling and their gradients (TensorOperations.spatialPooling,
// TensorOperations.kt:127; PoolingOperation.kt:5-15; kten-jvm: JVMSpatialMaxPooling.kt:24-69,
// JVMSpatialAvgPooling.kt:23-88; 1-D pooling is the same with a trailing extent of 1, TensorExtensions.kt:158-215).
//
// A window reduction over [planes, H, W] with planes = N * C: every value is read a few times through L1 / L2 and every
// result written once, so these are streaming kernels like the axis reductions, and they keep the reference's
// arithmetic to the bit:
//   * max forward: one thread per output; the window is walked in the reference's order (rows, then columns, both in
//     steps of the dilation) with its strict `>` from -infinity, so a NaN never wins, the first of equal values stays,
//     and a window without a winner gives -infinity and index -1.  The index is the position inside the plane
//     (y * W + x) as a float, as the reference stores it.
//   * average forward: the window clipped as the reference clips it (first to the padded extent -- that is the pool
//     size when the padding counts -- then to the plane), a float sum from 0f in row-major order, one float division.
//   * gradients: the reference scatters with `+=`, sequentially per plane in output order (i, then j).  Here every INPUT
//     position gathers instead: it visits the outputs whose window can contain it in the same (i, j) order and adds
//     their contributions in float from 0f -- the same additions in the same order, so the sums are identical, with no
//     atomics and no dependence on scheduling.  For max pooling a contribution is gradOut[i, j] where the saved index
//     equals the position; for average pooling gradOut[i, j] / itemsInPool(i, j).
#include <math_constants.h>

#include "ktc_internal.hpp"

namespace ktc {

namespace {

struct PoolGeom { int H, W, OH, OW, kh, kw, ph, pw, sh, sw, dh, dw; };

__device__ __forceinline__ int ceil_div_pos(int a, int b) { return a <= 0 ? 0 : (a + b - 1) / b; }

__global__ void __launch_bounds__(256) k_pool_max_forward(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ idx,
                                                          int64_t planes, const PoolGeom g) {
    const int64_t per = (int64_t)g.OH * g.OW, total = planes * per;
    for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t p = o / per;
        const int r = (int)(o - p * per), i = r / g.OW, j = r - i * g.OW;
        int h0 = i * g.sh - g.ph, w0 = j * g.sw - g.pw;
        const int h1 = min(h0 + (g.kh - 1) * g.dh + 1, g.H), w1 = min(w0 + (g.kw - 1) * g.dw + 1, g.W);
        while (h0 < 0) h0 += g.dh;
        while (w0 < 0) w0 += g.dw;
        const float* plane = in + p * (int64_t)g.H * g.W;
        float best = -CUDART_INF_F, at = -1.0f;
        for (int y = h0; y < h1; y += g.dh)
            for (int x = w0; x < w1; x += g.dw) {
                const float v = __ldg(plane + y * g.W + x);
                if (v > best) { best = v; at = (float)(y * g.W + x); }
            }
        out[o] = best;
        idx[o] = at;
    }
}

// the reference's window of output (i, j): [h0, h1) x [w0, w1) inside the plane, and the number of items it divides by
struct AvgWindow { int h0, h1, w0, w1, items; };
__device__ __forceinline__ AvgWindow avg_window(const PoolGeom& g, int i, int j, bool include_padding) {
    AvgWindow a;
    int h0 = i * g.sh - g.ph, w0 = j * g.sw - g.pw;
    int h1 = min(h0 + g.kh, g.H + g.ph), w1 = min(w0 + g.kw, g.W + g.pw);
    const int pool = (h1 - h0) * (w1 - w0);
    a.h0 = max(h0, 0); a.w0 = max(w0, 0); a.h1 = min(h1, g.H); a.w1 = min(w1, g.W);
    a.items = include_padding ? pool : (a.h1 - a.h0) * (a.w1 - a.w0);
    return a;
}

__global__ void __launch_bounds__(256) k_pool_avg_forward(const float* __restrict__ in, float* __restrict__ out, int64_t planes, const PoolGeom g,
                                                          int include_padding) {
    const int64_t per = (int64_t)g.OH * g.OW, total = planes * per;
    for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t p = o / per;
        const int r = (int)(o - p * per), i = r / g.OW, j = r - i * g.OW;
        const AvgWindow a = avg_window(g, i, j, include_padding != 0);
        const float* plane = in + p * (int64_t)g.H * g.W;
        float sum = 0.f;
        for (int y = a.h0; y < a.h1; ++y)
            for (int x = a.w0; x < a.w1; ++x) sum = __fadd_rn(sum, __ldg(plane + y * g.W + x));
        out[o] = __fdiv_rn(sum, (float)a.items);
    }
}

// the outputs whose window can reach input row y (column x): i in [lo, hi]
__device__ __forceinline__ void reach(int y, int pad, int span, int stride, int n_out, int* lo, int* hi) {
    *lo = ceil_div_pos(y + pad - span + 1, stride);
    *hi = min((y + pad) / stride, n_out - 1);
}

__global__ void __launch_bounds__(256) k_pool_max_backward(const float* __restrict__ gout, const float* __restrict__ idx, float* __restrict__ gin,
                                                           int64_t planes, const PoolGeom g) {
    const int64_t per = (int64_t)g.H * g.W, total = planes * per;
    const int span_h = (g.kh - 1) * g.dh + 1, span_w = (g.kw - 1) * g.dw + 1;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t p = e / per;
        const int pos = (int)(e - p * per), y = pos / g.W, x = pos - y * g.W;
        int i0, i1, j0, j1;
        reach(y, g.ph, span_h, g.sh, g.OH, &i0, &i1);
        reach(x, g.pw, span_w, g.sw, g.OW, &j0, &j1);
        const int64_t base = p * (int64_t)g.OH * g.OW;
        float acc = 0.f;
        for (int i = i0; i <= i1; ++i)
            for (int j = j0; j <= j1; ++j) {
                const int64_t o = base + (int64_t)i * g.OW + j;
                if ((int)__ldg(idx + o) == pos) acc = __fadd_rn(acc, __ldg(gout + o));      // Float.toInt() of the saved index
            }
        gin[e] = acc;
    }
}

__global__ void __launch_bounds__(256) k_pool_avg_backward(const float* __restrict__ gout, float* __restrict__ gin, int64_t planes, const PoolGeom g,
                                                           int include_padding) {
    const int64_t per = (int64_t)g.H * g.W, total = planes * per;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t p = e / per;
        const int pos = (int)(e - p * per), y = pos / g.W, x = pos - y * g.W;
        int i0, i1, j0, j1;
        reach(y, g.ph, g.kh, g.sh, g.OH, &i0, &i1);
        reach(x, g.pw, g.kw, g.sw, g.OW, &j0, &j1);
        const int64_t base = p * (int64_t)g.OH * g.OW;
        float acc = 0.f;
        for (int i = i0; i <= i1; ++i)
            for (int j = j0; j <= j1; ++j) {
                const AvgWindow a = avg_window(g, i, j, include_padding != 0);
                if (y >= a.h0 && y < a.h1 && x >= a.w0 && x < a.w1)
                    acc = __fadd_rn(acc, __fdiv_rn(__ldg(gout + base + (int64_t)i * g.OW + j), (float)a.items));
            }
        gin[e] = acc;
    }
}

int read_geometry(const char* what, const int* geom, PoolGeom* g) {
    if (!geom) return fail(KTC_EINVAL, "%s: no geometry", what);
    *g = PoolGeom{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], geom[8], geom[9], geom[10], geom[11]};
    if (g->H < 1 || g->W < 1 || g->OH < 1 || g->OW < 1) return fail(KTC_EINVAL, "%s: extents %d x %d -> %d x %d", what, g->H, g->W, g->OH, g->OW);
    if (g->kh < 1 || g->kw < 1) return fail(KTC_EINVAL, "%s: Kernel size should be greater than zero", what);
    if (g->sh < 1 || g->sw < 1) return fail(KTC_EINVAL, "%s: Stride should be greater than zero", what);
    if (g->dh < 1 || g->dw < 1) return fail(KTC_EINVAL, "%s: Dilation should be greater than zero", what);
    if (g->ph < 0 || g->pw < 0 || g->ph > g->kh / 2 || g->pw > g->kw / 2)
        return fail(KTC_EINVAL, "%s: Padding should be smaller than kernel size / 2, but got kernel: (%d, %d) and padding: (%d, %d)", what, g->kh, g->kw, g->ph, g->pw);
    if ((int64_t)g->H * g->W > 0x7fffffffLL || (int64_t)g->OH * g->OW > 0x7fffffffLL || (int64_t)g->H * g->W >= (1 << 24))
        return fail(KTC_ENOTSUP, "%s: planes of %d x %d (positions inside a plane are kept as floats: at most 2^24)", what, g->H, g->W);
    // A last window that starts beyond the plane (possible with useCeil and no padding) is empty: the reference then writes
    // -infinity / index -1, or 0f divided by its item count; the kernels do the same and read nothing outside the plane.
    return KTC_OK;
}

int grid_for(Device* d, int64_t items) {
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = (int64_t)d->sm_count * 32;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

int finish_pool(const char* what) {
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

// resolves the buffers of a call: `small` tensors hold planes * OH * OW floats, `big` ones planes * H * W
int resolve_all(const char* what, int64_t planes, const PoolGeom& g, const ktc_buf* small, int n_small, const ktc_buf* big, int n_big, Buf* bs, Buf* bb) {
    if (planes < 0) return fail(KTC_EINVAL, "%s: %lld planes", what, (long long)planes);
    int dev = -1;
    for (int k = 0; k < n_small + n_big; ++k) {
        Buf* b = k < n_small ? &bs[k] : &bb[k - n_small];
        KTC_TRY(resolve(k < n_small ? small[k] : big[k - n_small], b));
        if (dev < 0) dev = b->dev;
        if (b->dev != dev) return fail(KTC_EINVAL, "%s: buffers live on different devices", what);
        const int64_t need = planes * (k < n_small ? (int64_t)g.OH * g.OW : (int64_t)g.H * g.W);
        if (b->n < need) return fail(KTC_EINVAL, "%s: a buffer holds %lld floats, %lld needed", what, (long long)b->n, (long long)need);
    }
    for (int a = 0; a < n_small + n_big; ++a)
        for (int c = a + 1; c < n_small + n_big; ++c) {
            const Buf& x = a < n_small ? bs[a] : bb[a - n_small];
            const Buf& y = c < n_small ? bs[c] : bb[c - n_small];
            if (x.ptr == y.ptr) return fail(KTC_EINVAL, "%s: two of the tensors alias", what);
        }
    return KTC_OK;
}

}  // namespace

}  // namespace ktc

using namespace ktc;

// geom: {H, W, OH, OW, kernelH, kernelW, paddingH, paddingW, strideH, strideW, dilationH, dilationW}; in [planes, H, W],
// out and indices [planes, OH, OW].  The output extents are the caller's (the reference computes them on floats with
// ceil or floor and then drops a last window that would start in the padding, JVMSpatialPoolingBase.kt:27-77).
extern "C" int ktc_pool2d_max(ktc_buf out, ktc_buf indices, ktc_buf in, int64_t planes, const int* geom) {
    PoolGeom g;
    KTC_TRY(read_geometry("ktc_pool2d_max", geom, &g));
    const ktc_buf small[2] = {out, indices};
    Buf bs[2], bb[1];
    KTC_TRY(resolve_all("ktc_pool2d_max", planes, g, small, 2, &in, 1, bs, bb));
    if (planes == 0) return KTC_OK;
    Device* d = device(bb[0].dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    k_pool_max_forward<<<grid_for(d, planes * g.OH * g.OW), 256, 0, d->stream>>>(bb[0].ptr, bs[0].ptr, bs[1].ptr, planes, g);
    return finish_pool("pool2d_max");
}

// grad_in [planes, H, W] from grad_out and the indices saved by ktc_pool2d_max, both [planes, OH, OW]
extern "C" int ktc_pool2d_max_grad(ktc_buf grad_in, ktc_buf grad_out, ktc_buf indices, int64_t planes, const int* geom) {
    PoolGeom g;
    KTC_TRY(read_geometry("ktc_pool2d_max_grad", geom, &g));
    const ktc_buf small[2] = {grad_out, indices};
    Buf bs[2], bb[1];
    KTC_TRY(resolve_all("ktc_pool2d_max_grad", planes, g, small, 2, &grad_in, 1, bs, bb));
    if (planes == 0) return KTC_OK;
    Device* d = device(bb[0].dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    k_pool_max_backward<<<grid_for(d, planes * g.H * g.W), 256, 0, d->stream>>>(bs[0].ptr, bs[1].ptr, bb[0].ptr, planes, g);
    return finish_pool("pool2d_max_grad");
}

// average pooling (no dilation: geom[10] and geom[11] must be 1); include_padding: the divisor is the window clipped to
// the padded extent instead of the number of values summed
extern "C" int ktc_pool2d_avg(ktc_buf out, ktc_buf in, int64_t planes, const int* geom, int include_padding) {
    PoolGeom g;
    KTC_TRY(read_geometry("ktc_pool2d_avg", geom, &g));
    if (g.dh != 1 || g.dw != 1) return fail(KTC_EINVAL, "ktc_pool2d_avg: average pooling has no dilation");
    Buf bs[1], bb[1];
    KTC_TRY(resolve_all("ktc_pool2d_avg", planes, g, &out, 1, &in, 1, bs, bb));
    if (planes == 0) return KTC_OK;
    Device* d = device(bb[0].dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    k_pool_avg_forward<<<grid_for(d, planes * g.OH * g.OW), 256, 0, d->stream>>>(bb[0].ptr, bs[0].ptr, planes, g, include_padding);
    return finish_pool("pool2d_avg");
}

extern "C" int ktc_pool2d_avg_grad(ktc_buf grad_in, ktc_buf grad_out, int64_t planes, const int* geom, int include_padding) {
    PoolGeom g;
    KTC_TRY(read_geometry("ktc_pool2d_avg_grad", geom, &g));
    if (g.dh != 1 || g.dw != 1) return fail(KTC_EINVAL, "ktc_pool2d_avg_grad: average pooling has no dilation");
    Buf bs[1], bb[1];
    KTC_TRY(resolve_all("ktc_pool2d_avg_grad", planes, g, &grad_out, 1, &grad_in, 1, bs, bb));
    if (planes == 0) return KTC_OK;
    Device* d = device(bb[0].dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    k_pool_avg_backward<<<grid_for(d, planes * g.H * g.W), 256, 0, d->stream>>>(bs[0].ptr, bb[0].ptr, planes, g, include_padding);
    return finish_pool("pool2d_avg_grad");
}
