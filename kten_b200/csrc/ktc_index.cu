// ktc_index.cu -- data movement of the raw-tensor SPI: slices, transposes / permutes, gather /
// scatter / index-select / index-add (JVMRawTensor.kt:227-353, 437-518).
//
// Everything here is index arithmetic plus one pass over memory, so the kernels are judged by
// how close that pass comes to the HBM rate:
//   * k_copy_nd          dst[doff + i.dstr] = src[soff + i.sstr] over an N-d box (get / set by
//                        ranges, narrow, concat pieces, permutes that keep the innermost axis):
//                        dimensions are collapsed on the host; when both sides are contiguous
//                        along the innermost axis and 16-byte aligned the element type is float4;
//   * k_transpose_tiled  when the two sides are contiguous along DIFFERENT axes (transpose,
//                        permutes that move the innermost axis) a 32x32 tile goes through shared
//                        memory so that both the read and the write are coalesced;
//   * k_gather_axis / k_index_select   one thread per output element;
//   * k_scatter_axis_nd / k_index_add  one thread per column (all coordinates but the axis),
//                        sequential along the axis: the reference's loops are sequential in the
//                        index position (JVM:234-246, 508-516), so duplicates resolve in the same
//                        order -- last write wins, additions are summed in index order.
// Index values are float32 (as every kten tensor); an out-of-range index sets the device error
// word instead of faulting, and the entry point reports it like the reference's exception.
#include "ktc_internal.hpp"

namespace ktc {

namespace {

struct NdArgs {
    int ndim;
    int64_t shape[KTC_MAX_DIMS], dstr[KTC_MAX_DIMS], sstr[KTC_MAX_DIMS];
    int64_t total;
};

inline int finish(const char* what) {
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

// T = float or float4; FILL: no source
template <class T, bool FILL>
__global__ void __launch_bounds__(256) k_copy_nd(T* __restrict__ dst, const T* __restrict__ src, const __grid_constant__ NdArgs a, T v) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= a.total) return;
    int64_t rem = i, doff = 0, soff = 0;
    #pragma unroll 1
    for (int d = a.ndim - 1; d > 0; --d) {
        const int64_t q = rem / a.shape[d], c = rem - q * a.shape[d];
        doff += c * a.dstr[d];
        if (!FILL) soff += c * a.sstr[d];
        rem = q;
    }
    doff += rem * a.dstr[0];
    if (!FILL) soff += rem * a.sstr[0];
    dst[doff] = FILL ? v : src[soff];
}

// src is contiguous along dimension P, dst along dimension Q (P != Q): tiles of 32 x 32 over (P, Q).
struct TrArgs {
    int ndim, P, Q;
    int64_t shape[KTC_MAX_DIMS], dstr[KTC_MAX_DIMS], sstr[KTC_MAX_DIMS];
    int64_t tiles_p, tiles_q;
};

__global__ void __launch_bounds__(256) k_transpose_tiled(float* __restrict__ dst, const float* __restrict__ src, const __grid_constant__ TrArgs a) {
    __shared__ float tile[32][33];
    int64_t b = blockIdx.x;
    const int64_t tp = b % a.tiles_p; b /= a.tiles_p;
    const int64_t tq = b % a.tiles_q; b /= a.tiles_q;
    int64_t doff = 0, soff = 0;                          // the remaining (batch) dimensions
    #pragma unroll 1
    for (int d = a.ndim - 1; d >= 0; --d) {
        if (d == a.P || d == a.Q) continue;
        const int64_t q = b / a.shape[d], c = b - q * a.shape[d];
        doff += c * a.dstr[d]; soff += c * a.sstr[d];
        b = q;
    }
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t p0 = tp * 32, q0 = tq * 32;
    #pragma unroll
    for (int k = 0; k < 4; ++k) {                        // read: tx runs along P (stride 1 in src)
        const int64_t p = p0 + tx, q = q0 + ty + k * 8;
        if (p < a.shape[a.P] && q < a.shape[a.Q]) tile[ty + k * 8][tx] = src[soff + p * a.sstr[a.P] + q * a.sstr[a.Q]];
    }
    __syncthreads();
    #pragma unroll
    for (int k = 0; k < 4; ++k) {                        // write: tx runs along Q (stride 1 in dst)
        const int64_t q = q0 + tx, p = p0 + ty + k * 8;
        if (p < a.shape[a.P] && q < a.shape[a.Q]) dst[doff + p * a.dstr[a.P] + q * a.dstr[a.Q]] = tile[tx][ty + k * 8];
    }
}

struct AxisArgs {
    int ndim, axis;
    int64_t ishape[KTC_MAX_DIMS];                        // iteration space: the index tensor's shape
    int64_t istr[KTC_MAX_DIMS], tstr[KTC_MAX_DIMS], sstr[KTC_MAX_DIMS];
    int64_t t_axis_len;                                  // extent of the addressed tensor along the axis
    int64_t total;                                       // gather: index volume; scatter: index volume / extent along axis
};

__global__ void __launch_bounds__(256) k_gather_axis(float* __restrict__ out, const float* __restrict__ in, const float* __restrict__ index,
                                                     const __grid_constant__ AxisArgs a, int* err) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= a.total) return;
    int64_t rem = i, toff = 0;
    #pragma unroll 1
    for (int d = a.ndim - 1; d >= 0; --d) {
        const int64_t q = rem / a.ishape[d], c = rem - q * a.ishape[d];
        if (d != a.axis) toff += c * a.tstr[d];
        rem = q;
    }
    const int idx = (int)index[i];                        // Float.toInt(): truncation
    if (idx < 0 || idx >= a.t_axis_len) { *err = 1; return; }
    out[i] = in[toff + idx * a.tstr[a.axis]];
}

// MODE 0: target[.., idx, ..] = src   1: += src   2: = constant
template <int MODE>
__global__ void __launch_bounds__(128) k_scatter_axis_nd(float* __restrict__ target, const float* __restrict__ index, const float* __restrict__ src,
                                                         const __grid_constant__ AxisArgs a, float constant, int* err) {
    const int64_t col = (int64_t)blockIdx.x * 128 + threadIdx.x;
    if (col >= a.total) return;
    int64_t rem = col, ioff = 0, toff = 0, soff = 0;
    #pragma unroll 1
    for (int d = a.ndim - 1; d >= 0; --d) {
        if (d == a.axis) continue;
        const int64_t q = rem / a.ishape[d], c = rem - q * a.ishape[d];
        ioff += c * a.istr[d]; toff += c * a.tstr[d]; soff += c * a.sstr[d];
        rem = q;
    }
    const int64_t n = a.ishape[a.axis];
    for (int64_t i = 0; i < n; ++i) {                     // sequential in the index position, as the reference
        const int idx = (int)index[ioff + i * a.istr[a.axis]];
        if (idx < 0 || idx >= a.t_axis_len) { *err = 1; return; }
        float* t = target + toff + idx * a.tstr[a.axis];
        if (MODE == 0) *t = src[soff + i * a.sstr[a.axis]];
        else if (MODE == 1) *t = __fadd_rn(*t, src[soff + i * a.sstr[a.axis]]);
        else *t = constant;
    }
}

__global__ void __launch_bounds__(256) k_index_select(float* __restrict__ out, const float* __restrict__ in, const float* __restrict__ index,
                                                      int64_t outer, int64_t A, int64_t n_idx, int64_t inner, int* err) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= outer * n_idx * inner) return;
    const int64_t n = i % inner, r = i / inner, k = r % n_idx, o = r / n_idx;
    const int idx = (int)index[k];
    if (idx < 0 || idx >= A) { *err = 1; return; }
    out[i] = in[(o * A + idx) * inner + n];
}

__global__ void __launch_bounds__(128) k_index_add(float* __restrict__ target, const float* __restrict__ index, const float* __restrict__ src,
                                                   float alpha, int64_t outer, int64_t A, int64_t n_idx, int64_t inner, int* err) {
    const int64_t col = (int64_t)blockIdx.x * 128 + threadIdx.x;
    if (col >= outer * inner) return;
    const int64_t n = col % inner, o = col / inner;
    for (int64_t k = 0; k < n_idx; ++k) {                 // sequential: repeated indices add up in index order (JVM:508-516)
        const int idx = (int)index[k];
        if (idx < 0 || idx >= A) { *err = 1; return; }
        float* t = target + (o * A + idx) * inner + n;
        *t = __fadd_rn(*t, __fmul_rn(src[(o * n_idx + k) * inner + n], alpha));
    }
}

// reads the device error word (set by a kernel that met an invalid index), clears it, waits
int take_index_error(Device* d, const char* what, int64_t axis_len, int axis) {
    int h = 0;
    KTC_CUDA(cudaMemcpyAsync(&h, d->err_flag, sizeof(int), cudaMemcpyDeviceToHost, d->stream));
    KTC_CUDA(cudaMemsetAsync(d->err_flag, 0, sizeof(int), d->stream));
    KTC_CUDA(cudaStreamSynchronize(d->stream));
    if (h != 0) return fail(KTC_EINVAL, "%s got invalid index, index value is out of bounds 0 and %lld at axis: %d", what, (long long)axis_len, axis);
    return KTC_OK;
}

int64_t grid_of(int64_t items, int per_block) { return (items + per_block - 1) / per_block; }

}  // namespace

// dst / src already offset; strides in elements; shape/strides of `ndim` dimensions
int launch_copy_nd(Device* d, float* dst, const int64_t* dstr, const float* src, const int64_t* sstr,
                   const int64_t* shape, int ndim, bool fill, float value) {
    // drop extent-1 dimensions, merge neighbours that are contiguous on both sides
    int64_t S[KTC_MAX_DIMS], DS[KTC_MAX_DIMS], SS[KTC_MAX_DIMS];
    int m = 0;
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) {
        total *= shape[i];
        if (shape[i] == 1) continue;
        const int64_t ss = fill ? 0 : sstr[i];
        if (m > 0 && DS[m - 1] == dstr[i] * shape[i] && (fill || SS[m - 1] == ss * shape[i])) {
            S[m - 1] *= shape[i]; DS[m - 1] = dstr[i]; SS[m - 1] = ss;
        } else {
            S[m] = shape[i]; DS[m] = dstr[i]; SS[m] = ss; ++m;
        }
    }
    if (total == 0) return KTC_OK;
    if (m == 0) { S[0] = 1; DS[0] = 1; SS[0] = 1; m = 1; }

    // two different contiguous axes: tiled transpose
    if (!fill && m >= 2 && tune("copy_force_generic", 0) == 0) {
        int P = -1, Q = -1;
        for (int i = m - 1; i >= 0; --i) { if (P < 0 && SS[i] == 1) P = i; if (Q < 0 && DS[i] == 1) Q = i; }
        if (P >= 0 && Q >= 0 && P != Q && S[P] >= 8 && S[Q] >= 8) {
            TrArgs a{};
            a.ndim = m; a.P = P; a.Q = Q;
            int64_t batch = 1;
            for (int i = 0; i < m; ++i) { a.shape[i] = S[i]; a.dstr[i] = DS[i]; a.sstr[i] = SS[i]; if (i != P && i != Q) batch *= S[i]; }
            a.tiles_p = (S[P] + 31) / 32; a.tiles_q = (S[Q] + 31) / 32;
            const int64_t grid = a.tiles_p * a.tiles_q * batch;
            if (grid <= 0x7fffffffLL) {
                k_transpose_tiled<<<(int)grid, 256, 0, d->stream>>>(dst, src, a);
                return finish("transpose_tiled");
            }
        }
    }

    NdArgs a{};
    a.ndim = m;
    for (int i = 0; i < m; ++i) { a.shape[i] = S[i]; a.dstr[i] = DS[i]; a.sstr[i] = SS[i]; }
    // float4 elements when the innermost axis is contiguous on both sides and everything is 16-byte aligned
    bool vec = DS[m - 1] == 1 && (fill || SS[m - 1] == 1) && S[m - 1] % 4 == 0 && aligned16(dst) && (fill || aligned16(src));
    for (int i = 0; i < m - 1 && vec; ++i) vec = DS[i] % 4 == 0 && (fill || SS[i] % 4 == 0);
    if (vec) {
        a.shape[m - 1] /= 4;
        for (int i = 0; i < m - 1; ++i) { a.dstr[i] /= 4; a.sstr[i] /= 4; }
        a.total = total / 4;
        const int64_t grid = grid_of(a.total, 256);
        if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
        const float4 v4 = make_float4(value, value, value, value);
        if (fill) k_copy_nd<float4, true><<<(int)grid, 256, 0, d->stream>>>(reinterpret_cast<float4*>(dst), nullptr, a, v4);
        else k_copy_nd<float4, false><<<(int)grid, 256, 0, d->stream>>>(reinterpret_cast<float4*>(dst), reinterpret_cast<const float4*>(src), a, v4);
        return finish("copy_nd(vec)");
    }
    a.total = total;
    const int64_t grid = grid_of(total, 256);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    if (fill) k_copy_nd<float, true><<<(int)grid, 256, 0, d->stream>>>(dst, nullptr, a, value);
    else k_copy_nd<float, false><<<(int)grid, 256, 0, d->stream>>>(dst, src, a, value);
    return finish("copy_nd");
}

static void row_major(const int64_t* shape, int n, int64_t* str) {
    int64_t st = 1;
    for (int i = n - 1; i >= 0; --i) { str[i] = st; st *= shape[i]; }
}

int launch_gather_axis(Device* d, float* out, const float* in, const int64_t* in_shape, const float* index,
                       const int64_t* index_shape, int ndim, int axis) {
    AxisArgs a{};
    a.ndim = ndim; a.axis = axis; a.t_axis_len = in_shape[axis];
    row_major(in_shape, ndim, a.tstr);
    row_major(index_shape, ndim, a.istr);
    a.total = 1;
    for (int i = 0; i < ndim; ++i) { a.ishape[i] = index_shape[i]; a.total *= index_shape[i]; }
    if (a.total == 0) return KTC_OK;
    const int64_t grid = grid_of(a.total, 256);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    k_gather_axis<<<(int)grid, 256, 0, d->stream>>>(out, in, index, a, d->err_flag);
    KTC_TRY(finish("gather_axis"));
    return take_index_error(d, "Gather", a.t_axis_len, axis);
}

int launch_scatter_axis_nd(Device* d, int mode, float* target, const int64_t* target_shape, const float* index,
                           const int64_t* index_shape, const float* src, const int64_t* src_shape, int ndim, int axis, float constant) {
    AxisArgs a{};
    a.ndim = ndim; a.axis = axis; a.t_axis_len = target_shape[axis];
    row_major(target_shape, ndim, a.tstr);
    row_major(index_shape, ndim, a.istr);
    if (src_shape) row_major(src_shape, ndim, a.sstr);
    a.total = 1;
    for (int i = 0; i < ndim; ++i) { a.ishape[i] = index_shape[i]; if (i != axis) a.total *= index_shape[i]; }
    if (a.total == 0 || index_shape[axis] == 0) return KTC_OK;
    const int64_t grid = grid_of(a.total, 128);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    if (mode == KTC_SCATTER_SET) k_scatter_axis_nd<0><<<(int)grid, 128, 0, d->stream>>>(target, index, src, a, constant, d->err_flag);
    else if (mode == KTC_SCATTER_ADD) k_scatter_axis_nd<1><<<(int)grid, 128, 0, d->stream>>>(target, index, src, a, constant, d->err_flag);
    else k_scatter_axis_nd<2><<<(int)grid, 128, 0, d->stream>>>(target, index, nullptr, a, constant, d->err_flag);
    KTC_TRY(finish("scatter_axis_nd"));
    return take_index_error(d, "Scatter", a.t_axis_len, axis);
}

int launch_index_select(Device* d, float* out, const float* in, const float* index, int64_t outer, int64_t A, int64_t n_idx, int64_t inner) {
    const int64_t total = outer * n_idx * inner;
    if (total == 0) return KTC_OK;
    const int64_t grid = grid_of(total, 256);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    k_index_select<<<(int)grid, 256, 0, d->stream>>>(out, in, index, outer, A, n_idx, inner, d->err_flag);
    KTC_TRY(finish("index_select"));
    return take_index_error(d, "Index select", A, -1);
}

int launch_index_add(Device* d, float* target, const float* index, const float* src, float alpha,
                     int64_t outer, int64_t A, int64_t n_idx, int64_t inner) {
    const int64_t cols = outer * inner;
    if (cols == 0 || n_idx == 0) return KTC_OK;
    const int64_t grid = grid_of(cols, 128);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    k_index_add<<<(int)grid, 128, 0, d->stream>>>(target, index, src, alpha, outer, A, n_idx, inner, d->err_flag);
    KTC_TRY(finish("index_add"));
    return take_index_error(d, "Index Add", A, -1);
}

}  // namespace ktc

using namespace ktc;

namespace {

struct Dev2 {
    Device* d = nullptr; int dev = -1;
    int take(const Buf& b, const char* who) {
        if (dev < 0) { dev = b.dev; d = device(b.dev); if (!d) return KTC_ESTATE; return use_device(d); }
        if (b.dev != dev) return fail(KTC_EINVAL, "%s: operands live on different devices (%d and %d)", who, dev, b.dev);
        return KTC_OK;
    }
};

// the box [offset, offset + sum (shape-1)*stride] must lie inside a buffer of n floats
int check_box(const char* who, const char* what, int64_t n, int64_t offset, const int64_t* strides, const int64_t* shape, int ndim, int64_t* volume) {
    if (ndim < 0 || ndim > KTC_MAX_DIMS || (ndim > 0 && (!shape || !strides))) return fail(KTC_EINVAL, "%s: bad shape of %s", who, what);
    if (offset < 0) return fail(KTC_EINVAL, "%s: negative offset into %s", who, what);
    int64_t last = offset, vol = 1;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] < 0 || strides[i] < 0) return fail(KTC_EINVAL, "%s: negative extent or stride of %s", who, what);
        vol *= shape[i];
        if (shape[i] > 0) last += (shape[i] - 1) * strides[i];
    }
    if (vol > 0 && last >= n) return fail(KTC_EINVAL, "%s: %s holds %lld floats, element %lld addressed", who, what, (long long)n, (long long)last);
    *volume = vol;
    return KTC_OK;
}

int check_dims(const char* who, const int64_t* shape, int ndim, int64_t* volume) {
    if (ndim < 1 || ndim > KTC_MAX_DIMS || !shape) return fail(KTC_EINVAL, "%s: bad shape", who);
    int64_t v = 1;
    for (int i = 0; i < ndim; ++i) { if (shape[i] < 0) return fail(KTC_EINVAL, "%s: negative extent", who); v *= shape[i]; }
    *volume = v;
    return KTC_OK;
}

}  // namespace

extern "C" int ktc_copy_strided(ktc_buf dst, int64_t dst_offset, const int64_t* dst_strides,
                                ktc_buf src, int64_t src_offset, const int64_t* src_strides,
                                const int64_t* shape, int ndim) {
    Buf bd, bs; KTC_TRY(resolve(dst, &bd)); KTC_TRY(resolve(src, &bs));
    Dev2 g; KTC_TRY(g.take(bd, "ktc_copy_strided")); KTC_TRY(g.take(bs, "ktc_copy_strided"));
    int64_t vd, vs;
    KTC_TRY(check_box("ktc_copy_strided", "dst", bd.n, dst_offset, dst_strides, shape, ndim, &vd));
    KTC_TRY(check_box("ktc_copy_strided", "src", bs.n, src_offset, src_strides, shape, ndim, &vs));
    if (vd == 0) return KTC_OK;
    if (bd.ptr == bs.ptr) return fail(KTC_EINVAL, "ktc_copy_strided: dst aliases src");
    return launch_copy_nd(g.d, bd.ptr + dst_offset, dst_strides, bs.ptr + src_offset, src_strides, shape, ndim, false, 0.f);
}

extern "C" int ktc_fill_strided(ktc_buf dst, int64_t dst_offset, const int64_t* dst_strides, const int64_t* shape, int ndim, float value) {
    Buf bd; KTC_TRY(resolve(dst, &bd));
    Dev2 g; KTC_TRY(g.take(bd, "ktc_fill_strided"));
    int64_t vd;
    KTC_TRY(check_box("ktc_fill_strided", "dst", bd.n, dst_offset, dst_strides, shape, ndim, &vd));
    if (vd == 0) return KTC_OK;
    return launch_copy_nd(g.d, bd.ptr + dst_offset, dst_strides, nullptr, nullptr, shape, ndim, true, value);
}

extern "C" int ktc_gather_axis(ktc_buf out, ktc_buf in, const int64_t* in_shape, ktc_buf index, const int64_t* index_shape, int ndim, int axis) {
    Buf bo, bi, bx; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(in, &bi)); KTC_TRY(resolve(index, &bx));
    Dev2 g; KTC_TRY(g.take(bo, "ktc_gather_axis")); KTC_TRY(g.take(bi, "ktc_gather_axis")); KTC_TRY(g.take(bx, "ktc_gather_axis"));
    int64_t vi, vx;
    KTC_TRY(check_dims("ktc_gather_axis(in)", in_shape, ndim, &vi)); KTC_TRY(check_dims("ktc_gather_axis(index)", index_shape, ndim, &vx));
    if (axis < 0 || axis >= ndim) return fail(KTC_EINVAL, "ktc_gather_axis: axis %d out of range", axis);
    for (int i = 0; i < ndim; ++i)
        if (i != axis && index_shape[i] > in_shape[i]) return fail(KTC_EINVAL, "ktc_gather_axis: index extent %lld exceeds input extent %lld at dimension %d", (long long)index_shape[i], (long long)in_shape[i], i);
    if (bi.n < vi || bx.n < vx || bo.n < vx) return fail(KTC_EINVAL, "ktc_gather_axis: a buffer is smaller than its shape");
    if (bo.ptr == bi.ptr || bo.ptr == bx.ptr) return fail(KTC_EINVAL, "ktc_gather_axis: out aliases an input");
    return launch_gather_axis(g.d, bo.ptr, bi.ptr, in_shape, bx.ptr, index_shape, ndim, axis);
}

extern "C" int ktc_scatter_axis_nd(int mode, ktc_buf target, const int64_t* target_shape, ktc_buf index, const int64_t* index_shape,
                                   ktc_buf src, const int64_t* src_shape, int ndim, int axis, float constant) {
    if (mode < KTC_SCATTER_SET || mode > KTC_SCATTER_CONST) return fail(KTC_EINVAL, "ktc_scatter_axis_nd: unknown mode %d", mode);
    Buf bt, bx, bs{}; KTC_TRY(resolve(target, &bt)); KTC_TRY(resolve(index, &bx));
    Dev2 g; KTC_TRY(g.take(bt, "ktc_scatter_axis_nd")); KTC_TRY(g.take(bx, "ktc_scatter_axis_nd"));
    int64_t vt, vx, vs = 0;
    KTC_TRY(check_dims("ktc_scatter_axis_nd(target)", target_shape, ndim, &vt)); KTC_TRY(check_dims("ktc_scatter_axis_nd(index)", index_shape, ndim, &vx));
    if (axis < 0 || axis >= ndim) return fail(KTC_EINVAL, "ktc_scatter_axis_nd: axis %d out of range", axis);
    if (mode != KTC_SCATTER_CONST) {
        KTC_TRY(resolve(src, &bs)); KTC_TRY(g.take(bs, "ktc_scatter_axis_nd"));
        KTC_TRY(check_dims("ktc_scatter_axis_nd(src)", src_shape, ndim, &vs));
        if (bs.n < vs) return fail(KTC_EINVAL, "ktc_scatter_axis_nd: src is smaller than its shape");
        if (bs.ptr == bt.ptr) return fail(KTC_EINVAL, "ktc_scatter_axis_nd: src aliases the target");
    }
    for (int i = 0; i < ndim; ++i) {                       // ShapeFunctions.kt:346-371
        if (mode != KTC_SCATTER_CONST && index_shape[i] > src_shape[i])
            return fail(KTC_EINVAL, "Scatter requires that index.shape[a] <= src.shape[a] for all axis 'a'");
        if (i != axis && index_shape[i] > target_shape[i])
            return fail(KTC_EINVAL, "Scatter requires that index.shape[a] <= target.shape[a] for all axis 'a', except the specified 'axis' of the operation");
    }
    if (bt.n < vt || bx.n < vx) return fail(KTC_EINVAL, "ktc_scatter_axis_nd: a buffer is smaller than its shape");
    if (bx.ptr == bt.ptr) return fail(KTC_EINVAL, "ktc_scatter_axis_nd: index aliases the target");
    return launch_scatter_axis_nd(g.d, mode, bt.ptr, target_shape, bx.ptr, index_shape, mode == KTC_SCATTER_CONST ? nullptr : bs.ptr,
                                  mode == KTC_SCATTER_CONST ? nullptr : src_shape, ndim, axis, constant);
}

extern "C" int ktc_index_select(ktc_buf out, ktc_buf in, ktc_buf index, int64_t outer, int64_t axis_len, int64_t n_index, int64_t inner) {
    if (outer < 0 || axis_len < 0 || n_index < 0 || inner < 0) return fail(KTC_EINVAL, "ktc_index_select: negative extent");
    Buf bo, bi, bx; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(in, &bi)); KTC_TRY(resolve(index, &bx));
    Dev2 g; KTC_TRY(g.take(bo, "ktc_index_select")); KTC_TRY(g.take(bi, "ktc_index_select")); KTC_TRY(g.take(bx, "ktc_index_select"));
    if (bi.n < outer * axis_len * inner || bx.n < n_index || bo.n < outer * n_index * inner) return fail(KTC_EINVAL, "ktc_index_select: a buffer is smaller than its shape");
    if (bo.ptr == bi.ptr || bo.ptr == bx.ptr) return fail(KTC_EINVAL, "ktc_index_select: out aliases an input");
    return launch_index_select(g.d, bo.ptr, bi.ptr, bx.ptr, outer, axis_len, n_index, inner);
}

extern "C" int ktc_index_add(ktc_buf target, ktc_buf index, ktc_buf src, float alpha, int64_t outer, int64_t axis_len, int64_t n_index, int64_t inner) {
    if (outer < 0 || axis_len < 0 || n_index < 0 || inner < 0) return fail(KTC_EINVAL, "ktc_index_add: negative extent");
    Buf bt, bx, bs; KTC_TRY(resolve(target, &bt)); KTC_TRY(resolve(index, &bx)); KTC_TRY(resolve(src, &bs));
    Dev2 g; KTC_TRY(g.take(bt, "ktc_index_add")); KTC_TRY(g.take(bx, "ktc_index_add")); KTC_TRY(g.take(bs, "ktc_index_add"));
    if (bt.n < outer * axis_len * inner || bx.n < n_index || bs.n < outer * n_index * inner) return fail(KTC_EINVAL, "ktc_index_add: a buffer is smaller than its shape");
    if (bt.ptr == bs.ptr || bt.ptr == bx.ptr) return fail(KTC_EINVAL, "ktc_index_add: the target aliases an input");
    return launch_index_add(g.d, bt.ptr, bx.ptr, bs.ptr, alpha, outer, axis_len, n_index, inner);
}
