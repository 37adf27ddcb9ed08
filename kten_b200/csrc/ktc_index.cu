// ktc_index.cu -- data movement of the raw-tensor SPI: slices, transposes / permutes, gather /
// scatter / index-select / index-add (JVMRawTensor.kt:227-353, 437-518).
//
// Everything here is index arithmetic plus one pass over memory, so what matters for these kernels is
// how close that pass comes to the HBM rate:
//   * k_copy_nd          dst[doff + i.dstr] = src[soff + i.sstr] over an N-d box (get / set by
//                        ranges, narrow, concat pieces, permutes that keep the innermost axis):
//                        dimensions are collapsed on the host; when both sides are contiguous
//                        along the innermost axis and 16-byte aligned the element type is float4;
//   * k_transpose_tiled  when the two sides are contiguous along DIFFERENT axes (transpose,
//                        permutes that move the innermost axis) a 64x64 tile goes through shared
//                        memory so that both the read and the write are coalesced;
//   * k_gather_axis / k_index_select   one thread per output element (or per four); a gather along the last
//                        axis stages each input row in shared memory so that DRAM sees every element once;
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

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<unsigned long long>(p) & 15ull) == 0; }

inline int finish(const char* what) {
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

// T = float or float4; FILL: no source; I = type of the linear index that is decomposed (32-bit when the
// box is small enough).  A thread moves U items, 256 apart, and issues all its loads before the first store; every
// element is touched once, hence the streaming hints.
template <class T, bool FILL, class I, int U>
__global__ void __launch_bounds__(256) k_copy_nd(T* __restrict__ dst, const T* __restrict__ src, const __grid_constant__ NdArgs a, T v) {
    const int64_t base = (int64_t)blockIdx.x * (256 * U) + threadIdx.x;
    int64_t doff[U], soff[U];
    #pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t i = base + u * 256;
        I rem = (I)(i < a.total ? i : 0);
        int64_t dd = 0, ss = 0;
        #pragma unroll 1
        for (int d = a.ndim - 1; d > 0; --d) {
            const I ext = (I)a.shape[d];
            const I q = rem / ext, c = rem - q * ext;
            dd += (int64_t)c * a.dstr[d];
            if (!FILL) ss += (int64_t)c * a.sstr[d];
            rem = q;
        }
        doff[u] = dd + (int64_t)rem * a.dstr[0];
        soff[u] = FILL ? 0 : ss + (int64_t)rem * a.sstr[0];
    }
    T val[U];
    #pragma unroll
    for (int u = 0; u < U; ++u) val[u] = FILL ? v : ((base + u * 256 < a.total) ? __ldcs(src + soff[u]) : v);
    #pragma unroll
    for (int u = 0; u < U; ++u) if (base + u * 256 < a.total) __stcs(dst + doff[u], val[u]);
}

// src is contiguous along dimension P, dst along dimension Q (P != Q): tiles of 64 x 64 over (P, Q); a thread
// holds 16 elements and issues all its loads before the first shared-memory store.
struct TrArgs {
    int ndim, P, Q;
    int64_t shape[KTC_MAX_DIMS], dstr[KTC_MAX_DIMS], sstr[KTC_MAX_DIMS];
    int64_t tiles_p, tiles_q;
};

constexpr int kTrTile = 64;

__global__ void __launch_bounds__(256) k_transpose_tiled(float* __restrict__ dst, const float* __restrict__ src, const __grid_constant__ TrArgs a) {
    __shared__ float tile[kTrTile][kTrTile + 1];
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
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;            // 64 x 4 threads, 16 rows each
    const int64_t p0 = tp * kTrTile, q0 = tq * kTrTile;
    const int64_t SP = a.shape[a.P], SQ = a.shape[a.Q];
    const float* sp = src + soff + (p0 + tx) * a.sstr[a.P] + (q0 + ty) * a.sstr[a.Q];
    float v[16];
    if (p0 + kTrTile <= SP && q0 + kTrTile <= SQ) {                       // whole tile: every load before the first use
        #pragma unroll
        for (int k = 0; k < 16; ++k) v[k] = __ldcs(sp + (int64_t)(k * 4) * a.sstr[a.Q]);
    } else {
        #pragma unroll
        for (int k = 0; k < 16; ++k) v[k] = (p0 + tx < SP && q0 + ty + k * 4 < SQ) ? sp[(int64_t)(k * 4) * a.sstr[a.Q]] : 0.f;
    }
    #pragma unroll
    for (int k = 0; k < 16; ++k) tile[ty + k * 4][tx] = v[k];              // tile[q][p]
    __syncthreads();
    float* dp = dst + doff + (q0 + tx) * a.dstr[a.Q] + (p0 + ty) * a.dstr[a.P];
    if (p0 + kTrTile <= SP && q0 + kTrTile <= SQ) {
        #pragma unroll
        for (int k = 0; k < 16; ++k) __stcs(dp + (int64_t)(k * 4) * a.dstr[a.P], tile[tx][ty + k * 4]);
    } else {
        #pragma unroll
        for (int k = 0; k < 16; ++k)
            if (q0 + tx < SQ && p0 + ty + k * 4 < SP) dp[(int64_t)(k * 4) * a.dstr[a.P]] = tile[tx][ty + k * 4];
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

// gather when the index covers the input off the axis: both are [outer, *, inner]; a thread produces four
// consecutive outputs (one 128-bit index load, four independent gathers, one 128-bit store)
template <class I>
__global__ void __launch_bounds__(256) k_gather_axis3(float* __restrict__ out, const float* __restrict__ in, const float* __restrict__ index,
                                                      I A_in, I A_idx, I inner, I total4, int* err) {
    const I t = (I)blockIdx.x * 256 + threadIdx.x;
    if (t >= total4) return;
    const I i = t * 4;
    const float4 iv = __ldcs(reinterpret_cast<const float4*>(index) + t);
    I n = i % inner, r = i / inner, k = r % A_idx, o = r / A_idx;
    const float idxf[4] = {iv.x, iv.y, iv.z, iv.w};
    float res[4];
    bool bad = false;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int idx = (int)idxf[j];
        const bool ok = idx >= 0 && (I)idx < A_in;
        bad |= !ok;
        res[j] = ok ? in[(o * A_in + (I)idx) * inner + n] : 0.f;
        if (++n == inner) { n = 0; if (++k == A_idx) { k = 0; ++o; } }
    }
    if (bad) { *err = 1; return; }
    __stcs(reinterpret_cast<float4*>(out) + t, make_float4(res[0], res[1], res[2], res[3]));
}

// gather along the LAST axis with rows that fit in shared memory: one CTA per row stages the input row
// with coalesced loads, then serves the row's random reads from shared memory, so DRAM sees every input,
// index and output element exactly once (the generic kernels above read 32-byte sectors for 4-byte values)
__global__ void __launch_bounds__(512) k_gather_lastaxis_smem(float* __restrict__ out, const float* __restrict__ in, const float* __restrict__ index,
                                                              int A_in, int A_idx, int* err) {
    extern __shared__ float row[];
    const int64_t o = blockIdx.x;
    const float* src = in + o * A_in;
    const float* idx = index + o * A_idx;
    float* dst = out + o * A_idx;
    if ((A_in & 3) == 0 && aligned16_dev(src)) {
        for (int i = threadIdx.x; i < A_in / 4; i += 512) reinterpret_cast<float4*>(row)[i] = __ldcs(reinterpret_cast<const float4*>(src) + i);
    } else {
        for (int i = threadIdx.x; i < A_in; i += 512) row[i] = src[i];
    }
    __syncthreads();
    bool bad = false;
    if ((A_idx & 3) == 0 && aligned16_dev(idx) && aligned16_dev(dst)) {
        for (int k = threadIdx.x; k < A_idx / 4; k += 512) {
            const float4 iv = __ldcs(reinterpret_cast<const float4*>(idx) + k);
            const int j0 = (int)iv.x, j1 = (int)iv.y, j2 = (int)iv.z, j3 = (int)iv.w;
            const bool ok = (unsigned)j0 < (unsigned)A_in && (unsigned)j1 < (unsigned)A_in && (unsigned)j2 < (unsigned)A_in && (unsigned)j3 < (unsigned)A_in;
            if (!ok) { bad = true; continue; }
            __stcs(reinterpret_cast<float4*>(dst) + k, make_float4(row[j0], row[j1], row[j2], row[j3]));
        }
    } else {
        for (int k = threadIdx.x; k < A_idx; k += 512) {
            const int j = (int)idx[k];
            if ((unsigned)j >= (unsigned)A_in) { bad = true; continue; }
            dst[k] = row[j];
        }
    }
    if (bad) *err = 1;
}

// index select with a vectorisable inner extent: a thread moves four float4 of the output, 256 apart,
// and issues its four row loads before the stores
template <class I>
__global__ void __launch_bounds__(256) k_index_select_vec(float4* __restrict__ out, const float4* __restrict__ in, const float* __restrict__ index,
                                                          I A, I n_idx, I inner4, I total4, int* err) {
    const I base = (I)blockIdx.x * 1024 + threadIdx.x;
    float4 v[4];
    bool bad = false;
    #pragma unroll
    for (int u = 0; u < 4; ++u) {
        const I t = base + (I)(u * 256);
        if (t < total4) {
            const I n = t % inner4, r = t / inner4, k = r % n_idx, o = r / n_idx;
            const int idx = (int)index[k];
            const bool ok = idx >= 0 && (I)idx < A;
            bad |= !ok;
            if (ok) v[u] = in[(o * A + (I)idx) * inner4 + n];
        }
    }
    if (bad) { *err = 1; return; }
    #pragma unroll
    for (int u = 0; u < 4; ++u) {
        const I t = base + (I)(u * 256);
        if (t < total4) __stcs(out + t, v[u]);
    }
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

// ---- index add with many indices ------------------------------------------------------------
// One thread per column and a sequential walk over the indices has no parallelism when the
// columns are few and the indices many (an embedding gradient: 10^5 indices, 10^3 columns).
// The indices are therefore grouped by target row first -- count per row, exclusive scan,
// placement, and a sort of each row's (short) list by index position -- and then every
// (row, column) element adds its sources in index-position order: the same additions in the
// same order as the sequential loop of the reference (JVM:508-516), fully parallel over rows.
struct IaStats { int err; int max_count; };

__global__ void __launch_bounds__(256) k_ia_count(const float* __restrict__ index, int64_t n_idx, int64_t A, int* __restrict__ count, IaStats* st) {
    const int64_t k = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (k >= n_idx) return;
    const int idx = (int)index[k];
    if (idx < 0 || idx >= A) { st->err = 1; return; }
    const int c = atomicAdd(&count[idx], 1) + 1;
    if (c > 1) atomicMax(&st->max_count, c);
}

// exclusive scan of count[0, A) in three steps over blocks of 1024 rows
__global__ void __launch_bounds__(1024) k_ia_block_sums(const int* __restrict__ count, int64_t A, int* __restrict__ bsum) {
    __shared__ int sm[32];
    const int64_t j = (int64_t)blockIdx.x * 1024 + threadIdx.x;
    int v = j < A ? count[j] : 0;
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        int t = sm[threadIdx.x];
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
        if (threadIdx.x == 0) bsum[blockIdx.x] = t;
    }
}
__global__ void __launch_bounds__(1024) k_ia_scan_block_sums(int* bsum, int64_t nb) {      // one CTA, 1024 values per round
    __shared__ int sm[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int carry = 0;
    for (int64_t base = 0; base < nb; base += 1024) {
        const int64_t b = base + threadIdx.x;
        const int c = b < nb ? bsum[b] : 0;
        int v = c;
        #pragma unroll
        for (int off = 1; off < 32; off <<= 1) { const int t = __shfl_up_sync(0xffffffffu, v, off); if (lane >= off) v += t; }
        if (lane == 31) sm[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int t = sm[lane];
            #pragma unroll
            for (int off = 1; off < 32; off <<= 1) { const int u = __shfl_up_sync(0xffffffffu, t, off); if (lane >= off) t += u; }
            sm[lane] = t;
        }
        __syncthreads();
        if (b < nb) bsum[b] = carry + v - c + (warp > 0 ? sm[warp - 1] : 0);
        carry += sm[31];
        __syncthreads();
    }
}
__global__ void __launch_bounds__(1024) k_ia_offsets(const int* __restrict__ count, int64_t A, const int* __restrict__ bsum,
                                                     int* __restrict__ offsets, int* __restrict__ cursor) {
    __shared__ int sm[32];
    const int64_t j = (int64_t)blockIdx.x * 1024 + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = j < A ? count[j] : 0;
    int v = c;                                                         // inclusive scan inside the warp
    #pragma unroll
    for (int off = 1; off < 32; off <<= 1) { const int t = __shfl_up_sync(0xffffffffu, v, off); if (lane >= off) v += t; }
    if (lane == 31) sm[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = sm[lane];
        #pragma unroll
        for (int off = 1; off < 32; off <<= 1) { const int u = __shfl_up_sync(0xffffffffu, t, off); if (lane >= off) t += u; }
        sm[lane] = t;
    }
    __syncthreads();
    const int excl = v - c + (warp > 0 ? sm[warp - 1] : 0) + bsum[blockIdx.x];
    if (j < A) { offsets[j] = excl; cursor[j] = excl; }
}
__global__ void __launch_bounds__(256) k_ia_place(const float* __restrict__ index, int64_t n_idx, int* __restrict__ cursor, int* __restrict__ perm) {
    const int64_t k = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (k >= n_idx) return;
    perm[atomicAdd(&cursor[(int)index[k]], 1)] = (int)k;
}
__global__ void __launch_bounds__(256) k_ia_sort_lists(const int* __restrict__ offsets, const int* __restrict__ count, int64_t A, int* __restrict__ perm) {
    const int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (j >= A) return;
    const int c = count[j];
    if (c < 2) return;
    int* p = perm + offsets[j];
    for (int a = 1; a < c; ++a) {                                       // insertion sort: the placement order is arbitrary, lists are short
        const int v = p[a];
        int b = a - 1;
        while (b >= 0 && p[b] > v) { p[b + 1] = p[b]; --b; }
        p[b + 1] = v;
    }
}
// one thread per (outer, row, float4 of columns) or per element when V == 1
template <class T>
__global__ void __launch_bounds__(256) k_ia_apply(T* __restrict__ target, const T* __restrict__ src, const int* __restrict__ offsets,
                                                  const int* __restrict__ count, const int* __restrict__ perm, float alpha,
                                                  int64_t outer, int64_t A, int64_t n_idx, int64_t innerT) {
    const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (t >= outer * A * innerT) return;
    const int64_t n = t % innerT, r = t / innerT, j = r % A, o = r / A;
    const int c = count[j];
    if (c == 0) return;
    const int* p = perm + offsets[j];
    T acc = target[t];
    for (int a = 0; a < c; ++a) {
        const T v = src[(o * n_idx + p[a]) * innerT + n];
        if constexpr (sizeof(T) == 16) {
            acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, alpha)); acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, alpha));
            acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, alpha)); acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, alpha));
        } else {
            acc = __fadd_rn(acc, __fmul_rn(v, alpha));
        }
    }
    target[t] = acc;
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
            a.tiles_p = (S[P] + kTrTile - 1) / kTrTile; a.tiles_q = (S[Q] + kTrTile - 1) / kTrTile;
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
        const bool u8 = tune("copy_unroll", 4) == 8;              // items per thread: 8 gains nothing on rows of 8 K floats and loses 12 % on 1 K rows
        const int64_t grid = grid_of(a.total, u8 ? 2048 : 1024);
        if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
        const float4 v4 = make_float4(value, value, value, value);
        float4* d4 = reinterpret_cast<float4*>(dst);
        const float4* s4 = reinterpret_cast<const float4*>(src);
        const bool small = a.total < (1LL << 31);
#define KTC_CP(FILL, I) do { if (u8) k_copy_nd<float4, FILL, I, 8><<<(int)grid, 256, 0, d->stream>>>(d4, FILL ? nullptr : s4, a, v4); \
                             else k_copy_nd<float4, FILL, I, 4><<<(int)grid, 256, 0, d->stream>>>(d4, FILL ? nullptr : s4, a, v4); } while (0)
        if (fill) { if (small) KTC_CP(true, uint32_t); else KTC_CP(true, int64_t); }
        else      { if (small) KTC_CP(false, uint32_t); else KTC_CP(false, int64_t); }
#undef KTC_CP
        return finish("copy_nd(vec)");
    }
    a.total = total;
    const int64_t grid = grid_of(total, 1024);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    const bool small = total < (1LL << 31);
    if (fill) { if (small) k_copy_nd<float, true, uint32_t, 4><<<(int)grid, 256, 0, d->stream>>>(dst, nullptr, a, value);
                else k_copy_nd<float, true, int64_t, 4><<<(int)grid, 256, 0, d->stream>>>(dst, nullptr, a, value); }
    else      { if (small) k_copy_nd<float, false, uint32_t, 4><<<(int)grid, 256, 0, d->stream>>>(dst, src, a, value);
                else k_copy_nd<float, false, int64_t, 4><<<(int)grid, 256, 0, d->stream>>>(dst, src, a, value); }
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
    bool covers = true;                                   // the index spans the input off the axis: [outer, *, inner] on both sides
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < ndim; ++i) {
        if (i == axis) continue;
        covers = covers && index_shape[i] == in_shape[i];
        if (i < axis) outer *= index_shape[i]; else inner *= index_shape[i];
    }
    const int64_t in_total = outer * in_shape[axis] * inner;
    // last axis, rows of 4 KB ... 160 KB: one CTA per row, the row staged in shared memory -- when the index picks at
    // least one element in eight (a direct read costs a 32-byte sector per element; fewer picks, such as the one target
    // per row of SoftmaxCrossEntropy, are cheaper read directly)
    if (covers && inner == 1 && in_shape[axis] >= 1024 && in_shape[axis] <= 40960 && index_shape[axis] < (1LL << 31) &&
        index_shape[axis] * 8 >= in_shape[axis] &&
        outer <= 0x7fffffffLL && tune("gather_smem", 1) != 0) {
        const size_t smem = (size_t)in_shape[axis] * sizeof(float);
        if (smem > 48 * 1024)                                       // per device: cheap enough to repeat
            KTC_CUDA(cudaFuncSetAttribute(k_gather_lastaxis_smem, cudaFuncAttributeMaxDynamicSharedMemorySize, 40960 * (int)sizeof(float)));
        k_gather_lastaxis_smem<<<(int)outer, 512, smem, d->stream>>>(out, in, index, (int)in_shape[axis], (int)index_shape[axis], d->idx_err);
        KTC_TRY(finish("gather_lastaxis_smem"));
        return take_index_error(d, "Gather", a.t_axis_len, axis);
    }
    if (covers && a.total % 4 == 0 && aligned16(index) && aligned16(out) && tune("index_force_generic", 0) == 0) {
        const int64_t total4 = a.total / 4, grid = grid_of(total4, 256);
        if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
        if (a.total < (1LL << 31) && in_total < (1LL << 31))
            k_gather_axis3<uint32_t><<<(int)grid, 256, 0, d->stream>>>(out, in, index, (uint32_t)in_shape[axis], (uint32_t)index_shape[axis],
                                                                        (uint32_t)inner, (uint32_t)total4, d->idx_err);
        else
            k_gather_axis3<int64_t><<<(int)grid, 256, 0, d->stream>>>(out, in, index, in_shape[axis], index_shape[axis], inner, total4, d->idx_err);
        KTC_TRY(finish("gather_axis3"));
        return take_index_error(d, "Gather", a.t_axis_len, axis);
    }
    const int64_t grid = grid_of(a.total, 256);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    k_gather_axis<<<(int)grid, 256, 0, d->stream>>>(out, in, index, a, d->idx_err);
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
    if (mode == KTC_SCATTER_SET) k_scatter_axis_nd<0><<<(int)grid, 128, 0, d->stream>>>(target, index, src, a, constant, d->idx_err);
    else if (mode == KTC_SCATTER_ADD) k_scatter_axis_nd<1><<<(int)grid, 128, 0, d->stream>>>(target, index, src, a, constant, d->idx_err);
    else k_scatter_axis_nd<2><<<(int)grid, 128, 0, d->stream>>>(target, index, nullptr, a, constant, d->idx_err);
    KTC_TRY(finish("scatter_axis_nd"));
    return take_index_error(d, "Scatter", a.t_axis_len, axis);
}

int launch_index_select(Device* d, float* out, const float* in, const float* index, int64_t outer, int64_t A, int64_t n_idx, int64_t inner) {
    const int64_t total = outer * n_idx * inner;
    if (total == 0) return KTC_OK;
    const int64_t grid = grid_of(total, 256);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    if (inner % 4 == 0 && aligned16(out) && aligned16(in) && tune("index_force_generic", 0) == 0) {
        const int64_t total4 = total / 4, g4 = grid_of(total4, 1024);
        if (total < (1LL << 31) && outer * A * inner < (1LL << 31))
            k_index_select_vec<uint32_t><<<(int)g4, 256, 0, d->stream>>>(reinterpret_cast<float4*>(out), reinterpret_cast<const float4*>(in), index,
                                                                         (uint32_t)A, (uint32_t)n_idx, (uint32_t)(inner / 4), (uint32_t)total4, d->idx_err);
        else
            k_index_select_vec<int64_t><<<(int)g4, 256, 0, d->stream>>>(reinterpret_cast<float4*>(out), reinterpret_cast<const float4*>(in), index,
                                                                        A, n_idx, inner / 4, total4, d->idx_err);
        KTC_TRY(finish("index_select(vec)"));
        return take_index_error(d, "Index select", A, -1);
    }
    k_index_select<<<(int)grid, 256, 0, d->stream>>>(out, in, index, outer, A, n_idx, inner, d->idx_err);
    KTC_TRY(finish("index_select"));
    return take_index_error(d, "Index select", A, -1);
}

int launch_index_add(Device* d, float* target, const float* index, const float* src, float alpha,
                     int64_t outer, int64_t A, int64_t n_idx, int64_t inner) {
    const int64_t cols = outer * inner;
    if (cols == 0 || n_idx == 0) return KTC_OK;
    // many indices: group them by target row (see above); else one thread per column
    if (n_idx >= tune("index_add_group_min", 64) && A < (1LL << 31) && n_idx < (1LL << 31)) {
        const int64_t nb = (A + 1023) / 1024;
        Scratch sc;                                                      // count | offsets | cursor | block sums | perm | stats
        KTC_TRY(sc.get(d, 3 * A + nb + n_idx + 2));
        int* count = reinterpret_cast<int*>(sc.ptr);
        int* offsets = count + A; int* cursor = offsets + A; int* bsum = cursor + A; int* perm = bsum + nb;
        IaStats* st = reinterpret_cast<IaStats*>(perm + n_idx);
        KTC_CUDA(cudaMemsetAsync(count, 0, sizeof(int) * A, d->stream));
        KTC_CUDA(cudaMemsetAsync(st, 0, sizeof(IaStats), d->stream));
        k_ia_count<<<(int)grid_of(n_idx, 256), 256, 0, d->stream>>>(index, n_idx, A, count, st);
        KTC_TRY(finish("index_add(count)"));
        IaStats h{};
        KTC_CUDA(cudaMemcpyAsync(&h, st, sizeof(IaStats), cudaMemcpyDeviceToHost, d->stream));
        KTC_CUDA(cudaStreamSynchronize(d->stream));
        if (h.err) return fail(KTC_EINVAL, "Index Add got invalid index, index value is out of bounds 0 and %lld", (long long)A);
        if (h.max_count <= tune("index_add_max_list", 256)) {
            k_ia_block_sums<<<(int)nb, 1024, 0, d->stream>>>(count, A, bsum);
            k_ia_scan_block_sums<<<1, 1024, 0, d->stream>>>(bsum, nb);
            k_ia_offsets<<<(int)nb, 1024, 0, d->stream>>>(count, A, bsum, offsets, cursor);
            k_ia_place<<<(int)grid_of(n_idx, 256), 256, 0, d->stream>>>(index, n_idx, cursor, perm);
            if (h.max_count > 1) k_ia_sort_lists<<<(int)grid_of(A, 256), 256, 0, d->stream>>>(offsets, count, A, perm);
            count_launch(h.max_count > 1 ? 4 : 3);
            if (inner % 4 == 0 && aligned16(target) && aligned16(src)) {
                const int64_t items = outer * A * (inner / 4);
                if (grid_of(items, 256) > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
                k_ia_apply<float4><<<(int)grid_of(items, 256), 256, 0, d->stream>>>(reinterpret_cast<float4*>(target), reinterpret_cast<const float4*>(src),
                                                                                    offsets, count, perm, alpha, outer, A, n_idx, inner / 4);
            } else {
                const int64_t items = outer * A * inner;
                if (grid_of(items, 256) > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
                k_ia_apply<float><<<(int)grid_of(items, 256), 256, 0, d->stream>>>(target, src, offsets, count, perm, alpha, outer, A, n_idx, inner);
            }
            return finish("index_add(apply)");
        }
        // a row with a very long list: the sequential walk below handles it (its columns are the parallelism)
    }
    const int64_t grid = grid_of(cols, 128);
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "tensor too large for one launch");
    k_index_add<<<(int)grid, 128, 0, d->stream>>>(target, index, src, alpha, outer, A, n_idx, inner, d->idx_err);
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
