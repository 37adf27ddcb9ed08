// ktc_pool.cu -- spatial (2-D) max and average pooling and their gradients (TensorOperations.spatialPooling,
// TensorOperations.kt:127; PoolingOperation.kt:5-15; kten-jvm: JVMSpatialMaxPooling.kt:24-69,
// JVMSpatialAvgPooling.kt:23-88; 1-D pooling is the same with a trailing extent of 1, TensorExtensions.kt:158-215).
//
// A window reduction over [planes, H, W] with planes = N * C: every value is read a few times through L1 / L2 and every
// result written once, so these are streaming kernels like the axis reductions, and they keep the reference's
// arithmetic to the bit:
//   * max forward: one thread per output (a CTA owns four output rows of a plane); the window is walked in the reference's order (rows, then columns, both in
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
struct PoolLaunchArgs { unsigned grid; dim3 block; cudaStream_t stream; const float* p0; float* p1; float* p2; PoolGeom g; int flag; };

__device__ __forceinline__ int ceil_div_pos(int a, int b) { return a <= 0 ? 0 : (a + b - 1) / b; }

// Work decomposition shared by the four kernels: a CTA of bx x by = 256 threads (bx: a power of two that covers a row's
// items -- outputs for the forward kernels, groups of four input positions for the gradients -- up to 64) owns
// by * kRowsPerThread consecutive rows of one plane; threadIdx.y picks the row, threadIdx.x strides over the row.  The
// only division by a run-time value per CTA is plane = blockIdx / tiles.
constexpr int kRowsPerThread = 4;
struct Tile { int64_t plane; int row0; };
__device__ __forceinline__ Tile tile_of(int rows_per_plane) {
    const int per_cta = blockDim.y * kRowsPerThread;
    const int tiles = (rows_per_plane + per_cta - 1) / per_cta;
    Tile t;
    t.plane = blockIdx.x / tiles;
    t.row0 = (int)(blockIdx.x - t.plane * tiles) * per_cta + threadIdx.y;
    return t;
}
#define KTC_POOL_ROWS(var, limit) for (int var = t.row0, r_ = 0; r_ < kRowsPerThread && var < (limit); ++r_, var += blockDim.y)

__global__ void __launch_bounds__(256) k_pool_max_forward(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ idx, const PoolGeom g) {
    const Tile t = tile_of(g.OH);
    const float* plane = in + t.plane * (int64_t)g.H * g.W;
    KTC_POOL_ROWS(i, g.OH) {
    int h0 = i * g.sh - g.ph;
    const int h1 = min(h0 + (g.kh - 1) * g.dh + 1, g.H);
    while (h0 < 0) h0 += g.dh;
    const int64_t orow = (t.plane * g.OH + i) * (int64_t)g.OW;
    for (int j = threadIdx.x; j < g.OW; j += blockDim.x) {
        int w0 = j * g.sw - g.pw;
        const int w1 = min(w0 + (g.kw - 1) * g.dw + 1, g.W);
        while (w0 < 0) w0 += g.dw;
        float best = -CUDART_INF_F;
        int at = -1;
        for (int y = h0; y < h1; y += g.dh)
            for (int x = w0; x < w1; x += g.dw) {
                const float v = __ldg(plane + y * g.W + x);
                if (v > best) { best = v; at = y * g.W + x; }
            }
        __stcs(out + orow + j, best);
        __stcs(idx + orow + j, (float)at);
    }
    }
}

// the reference's window of output (i, j): [h0, h1) x [w0, w1) inside the plane, and the number of items it divides by
struct AvgSpan { int lo, hi, padded; };                      // clipped to the plane; `padded`: its length clipped to the padded extent only
__device__ __forceinline__ AvgSpan avg_span(int o, int stride, int pad, int kernel, int extent) {
    const int a = o * stride - pad, b = min(a + kernel, extent + pad);
    AvgSpan s;
    s.padded = b - a; s.lo = max(a, 0); s.hi = min(b, extent);
    return s;
}
// x / items in float: a power of two (the 2 x 2 and 4 x 4 windows) divides exactly as a multiplication by its reciprocal --
// both are roundings of the same real number, subnormal quotients included
__device__ __forceinline__ float div_items(float x, int items) {
    if (items > 0 && (items & (items - 1)) == 0) return __fmul_rn(x, __int_as_float((96 + __clz(items)) << 23));      // 2^-(31 - clz)
    return __fdiv_rn(x, (float)items);
}
__device__ __forceinline__ int avg_items(const AvgSpan& h, const AvgSpan& w, bool include_padding) {
    return include_padding ? h.padded * w.padded : (h.hi - h.lo) * (w.hi - w.lo);
}

__global__ void __launch_bounds__(256) k_pool_avg_forward(const float* __restrict__ in, float* __restrict__ out, const PoolGeom g, int include_padding) {
    const Tile t = tile_of(g.OH);
    const float* plane = in + t.plane * (int64_t)g.H * g.W;
    KTC_POOL_ROWS(i, g.OH) {
    const AvgSpan h = avg_span(i, g.sh, g.ph, g.kh, g.H);
    const int64_t orow = (t.plane * g.OH + i) * (int64_t)g.OW;
    for (int j = threadIdx.x; j < g.OW; j += blockDim.x) {
        const AvgSpan w = avg_span(j, g.sw, g.pw, g.kw, g.W);
        float sum = 0.f;
        for (int y = h.lo; y < h.hi; ++y)
            for (int x = w.lo; x < w.hi; ++x) sum = __fadd_rn(sum, __ldg(plane + y * g.W + x));
        __stcs(out + orow + j, div_items(sum, avg_items(h, w, include_padding != 0)));
    }
    }
}

// the outputs whose window can reach input row y (column x): i in [lo, hi]
__device__ __forceinline__ void reach(int y, int pad, int span, int stride, int n_out, int* lo, int* hi) {
    *lo = ceil_div_pos(y + pad - span + 1, stride);
    *hi = min((y + pad) / stride, n_out - 1);
}

// Gradients: a thread owns four neighbouring input positions (y, x0 .. x0 + 3).  It walks the outputs that can reach any
// of them in (i, j) order once and hands every contribution to the position it belongs to, so each position still sees
// its own contributions in output order.
__global__ void __launch_bounds__(256) k_pool_max_backward(const float* __restrict__ gout, const float* __restrict__ idx, float* __restrict__ gin, const PoolGeom g) {
    const Tile t = tile_of(g.H);
    const int span_h = (g.kh - 1) * g.dh + 1, span_w = (g.kw - 1) * g.dw + 1;
    const int64_t obase = t.plane * (int64_t)g.OH * g.OW;
    const bool vec = (g.W & 3) == 0 && (reinterpret_cast<uintptr_t>(gin) & 15) == 0;
    KTC_POOL_ROWS(y, g.H) {
    int i0, i1;
    reach(y, g.ph, span_h, g.sh, g.OH, &i0, &i1);
    float* row = gin + (t.plane * g.H + y) * (int64_t)g.W;
    for (int x0 = threadIdx.x * 4; x0 < g.W; x0 += 4 * blockDim.x) {
        int j0, j1, unused;
        reach(x0, g.pw, span_w, g.sw, g.OW, &j0, &unused);
        reach(min(x0 + 3, g.W - 1), g.pw, span_w, g.sw, g.OW, &unused, &j1);
        const int pos0 = y * g.W + x0;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = i0; i <= i1; ++i) {
            const int64_t o = obase + (int64_t)i * g.OW;
            for (int j = j0; j <= j1; ++j) {
                const unsigned k = (unsigned)((int)__ldg(idx + o + j) - pos0);      // Float.toInt() of the saved position
                if (k < 4u) {
                    const float v = __ldg(gout + o + j);
                    #pragma unroll
                    for (int c = 0; c < 4; ++c) if (k == (unsigned)c) acc[c] = __fadd_rn(acc[c], v);
                }
            }
        }
        if (vec) __stcs(reinterpret_cast<float4*>(row + x0), make_float4(acc[0], acc[1], acc[2], acc[3]));
        else
            for (int c = 0; c < 4 && x0 + c < g.W; ++c) row[x0 + c] = acc[c];
    }
    }
}

__global__ void __launch_bounds__(256) k_pool_avg_backward(const float* __restrict__ gout, float* __restrict__ gin, const PoolGeom g, int include_padding) {
    const Tile t = tile_of(g.H);
    const int64_t obase = t.plane * (int64_t)g.OH * g.OW;
    const bool vec = (g.W & 3) == 0 && (reinterpret_cast<uintptr_t>(gin) & 15) == 0;
    KTC_POOL_ROWS(y, g.H) {
    int i0, i1;
    reach(y, g.ph, g.kh, g.sh, g.OH, &i0, &i1);
    float* row = gin + (t.plane * g.H + y) * (int64_t)g.W;
    for (int x0 = threadIdx.x * 4; x0 < g.W; x0 += 4 * blockDim.x) {
        int j0, j1, unused;
        reach(x0, g.pw, g.kw, g.sw, g.OW, &j0, &unused);
        reach(min(x0 + 3, g.W - 1), g.pw, g.kw, g.sw, g.OW, &unused, &j1);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = i0; i <= i1; ++i) {
            const AvgSpan h = avg_span(i, g.sh, g.ph, g.kh, g.H);
            if (y < h.lo || y >= h.hi) continue;
            const int64_t o = obase + (int64_t)i * g.OW;
            for (int j = j0; j <= j1; ++j) {
                const AvgSpan w = avg_span(j, g.sw, g.pw, g.kw, g.W);
                const float c = div_items(__ldg(gout + o + j), avg_items(h, w, include_padding != 0));
                #pragma unroll
                for (int k = 0; k < 4; ++k) if (x0 + k >= w.lo && x0 + k < w.hi) acc[k] = __fadd_rn(acc[k], c);
            }
        }
        if (vec) __stcs(reinterpret_cast<float4*>(row + x0), make_float4(acc[0], acc[1], acc[2], acc[3]));
        else
            for (int c = 0; c < 4 && x0 + c < g.W; ++c) row[x0 + c] = acc[c];
    }
    }
}

// ---- square windows of 2 or 3 with stride 1 or 2 and no dilation: the same arithmetic with compile-time trip counts ----
// In the kernels above a window is a run-time loop whose every iteration loads a value and uses it at once: the loads of a
// thread go out one at a time.  With K and S known the loops unroll, every load of a thread's four rows is issued before
// the first comparison, and positions outside the plane take a neutral value instead of a branch: -infinity never wins
// the strict `>`, and +0f added to a sum that started at +0f changes nothing.
template <int K, int S, bool IS_MAX>
__global__ void __launch_bounds__(256) k_pool_forward_ks(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ idx, const PoolGeom g,
                                                         int include_padding) {
    constexpr int RT = K == 2 ? 4 : 2;                       // rows whose loads are issued together (9 values per row for K = 3)
    const Tile t = tile_of(g.OH);
    const float* plane = in + t.plane * (int64_t)g.H * g.W;
    float* oplane = out + t.plane * (int64_t)g.OH * g.OW;
    float* iplane = IS_MAX ? idx + t.plane * (int64_t)g.OH * g.OW : nullptr;
    for (int j = threadIdx.x; j < g.OW; j += blockDim.x) {
        const int xa = j * S - g.pw;
        bool xok[K];                                         // a window position is inside the plane if its row and its column are
        #pragma unroll
        for (int b = 0; b < K; ++b) xok[b] = (unsigned)(xa + b) < (unsigned)g.W;
        #pragma unroll 1
        for (int rb = 0; rb < kRowsPerThread; rb += RT) {
            float v[RT][K][K];
            #pragma unroll
            for (int r = 0; r < RT; ++r) {
                const int i = t.row0 + (rb + r) * blockDim.y, ya = i * S - g.ph;
                const float* corner = plane + ya * g.W + xa;  // may lie outside the plane: only dereferenced where yok && xok
                #pragma unroll
                for (int a = 0; a < K; ++a) {
                    const bool yok = i < g.OH && (unsigned)(ya + a) < (unsigned)g.H;
                    #pragma unroll
                    for (int b = 0; b < K; ++b)
                        v[r][a][b] = (yok && xok[b]) ? __ldg(corner + a * g.W + b) : (IS_MAX ? -CUDART_INF_F : 0.f);
                }
            }
            #pragma unroll
            for (int r = 0; r < RT; ++r) {
                const int i = t.row0 + (rb + r) * blockDim.y, ya = i * S - g.ph;
                if (i >= g.OH) break;
                const int o = i * g.OW + j;
                if (IS_MAX) {
                    float best = -CUDART_INF_F;
                    int at = -1;
                    #pragma unroll
                    for (int a = 0; a < K; ++a) {
                        #pragma unroll
                        for (int b = 0; b < K; ++b)
                            if (v[r][a][b] > best) { best = v[r][a][b]; at = (ya + a) * g.W + xa + b; }
                    }
                    __stcs(oplane + o, best);
                    __stcs(iplane + o, (float)at);
                } else {
                    const AvgSpan h = avg_span(i, S, g.ph, K, g.H), w = avg_span(j, S, g.pw, K, g.W);
                    float sum = 0.f;
                    #pragma unroll
                    for (int a = 0; a < K; ++a) {
                        #pragma unroll
                        for (int b = 0; b < K; ++b) sum = __fadd_rn(sum, v[r][a][b]);
                    }
                    __stcs(oplane + o, div_items(sum, avg_items(h, w, include_padding != 0)));
                }
            }
        }
    }
}

template <int K, int S, bool IS_MAX>
__global__ void __launch_bounds__(256) k_pool_backward_ks(const float* __restrict__ gout, const float* __restrict__ idx, float* __restrict__ gin, const PoolGeom g,
                                                          int include_padding) {
    constexpr int NI = (K + S - 1) / S;                      // outputs that can reach one input row
    constexpr int NJ = (K + 2) / S + 1;                      // ... four neighbouring input columns
    const Tile t = tile_of(g.H);
    const float* gp = gout + t.plane * (int64_t)g.OH * g.OW;      // offsets inside a plane fit 32 bits (read_geometry)
    const float* ip = idx + t.plane * (int64_t)g.OH * g.OW;
    float* plane_in = gin + t.plane * (int64_t)g.H * g.W;
    const bool vec = (g.W & 3) == 0 && (reinterpret_cast<uintptr_t>(gin) & 15) == 0;
    if (!IS_MAX && K == S && g.ph == 0 && g.pw == 0 && g.H == g.OH * K && g.W == g.OW * K && vec) {
        // average pooling whose windows tile the plane exactly: every position lies in ONE window of K * K items, so its
        // gradient is 0f + gradOut / (K * K) -- what the general walk below computes, without the walk
        KTC_POOL_ROWS(y, g.H) {
            const float* grow = gp + (y / K) * g.OW;
            float* row = plane_in + y * g.W;
            for (int x0 = threadIdx.x * 4; x0 < g.W; x0 += 4 * blockDim.x) {
                float r[4];
                #pragma unroll
                for (int c = 0; c < 4; ++c) r[c] = __fadd_rn(0.f, div_items(__ldg(grow + (x0 + c) / K), K * K));
                __stcs(reinterpret_cast<float4*>(row + x0), make_float4(r[0], r[1], r[2], r[3]));
            }
        }
        return;
    }
    for (int x0 = threadIdx.x * 4; x0 < g.W; x0 += 4 * blockDim.x) {
        int j0, j1, unused;                                  // the same for every row of the thread
        reach(x0, g.pw, K, S, g.OW, &j0, &unused);
        reach(min(x0 + 3, g.W - 1), g.pw, K, S, g.OW, &unused, &j1);
        AvgSpan wsp[NJ];                                     // average: the column spans of the outputs in reach, also the same for every row
        #pragma unroll
        for (int b = 0; b < NJ; ++b) wsp[b] = avg_span(j0 + b, S, g.pw, K, g.W);
        KTC_POOL_ROWS(y, g.H) {
            int i0, i1;
            reach(y, g.ph, K, S, g.OH, &i0, &i1);
            float go[NI][NJ], ix[NI][NJ];
            #pragma unroll
            for (int a = 0; a < NI; ++a) {
                const bool rok = i0 + a <= i1;
                const int orow = (i0 + a) * g.OW + j0;
                #pragma unroll
                for (int b = 0; b < NJ; ++b) {
                    const bool ok = rok && j0 + b <= j1;
                    const int o = ok ? orow + b : 0;
                    go[a][b] = __ldg(gp + o);
                    // max: an output outside the range takes a position no input has; average: it contributes through `ok` below
                    ix[a][b] = IS_MAX ? (ok ? __ldg(ip + o) : -2.0f) : (ok ? 1.0f : 0.0f);
                }
            }
            // positions are integers below 2^24 kept as floats: comparing the floats is comparing the positions
            const float p0 = (float)(y * g.W + x0), p1 = p0 + 1.f, p2 = p0 + 2.f, p3 = p0 + 3.f;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            #pragma unroll
            for (int a = 0; a < NI; ++a) {
                #pragma unroll
                for (int b = 0; b < NJ; ++b) {
                    if (IS_MAX) {
                        const float at = ix[a][b];               // Float.toInt() of the saved position, compared as a float
                        if (at == p0) acc[0] = __fadd_rn(acc[0], go[a][b]);
                        if (at == p1) acc[1] = __fadd_rn(acc[1], go[a][b]);
                        if (at == p2) acc[2] = __fadd_rn(acc[2], go[a][b]);
                        if (at == p3) acc[3] = __fadd_rn(acc[3], go[a][b]);
                    } else {
                        if (ix[a][b] == 0.0f) continue;
                        const AvgSpan h = avg_span(i0 + a, S, g.ph, K, g.H);
                        const AvgSpan& w = wsp[b];
                        if (y < h.lo || y >= h.hi) continue;
                        const float c = div_items(go[a][b], avg_items(h, w, include_padding != 0));
                        #pragma unroll
                        for (int k = 0; k < 4; ++k) if (x0 + k >= w.lo && x0 + k < w.hi) acc[k] = __fadd_rn(acc[k], c);
                    }
                }
            }
            float* row = plane_in + y * g.W;
            if (vec) __stcs(reinterpret_cast<float4*>(row + x0), make_float4(acc[0], acc[1], acc[2], acc[3]));
            else
                for (int c = 0; c < 4 && x0 + c < g.W; ++c) row[x0 + c] = acc[c];
        }
    }
}

// 0: no specialised kernel for this geometry; else K * 10 + S
int fast_shape(const PoolGeom& g) {
    if (g.kh != g.kw || g.sh != g.sw || g.dh != 1 || g.dw != 1 || !tune("pool_fast", 1)) return 0;
    if ((g.kh == 2 || g.kh == 3) && (g.sh == 1 || g.sh == 2)) return g.kh * 10 + g.sh;
    return 0;
}

template <bool IS_MAX>
bool launch_fast_forward(int shape, const PoolLaunchArgs& a) {
    switch (shape) {
    case 22: k_pool_forward_ks<2, 2, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    case 21: k_pool_forward_ks<2, 1, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    case 32: k_pool_forward_ks<3, 2, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    case 31: k_pool_forward_ks<3, 1, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    }
    return false;
}
template <bool IS_MAX>
bool launch_fast_backward(int shape, const PoolLaunchArgs& a) {
    switch (shape) {
    case 22: k_pool_backward_ks<2, 2, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    case 21: k_pool_backward_ks<2, 1, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    case 32: k_pool_backward_ks<3, 2, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    case 31: k_pool_backward_ks<3, 1, IS_MAX><<<a.grid, a.block, 0, a.stream>>>(a.p0, a.p1, a.p2, a.g, a.flag); return true;
    }
    return false;
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

// CTA shape for rows of `items` items and the grid for planes x rows; grid 0: more than a launch takes
struct PoolLaunch { dim3 block; int64_t grid; };
PoolLaunch launch_for(int64_t planes, int rows, int items) {
    int bx = 8;
    while (bx < 64 && bx < items) bx <<= 1;
    PoolLaunch l;
    l.block = dim3(bx, 256 / bx);
    const int per_cta = (256 / bx) * kRowsPerThread;
    const int64_t blocks = planes * ((rows + per_cta - 1) / per_cta);
    l.grid = blocks > 0x7fffffffLL ? 0 : blocks;
    return l;
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
    const PoolLaunch pl = launch_for(planes, g.OH, g.OW); const int64_t grid = pl.grid;
    if (!grid) return fail(KTC_ENOTSUP, "ktc_pool2d_max: tensor too large for one launch");
    if (!launch_fast_forward<true>(fast_shape(g), PoolLaunchArgs{(unsigned)grid, pl.block, d->stream, bb[0].ptr, bs[0].ptr, bs[1].ptr, g, 0}))
        k_pool_max_forward<<<(unsigned)grid, pl.block, 0, d->stream>>>(bb[0].ptr, bs[0].ptr, bs[1].ptr, g);
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
    const PoolLaunch pl = launch_for(planes, g.H, (g.W + 3) / 4); const int64_t grid = pl.grid;
    if (!grid) return fail(KTC_ENOTSUP, "ktc_pool2d_max_grad: tensor too large for one launch");
    if (!launch_fast_backward<true>(fast_shape(g), PoolLaunchArgs{(unsigned)grid, pl.block, d->stream, bs[0].ptr, bs[1].ptr, bb[0].ptr, g, 0}))
        k_pool_max_backward<<<(unsigned)grid, pl.block, 0, d->stream>>>(bs[0].ptr, bs[1].ptr, bb[0].ptr, g);
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
    const PoolLaunch pl = launch_for(planes, g.OH, g.OW); const int64_t grid = pl.grid;
    if (!grid) return fail(KTC_ENOTSUP, "ktc_pool2d_avg: tensor too large for one launch");
    if (!launch_fast_forward<false>(fast_shape(g), PoolLaunchArgs{(unsigned)grid, pl.block, d->stream, bb[0].ptr, bs[0].ptr, nullptr, g, include_padding}))
        k_pool_avg_forward<<<(unsigned)grid, pl.block, 0, d->stream>>>(bb[0].ptr, bs[0].ptr, g, include_padding);
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
    const PoolLaunch pl = launch_for(planes, g.H, (g.W + 3) / 4); const int64_t grid = pl.grid;
    if (!grid) return fail(KTC_ENOTSUP, "ktc_pool2d_avg_grad: tensor too large for one launch");
    if (!launch_fast_backward<false>(fast_shape(g), PoolLaunchArgs{(unsigned)grid, pl.block, d->stream, bs[0].ptr, nullptr, bb[0].ptr, g, include_padding}))
        k_pool_avg_backward<<<(unsigned)grid, pl.block, 0, d->stream>>>(bs[0].ptr, bb[0].ptr, g, include_padding);
    return finish_pool("pool2d_avg_grad");
}
