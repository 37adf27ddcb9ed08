// ktc_elementwise.cu -- contiguous and broadcast elementwise kernels (sm_100a).
//
// All of these are HBM-bandwidth kernels: every thread moves 128-bit vectors,
// issues all the loads of its tile before the first use (several independent
// 16-byte requests in flight per thread), reads with the streaming hint
// (ld.global.cs / evict-first: each element is used once) and writes with
// st.global.cs.  Nothing here is a contraction, so there is no tensor-core path.
//
//   map1  : out[i] = f(a[i])            unary maps, tensor-constant ops, clamp, compares
//   map2  : out[i] = f(a[i], b[i])      same-shape binary ops (also in place, out == a)
//   bcast : out[i0,i1,i2] = f(A, B)     broadcast binary ops on the collapsed 3-D view;
//           an operand is read directly (row base + i2), as one scalar per row
//           (inner stride 0), or from a row vector staged once per tile in
//           shared memory (broadcast along the middle dimension).  The
//           broadcast operand is never materialised in global memory
//           (the reference writes and re-reads a full-size copy:
//           JVMRawTensor.kt:51-73, kernels.cl:44-70).
#include "ktc_map.cuh"
#include "ktc_math_more.cuh"

namespace ktc {

__global__ void __launch_bounds__(256) k_fill_vec(float4* __restrict__ out, int64_t n4, float v) {
    const float4 vv = make_float4(v, v, v, v);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x)
        st_stream(out + i, vv);
}
__global__ void k_fill_scalar(float* __restrict__ out, int64_t n, float v) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = v;
}

int launch_fill(Device* d, float* out, int64_t n, float v) {
    if (n <= 0) return KTC_OK;
    // head up to the first 16-byte boundary, vector body, scalar tail
    int64_t head = 0;
    while (head < n && !aligned16(out + head)) ++head;
    int launches = 0;
    if (head) { k_fill_scalar<<<1, 32, 0, d->stream>>>(out, head, v); ++launches; }
    const int64_t n4 = (n - head) / 4;
    if (n4) { k_fill_vec<<<grid_for(d, n4, 256, 16), 256, 0, d->stream>>>((float4*)(out + head), n4, v); ++launches; }
    const int64_t tail = (n - head) - n4 * 4;
    if (tail) { k_fill_scalar<<<1, 32, 0, d->stream>>>(out + head + n4 * 4, tail, v); ++launches; }
    return finish_launch("fill", launches);
}

template <template <int> class W>
static int dispatch_scalar(Device* d, int op, float* out, const float* a, int64_t n, float s) {
    switch (op) {
    case KTC_PLUS:  return run_map1(d, out, a, n, W<KTC_PLUS>{s});
    case KTC_MINUS: return run_map1(d, out, a, n, W<KTC_MINUS>{s});
    case KTC_TIMES: return run_map1(d, out, a, n, W<KTC_TIMES>{s});
    case KTC_DIV:   return run_map1(d, out, a, n, W<KTC_DIV>{s});
    case KTC_POW:   return run_map1(d, out, a, n, W<KTC_POW>{s});
    }
    return fail(KTC_EINVAL, "unknown binary op %d", op);
}

int launch_map1(Device* d, int kind, int op, float* out, const float* a, int64_t n, float p0, float p1) {
    switch (kind) {
    case M1_UNARY:
        switch (op) {
        case KTC_EXP:        return run_map1(d, out, a, n, UnOp<KTC_EXP>());
        case KTC_LOG:        return run_map1(d, out, a, n, UnOp<KTC_LOG>());
        case KTC_TANH:       return run_map1(d, out, a, n, UnOp<KTC_TANH>());
        case KTC_SIGMOID:    return run_map1(d, out, a, n, UnOp<KTC_SIGMOID>());
        case KTC_RECIPROCAL: return run_map1(d, out, a, n, UnOp<KTC_RECIPROCAL>());
        case KTC_NEG:        return run_map1(d, out, a, n, UnOp<KTC_NEG>());
        }
        return fail(KTC_EINVAL, "unknown unary op %d", op);
    case M1_SCALAR_R:
        if (op == KTC_POW && p0 == 2.0f) return run_map1(d, out, a, n, Square());
        if (op == KTC_POW && p0 == 1.0f) return run_map1(d, out, a, n, Identity());
        return dispatch_scalar<ScalarRight>(d, op, out, a, n, p0);
    case M1_SCALAR_L:
        return dispatch_scalar<ScalarLeft>(d, op, out, a, n, p0);
    case M1_CLAMP:
        return run_map1(d, out, a, n, ClampOp{p0, p1});
    case M1_COMPARE:
        switch (op) {
        case KTC_LT:  return run_map1(d, out, a, n, CompareOp<KTC_LT>{p0});
        case KTC_LTE: return run_map1(d, out, a, n, CompareOp<KTC_LTE>{p0});
        case KTC_GT:  return run_map1(d, out, a, n, CompareOp<KTC_GT>{p0});
        case KTC_GTE: return run_map1(d, out, a, n, CompareOp<KTC_GTE>{p0});
        }
        return fail(KTC_EINVAL, "unknown compare op %d", op);
    }
    return fail(KTC_EINVAL, "unknown map kind %d", kind);
}

int launch_map2(Device* d, int op, float* out, const float* a, const float* b, int64_t n) {
    switch (op) {
    case KTC_PLUS:  return run_map2(d, out, a, b, n, BinOp<KTC_PLUS>());
    case KTC_MINUS: return run_map2(d, out, a, b, n, BinOp<KTC_MINUS>());
    case KTC_TIMES: return run_map2(d, out, a, b, n, BinOp<KTC_TIMES>());
    case KTC_DIV:   return run_map2(d, out, a, b, n, BinOp<KTC_DIV>());
    case KTC_POW:   return run_map2(d, out, a, b, n, BinOp<KTC_POW>());
    }
    return fail(KTC_EINVAL, "unknown binary op %d", op);
}

// ---- broadcast binary ------------------------------------------------------------
// Collapsed view: out[D0][D1][D2] contiguous; each operand has element strides
// (s0,s1,s2) with s2 in {0,1}.  A tile is RB rows of D1 by CW columns of D2 for
// one i0.  Operand access modes:
enum { AM_DIRECT = 0,    // s2 == 1: float4 at base + i0*s0 + i1*s1 + i2 (full-size, or broadcast along D0 only)
       AM_ROWSCALAR = 1, // s2 == 0: one float per (i0,i1) row; the tile's RB scalars are staged in shared memory
       AM_SMEMROW = 2,   // s2 == 1, s1 == 0: a row vector shared by all RB rows, staged once per tile in shared memory
       AM_NONE = 3 };    // operand not read (broadcast_to copies B only)

struct BcastArgs {
    const float* a; const float* b; float* out;
    int64_t D0, D1, D2;
    int64_t as0, as1, bs0, bs1;
    int rows_per_tile;       // RB
    int cols_per_tile;       // CW, multiple of 4
    int64_t tiles_d1, tiles_d2;
    int a_stream, b_stream;  // DIRECT operand is full-size: read it with the streaming hint
    int txc, txc_log2;       // threads across the columns of a tile (power of two <= 256)
};

template <int MODE>
__device__ __forceinline__ void stage_operand(float* sm, const float* base0, int64_t s1, int64_t r0, int64_t c0,
                                              int rows, int cols4) {
    if (MODE == AM_SMEMROW) {
        const float4* src = reinterpret_cast<const float4*>(base0 + c0);
        for (int c = threadIdx.x; c < cols4; c += blockDim.x) reinterpret_cast<float4*>(sm)[c] = __ldg(src + c);
    } else if (MODE == AM_ROWSCALAR) {
        for (int r = threadIdx.x; r < rows; r += blockDim.x) sm[r] = __ldg(base0 + (r0 + r) * s1);
    }
}

template <int MODE>
__device__ __forceinline__ float4 load_operand(const float* sm, const float* tile_base, int64_t s1, int row, int col, int stream) {
    if (MODE == AM_DIRECT) {
        const float4* p = reinterpret_cast<const float4*>(tile_base + (int64_t)row * s1 + col);
        return stream ? __ldcs(p) : __ldg(p);
    }
    if (MODE == AM_ROWSCALAR) { const float v = sm[row]; return make_float4(v, v, v, v); }
    if (MODE == AM_SMEMROW) return *reinterpret_cast<const float4*>(sm + col);
    return make_float4(0.f, 0.f, 0.f, 0.f);
}

template <class F> struct IsDiv { static constexpr bool value = false; };
template <> struct IsDiv<BinOp<KTC_DIV>> { static constexpr bool value = true; };

// A thread owns one column group (4 floats) and the rows ty, ty + TYC, ... of the tile,
// at most U of them per batch (U = 8: a tile of 8192 floats is one batch; U = 4 for the
// arithmetic-heavy functors, whose unrolled code would otherwise not fit the instruction cache).  The loads of the
// full-size (DIRECT) operands are issued first, then the broadcast operand is staged in
// shared memory, so the staging latency overlaps the main stream instead of preceding it.
template <int MODE_A, int MODE_B, int U, class F>
__global__ void __launch_bounds__(256, 3) k_bcast3(BcastArgs p, F f) {
    extern __shared__ __align__(16) float smem[];
    constexpr bool STAGE_A = (MODE_A == AM_SMEMROW || MODE_A == AM_ROWSCALAR);
    constexpr bool STAGE_B = (MODE_B == AM_SMEMROW || MODE_B == AM_ROWSCALAR);
    constexpr bool DIV_ROW = IsDiv<F>::value && MODE_B == AM_ROWSCALAR;      // one divisor per row: divide by its reciprocal
    const int sm_stride = max(p.cols_per_tile, (p.rows_per_tile + 3) & ~3);
    float* sm_a = smem;
    float* sm_b = smem + (STAGE_A ? sm_stride : 0);
    float* sm_r = sm_b + sm_stride;                                            // the rows' reciprocals (DIV_ROW)
    const int tx = threadIdx.x & (p.txc - 1), ty = threadIdx.x >> p.txc_log2;
    const int tyc = blockDim.x >> p.txc_log2;

    // tile counts fit 32 bits (the host falls back to the generic kernel otherwise): no 64-bit division on this path
    const uint32_t tiles_d2 = (uint32_t)p.tiles_d2;
    const uint32_t tiles_per_i0 = (uint32_t)p.tiles_d1 * tiles_d2;
    const uint32_t n_tiles = (uint32_t)p.D0 * tiles_per_i0;

    for (uint32_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const uint32_t i0u = t / tiles_per_i0;
        const uint32_t rem = t - i0u * tiles_per_i0;
        const uint32_t td1 = rem / tiles_d2, td2 = rem - td1 * tiles_d2;
        const int64_t i0 = i0u;
        const int64_t r0 = (int64_t)td1 * p.rows_per_tile, c0 = (int64_t)td2 * p.cols_per_tile;
        const int rows = (int)min((int64_t)p.rows_per_tile, p.D1 - r0);
        const int cols4 = (int)(min((int64_t)p.cols_per_tile, p.D2 - c0) >> 2);
        const float* abase = (MODE_A == AM_DIRECT) ? p.a + i0 * p.as0 + r0 * p.as1 + c0 : nullptr;
        const float* bbase = (MODE_B == AM_DIRECT) ? p.b + i0 * p.bs0 + r0 * p.bs1 + c0 : nullptr;
        float* obase = p.out + (i0 * p.D1 + r0) * p.D2 + c0;
        bool staged = false;

        for (int c4 = tx; c4 < cols4 || !staged; c4 += p.txc) {
            const int col = c4 << 2;
            const bool col_ok = c4 < cols4;
            for (int r = ty; r < rows || !staged; r += tyc * U) {
                float4 va[U], vb[U];
                // 1. direct operands of this batch
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int row = r + u * tyc;
                    if (col_ok && row < rows) {
                        if (MODE_A == AM_DIRECT) va[u] = load_operand<MODE_A>(sm_a, abase, p.as1, row, col, p.a_stream);
                        if (MODE_B == AM_DIRECT) vb[u] = load_operand<MODE_B>(sm_b, bbase, p.bs1, row, col, p.b_stream);
                    }
                }
                // 2. stage the broadcast operand(s) once per tile (every thread reaches this point in its first batch)
                if (!staged) {
                    if (STAGE_A || STAGE_B) {
                        __syncthreads();                 // readers of the previous tile are done
                        if (STAGE_A) stage_operand<MODE_A>(sm_a, p.a + i0 * p.as0, p.as1, r0, c0, rows, cols4);
                        if (STAGE_B) stage_operand<MODE_B>(sm_b, p.b + i0 * p.bs0, p.bs1, r0, c0, rows, cols4);
                        if (DIV_ROW) for (int rr = threadIdx.x; rr < rows; rr += blockDim.x) sm_r[rr] = kd_row_reciprocal(sm_b[rr]);   // its own value
                        __syncthreads();
                    }
                    staged = true;
                }
                // 3. staged operands, arithmetic, store
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int row = r + u * tyc;
                    if (col_ok && row < rows) {
                        if (MODE_A != AM_DIRECT) va[u] = load_operand<MODE_A>(sm_a, abase, p.as1, row, col, 0);
                        if (MODE_B != AM_DIRECT) vb[u] = load_operand<MODE_B>(sm_b, bbase, p.bs1, row, col, 0);
                        float4* dst = reinterpret_cast<float4*>(obase + (int64_t)row * p.D2 + col);
                        if (DIV_ROW) st_stream(dst, div_by_row(va[u], vb[u].x, sm_r[row]));
                        else st_stream(dst, apply2(f, va[u], vb[u]));
                    }
                }
            }
        }
    }
}

// The same tile when every tile of the launch is whole and exactly one batch (32 rows x 256 columns, 64 x 4 threads, 8 rows
// each: the geometry of any tensor whose extents are multiples of the tile): per-thread base pointers and strides are
// formed once and the body is straight-line -- about a third of the instructions of the guarded form, which matters when
// the clock drops under a power cap and a streaming kernel becomes bound by instruction issue.
template <int MODE_A, int MODE_B, int U, class F>
__global__ void __launch_bounds__(256, 3) k_bcast3_full(BcastArgs p, F f) {
    extern __shared__ __align__(16) float smem[];
    constexpr bool STAGE_A = (MODE_A == AM_SMEMROW || MODE_A == AM_ROWSCALAR);
    constexpr bool STAGE_B = (MODE_B == AM_SMEMROW || MODE_B == AM_ROWSCALAR);
    constexpr bool DIV_ROW = IsDiv<F>::value && MODE_B == AM_ROWSCALAR;
    const int sm_stride = max(p.cols_per_tile, (p.rows_per_tile + 3) & ~3);
    float* sm_a = smem;
    float* sm_b = smem + (STAGE_A ? sm_stride : 0);
    float* sm_r = sm_b + sm_stride;
    const int tx = threadIdx.x & (p.txc - 1), ty = threadIdx.x >> p.txc_log2;
    const int tyc = blockDim.x >> p.txc_log2;
    const uint32_t tiles_d2 = (uint32_t)p.tiles_d2;
    const uint32_t tiles_per_i0 = (uint32_t)p.tiles_d1 * tiles_d2;
    const uint32_t t = blockIdx.x;                                     // one tile per CTA
    const uint32_t i0u = t / tiles_per_i0;
    const uint32_t rem = t - i0u * tiles_per_i0;
    const uint32_t td1 = rem / tiles_d2, td2 = rem - td1 * tiles_d2;
    const int64_t i0 = i0u;
    const int64_t r0 = (int64_t)td1 * p.rows_per_tile, c0 = (int64_t)td2 * p.cols_per_tile;
    const int cols4 = p.cols_per_tile >> 2;
    const bool active = tx < cols4;
    const int col = tx << 2;
    const float* pa = (MODE_A == AM_DIRECT) ? p.a + i0 * p.as0 + (r0 + ty) * p.as1 + c0 + col : nullptr;
    const float* pb = (MODE_B == AM_DIRECT) ? p.b + i0 * p.bs0 + (r0 + ty) * p.bs1 + c0 + col : nullptr;
    float* po = p.out + (i0 * p.D1 + r0 + ty) * p.D2 + c0 + col;
    const int64_t sa = (int64_t)tyc * p.as1, sb = (int64_t)tyc * p.bs1, so = (int64_t)tyc * p.D2;
    float4 va[U], vb[U];
    if (active) {
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            if (MODE_A == AM_DIRECT) { const float4* q = reinterpret_cast<const float4*>(pa + u * sa); va[u] = p.a_stream ? __ldcs(q) : __ldg(q); }
            if (MODE_B == AM_DIRECT) { const float4* q = reinterpret_cast<const float4*>(pb + u * sb); vb[u] = p.b_stream ? __ldcs(q) : __ldg(q); }
        }
    }
    if (STAGE_A || STAGE_B) {
        if (STAGE_A) stage_operand<MODE_A>(sm_a, p.a + i0 * p.as0, p.as1, r0, c0, p.rows_per_tile, cols4);
        if (STAGE_B) stage_operand<MODE_B>(sm_b, p.b + i0 * p.bs0, p.bs1, r0, c0, p.rows_per_tile, cols4);
        if (DIV_ROW) for (int rr = threadIdx.x; rr < p.rows_per_tile; rr += blockDim.x) sm_r[rr] = kd_row_reciprocal(sm_b[rr]);
        __syncthreads();
    }
    if (active) {
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            const int row = ty + u * tyc;
            if (MODE_A != AM_DIRECT) va[u] = load_operand<MODE_A>(sm_a, nullptr, p.as1, row, col, 0);
            if (MODE_B != AM_DIRECT) vb[u] = load_operand<MODE_B>(sm_b, nullptr, p.bs1, row, col, 0);
            float4* dst = reinterpret_cast<float4*>(po + u * so);
            if (DIV_ROW) st_stream(dst, div_by_row(va[u], vb[u].x, sm_r[row]));
            else st_stream(dst, apply2(f, va[u], vb[u]));
        }
    }
}

// Fallback for anything the tiled kernel does not take (more than three
// collapsed dimensions, an inner extent that is not a multiple of 4, unaligned
// bases): one element per thread-iteration, index decomposed per element.
struct GenericArgs {
    int ndim;
    int64_t shape[KTC_MAX_DIMS];
    int64_t as[KTC_MAX_DIMS], bs[KTC_MAX_DIMS];
};

template <bool HAS_A, class F>
__global__ void k_bcast_generic(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                int64_t total, GenericArgs g, F f) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = e, oa = 0, ob = 0;
        for (int d = g.ndim - 1; d >= 0; --d) {
            const int64_t q = rem / g.shape[d], idx = rem - q * g.shape[d];
            rem = q; oa += idx * g.as[d]; ob += idx * g.bs[d];
        }
        out[e] = f(HAS_A ? __ldg(a + oa) : 0.0f, __ldg(b + ob));
    }
}

struct SelectB { __device__ __forceinline__ float operator()(float, float b) const { return b; } };

template <class F> struct BatchRows { static constexpr int value = 8; };
template <> struct BatchRows<BinOp<KTC_DIV>> { static constexpr int value = 4; };
template <> struct BatchRows<BinOp<KTC_POW>> { static constexpr int value = 4; };

template <int MA, int MB, class F>
static void launch_bcast3_modes(Device* d, const BcastArgs& p, int grid, size_t smem, F f) {
    constexpr bool kDivRow = IsDiv<F>::value && MB == AM_ROWSCALAR;
    constexpr int kU = kDivRow ? 8 : BatchRows<F>::value;                // three instructions per quotient: the full batch fits
    const int tyc = 256 >> p.txc_log2;
    const int64_t n_tiles = p.D0 * p.tiles_d1 * p.tiles_d2;
    // every tile whole, one batch per tile, one tile per CTA: the straight-line kernel
    const bool full = p.D1 % p.rows_per_tile == 0 && p.D2 % p.cols_per_tile == 0 && p.txc * 4 >= p.cols_per_tile
                      && tyc * kU == p.rows_per_tile && grid == n_tiles && tune("bcast_full_tiles", 1) != 0
                      && !(kDivRow && tune("bcast_div_batch", 8) != 8);
    if (full) { k_bcast3_full<MA, MB, kU, F><<<grid, 256, smem, d->stream>>>(p, f); return; }
    if (kDivRow && tune("bcast_div_batch", 8) == 8)
        k_bcast3<MA, MB, kU, F><<<grid, 256, smem, d->stream>>>(p, f);
    else
        k_bcast3<MA, MB, BatchRows<F>::value, F><<<grid, 256, smem, d->stream>>>(p, f);
}

template <class F>
static int run_bcast3(Device* d, int ma, int mb, const BcastArgs& p, int grid, size_t smem, F f) {
#define KTC_B3(MA, MB) if (ma == MA && mb == MB) { launch_bcast3_modes<MA, MB, F>(d, p, grid, smem, f); return finish_launch("bcast3"); }
    KTC_B3(AM_DIRECT, AM_DIRECT) KTC_B3(AM_DIRECT, AM_ROWSCALAR) KTC_B3(AM_DIRECT, AM_SMEMROW)
    KTC_B3(AM_ROWSCALAR, AM_DIRECT) KTC_B3(AM_ROWSCALAR, AM_ROWSCALAR) KTC_B3(AM_ROWSCALAR, AM_SMEMROW)
    KTC_B3(AM_SMEMROW, AM_DIRECT) KTC_B3(AM_SMEMROW, AM_ROWSCALAR) KTC_B3(AM_SMEMROW, AM_SMEMROW)
    KTC_B3(AM_NONE, AM_DIRECT) KTC_B3(AM_NONE, AM_ROWSCALAR) KTC_B3(AM_NONE, AM_SMEMROW)
#undef KTC_B3
    return fail(KTC_EINVAL, "bcast3: unsupported operand modes %d/%d", ma, mb);
}

template <class F>
static int run_bcast(Device* d, float* out, const int64_t* oshape, int ndim, const float* a, const int64_t* astride,
                     const float* b, const int64_t* bstride, F f) {
    // 1. drop unit dimensions, merge neighbours that are laid out contiguously in both operands
    int64_t S[KTC_MAX_DIMS], AS[KTC_MAX_DIMS], BS[KTC_MAX_DIMS];
    int m = 0;
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) total *= oshape[i];
    if (total == 0) return KTC_OK;
    for (int i = 0; i < ndim; ++i) {
        if (oshape[i] == 1) continue;
        const int64_t sa = a ? astride[i] : 0, sb = bstride[i];
        if (m > 0 && AS[m - 1] == sa * oshape[i] && BS[m - 1] == sb * oshape[i]) {
            S[m - 1] *= oshape[i]; AS[m - 1] = sa; BS[m - 1] = sb;
        } else { S[m] = oshape[i]; AS[m] = sa; BS[m] = sb; ++m; }
    }
    if (m == 0) { S[0] = 1; AS[0] = 0; BS[0] = 0; m = 1; }

    // 2. tiled path?
    bool tiled = (m <= 3) && (S[m - 1] % 4 == 0) && aligned16(out) && tune("bcast_force_generic", 0) == 0;
    int64_t D[3] = {1, 1, 1}, as[3] = {0, 0, 0}, bs[3] = {0, 0, 0};
    for (int i = 0; i < m && i < 3 && tiled; ++i) { D[3 - m + i] = S[i]; as[3 - m + i] = AS[i]; bs[3 - m + i] = BS[i]; }
    int ma = AM_NONE, mb = AM_DIRECT;
    auto classify = [&](const float* base, const int64_t* s, int* mode, int* stream) -> bool {
        *stream = 0;
        if (s[2] == 0) { *mode = AM_ROWSCALAR; return true; }
        if (s[2] != 1) return false;
        if (!aligned16(base) || (s[0] & 3) || (s[1] & 3)) return false;
        if (s[1] == 0 && D[1] > 1) { *mode = AM_SMEMROW; return true; }
        *mode = AM_DIRECT;
        *stream = (s[0] != 0 || D[0] == 1) ? 1 : 0;      // every element is read once
        return true;
    };
    BcastArgs p;
    if (tiled) {
        if (a) tiled = classify(a, as, &ma, &p.a_stream); else { ma = AM_NONE; p.a_stream = 0; }
        if (tiled) tiled = classify(b, bs, &mb, &p.b_stream);
    }
    if (tiled) {
        p.a = a; p.b = b; p.out = out;
        p.D0 = D[0]; p.D1 = D[1]; p.D2 = D[2];
        p.as0 = as[0]; p.as1 = as[1]; p.bs0 = bs[0]; p.bs1 = bs[1];
        const int tile_elems = tune("bcast_tile_elems", 8192);
        const int max_cols = tune("bcast_max_cols", 2048);
        p.cols_per_tile = (int)(D[2] < max_cols ? D[2] : max_cols);
        int64_t rb = tile_elems / p.cols_per_tile; if (rb < 1) rb = 1; if (rb > D[1]) rb = D[1];
        p.rows_per_tile = (int)rb;
        p.tiles_d1 = (D[1] + rb - 1) / rb;
        p.tiles_d2 = (D[2] + p.cols_per_tile - 1) / p.cols_per_tile;
        const int cw4 = p.cols_per_tile >> 2;
        p.txc = 1; p.txc_log2 = 0;
        while (p.txc < 256 && p.txc < cw4) { p.txc <<= 1; ++p.txc_log2; }
        const int64_t n_tiles = D[0] * p.tiles_d1 * p.tiles_d2;
        if (n_tiles >= 0x7fffffffLL) tiled = false;                  // the kernel decomposes the tile index with 32-bit arithmetic
    }
    if (tiled) {
        const int64_t n_tiles = D[0] * p.tiles_d1 * p.tiles_d2;
        const int bps = tune("bcast_blocks_per_sm", 0);             // <= 0: one tile per CTA, tiles in address order
        const int64_t cap = bps > 0 ? (int64_t)d->sm_count * bps : 0x7fffffffLL;
        const int grid = (int)(n_tiles < cap ? n_tiles : cap);
        const int sm_stride = p.cols_per_tile > ((p.rows_per_tile + 3) & ~3) ? p.cols_per_tile : ((p.rows_per_tile + 3) & ~3);
        const size_t smem = sizeof(float) * (size_t)sm_stride *              // a row-scalar b also gets room for the rows' reciprocals
            ((ma == AM_SMEMROW || ma == AM_ROWSCALAR ? 1 : 0) + (mb == AM_SMEMROW ? 1 : mb == AM_ROWSCALAR ? 2 : 0));
        return run_bcast3(d, ma, mb, p, grid, smem, f);
    }

    // 3. generic fallback
    GenericArgs g; g.ndim = m;
    for (int i = 0; i < m; ++i) { g.shape[i] = S[i]; g.as[i] = AS[i]; g.bs[i] = BS[i]; }
    const int grid = grid_for(d, total, 256, 16);
    if (a) k_bcast_generic<true, F><<<grid, 256, 0, d->stream>>>(a, b, out, total, g, f);
    else   k_bcast_generic<false, F><<<grid, 256, 0, d->stream>>>(a, b, out, total, g, f);
    return finish_launch("bcast(generic)");
}

// op < 0 selects the copy of operand b (broadcast_to)
int launch_bcast(Device* d, int op, float* out, const int64_t* oshape, int ndim,
                 const float* a, const int64_t* astride, const float* b, const int64_t* bstride, float param) {
    switch (op) {
    case kBcastSelectB:    return run_bcast(d, out, oshape, ndim, nullptr, nullptr, b, bstride, SelectB());
    case kBcastMaskedFill: return run_bcast(d, out, oshape, ndim, a, astride, b, bstride, MaskedFill{param});
    case KTC_PLUS:  return run_bcast(d, out, oshape, ndim, a, astride, b, bstride, BinOp<KTC_PLUS>());
    case KTC_MINUS: return run_bcast(d, out, oshape, ndim, a, astride, b, bstride, BinOp<KTC_MINUS>());
    case KTC_TIMES: return run_bcast(d, out, oshape, ndim, a, astride, b, bstride, BinOp<KTC_TIMES>());
    case KTC_DIV:   return run_bcast(d, out, oshape, ndim, a, astride, b, bstride, BinOp<KTC_DIV>());
    case KTC_POW:   return run_bcast(d, out, oshape, ndim, a, astride, b, bstride, BinOp<KTC_POW>());
    }
    return fail(KTC_EINVAL, "unknown binary op %d", op);
}

// ---- bounded device-side wait (test hook) -------------------------------------------
// Spins on a flag that nothing sets, gives up after limit_ns of %globaltimer and
// reports 1 in *status: the pattern every cross-kernel wait in this library must
// follow (no trap, no endless loop; the context stays usable).
__global__ void k_bounded_wait(const volatile int* flag, long long limit_ns, int* status) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    int st = 1;
    for (int iter = 0; iter < (1 << 28); ++iter) {
        if (*flag != 0) { st = 0; break; }
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if ((long long)(t - t0) > limit_ns) break;
        __nanosleep(200);
    }
    *status = st;
}

int launch_bounded_wait(Device* d, int64_t limit_ns, int* status) {
    int* dstatus = d->err_flag;       // reuse the error word as the status slot
    k_bounded_wait<<<1, 1, 0, d->stream>>>(d->wait_flag, (long long)limit_ns, dstatus);
    KTC_TRY(finish_launch("bounded_wait"));
    int h = -1;
    KTC_CUDA(cudaMemcpyAsync(&h, dstatus, sizeof(int), cudaMemcpyDeviceToHost, d->stream));
    KTC_CUDA(cudaMemsetAsync(dstatus, 0, sizeof(int), d->stream));
    KTC_CUDA(cudaStreamSynchronize(d->stream));
    if (status) *status = (h == 1) ? KTC_ETIMEOUT : KTC_OK;
    return KTC_OK;
}

}  // namespace ktc
