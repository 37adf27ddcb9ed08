// ktc_expr.cu -- fused evaluation of a chain of elementwise ops, optionally ending in a sum.
//
// kten's autograd issues one raw-tensor call per line of doForward / doBackward
// (kten-api/.../autograd/functions/BasicFunctions.kt, PointwiseFunctions.kt), and every call
// is a full pass over HBM: the sharded-graph benchmark step moves 34 tensor volumes where
// reading the input once or twice would do.  A backend can defer elementwise calls behind
// the SPI and hand the accumulated expression to this kernel when a value is finally needed
// (a host read, a reduction, an op outside the hot path).
//
// The expression arrives as a short program for a register machine:
//   * every register holds one float4 (four neighbouring elements of the innermost axis);
//   * each instruction applies ONE reference operation to whole registers, with exactly the
//     arithmetic of the stand-alone kernels (ktc_math.cuh), so a fused chain produces the same
//     bits as the chain of separate calls -- nothing is contracted or re-associated;
//   * LOAD reads a leaf tensor through its broadcast strides (0 where the leaf is broadcast;
//     nothing is materialised), STORE writes a full-size result, ACC feeds a sum.
// Registers live in shared memory (a dynamically indexed array cannot stay in hardware
// registers), laid out so that a warp's access is one conflict-free 128-bit row.
//
// Iteration space: the collapsed view [D0, D1, D2] of the result shape; a warp owns a
// 128-column tile (lane = 4 columns) of a segment of rows, like k_cols_warp.  Sinks:
//   KTC_EXPR_STORE_ONLY   results are written by STORE instructions;
//   KTC_EXPR_SUM_ALL      ACC values are summed over everything  -> out[1]  (optionally / count);
//   KTC_EXPR_SUM_ROWS     ACC values are summed over D0 and D1   -> out[D2] (the broadcast-gradient
//                         sum-to-shape of a row vector: mayUnexpand, Utils.kt:14-41).
// Sums use the accumulation scheme of ktc_reduce.cu (float runs folded into doubles, fixed
// combination order: eight segments per CTA, then a second pass).
#include "ktc_accum.cuh"
#include "ktc_expr_args.h"
#include "ktc_jit.hpp"
#include "ktc_p2p.cuh"
#include "ktc_softmax.cuh"

namespace ktc {


__device__ __forceinline__ float4 f4(float v) { return make_float4(v, v, v, v); }
#define KTC_EACH(expr_x, expr_y, expr_z, expr_w) make_float4(expr_x, expr_y, expr_z, expr_w)

// out-of-line so that the switch below stays small; same functors as the stand-alone kernels
static __device__ __noinline__ float4 expr_pow(float4 x, float4 y) {
    return apply2(BinOp<KTC_POW>(), x, y);
}
static __device__ __noinline__ float4 expr_sigmoid(float4 x) {
    return apply1(UnOp<KTC_SIGMOID>(), x);
}
static __device__ __noinline__ float4 expr_exp(float4 x) {
    return apply1(UnOp<KTC_EXP>(), x);
}
static __device__ __noinline__ float4 expr_log(float4 x) {
    UnOp<KTC_LOG> f; return KTC_EACH(f(x.x), f(x.y), f(x.z), f(x.w));
}
static __device__ __noinline__ float4 expr_tanh(float4 x) {
    UnOp<KTC_TANH> f; return KTC_EACH(f(x.x), f(x.y), f(x.z), f(x.w));
}

template <int SINK>
__global__ void __launch_bounds__(256) k_expr(const __grid_constant__ ExprArgs p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // launched early (launch_early below): the stream's earlier work is complete from here on
    __shared__ float4 regs[kExprRegs][256];
    __shared__ double sm_part[SINK == KTC_EXPR_SUM_ROWS ? 8 * 32 * 4 : 8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // item -> (row segment, column tile); the column tile varies fastest (address order)
    int64_t ct, seg;
    if (SINK == KTC_EXPR_STORE_ONLY) {
        const int64_t item = (int64_t)blockIdx.x * 8 + warp;
        if (item >= (int64_t)p.S * p.col_tiles) return;        // whole warps leave together; no barrier in this mode
        ct = item % p.col_tiles; seg = item / p.col_tiles;
    } else {
        ct = blockIdx.x % p.col_tiles;
        seg = (blockIdx.x / p.col_tiles) * 8 + warp;             // eight consecutive segments per CTA
    }
    const int64_t col = (ct * 32 + lane) * 4;
    const bool col_ok = col < p.D2;
    const int64_t rows_total = p.D0 * p.D1;
    const int64_t r0 = seg * p.seg_rows, r1 = min(rows_total, r0 + p.seg_rows);

    SumAcc acc[4];
    #pragma unroll
    for (int k = 0; k < 4; ++k) acc[k].init();

    if (col_ok && r0 < r1) {
        int64_t i0 = r0 / p.D1, i1 = r0 - i0 * p.D1;
        for (int64_t r = r0; r < r1; ++r) {
            #pragma unroll 1
            for (int pc = 0; pc < p.n_code; ++pc) {
                const uint32_t ins = p.code[pc];
                const int op = ins & 0xff, d = (ins >> 8) & 0xf, ra = (ins >> 12) & 0xf, rb = (ins >> 16) & 0xf, k = ins >> 20;
                const float4 x = regs[ra][tid], y = regs[rb][tid];
                float4 v;
                switch (op) {
                case KTC_X_LOAD: {
                    const float* base = p.leaf[k] + i0 * p.ls0[k] + i1 * p.ls1[k];
                    // plain (coherent) loads: an in-place program stores into the buffer one of its leaves reads
                    if (p.ls2[k]) v = __ldcs(reinterpret_cast<const float4*>(base + col));
                    else v = f4(*base);
                    break;
                }
                case KTC_X_CONST: v = f4(p.imm[k]); break;
                case KTC_X_ADD: v = KTC_EACH(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y), __fadd_rn(x.z, y.z), __fadd_rn(x.w, y.w)); break;
                case KTC_X_SUB: v = KTC_EACH(__fsub_rn(x.x, y.x), __fsub_rn(x.y, y.y), __fsub_rn(x.z, y.z), __fsub_rn(x.w, y.w)); break;
                case KTC_X_MUL: v = KTC_EACH(__fmul_rn(x.x, y.x), __fmul_rn(x.y, y.y), __fmul_rn(x.z, y.z), __fmul_rn(x.w, y.w)); break;
                case KTC_X_DIV: v = KTC_EACH(__fdiv_rn(x.x, y.x), __fdiv_rn(x.y, y.y), __fdiv_rn(x.z, y.z), __fdiv_rn(x.w, y.w)); break;
                case KTC_X_POW: v = expr_pow(x, y); break;
                case KTC_X_NEG: v = KTC_EACH(-x.x, -x.y, -x.z, -x.w); break;
                case KTC_X_RCP: v = KTC_EACH(__frcp_rn(x.x), __frcp_rn(x.y), __frcp_rn(x.z), __frcp_rn(x.w)); break;
                case KTC_X_SQUARE: v = KTC_EACH(__fmul_rn(x.x, x.x), __fmul_rn(x.y, x.y), __fmul_rn(x.z, x.z), __fmul_rn(x.w, x.w)); break;
                case KTC_X_EXP: v = expr_exp(x); break;
                case KTC_X_LOG: v = expr_log(x); break;
                case KTC_X_TANH: v = expr_tanh(x); break;
                case KTC_X_SIGMOID: v = expr_sigmoid(x); break;
                case KTC_X_CLAMP: { ClampOp c{p.imm[k], p.imm[k + 1]}; v = KTC_EACH(c(x.x), c(x.y), c(x.z), c(x.w)); break; }
                case KTC_X_CMP_LT: { const float t = p.imm[k]; v = KTC_EACH(x.x < t ? 1.f : 0.f, x.y < t ? 1.f : 0.f, x.z < t ? 1.f : 0.f, x.w < t ? 1.f : 0.f); break; }
                case KTC_X_CMP_LTE: { const float t = p.imm[k]; v = KTC_EACH(x.x <= t ? 1.f : 0.f, x.y <= t ? 1.f : 0.f, x.z <= t ? 1.f : 0.f, x.w <= t ? 1.f : 0.f); break; }
                case KTC_X_CMP_GT: { const float t = p.imm[k]; v = KTC_EACH(x.x > t ? 1.f : 0.f, x.y > t ? 1.f : 0.f, x.z > t ? 1.f : 0.f, x.w > t ? 1.f : 0.f); break; }
                case KTC_X_CMP_GTE: { const float t = p.imm[k]; v = KTC_EACH(x.x >= t ? 1.f : 0.f, x.y >= t ? 1.f : 0.f, x.z >= t ? 1.f : 0.f, x.w >= t ? 1.f : 0.f); break; }
                case KTC_X_SQRT: v = KTC_EACH(__fsqrt_rn(x.x), __fsqrt_rn(x.y), __fsqrt_rn(x.z), __fsqrt_rn(x.w)); break;
                case KTC_X_RSQRT: v = KTC_EACH(__fdiv_rn(1.0f, __fsqrt_rn(x.x)), __fdiv_rn(1.0f, __fsqrt_rn(x.y)), __fdiv_rn(1.0f, __fsqrt_rn(x.z)), __fdiv_rn(1.0f, __fsqrt_rn(x.w))); break;
                case KTC_X_ABS: v = KTC_EACH(fabsf(x.x), fabsf(x.y), fabsf(x.z), fabsf(x.w)); break;
                case KTC_X_SCATC: {
                    const int t = (int)y.x;                        // Float.toInt(): truncation; y holds the row's index in every column
                    if ((unsigned)t >= (unsigned)p.D2) *p.err = 1;
                    const float c = p.imm[k];
                    const int c0 = (int)col;
                    v = make_float4(c0 == t ? c : x.x, c0 + 1 == t ? c : x.y, c0 + 2 == t ? c : x.z, c0 + 3 == t ? c : x.w);
                    break;
                }
                case KTC_X_STORE:
                    __stcs(reinterpret_cast<float4*>(p.store[k] + r * p.D2 + col), x);
                    continue;
                case KTC_X_ACC:
                    if (SINK == KTC_EXPR_SUM_ROWS) {
                        acc[0].add(x.x, 0); acc[1].add(x.y, 0); acc[2].add(x.z, 0); acc[3].add(x.w, 0);
                    } else {
                        acc[0].add4(x, 0);
                    }
                    continue;
                default: continue;
                }
                regs[d][tid] = v;
            }
            if (SINK != KTC_EXPR_STORE_ONLY && ((r - r0) & 7) == 7) {       // fold the float runs every 8 rows (<= 32 values)
                #pragma unroll
                for (int k = 0; k < 4; ++k) acc[k].end();
            }
            if (++i1 == p.D1) { i1 = 0; ++i0; }
        }
        #pragma unroll
        for (int k = 0; k < 4; ++k) acc[k].end();
    }

    if (SINK == KTC_EXPR_SUM_ALL) {
        double v = acc[0].acc;
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) sm_part[warp] = v;
        __syncthreads();
        if (tid == 0) {
            double t = sm_part[0];
            #pragma unroll
            for (int w = 1; w < 8; ++w) t += sm_part[w];
            if (gridDim.x == 1) p.out[0] = (float)(p.divisor > 0.0 ? t / p.divisor : t);
            else p.part[blockIdx.x] = t;
        }
    } else if (SINK == KTC_EXPR_SUM_ROWS) {
        #pragma unroll
        for (int k = 0; k < 4; ++k) sm_part[(warp * 32 + lane) * 4 + k] = acc[k].acc;
        __syncthreads();
        if (warp == 0 && col_ok) {
            #pragma unroll
            for (int k = 0; k < 4; ++k) {
                double t = sm_part[lane * 4 + k];
                #pragma unroll
                for (int w = 1; w < 8; ++w) t += sm_part[(w * 32 + lane) * 4 + k];
                p.part[(blockIdx.x / p.col_tiles) * p.D2 + col + k] = t;
            }
        }
    }
}

// ---- second pass of a pass with several sums: ONE kernel for all of them ---------------------------------------
// Every sink's partials are combined exactly as its own second-pass kernel combines them (k_combine_warp: one warp per
// output, lanes stride over the segments, xor-shuffle tree; k_combine_thread: one thread per output, segments in order;
// a full sum: one block, threads stride over the partials, shuffles, then the warp leaders in order), so SUM_ROWS and
// SUM_LAST results keep the bits of the single-sink calls.  On top of that the kernel can
//   * add a result into another tensor in the same step (add_to: the gradient accumulated into a Variable,
//     Variable.kt:44-46 -- target = target + (float)sum, the very float addition the separate in-place call performs);
//   * sum tensors over the ranks when the last block has finished (x: the peer-memory exchange of ktc_p2p.cuh, run by
//     whichever block takes the last ticket of a device counter -- no block waits for another block).
// so that a training step's loss, gradients, accumulation and all-reduce are the producing pass plus this kernel.
struct CombineArgs {
    int n_sinks;
    int mode[kExprMaxSinks];               // 0 one warp per output, 1 one thread per output, 2 one block for a single output
    const double* part[kExprMaxSinks];
    float* out[kExprMaxSinks];
    float* add_to[kExprMaxSinks];          // nullptr: none
    int add_mode[kExprMaxSinks];           // 1: target += result; 2: target = 0f + result (a gradient that was just zeroed)
    int64_t n_out[kExprMaxSinks];
    int S[kExprMaxSinks];                  // partials per output
    double divisor[kExprMaxSinks];         // > 0: mean
    int block_end[kExprMaxSinks];          // sink j owns blocks [block_end[j-1], block_end[j])
    int exchange;                          // != 0: x is valid
    P2pArgs x;
};
__device__ unsigned int g_combine_tickets;  // blocks of the running k_combine_multi that have finished (back to 0 when the last one leaves)

__device__ __forceinline__ void combine_put(const CombineArgs& a, int j, int64_t o, double sum) {
    const float v = (float)(a.divisor[j] > 0.0 ? sum / a.divisor[j] : sum);
    a.out[j][o] = v;
    if (a.add_to[j]) a.add_to[j][o] = __fadd_rn(a.add_mode[j] == 2 ? 0.f : a.add_to[j][o], v);
}

__global__ void __launch_bounds__(256) k_combine_multi(const __grid_constant__ CombineArgs a) {
    // Launched with programmatic stream serialisation, this kernel's CTAs may be scheduled while the first pass drains; they
    // wait here until that grid has completed and its partial sums are visible (a no-op after an ordinary launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ double sm[8];
    __shared__ int last_block, timed_out;
    int j = 0;
    while (j + 1 < a.n_sinks && (int)blockIdx.x >= a.block_end[j]) ++j;
    const int block = (int)blockIdx.x - (j ? a.block_end[j - 1] : 0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const double* part = a.part[j];
    const int64_t n_out = a.n_out[j];
    const int S = a.S[j];
    if (a.mode[j] == 0) {
        const int64_t o = ((int64_t)block * 256 + tid) >> 5;
        if (o < n_out) {
            double acc = 0.0;
            for (int s = lane; s < S; s += 32) acc += part[(int64_t)s * n_out + o];
            #pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (lane == 0) combine_put(a, j, o, acc);
        }
    } else if (a.mode[j] == 1) {
        const int64_t o = (int64_t)block * 256 + tid;
        if (o < n_out) {
            double acc = 0.0;
            for (int s = 0; s < S; ++s) acc += part[(int64_t)s * n_out + o];
            combine_put(a, j, o, acc);
        }
    } else {
        double acc = 0.0;
        for (int s = tid; s < S; s += 256) acc += part[s];
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) sm[warp] = acc;
        __syncthreads();
        if (tid == 0) {
            double t = sm[0];
            #pragma unroll
            for (int w = 1; w < 8; ++w) t += sm[w];
            combine_put(a, j, 0, t);
        }
    }
    if (!a.exchange) return;
    // the block that takes the last ticket sees every other block's results (fence, then the ticket) and exchanges them
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&g_combine_tickets, 1u);
        last_block = ticket == gridDim.x - 1;
        if (last_block) g_combine_tickets = 0;
    }
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    p2p_exchange_block(a.x, &timed_out);
}

// Launches a kernel that begins with griddepcontrol.wait so that its CTAs may be scheduled while the kernel before it in the
// stream drains (programmatic stream serialisation): the stream's order, with the launch latency hidden.
template <class... Params, class... Args>
static inline void launch_early(void (*kernel)(Params...), dim3 grid, dim3 block, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = tune("expr_overlap_launches", 1) ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...) != cudaSuccess && cfg.numAttrs) {
        cudaGetLastError();                                  // an attribute the driver refuses: the ordinary way
        cfg.numAttrs = 0;
        cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    }
}

static inline int finish_launch_expr(const char* what) {
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return KTC_OK;
}

// The first pass over the iteration space: the kernel generated for this program when the space is
// large enough to pay for a compilation (tunable expr_jit_min_elems), else the interpreter.
static int launch_expr(Device* d, const ExprArgs& a, int n_leaves, int sink, int64_t grid, int64_t total) {
    if (tune("expr_jit", 1) && total >= (int64_t)tune("expr_jit_min_elems", 1 << 20)) {
        const int rc = jit_launch(d, a, n_leaves, sink, grid);
        if (rc != KTC_ENOTSUP) return rc;
    }
    if (sink == KTC_EXPR_MULTI) return fail(KTC_ENOTSUP, "ktc_expr_eval_multi: no generated kernel for this program (iteration space below expr_jit_min_elems, or NVRTC unavailable)");
    jit_count_interpreter_launch();
    if (sink == KTC_EXPR_STORE_ONLY) launch_early(k_expr<KTC_EXPR_STORE_ONLY>, dim3((unsigned)grid), dim3(256), d->stream, a);
    else if (sink == KTC_EXPR_SUM_ALL) launch_early(k_expr<KTC_EXPR_SUM_ALL>, dim3((unsigned)grid), dim3(256), d->stream, a);
    else launch_early(k_expr<KTC_EXPR_SUM_ROWS>, dim3((unsigned)grid), dim3(256), d->stream, a);
    return finish_launch_expr("expr");
}

}  // namespace ktc

using namespace ktc;

// sink == KTC_EXPR_MULTI: n_sinks sums described by sink_kinds / sink_outs / means; otherwise the single
// sink (sink, sink_out, mean).
static int expr_eval_impl(Device** scatc_dev, const uint32_t* code, int n_code, const float* imm, int n_imm,
                     const int64_t* shape, int ndim,
                     const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                     const ktc_buf* stores, int n_stores,
                     int sink, ktc_buf sink_out, int mean,
                     const int* sink_kinds, const ktc_buf* sink_outs, const int* means, int n_sinks,
                     const ktc_buf* add_to, const int* add_mode, ktc_p2p comm, const ktc_buf* x_bufs, const int64_t* x_counts, int n_x) {
    if (!code || n_code < 1 || n_code > kExprMaxInstr) return fail(KTC_EINVAL, "ktc_expr_eval: program of %d instructions (1..%d allowed)", n_code, kExprMaxInstr);
    if (n_imm < 0 || n_imm > kExprMaxImm || (n_imm > 0 && !imm)) return fail(KTC_EINVAL, "ktc_expr_eval: %d immediates (at most %d)", n_imm, kExprMaxImm);
    if (n_leaves < 0 || n_leaves > kExprMaxLeaves || n_stores < 0 || n_stores > kExprMaxStores)
        return fail(KTC_EINVAL, "ktc_expr_eval: %d leaves / %d stores (at most %d / %d)", n_leaves, n_stores, kExprMaxLeaves, kExprMaxStores);
    if (ndim < 1 || ndim > KTC_MAX_DIMS || !shape) return fail(KTC_EINVAL, "ktc_expr_eval: bad shape");
    if (sink < KTC_EXPR_STORE_ONLY || sink > KTC_EXPR_MULTI) return fail(KTC_EINVAL, "ktc_expr_eval: unknown sink %d", sink);      // SUM_LAST arrives as a one-sink MULTI
    const bool multi = sink == KTC_EXPR_MULTI;
    if (multi) {
        if (n_sinks < 1 || n_sinks > kExprMaxSinks || !sink_kinds || !sink_outs || !means) return fail(KTC_EINVAL, "ktc_expr_eval_multi: %d sinks (1..%d allowed)", n_sinks, kExprMaxSinks);
        for (int j = 0; j < n_sinks; ++j)
            if (sink_kinds[j] != KTC_EXPR_SUM_ALL && sink_kinds[j] != KTC_EXPR_SUM_ROWS && sink_kinds[j] != KTC_EXPR_SUM_LAST) return fail(KTC_EINVAL, "ktc_expr_eval_multi: sink %d is of unknown kind %d", j, sink_kinds[j]);
            else if (sink_kinds[j] != KTC_EXPR_SUM_ALL && means[j]) return fail(KTC_EINVAL, "ktc_expr_eval_multi: sink %d: only a SUM_ALL sink can be a mean", j);
    }
    const bool keep_inner = sink == KTC_EXPR_SUM_ROWS || multi;      // the innermost dimension of `shape` is not merged
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) { if (shape[i] < 1) return fail(KTC_EINVAL, "ktc_expr_eval: empty iteration space"); total *= shape[i]; }
    if (total > ((int64_t)1 << 40)) return fail(KTC_EINVAL, "ktc_expr_eval: iteration space too large");

    ExprArgs a{};
    Device* d = nullptr; int dev = -1;
    auto adopt = [&](const Buf& b) -> int {
        if (dev < 0) { dev = b.dev; d = device(dev); if (!d) return KTC_ESTATE; return use_device(d); }
        if (b.dev != dev) return fail(KTC_EINVAL, "ktc_expr_eval: buffers live on different devices");
        return KTC_OK;
    };

    // leaf strides through the right-aligned iteration shape (0 where the leaf is broadcast)
    int64_t lstr[kExprMaxLeaves][KTC_MAX_DIMS];
    for (int l = 0; l < n_leaves; ++l) {
        Buf b; KTC_TRY(resolve(leaves[l], &b)); KTC_TRY(adopt(b));
        const int64_t* ls = leaf_shapes + (int64_t)l * ndim;
        int64_t st = 1, vol = 1;
        for (int i = ndim - 1; i >= 0; --i) {
            if (!(ls[i] == shape[i] || ls[i] == 1)) return fail(KTC_EINVAL, "ktc_expr_eval: leaf %d extent %lld does not broadcast to %lld", l, (long long)ls[i], (long long)shape[i]);
            lstr[l][i] = (ls[i] == shape[i] && shape[i] != 1) ? st : 0;
            st *= ls[i]; vol *= ls[i];
        }
        if (b.n < vol) return fail(KTC_EINVAL, "ktc_expr_eval: leaf %d holds %lld floats, %lld needed", l, (long long)b.n, (long long)vol);
        a.leaf[l] = b.ptr;
    }
    for (int s = 0; s < n_stores; ++s) {
        Buf b; KTC_TRY(resolve(stores[s], &b)); KTC_TRY(adopt(b));
        if (b.n < total) return fail(KTC_EINVAL, "ktc_expr_eval: store target %d holds %lld floats, %lld needed", s, (long long)b.n, (long long)total);
        if (!aligned16(b.ptr)) return fail(KTC_ENOTSUP, "ktc_expr_eval: store target is not 16-byte aligned");
        a.store[s] = b.ptr;
    }

    // collapse to [D0, D1, D2]; for SUM_ROWS the innermost dimension of `shape` is the kept one and is not merged
    int64_t S[KTC_MAX_DIMS]; int64_t LS[kExprMaxLeaves][KTC_MAX_DIMS]; int m = 0;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] == 1) continue;
        bool merge = m > 0 && !(keep_inner && i == ndim - 1);
        for (int l = 0; l < n_leaves && merge; ++l) merge = (LS[l][m - 1] == lstr[l][i] * shape[i]);
        if (merge) { S[m - 1] *= shape[i]; for (int l = 0; l < n_leaves; ++l) LS[l][m - 1] = lstr[l][i]; }
        else { S[m] = shape[i]; for (int l = 0; l < n_leaves; ++l) LS[l][m] = lstr[l][i]; ++m; }
    }
    if (m == 0) { S[0] = 1; for (int l = 0; l < n_leaves; ++l) LS[l][0] = 0; m = 1; }
    if (keep_inner && shape[ndim - 1] == 1) return fail(KTC_ENOTSUP, "ktc_expr_eval: SUM_ROWS needs a kept innermost dimension");
    if (m > 3) return fail(KTC_ENOTSUP, "ktc_expr_eval: %d collapsed dimensions (at most 3 are fused)", m);
    int64_t D[3] = {1, 1, 1};
    for (int i = 0; i < m; ++i) D[3 - m + i] = S[i];
    if (D[2] % 4 != 0) return fail(KTC_ENOTSUP, "ktc_expr_eval: innermost extent %lld is not a multiple of 4", (long long)D[2]);
    for (int l = 0; l < n_leaves; ++l) {
        int64_t s3[3] = {0, 0, 0};
        for (int i = 0; i < m; ++i) s3[3 - m + i] = LS[l][i];
        if (s3[2] != 0 && s3[2] != 1) return fail(KTC_ENOTSUP, "ktc_expr_eval: leaf %d is not contiguous along the innermost axis", l);
        if (s3[2] == 1 && (!aligned16(a.leaf[l]) || (s3[0] & 3) || (s3[1] & 3))) return fail(KTC_ENOTSUP, "ktc_expr_eval: leaf %d rows are not 16-byte aligned", l);
        a.ls0[l] = s3[0]; a.ls1[l] = s3[1]; a.ls2[l] = (int)s3[2];
    }
    a.D0 = D[0]; a.D1 = D[1]; a.D2 = D[2];

    // validate the program: register and operand indices, opcodes
    a.n_code = n_code;
    bool has_acc = false, has_scatc = false;
    bool fed[kExprMaxSinks] = {false};
    for (int i = 0; i < n_code; ++i) {
        const uint32_t ins = code[i];
        const int op = ins & 0xff, dreg = (ins >> 8) & 0xf, ra = (ins >> 12) & 0xf, rb = (ins >> 16) & 0xf, k = ins >> 20;
        if (op < KTC_X_LOAD || op > KTC_X_ABS) return fail(KTC_EINVAL, "ktc_expr_eval: unknown opcode %d at %d", op, i);
        if (dreg >= kExprRegs || ra >= kExprRegs || rb >= kExprRegs) return fail(KTC_EINVAL, "ktc_expr_eval: register index out of range at %d", i);
        if (op == KTC_X_LOAD && k >= n_leaves) return fail(KTC_EINVAL, "ktc_expr_eval: LOAD of leaf %d (have %d)", k, n_leaves);
        if (op == KTC_X_STORE && k >= n_stores) return fail(KTC_EINVAL, "ktc_expr_eval: STORE to target %d (have %d)", k, n_stores);
        if (op == KTC_X_SCATC) has_scatc = true;
        if ((op == KTC_X_CONST || op == KTC_X_SCATC || (op >= KTC_X_CMP_LT && op <= KTC_X_CMP_GTE)) && k >= n_imm) return fail(KTC_EINVAL, "ktc_expr_eval: immediate %d (have %d)", k, n_imm);
        if (op == KTC_X_CLAMP && k + 1 >= n_imm) return fail(KTC_EINVAL, "ktc_expr_eval: clamp immediates %d,%d (have %d)", k, k + 1, n_imm);
        if (op == KTC_X_ACC) {
            if (sink == KTC_EXPR_STORE_ONLY) return fail(KTC_EINVAL, "ktc_expr_eval: ACC without a summing sink");
            if (multi) {
                if (k >= n_sinks || fed[k]) return fail(KTC_EINVAL, "ktc_expr_eval_multi: ACC at %d feeds sink %d (%d sinks, one ACC each)", i, k, n_sinks);
                fed[k] = true;
            }
            has_acc = true;
        }
        a.code[i] = ins;
    }
    for (int i = 0; i < n_imm; ++i) a.imm[i] = imm[i];
    if (sink != KTC_EXPR_STORE_ONLY && !has_acc) return fail(KTC_EINVAL, "ktc_expr_eval: a summing sink needs an ACC instruction");
    for (int j = 0; multi && j < n_sinks; ++j) if (!fed[j]) return fail(KTC_EINVAL, "ktc_expr_eval_multi: sink %d has no ACC instruction", j);

    const int64_t rows = D[0] * D[1];
    a.col_tiles = (D[2] / 4 + 31) / 32;
    int64_t seg_rows = tune("expr_item_kb", 32) * 1024 / 512;      // rows of 128 columns per warp
    if (seg_rows < 8) seg_rows = 8;
    // A shard of a strongly scaled step is small: with 32 KB items its grid is one wave and a bit (512 CTAs for 2^25
    // elements on 148 SMs x 3 resident CTAs, the second wave a quarter full: 86 us where 61 us would do).  Items shrink
    // (down to 8 rows) until the grid holds a few waves.
    if (d) {
        const int64_t want = (int64_t)d->sm_count * 3 * tune("expr_min_waves", 4);
        while (seg_rows > 8 && ((rows + seg_rows - 1) / seg_rows + 7) / 8 * a.col_tiles < want) seg_rows /= 2;
    }
    if (seg_rows > rows) seg_rows = rows;
    if ((multi || sink != KTC_EXPR_STORE_ONLY) && rows >= 64) {
        // a summing CTA folds eight segments: spread the rows evenly over whole groups of eight, so that a short row space
        // (256 rows of a batch-norm statistic: four segments of 64) does not leave half of every CTA's warps without work
        const int64_t groups8 = (rows + 8 * seg_rows - 1) / (8 * seg_rows);
        seg_rows = (rows + 8 * groups8 - 1) / (8 * groups8);
    }
    a.seg_rows = seg_rows;
    int64_t Sg = (rows + seg_rows - 1) / seg_rows;

    Buf bout{}; Scratch scratch;
    Buf mout[kExprMaxSinks];
    if (multi) {
        for (int j = 0; j < n_sinks; ++j) {
            KTC_TRY(resolve(sink_outs[j], &mout[j])); KTC_TRY(adopt(mout[j]));
            const int64_t need_out = sink_kinds[j] == KTC_EXPR_SUM_ALL ? 1 : sink_kinds[j] == KTC_EXPR_SUM_ROWS ? D[2] : rows;
            if (mout[j].n < need_out) return fail(KTC_EINVAL, "ktc_expr_eval_multi: output of sink %d holds %lld floats, %lld needed", j, (long long)mout[j].n, (long long)need_out);
        }
        Sg = (Sg + 7) & ~(int64_t)7;
    } else if (sink != KTC_EXPR_STORE_ONLY) {
        KTC_TRY(resolve(sink_out, &bout)); KTC_TRY(adopt(bout));
        const int64_t need_out = sink == KTC_EXPR_SUM_ALL ? 1 : D[2];
        if (bout.n < need_out) return fail(KTC_EINVAL, "ktc_expr_eval: sink output holds %lld floats, %lld needed", (long long)bout.n, (long long)need_out);
        Sg = (Sg + 7) & ~(int64_t)7;
    }
    if (!d) return fail(KTC_EINVAL, "ktc_expr_eval: no buffers given");
    a.S = (int)Sg;
    a.err = d->idx_err;
    if (has_scatc && a.D2 != shape[ndim - 1]) return fail(KTC_ENOTSUP, "ktc_expr_eval: a scatter along the last axis needs that axis uncollapsed");
    if (has_scatc && scatc_dev) *scatc_dev = d;           // the caller reads the index check after the launches

    if (sink == KTC_EXPR_STORE_ONLY) {
        const int64_t grid = (Sg * a.col_tiles + 7) / 8;
        if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "ktc_expr_eval: grid too large");
        return launch_expr(d, a, n_leaves, sink, grid, total);
    }
    const int64_t groups = Sg / 8;
    const int64_t grid = groups * a.col_tiles;
    if (grid > 0x7fffffffLL) return fail(KTC_ENOTSUP, "ktc_expr_eval: grid too large");
    if (multi) {
        // one partial-sum area per sink, laid out as the single-sink launches lay theirs out, then each
        // sink's own second pass
        auto part_size = [&](int kind) { return kind == KTC_EXPR_SUM_ALL ? grid : kind == KTC_EXPR_SUM_ROWS ? groups * D[2] : a.col_tiles * rows; };
        int64_t need = 0;
        for (int j = 0; j < n_sinks; ++j) need += part_size(sink_kinds[j]);
        KTC_TRY(scratch.get(d, need * 2));
        double* base = reinterpret_cast<double*>(scratch.ptr);
        a.n_sinks = n_sinks;
        for (int j = 0; j < n_sinks; ++j) {
            a.sink_kind[j] = sink_kinds[j];
            a.mpart[j] = base;
            base += part_size(sink_kinds[j]);
        }
        // everything that can fail is checked before the first launch
        CombineArgs c{};
        c.n_sinks = n_sinks;
        int blocks = 0;
        for (int j = 0; j < n_sinks; ++j) {
            c.part[j] = a.mpart[j]; c.out[j] = mout[j].ptr; c.divisor[j] = means[j] ? (double)total : 0.0;
            if (sink_kinds[j] == KTC_EXPR_SUM_ALL) { c.mode[j] = 2; c.n_out[j] = 1; c.S[j] = (int)grid; blocks += 1; }
            else if (sink_kinds[j] == KTC_EXPR_SUM_LAST) { c.mode[j] = 1; c.n_out[j] = rows; c.S[j] = (int)a.col_tiles; blocks += (int)((rows + 255) / 256); }
            else if (groups >= 64 || D[2] < 4096) { c.mode[j] = 0; c.n_out[j] = D[2]; c.S[j] = (int)groups; blocks += (int)((D[2] * 32 + 255) / 256); }
            else { c.mode[j] = 1; c.n_out[j] = D[2]; c.S[j] = (int)groups; blocks += (int)((D[2] + 255) / 256); }
            c.block_end[j] = blocks;
            if (add_to && add_to[j]) {
                Buf t; KTC_TRY(resolve(add_to[j], &t)); KTC_TRY(adopt(t));
                if (t.n < c.n_out[j]) return fail(KTC_EINVAL, "ktc_expr_eval_multi_fused: the tensor sink %d is added to holds %lld floats, %lld needed", j, (long long)t.n, (long long)c.n_out[j]);
                if (t.ptr == mout[j].ptr) return fail(KTC_EINVAL, "ktc_expr_eval_multi_fused: sink %d is added to its own output", j);
                c.add_to[j] = t.ptr;
                c.add_mode[j] = add_mode ? add_mode[j] : 1;
                if (c.add_mode[j] != 1 && c.add_mode[j] != 2) return fail(KTC_EINVAL, "ktc_expr_eval_multi_fused: add_mode %d of sink %d (1: add, 2: add to zero)", c.add_mode[j], j);
            }
        }
        if (comm) {
            Device* xd = nullptr;
            KTC_TRY(p2p_prepare(comm, x_bufs, x_counts, n_x, &c.x, &xd));
            if (xd != d) return fail(KTC_EINVAL, "ktc_expr_eval_multi_fused: the communicator lives on another device");
            c.exchange = 1;
        }
        KTC_TRY(launch_expr(d, a, n_leaves, sink, grid, total));
        // the second pass follows the first in the stream, but its launch need not wait for the first to end: it starts early and
        // waits for the first pass itself (griddepcontrol.wait at its top)
        if (tune("expr_overlap_second_pass", 1)) launch_early(k_combine_multi, dim3((unsigned)blocks), dim3(256), d->stream, c);
        else k_combine_multi<<<blocks, 256, 0, d->stream>>>(c);
        KTC_TRY(finish_launch_expr("expr(combine)"));
        return KTC_OK;
    }
    a.divisor = mean ? (double)total : 0.0;
    if (sink == KTC_EXPR_SUM_ALL) {
        a.out = bout.ptr;
        if (grid > 1) { KTC_TRY(scratch.get(d, grid * 2)); a.part = reinterpret_cast<double*>(scratch.ptr); }
        KTC_TRY(launch_expr(d, a, n_leaves, sink, grid, total));
        if (grid > 1) {
            if (mean) k_combine_block<1, SumAcc><<<1, 512, 0, d->stream>>>(a.part, bout.ptr, nullptr, 1, (int)grid, total);
            else      k_combine_block<0, SumAcc><<<1, 512, 0, d->stream>>>(a.part, bout.ptr, nullptr, 1, (int)grid, total);
            KTC_TRY(finish_launch_expr("expr(combine)"));
        }
        return KTC_OK;
    }
    // SUM_ROWS: partial[group][column] then one pass over the groups
    KTC_TRY(scratch.get(d, groups * D[2] * 2));
    a.part = reinterpret_cast<double*>(scratch.ptr);
    KTC_TRY(launch_expr(d, a, n_leaves, sink, grid, total));
    if (groups >= 64 || D[2] < 4096) {
        const int64_t blocks = (D[2] * 32 + 255) / 256;
        k_combine_warp<0, SumAcc><<<(int)blocks, 256, 0, d->stream>>>(a.part, bout.ptr, nullptr, D[2], (int)groups, rows);
    } else {
        k_combine_thread<0, SumAcc><<<(int)((D[2] + 255) / 256), 256, 0, d->stream>>>(a.part, bout.ptr, nullptr, D[2], (int)groups, rows);
    }
    return finish_launch_expr("expr(combine)");
}

static int expr_eval(const uint32_t* code, int n_code, const float* imm, int n_imm,
                     const int64_t* shape, int ndim,
                     const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                     const ktc_buf* stores, int n_stores,
                     int sink, ktc_buf sink_out, int mean,
                     const int* sink_kinds, const ktc_buf* sink_outs, const int* means, int n_sinks,
                     const ktc_buf* add_to = nullptr, const int* add_mode = nullptr, ktc_p2p comm = 0, const ktc_buf* x_bufs = nullptr,
                     const int64_t* x_counts = nullptr, int n_x = 0) {
    Device* scatc_dev = nullptr;
    KTC_TRY(expr_eval_impl(&scatc_dev, code, n_code, imm, n_imm, shape, ndim, leaves, leaf_shapes, n_leaves, stores, n_stores, sink, sink_out, mean,
                           sink_kinds, sink_outs, means, n_sinks, add_to, add_mode, comm, x_bufs, x_counts, n_x));
    if (scatc_dev) return take_index_error(scatc_dev, "Scatter", shape[ndim - 1], ndim - 1);      // a recorded inplaceScatter ran inside the program
    return KTC_OK;
}

extern "C" int ktc_expr_eval(const uint32_t* code, int n_code, const float* imm, int n_imm,
                             const int64_t* shape, int ndim,
                             const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                             const ktc_buf* stores, int n_stores,
                             int sink, ktc_buf sink_out, int mean) {
    if (sink == KTC_EXPR_MULTI) return fail(KTC_EINVAL, "ktc_expr_eval: several sinks go through ktc_expr_eval_multi");
    if (sink == KTC_EXPR_SUM_LAST) {
        const int kind = KTC_EXPR_SUM_LAST;
        return expr_eval(code, n_code, imm, n_imm, shape, ndim, leaves, leaf_shapes, n_leaves, stores, n_stores, KTC_EXPR_MULTI, 0, 0, &kind, &sink_out, &mean, 1);
    }
    return expr_eval(code, n_code, imm, n_imm, shape, ndim, leaves, leaf_shapes, n_leaves, stores, n_stores, sink, sink_out, mean, nullptr, nullptr, nullptr, 0);
}

extern "C" int ktc_expr_eval_multi_fused(const uint32_t* code, int n_code, const float* imm, int n_imm,
                                         const int64_t* shape, int ndim,
                                         const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                                         const ktc_buf* stores, int n_stores,
                                         const int* sink_kinds, const ktc_buf* sink_outs, const int* means, int n_sinks,
                                         const ktc_buf* add_to, const int* add_mode, ktc_p2p comm, const ktc_buf* x_bufs, const int64_t* x_counts, int n_x) {
    if (comm && (!x_bufs || !x_counts || n_x < 1)) return fail(KTC_EINVAL, "ktc_expr_eval_multi_fused: a communicator without tensors to exchange");
    return expr_eval(code, n_code, imm, n_imm, shape, ndim, leaves, leaf_shapes, n_leaves, stores, n_stores, KTC_EXPR_MULTI, 0, 0, sink_kinds, sink_outs, means, n_sinks,
                     add_to, add_mode, comm, x_bufs, x_counts, n_x);
}

extern "C" int ktc_expr_eval_multi(const uint32_t* code, int n_code, const float* imm, int n_imm,
                                   const int64_t* shape, int ndim,
                                   const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves,
                                   const ktc_buf* stores, int n_stores,
                                   const int* sink_kinds, const ktc_buf* sink_outs, const int* means, int n_sinks) {
    return expr_eval(code, n_code, imm, n_imm, shape, ndim, leaves, leaf_shapes, n_leaves, stores, n_stores, KTC_EXPR_MULTI, 0, 0, sink_kinds, sink_outs, means, n_sinks);
}

// The forward of SoftmaxCrossEntropy (ktc_softmax_xent_forward) with an elementwise program as its epilogue: leaf
// `soft_leaf` of the program is the row's softmax while it is still in registers, so a consumer of the saved tensor --
// the function's backward, (softmax with -1 added at the target) / rows, SoftmaxCrossEntropy.kt:61-67 -- runs in the pass
// that reads the logits, and `softmax` may be 0 (not written).  The other leaves are [rows | 1, cols | 1] tensors
// (leaf_shapes: two extents per leaf; the entry of soft_leaf is ignored), STORE k writes stores[k], [rows, cols]; no ACC.
// Every instruction is the reference operation of the stand-alone call, so the stored values are those of the forward
// followed by the separate program.  KTC_ENOTSUP: rows the one-pass kernel does not take, or no run-time compiler -- run
// the two separately.
extern "C" int ktc_softmax_xent_forward_expr(ktc_buf softmax, ktc_buf nll, ktc_buf logits, ktc_buf targets, int64_t rows, int64_t cols, float lo, float hi,
                                             const uint32_t* code, int n_code, const float* imm, int n_imm,
                                             const ktc_buf* leaves, const int64_t* leaf_shapes, int n_leaves, int soft_leaf,
                                             const ktc_buf* stores, int n_stores) {
    const char* me = "ktc_softmax_xent_forward_expr";
    if (rows < 0 || cols < 1) return fail(KTC_EINVAL, "%s: bad shape [%lld, %lld]", me, (long long)rows, (long long)cols);
    if (!code || n_code < 1 || n_code > kExprMaxInstr) return fail(KTC_EINVAL, "%s: program of %d instructions (1..%d allowed)", me, n_code, kExprMaxInstr);
    if (n_imm < 0 || n_imm > kExprMaxImm || (n_imm > 0 && !imm)) return fail(KTC_EINVAL, "%s: %d immediates (at most %d)", me, n_imm, kExprMaxImm);
    if (n_leaves < 1 || n_leaves > kExprMaxLeaves || !leaves || !leaf_shapes || soft_leaf < 0 || soft_leaf >= n_leaves || n_stores < 0 || n_stores > kExprMaxStores || (n_stores && !stores))
        return fail(KTC_EINVAL, "%s: %d leaves (softmax: %d) / %d stores (at most %d / %d)", me, n_leaves, soft_leaf, n_stores, kExprMaxLeaves, kExprMaxStores);
    Buf bs{}, bn, bl, bt;
    if (softmax) KTC_TRY(resolve(softmax, &bs));
    KTC_TRY(resolve(nll, &bn)); KTC_TRY(resolve(logits, &bl)); KTC_TRY(resolve(targets, &bt));
    if ((softmax && bs.dev != bl.dev) || bn.dev != bl.dev || bt.dev != bl.dev) return fail(KTC_EINVAL, "%s: buffers live on different devices", me);
    const int64_t total = rows * cols;
    if (bl.n < total || (softmax && bs.n < total) || bn.n < rows || bt.n < rows) return fail(KTC_EINVAL, "%s: a buffer is too small for [%lld, %lld]", me, (long long)rows, (long long)cols);
    if (softmax && bs.ptr == bl.ptr) return fail(KTC_EINVAL, "%s: softmax aliases logits", me);
    if (!softmax_row_length_ok(cols) || !aligned16(bl.ptr) || (softmax && !aligned16(bs.ptr)))
        return fail(KTC_ENOTSUP, "%s: rows of %lld columns are not handled in one pass", me, (long long)cols);
    if (rows == 0) return KTC_OK;
    ExprArgs a{};
    for (int l = 0; l < n_leaves; ++l) {
        if (l == soft_leaf) { a.leaf[l] = nullptr; a.ls1[l] = cols; a.ls2[l] = 1; continue; }
        Buf b; KTC_TRY(resolve(leaves[l], &b));
        if (b.dev != bl.dev) return fail(KTC_EINVAL, "%s: leaf %d lives on another device", me, l);
        const int64_t r = leaf_shapes[2 * l], c = leaf_shapes[2 * l + 1];
        if ((r != rows && r != 1) || (c != cols && c != 1)) return fail(KTC_EINVAL, "%s: leaf %d of shape [%lld, %lld] does not broadcast to [%lld, %lld]", me, l, (long long)r, (long long)c, (long long)rows, (long long)cols);
        if (b.n < r * c) return fail(KTC_EINVAL, "%s: leaf %d holds %lld floats, %lld needed", me, l, (long long)b.n, (long long)(r * c));
        a.leaf[l] = b.ptr;
        a.ls2[l] = c == cols ? 1 : 0;
        a.ls1[l] = (r == rows && rows != 1) ? c : 0;
        if (a.ls2[l] && !aligned16(b.ptr)) return fail(KTC_ENOTSUP, "%s: leaf %d rows are not 16-byte aligned", me, l);
    }
    for (int k = 0; k < n_stores; ++k) {
        Buf b; KTC_TRY(resolve(stores[k], &b));
        if (b.dev != bl.dev) return fail(KTC_EINVAL, "%s: store target %d lives on another device", me, k);
        if (b.n < total) return fail(KTC_EINVAL, "%s: store target %d holds %lld floats, %lld needed", me, k, (long long)b.n, (long long)total);
        if (!aligned16(b.ptr)) return fail(KTC_ENOTSUP, "%s: store target is not 16-byte aligned", me);
        if (b.ptr == bl.ptr || (softmax && b.ptr == bs.ptr)) return fail(KTC_EINVAL, "%s: store target %d aliases the logits or the softmax", me, k);
        a.store[k] = b.ptr;
    }
    a.n_code = n_code;
    for (int i = 0; i < n_code; ++i) {
        const uint32_t ins = code[i];
        const int op = ins & 0xff, dreg = (ins >> 8) & 0xf, ra = (ins >> 12) & 0xf, rb = (ins >> 16) & 0xf, k = ins >> 20;
        if (op < KTC_X_LOAD || op > KTC_X_ABS || op == KTC_X_ACC) return fail(KTC_EINVAL, "%s: opcode %d at %d", me, op, i);
        if (dreg >= kExprRegs || ra >= kExprRegs || rb >= kExprRegs) return fail(KTC_EINVAL, "%s: register index out of range at %d", me, i);
        if (op == KTC_X_LOAD && k >= n_leaves) return fail(KTC_EINVAL, "%s: LOAD of leaf %d (have %d)", me, k, n_leaves);
        if (op == KTC_X_STORE && k >= n_stores) return fail(KTC_EINVAL, "%s: STORE to target %d (have %d)", me, k, n_stores);
        if ((op == KTC_X_CONST || op == KTC_X_SCATC || (op >= KTC_X_CMP_LT && op <= KTC_X_CMP_GTE)) && k >= n_imm) return fail(KTC_EINVAL, "%s: immediate %d (have %d)", me, k, n_imm);
        if (op == KTC_X_CLAMP && k + 1 >= n_imm) return fail(KTC_EINVAL, "%s: clamp immediates %d,%d (have %d)", me, k, k + 1, n_imm);
        a.code[i] = ins;
    }
    for (int i = 0; i < n_imm; ++i) a.imm[i] = imm[i];
    Device* d = device(bl.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    a.D0 = 1; a.D1 = rows; a.D2 = cols; a.col_tiles = (cols / 4 + 31) / 32; a.seg_rows = 1; a.S = 0;
    a.err = d->idx_err;
    const SxArgs sa{bl.ptr, bt.ptr, bs.ptr, bn.ptr, rows, (int)cols, lo, hi, d->idx_err};
    const int rc = jit_launch_softmax(d, a, n_leaves, soft_leaf, sa);
    if (rc == KTC_ENOTSUP) return fail(KTC_ENOTSUP, "%s: no generated kernel for this program (NVRTC unavailable or the compilation failed)", me);
    KTC_TRY(rc);
    return take_index_error(d, "SoftmaxCrossEntropy target", cols, 1);
}
