// ktc_expr_args.h -- launch parameters of the fused expression kernels.  Shared by the built-in
// interpreter kernel (ktc_expr.cu) and by the kernels generated at run time (ktc_jit.cu), whose
// source embeds this file: plain types only, nothing but <stdint.h> names.
#pragma once

#include "../../include/kten_cuda.h"

namespace ktc {

constexpr int kExprMaxInstr = KTC_EXPR_MAX_INSTR;
constexpr int kExprMaxImm = KTC_EXPR_MAX_IMM;
constexpr int kExprMaxLeaves = KTC_EXPR_MAX_LEAVES;
constexpr int kExprMaxStores = KTC_EXPR_MAX_STORES;
constexpr int kExprRegs = KTC_EXPR_REGS;
constexpr int kExprMaxSinks = KTC_EXPR_MAX_SINKS;

// Iteration space: the collapsed view [D0, D1, D2] of the result shape; a warp owns a 128-column
// tile (lane = 4 columns) of `seg_rows` consecutive rows of the D0*D1 row space.
struct ExprArgs {
    int n_code;
    uint32_t code[kExprMaxInstr];          // op | dst << 8 | a << 12 | b << 16 | k << 20
    float imm[kExprMaxImm];
    const float* leaf[kExprMaxLeaves];
    int64_t ls0[kExprMaxLeaves], ls1[kExprMaxLeaves];
    int ls2[kExprMaxLeaves];               // 0 or 1
    float* store[kExprMaxStores];
    int64_t D0, D1, D2;
    int64_t col_tiles;                     // ceil(D2 / 128)
    int64_t seg_rows;                      // rows (of D0*D1) per warp
    int S;                                 // segments of the row space (multiple of 8 for the summing sinks)
    double* part;                          // partial sums of the summing sinks
    float* out;                            // final result when a single CTA suffices (unused otherwise)
    double divisor;                        // > 0: mean
    // several sums in one pass (KTC_EXPR_MULTI): an ACC instruction's k field names its sink
    int n_sinks;
    int sink_kind[kExprMaxSinks];          // KTC_EXPR_SUM_ALL or KTC_EXPR_SUM_ROWS
    double* mpart[kExprMaxSinks];          // partial sums of each sink
    int* err;                              // device word set when a SCATC instruction meets an index outside its row
};

}  // namespace ktc
