// ktc_jit.hpp -- run-time generated variants of the fused expression kernel (ktc_jit.cu).
#pragma once

#include "ktc_expr_args.h"
#include "ktc_internal.hpp"

namespace ktc {

// Launches the kernel generated for a's program on d's compute stream with the grid of k_expr.
// KTC_OK: launched.  KTC_ENOTSUP: no generated kernel for this program (NVRTC missing, compilation
// failed): the caller runs the interpreter kernel.  Other codes: launch errors.
int jit_launch(Device* d, const ExprArgs& a, int n_leaves, int sink, int64_t grid);
void jit_count_interpreter_launch();

// The softmax row kernel (ktc_softmax.cuh) generated with a's program as its epilogue: leaf `soft_leaf` of the program
// is the row's softmax, in registers.  Same return codes.
struct SxArgs;
bool softmax_row_length_ok(int64_t cols);
bool softmax_row_takes_cta(int64_t cols);           // ktc_softmax.cu: one CTA per row (sx_rows_cta) instead of one warp          // ktc_softmax.cu: the row lengths the one-pass kernels take
int jit_launch_softmax(Device* d, const ExprArgs& a, int n_leaves, int soft_leaf, const SxArgs& sa);

}  // namespace ktc
