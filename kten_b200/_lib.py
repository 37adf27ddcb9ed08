"""ctypes binding of libkten_cuda.so (the C ABI declared in include/kten_cuda.h).

The library is the product; this module only loads it and declares the
prototypes.  There is no fallback of any kind: if the shared object is missing
the import of the symbol table fails, and if no CUDA device is usable
`ktc_init` fails, each with an error that says so.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkten_cuda.so")

# status codes (include/kten_cuda.h)
KTC_OK, KTC_EINVAL, KTC_ESTATE, KTC_ENOMEM, KTC_ECUDA, KTC_ECOMM, KTC_ETIMEOUT, KTC_ENOTSUP = 0, -1, -2, -3, -4, -5, -6, -7
# op codes
PLUS, MINUS, TIMES, DIV, POW = range(5)
EXP, LOG, TANH, SIGMOID, RECIPROCAL, NEG = range(6)
SUM, MEAN, MAX, MIN, ARGMAX, ARGMIN = range(6)
(SINH, COSH, ABS, SIGN, SQRT, SIN, COS, TAN, ASIN, ACOS, ATAN, FLOOR, CEIL, ROUND, TRUNC, RSQRT) = range(6, 22)
RECORDABLE_UNARY = frozenset(range(0, 6)) | {SQRT, RSQRT, ABS}      # the unary operations that are expression instructions
LT, LTE, GT, GTE, EQ, NEQ = range(6)
SCATTER_SET, SCATTER_ADD, SCATTER_CONST = 0, 1, 2
MAX_DIMS = 10
COPY_ASYNC, COPY_SYNC, COPY_OVERLAP, COPY_OVERLAP_UNFENCED = 0, 1, 2, 3
COMM_ID_BYTES = 128
P2P_HANDLE_BYTES, P2P_MAX_RANKS, P2P_MAX_FLOATS, P2P_MAX_TENSORS = 64, 16, 16384, 8
# fused expression programs (ktc_expr_eval)
(X_LOAD, X_CONST, X_ADD, X_SUB, X_MUL, X_DIV, X_POW, X_NEG, X_RCP, X_SQUARE, X_EXP, X_LOG, X_TANH, X_SIGMOID, X_CLAMP,
 X_CMP_LT, X_CMP_LTE, X_CMP_GT, X_CMP_GTE, X_STORE, X_ACC, X_SCATC, X_SQRT, X_RSQRT, X_ABS) = range(1, 26)
EXPR_STORE_ONLY, EXPR_SUM_ALL, EXPR_SUM_ROWS, EXPR_MULTI, EXPR_SUM_LAST = 0, 1, 2, 3, 4
EXPR_MAX_INSTR, EXPR_MAX_IMM, EXPR_MAX_LEAVES, EXPR_MAX_STORES, EXPR_REGS, EXPR_MAX_SINKS = 32, 16, 8, 3, 8, 4
NOALLOC_SCRATCH_BYTES = 16384
NOALLOC_MAX_ELEMS = 1 << 30

i32, i64, u64, f32 = C.c_int, C.c_int64, C.c_uint64, C.c_float
p_i32, p_i64, p_u64, p_f32 = C.POINTER(i32), C.POINTER(i64), C.POINTER(u64), C.POINTER(f32)

_PROTOTYPES = {
    "ktc_init": (i32, [p_i32]),
    "ktc_shutdown": (i32, []),
    "ktc_device_info": (i32, [i32, C.c_char_p, C.c_size_t, p_i64, p_i32]),
    "ktc_last_error": (C.c_char_p, []),
    "ktc_version": (C.c_char_p, []),
    "ktc_alloc": (i32, [i32, i64, p_u64]),
    "ktc_wrap": (i32, [i32, C.c_void_p, i64, p_u64]),
    "ktc_view": (i32, [u64, i64, i64, p_u64]),
    "ktc_retain": (i32, [u64]),
    "ktc_release": (i32, [u64]),
    "ktc_refcount": (i32, [u64, p_i32]),
    "ktc_buf_info": (i32, [u64, p_i32, p_i64, C.POINTER(C.c_void_p)]),
    "ktc_pool_stats": (i32, [i32, p_i64, p_i64, p_i64, p_i64]),
    "ktc_pool_trim": (i32, [i32]),
    "ktc_pool_limit": (i32, [i32, i64]),
    "ktc_host_alloc": (i32, [i64, C.POINTER(p_f32)]),
    "ktc_host_free": (i32, [p_f32]),
    "ktc_h2d": (i32, [u64, i64, C.c_void_p, i64, i32]),
    "ktc_d2h": (i32, [C.c_void_p, u64, i64, i64, i32]),
    "ktc_d2d": (i32, [u64, i64, u64, i64, i64]),
    "ktc_fill": (i32, [u64, i64, i64, f32]),
    "ktc_sync": (i32, [i32]),
    "ktc_copy_fence": (i32, [i32]),
    "ktc_binary": (i32, [i32, u64, u64, u64, i64]),
    "ktc_binary_bcast": (i32, [i32, u64, u64, p_i64, i32, u64, p_i64, i32]),
    "ktc_binary_inplace": (i32, [i32, u64, u64, i64]),
    "ktc_scalar": (i32, [i32, u64, u64, f32, i64, i32]),
    "ktc_scalar_inplace": (i32, [i32, u64, f32, i64]),
    "ktc_unary": (i32, [i32, u64, u64, i64]),
    "ktc_clamp": (i32, [u64, u64, f32, f32, i64]),
    "ktc_compare_scalar": (i32, [i32, u64, u64, f32, i64]),
    "ktc_compare_scalar_eps": (i32, [i32, u64, u64, f32, f32, i64]),
    "ktc_compare_tensor": (i32, [i32, u64, u64, u64, f32, i64]),
    "ktc_masked_fill": (i32, [u64, u64, p_i64, i32, u64, p_i64, i32, f32]),
    "ktc_contains_nan": (i32, [u64, i64, p_i32]),
    "ktc_copy_strided": (i32, [u64, i64, p_i64, u64, i64, p_i64, p_i64, i32]),
    "ktc_fill_strided": (i32, [u64, i64, p_i64, p_i64, i32, f32]),
    "ktc_gather_axis": (i32, [u64, u64, p_i64, u64, p_i64, i32, i32]),
    "ktc_scatter_axis_nd": (i32, [i32, u64, p_i64, u64, p_i64, u64, p_i64, i32, i32, f32]),
    "ktc_index_select": (i32, [u64, u64, u64, i64, i64, i64, i64]),
    "ktc_index_add": (i32, [u64, u64, u64, f32, i64, i64, i64, i64]),
    "ktc_broadcast_to": (i32, [u64, p_i64, i32, u64, p_i64, i32]),
    "ktc_reduce_axis": (i32, [i32, u64, u64, i64, i64, i64]),
    "ktc_reduce_axis_validx": (i32, [i32, u64, u64, u64, i64, i64, i64]),
    "ktc_reduce_all": (i32, [i32, u64, u64, i64]),
    "ktc_reduce_all_noalloc": (i32, [i32, u64, u64, i64]),
    "ktc_expr_eval": (i32, [C.POINTER(C.c_uint32), i32, p_f32, i32, p_i64, i32, p_u64, p_i64, i32, p_u64, i32, i32, u64, i32]),
    "ktc_expr_stats": (i32, [p_i64]),
    "ktc_expr_jit_log": (i32, [C.c_char_p, i32]),
    "ktc_expr_eval_multi": (i32, [C.POINTER(C.c_uint32), i32, p_f32, i32, p_i64, i32, p_u64, p_i64, i32, p_u64, i32, C.POINTER(C.c_int), p_u64, C.POINTER(C.c_int), i32]),
    "ktc_test_expr_compile_multi": (i32, [C.POINTER(C.c_uint32), i32, i32, C.POINTER(C.c_int), C.POINTER(C.c_int), i32, C.POINTER(C.c_int), i32, p_i64, C.POINTER(C.c_double)]),
    "ktc_test_expr_compile": (i32, [C.POINTER(C.c_uint32), i32, i32, C.POINTER(C.c_int), C.POINTER(C.c_int), i32, i32, p_i64, C.POINTER(C.c_double)]),
    "ktc_lazy_leaf": (i32, [u64, p_i64, i32, p_u64]),
    "ktc_lazy_free": (i32, [u64]),
    "ktc_lazy_unary": (i32, [i32, u64, p_u64]),
    "ktc_lazy_binary": (i32, [i32, u64, u64, p_u64]),
    "ktc_lazy_scalar": (i32, [i32, u64, f32, i32, p_u64]),
    "ktc_lazy_clamp": (i32, [u64, f32, f32, p_u64]),
    "ktc_lazy_compare_scalar": (i32, [i32, u64, f32, p_u64]),
    "ktc_lazy_broadcast_to": (i32, [u64, p_i64, i32, p_u64]),
    "ktc_lazy_assign_binary": (i32, [i32, u64, u64, p_i32]),
    "ktc_lazy_assign_scalar": (i32, [i32, u64, f32, p_i32]),
    "ktc_lazy_sum": (i32, [u64, i32, i32, p_i64, i32, p_u64]),
    "ktc_lazy_buffer": (i32, [u64, p_u64]),
    "ktc_lazy_info": (i32, [u64, p_i32, p_i32, p_i64, p_i32]),
    "ktc_lazy_flush": (i32, [u64]),
    "ktc_lazy_run_pending": (i32, []),
    "ktc_lazy_option": (i32, [C.c_char_p, i32]),
    "ktc_lazy_stats": (i32, [p_i64]),
    "ktc_lazy_allreduce": (i32, [u64, p_u64, i32]),
    "ktc_expr_eval_multi_fused": (i32, [C.POINTER(C.c_uint32), i32, p_f32, i32, p_i64, i32, p_u64, p_i64, i32, p_u64, i32, C.POINTER(C.c_int), p_u64, C.POINTER(C.c_int), i32,
                                        p_u64, p_i32, u64, p_u64, p_i64, i32]),
    "ktc_lazy_full": (i32, [i32, p_i64, i32, f32, p_u64]),
    "ktc_lazy_assign_fill": (i32, [u64, f32, p_i32]),
    "ktc_lazy_assign_scatter_const": (i32, [u64, u64, f32, p_i32]),
    "ktc_lazy_softmax_xent_forward": (i32, [u64, u64, f32, f32, p_u64, p_u64]),
    "ktc_softmax_xent_forward": (i32, [u64, u64, u64, u64, i64, i64, f32, f32]),
    "ktc_softmax_xent_forward_expr": (i32, [u64, u64, u64, u64, i64, i64, f32, f32, C.POINTER(C.c_uint32), i32, C.POINTER(C.c_float), i32,
                                            C.POINTER(u64), p_i64, i32, i32, C.POINTER(u64), i32]),
    "ktc_test_softmax_expr_compile": (i32, [C.POINTER(C.c_uint32), i32, i32, C.POINTER(C.c_int), C.POINTER(C.c_int), i32, i32, p_i64, C.POINTER(C.c_double)]),
    "ktc_upsample2d_nearest": (i32, [u64, u64, i64, i64, i32]),
    "ktc_upsample2d_nearest_grad": (i32, [u64, u64, i64, i64, i32]),
    "ktc_pool2d_max": (i32, [u64, u64, u64, i64, C.POINTER(C.c_int)]),
    "ktc_pool2d_max_grad": (i32, [u64, u64, u64, i64, C.POINTER(C.c_int)]),
    "ktc_pool2d_avg": (i32, [u64, u64, i64, C.POINTER(C.c_int), i32]),
    "ktc_pool2d_avg_grad": (i32, [u64, u64, i64, C.POINTER(C.c_int), i32]),
    "ktc_sum_to_shape": (i32, [u64, p_i64, i32, u64, p_i64, i32]),
    "ktc_scatter_axis": (i32, [u64, u64, u64, i64, i64, i64]),
    "ktc_comm_unique_id": (i32, [C.c_char_p]),
    "ktc_comm_init_rank": (i32, [i32, i32, i32, C.c_char_p, p_u64]),
    "ktc_allreduce_sum": (i32, [u64, u64, i64, i64]),
    "ktc_comm_destroy": (i32, [u64]),
    "ktc_p2p_create": (i32, [i32, i32, i32, p_u64, C.c_char_p]),
    "ktc_p2p_connect": (i32, [u64, C.c_char_p]),
    "ktc_p2p_allreduce_sum": (i32, [u64, p_u64, p_i64, i32]),
    "ktc_p2p_status": (i32, [u64, p_i32]),
    "ktc_p2p_destroy": (i32, [u64]),
    "ktc_test_p2p_connect_self": (i32, [u64]),
    "ktc_timer_start": (i32, [i32]),
    "ktc_timer_stop": (i32, [i32, p_f32]),
    "ktc_launch_count": (i64, []),
    "ktc_flush_l2": (i32, [i32]),
    "ktc_tune_set": (i32, [C.c_char_p, i32]),
    "ktc_test_inject_comm_error": (i32, [i32]),
    "ktc_test_bounded_wait": (i32, [i32, i64, p_i32]),
}

_lib = None


class KtenCudaError(RuntimeError):
    """A KTC_E* status from the library; `.status` holds the code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}] {message}")
        self.status = status


def _preload_newest_nccl() -> None:
    """libkten_cuda.so binds `libnccl.so.2` with dlopen at its first collective call, and a process holds one
    library per soname.  Where a Python environment ships its own NCCL next to PyTorch (the `nvidia.nccl`
    wheel), that copy must be the one in the process: if the system's older libnccl were picked up first, a
    later `import torch` in the same process would fail on the symbols it lacks.  Loading the wheel's copy
    here (when there is one) makes the order of imports irrelevant; without the wheel the system library is
    used."""
    import importlib.util
    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        spec = None
    for base in (spec.submodule_search_locations if spec is not None and spec.submodule_search_locations else []):
        path = os.path.join(base, "lib", "libnccl.so.2")
        if os.path.exists(path):
            try:
                C.CDLL(path, mode=C.RTLD_GLOBAL if hasattr(C, "RTLD_GLOBAL") else 0)
            except OSError:
                pass
            return


def load() -> C.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m kten_b200.build` "
            "(nvcc, sm_100a).  kten_b200 has no CPU or PyTorch fallback.")
    _preload_newest_nccl()
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL if hasattr(C, "RTLD_GLOBAL") else 0)
    for name, (res, args) in _PROTOTYPES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    """Map a negative status to the exception the JVM backend would throw:
    KTC_EINVAL -> ValueError (IllegalArgumentException), KTC_ESTATE ->
    RuntimeError (IllegalStateException), KTC_ENOMEM -> MemoryError."""
    if status == KTC_OK:
        return
    msg = load().ktc_last_error().decode("utf-8", "replace")
    if status == KTC_EINVAL:
        raise ValueError(msg)
    if status == KTC_ENOMEM:
        raise MemoryError(msg)
    if status == KTC_ETIMEOUT:
        raise TimeoutError(msg)
    raise KtenCudaError(status, msg)


def shape_array(shape):
    arr = (i64 * max(len(shape), 1))(*shape)
    return arr, len(shape)
