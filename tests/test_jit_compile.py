"""Run-time generated expression kernels, checked where no device is needed: NVRTC compiles for
sm_100a on a machine without a GPU, so the source generator is exercised here for every opcode,
every sink, both row-index forms and programs produced by the deferred-expression compiler."""
import ctypes as C

import pytest

import numpy as np

from kten_b200 import _lib as L
from tests import fake_lib


def ins(op, d=0, a=0, b=0, k=0):
    return op | (d << 8) | (a << 12) | (b << 16) | (k << 20)


def compile_only(prog, inner, fixed, rank3, sink):
    lib = L.load()
    code = (C.c_uint32 * len(prog))(*prog)
    n = len(inner)
    nbytes, ms = C.c_int64(0), C.c_double(0)
    rc = lib.ktc_test_expr_compile(code, len(prog), n, (C.c_int * max(1, n))(*inner), (C.c_int * max(1, n))(*fixed),
                                   rank3, sink, C.byref(nbytes), C.byref(ms))
    if rc == L.KTC_ENOTSUP:
        pytest.skip("NVRTC is not installed here: " + lib.ktc_last_error().decode())
    assert rc == L.KTC_OK, lib.ktc_last_error().decode()[:4000]
    assert nbytes.value > 1000
    return nbytes.value, ms.value


def test_every_opcode_compiles_for_every_sink():
    body = [ins(L.X_LOAD, 0, k=0), ins(L.X_LOAD, 1, k=1), ins(L.X_LOAD, 2, k=2), ins(L.X_CONST, 3, k=0),
            ins(L.X_ADD, 4, 0, 1), ins(L.X_SUB, 4, 4, 2), ins(L.X_MUL, 4, 4, 3), ins(L.X_DIV, 4, 4, 1), ins(L.X_POW, 5, 0, 4),
            ins(L.X_NEG, 5, 5), ins(L.X_RCP, 5, 5), ins(L.X_SQUARE, 5, 5), ins(L.X_EXP, 6, 5), ins(L.X_LOG, 6, 6),
            ins(L.X_TANH, 6, 6), ins(L.X_SIGMOID, 6, 6), ins(L.X_CLAMP, 6, 6, k=1), ins(L.X_CMP_LT, 7, 6, k=3),
            ins(L.X_CMP_LTE, 7, 7, k=3), ins(L.X_CMP_GT, 7, 7, k=3), ins(L.X_CMP_GTE, 7, 7, k=3), ins(L.X_MUL, 7, 7, 6),
            ins(L.X_ABS, 6, 6), ins(L.X_SQRT, 6, 6), ins(L.X_RSQRT, 6, 6), ins(L.X_ADD, 7, 7, 6)]
    for sink, tail in ((L.EXPR_STORE_ONLY, [ins(L.X_STORE, a=7, k=0), ins(L.X_STORE, a=4, k=1)]),
                       (L.EXPR_SUM_ALL, [ins(L.X_STORE, a=4, k=0), ins(L.X_ACC, a=7)]),
                       (L.EXPR_SUM_ROWS, [ins(L.X_ACC, a=7)])):
        for rank3 in (0, 1):
            compile_only(body + tail, inner=[1, 1, 0], fixed=[0, 1, 0], rank3=rank3, sink=sink)


def test_ill_formed_program_is_rejected():
    lib = L.load()
    prog = [ins(L.X_ADD, 0, 1, 2), ins(L.X_STORE, a=0, k=0)]           # reads registers nothing wrote
    code = (C.c_uint32 * 2)(*prog)
    rc = lib.ktc_test_expr_compile(code, 2, 0, None, None, 0, L.EXPR_STORE_ONLY, None, None)
    assert rc == L.KTC_EINVAL
    bad = (C.c_uint32 * 1)(ins(77))
    assert lib.ktc_test_expr_compile(bad, 1, 0, None, None, 0, L.EXPR_STORE_ONLY, None, None) == L.KTC_EINVAL


def recorded_step(one_pass: bool):
    """The sharded benchmark step -- loss = sum(sigmoid(x*w + b) pow 2), backward for w and b -- issued through
    the autograd caller over the stand-in library with everything deferred; returns the programs the recorder
    handed to ktc_expr_eval."""
    ops = fake_lib.make_ops()
    ops.lazy, ops.deferSums = True, one_pass
    rng = np.random.default_rng(3)
    shape = [32, 64]
    from kten_b200.sharded import ShardedSigmoidGraph
    x = ops.createRaw(shape, rng.uniform(-1, 1, shape).astype(np.float32))
    w = ops.createRaw([1, 64], rng.normal(0, 0.02, [1, 64]).astype(np.float32))
    b = ops.createRaw([64], np.zeros(64, np.float32))
    graph = ShardedSigmoidGraph(ops, x, w, b)
    with ops.garbageCollector():
        for r in graph.step():
            r.toArray()
        graph.release_step()
    return ops.lib.programs


def flags(prog):
    inner = [1 if sh[-1] != 1 else 0 for sh in prog["leaf_shapes"]]
    fixed = [1 if sh[0] == 1 else 0 for sh in prog["leaf_shapes"]]
    return inner, fixed


def test_program_from_the_expression_compiler_compiles():
    """The step's backward formula with its leading-axis sum, as the recorder emits it (one sum per pass)."""
    progs = [p for p in recorded_step(one_pass=False) if p["sink"] == L.EXPR_SUM_ROWS]
    assert progs
    prog = max(progs, key=lambda p: len(p["code"]))
    inner, fixed = flags(prog)
    nbytes, ms = compile_only(prog["code"], inner, fixed, 0, L.EXPR_SUM_ROWS)
    assert ms < 20000


def test_multi_sink_program_compiles():
    """Loss, weight gradient and bias gradient of the step as ONE program with three sinks (SUM_ALL, SUM_ROWS,
    SUM_ROWS), as the recorder emits it once sums are deferred too."""
    progs = [p for p in recorded_step(one_pass=True) if p["sinks"] and len(p["sinks"]) == 3]
    assert len(progs) == 1
    prog = progs[0]
    accs = [(c >> 20) for c in prog["code"] if (c & 0xff) == L.X_ACC]
    assert sorted(accs) == [0, 1, 2]
    assert sorted(k for k, _, _ in prog["sinks"]) == [L.EXPR_SUM_ALL, L.EXPR_SUM_ROWS, L.EXPR_SUM_ROWS]
    inner, fixed = flags(prog)
    lib_ = L.load()
    code = (C.c_uint32 * len(prog["code"]))(*prog["code"])
    n = len(inner)
    nbytes, ms = C.c_int64(0), C.c_double(0)
    kinds = (C.c_int * 3)(*[k for k, _, _ in prog["sinks"]])
    for rank3 in (0, 1):
        rc = lib_.ktc_test_expr_compile_multi(code, len(prog["code"]), n, (C.c_int * n)(*inner), (C.c_int * n)(*fixed), rank3, kinds, 3,
                                              C.byref(nbytes), C.byref(ms))
        if rc == L.KTC_ENOTSUP:
            pytest.skip("NVRTC is not installed here: " + lib_.ktc_last_error().decode())
        assert rc == L.KTC_OK, lib_.ktc_last_error().decode()[:4000]
        assert nbytes.value > 1000
    bad = (C.c_int * 1)(L.EXPR_STORE_ONLY)
    assert lib_.ktc_test_expr_compile_multi(code, len(prog["code"]), n, (C.c_int * n)(*inner), (C.c_int * n)(*fixed), 0, bad, 1, None, None) == L.KTC_EINVAL


def test_last_axis_sum_sink_compiles():
    """exp(x - rowmax) with its row sums (the first softmax normalisation), alone and beside other sums."""
    body = [ins(L.X_LOAD, 0, k=0), ins(L.X_LOAD, 1, k=1), ins(L.X_SUB, 2, 0, 1), ins(L.X_EXP, 3, 2), ins(L.X_STORE, a=3, k=0)]
    lib = L.load()
    for kinds, tail in (((L.EXPR_SUM_LAST,), [ins(L.X_ACC, a=3, k=0)]),
                        ((L.EXPR_SUM_LAST, L.EXPR_SUM_ALL), [ins(L.X_ACC, a=3, k=0), ins(L.X_ACC, a=2, k=1)]),
                        ((L.EXPR_SUM_ROWS, L.EXPR_SUM_LAST, L.EXPR_SUM_LAST), [ins(L.X_ACC, a=3, k=0), ins(L.X_ACC, a=3, k=1), ins(L.X_ACC, a=2, k=2)])):
        prog = body + tail
        code = (C.c_uint32 * len(prog))(*prog)
        for rank3 in (0, 1):
            nbytes = C.c_int64(0)
            rc = lib.ktc_test_expr_compile_multi(code, len(prog), 2, (C.c_int * 2)(1, 0), (C.c_int * 2)(0, 0), rank3,
                                                 (C.c_int * len(kinds))(*kinds), len(kinds), C.byref(nbytes), None)
            if rc == L.KTC_ENOTSUP:
                pytest.skip("NVRTC is not installed here: " + lib.ktc_last_error().decode())
            assert rc == L.KTC_OK, lib.ktc_last_error().decode()[:4000]
            assert nbytes.value > 1000


@pytest.mark.parametrize("cols", [2048, 1024, 512, 640, 4096, 12288])
def test_softmax_row_kernel_with_an_epilogue_program_compiles(cols):
    """The generated form of the softmax forward (ktc_softmax_xent_forward_expr): the backward of SoftmaxCrossEntropy as
    its epilogue -- (0 with -1 at the target + softmax) / rows, then the accumulation into a zeroed gradient -- and a
    program that touches every other kind of leaf, for each row-length specialisation."""
    lib = L.load()
    # leaves: 0 targets [rows, 1], 1 the softmax (registers), 2 a row vector [1, cols], 3 a [rows, cols] tensor, 4 a scalar [1, 1]
    prog = [ins(L.X_CONST, 0, k=0), ins(L.X_LOAD, 1, k=0), ins(L.X_SCATC, 0, 0, 1, k=1), ins(L.X_LOAD, 1, k=1), ins(L.X_ADD, 0, 0, 1),
            ins(L.X_CONST, 1, k=2), ins(L.X_DIV, 0, 0, 1), ins(L.X_CONST, 1, k=0), ins(L.X_ADD, 0, 1, 0), ins(L.X_STORE, a=0, k=0),
            ins(L.X_LOAD, 2, k=2), ins(L.X_MUL, 2, 2, 0), ins(L.X_LOAD, 3, k=3), ins(L.X_SUB, 2, 2, 3), ins(L.X_LOAD, 3, k=4), ins(L.X_MUL, 2, 2, 3),
            ins(L.X_EXP, 2, 2), ins(L.X_STORE, a=2, k=1)]
    code = (C.c_uint32 * len(prog))(*prog)
    inner, fixed = (C.c_int * 5)(0, 1, 1, 1, 0), (C.c_int * 5)(0, 0, 1, 0, 1)
    nbytes, ms = C.c_int64(0), C.c_double(0)
    rc = lib.ktc_test_softmax_expr_compile(code, len(prog), 5, inner, fixed, 1, cols, C.byref(nbytes), C.byref(ms))
    if rc == L.KTC_ENOTSUP:
        pytest.skip("NVRTC is not installed here: " + lib.ktc_last_error().decode())
    assert rc == L.KTC_OK, lib.ktc_last_error().decode()[:4000]
    assert nbytes.value > 1000
    acc = (C.c_uint32 * 2)(ins(L.X_LOAD, 0, k=1), ins(L.X_ACC, a=0))
    assert lib.ktc_test_softmax_expr_compile(acc, 2, 5, inner, fixed, 1, cols, None, None) == L.KTC_EINVAL
