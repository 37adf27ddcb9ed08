"""Run-time generated expression kernels, checked where no device is needed: NVRTC compiles for
sm_100a on a machine without a GPU, so the source generator is exercised here for every opcode,
every sink, both row-index forms and programs produced by the deferred-expression compiler."""
import ctypes as C

import pytest

from kten_b200 import _lib as L
from kten_b200 import lazy as Z
from tests.test_lazy_host import FakeLib


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
            ins(L.X_CMP_LTE, 7, 7, k=3), ins(L.X_CMP_GT, 7, 7, k=3), ins(L.X_CMP_GTE, 7, 7, k=3), ins(L.X_MUL, 7, 7, 6)]
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


def test_program_from_the_expression_compiler_compiles():
    """The sharded benchmark step's backward formula, as the deferred layer emits it."""
    lib = FakeLib()
    shape = [4096, 1024]
    x, w, b, g = Z.leaf(lib, 1, shape), Z.leaf(lib, 2, [1, 1024]), Z.leaf(lib, 3, [1024]), Z.leaf(lib, 4, [1])
    bin_ = lambda op, p, q: Z.Node("bin", shape, op, (p, q))
    s = Z.Node("un", shape, L.SIGMOID, (bin_(L.PLUS, bin_(L.TIMES, x, w), b),))
    gp = bin_(L.TIMES, bin_(L.TIMES, Z.Node("bcast", shape, 0, (g,)), Z.const(2.0)), s)       # PowConstant backward
    t = bin_(L.PLUS, Z.Node("un", shape, L.NEG, (s,)), Z.const(1.0))                            # Sigmoid backward
    dz = bin_(L.TIMES, bin_(L.TIMES, t, s), gp)
    prog, _, _ = Z.compile_program(shape, [], bin_(L.TIMES, dz, x), 0)
    inner = [1 if sh[-1] != 1 else 0 for _, sh in prog.leaves]
    fixed = [1 if sh[0] == 1 else 0 for _, sh in prog.leaves]
    nbytes, ms = compile_only(prog.code, inner, fixed, 0, L.EXPR_SUM_ROWS)
    assert ms < 20000


def test_multi_sink_program_compiles():
    """Loss, weight gradient and bias gradient of the sharded step as ONE program with three sinks
    (SUM_ALL mean, SUM_ROWS, SUM_ROWS), as the deferred layer emits it once sums are deferred too."""
    lib = FakeLib()
    shape = [4096, 1024]
    x, w, b, y, g = (Z.leaf(lib, 1, shape), Z.leaf(lib, 2, [1, 1024]), Z.leaf(lib, 3, [1024]), Z.leaf(lib, 5, shape), Z.leaf(lib, 4, [1]))
    bin_ = lambda op, p, q: Z.Node("bin", shape, op, (p, q))
    s = Z.Node("un", shape, L.SIGMOID, (bin_(L.PLUS, bin_(L.TIMES, x, w), b),))
    d = bin_(L.MINUS, s, y)
    loss = Z.Node("square", shape, 0, (d,))
    gp = bin_(L.TIMES, bin_(L.TIMES, Z.Node("bcast", shape, 0, (g,)), Z.const(2.0)), d)
    t = bin_(L.PLUS, Z.Node("un", shape, L.NEG, (s,)), Z.const(1.0))
    dz = bin_(L.TIMES, bin_(L.TIMES, t, s), gp)
    prog, _, _ = Z.compile_program(shape, [], [loss, bin_(L.TIMES, dz, x), dz], 0)
    accs = [(c >> 20) for c in prog.code if (c & 0xff) == L.X_ACC]
    assert sorted(accs) == [0, 1, 2]
    inner = [1 if sh[-1] != 1 else 0 for _, sh in prog.leaves]
    fixed = [1 if sh[0] == 1 else 0 for _, sh in prog.leaves]
    lib_ = L.load()
    code = (C.c_uint32 * len(prog.code))(*prog.code)
    n = len(inner)
    nbytes, ms = C.c_int64(0), C.c_double(0)
    kinds = (C.c_int * 3)(L.EXPR_SUM_ALL, L.EXPR_SUM_ROWS, L.EXPR_SUM_ROWS)
    for rank3 in (0, 1):
        rc = lib_.ktc_test_expr_compile_multi(code, len(prog.code), n, (C.c_int * n)(*inner), (C.c_int * n)(*fixed), rank3, kinds, 3,
                                              C.byref(nbytes), C.byref(ms))
        if rc == L.KTC_ENOTSUP:
            pytest.skip("NVRTC is not installed here: " + lib_.ktc_last_error().decode())
        assert rc == L.KTC_OK, lib_.ktc_last_error().decode()[:4000]
        assert nbytes.value > 1000
    bad = (C.c_int * 1)(L.EXPR_STORE_ONLY)
    assert lib_.ktc_test_expr_compile_multi(code, len(prog.code), n, (C.c_int * n)(*inner), (C.c_int * n)(*fixed), 0, bad, 1, None, None) == L.KTC_EINVAL


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
