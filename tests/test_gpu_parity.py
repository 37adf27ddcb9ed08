"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a real GPU.

Bars (kten-jvm is the target semantics):
  + - * /, compares, clamp, max/min, arg indices, shapes ...... bit-exact
  pow / exp / log / tanh / sigmoid ............................. <= 2 ulp
  sum / mean / sum-to-shape .................................... |err| <= 1e-5 * sum(|x|)  (bit-exact on exact data)
"""
import ctypes as C
import itertools
import os

import numpy as np
import pytest

from kten_b200 import _lib as L
from kten_b200 import autograd as AG
from kten_b200 import datagen as D
from oracle import oracle as O
from tests.kten_cases import CASES, CASE_IDS, run_case

pytestmark = pytest.mark.gpu

ULP_TOL = 2                  # transcendental functions, in units in the last place
RED_RTOL = 1e-5              # reductions, relative to sum(|x|)
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_fixtures.npz"))

BIN = {"plus": (L.PLUS, O.PLUS), "minus": (L.MINUS, O.MINUS), "times": (L.TIMES, O.TIMES), "div": (L.DIV, O.DIV), "pow": (L.POW, O.POW)}
UN = {"exp": (L.EXP, O.EXP), "log": (L.LOG, O.LOG), "tanh": (L.TANH, O.TANH), "sigmoid": (L.SIGMOID, O.SIGMOID),
      "reciprocal": (L.RECIPROCAL, O.RECIPROCAL), "neg": (L.NEG, O.NEG)}
RED = {"sum": (L.SUM, O.SUM), "mean": (L.MEAN, O.MEAN), "max": (L.MAX, O.MAX), "min": (L.MIN, O.MIN),
       "argmax": (L.ARGMAX, O.ARGMAX), "argmin": (L.ARGMIN, O.ARGMIN)}
EXACT_BIN = ("plus", "minus", "times", "div")


def same_bits(a, b):
    a = np.asarray(a, dtype=np.float32).reshape(-1)
    b = np.asarray(b, dtype=np.float32).reshape(-1)
    both_nan = np.isnan(a) & np.isnan(b)
    return bool(np.all((a.view(np.uint32) == b.view(np.uint32)) | both_nan))


def check_elementwise(name, got, want):
    if name in EXACT_BIN or name in ("reciprocal", "neg"):
        assert same_bits(got, want), f"{name}: not bit-exact"
    else:
        d = O.ulp_distance(got, want)
        assert d.max(initial=0) <= ULP_TOL, f"{name}: {d.max()} ulp at {int(d.argmax())}"


def special_values():
    return np.array([0.0, -0.0, 1.0, -1.0, 0.5, 2.0, 3.0, -2.0, 1e-45, -1e-45, 1e-38, 1.17549435e-38, 3.4028235e38,
                     -3.4028235e38, np.inf, -np.inf, np.nan, 88.0, -88.0, 89.0, -104.0, 0.1, 10.0, 1e-20, 1e20, 7.5, -7.5,
                     16.0, 1e-3, -1e-3, 0.99999994, 1.0000001], dtype=np.float32)


# --------------------------------------------------------------------------------------
# the reference's own known-answer tests, on the CUDA backend
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_reference_vectors_on_cuda(cuda_ops, gc_scope, case):
    run_case(cuda_ops, case)


# --------------------------------------------------------------------------------------
# contiguous elementwise
# --------------------------------------------------------------------------------------
SIZES = [1, 2, 3, 4, 5, 7, 255, 1024, 1027, 4096, 65537, (1 << 20) + 3]


@pytest.mark.parametrize("name", list(BIN))
def test_binary_same_shape(cuda_ops, gc_scope, name):
    k, o = BIN[name]
    for n in SIZES:
        a, b = D.uniform(n, 1, 0.1, 2.0), D.uniform(n, 2, 0.1, 2.0)
        if name != "pow":
            a = a - np.float32(1.0)                      # mixed signs for the exact ops
        ra, rb = cuda_ops.createRaw([n], a), cuda_ops.createRaw([n], b)
        got = ra._binary(k, rb).toArray()
        check_elementwise(name, got, O.binary_same(o, a, b))


@pytest.mark.parametrize("name", list(BIN))
def test_binary_special_values(cuda_ops, gc_scope, name):
    k, o = BIN[name]
    sv = special_values()
    a = np.repeat(sv, sv.size)
    b = np.tile(sv, sv.size)
    got = cuda_ops.createRaw([a.size], a)._binary(k, cuda_ops.createRaw([b.size], b)).toArray()
    check_elementwise(name, got, O.binary_same(o, a, b))


@pytest.mark.parametrize("name", list(BIN))
def test_binary_inplace_and_scalar(cuda_ops, gc_scope, name):
    k, o = BIN[name]
    n = 10007
    a, b = D.uniform(n, 11, 0.1, 2.0), D.uniform(n, 12, 0.1, 2.0)
    ra, rb = cuda_ops.createRaw([n], a), cuda_ops.createRaw([n], b)
    ra._binary_assign(k, rb)
    check_elementwise(name, ra.toArray(), O.binary_same(o, a, b))
    for s in (2.0, 0.5, -1.25, 3.0, 1.0, 0.0):
        rc = cuda_ops.createRaw([n], a)
        check_elementwise(name, rc._scalar(k, s).toArray(), O.scalar(o, a, s))
        check_elementwise(name, rc._scalar(k, s, scalar_first=True).toArray(), O.scalar(o, a, s, scalar_first=True))
        rc._scalar_assign(k, s)
        check_elementwise(name, rc.toArray(), O.scalar(o, a, s))


def test_inplace_rejects_unequal_shapes(cuda_ops, gc_scope):
    a, b = cuda_ops.createRaw([2, 3]), cuda_ops.createRaw([3])
    with pytest.raises(ValueError, match="Shapes does not match for inplace operation"):
        a.plusAssign(b)


@pytest.mark.parametrize("name", list(UN))
def test_unary(cuda_ops, gc_scope, name):
    k, o = UN[name]
    for n in SIZES:
        a = D.uniform(n, 5, 0.1, 2.0)
        check_elementwise(name, cuda_ops.createRaw([n], a)._unary(k).toArray(), O.unary(o, a))
    wide = np.concatenate([special_values(), D.uniform(200000, 6, -20.0, 20.0), D.normal(200000, 7, 0.0, 1e-3),
                           D.uniform(50000, 8, -100.0, 100.0)])
    check_elementwise(name, cuda_ops.createRaw([wide.size], wide)._unary(k).toArray(), O.unary(o, wide))


def test_clamp_and_compares(cuda_ops, gc_scope):
    x = np.concatenate([special_values(), D.uniform(5000, 9, -2.0, 2.0)])
    r = cuda_ops.createRaw([x.size], x)
    for lo, hi in ((-0.5, 0.5), (0.15, 0.55), (-0.0, 0.0), (0.0, -0.0), (-np.inf, np.inf)):
        assert same_bits(r.clamp(lo, hi).toArray(), O.clamp(x, lo, hi))
    oracle_r = O.OracleTensorOperations().createRaw([x.size], x)
    for cmp in ("lt", "lte", "gt", "gte"):
        for v in (0.0, 0.5, -1.0):
            assert same_bits(getattr(r, cmp)(v).toArray(), getattr(oracle_r, cmp)(v).toArray())


# --------------------------------------------------------------------------------------
# broadcast elementwise
# --------------------------------------------------------------------------------------
def bcast_pairs():
    pairs = [([32, 64, 128], [64, 1]), ([32, 64, 128], [128]), ([8, 16, 64], [1, 16, 1]), ([8, 16, 64], [8, 1, 64]),
             ([64, 1], [32, 64, 128]), ([128], [32, 64, 128]), ([6, 8, 12], [8, 1]), ([6, 8, 12], [12]), ([6, 8, 12], [6, 1, 12]),
             ([3, 1], [1, 4]), ([4, 1, 8], [1, 5, 1]), ([1], [7, 9]), ([7, 9], [1]), ([5, 4], [5, 4]), ([2, 3, 4, 5, 6], [3, 1, 5, 1]),
             ([2, 1, 3, 1, 2, 1, 3], [1, 2, 1, 3, 1, 2, 1]), ([16, 1024], [1, 1024]), ([16, 1024], [1024]), ([16, 1024], [16, 1]),
             ([4, 4100], [4100]), ([3, 5000, 8], [5000, 1]), ([2, 3, 8192], [3, 1]), ([2, 2, 2, 2, 2, 2, 2, 2, 2, 4], [2, 1, 2, 1, 2, 1, 2, 1, 4])]
    dims = (1, 2, 3, 5)
    for sa in itertools.product(dims, repeat=3):
        for mask in range(1, 8):
            sb = [1 if (mask >> i) & 1 else sa[i] for i in range(3)]
            pairs.append((list(sa), sb))
    return pairs


@pytest.mark.parametrize("name", EXACT_BIN)
def test_broadcast_patterns(cuda_ops, gc_scope, name):
    k, o = BIN[name]
    for i, (sa, sb) in enumerate(bcast_pairs()):
        a = D.uniform(O.volume(sa), 100 + i, 0.5, 2.0)
        b = D.uniform(O.volume(sb), 200 + i, 0.5, 2.0)
        got = cuda_ops.createRaw(sa, a)._binary(k, cuda_ops.createRaw(sb, b))
        want, cs = O.binary(o, a, sa, b, sb)
        assert got.shape == cs
        assert same_bits(got.toArray(), want), f"{name} {sa} x {sb}"


def test_broadcast_pow_and_tile_settings(cuda_ops, gc_scope):
    lib = cuda_ops.lib
    sa, sb, sc = [8, 33, 64], [1, 33, 1], [8, 1, 64]
    a, b, c = D.uniform(O.volume(sa), 1, 0.1, 2.0), D.uniform(33, 2, 0.5, 2.0), D.uniform(512, 3, 0.1, 2.0)
    ra, rb, rc = cuda_ops.createRaw(sa, a), cuda_ops.createRaw(sb, b), cuda_ops.createRaw(sc, c)
    try:
        for tile, cols, generic in ((8192, 2048, 0), (256, 16, 0), (64, 64, 0), (8192, 2048, 1)):
            lib.ktc_tune_set(b"bcast_tile_elems", tile); lib.ktc_tune_set(b"bcast_max_cols", cols)
            lib.ktc_tune_set(b"bcast_force_generic", generic)
            assert same_bits(ra.times(rb).toArray(), O.binary(O.TIMES, a, sa, b, sb)[0])
            assert same_bits(ra.plus(rc).toArray(), O.binary(O.PLUS, a, sa, c, sc)[0])
            assert same_bits(rb.minus(rc).toArray(), O.binary(O.MINUS, b, sb, c, sc)[0])
            d = O.ulp_distance(ra.pow(rc).toArray(), O.binary(O.POW, a, sa, c, sc)[0])
            assert d.max() <= ULP_TOL
    finally:
        lib.ktc_tune_set(b"bcast_tile_elems", 8192); lib.ktc_tune_set(b"bcast_max_cols", 2048)
        lib.ktc_tune_set(b"bcast_force_generic", 0)


def test_broadcast_division_by_row_scalars(cuda_ops, gc_scope):
    """a[I, J, K] / b[1, J, 1] divides by the rows' reciprocals where that is the IEEE quotient and by IEEE division
    elsewhere: dividends and divisors of every kind (zeros of both signs, subnormals, huge, tiny, infinite, NaN,
    negative), each divisor meeting each dividend, both batch sizes of the kernel, also as the scalar-first form
    b / a, which must keep the ordinary path."""
    lib = cuda_ops.lib
    sv = special_values()
    extra = np.array([1e-19, -1e-19, 1.0842e-19, 1.8e19, -1.8e19, 9.2e18, 2.0 ** -63, 2.0 ** 64, 2.0 ** 63.5, 2.0 ** -64,
                      1e-30, 1e30, 3.0, 1.0 / 3.0, 0.99999994, 5e-39], dtype=np.float32)
    vals = np.concatenate([sv, extra, D.normal(80, 5, 0.0, 1.0)])                    # 128 values
    J, K = vals.size, 64
    divisors = np.concatenate([sv, extra, np.array([2.0 ** -60, 2.0 ** 60, 2.0 ** -61, 2.0 ** 61, -(2.0 ** 60)], dtype=np.float32),
                               D.uniform(J - sv.size - extra.size - 5, 6, 0.5, 2.0)]).astype(np.float32)
    a = np.empty((3, J, K), dtype=np.float32)
    for i in range(3):
        for j in range(J):
            a[i, j] = np.roll(vals, i * 7 + j)[:K]                                   # every divisor meets many kinds of dividends
    a[1, :, :vals.size // 2] = vals[None, ::2]
    a = a.reshape(-1)
    ra, rb = cuda_ops.createRaw([3, J, K], a), cuda_ops.createRaw([1, J, 1], divisors)
    want = O.binary(O.DIV, a, [3, J, K], divisors, [1, J, 1])[0]
    want_rev = O.binary(O.DIV, divisors, [1, J, 1], a, [3, J, K])[0]
    try:
        for batch in (8, 4):
            lib.ktc_tune_set(b"bcast_div_batch", batch)
            assert same_bits(ra.div(rb).toArray(), want), batch
            assert same_bits(rb.div(ra).toArray(), want_rev), batch
    finally:
        lib.ktc_tune_set(b"bcast_div_batch", 8)
    big = D.normal(64 * 1024 * 256, 9, 0.0, 1.0)
    big[::1000] = 0.0
    bdiv = D.uniform(1024, 10, 0.5, 2.0)
    got = cuda_ops.createRaw([64, 1024, 256], big).div(cuda_ops.createRaw([1, 1024, 1], bdiv)).toArray()
    assert same_bits(got, O.binary(O.DIV, big, [64, 1024, 256], bdiv, [1, 1024, 1])[0])


def test_broadcast_shape_mismatch_is_rejected(cuda_ops, gc_scope):
    a, b = cuda_ops.createRaw([2, 3]), cuda_ops.createRaw([4, 3])
    with pytest.raises(ValueError, match="non-singleton"):
        a.plus(b)
    h = C.c_uint64(0)
    sa, na = L.shape_array([2, 3]); sb, nb = L.shape_array([4, 3])
    assert cuda_ops.lib.ktc_binary_bcast(L.PLUS, a.storeReference, a.storeReference, sa, na, b.storeReference, sb, nb) == L.KTC_EINVAL


def test_broadcast_to(cuda_ops, gc_scope):
    for src, dst in (([64, 1], [32, 64, 128]), ([1], [5, 7]), ([128], [3, 4, 128]), ([3, 1, 5], [2, 3, 4, 5]), ([1, 1024], [64, 1024])):
        a = D.uniform(O.volume(src), 31, -1.0, 1.0)
        r = cuda_ops.createRaw(src, a)
        got = r.broadcastTo(dst)
        assert got.shape == dst and same_bits(got.toArray(), O.broadcast_to(a, src, dst))
    r = cuda_ops.createRaw([2, 3])
    assert r.broadcastTo([2, 3]) is r                      # same shape returns this (JVMRawTensor.kt:52-53)
    with pytest.raises(ValueError):
        r.broadcastTo([3])


# --------------------------------------------------------------------------------------
# reductions
# --------------------------------------------------------------------------------------
RED_SHAPES = [(o, a, i) for o in (1, 3, 70) for a in (1, 2, 3, 31, 32, 33, 128, 513, 1024, 4096, 5000) for i in (1, 2, 3, 4, 128, 130)
              if o * a * i <= 3_000_000]
RED_SHAPES += [(2048, 128, 1), (1, 2048, 128), (64, 32, 64), (1, 1 << 22, 1), (1, (1 << 22) + 5, 1), (1, 100000, 8), (5, 70000, 1),
               (1, 1 << 16, 1024), (4000, 8, 1), (4, 8192, 4)]


@pytest.mark.parametrize("name", list(RED))
def test_axis_reductions_exact_data(cuda_ops, gc_scope, name):
    """Multiples of 1/16 with small totals: every accumulation order is exact, so
    sums must be bit-identical; ties are frequent, so arg ops exercise the
    lowest-index rule."""
    k, o = RED[name]
    for idx, (outer, A, inner) in enumerate(RED_SHAPES):
        x = D.normal(outer * A * inner, 40 + idx, 0.0, 1.0, quantum=16.0)
        r = cuda_ops.createRaw([outer, A, inner], x)
        got = r._aggregate(1, False, k)
        want = O.aggregate(o, x, outer, A, inner, mode=1)
        assert same_bits(got.toArray(), want), f"{name} {(outer, A, inner)}"
        assert same_bits(want, O.aggregate(o, x, outer, A, inner, mode=0))      # and kten-jvm's own order agrees


@pytest.mark.parametrize("name", ("sum", "mean"))
def test_axis_reductions_float_data(cuda_ops, gc_scope, name):
    k, o = RED[name]
    for idx, (outer, A, inner) in enumerate(RED_SHAPES):
        x = D.uniform(outer * A * inner, 300 + idx, -1.0, 1.0) * np.float32(37.0)
        got = cuda_ops.createRaw([outer, A, inner], x)._aggregate(1, True, k).toArray().reshape(-1).astype(np.float64)
        want = O.aggregate(o, x, outer, A, inner, mode=1).astype(np.float64)
        scale = np.abs(x.reshape(outer, A, inner).astype(np.float64)).sum(axis=1).reshape(-1)
        if name == "mean":
            scale = scale / A
        assert np.all(np.abs(got - want) <= RED_RTOL * scale + 1e-30), f"{name} {(outer, A, inner)}"


def test_reductions_nan_inf_and_ties(cuda_ops, gc_scope):
    nan, inf = np.nan, np.inf
    rows = np.array([[1, nan, 3, 2], [nan, nan, nan, nan], [-inf, -inf, -inf, -inf], [inf, 1, inf, 0], [2, 2, 2, 2],
                     [-0.0, 0.0, -0.0, 0.0], [0.0, -0.0, 0.0, -0.0], [-1, -2, -1, -2], [inf, -inf, nan, 0]], dtype=np.float32)
    for layout in ("rows", "cols"):
        x = rows if layout == "rows" else np.ascontiguousarray(rows.T)
        outer, A, inner = (rows.shape[0], 4, 1) if layout == "rows" else (1, 4, rows.shape[0])
        r = cuda_ops.createRaw([outer, A, inner], x)
        for name, (k, o) in RED.items():
            got = r._aggregate(1, False, k).toArray()
            assert same_bits(got, O.aggregate(o, x, outer, A, inner, mode=1)), f"{name} {layout}"
    # long rows (block kernel and split path) with NaN / ties far apart
    for A in (5000, 1 << 20):
        x = np.zeros(A, dtype=np.float32); x[A // 3] = 7; x[A - 2] = 7; x[17] = nan
        r = cuda_ops.createRaw([1, A, 1], x)
        for name, (k, o) in RED.items():
            assert same_bits(r._aggregate(1, False, k).toArray(), O.aggregate(o, x, 1, A, 1, mode=1)), f"{name} A={A}"


def test_full_reductions(cuda_ops, gc_scope):
    for n in (1, 5, 1000, 4096, 100003, 1 << 22, (1 << 24) + 5):
        q = D.normal(n, 77, 0.0, 1.0, quantum=16.0)
        r = cuda_ops.createRaw([n], q)
        s, m = r.sum(), r.mean()
        assert s.shape == [1] and m.shape == [1]
        assert same_bits(s.toArray(), [O.reduce_all(O.SUM, q, 1)])
        assert same_bits(m.toArray(), [O.reduce_all(O.MEAN, q, 1)])
        x = D.uniform(n, 78, 0.0, 1.0)               # all positive: the case kten-jvm's float sum gets wrong at scale
        r = cuda_ops.createRaw([n], x)
        tol = RED_RTOL * O.abs_sum(x)
        assert abs(float(r.sum().toArray()[0]) - float(O.reduce_all(O.SUM, x, 1))) <= tol
        assert abs(float(r.mean().toArray()[0]) - float(O.reduce_all(O.MEAN, x, 1))) <= tol / n
    empty = cuda_ops.createRaw([0])
    assert float(empty.sum().toArray()[0]) == 0.0 and np.isnan(empty.mean().toArray()[0])


def test_aggregate_shapes_follow_the_spi(cuda_ops, gc_scope):
    r = cuda_ops.createRaw([3, 4, 5], np.arange(60, dtype=np.float32))
    assert r.sum(1).shape == [3, 5] and r.sum(1, True).shape == [3, 1, 5] and r.sum(-1).shape == [3, 4]
    assert r.argMax(0, True).shape == [1, 4, 5] and r.max(2).shape == [3, 4]
    v = cuda_ops.createRaw([7], np.arange(7, dtype=np.float32))
    assert v.sum(0).shape == [1] and v.argMax().shape == [1] and v.argMax().toArray()[0] == 6.0   # 1-D keeps [1]
    with pytest.raises(ValueError, match="Cannot address axis"):
        r.sum(3)


def test_fused_value_and_index(cuda_ops, gc_scope):
    for idx, (outer, A, inner) in enumerate([(70, 33, 1), (3, 513, 4), (1, 5000, 130), (2048, 128, 1), (5, 70000, 1), (64, 32, 64)]):
        x = D.normal(outer * A * inner, 500 + idx, 0.0, 1.0, quantum=16.0)
        r = cuda_ops.createRaw([outer, A, inner], x)
        for is_max, (ov, oi) in ((True, (O.MAX, O.ARGMAX)), (False, (O.MIN, O.ARGMIN))):
            val, ind = r.maxWithIndices(1, False, is_max)
            assert same_bits(val.toArray(), O.aggregate(ov, x, outer, A, inner))
            assert same_bits(ind.toArray(), O.aggregate(oi, x, outer, A, inner))


SUM_TO_SHAPE = [([32, 64, 128], [64, 1]), ([32, 64, 128], [128]), ([32, 64, 128], [32, 64, 128]), ([32, 64, 128], [1]),
                ([32, 64, 128], [1, 1, 1]), ([32, 64, 128], [32, 1, 128]), ([4096, 1024], [1, 1024]), ([4096, 1024], [1024]),
                ([4096, 1024], [4096, 1]), ([3, 3], [3]), ([3, 3], [3, 1]), ([3, 3], [1]), ([2, 3, 4, 5, 6], [3, 1, 5, 1]),
                ([2, 3, 4, 5, 6], [1, 1, 1, 6]), ([7, 5, 3], [5, 3]), ([6, 1, 5], [1, 5])]


def test_sum_to_shape(cuda_ops, gc_scope):
    for i, (shape, old) in enumerate(SUM_TO_SHAPE):
        q = D.normal(O.volume(shape), 600 + i, 0.0, 1.0, quantum=16.0)
        got = cuda_ops.createRaw(shape, q).sumToShape(old)
        assert got.shape == old
        assert same_bits(got.toArray(), O.sum_to_shape(q, shape, old, mode=1)), f"{shape} -> {old}"
        assert same_bits(got.toArray(), O.sum_to_shape(q, shape, old, mode=0))
        x = D.uniform(O.volume(shape), 700 + i, -1.0, 1.0)
        got = cuda_ops.createRaw(shape, x).sumToShape(old).toArray().reshape(-1).astype(np.float64)
        want = O.sum_to_shape(x, shape, old, mode=1).astype(np.float64)
        scale = O.sum_to_shape(np.abs(x), shape, old, mode=1).astype(np.float64)
        assert np.all(np.abs(got - want) <= RED_RTOL * scale + 1e-30)
    with pytest.raises(ValueError):
        cuda_ops.createRaw([3, 4]).sumToShape([5])


def test_may_unexpand_chain_equals_fused(cuda_ops, gc_scope):
    shape, old = [32, 64, 128], [64, 1]
    q = D.normal(O.volume(shape), 9, 0.0, 1.0, quantum=16.0)
    r = cuda_ops.createRaw(shape, q)
    chain = AG.may_unexpand(r, old, cuda_ops)
    fused = AG.may_unexpand(r, old, cuda_ops, fused=True)
    assert chain.shape == fused.shape == old and same_bits(chain.toArray(), fused.toArray())


def test_scatter_axis_rejects_bad_index(cuda_ops, gc_scope, index_checks_at_call):
    t = cuda_ops.createRawFill([2, 3], 0.0)
    src = cuda_ops.createRaw([2, 1], [5.0, 6.0])
    t.inplaceScatter(1, cuda_ops.createRaw([2, 1], [2.0, 0.0]), src)
    assert t.toArray().tolist() == [[0, 0, 5], [6, 0, 0]]
    with pytest.raises(ValueError, match="Scatter got invalid index"):
        t.inplaceScatter(1, cuda_ops.createRaw([2, 1], [3.0, 0.0]), src)
    assert t.toArray().tolist() == [[0, 0, 5], [6, 0, 0]]       # and the context is still usable


# --------------------------------------------------------------------------------------
# committed golden fixtures and configuration 1
# --------------------------------------------------------------------------------------
def test_committed_elementwise_fixture(cuda_ops, gc_scope):
    a, b = GOLD["ew_a"], GOLD["ew_b"]
    assert np.array_equal(a, D.uniform(a.size, 1, 0.1, 2.0)) and np.array_equal(b, D.uniform(b.size, 2, 0.1, 2.0))
    ra, rb = cuda_ops.createRaw([a.size], a), cuda_ops.createRaw([b.size], b)
    for name in ("plus", "times", "div", "pow"):
        check_elementwise(name, ra._binary(BIN[name][0], rb).toArray(), GOLD[f"ew_{name}"])
    for name in ("exp", "log", "tanh", "sigmoid"):
        check_elementwise(name, ra._unary(UN[name][0]).toArray(), GOLD[f"ew_{name}"])


def test_committed_reduction_fixture(cuda_ops, gc_scope):
    q = GOLD["red_in"]
    last, first = cuda_ops.createRaw([37, 129], q), cuda_ops.createRaw([37, 129], q)
    for name, (k, _) in RED.items():
        assert same_bits(last._aggregate(1, False, k).toArray(), GOLD[f"red_last_{name}"])
        assert same_bits(first._aggregate(0, False, k).toArray(), GOLD[f"red_first_{name}"])


def config1_inputs():
    x = D.uniform(32 * 64 * 128, 0, -1.0, 1.0, stream=0)
    y = D.uniform(64, 0, 0.5, 1.5, stream=1)
    return x, y, GOLD["c1_z"]


def run_config1(ops, x, y, z):
    tx = AG.Variable(ops, ops.createRaw([32, 64, 128], x))
    ty = AG.Variable(ops, ops.createRaw([64, 1], y))
    tz = AG.NoGradVariable(ops, ops.createRaw([128], z))
    r = ((tx * ty + tz).pow(2.0)).sum(axis=2)
    loss = r.mean()
    r.forward()                      # keeps r's value across backward()
    loss.backward()
    return r.toArray(), loss.toArray(), tx.grad().toArray(), ty.grad().toArray()


def test_config1_plumbing_graph(cuda_ops, gc_scope):
    """x[32,64,128] ~ U(-1,1), y[64,1] ~ U(0.5,1.5), z[128] ~ N(0,1), seed 0:
    r = sum((x*y + z) pow 2, axis=2), loss = mean(r), backward for x and y."""
    x, y, z = config1_inputs()
    r, loss, gx, gy = run_config1(cuda_ops, x, y, z)
    # forward elementwise chain, bit-exact against the oracle
    raw = lambda s, v: cuda_ops.createRaw(s, v)
    xy_want, _ = O.binary(O.TIMES, x, [32, 64, 128], y, [64, 1])
    xyz_want, _ = O.binary(O.PLUS, xy_want, [32, 64, 128], z, [128])
    sq_want = O.scalar(O.POW, xyz_want, 2.0)
    xy_got = raw([32, 64, 128], x).times(raw([64, 1], y))
    xyz_got = xy_got.plus(raw([128], z))
    sq_got = xyz_got.pow(2.0)
    assert same_bits(xy_got.toArray(), xy_want) and same_bits(xyz_got.toArray(), xyz_want) and same_bits(sq_got.toArray(), sq_want)
    # reductions and gradients within 1e-5 * sum|terms| of the exact oracle (committed fixture)
    sq64 = sq_want.astype(np.float64).reshape(32, 64, 128)
    assert np.all(np.abs(r.astype(np.float64) - GOLD["c1_r_exact"]) <= RED_RTOL * sq64.sum(axis=2))
    assert abs(float(loss[0]) - float(GOLD["c1_loss_exact"][0])) <= RED_RTOL * sq64.sum() / 2048
    g = 2.0 * np.abs(xyz_want.astype(np.float64)).reshape(32, 64, 128) / 2048.0          # |d loss / d (x*y+z)|
    gx_terms = (g * np.abs(y.astype(np.float64)).reshape(1, 64, 1)).reshape(-1)
    assert np.all(np.abs(gx.reshape(-1)[::257].astype(np.float64) - GOLD["c1_gx_exact_every257"]) <= RED_RTOL * gx_terms[::257] + 1e-12)
    gy_terms = (g * np.abs(x.astype(np.float64)).reshape(32, 64, 128)).sum(axis=(0, 2))
    assert np.all(np.abs(gy.reshape(-1).astype(np.float64) - GOLD["c1_gy_exact"].reshape(-1)) <= RED_RTOL * gy_terms)
    # and against the oracle run live on the same inputs
    ro, lo, gxo, gyo = run_config1(O.OracleTensorOperations(1), x, y, z)
    assert np.all(np.abs(gx.astype(np.float64) - gxo) <= RED_RTOL * gx_terms.reshape(32, 64, 128) + 1e-12)
    assert np.all(np.abs(r.astype(np.float64) - ro) <= RED_RTOL * sq64.sum(axis=2))


def test_config5_sharded_graph_on_one_gpu(cuda_ops, gc_scope):
    """loss = sum(sigmoid(x*w + b) pow 2) with gradients for w [1,C] and b [C] (sum-to-shape over
    the leading axis); whole tensor vs two row shards summed, vs the CPU oracle running the same
    call sequence, vs float64 ground truth."""
    from kten_b200.sharded import ShardedSigmoidGraph, shard_rows
    rows, cols = 2048, 1024
    x = D.uniform(rows * cols, 0, -1.0, 1.0, stream=0)
    w = D.normal(cols, 0, 0.0, 0.02, stream=1)
    b = D.uniform(cols, 0, -0.1, 0.1, stream=2)

    def run(ops, xs, n, fused=False):
        g = ShardedSigmoidGraph(ops, ops.createRaw([n, cols], xs), ops.createRaw([1, cols], w), ops.createRaw([cols], b))
        loss, gw, gb = g.step()
        return float(loss.toArray()[0]), gw.toArray().reshape(-1).astype(np.float64), gb.toArray().astype(np.float64)

    loss, gw, gb = run(cuda_ops, x, rows)
    parts = [run(cuda_ops, x[f * cols:(f + c) * cols], c) for f, c in (shard_rows(rows, 2, r) for r in range(2))]
    lo, gwo, gbo = run(O.OracleTensorOperations(1), x, rows)
    X = x.reshape(rows, cols).astype(np.float64)
    s = 1.0 / (1.0 + np.exp(-(X * w + b)))
    g = 2 * s * s * (1 - s)
    for got_loss, got_gw, got_gb in ((loss, gw, gb), (parts[0][0] + parts[1][0], parts[0][1] + parts[1][1], parts[0][2] + parts[1][2])):
        assert abs(got_loss - (s * s).sum()) <= RED_RTOL * (s * s).sum()
        assert abs(got_loss - lo) <= RED_RTOL * (s * s).sum()
        assert np.all(np.abs(got_gb - g.sum(axis=0)) <= RED_RTOL * np.abs(g).sum(axis=0))
        assert np.all(np.abs(got_gw - (g * X).sum(axis=0)) <= RED_RTOL * np.abs(g * X).sum(axis=0))
        assert np.all(np.abs(got_gb - gbo) <= RED_RTOL * np.abs(g).sum(axis=0))
        assert np.all(np.abs(got_gw - gwo) <= RED_RTOL * np.abs(g * X).sum(axis=0))


def test_single_rank_communicator_and_injected_failure(cuda_ops, gc_scope):
    """A one-rank communicator exercises the collective wrapper on one GPU: the all-reduce
    is the identity; a failure injected on the host is reported as KTC_ECOMM (nothing on the
    GPU is made to fail) and the next call works again."""
    lib = cuda_ops.lib
    ident = C.create_string_buffer(L.COMM_ID_BYTES)
    L.check(lib.ktc_comm_unique_id(ident))
    comm = C.c_uint64(0)
    L.check(lib.ktc_comm_init_rank(0, 1, 0, ident.raw, C.byref(comm)))
    try:
        x = D.uniform(2049, 3, -1.0, 1.0)
        r = cuda_ops.createRaw([2049], x)
        L.check(lib.ktc_allreduce_sum(comm.value, r.storeReference, 0, 2049))
        assert same_bits(r.toArray(), x)
        L.check(lib.ktc_test_inject_comm_error(1))
        assert lib.ktc_allreduce_sum(comm.value, r.storeReference, 0, 2049) == L.KTC_ECOMM
        assert b"injected" in lib.ktc_last_error()
        L.check(lib.ktc_allreduce_sum(comm.value, r.storeReference, 1, 2048))
        assert same_bits(r.toArray(), x)
        assert lib.ktc_allreduce_sum(comm.value, r.storeReference, 2, 2048) == L.KTC_EINVAL      # range outside the buffer
        assert lib.ktc_allreduce_sum(comm.value + 7, r.storeReference, 0, 1) == L.KTC_ESTATE
    finally:
        L.check(lib.ktc_test_inject_comm_error(0))
        L.check(lib.ktc_comm_destroy(comm.value))


# --------------------------------------------------------------------------------------
# runtime behaviour: handles, pool, transfers, errors
# --------------------------------------------------------------------------------------
def test_refcount_release_and_stale_handles(cuda_ops):
    lib = cuda_ops.lib
    h = C.c_uint64(0)
    L.check(lib.ktc_alloc(0, 1000, C.byref(h)))
    cnt = C.c_int(0)
    L.check(lib.ktc_retain(h)); L.check(lib.ktc_refcount(h, C.byref(cnt))); assert cnt.value == 2
    L.check(lib.ktc_release(h)); L.check(lib.ktc_release(h))
    assert lib.ktc_release(h) == L.KTC_ESTATE and b"already released" in lib.ktc_last_error()
    assert lib.ktc_fill(h, 0, 10, 1.0) == L.KTC_ESTATE                  # use after release is detected
    assert lib.ktc_fill(0, 0, 10, 1.0) == L.KTC_ESTATE
    raw = cuda_ops.createRaw([4])
    raw.release()
    with pytest.raises(RuntimeError, match="already released"):
        raw.plus(1.0)


def test_gc_scope_releases_what_it_created(cuda_ops):
    before = cuda_ops.getMetrics()["liveMB"]
    keep = None
    with cuda_ops.garbageCollector():
        a = cuda_ops.createRaw([1 << 20])
        b = a.plus(1.0)
        keep = b.times(2.0)
        cuda_ops.incrementRef(keep)                    # what Function.output does
        with cuda_ops.garbageCollector():              # nested scopes are no-ops
            c = keep.plus(1.0)
        assert not c._released
    assert a._released and b._released and c._released and not keep._released
    assert abs(cuda_ops.getMetrics()["liveMB"] - before - 4.0) < 0.01
    keep.release()
    assert keep._released and abs(cuda_ops.getMetrics()["liveMB"] - before) < 0.01


def test_pool_reuses_exact_sizes_and_honours_limit(cuda_ops):
    lib = cuda_ops.lib
    m0 = cuda_ops.getMetrics()
    for _ in range(5):
        r = cuda_ops.createRaw([123457]); r.release()
    m1 = cuda_ops.getMetrics()
    assert m1["poolHits"] - m0["poolHits"] >= 4
    live = C.c_int64(0)
    L.check(lib.ktc_pool_stats(0, C.byref(live), None, None, None))
    L.check(lib.ktc_pool_limit(0, live.value + (1 << 20)))
    try:
        with pytest.raises(MemoryError, match="pool limit"):
            cuda_ops.createRaw([1 << 22])
    finally:
        L.check(lib.ktc_pool_limit(0, 0))
    L.check(lib.ktc_pool_trim(0))
    assert cuda_ops.getMetrics()["pooledMB"] == 0.0


def test_transfers_fill_copy_and_ranges(cuda_ops, gc_scope):
    lib = cuda_ops.lib
    x = np.arange(1000, dtype=np.float32)
    r = cuda_ops.createRaw([1000], x)
    assert r.getSingleValue([999]) == 999.0 and r.getSingleValue([-1]) == 999.0
    for off, n, v in ((0, 1000, 1.5), (1, 7, 2.5), (3, 996, -1.0), (999, 1, 9.0)):
        L.check(lib.ktc_fill(r.storeReference, off, n, v)); x[off:off + n] = v
        assert np.array_equal(r.toArray(), x)
    shallow, deep = r.copy(shallow=True), r.copy()
    r.inplaceFill(4.0)
    assert np.all(shallow.toArray() == 4.0) and np.array_equal(deep.toArray(), x)
    v = r.view([10, -1]); assert v.shape == [10, 100]
    out = np.zeros(4, dtype=np.float32)
    assert lib.ktc_d2h(out.ctypes.data_as(C.c_void_p), r.storeReference, 998, 4, 1) == L.KTC_EINVAL
    assert lib.ktc_h2d(r.storeReference, -1, out.ctypes.data_as(C.c_void_p), 4, 1) == L.KTC_EINVAL
    assert lib.ktc_binary(L.PLUS, r.storeReference, r.storeReference, r.storeReference, 1001) == L.KTC_EINVAL
    assert lib.ktc_binary(99, r.storeReference, r.storeReference, r.storeReference, 10) == L.KTC_EINVAL
    assert lib.ktc_reduce_axis(L.SUM, r.storeReference, r.storeReference, 1, 1000, 1) == L.KTC_EINVAL      # aliasing


def test_views_and_overlapped_copy_pipeline(cuda_ops, gc_scope):
    """Sub-range handles keep their parent alive, and a chunked upload / compute / download
    pipeline in KTC_COPY_OVERLAP mode gives the same bits as the one-shot path."""
    lib = cuda_ops.lib
    n, chunk = 1 << 20, 1 << 16
    a, b = D.uniform(n, 21, -1.0, 1.0), D.uniform(n, 22, 0.5, 2.0)
    want = O.binary_same(O.DIV, a, b)
    ra, rb, ro = cuda_ops.createRaw([n]), cuda_ops.createRaw([n]), cuda_ops.createRaw([n])
    views = []
    for mode in (L.COPY_OVERLAP, L.COPY_OVERLAP_UNFENCED):
        got = np.zeros(n, dtype=np.float32)
        L.check(lib.ktc_copy_fence(0))
        for i in range(n // chunk):
            hs = [C.c_uint64(0) for _ in range(3)]
            for h, r in zip(hs, (ra, rb, ro)):
                L.check(lib.ktc_view(r.storeReference, i * chunk, chunk, C.byref(h)))
            va, vb, vo = (h.value for h in hs)
            sl = slice(i * chunk, (i + 1) * chunk)
            L.check(lib.ktc_h2d(va, 0, a[sl].ctypes.data_as(C.c_void_p), chunk, mode))
            L.check(lib.ktc_h2d(vb, 0, b[sl].ctypes.data_as(C.c_void_p), chunk, mode))
            L.check(lib.ktc_binary(L.DIV, vo, va, vb, chunk))
            L.check(lib.ktc_d2h(got[sl].ctypes.data_as(C.c_void_p), vo, 0, chunk, mode))
            for v in (va, vb, vo):
                L.check(lib.ktc_release(v))
        cuda_ops.synchronize()
        assert same_bits(got, want)
        ro.inplaceFill(0.0)
    got = np.zeros(n, dtype=np.float32)
    for i in range(n // chunk):
        hs = [C.c_uint64(0) for _ in range(3)]
        for h, r in zip(hs, (ra, rb, ro)):
            L.check(lib.ktc_view(r.storeReference, i * chunk, chunk, C.byref(h)))
        va, vb, vo = (h.value for h in hs)
        views += [va, vb, vo]
        sl = slice(i * chunk, (i + 1) * chunk)
        L.check(lib.ktc_h2d(va, 0, a[sl].ctypes.data_as(C.c_void_p), chunk, L.COPY_OVERLAP))
        L.check(lib.ktc_h2d(vb, 0, b[sl].ctypes.data_as(C.c_void_p), chunk, L.COPY_OVERLAP))
        L.check(lib.ktc_binary(L.DIV, vo, va, vb, chunk))
        L.check(lib.ktc_d2h(got[sl].ctypes.data_as(C.c_void_p), vo, 0, chunk, L.COPY_OVERLAP))
    cuda_ops.synchronize()
    assert same_bits(got, want)
    assert same_bits(ro.toArray(), want)
    # a view outlives the tensor object that created its parent
    cnt = C.c_int(0)
    L.check(lib.ktc_refcount(ra.storeReference, C.byref(cnt))); assert cnt.value == 1 + n // chunk
    h_parent = ra.storeReference
    ra.release()
    L.check(lib.ktc_refcount(h_parent, C.byref(cnt))); assert cnt.value == n // chunk
    out = np.zeros(4, dtype=np.float32)
    L.check(lib.ktc_d2h(out.ctypes.data_as(C.c_void_p), views[0], 0, 4, L.COPY_SYNC))
    assert same_bits(out, a[:4])
    h = C.c_uint64(0)
    assert lib.ktc_view(rb.storeReference, n - 2, 4, C.byref(h)) == L.KTC_EINVAL
    for v in views:
        L.check(lib.ktc_release(v))
    assert lib.ktc_d2h(out.ctypes.data_as(C.c_void_p), h_parent, 0, 4, L.COPY_SYNC) == L.KTC_ESTATE   # last view gone -> parent freed


def test_wrap_external_device_memory(cuda_ops, gc_scope):
    torch = pytest.importorskip("torch")
    t = torch.arange(4096, dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()
    h = C.c_uint64(0)
    L.check(cuda_ops.lib.ktc_wrap(0, C.c_void_p(t.data_ptr()), t.numel(), C.byref(h)))
    from kten_b200.raw_tensor import CUDARawTensor
    w = CUDARawTensor([4096], h.value, cuda_ops)
    assert float(w.sum().toArray()[0]) == float(4095 * 4096 // 2)
    w.timesAssign(2.0)
    cuda_ops.synchronize()
    assert float(t.sum().item()) == float(4095 * 4096)


def test_determinism_bit_stable(cuda_ops, gc_scope):
    x = D.uniform(1 << 22, 5, -1.0, 1.0)
    r = cuda_ops.createRaw([1 << 12, 1 << 10], x)
    runs = [(r.sum().toArray(), r.sum(0).toArray(), r.sum(1).toArray(), r.sumToShape([1, 1 << 10]).toArray()) for _ in range(3)]
    for other in runs[1:]:
        for a, b in zip(runs[0], other):
            assert same_bits(a, b)


def test_bounded_device_wait_times_out_cleanly(cuda_ops):
    """A wait on a flag nothing sets gives up after its limit and reports it; the
    context stays usable (no trap, no endless loop)."""
    st = C.c_int(0)
    L.check(cuda_ops.lib.ktc_test_bounded_wait(0, 2_000_000, C.byref(st)))       # 2 ms
    assert st.value == L.KTC_ETIMEOUT
    r = cuda_ops.createRawFill([16], 1.0)
    assert float(r.sum().toArray()[0]) == 16.0
    r.release()


def test_vector_math_equals_scalar_math_and_the_host_build(cuda_ops, gc_scope):
    """exp, sigmoid and pow test their rare slow paths once per float4 in the vector kernels and once per
    element in the scalar kernels that serve unaligned buffers: both must produce the same bits.  The
    unaligned case is a view that starts one float into the buffer.  The same header compiled for the host
    (tests/host_math) must give the device's bits too, which is what makes the accuracy measured on the CPU
    (tests/test_fastmath_host.py) a statement about the GPU."""
    lib = cuda_ops.lib
    n = (1 << 18) + 1
    x = np.concatenate([D.uniform(n - 40, 61, -30.0, 30.0), special_values()[:20], np.array([88.0, -88.0, 87.0, -87.0, 100.0, -100.0, 0.0, -0.0,
                        1e-30, -1e-30, 1.0, -1.0, 0.5, 2.0, 3.0, 1e5, -1e5, 1e-10, 40.0, -40.0], dtype=np.float32)])[:n].astype(np.float32)
    y = np.concatenate([D.uniform(n - 8, 62, -4.0, 4.0), np.array([0.0, -0.0, 1.0, 2.0, 0.5, -1.0, 1e3, -1e3], dtype=np.float32)])[:n].astype(np.float32)
    base = np.abs(x) + np.float32(1e-3)
    ta, tb = cuda_ops.createRaw([n], x), cuda_ops.createRaw([n], y)
    tp = cuda_ops.createRaw([n], base)
    out_v, out_s = cuda_ops.createRaw([n]), cuda_ops.createRaw([n])

    def view(t):
        h = C.c_uint64(0)
        L.check(lib.ktc_view(t.storeReference, 1, n - 1, C.byref(h)))
        return h.value

    va, vb, vp, vo = view(ta), view(tb), view(tp), view(out_s)
    for code in (L.EXP, L.SIGMOID):
        L.check(lib.ktc_unary(code, out_v.storeReference, ta.storeReference, n))          # aligned: packed
        L.check(lib.ktc_unary(code, vo, va, n - 1))                                       # unaligned: scalar
        assert same_bits(out_v.toArray()[1:], out_s.toArray()[1:]), code
    L.check(lib.ktc_binary(L.POW, out_v.storeReference, tp.storeReference, tb.storeReference, n))
    L.check(lib.ktc_binary(L.POW, vo, vp, vb, n - 1))
    assert same_bits(out_v.toArray()[1:], out_s.toArray()[1:])
    for h in (va, vb, vp, vo):
        L.check(lib.ktc_release(h))
    from tests.test_fastmath_host import host_math_library, host_unary, host_pow
    host = host_math_library()
    got = ta.sigmoid().toArray()
    assert same_bits(got, host_unary(host, "kfh_sigmoid", x))
    assert same_bits(ta.exp().toArray(), host_unary(host, "kfh_exp", x))
    want, ok = host_pow(host, base, y)
    assert ok.mean() > 0.9 and same_bits(tp.pow(tb).toArray()[ok], want[ok])
    # against the reference: e = (float)Math.exp(-1f * x), then its two IEEE operations (JVMRawTensor.kt:399)
    d = O.ulp_distance(got, O.unary(O.SIGMOID, x))
    assert d.max() <= 2 and int((d > 0).sum()) <= 2


def test_peer_memory_allreduce_single_rank_and_bounded_wait(cuda_ops, gc_scope):
    """World of one: the kernel publishes into its own mailbox and sums one slot (identity), several
    tensors per call, twice in a row (both slot sets).  Then a communicator whose second rank never
    arrives: the wait must give up after its limit, report KTC_ETIMEOUT, leave the tensors untouched
    and the device usable."""
    lib = cuda_ops.lib
    vals = [D.uniform(n, 70 + i, -1.0, 1.0) for i, n in enumerate((1, 1024, 1024, 5000))]
    ts = [cuda_ops.createRaw([v.size], v) for v in vals]
    handle = C.create_string_buffer(L.P2P_HANDLE_BYTES)
    comm = C.c_uint64(0)
    L.check(lib.ktc_p2p_create(0, 1, 0, C.byref(comm), handle))
    L.check(lib.ktc_p2p_connect(comm.value, handle.raw))
    bufs = (C.c_uint64 * 4)(*[t.storeReference for t in ts])
    counts = (C.c_int64 * 4)(*[t.size for t in ts])
    st = C.c_int(-99)
    for _ in range(3):
        L.check(lib.ktc_p2p_allreduce_sum(comm.value, bufs, counts, 4))
    L.check(lib.ktc_p2p_status(comm.value, C.byref(st)))
    assert st.value == L.KTC_OK
    for t, v in zip(ts, vals):
        assert same_bits(t.toArray(), v)
    too_many = (C.c_int64 * 1)(L.P2P_MAX_FLOATS + 1)
    big = cuda_ops.createRaw([L.P2P_MAX_FLOATS + 1])
    assert lib.ktc_p2p_allreduce_sum(comm.value, (C.c_uint64 * 1)(big.storeReference), too_many, 1) == L.KTC_EINVAL
    L.check(lib.ktc_p2p_destroy(comm.value))
    assert lib.ktc_p2p_allreduce_sum(comm.value, bufs, counts, 4) == L.KTC_ESTATE
    # a rank that never arrives
    L.check(lib.ktc_tune_set(b"p2p_wait_ms", 50))
    try:
        L.check(lib.ktc_p2p_create(0, 2, 0, C.byref(comm), handle))
        L.check(lib.ktc_test_p2p_connect_self(comm.value))
        L.check(lib.ktc_p2p_allreduce_sum(comm.value, bufs, counts, 4))
        L.check(lib.ktc_p2p_status(comm.value, C.byref(st)))
        assert st.value == L.KTC_ETIMEOUT
        L.check(lib.ktc_p2p_status(comm.value, C.byref(st)))
        assert st.value == L.KTC_OK                                   # the flag was cleared by the read
        L.check(lib.ktc_p2p_destroy(comm.value))
    finally:
        L.check(lib.ktc_tune_set(b"p2p_wait_ms", 10000))
    for t, v in zip(ts, vals):
        assert same_bits(t.toArray(), v)                              # nothing was summed
    assert same_bits(ts[1].plus(ts[2]).toArray(), vals[1] + vals[2])  # the device still works
