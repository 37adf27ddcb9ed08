"""Deferred elementwise expressions (ops.lazy = True) on the GPU: every result must equal the
call-by-call execution of the same backend -- bit for bit for elementwise values, within the
reduction tolerance (exact on exactly summable data) for fused sums -- and the aliasing rules of
the raw-tensor SPI (shallow copies share storage, in-place calls are visible through aliases,
deep copies are independent) must hold whether or not a tensor has storage yet."""
import ctypes as C

import numpy as np

from oracle import oracle as O
import pytest

from kten_b200 import _lib as L
from kten_b200 import autograd as AG
from kten_b200 import datagen as D
from tests.kten_cases import CASES, CASE_IDS, run_case

pytestmark = pytest.mark.gpu
RED_RTOL = 1e-5


def same_bits(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.fixture()
def lazy_ops(cuda_ops):
    """Deferred elementwise calls; every sum runs where it is written (one sink per program)."""
    cuda_ops.lazy, cuda_ops.deferSums = True, False
    try:
        with cuda_ops.garbageCollector():
            yield cuda_ops
    finally:
        cuda_ops.lazy, cuda_ops.deferSums = False, True


@pytest.fixture()
def lazy_sums_ops(cuda_ops):
    """The default deferred mode: sums wait as well and share passes (ops.deferSums)."""
    cuda_ops.lazy, cuda_ops.deferSums = True, True
    try:
        with cuda_ops.garbageCollector():
            yield cuda_ops
    finally:
        cuda_ops.lazy = False


def both(ops, fn):
    """Run fn(ops) eagerly and deferred; returns (eager results, deferred results) as arrays."""
    out = []
    for mode in (False, True):
        ops.lazy = mode
        with ops.garbageCollector():
            res = fn(ops)
            res = res if isinstance(res, (list, tuple)) else [res]
            out.append([r.toArray() for r in res])
    ops.lazy = True
    return out


@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_reference_vectors_deferred(lazy_ops, case):
    run_case(lazy_ops, case)


@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_reference_vectors_deferred_with_pending_sums(lazy_sums_ops, case):
    run_case(lazy_sums_ops, case)


SHAPES = [([64, 128], [64, 128], [128]), ([8, 16, 32], [16, 1], [32]), ([5, 12], [1, 12], [5, 1]),
          ([3, 5, 7], [5, 7], [7]),                       # innermost extent not a multiple of 4: separate calls
          ([2, 3, 4, 2, 8], [3, 1, 2, 1], [4, 1, 8]),     # more collapsed dimensions than the kernel fuses
          ([1 << 16], [1 << 16], [1])]


@pytest.mark.parametrize("shapes", SHAPES, ids=[str(s[0]) for s in SHAPES])
def test_chains_equal_call_by_call(lazy_ops, shapes):
    sa, sb, sc = shapes
    vol = lambda s: int(np.prod(s))
    a = D.uniform(vol(sa), 3, 0.25, 2.0, stream=0)
    b = D.uniform(vol(sb), 3, -1.0, 1.0, stream=1)
    c = D.uniform(vol(sc), 3, 0.5, 1.5, stream=2)

    def chain(ops):
        ta, tb, tc = ops.createRaw(sa, a), ops.createRaw(sb, b), ops.createRaw(sc, c)
        u = ta.times(tb).plus(tc)                 # broadcast binary ops
        v = u.sigmoid().pow(2.0).minus(0.25)      # unary, square, scalar
        w = ta.log().div(tc).tanh().clamp(-0.5, 0.4)
        x = v.times(w).plus(u.exp().reciprocal()).unaryMinus()
        y = ta.pow(tc).minus(ops.pow(1.5, tb)).lt(0.75)
        z = ta.pow(1.0).plus(3.0)
        q = tb.abs().plus(1.0).rsqrt().times(tc.sqrt()).plus(ta)      # abs, 1 / sqrt and sqrt are expression instructions too
        return [u, v, w, x, y, z, q]

    eager, lazy = both(lazy_ops, chain)
    for e, l in zip(eager, lazy):
        assert same_bits(e, l)
    # and directly against the oracle: the exact operations reproduce it bit for bit; exp, sigmoid and pow differ from
    # the narrowed double libm in fewer than one element per million, so chains of those agree in (nearly) every
    # element; log and tanh are within 1 and 2 ulp (w, x)
    want = [r.toArray() for r in chain(O.OracleTensorOperations())]
    for name, l, o in zip("uvwxyzq", lazy, want):
        assert l.shape == o.shape, name
        differing = int(np.count_nonzero(l.view(np.uint32) != o.view(np.uint32)))
        if name in "uvyzq":
            assert differing <= max(1, l.size // 1000), (name, differing, l.size)
        if name != "y":                                            # y is a comparison: 0 or 1
            assert np.allclose(l, o, rtol=4e-6, atol=4e-6), name
        if name in "uzq":                                          # only exact operations
            assert differing == 0, name


def test_fused_path_is_the_one_that_runs(lazy_ops):
    ops = lazy_ops
    a = ops.createRaw([256, 512], D.uniform(256 * 512, 5, -1.0, 1.0))
    b = ops.createRaw([512], D.uniform(512, 5, 0.5, 1.5, stream=1))
    f0, u0, l0 = ops.fusedEvaluations, ops.unfusedEvaluations, ops.lib.ktc_launch_count()
    r = a.times(b).plus(1.0).sigmoid().pow(2.0)
    assert r.isDeferred and ops.lib.ktc_launch_count() == l0          # nothing ran yet
    total = r.sum()
    assert r.isDeferred and ops.fusedEvaluations == f0 + 1 and ops.unfusedEvaluations == u0
    assert ops.lib.ktc_launch_count() - l0 <= 2                       # one fused kernel (+ its partial combine)
    r.toArray()
    assert not r.isDeferred and ops.fusedEvaluations == f0 + 2
    want = a.toArray().astype(np.float64) * b.toArray() + 1.0
    want = (1.0 / (1.0 + np.exp(-want))) ** 2
    assert abs(float(total.toArray()[0]) - want.sum()) <= RED_RTOL * want.sum()


def test_fused_sums_match_reductions(lazy_ops):
    ops = lazy_ops
    rows, cols = 1000, 384
    xi = np.round(D.uniform(rows * cols, 9, -8.0, 8.0)).astype(np.float32)      # small integers: sums are exact
    wi = np.round(D.uniform(cols, 9, -4.0, 4.0, stream=1)).astype(np.float32)

    def sums(o):
        x, w = o.createRaw([rows, cols], xi), o.createRaw([1, cols], wi)
        p = x.times(w).plus(2.0)
        return [p.sum(), p.mean(), p.sum(0), p.sum(0, keepDimensions=True), x.plus(1.0).sum(axis=1)]

    eager, lazy = both(ops, sums)
    want = xi.reshape(rows, cols).astype(np.float64) * wi + 2.0
    assert float(lazy[0][0]) == want.sum() and same_bits(lazy[0], eager[0])
    assert abs(float(lazy[1][0]) - want.mean()) <= 1e-6 * abs(want.mean()) + 1e-7
    assert same_bits(lazy[2], eager[2]) and np.array_equal(lazy[2].astype(np.float64), want.sum(axis=0))
    assert lazy[3].shape == (1, cols) and same_bits(lazy[3], eager[3])
    assert same_bits(lazy[4], eager[4])
    # float data: within the reduction tolerance of the float64 value
    xf = D.uniform(rows * cols, 10, -1.0, 1.0)
    e2, l2 = both(ops, lambda o: [o.createRaw([rows, cols], xf).sigmoid().sum(0), o.createRaw([rows, cols], xf).exp().mean()])
    s64 = 1.0 / (1.0 + np.exp(-xf.reshape(rows, cols).astype(np.float64)))
    assert np.all(np.abs(l2[0] - s64.sum(axis=0)) <= RED_RTOL * s64.sum(axis=0))
    assert np.all(np.abs(l2[0] - e2[0]) <= RED_RTOL * s64.sum(axis=0))
    assert abs(float(l2[1][0]) - np.exp(xf.astype(np.float64)).mean()) <= RED_RTOL * np.exp(xf.astype(np.float64)).mean()


def test_inplace_and_alias_rules(lazy_ops):
    n = 4096
    av, bv, cv = (D.uniform(n, 11, -1.0, 1.0, stream=s) for s in range(3))

    def script(o):
        a, b, c = o.createRaw([n], av), o.createRaw([n], bv), o.createRaw([n], cv)
        d = a.plus(b)                    # reads a ...
        a.plusAssign(c)                  # ... which then changes in place: d keeps the old value
        a.timesAssign(0.5)
        e = d.times(2.0)
        s = e.copy(shallow=True)         # alias of a (possibly pending) value
        s.timesAssign(b)                 # visible through e
        s.plusAssign(1.0)
        deep = e.copy()                  # independent of later writes to e
        e.divAssign(4.0)
        f = o.createRaw([n], bv).minus(c)
        f.inplaceFill(7.0)               # overwrites a pending value
        g = d.exp()
        d.release()                      # released before its consumer is evaluated
        v = c.view([64, 64]).times(2.0)
        c.plusAssign(1.0)                # the view's consumer keeps the old contents
        return [a, e, s, deep, f, g, v, c]

    eager, lazy = both(lazy_ops, script)
    for k, (e, l) in enumerate(zip(eager, lazy)):
        assert same_bits(e, l), f"result {k}"
    assert np.array_equal(lazy[1], lazy[2])                 # alias and original agree
    assert same_bits(lazy[4], np.full(n, 7.0, np.float32))


def test_cheap_values_are_recomputed_heavy_ones_stored(lazy_ops):
    ops = lazy_ops
    assert ops.recomputeLimit == 2 and ops.storeCost == 8
    n = 1 << 14
    xv = D.uniform(n, 13, -2.0, 2.0)
    x = ops.createRaw([n], xv)
    c = x.times(2.0).plus(1.0)            # cheap: recomputed from x, which is read either way
    first = c.plus(1.0).sum()
    second = c.times(c).sum()
    assert c.isDeferred
    third = c.times(0.5).sum()            # the third use stores it
    assert not c.isDeferred
    s = x.sigmoid()                       # behind a transcendental: stored by the first program that computes it
    fourth = s.times(s).sum()
    assert not s.isDeferred
    ops.lazy = False
    xe = ops.createRaw([n], xv)
    assert same_bits(c.toArray(), xe.times(2.0).plus(1.0).toArray())
    assert same_bits(s.toArray(), xe.sigmoid().toArray())
    c64, s64 = c.toArray().astype(np.float64), s.toArray().astype(np.float64)
    for got, want in ((first, c64 + 1), (second, c64 * c64), (third, c64 * 0.5), (fourth, s64 * s64)):
        assert abs(float(got.toArray()[0]) - want.sum()) <= RED_RTOL * np.abs(want).sum()


def test_programs_beyond_the_kernel_limits_are_split(lazy_ops):
    ops = lazy_ops
    n = 2048
    vals = [D.uniform(n, 17, 0.5, 1.5, stream=s) for s in range(9)]

    def wide(o):
        ts = [o.createRaw([n], v) for v in vals]
        acc = ts[0]
        for t in ts[1:]:                  # nine distinct operands: more than one program can load
            acc = acc.times(t).plus(t)
        deep = ts[0]
        for i in range(40):               # longer than one program
            deep = deep.plus(float(i)).times(0.99)
        return [acc, deep]

    eager, lazy = both(ops, wide)
    assert same_bits(eager[0], lazy[0]) and same_bits(eager[1], lazy[1])
    assert ops.unfusedEvaluations > 0


def test_config1_graph_deferred_equals_eager(lazy_ops):
    x = D.uniform(32 * 64 * 128, 0, -1.0, 1.0, stream=0)
    y = D.uniform(64, 0, 0.5, 1.5, stream=1)
    z = D.normal(128, 0, 0.0, 1.0, stream=2)
    out = []
    for mode in (False, True):
        lazy_ops.lazy = mode
        with lazy_ops.garbageCollector():
            tx = AG.Variable(lazy_ops, lazy_ops.createRaw([32, 64, 128], x))
            ty = AG.Variable(lazy_ops, lazy_ops.createRaw([64, 1], y))
            tz = AG.NoGradVariable(lazy_ops, lazy_ops.createRaw([128], z))
            r = ((tx * ty + tz).pow(2.0)).sum(axis=2)
            loss = r.mean()
            r.forward()
            loss.backward()
            out.append((r.toArray(), loss.toArray(), tx.grad().toArray(), ty.grad().toArray()))
    (re, le, gxe, gye), (rl, ll, gxl, gyl) = out
    assert same_bits(re, rl) and same_bits(le, ll)          # axis-2 sum runs on stored values in both modes
    assert same_bits(gxe, gxl)                              # elementwise gradient: identical operations
    sq = (x.reshape(32, 64, 128).astype(np.float64) * y.reshape(64, 1) + z)
    terms = (2.0 * np.abs(sq) / 2048.0 * np.abs(x.reshape(32, 64, 128))).sum(axis=(0, 2))
    assert np.all(np.abs(gye.reshape(-1).astype(np.float64) - gyl.reshape(-1)) <= RED_RTOL * terms)


def test_config5_graph_deferred(lazy_ops):
    from kten_b200.sharded import ShardedSigmoidGraph
    rows, cols = 4096, 1024
    x = D.uniform(rows * cols, 0, -1.0, 1.0, stream=0)
    w = D.normal(cols, 0, 0.0, 0.02, stream=1)
    b = D.uniform(cols, 0, -0.1, 0.1, stream=2)
    res = []
    for mode in (False, True):
        lazy_ops.lazy = mode
        with lazy_ops.garbageCollector():
            g = ShardedSigmoidGraph(lazy_ops, lazy_ops.createRaw([rows, cols], x), lazy_ops.createRaw([1, cols], w),
                                    lazy_ops.createRaw([cols], b))
            f0, l0 = lazy_ops.fusedEvaluations, lazy_ops.lib.ktc_launch_count()
            for _ in range(2):                               # two steps: state from the first must not leak
                loss, gw, gb = g.step()
                vals = (float(loss.toArray()[0]), gw.toArray().reshape(-1).astype(np.float64), gb.toArray().astype(np.float64))
                g.release_step()
            res.append(vals + (lazy_ops.fusedEvaluations - f0, lazy_ops.lib.ktc_launch_count() - l0))
    X = x.reshape(rows, cols).astype(np.float64)
    s = 1.0 / (1.0 + np.exp(-(X * w + b)))
    gz = 2 * s * s * (1 - s)
    for loss, gw, gb, _, _ in res:
        assert abs(loss - (s * s).sum()) <= RED_RTOL * (s * s).sum()
        assert np.all(np.abs(gb - gz.sum(axis=0)) <= RED_RTOL * np.abs(gz).sum(axis=0))
        assert np.all(np.abs(gw - (gz * X).sum(axis=0)) <= RED_RTOL * np.abs(gz * X).sum(axis=0))
    assert res[0][3] == 0 and res[1][3] >= 6                # the deferred run went through the fused kernel ...
    assert res[1][4] < res[0][4]                            # ... with fewer launches than call by call


def expr_stats(ops):
    out = (C.c_int64 * 6)()
    L.check(ops.lib.ktc_expr_stats(out))
    return dict(zip(("compiled", "jit_launches", "interp_launches", "failures", "compile_us", "nvrtc"), out))


def test_generated_kernels_equal_the_interpreter(lazy_ops):
    """Programs run by kernels generated at run time (NVRTC) and by the built-in interpreter kernel:
    same operations, same summation order, so stores and sums agree bit for bit."""
    ops = lazy_ops
    cases = [([512, 1024], [1, 1024], [1024]), ([24, 16, 128], [16, 1], [24, 1, 128]), ([96, 8, 64], [96, 1, 64], [1])]
    vol = lambda s: int(np.prod(s))

    def script(o, sa, sb, sc, a, b, c):
        ta, tb, tc = o.createRaw(sa, a), o.createRaw(sb, b), o.createRaw(sc, c)
        u = ta.times(tb).plus(tc).sigmoid()
        v = u.pow(2.0).minus(ta.exp().div(3.0)).clamp(-2.0, 2.0)
        w = ta.pow(tb.plus(2.0)).log().tanh().reciprocal().unaryMinus().gt(-1.5)
        acc = o.createRaw(sa, a)
        acc.plusAssign(v)                                    # in place into a stored tensor
        acc.timesAssign(0.5)
        return [v, w, acc, u.times(v).sum(), v.mean(), u.times(ta).sum(0), u.sum(0, keepDimensions=True)]

    before = expr_stats(ops)
    results = {}
    for mode, (jit, min_elems) in {"interpreter": (0, 1 << 20), "generated": (1, 0)}.items():
        L.check(ops.lib.ktc_tune_set(b"expr_jit", jit))
        L.check(ops.lib.ktc_tune_set(b"expr_jit_min_elems", min_elems))
        try:
            out = []
            for sa, sb, sc in cases:
                a = D.uniform(vol(sa), 21, 0.25, 2.0, stream=0)
                b = D.uniform(vol(sb), 21, -1.0, 1.0, stream=1)
                c = D.uniform(vol(sc), 21, 0.5, 1.5, stream=2)
                with ops.garbageCollector():
                    out.append([r.toArray() for r in script(ops, sa, sb, sc, a, b, c)])
            results[mode] = out
        finally:
            L.check(ops.lib.ktc_tune_set(b"expr_jit", 1))
            L.check(ops.lib.ktc_tune_set(b"expr_jit_min_elems", 1 << 20))
    after = expr_stats(ops)
    if after["nvrtc"] == 0:
        pytest.fail("NVRTC is missing on this machine: generated kernels did not run")
    log = C.create_string_buffer(4000)
    ops.lib.ktc_expr_jit_log(log, 4000)
    assert after["failures"] == before["failures"], log.value.decode()
    assert after["jit_launches"] > before["jit_launches"] and after["interp_launches"] > before["interp_launches"]
    for ci, (ri, rg) in enumerate(zip(results["interpreter"], results["generated"])):
        for k, (x, y) in enumerate(zip(ri, rg)):
            assert same_bits(x, y), f"case {ci} result {k}"


def test_large_programs_use_generated_kernels_by_default(lazy_ops):
    ops = lazy_ops
    rows, cols = 2048, 1024                                   # 2^21 elements: above the default threshold
    x = ops.createRaw([rows, cols], D.uniform(rows * cols, 23, -1.0, 1.0))
    before = expr_stats(ops)
    got = x.times(2.0).plus(1.0).tanh().sum(0).toArray()
    after = expr_stats(ops)
    assert after["jit_launches"] == before["jit_launches"] + 1 and after["failures"] == before["failures"]
    want = np.tanh(x.toArray().astype(np.float64) * 2.0 + 1.0)
    assert np.all(np.abs(got - want.sum(axis=0)) <= RED_RTOL * np.abs(want).sum(axis=0))


def test_config5_step_is_one_pass_with_three_sinks(lazy_sums_ops):
    """With the sums deferred as well, loss, weight gradient and bias gradient of the sharded step come out
    of ONE generated kernel that reads x once.  The gradients equal those of the one-sink-per-program mode
    bit for bit (same element values, same partition, same combination order); the loss agrees within the
    reduction tolerance."""
    from kten_b200.sharded import ShardedSigmoidGraph
    ops = lazy_sums_ops
    rows, cols = 4096, 1024                                   # 2^22 elements: generated kernels by default
    x = D.uniform(rows * cols, 0, -1.0, 1.0, stream=0)
    w = D.normal(cols, 0, 0.0, 0.02, stream=1)
    b = D.uniform(cols, 0, -0.1, 0.1, stream=2)
    res = []
    for defer in (False, True):
        ops.deferSums = defer
        with ops.garbageCollector():
            g = ShardedSigmoidGraph(ops, ops.createRaw([rows, cols], x), ops.createRaw([1, cols], w), ops.createRaw([cols], b))
            m0, l0, before = ops.multiSinkEvaluations, ops.lib.ktc_launch_count(), expr_stats(ops)
            for _ in range(2):
                loss, gw, gb = g.step()
                vals = (loss.toArray().copy(), gw.toArray().copy(), gb.toArray().copy())
                g.release_step()
            after = expr_stats(ops)
            res.append(vals + (ops.multiSinkEvaluations - m0, ops.lib.ktc_launch_count() - l0, after["failures"] - before["failures"]))
    ops.deferSums = True
    (l1, gw1, gb1, m1, n1, f1), (l2, gw2, gb2, m2, n2, f2) = res
    assert f1 == 0 and f2 == 0
    assert m1 == 0 and m2 == 2                                # one multi-sink pass per step
    assert n2 < n1
    assert same_bits(gw1, gw2) and same_bits(gb1, gb2)
    assert abs(float(l1[0]) - float(l2[0])) <= RED_RTOL * abs(float(l1[0]))


def test_pending_sums_keep_the_semantics_of_sums_that_run_at_once(lazy_sums_ops):
    rows, cols = 2048, 512                                    # 2^20 elements: the multi-sink kernel runs
    xv, yv = D.uniform(rows * cols, 21, -1.0, 1.0), D.uniform(rows * cols, 22, -1.0, 1.0)
    gv = D.uniform(cols, 23, -1.0, 1.0)

    def script(o):
        x, y = o.createRaw([rows, cols], xv), o.createRaw([rows, cols], yv)
        g1, g2 = o.createRaw([1, cols], gv), o.createRaw([cols], gv)
        d = x.minus(y)
        loss = d.pow(2.0).mean()                          # pending
        x.timesAssign(2.0)                                # overwrites an operand: the mean is of the old x
        g1.plusAssign(d.times(y).sum(0, keepDimensions=True))
        g1.plusAssign(d.sum(0, keepDimensions=True))      # a second update of the same buffer, in order
        g2.plusAssign(d.times(0.5).sum(0))
        g2.timesAssign(3.0)                               # in-place write to a buffer with a pending update
        nested = d.minus(d.mean()).pow(2.0).sum()         # a sum over an expression that holds a pending sum
        spread = g2.broadcastTo([rows, cols]).plus(1.0).sum()
        p, q, r, t = d.exp().sum(), d.exp().sum(0), d.times(d).mean(), d.plus(y).sum(0, keepDimensions=True)    # four sinks, one pass
        view = g1.view([cols])
        return [loss, g1, g2, nested, spread, p, q, r, t, view, x]

    m0 = lazy_sums_ops.multiSinkEvaluations
    eager, lazy = both(lazy_sums_ops, script)
    assert lazy_sums_ops.multiSinkEvaluations > m0
    for k, (a, c) in enumerate(zip(eager, lazy)):
        scale = np.abs(a).max() + 1.0
        assert np.all(np.abs(a.astype(np.float64) - c) <= 2e-5 * scale), f"result {k}"
    assert same_bits(eager[10], lazy[10]) and same_bits(lazy[1].reshape(-1), lazy[9])


def test_multi_sink_call_checks_its_arguments(cuda_ops, gc_scope):
    lib = cuda_ops.lib
    rows, cols = 8, 128
    x = cuda_ops.createRaw([rows, cols], D.uniform(rows * cols, 31, -1.0, 1.0))
    o1, o2 = cuda_ops.createRaw([1]), cuda_ops.createRaw([cols])
    ins = lambda op, d=0, a=0, b=0, k=0: op | (d << 8) | (a << 12) | (b << 16) | (k << 20)
    shape, leaves, lsh = (C.c_int64 * 2)(rows, cols), (C.c_uint64 * 1)(x._buf()), (C.c_int64 * 2)(rows, cols)
    outs, means = (C.c_uint64 * 2)(o1._buf(), o2._buf()), (C.c_int * 2)(0, 0)

    def call(code, kinds, n_sinks=2):
        arr = (C.c_uint32 * len(code))(*code)
        return lib.ktc_expr_eval_multi(arr, len(code), None, 0, shape, 2, leaves, lsh, 1, None, 0, (C.c_int * 2)(*kinds), outs, means, n_sinks)

    good = [ins(L.X_LOAD, 0, k=0), ins(L.X_ACC, a=0, k=0), ins(L.X_ACC, a=0, k=1)]
    assert call(good, (L.EXPR_SUM_ALL, L.EXPR_SUM_ROWS)) == L.KTC_ENOTSUP           # 1024 elements: below expr_jit_min_elems
    assert call(good, (L.EXPR_SUM_ALL, L.EXPR_STORE_ONLY)) == L.KTC_EINVAL          # not a summing kind
    assert call(good[:2], (L.EXPR_SUM_ALL, L.EXPR_SUM_ROWS)) == L.KTC_EINVAL        # sink 1 is never fed
    assert call(good, (L.EXPR_SUM_ALL, L.EXPR_SUM_ROWS), n_sinks=5) == L.KTC_EINVAL
    assert call([ins(L.X_LOAD, 0, k=0), ins(L.X_ACC, a=0, k=0), ins(L.X_ACC, a=0, k=0)], (L.EXPR_SUM_ALL, L.EXPR_SUM_ROWS)) == L.KTC_EINVAL
    L.check(lib.ktc_tune_set(b"expr_jit_min_elems", 0))
    try:
        L.check(call(good, (L.EXPR_SUM_ALL, L.EXPR_SUM_ROWS)))
    finally:
        L.check(lib.ktc_tune_set(b"expr_jit_min_elems", 1 << 20))
    xa = x.toArray().astype(np.float64)
    assert abs(float(o1.toArray()[0]) - xa.sum()) <= RED_RTOL * np.abs(xa).sum()
    assert np.all(np.abs(o2.toArray() - xa.sum(axis=0)) <= RED_RTOL * np.abs(xa).sum(axis=0))


def test_generated_kernel_shape_tunables_do_not_change_a_bit(lazy_sums_ops):
    """Rows per batch, the occupancy hint and where the double accumulators live only reshape the generated code:
    the sharded step's loss and gradients are the same bits under every setting."""
    from kten_b200.sharded import ShardedSigmoidGraph
    ops = lazy_sums_ops
    rows, cols = 2048, 1024
    x = D.uniform(rows * cols, 40, -1.0, 1.0)
    w = D.normal(cols, 40, 0.0, 0.5, stream=1)
    b = D.uniform(cols, 40, -0.1, 0.1, stream=2)
    keys = (b"expr_jit_multi_rows", b"expr_jit_multi_min_blocks", b"expr_jit_multi_smem_acc")
    results = []
    before = expr_stats(ops)
    try:
        for setting in ((4, 3, 1), (1, 0, 0), (2, 4, 1), (8, 0, 0), (4, 0, 0)):
            for key, v in zip(keys, setting):
                L.check(ops.lib.ktc_tune_set(key, v))
            with ops.garbageCollector():
                g = ShardedSigmoidGraph(ops, ops.createRaw([rows, cols], x), ops.createRaw([1, cols], w), ops.createRaw([cols], b))
                m0 = ops.multiSinkEvaluations
                loss, gw, gb = g.step()
                results.append((loss.toArray().copy(), gw.toArray().copy(), gb.toArray().copy()))
                assert ops.multiSinkEvaluations == m0 + 1
                g.release_step()
    finally:
        for key, v in zip(keys, (4, 3, 1)):
            L.check(ops.lib.ktc_tune_set(key, v))
    after = expr_stats(ops)
    assert after["failures"] == before["failures"] and after["compiled"] >= before["compiled"] + 4
    for other in results[1:]:
        for p, q in zip(results[0], other):
            assert same_bits(p, q)


@pytest.mark.parametrize("shape", [[4096, 260], [64, 32, 516], [1024, 1024], [3, 128, 2052]], ids=str)
def test_last_axis_sum_sink(cuda_ops, gc_scope, shape):
    """ktc_expr_eval with the SUM_LAST sink (generated kernel): exp(x) stored and summed along the innermost axis, on
    extents that leave the last 128-column tile partly (or almost entirely) empty."""
    lib = cuda_ops.lib
    n = int(np.prod(shape))
    rows = n // shape[-1]
    xv = D.uniform(n, 51, -1.0, 1.0)
    x = cuda_ops.createRaw(shape, xv)
    e, sums = cuda_ops.createRaw(shape), cuda_ops.createRaw([rows])
    ins = lambda op, d=0, a=0, b=0, k=0: op | (d << 8) | (a << 12) | (b << 16) | (k << 20)
    code = [ins(L.X_LOAD, 0, k=0), ins(L.X_EXP, 1, 0), ins(L.X_STORE, a=1, k=0), ins(L.X_ACC, a=1, k=0)]
    arr = (C.c_uint32 * len(code))(*code)
    nd = len(shape)
    shp = (C.c_int64 * nd)(*shape)
    L.check(lib.ktc_tune_set(b"expr_jit_min_elems", 0))
    try:
        before = expr_stats(cuda_ops)
        L.check(lib.ktc_expr_eval(arr, len(code), None, 0, shp, nd, (C.c_uint64 * 1)(x._buf()), shp, 1, (C.c_uint64 * 1)(e._buf()), 1,
                                  L.EXPR_SUM_LAST, sums._buf(), 0))
        after = expr_stats(cuda_ops)
    finally:
        L.check(lib.ktc_tune_set(b"expr_jit_min_elems", 1 << 20))
    assert after["jit_launches"] == before["jit_launches"] + 1 and after["failures"] == before["failures"]
    got_e = e.toArray().reshape(rows, shape[-1])
    assert same_bits(got_e.reshape(-1), cuda_ops.createRaw([n], xv).exp().toArray())
    want = got_e.astype(np.float64).sum(axis=1)
    assert np.all(np.abs(sums.toArray() - want) <= RED_RTOL * want)
    assert lib.ktc_expr_eval(arr, len(code), None, 0, shp, nd, (C.c_uint64 * 1)(x._buf()), shp, 1, (C.c_uint64 * 1)(e._buf()), 1,
                             L.EXPR_SUM_LAST, sums._buf(), 1) == L.KTC_EINVAL          # a mean over the last axis is not offered


def test_softmax_normalisations_as_pending_last_axis_sums(lazy_sums_ops):
    rows, cols = 2048, 512                                   # 2^20 elements: generated kernels
    xv = D.uniform(rows * cols, 31, -2.0, 2.0)

    def script(o):
        x = o.createRaw([rows, cols], xv)
        m = x.max(-1, keepDimensions=True)
        e = x.minus(m).exp()
        z = e.sum(-1, keepDimensions=True)
        total = e.sum()                                    # same iteration space: one pass with two sinks
        sm = e.div(z)
        z2 = sm.sum(-1)                                    # holds the pending z: waits for it
        norm = sm.div(z2.view([rows, 1])).clamp(1e-7, 1.0 - 1e-7).log()
        return [z, total, z2, norm, sm]

    m0, u0 = lazy_sums_ops.multiSinkEvaluations, lazy_sums_ops.unfusedEvaluations
    eager, lazy = both(lazy_sums_ops, script)
    assert lazy_sums_ops.multiSinkEvaluations == m0 + 1 and lazy_sums_ops.unfusedEvaluations == u0
    for k, (a, c) in enumerate(zip(eager, lazy)):
        assert a.shape == c.shape
        assert np.all(np.abs(a.astype(np.float64) - c) <= 1e-5 * (np.abs(a) + 1e-3)), f"result {k}"
