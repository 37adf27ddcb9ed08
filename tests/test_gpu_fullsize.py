"""The benchmark's full-size configurations (2^28 elements per operand), checked through
properties that do not need a full CPU pass: oracle comparison on windows of the output,
checksums of checksums for the reductions, and value-at-index consistency for argmax."""
import ctypes as C

import numpy as np
import pytest

from kten_b200 import _lib as L
from kten_b200 import datagen as D
from oracle import oracle as O

pytestmark = pytest.mark.gpu

N = 1 << 28
WIN = 1 << 16
OFFSETS = [0, 4096 * 7 + 4, (N // 3) & ~3, N // 2 - WIN // 2, N - WIN - 12, N - WIN]


def window(ops, raw, off, n=WIN):
    out = np.empty(n, dtype=np.float32)
    L.check(ops.lib.ktc_d2h(out.ctypes.data_as(C.c_void_p), raw.storeReference, off, n, 1))
    return out


def same_bits(a, b):
    a, b = np.asarray(a, np.float32).reshape(-1), np.asarray(b, np.float32).reshape(-1)
    return bool(np.all((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))))


def test_config2_contiguous_sweep_windows(cuda_ops, gc_scope):
    ha, hb = D.uniform(N, 1, 0.1, 2.0), D.uniform(N, 2, 0.1, 2.0)
    a, b = cuda_ops.createRaw([N], ha), cuda_ops.createRaw([N], hb)
    for name, k, o in (("plus", L.PLUS, O.PLUS), ("times", L.TIMES, O.TIMES), ("div", L.DIV, O.DIV), ("pow", L.POW, O.POW)):
        r = a._binary(k, b)
        for off in OFFSETS:
            got, want = window(cuda_ops, r, off), O.binary_same(o, ha[off:off + WIN], hb[off:off + WIN])
            if name == "pow":
                assert O.ulp_distance(got, want).max() <= 2
            else:
                assert same_bits(got, want), f"{name} at {off}"
        r.release()
    for name, k, o in (("exp", L.EXP, O.EXP), ("log", L.LOG, O.LOG), ("tanh", L.TANH, O.TANH), ("sigmoid", L.SIGMOID, O.SIGMOID)):
        r = a._unary(k)
        for off in OFFSETS:
            d = O.ulp_distance(window(cuda_ops, r, off), O.unary(o, ha[off:off + WIN]))
            assert d.max() <= 2, f"{name} at {off}: {d.max()} ulp"
        r.release()


def test_config3_broadcast_windows(cuda_ops, gc_scope):
    shape = [1024, 1024, 256]
    ha = D.normal(N, 3, 0.0, 1.0)
    hb, hc = D.uniform(1024, 4, 0.5, 2.0), D.uniform(1024 * 256, 5, -1.0, 1.0)
    a, b, c = cuda_ops.createRaw(shape, ha), cuda_ops.createRaw([1, 1024, 1], hb), cuda_ops.createRaw([1024, 1, 256], hc)
    t = a.times(b)
    tc = t.plus(c)
    q = a.div(b)
    assert tc.shape == shape and q.shape == shape
    rows = WIN // 256                                    # a window is `rows` consecutive [256]-rows
    for off in OFFSETS:
        off = off // 256 * 256
        r0 = off // 256                                   # flat row index = i0 * 1024 + i1
        i0, i1 = np.divmod(np.arange(r0, r0 + rows), 1024)
        aw = ha[off:off + WIN].reshape(rows, 256)
        bw = hb[i1].reshape(rows, 1)
        cw = hc.reshape(1024, 256)[i0]
        want_t = (aw * bw).astype(np.float32)
        assert same_bits(window(cuda_ops, t, off), want_t)
        assert same_bits(window(cuda_ops, tc, off), (want_t + cw).astype(np.float32))
        assert same_bits(window(cuda_ops, q, off), (aw / bw).astype(np.float32))


def test_config4_reductions_checksums(cuda_ops, gc_scope):
    hx = D.normal(N, 6, 0.0, 1.0, quantum=16.0)          # multiples of 1/16: every summation order is exact
    x = cuda_ops.createRaw([65536, 4096], hx)
    row_sum, row_mean = x.sum(1), x.mean(1)
    row_max, row_arg = x.max(1), x.argMax(1)
    full = x.sum()
    x.shape = [512, 4096, 128]
    mid_sum, mid_max = x.sum(1), x.max(1)
    # checksum of checksums: all three routes to the grand total agree bit for bit
    total = float(full.toArray()[0])
    assert total == float(row_sum.sum().toArray()[0]) == float(mid_sum.sum().toArray()[0])
    assert total == float(hx.astype(np.float64).sum())
    # rows against the oracle on a sample of rows, and against numpy for all rows
    rs, rm, rx, ra = row_sum.toArray(), row_mean.toArray(), row_max.toArray(), row_arg.toArray()
    h2 = hx.reshape(65536, 4096)
    assert np.array_equal(rs, h2.astype(np.float64).sum(axis=1).astype(np.float32))
    assert np.array_equal(rm, (h2.astype(np.float64).sum(axis=1) / 4096).astype(np.float32))
    assert np.array_equal(rx, h2.max(axis=1))
    assert np.array_equal(ra, h2.argmax(axis=1).astype(np.float32))        # numpy also returns the first maximum
    idx = ra.astype(np.int64)
    assert np.array_equal(h2[np.arange(65536), idx], rx)                    # the value at the index is the maximum
    ties = (h2 == rx[:, None]).sum(axis=1)
    assert (ties > 1).mean() > 0.05                                          # ties do occur, so the rule was exercised
    sample = slice(1000, 1064)
    assert same_bits(rs[sample], O.aggregate(O.SUM, h2[sample], 64, 4096, 1, mode=0))      # kten-jvm's own order agrees too
    assert same_bits(ra[sample], O.aggregate(O.ARGMAX, h2[sample], 64, 4096, 1))
    # middle axis
    h3 = hx.reshape(512, 4096, 128)
    assert np.array_equal(mid_sum.toArray(), h3.astype(np.float64).sum(axis=1).astype(np.float32))
    assert np.array_equal(mid_max.toArray(), h3.max(axis=1))
    # the grand maximum through both routes
    assert float(row_max.max(0).toArray()[0]) == float(mid_max.max(0).max(0).toArray()[0]) == float(hx.max())


def test_config5_step_modes_agree_at_full_size(cuda_ops, gc_scope):
    """The sharded-graph step on the whole x[262144, 1024] in the backend's three execution modes -- call by call,
    deferred with one sum per pass, deferred with loss and both gradients in ONE pass -- and as two row shards
    whose partial results are added (what the ranks of a sharded run compute).  The two deferred modes give the
    same gradient bits; everything else agrees within 1e-5 of the sum of the absolute terms, which the device
    computes itself (the terms of the loss and of grad b are positive, so those sums are their own bound)."""
    from kten_b200.sharded import ShardedSigmoidGraph
    ops = cuda_ops
    rows, cols = 262144, 1024
    hx = D.uniform(rows * cols, 0, -1.0, 1.0)
    hw = D.normal(cols, 0, 0.0, 0.02, stream=1)
    hb = D.uniform(cols, 0, -0.1, 0.1, stream=2)
    x, w, b = ops.createRaw([rows, cols], hx), ops.createRaw([1, cols], hw), ops.createRaw([cols], hb)

    def run(xr, lazy, defer):
        ops.lazy, ops.deferSums = lazy, defer
        try:
            g = ShardedSigmoidGraph(ops, xr, w, b)
            loss, gw, gb = g.step()
            out = (float(loss.toArray()[0]), gw.toArray().reshape(-1).astype(np.float64), gb.toArray().astype(np.float64))
            g.release_step()
            return out
        finally:
            ops.lazy, ops.deferSums = False, True

    m0 = ops.multiSinkEvaluations
    eager = run(x, False, True)
    single = run(x, True, False)
    multi = run(x, True, True)
    assert ops.multiSinkEvaluations == m0 + 1
    half = rows // 2
    top, bottom = x.narrow(0, 0, half), x.narrow(0, half, half)
    parts = [run(top, True, True), run(bottom, True, True)]
    sharded = tuple(p + q for p, q in zip(*parts))
    # bound on the absolute terms: s = sigmoid(x*w+b), gz = 2 s s (1-s) >= 0, so sum|gz| = grad b and sum|gz x| = sum(gz |x|)
    s = x.times(w).plus(b).sigmoid()
    gz = s.times(s).times(s.unaryMinus().plus(1.0)).times(2.0)
    abs_gw = gz.times(x.abs()).sum(0).toArray().astype(np.float64)
    assert np.array_equal(single[1], multi[1]) and np.array_equal(single[2], multi[2])
    for other in (single, multi, sharded):
        assert abs(other[0] - eager[0]) <= 1e-5 * eager[0]
        assert np.all(np.abs(other[2] - eager[2]) <= 1e-5 * eager[2])
        assert np.all(np.abs(other[1] - eager[1]) <= 1e-5 * abs_gw)
    # closed form in float64 on a sample of columns
    colsamp = [0, 1, 511, 1023]
    X = hx.reshape(rows, cols)[:, colsamp].astype(np.float64)
    S = 1.0 / (1.0 + np.exp(-(X * hw[colsamp] + hb[colsamp])))
    GZ = 2.0 * S * S * (1.0 - S)
    assert np.all(np.abs(multi[2][colsamp] - GZ.sum(axis=0)) <= 1e-5 * GZ.sum(axis=0))
    assert np.all(np.abs(multi[1][colsamp] - (GZ * X).sum(axis=0)) <= 1e-5 * np.abs(GZ * X).sum(axis=0))
