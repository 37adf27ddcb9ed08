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
