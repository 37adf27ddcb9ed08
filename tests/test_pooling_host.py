"""Spatial pooling on the CPU: the oracle's restatement of kten-jvm's loops against the reference's own fixture and against
definitions written without the reference's clipping tricks, and the shape rules of the host side (the same code computes
the output extents for the CUDA backend)."""
import numpy as np
import pytest

from kten_b200 import autograd as AG
from kten_b200.nn import PoolingOptions, PoolingType, pooled_size
from oracle import oracle as O
from tests.fake_lib import make_ops
from tests.kten_cases import max_pooling_1d_golden

ORACLE = O.OracleTensorOperations()


def test_reference_fixture_max_pooling_1d():
    res, total, grad = max_pooling_1d_golden(ORACLE)
    assert res.shape == (2, 3, 5) and grad.shape == (2, 3, 10)
    assert set(np.unique(grad)) <= {0.0, 1.0, 2.0, 3.0}


def brute_max(x, k, s, p, d, OH, OW):
    P, H, W = x.shape
    out = np.full((P, OH, OW), -np.inf, np.float32)
    idx = np.full((P, OH, OW), -1.0, np.float32)
    for q in range(P):
        for i in range(OH):
            for j in range(OW):
                for a in range(k[0]):
                    for b in range(k[1]):
                        y, xx = i * s[0] - p[0] + a * d[0], j * s[1] - p[1] + b * d[1]
                        if 0 <= y < H and 0 <= xx < W and x[q, y, xx] > out[q, i, j]:
                            out[q, i, j], idx[q, i, j] = x[q, y, xx], y * W + xx
    return out, idx


CONFIGS = [((2, 2), (2, 2), (0, 0), (1, 1), False), ((3, 3), (2, 2), (1, 1), (1, 1), False), ((3, 2), (1, 2), (1, 0), (2, 1), True),
           ((3, 3), (2, 3), (1, 1), (2, 2), True), ((1, 1), (3, 3), (0, 0), (1, 1), True), ((5, 3), (3, 1), (2, 1), (1, 2), False)]


@pytest.mark.parametrize("k,s,p,d,ceil", CONFIGS)
def test_oracle_max_pooling_against_the_definition(k, s, p, d, ceil):
    rng = np.random.default_rng(5)
    x = rng.normal(size=(2, 3, 11, 9)).astype(np.float32)
    x[0, 0, 3, 4] = np.nan
    x[1, 2] = np.round(x[1, 2])                                    # ties
    op = ORACLE.spatialPooling(k, p, s, d, PoolingOptions(PoolingType.MAX, ceil))
    raw = ORACLE.createRaw(list(x.shape), x.reshape(-1))
    out, idx = op.updateOutput(raw)
    OH, OW = out.shape[-2:]
    want, widx = brute_max(x.reshape(6, 11, 9), k, s, p, d, OH, OW)
    assert np.array_equal(out.toArray().reshape(want.shape), want) and np.array_equal(idx.toArray().reshape(widx.shape), widx)
    g = rng.normal(size=out.shape).astype(np.float32)
    gin = op.calculateGradInput(raw, ORACLE.createRaw(list(out.shape), g.reshape(-1)), idx).toArray().reshape(6, 99)
    want_g = np.zeros((6, 99), np.float32)
    for q in range(6):
        for o in range(OH * OW):
            t = int(widx.reshape(6, -1)[q, o])
            if t >= 0:
                want_g[q, t] = np.float32(want_g[q, t] + g.reshape(6, -1)[q, o])
    assert np.array_equal(gin, want_g)


@pytest.mark.parametrize("k,s,p,ceil,incl", [((2, 2), (2, 2), (0, 0), False, False), ((3, 3), (2, 2), (1, 1), False, True), ((3, 3), (2, 2), (1, 1), True, False),
                                             ((4, 2), (3, 1), (2, 1), True, True), ((1, 3), (2, 2), (0, 1), False, False)])
def test_oracle_average_pooling_against_the_definition(k, s, p, ceil, incl):
    rng = np.random.default_rng(6)
    x = rng.normal(size=(4, 10, 7)).astype(np.float32)
    op = ORACLE.spatialPooling(k, p, s, (1, 1), PoolingOptions(PoolingType.AVG, ceil, incl))
    raw = ORACLE.createRaw([4, 10, 7], x.reshape(-1))
    out, idx = op.updateOutput(raw)
    assert idx is None
    OH, OW = out.shape[-2:]
    got = out.toArray().reshape(4, OH, OW)
    for i in range(OH):
        for j in range(OW):
            ys = [y for y in range(i * s[0] - p[0], i * s[0] - p[0] + k[0]) if y < 10 + p[0]]
            xs = [c for c in range(j * s[1] - p[1], j * s[1] - p[1] + k[1]) if c < 7 + p[1]]
            inside = [(y, c) for y in ys for c in xs if 0 <= y < 10 and 0 <= c < 7]
            n = len(ys) * len(xs) if incl else len(inside)
            want = sum((x[:, y, c].astype(np.float64) for y, c in inside), np.zeros(4)) / n
            assert np.allclose(got[:, i, j], want, rtol=1e-6, atol=1e-7)
    # the gradient of sum(out * g) by finite reasoning: every input receives g / n from each window that holds it
    g = rng.normal(size=(4, OH, OW)).astype(np.float32)
    gin = op.calculateGradInput(raw, ORACLE.createRaw([4, OH, OW], g.reshape(-1)), None).toArray().reshape(4, 10, 7)
    want_g = np.zeros((4, 10, 7))
    for i in range(OH):
        for j in range(OW):
            ys = [y for y in range(i * s[0] - p[0], i * s[0] - p[0] + k[0]) if y < 10 + p[0]]
            xs = [c for c in range(j * s[1] - p[1], j * s[1] - p[1] + k[1]) if c < 7 + p[1]]
            inside = [(y, c) for y in ys for c in xs if 0 <= y < 10 and 0 <= c < 7]
            n = len(ys) * len(xs) if incl else len(inside)
            for y, c in inside:
                want_g[:, y, c] += g[:, i, j].astype(np.float64) / n
    assert np.allclose(gin, want_g, rtol=1e-5, atol=1e-6)


def test_output_extents_and_checks():
    assert pooled_size(10, 2, 3, 1, 2, True) == 5 and pooled_size(10, 2, 3, 1, 2, False) == 4
    assert pooled_size(11, 1, 1, 0, 3, True) == 5                   # a last window beyond the plane: kept when there is no padding
    x = ORACLE.createRaw([1, 2, 8, 8], np.zeros(128, np.float32))
    with pytest.raises(ValueError, match="Padding should be smaller"):
        ORACLE.spatialPooling((2, 2), (2, 2), (1, 1), (1, 1), PoolingOptions(PoolingType.MAX)).updateOutput(x)
    with pytest.raises(ValueError, match="Input must be 3D or 4D"):
        ORACLE.spatialPooling((2, 2), (0, 0), (1, 1), (1, 1), PoolingOptions(PoolingType.MAX)).updateOutput(ORACLE.createRaw([8, 8], np.zeros(64, np.float32)))
    with pytest.raises(ValueError, match="too small"):
        ORACLE.spatialPooling((9, 9), (0, 0), (1, 1), (1, 1), PoolingOptions(PoolingType.AVG)).updateOutput(x)
    op = ORACLE.spatialPooling((2, 2), (0, 0), (2, 2), (1, 1), PoolingOptions(PoolingType.MAX))
    out, idx = op.updateOutput(x)
    with pytest.raises(ValueError, match="Invalid gradient shape"):
        op.calculateGradInput(x, ORACLE.createRaw([1, 2, 3, 4], np.zeros(24, np.float32)), idx)
    # with padding, a last window that would start in the right padding is dropped (JVMSpatialPoolingBase.kt:64-69)
    op = ORACLE.spatialPooling((2, 2), (1, 1), (2, 2), (1, 1), PoolingOptions(PoolingType.MAX, True))
    assert op.updateOutput(ORACLE.createRaw([1, 5, 5], np.zeros(25, np.float32)))[0].shape == [1, 3, 3]
    t = AG.tensorOf(ORACLE, np.zeros((2, 8), np.float32))
    with pytest.raises(RuntimeError, match="1D pooling cannot be applied"):
        t.maxPooling1d(2)


def test_the_backend_host_code_on_the_stand_in_library():
    """The CUDA backend's own host part (kten_b200/nn.py: checks, output extents, result tensors; the autograd function) over
    the stand-in library, whose pooling entry points run the oracle's loops on the extents they are given: the reference
    fixture, both execution modes, and every geometry of the oracle tests against the oracle backend."""
    for lazy in (False, True):
        ops = make_ops()
        ops.lazy = lazy
        with ops.garbageCollector():
            got = max_pooling_1d_golden(ops)
            want = max_pooling_1d_golden(ORACLE)
            assert all(np.array_equal(a, b) for a, b in zip(got, want))
    rng = np.random.default_rng(8)
    x = rng.normal(size=(2, 3, 11, 9)).astype(np.float32)
    ops = make_ops()
    with ops.garbageCollector():
        for k, s, p, d, ceil in CONFIGS:
            for kind in (PoolingType.MAX, PoolingType.AVG):
                opt = PoolingOptions(kind, ceil, includePadding=(kind == PoolingType.AVG and ceil))
                res = []
                for backend in (ORACLE, ops):
                    op = backend.spatialPooling(k, p, s, d, opt)
                    raw = backend.createRaw(list(x.shape), x.reshape(-1))
                    out, idx = op.updateOutput(raw)
                    g = backend.createRaw(list(out.shape), np.arange(int(np.prod(out.shape)), dtype=np.float32))
                    gin = op.calculateGradInput(raw, g, idx)
                    res.append((list(out.shape), out.toArray(), gin.toArray()))
                assert res[0][0] == res[1][0] and np.array_equal(res[0][1], res[1][1], equal_nan=True) and np.array_equal(res[0][2], res[1][2], equal_nan=True)
        with pytest.raises(ValueError, match="Padding should be smaller"):
            ops.spatialPooling((2, 2), (2, 2), (1, 1), (1, 1), PoolingOptions(PoolingType.MAX)).updateOutput(ops.createRaw([1, 2, 8, 8], np.zeros(128, np.float32)))
        with pytest.raises(ValueError, match="too small"):
            ops.spatialPooling((9, 9), (0, 0), (1, 1), (1, 1), PoolingOptions(PoolingType.AVG)).updateOutput(ops.createRaw([1, 2, 8, 8], np.zeros(128, np.float32)))
