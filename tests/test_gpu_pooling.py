"""Spatial pooling on the GPU (ktc_pool.cu through the C ABI): the reference's own fixture, and results, winner positions
and gradients bit-identical to the oracle's restatement of kten-jvm's loops -- NaN, ties, -infinity, padding, dilation, both
rounding modes of the output extent, 3-D and 4-D inputs."""
import ctypes as C

import numpy as np
import pytest

from kten_b200 import _lib as L
from kten_b200.nn import PoolingOptions, PoolingType
from oracle import oracle as O
from tests import kten_cases as K

pytestmark = pytest.mark.gpu
ORACLE = O.OracleTensorOperations()


def same_bits(a, b):
    """Bit-identical; a NaN matches a NaN (0f / 0 of an empty average window has no payload worth comparing)."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    if a.shape != b.shape:
        return False
    both_nan = np.isnan(a) & np.isnan(b)
    return bool(np.all((a.view(np.uint32) == b.view(np.uint32)) | both_nan))


def test_reference_fixture_max_pooling_1d(cuda_ops, gc_scope):
    got = K.max_pooling_1d_golden(cuda_ops)
    want = K.max_pooling_1d_golden(ORACLE)
    assert same_bits(got[0], want[0]) and same_bits(got[2], want[2])


MAX_CONFIGS = [((2, 2), (2, 2), (0, 0), (1, 1), False), ((3, 3), (2, 2), (1, 1), (1, 1), False), ((3, 2), (1, 2), (1, 0), (2, 1), True),
               ((3, 3), (2, 3), (1, 1), (2, 2), True), ((1, 1), (3, 3), (0, 0), (1, 1), True), ((5, 3), (3, 1), (2, 1), (1, 2), False),
               ((3, 3), (1, 1), (1, 1), (1, 1), False)]


@pytest.mark.parametrize("shape", [[3, 37, 29], [2, 5, 64, 48]], ids=["chw", "nchw"])
@pytest.mark.parametrize("k,s,p,d,ceil", MAX_CONFIGS)
def test_max_pooling_matches_the_oracle_bit_for_bit(cuda_ops, gc_scope, shape, k, s, p, d, ceil):
    rng = np.random.default_rng(11)
    x = rng.normal(size=shape).astype(np.float32)
    flat = x.reshape(-1)
    flat[::97] = np.nan
    flat[5::131] = -np.inf
    x.reshape(-1, shape[-2], shape[-1])[1] = np.round(x.reshape(-1, shape[-2], shape[-1])[1])        # ties: the first in window order wins
    opt = PoolingOptions(PoolingType.MAX, ceil)
    res = []
    for ops in (ORACLE, cuda_ops):
        op = ops.spatialPooling(k, p, s, d, opt)
        raw = ops.createRaw(shape, x.reshape(-1))
        out, idx = op.updateOutput(raw)
        g = np.random.default_rng(12).normal(size=out.shape).astype(np.float32)
        gin = op.calculateGradInput(raw, ops.createRaw(list(out.shape), g.reshape(-1)), idx)
        res.append((list(out.shape), out.toArray(), idx.toArray(), gin.toArray()))
    assert res[0][0] == res[1][0]
    for a, b in zip(res[0][1:], res[1][1:]):
        assert same_bits(a, b)
    assert (res[1][2] == -1).any() or not np.isinf(res[1][1]).any()      # a window without a winner: -infinity and index -1 go together


@pytest.mark.parametrize("shape", [[3, 37, 29], [2, 5, 64, 48]], ids=["chw", "nchw"])
@pytest.mark.parametrize("k,s,p,ceil,incl", [((2, 2), (2, 2), (0, 0), False, False), ((3, 3), (2, 2), (1, 1), False, True), ((3, 3), (2, 2), (1, 1), True, False),
                                             ((4, 2), (3, 1), (2, 1), True, True), ((1, 3), (2, 2), (0, 1), False, False), ((3, 3), (1, 1), (1, 1), False, False),
                                             ((1, 1), (3, 3), (0, 0), True, False)])
def test_average_pooling_matches_the_oracle_bit_for_bit(cuda_ops, gc_scope, shape, k, s, p, ceil, incl):
    x = np.random.default_rng(13).normal(size=shape).astype(np.float32)
    opt = PoolingOptions(PoolingType.AVG, ceil, incl)
    res = []
    for ops in (ORACLE, cuda_ops):
        op = ops.spatialPooling(k, p, s, (1, 1), opt)
        raw = ops.createRaw(shape, x.reshape(-1))
        out, idx = op.updateOutput(raw)
        assert idx is None
        g = np.random.default_rng(14).normal(size=out.shape).astype(np.float32)
        gin = op.calculateGradInput(raw, ops.createRaw(list(out.shape), g.reshape(-1)), None)
        res.append((list(out.shape), out.toArray(), gin.toArray()))
    assert res[0][0] == res[1][0]
    for a, b in zip(res[0][1:], res[1][1:]):
        assert same_bits(a, b)


def test_pooling_through_autograd_in_both_modes(cuda_ops, gc_scope):
    from kten_b200 import autograd as AG
    x = np.random.default_rng(15).normal(size=(4, 6, 32, 32)).astype(np.float32)
    want = None
    for lazy in (False, True):
        cuda_ops.lazy = lazy
        try:
            t = AG.tensorOf(cuda_ops, x, requiresGrad=True)
            yv = t.maxPooling2d((3, 3), (2, 2), (1, 1)).avgPooling2d((2, 2), includePadding=True).toArray()
            y = t.maxPooling2d((3, 3), (2, 2), (1, 1)).avgPooling2d((2, 2), includePadding=True)
            loss = y.pow(2.0).sum()
            loss.backward()                                  # frees the intermediate results of the graph
            got = (yv, t.grad().toArray())
        finally:
            cuda_ops.lazy = False
        if want is None:
            want = got
            to = AG.tensorOf(ORACLE, x, requiresGrad=True)
            yo = to.maxPooling2d((3, 3), (2, 2), (1, 1)).avgPooling2d((2, 2), includePadding=True)
            yo.pow(2.0).sum().backward()
            assert same_bits(got[0], yo.toArray()) and np.allclose(got[1], to.grad().toArray(), rtol=1e-6, atol=1e-7)
        else:
            assert same_bits(got[0], want[0]) and same_bits(got[1], want[1])


def test_argument_checks(cuda_ops, gc_scope):
    lib = cuda_ops.lib
    x = cuda_ops.createRaw([2, 8, 8], np.zeros(128, np.float32))
    out, idx = cuda_ops.createRaw([2, 4, 4]), cuda_ops.createRaw([2, 4, 4])
    geom = lambda *v: (C.c_int * 12)(*v)
    ok = geom(8, 8, 4, 4, 2, 2, 0, 0, 2, 2, 1, 1)
    L.check(lib.ktc_pool2d_max(out.storeReference, idx.storeReference, x.storeReference, 2, ok))
    assert lib.ktc_pool2d_max(out.storeReference, idx.storeReference, x.storeReference, 2, geom(8, 8, 4, 4, 2, 2, 2, 2, 2, 2, 1, 1)) == L.KTC_EINVAL      # padding > kernel / 2
    assert lib.ktc_pool2d_max(out.storeReference, idx.storeReference, x.storeReference, 2, geom(8, 8, 4, 4, 0, 2, 0, 0, 2, 2, 1, 1)) == L.KTC_EINVAL
    assert lib.ktc_pool2d_max(out.storeReference, idx.storeReference, x.storeReference, 2, geom(8, 8, 4, 4, 2, 2, 0, 0, 0, 2, 1, 1)) == L.KTC_EINVAL
    assert lib.ktc_pool2d_max(out.storeReference, idx.storeReference, x.storeReference, 2, geom(8, 8, 9, 9, 2, 2, 0, 0, 1, 1, 1, 1)) == L.KTC_EINVAL      # out too small for 9 x 9
    assert lib.ktc_pool2d_max(out.storeReference, out.storeReference, x.storeReference, 2, ok) == L.KTC_EINVAL                                            # aliasing
    assert lib.ktc_pool2d_avg(out.storeReference, x.storeReference, 2, geom(8, 8, 4, 4, 2, 2, 0, 0, 2, 2, 2, 1), 0) == L.KTC_EINVAL                      # no dilation
    assert lib.ktc_pool2d_avg(out.storeReference, x.storeReference, 3, ok, 0) == L.KTC_EINVAL                                                            # three planes do not fit
    with pytest.raises(ValueError, match="Padding should be smaller"):
        cuda_ops.spatialPooling((2, 2), (2, 2), (1, 1), (1, 1), PoolingOptions(PoolingType.MAX)).updateOutput(x)


def test_random_geometries_match_the_oracle(cuda_ops, gc_scope):
    """Sixty seeded geometries -- kernels 1 to 5, strides 1 to 4, any admissible padding, dilations 1 to 3, both rounding modes,
    odd plane sizes -- for max and average pooling: results, positions and gradients bit-identical to the oracle (windows
    other than 2 and 3, strides above 2 and dilations take the kernels with run-time window loops)."""
    rng = np.random.default_rng(2024)
    done = 0
    while done < 60:
        kh, kw = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        sh, sw = int(rng.integers(1, 5)), int(rng.integers(1, 5))
        ph, pw = int(rng.integers(0, kh // 2 + 1)), int(rng.integers(0, kw // 2 + 1))
        is_max = bool(rng.integers(0, 2))
        dh, dw = (int(rng.integers(1, 4)), int(rng.integers(1, 4))) if is_max else (1, 1)
        H, W = int(rng.integers(4, 40)), int(rng.integers(4, 40))
        shape = [int(rng.integers(1, 4)), int(rng.integers(1, 5)), H, W] if rng.integers(0, 2) else [int(rng.integers(1, 6)), H, W]
        opt = PoolingOptions(PoolingType.MAX if is_max else PoolingType.AVG, bool(rng.integers(0, 2)), bool(rng.integers(0, 2)))
        x = rng.normal(size=shape).astype(np.float32)
        if is_max:
            x.reshape(-1)[::53] = np.round(x.reshape(-1)[::53])
        res = []
        try:
            for ops in (ORACLE, cuda_ops):
                op = ops.spatialPooling((kh, kw), (ph, pw), (sh, sw), (dh, dw), opt)
                raw = ops.createRaw(shape, x.reshape(-1))
                out, idx = op.updateOutput(raw)
                g = np.random.default_rng(done).normal(size=out.shape).astype(np.float32)
                gin = op.calculateGradInput(raw, ops.createRaw(list(out.shape), g.reshape(-1)), idx)
                res.append((list(out.shape), out.toArray(), gin.toArray()) + ((idx.toArray(),) if idx is not None else ()))
        except ValueError as exc:                                    # the window does not fit the plane: both backends must say so
            assert "too small" in str(exc) and not res
            with pytest.raises(ValueError, match="too small"):
                cuda_ops.spatialPooling((kh, kw), (ph, pw), (sh, sw), (dh, dw), opt).updateOutput(cuda_ops.createRaw(shape, x.reshape(-1)))
            continue
        what = (kh, kw, sh, sw, ph, pw, dh, dw, shape, opt.type, opt.useCeil, opt.includePadding)
        assert res[0][0] == res[1][0], what
        for a, b in zip(res[0][1:], res[1][1:]):
            assert same_bits(a, b), what
        done += 1
