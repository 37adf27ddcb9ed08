"""Batch normalisation and nearest-neighbour upsampling: the oracle's restatement of kten-jvm against the reference's own
property tests, and the CUDA backend's composition of recorded raw-tensor calls (kten_b200/nn.py) against the oracle
on the stand-in library."""
import numpy as np
import pytest

from oracle import oracle as O
from tests import kten_cases as K
from tests.fake_lib import make_ops


@pytest.mark.parametrize("mode", [1, 0], ids=["exact", "jvm-faithful"])
def test_reference_property_tests_on_the_oracle(mode):
    ops = O.OracleTensorOperations(mode)
    K.batch_norm_training_property(ops, True)
    K.batch_norm_training_property(ops, False)
    K.batch_norm_inference_property(ops, True)
    K.batch_norm_inference_property(ops, False)
    K.upsample_nearest_property(ops)


def bn_both(ops_c, ops_o, rng, shape, axis, training, affine, running):
    """The same batch norm forward + backward on two backends; returns the two lists of arrays."""
    C = shape[axis]
    x, go = rng.normal(0, 1, shape).astype(np.float32), rng.normal(0, 1, shape).astype(np.float32)
    g = rng.uniform(0.5, 1.5, C).astype(np.float32) if affine else None
    b = rng.uniform(-1, 1, C).astype(np.float32) if affine else None
    rm0, rv0 = rng.uniform(-1, 1, C).astype(np.float32), rng.uniform(0.5, 2, C).astype(np.float32)
    res = []
    for ops in (ops_c, ops_o):
        mk = lambda a, s: None if a is None else ops.createRaw(s, a.reshape(-1))
        rx, rgo = mk(x, list(shape)), mk(go, list(shape))
        rm, rv = (mk(rm0.copy(), [C]), mk(rv0.copy(), [C])) if running else (None, None)
        bn = ops.batchNorm(axis, 0.1, 1e-3, training)
        out, mean, std = bn.calculateOutput(rx, rm, rv, mk(g, [C]), mk(b, [C]))
        gi, gg, gb = bn.calculateGrads(rx, rm, rv, mean, std, mk(g, [C]), rgo, True, affine, affine)
        arr = lambda t: None if t is None else np.asarray(t.toArray()).reshape(-1)
        res.append({"out": arr(out), "mean": arr(mean), "std": arr(std), "running mean": arr(rm), "running var": arr(rv),
                    "grad in": arr(gi), "grad gamma": arr(gg), "grad beta": arr(gb)})
    return res


def assert_bn_close(got, want, what, rtol=2e-5):
    for name in want:
        a, o = got[name], want[name]
        assert (a is None) == (o is None), (name, what)
        if a is None:
            continue
        err = float(np.abs(a.astype(np.float64) - o.astype(np.float64)).max(initial=0.0))
        assert err <= rtol * max(1.0, float(np.abs(o).max(initial=0.0))), (name, err, what)


@pytest.mark.parametrize("lazy", [False, True], ids=["call by call", "deferred"])
def test_batch_norm_composition_matches_the_oracle(lazy):
    rng = np.random.default_rng(3)
    ops_c, ops_o = make_ops(), O.OracleTensorOperations()
    ops_c.lazy = lazy
    with ops_c.garbageCollector():
        for shape, axis in (([6, 4, 8], 1), ([5, 8], 1), ([8, 12], 0), ([3, 4, 2, 8], 2), ([4, 3, 4, 4], 1), ([1, 4, 8], 1)):
            for training in (True, False):
                for affine in (True, False):
                    got, want = bn_both(ops_c, ops_o, rng, shape, axis, training, affine, True)
                    assert_bn_close(got, want, (shape, axis, training, affine))
            got, want = bn_both(ops_c, ops_o, rng, shape, axis, True, True, False)          # no running statistics
            assert_bn_close(got, want, (shape, axis, "no running statistics"))
    assert ops_c.lazy == lazy                                       # the operation records inside and restores the mode


def test_batch_norm_with_zero_epsilon_and_constant_channel():
    """sum == 0 and epsilon == 0: the reference leaves the inverse deviation at 0 (JVMBatchNorm.kt:63-65)."""
    ops_c, ops_o = make_ops(), O.OracleTensorOperations()
    x = np.random.default_rng(1).normal(0, 1, (4, 3, 8)).astype(np.float32)
    x[:, 1, :] = 2.5
    outs = []
    for ops in (ops_c, ops_o):
        bn = ops.batchNorm(1, 0.1, 0.0, True)
        out, mean, std = bn.calculateOutput(ops.createRaw([4, 3, 8], x.reshape(-1)), None, None, None, None)
        outs.append((np.asarray(out.toArray()).reshape(4, 3, 8), np.asarray(std.toArray()).reshape(-1)))
    assert outs[0][1][1] == 0.0 and outs[1][1][1] == 0.0
    assert np.all(outs[0][0][:, 1, :] == 0.0)
    assert np.allclose(outs[0][0], outs[1][0], atol=2e-6)


def test_upsample_composition_matches_the_oracle():
    rng = np.random.default_rng(2)
    ops_c, ops_o = make_ops(), O.OracleTensorOperations()
    for shape, scale in (([2, 3, 4, 8], 2), ([3, 6, 4], 4), ([1, 1, 1, 4], 3)):
        x = rng.normal(0, 1, shape).astype(np.float32)
        up, upo = ops_c.upsample("NEAREST", scale), ops_o.upsample("NEAREST", scale)
        a, o = up.upsample(ops_c.createRaw(shape, x.reshape(-1))), upo.upsample(ops_o.createRaw(shape, x.reshape(-1)))
        assert a.shape == o.shape == shape[:-2] + [shape[-2] * scale, shape[-1] * scale]
        assert np.array_equal(np.asarray(a.toArray()).reshape(-1), np.asarray(o.toArray()).reshape(-1))
        ga, g0 = up.calculateGrad(a, shape), upo.calculateGrad(o, shape)
        assert ga.shape == g0.shape == shape
        assert np.allclose(np.asarray(ga.toArray()).reshape(-1), np.asarray(g0.toArray()).reshape(-1), atol=2e-6)
    with pytest.raises(ValueError, match="3 or 4 dimensions"):
        ops_c.upsample("NEAREST", 2).upsample(ops_c.createRaw([4, 4]))
    with pytest.raises(ValueError, match="does not align"):
        ops_c.upsample("NEAREST", 2).calculateGrad(ops_c.createRaw([2, 3, 8, 8]), [2, 3, 4, 8])
