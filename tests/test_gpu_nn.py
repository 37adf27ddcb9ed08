"""Batch normalisation and nearest-neighbour upsampling on the GPU: the reference's property tests
(TensorTestsBase.kt:2015-2200) in both execution modes, and the operations themselves against the oracle's
restatement of kten-jvm on shapes that exercise every layout (channel axis first, last, in the middle)."""
import numpy as np
import pytest

from oracle import oracle as O
from tests import kten_cases as K
from tests.test_nn_host import assert_bn_close, bn_both

pytestmark = pytest.mark.gpu
ORACLE = O.OracleTensorOperations()


@pytest.fixture(params=[False, True], ids=["call by call", "deferred"])
def ops(request, cuda_ops):
    cuda_ops.lazy = request.param
    try:
        with cuda_ops.garbageCollector():
            yield cuda_ops
    finally:
        cuda_ops.lazy = False


def test_reference_property_tests(ops):
    want = K.batch_norm_training_property(ORACLE, True)
    got = K.batch_norm_training_property(ops, True)
    for k in want:                                                   # same seeds: the device agrees with the oracle, not only with itself
        assert np.allclose(got[k], want[k], rtol=2e-5, atol=2e-6), k
    K.batch_norm_training_property(ops, False)
    assert np.allclose(K.batch_norm_inference_property(ops, True), K.batch_norm_inference_property(ORACLE, True), atol=1e-6)
    K.batch_norm_inference_property(ops, False)
    out, grad = K.upsample_nearest_property(ops)
    want_out, want_grad = K.upsample_nearest_property(ORACLE)
    assert np.array_equal(out, want_out) and np.allclose(grad, want_grad, atol=4e-6)


@pytest.mark.parametrize("shape,axis", [([64, 16, 24, 24], 1), ([512, 128], 1), ([96, 4096], 0), ([8, 5, 3, 33], 2), ([1, 32, 4096], 1), ([300, 7, 5], 1)],
                         ids=["nchw", "channel last", "channel first", "odd extents", "one image", "small inner"])
def test_batch_norm_matches_the_oracle(ops, shape, axis):
    rng = np.random.default_rng(11)
    for training in (True, False):
        for affine in (True, False):
            got, want = bn_both(ops, ORACLE, rng, shape, axis, training, affine, True)
            assert_bn_close(got, want, (shape, axis, training, affine))
    got, want = bn_both(ops, ORACLE, rng, shape, axis, True, True, False)
    assert_bn_close(got, want, (shape, axis, "no running statistics"))


def test_batch_norm_output_has_the_bits_of_the_reference_given_its_statistics(ops):
    """Inference mode takes the statistics as inputs, so nothing but the reference's per-element float operations is
    left: (x - mean) * stdev * gamma + beta, bit for bit."""
    rng = np.random.default_rng(12)
    shape, C = [32, 8, 16, 16], 8
    x = rng.normal(0, 2, shape).astype(np.float32)
    x.reshape(-1)[::97] = 0.0
    rm, rv = rng.normal(0, 1, C).astype(np.float32), rng.uniform(0.1, 3, C).astype(np.float32)
    g, b = rng.normal(0, 1, C).astype(np.float32), rng.normal(0, 1, C).astype(np.float32)
    outs = []
    for backend in (ops, ORACLE):
        mk = lambda a, s: backend.createRaw(s, a.reshape(-1))
        out, _, _ = backend.batchNorm(1, 0.1, 1e-3, False).calculateOutput(mk(x, shape), mk(rm, [C]), mk(rv, [C]), mk(g, [C]), mk(b, [C]))
        outs.append(np.asarray(out.toArray(), np.float32).reshape(-1))
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))


def test_batch_norm_training_is_three_passes_forward_and_two_backward(cuda_ops):
    """Recorded, the forward reads the input three times (mean, centred squares, normalise) and the backward takes
    both sums in one pass with two sinks before the gradient pass."""
    ops = cuda_ops
    rng = np.random.default_rng(13)
    shape, C = [256, 32, 32, 32], 32                                 # 2^23 elements: the generated kernels run
    with ops.garbageCollector():
        x = ops.createRaw(shape, rng.normal(0, 1, shape).astype(np.float32).reshape(-1))
        go = ops.createRaw(shape, rng.normal(0, 1, shape).astype(np.float32).reshape(-1))
        g, b = ops.createRaw([C], np.ones(C, np.float32)), ops.createRaw([C], np.zeros(C, np.float32))
        bn = ops.batchNorm(1, 0.1, 1e-3, True)
        for _ in range(2):                                           # the second round hits the program cache
            s0 = ops._recorder.stats()
            out, mean, std = bn.calculateOutput(x, None, None, g, b)
            s1 = ops._recorder.stats()
            gi, gg, gb = bn.calculateGrads(x, None, None, mean, std, g, go, True, True, True)
            gi._buf(); gg._buf(); gb._buf()
            s2 = ops._recorder.stats()
        assert s2["multi_sink"] - s1["multi_sink"] == 1              # sum(gradOut) and sum((x - mean) * gradOut) share a pass
        assert s1["unfused"] == s0["unfused"] and s2["unfused"] == s1["unfused"]
        want = ORACLE.batchNorm(1, 0.1, 1e-3, True)
        o_out, o_mean, o_std = want.calculateOutput(ORACLE.createRaw(shape, x.toArray().reshape(-1)), None, None,
                                                    ORACLE.createRaw([C], np.ones(C, np.float32)), ORACLE.createRaw([C], np.zeros(C, np.float32)))
        assert np.allclose(out.toArray().reshape(-1), o_out.toArray().reshape(-1), atol=2e-5)
        assert np.allclose(mean.toArray(), o_mean.toArray(), atol=1e-6) and np.allclose(std.toArray(), o_std.toArray(), rtol=1e-5)


@pytest.mark.parametrize("shape,scale", [([8, 3, 32, 48], 2), ([3, 6, 5], 4), ([2, 2, 7, 9], 3), ([64, 4, 64, 64], 2)])
def test_upsample_matches_the_oracle(ops, shape, scale):
    rng = np.random.default_rng(14)
    x = rng.normal(0, 1, shape).astype(np.float32)
    up, upo = ops.upsample("NEAREST", scale), ORACLE.upsample("NEAREST", scale)
    a, o = up.upsample(ops.createRaw(shape, x.reshape(-1))), upo.upsample(ORACLE.createRaw(shape, x.reshape(-1)))
    assert a.shape == o.shape
    assert np.array_equal(a.toArray().reshape(-1), o.toArray().reshape(-1))
    g = rng.normal(0, 1, a.shape).astype(np.float32)
    ga, g0 = up.calculateGrad(ops.createRaw(a.shape, g.reshape(-1)), shape), upo.calculateGrad(ORACLE.createRaw(a.shape, g.reshape(-1)), shape)
    assert ga.shape == g0.shape == shape
    assert np.allclose(ga.toArray().reshape(-1), g0.toArray().reshape(-1), atol=1e-5)
    # the library's kernel adds the block in kten-jvm's order in float: the bits of the oracle in its kten-jvm-faithful mode
    faithful = O.OracleTensorOperations(mode=0)
    gf = faithful.upsample("NEAREST", scale).calculateGrad(faithful.createRaw(a.shape, g.reshape(-1)), shape)
    assert np.array_equal(ga.toArray().reshape(-1).view(np.uint32), gf.toArray().reshape(-1).view(np.uint32))
