"""Pins the CPU oracle (and the autograd caller) against the reference's own
known-answer tests.  No GPU involved."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.kten_cases import CASES, CASE_IDS, run_case


@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_reference_vectors_on_oracle(oracle_ops, case):
    run_case(oracle_ops, case)


@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_reference_vectors_on_jvm_faithful_oracle(case):
    # same vectors with kten-jvm's own accumulation (float, sequential)
    run_case(O.OracleTensorOperations(mode=0), case)


def test_java_max_min_semantics():
    nan = np.float32("nan")
    # Math.max/min propagate NaN and order -0 < +0 (JVMRawTensor.kt:159-160, 409-411)
    assert np.isnan(O.aggregate(O.MAX, [1.0, nan, 3.0], 1, 3, 1)[0])
    assert np.isnan(O.aggregate(O.MIN, [1.0, nan, 3.0], 1, 3, 1)[0])
    r = O.aggregate(O.MAX, [-0.0, 0.0], 1, 2, 1)
    assert r[0] == 0 and not np.signbit(r[0])
    r = O.aggregate(O.MIN, [0.0, -0.0], 1, 2, 1)
    assert r[0] == 0 and np.signbit(r[0])
    assert np.isnan(O.clamp([nan], 0.0, 1.0)[0])


def test_arg_semantics():
    nan, inf = np.float32("nan"), np.float32("inf")
    # strict compares from -inf: NaN never selected, ties -> lowest index, all -inf -> 0 (JVMRawTensor.kt:166-184)
    assert O.aggregate(O.ARGMAX, [nan, 2.0, 2.0], 1, 3, 1)[0] == 1
    assert O.aggregate(O.ARGMAX, [-inf, -inf], 1, 2, 1)[0] == 0
    assert O.aggregate(O.ARGMAX, [nan, nan], 1, 2, 1)[0] == 0
    assert O.aggregate(O.ARGMIN, [3.0, 1.0, 1.0], 1, 3, 1)[0] == 1
    assert O.aggregate(O.ARGMAX, [1.0, inf, inf], 1, 3, 1)[0] == 1


def test_java_pow_corner_cases():
    nan, inf = float("nan"), float("inf")
    p = lambda x, y: O.binary_same(O.POW, [x], [y])[0]
    assert p(nan, 0.0) == 1.0 and p(5.0, -0.0) == 1.0
    assert np.isnan(p(1.0, nan))            # Java: NaN exponent -> NaN (C99 would give 1)
    assert np.isnan(p(-1.0, inf)) and np.isnan(p(1.0, -inf))   # Java: |x| == 1, infinite exponent -> NaN
    assert p(2.0, 10.0) == 1024.0 and p(-2.0, 3.0) == -8.0 and np.isnan(p(-2.0, 0.5))
    assert p(0.0, -1.0) == inf and p(4.0, 0.5) == 2.0


def test_pow_two_equals_square_bit_exact():
    x = np.random.default_rng(0).uniform(-3, 3, 100000).astype(np.float32)
    assert np.array_equal(O.scalar(O.POW, x, 2.0), x * x)


def test_jvm_faithful_sum_stalls_exact_does_not():
    # the hazard that makes the exact mode the reduction target: sequential float
    # accumulation stops growing once the total reaches 2^24 ulps of the addend
    x = np.full(1 << 25, 0.25, dtype=np.float32)
    assert O.reduce_all(O.SUM, x, mode=0) == np.float32(4194304.0)     # 2^22: 0.25 is half an ulp there
    assert O.reduce_all(O.SUM, x, mode=1) == np.float32(8388608.0)
    assert O.reduce_all(O.MEAN, x, mode=0) == np.float32(0.25)         # mean() accumulates in double


def test_sum_to_shape_modes_agree_on_exact_data():
    rng = np.random.default_rng(1)
    x = (np.rint(rng.normal(size=(4, 6, 5)) * 16) / 16).astype(np.float32)
    for old in ([6, 1], [5], [1, 6, 5], [4, 1, 1], [4, 6, 5], [1]):
        a = O.sum_to_shape(x, [4, 6, 5], old, mode=0)
        b = O.sum_to_shape(x, [4, 6, 5], old, mode=1)
        assert np.array_equal(a, b)
        axes = tuple(range(3 - len(old))) + tuple(3 - len(old) + i for i, d in enumerate(old) if d == 1 and x.shape[3 - len(old) + i] != 1)
        ref = x.astype(np.float64).sum(axis=axes, keepdims=True).reshape(old)
        assert np.array_equal(a.reshape(old), ref.astype(np.float32))


def test_broadcast_shape_errors():
    with pytest.raises(ValueError):
        O.common_shape([2, 3], [4, 3])
    assert O.common_shape([32, 64, 128], [64, 1]) == [32, 64, 128]
    assert O.common_shape([3], [2, 1]) == [2, 3]


def test_softmax_cross_entropy_property_and_closed_form(oracle_ops):
    """The reference's own property (function node == one-hot spelling), then the closed form in
    float64: loss = mean(-log softmax[target]), gradient = (softmax - onehot) / rows."""
    from tests.kten_cases import softmax_cross_entropy_property
    loss, grad, x, t = softmax_cross_entropy_property(oracle_ops, rows=64, classes=512)
    xs = x.astype(np.float64)
    p = np.exp(xs - xs.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    rows = np.arange(x.shape[0])
    assert abs(float(loss[0]) + np.log(p[rows, t.astype(int)]).mean()) < 1e-5
    g = p.copy()
    g[rows, t.astype(int)] -= 1.0
    assert np.abs(g / x.shape[0] - grad).max() < 1e-7


def test_softmax_cross_entropy_argument_checks(oracle_ops):
    from kten_b200 import autograd as AG
    logits = AG.tensorOf(oracle_ops, np.zeros((2, 3), np.float32), requiresGrad=True)
    with pytest.raises(ValueError, match="2D logits"):
        AG.tensorOf(oracle_ops, np.zeros(3, np.float32), requiresGrad=True).softmaxCrossEntropy(AG.tensorOf(oracle_ops, [0.0, 1.0, 2.0]))
    with pytest.raises(ValueError, match="1D targets"):
        logits.softmaxCrossEntropy(AG.tensorOf(oracle_ops, np.zeros((2, 1), np.float32)))
    with pytest.raises(ValueError, match="same size at the first dimension"):
        logits.softmaxCrossEntropy(AG.tensorOf(oracle_ops, [0.0, 1.0, 2.0]))
    with pytest.raises(ValueError, match="don't require gradients"):
        logits.softmaxCrossEntropy(AG.tensorOf(oracle_ops, [0.0, 1.0], requiresGrad=True))
