"""Runs the reference's known-answer graphs (tests/golden/reference_test_vectors.json)
on any backend that offers the RawTensor / TensorOperations methods."""
from __future__ import annotations

import json
import os

import numpy as np

from kten_b200 import autograd as AG

HERE = os.path.dirname(os.path.abspath(__file__))

with open(os.path.join(HERE, "golden", "reference_test_vectors.json")) as fh:
    CASES = json.load(fh)["cases"]
CASE_IDS = [c["name"] for c in CASES]


def _t(ops, spec, grad=False):
    return AG.tensorOf(ops, spec["data"], spec["shape"], requiresGrad=grad)


def _expect(spec):
    if "fill" in spec:
        return np.full(spec["shape"], spec["fill"], dtype=np.float32)
    return np.asarray(spec["data"], dtype=np.float32).reshape(spec["shape"])


def assert_tensor_equals(expected_spec, actual, tol):
    """assertTensorEquals (kten-testing/.../TestUtils.kt:9-29): equal shapes, then
    per-element absolute difference <= tolerance."""
    exp = _expect(expected_spec)
    act = actual.toArray() if hasattr(actual, "toArray") else np.asarray(actual)
    assert list(act.shape) == list(exp.shape), f"shape {list(act.shape)} != {list(exp.shape)}"
    diff = np.abs(exp.astype(np.float64) - act.astype(np.float64))
    assert np.all(diff <= tol + 1e-12), f"expected {exp.tolist()} but was {act.tolist()}"


def run_case(ops, case):
    g, tol = case["graph"], case["tol"]
    if g == "plus":
        res = _t(ops, case["a"]) + _t(ops, case["b"])
        assert_tensor_equals(case["res"], res, tol)
    elif g in ("mean((a-b) pow 2)", "sum((a+b) pow 2)", "sum(a-b)", "sum(a*b)", "sum(a/b)", "sum(a pow b)"):
        a, b = _t(ops, case["a"], True), _t(ops, case["b"], True)
        res = {"mean((a-b) pow 2)": lambda: ((a - b).pow(2.0)).mean(),
               "sum((a+b) pow 2)": lambda: ((a + b).pow(2.0)).sum(),
               "sum(a-b)": lambda: (a - b).sum(),
               "sum(a*b)": lambda: (a * b).sum(),
               "sum(a/b)": lambda: (a / b).sum(),
               "sum(a pow b)": lambda: a.pow(b).sum()}[g]()
        assert_tensor_equals(case["res"], res, tol)
        res.backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
        assert_tensor_equals(case["grad_b"], b.grad(), tol)
    elif g == "sum(max(a, axis=-1))":
        a = _t(ops, case["a"], True)
        m = a.max(axis=-1)
        assert_tensor_equals(case["res"], m, tol)
        m.sum().backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g in ("a+c ; c+a", "a-c ; c-a", "a*c ; c*a", "a/c ; c/a"):
        a, c = _t(ops, case["a"], True), case["c"]
        tc = {"a+c ; c+a": lambda: a + c, "a-c ; c-a": lambda: a - c, "a*c ; c*a": lambda: a * c, "a/c ; c/a": lambda: a / c}[g]()
        ct = {"a+c ; c+a": lambda: c + a, "a-c ; c-a": lambda: c - a, "a*c ; c*a": lambda: c * a, "a/c ; c/a": lambda: c / a}[g]()
        assert_tensor_equals(case["res_tc"], tc, tol)
        assert_tensor_equals(case["res_ct"], ct, tol)
        tc.sum().backward()
        assert_tensor_equals(case["grad_tc"], a.grad(), tol)
        a.zeroGrad()
        ct.sum().backward()
        assert_tensor_equals(case["grad_ct"], a.grad(), tol)
    elif g == "sum(c pow a)":
        a = _t(ops, case["a"], True)
        res = case["c"] ** a
        assert_tensor_equals(case["res"], res, 1e-6)
        res.sum().backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "agg":
        a = _t(ops, case["a"], True)
        res = getattr(a, case["op"])(axis=case["axis"], keepDimensions=case["keep"])
        assert_tensor_equals(case["res"], res, tol)
        res.backward(_t(ops, case["seed"]))
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "agg_sum":
        a = _t(ops, case["a"], True)
        res = getattr(a, case["op"])(axis=case["axis"], keepDimensions=case["keep"])
        assert_tensor_equals(case["res"], res, tol)
        res.sum().backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "arg":
        a = _t(ops, case["a"])
        res = getattr(a, case["op"])(axis=case["axis"], keepDimensions=case["keep"])
        assert_tensor_equals(case["res"], res, tol)
    elif g in ("unary_mean", "unary_sum"):
        a = _t(ops, case["a"], True)
        res = a.clamp(case["min"], case["max"]) if case["op"] == "clamp" else getattr(a, case["op"])()
        assert_tensor_equals(case["res"], res, tol)
        (res.mean() if g == "unary_mean" else res.sum()).backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "sum(expand(a))":
        a = _t(ops, case["a"], True)
        a.expand(*case["expand"]).sum().backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "long_graph":
        ones = {"shape": [5, 5], "data": [1.0] * 25}
        t1, t2 = _t(ops, ones, True), _t(ops, ones, True)
        a, b, c = t1 + 2.0, t2 + 2.0, t1 + 2.0
        add2 = (a + b) + c
        for _ in range(4):
            a, b, c = a * 2.0, b * 2.0, c * 2.0
        out = add2 + ((a + b) + c)
        out.backward(_t(ops, ones))
        assert_tensor_equals(case["grad_a"], t1.grad(), tol)
        assert_tensor_equals(case["grad_b"], t2.grad(), tol)
    elif g in ("unary_sum_after_set", "unary_chain_sum"):
        if g == "unary_sum_after_set":                     # elementwiseTestTensor().noGrad(); t1[1, 1] = -0.4f; asVariable
            a = _t(ops, case["a"])
            a[tuple(case["set_index"])] = case["set_value"]
            a = a.asVariable(requiresGrad=True)
            res = getattr(a, case["op"])()
        else:
            a = _t(ops, case["a"], True)
            res = a
            for op in case["ops"]:
                res = getattr(res, op)()
        assert_tensor_equals(case["res"], res, tol)
        res.sum().backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "set_element_from_tensor":
        t1, t2 = _t(ops, case["t1"], True), _t(ops, case["t2"], True)
        t2[1, 1] = t1[1].pow(2.0)
        t2.sum().backward()
        t1.sum().backward()
        assert_tensor_equals(case["res_t2"], t2, tol)
        assert_tensor_equals(case["grad_t1"], t1.grad(), tol)
    elif g == "set_element_range_from_tensor":
        t1 = AG.tensorOf(ops, [0.1]).expand(3, 3).asVariable(requiresGrad=True)
        t2 = AG.tensorOf(ops, [1.0]).expand(3, 3, 3).asVariable(requiresGrad=True)
        t2[(1, 1), None, (1, -1)] = t1[None, (1, -1)].pow(2.0).unsqueeze(0)
        t2.sum().backward()
        t1.sum().backward()
        assert_tensor_equals(case["res_t2"], t2, tol)
        assert_tensor_equals(case["grad_t1"], t1.grad(), tol)
    elif g == "set_constant":
        t1 = AG.tensorOf(ops, [0.1]).expand(2, 4).asVariable(requiresGrad=True)
        index = tuple(tuple(i) if isinstance(i, list) else i for i in case["index"])
        t1[index] = case["value"]
        assert_tensor_equals(case["res"], t1, tol)
        t1.sum().backward()
        assert_tensor_equals(case["res"], t1, tol)
        assert_tensor_equals(case["grad"], t1.grad(), tol)
    elif g == "transpose":
        a = _t(ops, case["a"], True)
        res = a.transpose(0, 1)
        assert_tensor_equals(case["res"], res, tol)
        res.backward(_t(ops, case["seed"]))
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "permute":
        a = _t(ops, case["a"], True)
        res = a.permute(*case["axes"])
        assert_tensor_equals(case["res"], res, tol)
        res.pow(2.0).sum().backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "concat":
        t1 = AG.tensorOf(ops, [1.0, 2.0, 3.0]).expand(2, 3).asVariable(requiresGrad=True)
        t2 = AG.tensorOf(ops, [4.0, 5.0, 6.0]).expand(1, 3).asVariable(requiresGrad=True)
        t3 = AG.tensorOf(ops, [7.0, 8.0, 9.0]).expand(1, 3).asVariable(requiresGrad=True)
        res = AG.concat([t1, t2, t3])
        assert_tensor_equals(case["res"], res, tol)
        res.pow(2.0).sum().backward()
        for t, key in ((t1, "grad_t1"), (t2, "grad_t2"), (t3, "grad_t3")):
            assert_tensor_equals(case[key], t.grad(), tol)
    elif g == "gather":
        a = _t(ops, case["a"], True)
        res = a.gather(case["axis"], _t(ops, case["index"]))
        assert_tensor_equals(case["res"], res, tol)
        res.sum().backward()
        assert_tensor_equals(case["grad_a"], a.grad(), tol)
    elif g == "scatter":
        t1 = AG.tensorOf(ops, np.arange(1, 11, dtype=np.float32), [2, 5])          # Tensor.arrange(11f, start = 1f).reshape(2, 5)
        zeros = lambda: AG.tensorOf(ops, np.zeros(15, dtype=np.float32), [3, 5])
        assert_tensor_equals(case["res1"], zeros().scatter(0, _t(ops, case["index1"]), t1), tol)
        assert_tensor_equals(case["res2"], zeros().scatter(1, _t(ops, case["index2"]), t1), tol)
    elif g == "scatter_with_grads":
        t1 = AG.tensorOf(ops, np.arange(1, 11, dtype=np.float32), [2, 5], requiresGrad=True)
        target = AG.tensorOf(ops, np.zeros(15, dtype=np.float32), [3, 5], requiresGrad=True)
        res = (target + 1.0).scatter(1, _t(ops, case["index"]), t1).pow(2.0)
        assert_tensor_equals(case["res"], res, tol)
        res.sum().backward()
        assert_tensor_equals(case["grad_t1"], t1.grad(), tol)
        assert_tensor_equals(case["grad_target"], target.grad(), tol)
    elif g == "index_select":
        t = AG.tensorOf(ops, np.arange(27, dtype=np.float32), [3, 3, 3], requiresGrad=True)
        res = t.indexSelect(case["axis"], _t(ops, case["index"]))
        assert_tensor_equals(case["res"], res, tol)
        res.sum().backward()
        assert_tensor_equals(case["grad"], t.grad(), tol)
    elif g == "fill_partially":
        t1 = AG.tensorOf(ops, np.ones(6, dtype=np.float32), [2, 3])
        t1.getRawValue().timesAssign(2.0)                                           # t1 *= 2f on a no-grad tensor
        t1[(0, 0), (1, 2)] = 0.0
        assert_tensor_equals(case["res"], t1, tol)
    else:
        raise AssertionError(f"unknown graph {g}")


def softmax_cross_entropy_property(ops, rows=256, classes=2048, seed=77, tol=1e-6):
    """should_calculate_softmax_cross_entropy_from_logits (kten-testing/.../TensorTestsBase.kt:2204-2224):
    the fused function node and the same loss spelled with one-hot targets agree in value and in
    gradient within assertTensorEquals' default tolerance.  The reference draws the logits and the
    targets from an unseeded generator; here they are seeded (standard-normal-range logits, uniform
    integer targets).  Returns (loss, gradient, logits, targets) as arrays for further checks."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1.0, 1.0, (rows, classes)).astype(np.float32)
    t = rng.integers(0, classes, rows).astype(np.float32)
    tensor = AG.tensorOf(ops, x, requiresGrad=True)
    tensor2 = tensor.copy().asVariable(requiresGrad=True)
    targets = AG.tensorOf(ops, t)
    one_hot = AG.oneHot(ops, targets, classes)

    res = tensor.softmaxCrossEntropy(targets)
    res.backward()

    exp_val = (tensor2 - tensor2.max(-1, keepDimensions=True)).exp()
    softmax = exp_val / exp_val.sum(-1, keepDimensions=True)
    eps = ops.epsilon
    softmax_norm = (softmax / softmax.sum(-1, keepDimensions=True)).clamp(eps, 1.0 - eps)
    res2 = (-(one_hot * softmax_norm.log()).sum(-1)).mean()
    res2.backward()

    got, want = res.toArray(), res2.toArray()
    assert got.shape == want.shape == (1,)
    assert abs(float(got[0]) - float(want[0])) <= tol, (got, want)
    g1, g2 = tensor.grad().toArray(), tensor2.grad().toArray()
    assert g1.shape == g2.shape == (rows, classes)
    assert float(np.abs(g1.astype(np.float64) - g2.astype(np.float64)).max()) <= tol
    return got, g1, x, t


def _close(a, b, tol):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    assert float(np.abs(a - b).max(initial=0.0)) <= tol, float(np.abs(a - b).max())


def batch_norm_training_property(ops, with_affine=True, seed=5, tol=1e-4):
    """should_calculate_batch_norm_for_specified_axis_in_train_mode and ..._in_training_mode_without_gamma_and_beta
    (kten-testing/.../TensorTestsBase.kt:2015-2064, 2099-2131): batchNorm along axis 1 of a [10, 3, 4, 5] tensor against
    the same normalisation spelled with mean / variance tensors -- output (the reference allows 0.02 / 0.01 here: the
    spelled form divides by the unbiased variance), running statistics, and the gradients of input, gamma and beta.
    The reference draws its tensors from an unseeded generator; here they are seeded.  Returns the arrays."""
    rng = np.random.default_rng(seed)
    rnd = lambda *shape: rng.uniform(0.0, 1.0, shape).astype(np.float32)
    axis, momentum, epsilon = 1, 0.1, 1e-3
    tensor = AG.tensorOf(ops, rnd(10, 3, 4, 5), requiresGrad=True)
    gamma = AG.tensorOf(ops, rnd(1, 3, 1, 1), requiresGrad=True) if with_affine else None
    beta = AG.tensorOf(ops, rnd(1, 3, 1, 1), requiresGrad=True) if with_affine else None
    running_mean_base, running_var_base = AG.tensorOf(ops, rnd(1, 3, 1, 1)), AG.tensorOf(ops, rnd(1, 3, 1, 1))

    t = tensor.permute(1, 0, 2, 3).view(3, -1)
    m, v = t.meanVariance(1)
    mean, variance = m.view(1, 3, 1, 1), v.view(1, 3, 1, 1)
    running_mean = (mean.noGrad() * momentum) + running_mean_base * (1.0 - momentum)
    running_var = (variance.noGrad() * momentum) + running_var_base * (1.0 - momentum)
    result = (tensor - mean) / (variance + epsilon).sqrt()
    if with_affine:
        result = result * gamma + beta
    result.sum().backward()
    want = {"out": result.toArray(), "gx": tensor.grad().toArray(), "rm": running_mean.toArray().reshape(3), "rv": running_var.toArray().reshape(3)}
    if with_affine:
        want["gg"], want["gb"] = gamma.grad().toArray(), beta.grad().toArray()
    for var in (tensor, gamma, beta):
        if var is not None:
            var.zeroGrad()

    running_mean2, running_var2 = running_mean_base.reshape(3), running_var_base.reshape(3)
    result2 = tensor.batchNorm(axis, running_mean2, running_var2, True, momentum, epsilon,
                               gamma.view(3) if with_affine else None, beta.view(3) if with_affine else None)
    result2.sum().backward()
    got = {"out": result2.toArray(), "gx": tensor.grad().toArray(), "rm": running_mean2.toArray(), "rv": running_var2.toArray()}
    if with_affine:
        got["gg"], got["gb"] = gamma.grad().toArray(), beta.grad().toArray()
    _close(got["out"], want["out"], 0.02 if with_affine else 0.01)
    for k in ("rm", "rv", "gx") + (("gg", "gb") if with_affine else ()):
        _close(got[k], want[k], tol)
    return got


def batch_norm_inference_property(ops, with_affine=True, seed=6, tol=1e-6):
    """should_calculate_batch_norm_for_specified_axis_in_inference_mode and ..._without_gamma_and_beta
    (TensorTestsBase.kt:2066-2090, 2133-2150): axis 2 of [10, 3, 4, 5], running statistics given."""
    rng = np.random.default_rng(seed)
    rnd = lambda *shape: rng.uniform(0.0, 1.0, shape).astype(np.float32)
    tensor = AG.tensorOf(ops, rnd(10, 3, 4, 5))
    gamma = AG.tensorOf(ops, rnd(1, 1, 4, 1)) if with_affine else None
    beta = AG.tensorOf(ops, rnd(1, 1, 4, 1)) if with_affine else None
    running_mean, running_var = AG.tensorOf(ops, rnd(1, 1, 4, 1)), AG.tensorOf(ops, rnd(1, 1, 4, 1))
    result = (tensor - running_mean) / (running_var + 1e-3).sqrt()
    if with_affine:
        result = result * gamma + beta
    result2 = tensor.batchNorm(2, running_mean.reshape(4), running_var.reshape(4), False, 0.1, 1e-3,
                               gamma.view(4) if with_affine else None, beta.view(4) if with_affine else None)
    got, want = result2.toArray(), result.toArray()
    _close(got, want, tol)
    return got


def upsample_nearest_property(ops, seed=7, tol=4e-6):        # block sums reach 24: two float roundings against one are 2 ulp = 3.8e-6
    """should_calculate_upsample_nearest_with_grads (TensorTestsBase.kt:2152-2180): upsample2d of [5, 3, 4, 5] by 3
    against view / expand / view, values and the gradients of sum(exp(.))."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(0.0, 1.0, (5, 3, 4, 5)).astype(np.float32)
    scale = 3
    tensor = AG.tensorOf(ops, x, requiresGrad=True)
    spelled = tensor.view(5, 3, 4, 1, 5, 1).expand(5, 3, 4, scale, 5, scale).view(5, 3, scale * 4, scale * 5)
    want_out = spelled.noGrad().toArray()
    spelled.exp().sum().backward()
    want_grad = tensor.grad().toArray()
    tensor.zeroGrad()
    ups = tensor.upsample2d(scale)
    got_out = ups.noGrad().toArray()
    ups.exp().sum().backward()
    got_grad = tensor.grad().toArray()
    assert np.array_equal(got_out, want_out)
    _close(got_grad, want_grad, tol)
    return got_out, got_grad


def max_pooling_1d_golden(ops):
    """should_calculate_max_pooling_for_1d_cases (kten-testing/.../nn/PoolingTestsBase.kt:13-42) on the reference's own
    fixture (tests/golden/maxpool1d_k3_s2_p1_d2_on_2x3x10_ceil.json, made from its XML): result, sum of the result and the
    input's gradient within the test's 1e-4."""
    with open(os.path.join(HERE, "golden", "maxpool1d_k3_s2_p1_d2_on_2x3x10_ceil.json")) as fh:
        case = json.load(fh)
    t1 = AG.tensorOf(ops, np.array(case["t1"], np.float32), requiresGrad=True)
    o = case["op"]
    res = t1.maxPooling1d(kernel=o["kernel"], stride=o["stride"], padding=o["padding"], dilation=o["dilation"], useCeil=o["useCeil"])
    total = res.sum()
    total.backward()
    got = res.toArray(), total.toArray(), t1.grad().toArray()
    _close(got[0], np.array(case["res"], np.float32), case["tol"])
    _close(got[1], np.array(case["sumRes"], np.float32), case["tol"])
    _close(got[2], np.array(case["t1Grad"], np.float32), case["tol"])
    return got
