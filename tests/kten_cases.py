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
    else:
        raise AssertionError(f"unknown graph {g}")
