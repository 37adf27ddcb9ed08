"""Writes tests/golden/maxpool1d_k3_s2_p1_d2_on_2x3x10_ceil.json from the reference's own fixture for its pooling test
(kten-testing/src/main/resources/maxpool1d_k3_s2_p1_d2_on_2x3x10_ceil.xml, used by PoolingTestsBase.kt:13-18): the input,
the pooled result, its sum and the input's gradient, as that file gives them.

    python tests/golden/make_pooling_golden.py <path of the kten checkout>

The reference checkout is only needed to (re)generate the file; the tests read the committed JSON.
"""
import json
import os
import re
import sys


def main():
    root = sys.argv[1]
    name = "maxpool1d_k3_s2_p1_d2_on_2x3x10_ceil"
    text = open(os.path.join(root, "kten-testing", "src", "main", "resources", name + ".xml")).read()
    out = {"_about": "Fixture of the reference's pooling test (PoolingTestsBase.kt:13-18, poolingTestCase :20-42): "
                     "maxPooling1d(kernel = 3, stride = 2, padding = 1, dilation = 2, useCeil = true) on t1 [2, 3, 10]; res, sumRes = sum(res) "
                     "and t1Grad = d sumRes / d t1, each compared with tolerance 1e-4 there.",
           "op": {"kernel": 3, "stride": 2, "padding": 1, "dilation": 2, "useCeil": True}, "tol": 1e-4}
    for m in re.finditer(r'<tensor name="(\w+)">\s*(\{.*?\})\s*</tensor>', text, re.S):
        data = json.loads(re.sub(r"(\d)\.(?=[,\]\s])", r"\1.0", m.group(2)))["data"]      # "0." -> "0.0"
        out[m.group(1)] = data
    assert set(out) >= {"t1", "res", "sumRes", "t1Grad"}
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, name + ".json"), "w") as fh:
        json.dump(out, fh, indent=1)
    print("wrote", name + ".json")


if __name__ == "__main__":
    main()
