"""Accuracy of the table-driven exp / sigmoid / pow (kten_b200/csrc/ktc_fastmath_d.h), measured
on the host.  The header uses only IEEE float and double add / mul / fma, conversions and
integer operations, so the bits checked here are the bits the GPU produces
(tests/test_gpu_parity.py compares the two)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from oracle import oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "host_math", "fastmath_host.cpp")
SO = os.path.join(HERE, "host_math", "libfastmath_host.so")
HDR = os.path.join(HERE, "..", "kten_b200", "csrc", "ktc_fastmath_d.h")


def host_math_library():
    """Builds (when stale) and loads the host build of the header."""
    if not os.path.exists(SO) or os.path.getmtime(SO) < max(os.path.getmtime(SRC), os.path.getmtime(HDR)):
        flags = ["-O2", "-fopenmp", "-fPIC", "-shared", "-ffp-contract=off", "-std=c++17"]
        with open("/proc/cpuinfo") as fh:
            if " fma " in fh.read():
                flags.append("-mfma")            # std::fma as one instruction; the library routine gives the same bits
        subprocess.run(["g++", *flags, "-o", SO, SRC], check=True)
    lib = C.CDLL(SO)
    lib.kfh_sweep.restype = C.c_int64
    lib.kfh_sweep.argtypes = [C.c_int, C.c_uint32, C.POINTER(C.c_int64)]
    lib.kfh_div.restype = C.c_int64
    lib.kfh_div.argtypes = [C.c_int, C.c_int64]
    lib.kfh_div_pow2.restype = C.c_int64
    lib.kfh_div_pow2.argtypes = [C.c_int64]
    lib.kfh_div_accepts.restype = C.c_int
    lib.kfh_div_accepts.argtypes = [C.c_float, C.c_float]
    return lib


@pytest.fixture(scope="module")
def fm():
    return host_math_library()


def host_unary(lib, fn, x):
    out = np.empty_like(x)
    getattr(lib, fn)(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_int64(x.size))
    return out


def host_pow(lib, x, y):
    out, ok = np.empty_like(x), np.empty(x.size, dtype=np.uint8)
    lib.kfh_pow(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p),
                ok.ctypes.data_as(C.c_void_p), C.c_int64(x.size))
    return out, ok.astype(bool)


def test_exp_every_eleventh_float(fm):
    """Every 11th float bit pattern -- both signs, subnormals, arguments whose exp overflows or
    underflows, infinities, NaNs: at most 1 ulp from the narrowed double exp, and fewer than one
    argument in a million differs at all."""
    counts = (C.c_int64 * 4)()
    worst = fm.kfh_sweep(0, 11, counts)
    n = sum(counts)
    assert n > 390_000_000
    assert worst <= 1
    assert counts[1] <= n // 1_000_000


def test_sigmoid_every_eleventh_float(fm):
    """The composite 1f / (1f + (float)exp(-1f * x)) over every 11th float: at most 2 ulp from the
    reference's value, fewer than one argument in a million differs."""
    counts = (C.c_int64 * 4)()
    worst = fm.kfh_sweep(1, 11, counts)
    n = sum(counts)
    assert worst <= 2
    assert counts[1] + counts[2] <= n // 1_000_000 and counts[3] == 0


def test_forms_without_clamps_are_the_same_functions_inside_their_range(fm):
    """The vector kernels skip the clamps and the denominator test when all four arguments lie within +-80 (or are NaN):
    every 7th float of that range gives the bits of the full form."""
    for fn in (2, 3):                                   # sigmoid within +-80, exp within +-104
        counts = (C.c_int64 * 4)()
        worst = fm.kfh_sweep(fn, 7, counts)
        assert worst == 0 and counts[0] > 200_000_000 and counts[1] + counts[2] + counts[3] == 0


@pytest.mark.parametrize("domain", ["config2", "wide", "large_exponent", "huge_base", "near_one", "subnormal_result"])
def test_pow(fm, domain):
    rng = np.random.default_rng(len(domain) * 131)
    n = 4_000_000
    if domain == "config2":
        x, y = rng.uniform(0.1, 2.0, n), rng.uniform(0.1, 2.0, n)
    elif domain == "wide":
        x, y = np.exp(rng.uniform(np.log(1e-3), np.log(1e3), n)), rng.uniform(-8, 8, n)
    elif domain == "large_exponent":
        x, y = rng.uniform(0.5, 2.0, n), rng.uniform(-150, 150, n)
    elif domain == "huge_base":
        x, y = np.exp(rng.uniform(np.log(1e-30), np.log(1e30), n)), rng.uniform(-1.2, 1.2, n)
    elif domain == "near_one":
        x, y = 1.0 + rng.uniform(-1e-3, 1e-3, n), rng.uniform(-1e5, 1e5, n)
    else:
        x, y = rng.uniform(0.01, 0.5, n), rng.uniform(20, 60, n)      # results from 1e-30 down through the subnormals to 0
    x, y = x.astype(np.float32), y.astype(np.float32)
    got, ok = host_pow(fm, x, y)
    assert ok.mean() > 0.85
    want = O.binary_same(O.POW, x, y, tuned=True)
    d = O.ulp_distance(got[ok], want[ok])
    assert d.max() <= 1
    assert int((d > 0).sum()) <= n // 100_000


def test_pow_declines_special_operands_and_keeps_zero_exponents(fm):
    x = np.array([0.0, -1.0, np.inf, np.nan, 1e-40, 2.0, 2.0, 2.0, 1.0, 1.0, 3.0, 0.5, -0.0, -np.inf], dtype=np.float32)
    y = np.array([2.0, 2.0, 2.0, 2.0, 2.0, np.inf, np.nan, 200.0, np.nan, np.inf, -130.0, 170.0, 3.0, 3.0], dtype=np.float32)
    _, ok = host_pow(fm, x, y)
    assert not ok.any()
    x = np.array([2.0, 0.5, 1.0, 3.4e38, 1.2e-38], dtype=np.float32)
    got, ok = host_pow(fm, x, np.array([0.0, -0.0, 0.0, 0.0, -0.0], dtype=np.float32))
    assert ok.all() and np.all(got == 1.0)


def test_special_arguments_of_exp_and_sigmoid(fm):
    x = np.array([np.inf, -np.inf, np.nan, 88.7228394, 88.72284, 89.0, 1e30, -103.97, -103.98, -104.5, -1e30, 0.0, -0.0,
                  -88.5, -88.8, -87.0, -86.0, 17.0, 30.0, 31.0, 1e-45, -1e-45], dtype=np.float32)
    for fn, code in (("kfh_exp", O.EXP), ("kfh_sigmoid", O.SIGMOID)):
        got, want = host_unary(fm, fn, x), O.unary(code, x, tuned=True)
        assert np.array_equal(np.isnan(got), np.isnan(want)), fn
        keep = ~np.isnan(want)
        assert np.array_equal(got[keep].view(np.uint32), want[keep].view(np.uint32)), (fn, got, want)


def test_division_by_a_shared_divisor_is_the_ieee_quotient(fm):
    """q = x r, then q + (x - q b) r with r = RN(1 / b): the quotient of the broadcast division kernel.  Every
    dividend mantissa against 1024 divisors (those nearest to all-ones and to 1.0 among them), and 2^28 seeded
    pairs over the whole exponent window: not one bit differs from x / b."""
    assert fm.kfh_div(0, 1024) == 0
    assert fm.kfh_div(1, 1 << 28) == 0


def test_division_by_a_power_of_two_is_a_multiplication(fm):
    """x / 2^k == x * 2^-k bit for bit for every k in [-60, 60], both signs, over a million seeded dividends of any bit
    pattern each (zeros, subnormals, infinities; NaN stays NaN), and nothing else is taken for a power of two."""
    assert fm.kfh_div_pow2(1 << 20) == 0


def test_division_by_a_shared_divisor_declines_what_it_cannot_do(fm):
    inf, nan = float("inf"), float("nan")
    for x, b in ((0.0, 2.0), (-0.0, 2.0), (inf, 2.0), (nan, 2.0), (1e-30, 2.0), (1e30, 2.0), (1e-45, 3.0),
                 (1.0, 0.0), (1.0, inf), (1.0, nan), (1.0, 1e-30), (1.0, 1e30), (1.0, 1e-45), (3e38, 3.0)):
        assert fm.kfh_div_accepts(x, b) == 0, (x, b)
    for x, b in ((1.0, 3.0), (-7.5, 1e-18), (1.1e-19, -1e18), (1.8e19, 9e17)):
        assert fm.kfh_div_accepts(x, b) == 1, (x, b)


def test_tables_of_the_header_are_what_the_generator_prints():
    pytest.importorskip("mpmath")
    import sys
    gen = os.path.join(HERE, "..", "kten_b200", "csrc", "gen_fastmath_d_tables.py")
    r = subprocess.run([sys.executable, gen, "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
