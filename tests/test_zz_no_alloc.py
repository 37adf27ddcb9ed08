"""ktc_reduce_all_noalloc: the full sum / mean for callers that may not allocate
(their device memory belongs to another allocator, or they cannot take the
device-wide stall of cudaMalloc in the middle of a step).  It keeps its per-CTA
partials in a fixed array inside the library instead of pool memory.

Checked here through the C ABI against ktc_reduce_all, the pooled entry point it
mirrors, on two calls in a row (the array is shared by all calls and is not
cleared between them, so the second call runs on the first one's leftovers).
This file sorts last on purpose: a run that stops at the first failure has
already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

from kten_b200 import _lib as L
from kten_b200 import datagen as D

pytestmark = pytest.mark.gpu

RED_RTOL = 1e-5          # same bar as the other reduction tests: relative to sum(|x|)


def _alloc(lib, n):
    h = C.c_uint64(0)
    L.check(lib.ktc_alloc(0, n, C.byref(h)))
    return h.value


def _upload(lib, h, x):
    L.check(lib.ktc_h2d(h, 0, x.ctypes.data_as(C.c_void_p), x.size, 1))


def _read1(lib, h):
    out = np.zeros(1, dtype=np.float32)
    L.check(lib.ktc_d2h(out.ctypes.data_as(C.c_void_p), h, 0, 1, 1))
    return out[0]


def test_noalloc_sum_matches_pooled_entry_point_twice_in_a_row():
    lib = L.load()
    n_dev = C.c_int(0)
    L.check(lib.ktc_init(C.byref(n_dev)))
    sizes = [(1 << 22) + 3, 1000]                 # a long input first, then a short one over its leftovers
    bufs = []
    try:
        for call, n in enumerate(sizes):
            exact = D.normal(n, 90 + call, 0.0, 1.0, quantum=16.0)     # sums are exact in any order
            rough = D.uniform(n, 95 + call, 0.0, 1.0)                   # all positive, rounding matters
            for x, bit_exact in ((exact, True), (rough, False)):
                h_in, h_ref, h_new = _alloc(lib, n), _alloc(lib, 1), _alloc(lib, 1)
                bufs += [h_in, h_ref, h_new]
                _upload(lib, h_in, x)
                for op in (L.SUM, L.MEAN):
                    L.check(lib.ktc_reduce_all(op, h_ref, h_in, n))
                    calls_before = C.c_int64(0)
                    L.check(lib.ktc_pool_stats(0, None, None, C.byref(calls_before), None))
                    L.check(lib.ktc_reduce_all_noalloc(op, h_new, h_in, n))
                    calls_after = C.c_int64(0)
                    L.check(lib.ktc_pool_stats(0, None, None, C.byref(calls_after), None))
                    assert calls_after.value == calls_before.value          # the pool was not touched
                    ref, new = _read1(lib, h_ref), _read1(lib, h_new)
                    if bit_exact:
                        assert ref.view(np.uint32) == new.view(np.uint32)
                    scale = float(np.abs(x.astype(np.float64)).sum()) / (n if op == L.MEAN else 1)
                    assert abs(float(ref) - float(new)) <= RED_RTOL * scale
                    want = x.astype(np.float64).sum() / (n if op == L.MEAN else 1)
                    assert abs(float(new) - want) <= RED_RTOL * scale
    finally:
        for h in bufs:
            lib.ktc_release(h)


def test_noalloc_rejects_what_it_was_not_built_for():
    lib = L.load()
    n_dev = C.c_int(0)
    L.check(lib.ktc_init(C.byref(n_dev)))
    h_in, h_out = _alloc(lib, 16), _alloc(lib, 1)
    try:
        assert lib.ktc_reduce_all_noalloc(L.SUM, h_out, h_in, L.NOALLOC_MAX_ELEMS + 1) == L.KTC_EINVAL
        assert b"exceed the limit" in lib.ktc_last_error()
        assert lib.ktc_reduce_all_noalloc(L.SUM, h_out, h_in, 17) == L.KTC_EINVAL        # more than the buffer holds
        assert lib.ktc_reduce_all_noalloc(L.MAX, h_out, h_in, 16) == L.KTC_EINVAL
        assert lib.ktc_reduce_all_noalloc(L.SUM, h_in, h_in, 16) == L.KTC_EINVAL          # out aliases in
        inside = C.c_uint64(0)
        L.check(lib.ktc_view(h_in, 5, 1, C.byref(inside)))                                # a view inside the input
        assert lib.ktc_reduce_all_noalloc(L.SUM, inside.value, h_in, 16) == L.KTC_EINVAL
        L.check(lib.ktc_reduce_all_noalloc(L.SUM, inside.value, h_in, 5))                  # behind the elements that are read: fine
        lib.ktc_release(inside.value)
        _upload(lib, h_in, np.arange(16, dtype=np.float32))
        L.check(lib.ktc_reduce_all_noalloc(L.MEAN, h_out, h_in, 16))
        assert _read1(lib, h_out) == np.float32(7.5)
        L.check(lib.ktc_reduce_all_noalloc(L.MEAN, h_out, h_in, 0))
        assert np.isnan(_read1(lib, h_out))
    finally:
        lib.ktc_release(h_in); lib.ktc_release(h_out)
