"""The expression recorder behind `ktc_lazy_*` (kten_b200/csrc/ktc_lazy.cpp) without a device: the
recorder is compiled alone and drives the stand-in library (tests/fake_lib.py), whose ktc_expr_eval is
a numpy interpreter of the program encoding and keeps every program it is handed.  Results must equal
the direct numpy evaluation of the same expressions; the programs show register reuse, shared
sub-expressions, broadcast markers, side outputs and what happens at the limits that make the kernel
decline."""
import numpy as np

from kten_b200 import _lib as L
from tests import fake_lib


def ops_with(*arrays):
    ops = fake_lib.make_ops()
    ops.lazy = True
    return ops, [ops.createRaw(list(a.shape), a) for a in arrays]


def opcodes(program):
    return [w & 0xFF for w in program["code"]]


def rnd(shape, seed):
    return np.random.default_rng(seed).uniform(0.5, 2.0, shape).astype(np.float32)


def test_program_equals_direct_evaluation():
    X, W, B = rnd([6, 8], 1), rnd([1, 8], 2), rnd([8], 3)
    ops, (x, w, b) = ops_with(X, W, B)
    z = x.times(w).plus(b)
    e = z.exp()
    out = e.pow(2.0).minus(z.div(4.0))                       # z is used twice
    cl = out.clamp(0.0, 50.0)
    got = cl.toArray()
    zz = (X * W).astype(np.float32) + B
    ee = np.exp(zz.astype(np.float64)).astype(np.float32)
    want = np.clip((ee * ee).astype(np.float32) - (zz / np.float32(4.0)).astype(np.float32), 0.0, 50.0)
    assert np.array_equal(got, want)
    prog = ops.lib.programs[-1]
    assert ops.lib.expr_calls == 1 and ops.lib.calls == ["expr_eval"]
    assert opcodes(prog).count(L.X_LOAD) == 3                                      # every leaf is loaded once
    assert prog["leaf_shapes"] == [[6, 8], [1, 8], [1, 8]]
    assert prog["n_stores"] == 2                                                   # cl, and e on the side (a transcendental a tensor still waits for)
    assert np.array_equal(e.toArray(), ee) and ops.lib.expr_calls == 1             # ... so reading e costs nothing
    assert np.array_equal(z.toArray(), zz) and ops.lib.expr_calls == 2             # z was cheap: recomputed on demand


def test_broadcast_markers_cost_nothing():
    G, X = rnd([1], 5), rnd([4, 8], 6)
    ops, (g, x) = ops_with(G, X)
    xp = x.unaryMinus()
    alias = xp.copy()                                                              # a deep copy that is not made yet
    prod = g.broadcastTo([4, 8]).times(alias)
    assert np.array_equal(prod.toArray(), (G[0] * -X).astype(np.float32))
    assert opcodes(ops.lib.programs[-1]) == [L.X_LOAD, L.X_LOAD, L.X_NEG, L.X_MUL, L.X_STORE]
    assert alias.isDeferred and np.array_equal(alias.toArray(), -X)
    assert alias.storeReference != xp.storeReference                               # storage of its own, as a deep copy has


def test_registers_are_reused_and_limits_fall_back_to_separate_calls():
    X = rnd([16], 10)
    ops, (x,) = ops_with(X)
    cur, want = x, X.copy()
    for i in range(12):                                                             # a long chain needs two registers
        cur, want = cur.plus(float(i)), (want + np.float32(i)).astype(np.float32)
    assert np.array_equal(cur.toArray(), want) and ops.lib.expr_calls == 1 and ops.unfusedEvaluations == 0
    for _ in range(8):                                                              # 12 + 8 constants > 16 immediates
        cur, want = cur.plus(0.5), (want + np.float32(0.5)).astype(np.float32)
    assert np.array_equal(cur.toArray(), want)
    many, wantm = x, X.copy()
    others = [rnd([16], 20 + h) for h in range(9)]
    for o in others:                                                                # 10 distinct leaves > 8
        many, wantm = many.times(ops.createRaw([16], o)), (wantm * o).astype(np.float32)
    before = ops.unfusedEvaluations
    assert np.array_equal(many.toArray(), wantm) and ops.unfusedEvaluations > before

    def tree(depth, base):                                                          # needs more live values than there are registers
        if depth == 0:
            return x.plus(float(base)), (X + np.float32(base)).astype(np.float32)
        (a, wa), (b, wb) = tree(depth - 1, base), tree(depth - 1, base + (1 << depth))
        return a.times(b), (wa * wb).astype(np.float32)
    t, wt = tree(4, 0)
    before = ops.unfusedEvaluations
    assert np.array_equal(t.toArray(), wt) and ops.unfusedEvaluations > before


def test_side_outputs_only_for_values_a_tensor_still_waits_for():
    X = rnd([8, 8], 30)
    ss = np.exp((X + np.float32(1.0)).astype(np.float64)).astype(np.float32)
    # recompute rule alone: a value is recomputed `recomputeLimit` times, then stored if its tensor is still alive
    ops, (x,) = ops_with(X)
    ops.storeCost, ops.recomputeLimit = 0, 1
    z = x.plus(1.0)
    s = z.exp()
    assert np.array_equal(s.times(s).toArray(), (ss * ss).astype(np.float32))
    assert ops.lib.programs[-1]["n_stores"] == 1                                   # first evaluation: nothing on the side
    assert np.array_equal(s.plus(s).toArray(), (ss + ss).astype(np.float32))
    assert ops.lib.programs[-1]["n_stores"] == 2                                   # s is stored; z below it is not
    n = ops.lib.expr_calls
    assert np.array_equal(s.toArray(), ss) and ops.lib.expr_calls == n
    assert np.array_equal(z.toArray(), X + np.float32(1.0)) and ops.lib.expr_calls == n + 1
    # a higher limit: not yet
    ops, (x,) = ops_with(X)
    ops.storeCost, ops.recomputeLimit = 0, 2
    z = x.plus(1.0); s = z.exp()
    s.times(s).toArray(); s.plus(s).toArray()
    assert [p["n_stores"] for p in ops.lib.programs] == [1, 1]
    # the tensor moved on: no side output for it, but the value below it, now reachable, is a candidate
    ops, (x,) = ops_with(X)
    ops.storeCost, ops.recomputeLimit = 0, 1
    z = x.plus(1.0); s = z.exp()
    s.times(s).toArray()
    top = s.plus(s)
    s.release()
    assert np.array_equal(top.toArray(), (ss + ss).astype(np.float32)) and ops.lib.programs[-1]["n_stores"] == 2
    n = ops.lib.expr_calls
    assert np.array_equal(z.toArray(), X + np.float32(1.0)) and ops.lib.expr_calls == n        # z was the side output
    # cost rule: a value behind a transcendental is stored the first time, a cheap one is not
    ops, (x,) = ops_with(X)
    ops.storeCost, ops.recomputeLimit = 8, 2
    z = x.plus(1.0); s = z.exp()
    s.times(s).toArray()
    assert ops.lib.programs[-1]["n_stores"] == 2
    ops, (x,) = ops_with(X)
    z = x.plus(1.0); s = z.exp()
    top = s.times(s)
    s.release()
    top.toArray()
    assert ops.lib.programs[-1]["n_stores"] == 1                                   # z alone is one addition


def test_a_stored_value_replaces_its_operands_and_references_are_returned():
    X = rnd([8], 40)
    ops, (x,) = ops_with(X)
    base = ops.lib.live_buffers()
    mid = x.exp()
    top = mid.plus(1.0)
    mm = np.exp(X.astype(np.float64)).astype(np.float32)
    assert np.array_equal(mid.toArray(), mm)
    assert np.array_equal(top.toArray(), mm + np.float32(1.0))
    assert ops.lib.programs[-1]["leaves"] == [mid.storeReference]                  # x is no longer read
    for t in (mid, top):
        t.release()
    assert ops.lib.live_buffers() == base
    x.release()
    st = ops._recorder.stats()
    assert ops.lib.live_buffers() == base - 1 and st["live_nodes"] == 0 and st["live_cells"] == 0


def test_program_cache_tells_one_buffer_read_twice_from_two_buffers():
    """A program compiled for a DAG that reads ONE buffer through two operands of different rank must not be
    reused for a DAG of the same structure that reads two different buffers."""
    X, Bv, Cv = rnd([3, 4], 50), rnd([4], 51), rnd([1, 4], 52)
    ops, (x, b, c) = ops_with(X, Bv, Cv)
    first = x.plus(b).times(b.view([1, 4])).toArray()
    second = x.plus(b).times(c).toArray()
    assert np.array_equal(first, ((X + Bv).astype(np.float32) * Bv).astype(np.float32))
    assert np.array_equal(second, ((X + Bv).astype(np.float32) * Cv).astype(np.float32))
    assert len(ops.lib.programs[0]["leaves"]) == 2 and len(ops.lib.programs[1]["leaves"]) == 3
    st = ops._recorder.stats()
    assert st["compiled"] == 2 and st["cache_hits"] == 0
    third = x.plus(b).times(c).toArray()                                           # the same structure again: re-bound, not recompiled
    assert np.array_equal(third, second) and ops._recorder.stats()["cache_hits"] == 1


def test_sqrt_rsqrt_and_abs_are_expression_instructions():
    """The step of an optimiser, m / (sqrt(v) + eps), and a normalisation, x * rsqrt(abs(x) + 1), stay one program each
    and give the bits of the separate calls."""
    M, V = rnd([8, 16], 70), np.abs(rnd([8, 16], 71)) + np.float32(0.01)
    ops, (m, v) = ops_with(M, V)
    upd = m.div(v.sqrt().plus(1e-8))
    norm = m.times(m.abs().plus(1.0).rsqrt())
    want_upd = (M / (np.sqrt(V, dtype=np.float32) + np.float32(1e-8))).astype(np.float32)
    want_norm = (M * (np.float32(1.0) / np.sqrt(np.abs(M) + np.float32(1.0), dtype=np.float32))).astype(np.float32)
    n0 = ops.lib.expr_calls
    assert np.array_equal(upd.toArray(), want_upd) and np.array_equal(norm.toArray(), want_norm)
    assert ops.lib.expr_calls == n0 + 2 and ops.unfusedEvaluations == 0
    assert L.X_SQRT in opcodes(ops.lib.programs[-2]) and {L.X_ABS, L.X_RSQRT} <= set(opcodes(ops.lib.programs[-1]))
