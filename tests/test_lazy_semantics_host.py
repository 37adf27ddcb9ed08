"""The deferred-expression layer on a machine without a GPU: the host logic (storage cells, aliasing,
in-place rules, side outputs, splitting of programs the kernel declines, reference counting) driven
against a stand-in for the library (tests/fake_lib.py).  Every script runs call by call and deferred
on the same stand-in; the results must be bit-identical and no buffer may leak."""
import gc

import numpy as np
import pytest

from kten_b200 import datagen as D
from tests.fake_lib import make_ops
from tests.kten_cases import CASES, CASE_IDS, run_case


def same_bits(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def both(fn):
    out, stats = [], []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            res = fn(ops)
            out.append([r.toArray() for r in res])
        stats.append((ops.lib.live_buffers(), ops.lib.expr_calls, list(ops.lib.calls), ops.fusedEvaluations, ops.unfusedEvaluations))
    return out[0], out[1], stats


@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_reference_vectors_deferred_on_the_stand_in(case):
    live = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        try:
            with ops.garbageCollector():
                run_case(ops, case)
        except AttributeError as exc:
            if "FakeLib" in str(exc):
                pytest.skip(f"the stand-in does not provide this entry point: {exc}")
            raise
        gc.collect()
        live.append(ops.lib.live_buffers())
    assert live[1] <= live[0]            # what stays alive are the kept outputs of the graph, as in the eager run


def test_inplace_and_alias_rules():
    n = 256
    av, bv, cv = (D.uniform(n, 11, -1.0, 1.0, stream=s) for s in range(3))

    def script(o):
        a, b, c = o.createRaw([n], av), o.createRaw([n], bv), o.createRaw([n], cv)
        d = a.plus(b)                    # reads a ...
        a.plusAssign(c)                  # ... which then changes in place: d keeps the old value
        a.timesAssign(0.5)
        e = d.times(2.0)
        s = e.copy(shallow=True)         # alias of a pending value
        s.timesAssign(b)                 # visible through e
        s.plusAssign(1.0)
        deep = e.copy()                  # independent of later writes to e
        e.divAssign(4.0)
        f = o.createRaw([n], bv).minus(c)
        f.inplaceFill(7.0)               # overwrites a pending value
        g = d.exp()
        d.release()                      # released before its consumer is evaluated
        v = c.view([16, 16]).times(2.0)
        c.plusAssign(1.0)                # the view's consumer keeps the old contents
        w = a.pow(2.0).pow(1.0)
        t = b.copy(shallow=True)         # alias of a stored tensor
        t.timesAssign(3.0)               # visible through b
        return [a, e, s, deep, f, g, v, c, w, b, t]

    eager, lazy, stats = both(script)
    for k, (x, y) in enumerate(zip(eager, lazy)):
        assert same_bits(x, y), f"result {k}"
    assert np.array_equal(lazy[1], lazy[2]) and np.array_equal(lazy[9], lazy[10])
    assert stats[0][0] == 0 and stats[1][0] == 0                      # every buffer went back
    assert stats[1][1] > 0 and stats[0][1] == 0                       # the deferred run used fused programs, the eager run none


def test_chains_sums_and_side_outputs():
    rows, cols = 24, 16
    xv, wv = D.uniform(rows * cols, 3, -1.0, 1.0), D.uniform(cols, 3, 0.5, 1.5, stream=1)

    def script(o):
        x, w = o.createRaw([rows, cols], xv), o.createRaw([1, cols], wv)
        z = x.times(w).plus(0.25)
        s = z.sigmoid()
        loss = s.pow(2.0).sum()
        g = s.unaryMinus().plus(1.0).times(s)                         # (1 - s) s
        gw = g.times(x).sum(0, keepDimensions=True)
        gb = g.sum(0)
        m = z.mean()
        return [loss, gw, gb, m, s, z]

    eager, lazy, stats = both(script)
    for k in (4, 5):
        assert same_bits(eager[k], lazy[k])
    for k in (0, 1, 2, 3):                                            # fused sums: same values up to summation order
        assert np.allclose(eager[k], lazy[k], rtol=1e-6, atol=1e-6)
    calls = stats[1][2]
    assert calls.count("expr_eval") >= 1 and "unary" not in calls     # sigmoid ran inside a program, never as a separate call
    assert stats[1][0] == 0


def test_cheap_values_are_recomputed_heavy_ones_stored():
    ops = make_ops()
    ops.lazy = True
    ops.deferSums = False                                               # every sum below runs where it is written
    n = 64
    with ops.garbageCollector():
        x = ops.createRaw([n], D.uniform(n, 13, -2.0, 2.0))
        c = x.times(2.0).plus(1.0)
        c.plus(1.0).sum(); c.times(c).sum()
        assert c.isDeferred                                             # recomputed twice from x
        c.times(0.5).sum()
        assert not c.isDeferred                                         # the third use stored it
        s = x.sigmoid()
        s.times(s).sum()
        assert not s.isDeferred                                         # behind a transcendental: stored at once
    assert ops.lib.live_buffers() == 0


def test_programs_the_kernel_declines_are_split():
    n = 64
    vals = [D.uniform(n, 17, 0.5, 1.5, stream=s) for s in range(9)]

    def wide(o):
        ts = [o.createRaw([n], v) for v in vals]
        acc = ts[0]
        for t in ts[1:]:                                                # nine operands: more than one program loads
            acc = acc.times(t).plus(t)
        deep = ts[0]
        for i in range(40):                                             # longer than one program
            deep = deep.plus(float(i)).times(0.99)
        odd = o.createRaw([3, 5, 7], D.uniform(105, 18, 0.5, 1.5)).exp().times(2.0).plus(o.createRaw([7], vals[0][:7]))
        return [acc, deep, odd]                                         # innermost extent 7: the call declines it

    eager, lazy, stats = both(wide)
    for x, y in zip(eager, lazy):
        assert same_bits(x, y)
    assert stats[1][4] > 0 and stats[1][0] == 0


def test_sharded_graph_step_deferred_equals_call_by_call():
    """The config-5 autograd step through the stand-in: same loss and gradients in both execution modes; the deferred
    mode runs ONE pass with three sinks (loss, both broadcast gradients) whose second pass also performs the two
    in-place gradient accumulations, instead of two dozen calls -- three single-sink passes with ops.deferSums
    off --, nothing left allocated."""
    from kten_b200.sharded import ShardedSigmoidGraph
    rows, cols = 32, 16
    x, w, b = D.uniform(rows * cols, 0, -1.0, 1.0), D.normal(cols, 0, 0.0, 0.5, stream=1), D.uniform(cols, 0, -0.1, 0.1, stream=2)
    res = []
    for mode in (False, True, "sums at once"):
        ops = make_ops()
        ops.lazy = bool(mode)
        ops.deferSums = mode is True
        with ops.garbageCollector():
            g = ShardedSigmoidGraph(ops, ops.createRaw([rows, cols], x), ops.createRaw([1, cols], w), ops.createRaw([cols], b))
            for _ in range(2):
                n0 = len(ops.lib.calls)
                loss, gw, gb = g.step()
                vals = (loss.toArray().copy(), gw.toArray().copy(), gb.toArray().copy())
                g.release_step()
            res.append((vals, ops.lib.calls[n0:], ops.lib.multi_calls, ops.lib.programs[-1].get("folded_updates") if ops.lib.programs else None))
            for v in (g.x, g.w, g.b):
                v.getRawValue().release()
            g.w.gradient.release(); g.b.gradient.release()
        gc.collect()
        assert ops.lib.live_buffers() == 0
    (ve, ce, _, _), (vl, cl, multi, folded), (vs, cs, multi_off, _) = res[0], res[1], res[2]
    for a, c, d in zip(ve, vl, vs):
        assert np.allclose(a, c, rtol=1e-6, atol=1e-6) and np.allclose(a, d, rtol=1e-6, atol=1e-6)
    # sums that run where they are written: three passes with one sum each, and the two accumulations into the zeroed
    # (pending-constant) gradients as two small programs
    assert ce.count("expr_eval") == 0 and cs == ["expr_eval"] * 5 and multi_off == 0
    assert cl == ["expr_eval"] and multi == 2 and folded == 2, cl      # one pass per step (two steps), both `+=` inside it


def test_pending_sums_keep_the_semantics_of_sums_that_run_at_once():
    """ops.deferSums: a sum is computed when its value (or a buffer it updates) is first looked at, but must
    see the operands as they were where the sum was written."""
    rows, cols = 16, 8
    xv, yv = D.uniform(rows * cols, 21, -1.0, 1.0), D.uniform(rows * cols, 22, -1.0, 1.0)
    gv = D.uniform(cols, 23, -1.0, 1.0)

    def script(o):
        x, y = o.createRaw([rows, cols], xv), o.createRaw([rows, cols], yv)
        g1, g2 = o.createRaw([1, cols], gv), o.createRaw([cols], gv)
        d = x.minus(y)
        loss = d.pow(2.0).mean()                          # pending
        x.timesAssign(2.0)                                # overwrites an operand: the mean is of the old x
        g1.plusAssign(d.times(y).sum(0, keepDimensions=True))      # pending update of g1 (d already evaluated by the write above)
        g1.plusAssign(d.sum(0, keepDimensions=True))      # a second update of the same buffer, in order
        g2.plusAssign(d.times(0.5).sum(0))
        g2.timesAssign(3.0)                               # in-place write to a buffer with a pending update
        nested = d.minus(d.mean()).pow(2.0).sum()         # a sum over an expression that holds a pending sum
        spread = g2.broadcastTo([rows, cols]).plus(1.0).sum()
        odd = o.createRaw([3, 7], xv[:21]).times(2.0).sum()        # innermost extent 7: not fusable, reduced by the library call
        view = g1.view([cols])                            # shares g1's buffer
        return [loss, g1, g2, nested, spread, odd, view, x]

    eager, lazy, stats = both(script)
    for k, (a, c) in enumerate(zip(eager, lazy)):
        assert np.allclose(a, c, rtol=1e-6, atol=1e-6), f"result {k}: {a} != {c}"
    assert same_bits(eager[7], lazy[7]) and same_bits(lazy[1].reshape(-1), lazy[6])
    assert stats[1][0] == 0 and stats[0][0] == 0


def test_a_pending_sum_nobody_reads_is_never_computed():
    ops = make_ops()
    ops.lazy = True
    with ops.garbageCollector():
        x = ops.createRaw([16, 8], D.uniform(128, 24, -1.0, 1.0))
        ops.release(x.times(2.0).sum())                     # released before anyone looked at it
        kept = x.plus(1.0).sum(0)
        assert ops.lib.calls == []                          # nothing has run yet
        assert kept.toArray().shape == (8,)
        assert ops.lib.calls == ["expr_eval"] and ops.lib.multi_calls == 0     # only the sum that was read
    assert ops.lib.live_buffers() == 0


def test_last_axis_sums_wait_and_share_a_pass():
    """The two normalisations of a softmax (SoftmaxCrossEntropy.kt:40-52): the row sums are pending sums over the
    last axis, the second one waits for the first, and a full sum over the same expression joins the pass."""
    rows, cols = 12, 16
    xv = D.uniform(rows * cols, 31, -2.0, 2.0)

    def script(o):
        x = o.createRaw([rows, cols], xv)
        m = x.max(-1, keepDimensions=True)
        e = x.minus(m).exp()
        z = e.sum(-1, keepDimensions=True)
        total = e.sum()                                    # same iteration space: one pass with two sinks
        sm = e.div(z)
        z2 = sm.sum(-1)                                    # holds the pending z: waits for it
        norm = sm.div(z2.view([rows, 1])).clamp(1e-7, 1.0 - 1e-7).log()
        return [z, total, z2, norm, sm]

    eager, lazy, stats = both(script)
    for k, (a, c) in enumerate(zip(eager, lazy)):
        assert a.shape == c.shape and np.allclose(a, c, rtol=2e-6, atol=1e-6), f"result {k}"
    assert eager[0].shape == (rows, 1) and eager[2].shape == (rows,)
    assert stats[1][0] == 0
    calls = stats[1][2]
    assert "unary" not in calls and calls.count("reduce_axis") == 1          # only the row maximum ran as a reduction call


def test_gather_of_a_pending_expression_gathers_its_operands():
    """One pick per row from log(clamp(e / z)) (SoftmaxCrossEntropy.kt:50-53): the deferred mode gathers e and
    rebuilds the expression on [rows, 1]; same bits as evaluating everything and gathering then."""
    rows, cols = 16, 32
    xv = D.uniform(rows * cols, 41, 0.1, 2.0)
    zv = D.uniform(rows, 42, 1.0, 3.0)
    tv = np.floor(D.uniform(rows, 43, 0.0, cols - 0.01)).astype(np.float32)

    def script(o):
        x, z, t = o.createRaw([rows, cols], xv), o.createRaw([rows, 1], zv), o.createRaw([rows, 1], tv)
        full = x.exp().div(z).clamp(1e-7, 1.0).log()
        picked = full.gather(-1, t)
        dense = full.gather(-1, o.createRaw([rows, cols], np.tile(tv.reshape(rows, 1), (1, cols))))      # many picks: evaluated first
        return [picked, picked.unaryMinus().mean(), dense]

    eager, lazy, stats = both(script)
    for k, (a, c) in enumerate(zip(eager, lazy)):
        assert a.shape == c.shape
    assert same_bits(eager[0], lazy[0]) and same_bits(eager[2], lazy[2])
    assert np.allclose(eager[1], lazy[1], rtol=1e-6)
    assert stats[1][0] == 0 and stats[0][0] == 0
    assert stats[1][2].count("gather") == 2 and stats[0][2].count("gather") == 2


def test_softmax_cross_entropy_on_the_stand_in():
    """The reference's property test of SoftmaxCrossEntropy through the stand-in, call by call and deferred: the deferred
    run takes the row sums as pending last-axis sums, gathers the targets through the pending log-softmax expression
    (no full-size logarithm is ever computed) and leaves nothing allocated."""
    import gc
    from tests.kten_cases import softmax_cross_entropy_property
    res = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            loss, grad, _, _ = softmax_cross_entropy_property(ops, rows=16, classes=64)
            res.append((loss, grad, list(ops.lib.calls)))
        gc.collect()
    (le, ge, ce), (ll, gl, cl) = res
    assert abs(float(le[0]) - float(ll[0])) <= 1e-6 and np.abs(ge - gl).max() <= 1e-8
    # exp runs inside a program; what is left as separate calls are the operations on the picked [rows, 1] values, which
    # this stand-in (unlike the library, which collapses the trailing 1) declines to fuse
    assert len(cl) < len(ce) and cl.count("unary") < ce.count("unary") / 2


def test_inplace_chain_on_a_buffer_nobody_else_holds_waits():
    """`g += pending; g /= c; acc += g` (the backward of SoftmaxCrossEntropy.kt:74-77 and the accumulation into the
    Variable): with no second holder of g's or acc's buffer the three in-place calls become one program; a buffer that a
    view also holds is written in place at once, and the view sees it."""
    rows, cols = 8, 16
    xv, zv, av = D.uniform(rows * cols, 51, -1.0, 1.0), D.uniform(rows, 52, 1.0, 2.0), D.uniform(rows * cols, 53, -1.0, 1.0)

    def script(o):
        x, z = o.createRaw([rows, cols], xv), o.createRaw([rows, 1], zv)
        g = o.createRawFill([rows, cols], 0.0)
        g.inplaceScatter(-1, o.createRaw([rows, 1], np.arange(rows, dtype=np.float32)), -1.0)
        g.plusAssign(x.exp().div(z))
        g.divAssign(float(rows))
        acc = o.createRaw([rows, cols], av)
        acc.plusAssign(g)
        held = o.createRaw([rows, cols], av)
        view = held.view([cols, rows])                     # a second holder of the buffer
        held.plusAssign(x.exp().div(z))
        return [acc, g, held, view]

    eager, lazy, stats = both(script)
    for k, (a, c) in enumerate(zip(eager, lazy)):
        assert same_bits(a, c), f"result {k}"
    assert same_bits(lazy[2].reshape(-1), lazy[3].reshape(-1))
    assert stats[1][0] == 0 and stats[0][0] == 0
    calls = stats[1][2]
    # deferred: acc and g in one program each when they are read (g's is a side output or a second program), held at once
    assert calls.count("expr_eval") <= 3 and calls.count("binary") == 0 and calls.count("scalar") == 0


def test_updates_of_one_buffer_apply_in_the_order_they_were_written():
    """`t += s2; t += s1` with s1 created first: float addition does not commute with rounding, so the pending
    updates must be applied in the order of the calls, not in the order the sums came into being."""
    def script(o):
        a = o.createRaw([4, 8], np.full(32, 1.0 / 32, np.float32))
        b = o.createRaw([4, 8], np.full(32, -1e8 / 32, np.float32))
        t = o.createRaw([1], np.array([1e8], np.float32))
        s1 = a.times(1.0).sum()              # 1.0, created first
        s2 = b.times(1.0).sum()              # -1e8
        t.plusAssign(s2)
        t.plusAssign(s1)                     # (1e8 - 1e8) + 1 = 1; the other order gives (1e8 + 1) - 1e8 = 0
        return [t]
    eager, lazy, stats = both(script)
    assert eager[0][0] == 1.0 and same_bits(eager[0], lazy[0])
    assert stats[1][1] == 1                  # both sums in one pass


def test_allreduce_through_the_recorder_joins_the_pass_when_it_can():
    """ktc_lazy_allreduce on (loss, grad w, grad b): with everything deferred the step is one pass whose second pass
    applies both updates and performs the exchange (no call of the collective's own); call by call, or with sums that
    run where they are written, the values are computed first and the collective is called on their buffers."""
    from kten_b200.sharded import ShardedSigmoidGraph

    class RecorderCollective:                      # what PeerMemoryCollective.allreduce_sum does, without a communicator to create
        def __init__(self, ops):
            self.ops = ops

        def allreduce_sum(self, raws):
            self.ops._recorder.allreduce(7, [r._lz(apply_updates=False) for r in raws])

    rows, cols = 32, 16
    x, w, b = D.uniform(rows * cols, 0, -1.0, 1.0), D.normal(cols, 0, 0.0, 0.5, stream=1), D.uniform(cols, 0, -0.1, 0.1, stream=2)
    # steps whose results nobody reads in between (a training loop on several ranks): the gradient buffers are held by
    # the recorder alone, zeroGrad still becomes a pending constant, and every step is the one call
    ops = make_ops()
    ops.lazy = True
    with ops.garbageCollector():
        g = ShardedSigmoidGraph(ops, ops.createRaw([rows, cols], x), ops.createRaw([1, cols], w), ops.createRaw([cols], b), RecorderCollective(ops))
        for step in range(3):
            n0 = len(ops.lib.calls)
            g.step()
            assert ops.lib.calls[n0:] == ["expr_eval"], (step, ops.lib.calls[n0:])
            g.release_step()
    vals = {}
    for mode in ("eager", "deferred", "sums at once"):
        ops = make_ops()
        ops.lazy = mode != "eager"
        ops.deferSums = mode == "deferred"
        with ops.garbageCollector():
            g = ShardedSigmoidGraph(ops, ops.createRaw([rows, cols], x), ops.createRaw([1, cols], w), ops.createRaw([cols], b), RecorderCollective(ops))
            for _ in range(2):
                n0 = len(ops.lib.calls)
                loss, gw, gb = g.step()
                calls = ops.lib.calls[n0:]
                vals[mode] = (loss.toArray().copy(), gw.toArray().copy(), gb.toArray().copy())
                g.release_step()
            if mode == "deferred":
                last = ops.lib.programs[-1]
                assert calls == ["expr_eval"] and last["folded_updates"] == 2
                assert last["exchange"] == [loss.storeReference, gw.storeReference, gb.storeReference]
                assert ops._recorder.stats()["folded_exchanges"] == 2
            else:
                assert calls[-1] == "p2p_allreduce" and calls.count("p2p_allreduce") == 1
                assert ops._recorder.stats()["folded_exchanges"] == 0
    for a, c, d in zip(vals["eager"], vals["deferred"], vals["sums at once"]):
        assert np.allclose(a, c, rtol=1e-6, atol=1e-6) and np.allclose(a, d, rtol=1e-6, atol=1e-6)
