"""SoftmaxCrossEntropy's forward as a pending value of the recorder (ktc_lazy_softmax_xent_forward): which kernel the
recorder asks for, in which order, and what it keeps in memory -- driven against the stand-in library on a machine without
a GPU.  The deferred results must carry the bits of the call-by-call run."""
import gc

import numpy as np

from kten_b200 import autograd as AG
from kten_b200 import datagen as D
from tests.fake_lib import make_ops

ROWS, COLS = 12, 128


def same_bits(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def _inputs():
    x = D.uniform(ROWS * COLS, 31, -2.0, 2.0).reshape(ROWS, COLS)
    t = np.floor(D.uniform(ROWS, 32, 0.0, COLS - 0.01)).astype(np.float32)
    return x, t


def _step(ops, loss_first=False, hold=None):
    """forward + backward through the autograd caller; returns (loss, gradient, calls)."""
    x, t = _inputs()
    logits = AG.Variable(ops, ops.createRaw([ROWS, COLS], x))
    targets = AG.NoGradVariable(ops, ops.createRaw([ROWS], t))
    loss = logits.softmaxCrossEntropy(targets)
    if hold is not None:
        hold.append(loss)
    loss.backward()
    if loss_first:
        lv = loss.toArray()
        gv = logits.grad().toArray()
    else:
        gv = logits.grad().toArray()
        lv = loss.toArray()
    return lv, gv, list(ops.lib.calls)


def _eager():
    ops = make_ops()
    with ops.garbageCollector():
        res = _step(ops)
    gc.collect()
    return res + (ops.lib.live_buffers(),)         # the Variable's value and gradient outlive the scope


def test_backward_runs_inside_the_forward_kernel_and_the_softmax_is_not_written():
    le, ge, ce, live = _eager()
    assert ce.count("softmax_xent_forward") == 1 and "softmax_xent_forward_expr" not in ce
    for loss_first in (False, True):
        ops = make_ops()
        ops.lazy = True
        kept = []
        real = ops.lib.ktc_softmax_xent_forward_expr

        def spy(softmax, *rest):
            kept.append(int(softmax))
            return real(softmax, *rest)

        ops.lib.ktc_softmax_xent_forward_expr = spy
        ops.lib._attach_recorder()                      # the recorder's table picks up the wrapped entry
        with ops.garbageCollector():
            ll, gl, cl = _step(ops, loss_first=loss_first)
        gc.collect()
        assert same_bits(le, ll) and same_bits(ge, gl)
        assert cl.count("softmax_xent_forward_expr") == 1 and "softmax_xent_forward" not in cl, cl
        assert kept == [0]                              # nothing holds the saved tensor any more: it never reaches memory
        assert ops.lib.live_buffers() == live


def test_a_held_softmax_is_written_by_the_same_kernel():
    x, t = _inputs()
    res = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            lg, tg = ops.createRaw([ROWS, COLS], x), ops.createRaw([ROWS, 1], t)
            softmax, nll = lg.softmaxCrossEntropyForward(tg, 1e-7, 1.0 - 1e-7)
            g = softmax.times(2.0).plus(1.0)
            res.append((g.toArray(), softmax.toArray(), nll.toArray(), list(ops.lib.calls)))
    (ge, se, ne, ce), (gl, sl, nl, cl) = res
    assert same_bits(ge, gl) and same_bits(se, sl) and same_bits(ne, nl)
    assert cl.count("softmax_xent_forward_expr") == 1 and "softmax_xent_forward" not in cl and "scalar" not in cl, cl


def test_other_consumers_get_the_forward_on_its_own():
    """A sum over the softmax, a consumer of another shape, the nll inside an expression: the forward runs alone first."""
    x, t = _inputs()
    res = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            lg, tg = ops.createRaw([ROWS, COLS], x), ops.createRaw([ROWS, 1], t)
            softmax, nll = lg.softmaxCrossEntropyForward(tg, 1e-7, 1.0 - 1e-7)
            col_sums = softmax.sum(0)
            scaled = nll.times(3.0)
            res.append((col_sums.toArray(), scaled.toArray(), softmax.exp().toArray(), list(ops.lib.calls)))
    (a0, b0, c0, _), (a1, b1, c1, cl) = res
    assert np.allclose(a0, a1, rtol=1e-6) and same_bits(b0, b1) and same_bits(c0, c1)
    assert cl.count("softmax_xent_forward") + cl.count("softmax_xent_forward_expr") == 1, cl


def test_without_a_generated_kernel_the_two_run_separately():
    le, ge, _, live = _eager()
    ops = make_ops()
    ops.lazy = True
    ops.lib.no_softmax_epilogue = True
    with ops.garbageCollector():
        ll, gl, cl = _step(ops)
    assert same_bits(le, ll) and same_bits(ge, gl)
    assert cl.count("softmax_xent_forward") == 1 and "softmax_xent_forward_expr" not in cl
    gc.collect()
    assert ops.lib.live_buffers() == live


def test_logits_written_in_place_after_the_forward_was_recorded():
    x, t = _inputs()
    res = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            lg, tg = ops.createRaw([ROWS, COLS], x), ops.createRaw([ROWS, 1], t)
            softmax, nll = lg.softmaxCrossEntropyForward(tg, 1e-7, 1.0 - 1e-7)
            lg.timesAssign(0.0)                         # the recorded forward read the old logits
            res.append((softmax.toArray(), nll.toArray(), lg.toArray()))
    assert all(same_bits(a, b) for a, b in zip(*res))
    assert not np.any(res[1][2])


def test_rows_the_kernel_does_not_take_fall_back_to_the_calls():
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (6, 48)).astype(np.float32)
    t = rng.integers(0, 48, 6).astype(np.float32)
    out = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            logits = AG.Variable(ops, ops.createRaw([6, 48], x))
            loss = logits.softmaxCrossEntropy(AG.NoGradVariable(ops, ops.createRaw([6], t)))
            loss.backward()
            out.append((loss.toArray(), logits.grad().toArray(), list(ops.lib.calls)))
    assert abs(float(out[0][0][0]) - float(out[1][0][0])) <= 1e-6 and np.abs(out[0][1] - out[1][1]).max() <= 1e-7
    assert not any(c.startswith("softmax_xent") for c in out[1][2])


def test_an_interior_value_read_later_is_recomputed_from_the_logits():
    x, t = _inputs()
    res = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            lg, tg = ops.createRaw([ROWS, COLS], x), ops.createRaw([ROWS, 1], t)
            softmax, nll = lg.softmaxCrossEntropyForward(tg, 1e-7, 1.0 - 1e-7)
            g = softmax.times(2.0)
            h = g.plus(1.0)
            softmax.release()
            hv = h.toArray()                            # one kernel: forward + both operations; neither softmax nor g is written
            gv = g.toArray()                            # asked for after all: the forward runs once more with g as its epilogue
            res.append((hv, gv, nll.toArray(), list(ops.lib.calls)))
    (h0, g0, n0, _), (h1, g1, n1, cl) = res
    assert same_bits(h0, h1) and same_bits(g0, g1) and same_bits(n0, n1)
    assert cl.count("softmax_xent_forward_expr") == 2 and "softmax_xent_forward" not in cl, cl


def test_gradient_accumulated_over_two_steps():
    """Two forward + backward passes into the same Variable without clearing or reading its gradient in between.  One
    expression over two pending forwards is not a form a forward can take into its kernel, so when the second step's
    gradient arrives the first step's is evaluated (with its forward), and the second step's kernel adds to the stored
    result: two kernels, the bits of the call-by-call run."""
    x, t = _inputs()
    res = []
    for mode in (False, True):
        ops = make_ops()
        ops.lazy = mode
        with ops.garbageCollector():
            logits = AG.Variable(ops, ops.createRaw([ROWS, COLS], x))
            targets = AG.NoGradVariable(ops, ops.createRaw([ROWS], t))
            for _ in range(2):
                loss = logits.softmaxCrossEntropy(targets)
                loss.backward()
            res.append((logits.grad().toArray(), loss.toArray(), list(ops.lib.calls)))
    (g0, l0, _), (g1, l1, cl) = res
    assert same_bits(g0, g1) and same_bits(l0, l1)
    assert cl.count("softmax_xent_forward_expr") == 2 and "softmax_xent_forward" not in cl, cl
