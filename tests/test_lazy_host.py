"""Host logic of the deferred-expression layer (kten_b200.lazy) without a device: expression DAGs
are compiled into register programs for ktc_expr_eval and the programs are executed here by a
small numpy interpreter of the instruction encoding; the results must equal the direct numpy
evaluation of the same DAG.  Covers register reuse, shared sub-expressions, broadcast markers,
side outputs and the limits that make the compiler decline."""
import weakref

import numpy as np
import pytest

from kten_b200 import _lib as L
from kten_b200 import lazy as Z


class FakeLib:
    """Counts references per handle; nothing else of the library is needed to build nodes."""

    def __init__(self):
        self.refs = {}

    def ktc_retain(self, h):
        self.refs[h] = self.refs.get(h, 0) + 1
        return 0

    def ktc_release(self, h):
        self.refs[h] -= 1
        return 0


class FakeCell:
    __slots__ = ("store", "node", "share", "__weakref__")

    def __init__(self, node):
        self.store, self.node, self.share = None, node, 1


def interpret(prog, buffers, n_stores):
    """Run a compiled program over the whole iteration space at once."""
    shape = prog.shape
    regs = [None] * L.EXPR_REGS
    stores = [None] * n_stores
    acc = None
    f32 = np.float32
    for word in prog.code:
        op, d, a, b, k = word & 0xFF, (word >> 8) & 0xF, (word >> 12) & 0xF, (word >> 16) & 0xF, word >> 20
        if op == L.X_LOAD:
            h, lshape = prog.leaves[k]
            regs[d] = np.broadcast_to(buffers[h].reshape(lshape), shape).astype(f32)
        elif op == L.X_CONST:
            regs[d] = np.full(shape, prog.imm[k], f32)
        elif op in (L.X_ADD, L.X_SUB, L.X_MUL, L.X_DIV):
            fn = {L.X_ADD: np.add, L.X_SUB: np.subtract, L.X_MUL: np.multiply, L.X_DIV: np.divide}[op]
            regs[d] = fn(regs[a], regs[b]).astype(f32)
        elif op == L.X_NEG:
            regs[d] = -regs[a]
        elif op == L.X_RCP:
            regs[d] = (f32(1.0) / regs[a]).astype(f32)
        elif op == L.X_SQUARE:
            regs[d] = (regs[a] * regs[a]).astype(f32)
        elif op == L.X_EXP:
            regs[d] = np.exp(regs[a].astype(np.float64)).astype(f32)
        elif op == L.X_CLAMP:
            regs[d] = np.minimum(np.maximum(regs[a], f32(prog.imm[k])), f32(prog.imm[k + 1]))
        elif op == L.X_CMP_LT:
            regs[d] = (regs[a] < f32(prog.imm[k])).astype(f32)
        elif op == L.X_STORE:
            stores[k] = regs[a].copy()
        elif op == L.X_ACC:
            acc = regs[a].copy()
        else:
            raise AssertionError(f"opcode {op} not covered by the interpreter")
    return stores, acc


@pytest.fixture()
def env():
    lib = FakeLib()
    rng = np.random.default_rng(7)
    bufs = {}

    def leaf(handle, shape):
        bufs[handle] = rng.uniform(0.5, 2.0, int(np.prod(shape))).astype(np.float32)
        return Z.leaf(lib, handle, shape)

    return lib, bufs, leaf


def bin_(op, a, b, shape):
    return Z.Node("bin", shape, op, (a, b))


def test_program_equals_direct_evaluation(env):
    lib, bufs, leaf = env
    shape = [6, 8]
    x, w, b = leaf(1, shape), leaf(2, [1, 8]), leaf(3, [8])
    z = bin_(L.PLUS, bin_(L.TIMES, x, w, shape), b, shape)
    e = Z.Node("un", shape, L.EXP, (z,))
    sq = Z.Node("square", shape, 0, (e,))
    out = bin_(L.MINUS, sq, bin_(L.DIV, z, Z.const(4.0), shape), shape)            # z is used twice
    cl = Z.Node("clamp", shape, 0, (out,), imm=(0.0, 50.0))
    prog, store_nodes, n_req = Z.compile_program(shape, [cl, z], e, recompute_limit=1)
    assert n_req == 2 and len(store_nodes) == 2 and prog.n_stores == 2
    stores, acc = interpret(prog, bufs, 2)
    X, W, B = bufs[1].reshape(shape), bufs[2].reshape(1, 8), bufs[3].reshape(8)
    zz = (X * W).astype(np.float32) + B
    ee = np.exp(zz.astype(np.float64)).astype(np.float32)
    want = np.clip((ee * ee).astype(np.float32) - (zz / np.float32(4.0)).astype(np.float32), 0.0, 50.0)
    assert np.array_equal(stores[0], want) and np.array_equal(stores[1], zz) and np.array_equal(acc, ee)
    assert len(prog.leaves) == 3 and [s for _, s in prog.leaves] == [[6, 8], [1, 8], [1, 8]]
    loads = sum(1 for wd in prog.code if (wd & 0xFF) == L.X_LOAD)
    assert loads == 3                                                              # every leaf is loaded once


def test_broadcast_markers_cost_nothing(env):
    lib, bufs, leaf = env
    g = leaf(5, [1])
    x = leaf(6, [4, 8])
    gb = Z.Node("bcast", [4, 8], 0, (g,))
    alias = Z.Node("bcast", [4, 8], 0, (x,))                                        # a deep copy that is not made yet
    prod = bin_(L.TIMES, gb, alias, [4, 8])
    prog, nodes, _ = Z.compile_program([4, 8], [prod], None, recompute_limit=0)
    stores, _ = interpret(prog, bufs, 1)
    assert np.array_equal(stores[0], (bufs[5][0] * bufs[6]).reshape(4, 8))
    assert len(prog.code) == 4                                                     # 2 loads, 1 multiply, 1 store
    assert Z.strip(alias) is x and Z.strip(gb) is g


def test_registers_are_reused_and_limits_decline(env):
    lib, bufs, leaf = env
    shape = [16]
    x = leaf(10, shape)
    cur = x
    for i in range(12):                                                             # a long chain needs two registers
        cur = bin_(L.PLUS, cur, Z.const(float(i)), shape)
    prog, _, _ = Z.compile_program(shape, [cur], None, 0)
    stores, _ = interpret(prog, bufs, 1)
    want = bufs[10].copy()
    for i in range(12):
        want = (want + np.float32(i)).astype(np.float32)
    assert np.array_equal(stores[0], want)
    for _ in range(8):                                                              # 12 + 8 constants > 16 immediates
        cur = bin_(L.PLUS, cur, Z.const(0.5), shape)
    with pytest.raises(Z.NotFusable):
        Z.compile_program(shape, [cur], None, 0)
    many = leaf(20, shape)
    for h in range(21, 28):                                                         # 8 distinct leaves > 6
        many = bin_(L.TIMES, many, leaf(h, shape), shape)
    with pytest.raises(Z.NotFusable):
        Z.compile_program(shape, [many], None, 0)
    # a wide tree that needs more live values than there are registers
    def tree(depth, base):
        if depth == 0:
            return bin_(L.PLUS, x, Z.const(float(base)), shape)
        return bin_(L.TIMES, tree(depth - 1, base), tree(depth - 1, base + (1 << depth)), shape)
    with pytest.raises(Z.NotFusable):
        Z.compile_program(shape, [tree(4, 0)], None, 0)


def test_side_outputs_only_for_values_a_tensor_still_waits_for(env):
    lib, bufs, leaf = env
    shape = [8, 8]
    x = leaf(30, shape)
    z = bin_(L.PLUS, x, Z.const(1.0), shape)
    s = Z.Node("un", shape, L.EXP, (z,))
    cells = {"z": FakeCell(z), "s": FakeCell(s)}
    z.owner = lambda: cells["z"]
    s.owner = lambda: cells["s"]
    top = bin_(L.TIMES, s, s, shape)
    _, nodes, n_req = Z.compile_program(shape, [top], None, 1)
    assert len(nodes) == 1                                                          # first evaluation: nothing on the side
    z.evals = s.evals = 1
    prog, nodes, n_req = Z.compile_program(shape, [top], None, 1)
    assert n_req == 1 and nodes[1:] == [s]                                         # s is stored; z below it is not
    stores, _ = interpret(prog, bufs, 2)
    ss = np.exp((bufs[30] + np.float32(1.0)).astype(np.float64)).astype(np.float32).reshape(shape)
    assert np.array_equal(stores[1], ss) and np.array_equal(stores[0], (ss * ss).astype(np.float32))
    _, nodes, _ = Z.compile_program(shape, [top], None, 2)
    assert len(nodes) == 1                                                          # a higher recompute limit: not yet
    cells["s"].node = None                                                          # the tensor moved on: no side output
    _, nodes, _ = Z.compile_program(shape, [top], None, 1)
    assert nodes[1:] == [z]                                                         # ... but z, now reachable, is a candidate
    # cost rule: a value behind a transcendental is stored the first time, a cheap one is not
    cells["s"].node = s
    z.evals = s.evals = 0
    _, nodes, _ = Z.compile_program(shape, [top], None, 2, store_cost=8)
    assert nodes[1:] == [s]
    cells["s"].node = None
    _, nodes, _ = Z.compile_program(shape, [top], None, 2, store_cost=8)
    assert len(nodes) == 1                                                          # z alone is one addition


def test_set_stored_updates_dependents_and_references(env):
    lib, bufs, leaf = env
    shape = [8]
    x = leaf(40, shape)
    assert lib.refs[40] == 1
    mid = Z.Node("un", shape, L.EXP, (x,))
    top = bin_(L.PLUS, mid, Z.const(1.0), shape)
    assert top.leaves == {40}
    cell = FakeCell(top)
    top.owner = weakref.ref(cell)
    registry = {}
    mid.set_stored(Z.BufferRef(lib, 41), registry)
    assert mid.stored() and mid.args == () and 41 in top.leaves and any(r() is cell for r in registry[41])
    prog, _, _ = Z.compile_program(shape, [top], None, 0)
    assert [h for h, _ in prog.leaves] == [41]                                     # x is no longer read
    del mid, top, prog, cell
    import gc
    gc.collect()
    assert lib.refs[41] == 0 and lib.refs[40] == 1
    del x
    gc.collect()
    assert lib.refs[40] == 0
