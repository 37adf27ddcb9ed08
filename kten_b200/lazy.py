"""Deferred elementwise expressions behind the RawTensor SPI.

kten's autograd issues one raw-tensor call per line of doForward / doBackward
(kten-api/.../autograd/functions/BasicFunctions.kt, PointwiseFunctions.kt,
AggregatingFunctions.kt); executed one by one, the sharded-graph step of the benchmark
moves 34 tensor volumes through HBM.  With `ops.lazy = True` a CUDARawTensor produced by
an elementwise call holds an expression node instead of storage; the expression is
compiled into a program for `ktc_expr_eval` when a value is needed -- a host read, a sum
(`sum()`, `mean()`, the leading-axis sums of mayUnexpand), or any call outside the
elementwise set.  Every instruction of the program is one of the library's reference
operations with its own rounding, so results equal the call-by-call execution bit for
bit; only the order of summation inside a fused sum differs (within the reduction
tolerance, exact on exactly summable data).

Rules that keep the semantics of the eager backend:
  * nodes are immutable; an in-place call on a deferred tensor replaces its node, an
    in-place call on a stored tensor is evaluated at once into its own buffer;
  * before a stored tensor is written in place, every deferred tensor that reads it is
    evaluated (a registry maps buffers to the deferred tensors depending on them);
  * a shallow copy of a deferred tensor evaluates it first, so aliases keep sharing
    storage exactly as in the eager backend;
  * an interior node is recomputed inside at most `ops.recomputeLimit` programs (recomputing a
    short chain from an operand that is read anyway costs no memory traffic); the next
    evaluation, if its tensor is still alive, stores it as a side output and later programs
    read it from memory; a value behind a transcendental (`ops.storeCost`) is stored by the
    first program that computes it, since that program is issue-bound and the store rides along;
  * with `ops.deferSums`, sum() / mean() and the leading-axis sums of a deferred tensor are
    deferred as well, and `stored += pending sum` (a gradient accumulated into a Variable) is
    remembered as a pending update of that buffer; the first read of any of them -- or of the
    updated buffer -- runs all pending sums, those over the same iteration space as ONE pass with
    several sinks (the loss and both broadcast gradients of a training step read x once);
  * `gather` with few picks from a pending expression gathers the expression's operands and rebuilds the
    expression over the index's shape (elementwise operations commute with the pick);
  * with `ops.deferInplace`, an in-place call with a pending operand on a stored tensor whose buffer nobody
    else holds makes the tensor deferred (its node reads the old buffer) instead of rewriting the buffer at
    once, so that a chain of in-place calls becomes one program;
  * compiled programs are cached by the structure of the expression DAG, so a training step that
    rebuilds the same graph with fresh tensors pays for register allocation once.
Whatever the kernel does not fuse (more than three collapsed dimensions, an innermost
extent that is not a multiple of four, programs beyond its size limits) falls back to
the library's separate calls -- never to the host.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, List, Optional, Sequence, Tuple

from . import _lib as L
from . import shape_functions as SF

BIN_X = {L.PLUS: L.X_ADD, L.MINUS: L.X_SUB, L.TIMES: L.X_MUL, L.DIV: L.X_DIV, L.POW: L.X_POW}
UN_X = {L.EXP: L.X_EXP, L.LOG: L.X_LOG, L.TANH: L.X_TANH, L.SIGMOID: L.X_SIGMOID, L.RECIPROCAL: L.X_RCP, L.NEG: L.X_NEG}
CMP_X = {L.LT: L.X_CMP_LT, L.LTE: L.X_CMP_LTE, L.GT: L.X_CMP_GT, L.GTE: L.X_CMP_GTE}


class BufferRef:
    """One retained reference on a library buffer, dropped when the last node using it dies."""

    __slots__ = ("lib", "handle", "__weakref__")

    def __init__(self, lib, handle: int, retain: bool = True):
        self.lib, self.handle = lib, handle
        if retain:
            L.check(lib.ktc_retain(handle))

    def __del__(self):
        try:
            self.lib.ktc_release(self.handle)
        except Exception:
            pass


class Node:
    """kind: leaf | const | un | bin | clamp | cmp | square | bcast | reduce.  Immutable value; `buf`
    is set once the value has been written to memory (the node then acts as a leaf).  A `reduce`
    node is a sum that has not run yet: args[0] is the summed expression, op the sink kind
    (EXPR_SUM_ALL / EXPR_SUM_ROWS), imm[0] != 0 a mean; it is never part of a program -- whoever
    needs its value runs the pending sums first, several of them in one pass where they share an
    iteration space."""

    __slots__ = ("kind", "op", "args", "shape", "imm", "buf", "leaves", "evals", "owner", "parents", "has_sum", "__weakref__")

    def __init__(self, kind, shape, op=0, args=(), imm=(), buf: Optional[BufferRef] = None):
        self.kind, self.op, self.args, self.shape, self.imm, self.buf = kind, op, tuple(args), list(shape), tuple(imm), buf
        self.evals = 0
        self.owner = None                      # weakref to the storage cell (raw_tensor._Cell) waiting for this value
        self.parents = None                    # weak references to the nodes built on this one (list, pruned as it grows)
        self.has_sum = kind == "reduce"        # a pending sum may sit underneath (never reset: a stale True only costs a look)
        if buf is not None:
            self.leaves = {buf.handle}
            return
        handles = set()
        me = None
        for a in self.args:
            if a.has_sum and a.buf is None:
                self.has_sum = True
            if a.buf is not None:
                handles.add(a.buf.handle)
            else:
                handles |= a.leaves
            if a.kind != "const":
                if me is None:
                    me = weakref.ref(self)
                ps = a.parents
                if ps is None:
                    a.parents = [me]
                else:
                    ps.append(me)
                    if len(ps) > 64 and (len(ps) & (len(ps) - 1)) == 0:      # at powers of two: drop the dead ones
                        a.parents = [r for r in ps if r() is not None]
        self.leaves = handles                  # buffers this value is read from (grows when a descendant is stored)

    def stored(self) -> bool:
        return self.buf is not None

    def ancestors(self):
        seen, stack = set(), [r() for r in (self.parents or ())]
        while stack:
            n = stack.pop()
            if n is None or n in seen:
                continue
            seen.add(n)
            yield n
            if n.parents:
                stack.extend(r() for r in n.parents)

    def set_stored(self, buf: BufferRef, registry) -> None:
        """The value now lives in `buf`: forget how it was computed, and make everything that is
        computed from it depend on the new buffer."""
        self.buf = buf
        self.args = ()
        for anc in self.ancestors():
            anc.leaves.add(buf.handle)
            if anc.owner is not None and anc.owner() is not None:
                registry.setdefault(buf.handle, []).append(anc.owner)


def leaf(lib, handle: int, shape) -> Node:
    return Node("leaf", shape, buf=BufferRef(lib, handle))


def const(value: float) -> Node:
    return Node("const", [1], imm=(float(value),))


class NotFusable(Exception):
    pass


class Program:
    def __init__(self, shape):
        self.shape = list(shape)
        self.code: List[int] = []
        self.imm: List[float] = []
        self.leaves: List[Tuple[int, List[int]]] = []       # (handle, right-aligned shape)
        self.n_stores = 0
        self.free = list(range(L.EXPR_REGS - 1, -1, -1))
        self.imm_src: List[Tuple[int, int]] = []             # per immediate: (position of its node in the order, index in node.imm)
        self.leaf_src: List[int] = []                        # per leaf: position of the (first) stored node it came from
        self.order: List["Node"] = []

    def emit(self, op, d=0, a=0, b=0, k=0):
        if len(self.code) >= L.EXPR_MAX_INSTR:
            raise NotFusable("program too long")
        self.code.append(op | (d << 8) | (a << 12) | (b << 16) | (k << 20))

    def imm_index(self, values, src: int = -1) -> int:
        if len(self.imm) + len(values) > L.EXPR_MAX_IMM:
            raise NotFusable("too many immediates")
        k = len(self.imm)
        self.imm.extend(values)
        self.imm_src.extend((src, j) for j in range(len(values)))
        return k

    def leaf_index(self, handle, shape, src: int = -1) -> int:
        nd = len(self.shape)
        padded = [1] * (nd - len(shape)) + list(shape)
        if len(padded) != nd:
            raise NotFusable("leaf has more dimensions than the iteration space")
        for i, (h, s) in enumerate(self.leaves):
            if h == handle and s == padded:
                return i
        if len(self.leaves) >= L.EXPR_MAX_LEAVES:
            raise NotFusable("too many leaves")
        self.leaves.append((handle, padded))
        self.leaf_src.append(src)
        return len(self.leaves) - 1

    def alloc(self) -> int:
        if not self.free:
            raise NotFusable("out of registers")
        return self.free.pop()


def strip(n: Node) -> Node:
    """Look through broadcast markers: they change the shape, not the value of an element."""
    while n.kind == "bcast" and not n.stored():
        n = n.args[0]
    return n


def _toposort(roots: Sequence[Node]) -> Tuple[List[Node], Dict[Node, int]]:
    """Children-first order of the unstored DAG under `roots` (broadcast markers looked through) and
    the number of uses of every node (one per consumer, one per root)."""
    order: List[Node] = []
    uses: Dict[Node, int] = {}
    stack = []
    for r in roots:
        while r.kind == "bcast" and r.buf is None:
            r = r.args[0]
        stack.append((r, False))
    # iterative post-order; a node is expanded the first time it is seen
    stack.reverse()
    while stack:
        n, done = stack.pop()
        if done:
            order.append(n)
            continue
        c = uses.get(n)
        if c is not None:
            uses[n] = c + 1
            continue
        uses[n] = 1
        stack.append((n, True))
        if n.buf is None:
            for a in reversed(n.args):
                while a.kind == "bcast" and a.buf is None:
                    a = a.args[0]
                stack.append((a, False))
    return order, uses


# rough issue cost of recomputing one element of a node, in units of a float add
HEAVY = {L.EXP: 10, L.LOG: 10, L.TANH: 12, L.SIGMOID: 16, L.RECIPROCAL: 2, L.NEG: 1}


def _weight(n: Node) -> int:
    if n.kind == "un":
        return HEAVY.get(n.op, 1)
    if n.kind == "bin":
        return 30 if n.op == L.POW else 3 if n.op == L.DIV else 1
    return 0 if n.kind in ("leaf", "const", "bcast") else 1


def compile_program(shape, stores: Sequence[Node], acc, recompute_limit: int = 0, store_cost: int = 0):
    """Linearise the DAG under `stores` + `acc` into a register program over the iteration
    space `shape`.  `acc`: the summed node of a single-sink program (or None), or a list of
    nodes, one per sink of a multi-sink program (the ACC of list entry j carries sink index j).  Returns (Program, nodes written by STORE, in store-index order; the first
    len(stores) entries are the requested ones).  Side outputs: a value that a tensor still waits
    for is stored on the way when it was already computed `recompute_limit` times, or when
    recomputing it from memory would cost `store_cost` or more (both 0: nothing is stored but what
    was asked for).  Raises NotFusable."""
    accs = [strip(a) for a in acc] if isinstance(acc, (list, tuple)) else ([strip(acc)] if acc is not None else [])
    sinks = [strip(n) for n in stores] + accs
    order, uses = _toposort(sinks)
    full_volume = SF.to_store_size(shape)
    # The program depends on the structure of the DAG (operations, sharing, which values are in memory and which
    # leaves are the same buffer) and on the per-node facts the side-output rule looks at -- not on buffer handles
    # or constants.  Graphs are rebuilt with fresh nodes every step, so the compiled form is cached by that
    # structure and re-bound to the current nodes: immediates, leaf handles and store nodes are looked up by
    # position in the topological order.
    pos = {n: i for i, n in enumerate(order)}
    sig, first_leaf = [], {}
    for i, n in enumerate(order):
        if n.buf is not None:
            sig.append((0, tuple(n.shape), first_leaf.setdefault((n.buf.handle, tuple(n.shape)), i)))
        elif n.kind == "const":
            sig.append(1)
        else:
            cell = n.owner() if n.owner is not None else None
            waiting = cell is not None and cell.store is None and cell.node is n and SF.to_store_size(n.shape) == full_volume
            sig.append((n.kind, n.op, len(n.imm), tuple([pos[strip(a)] for a in n.args]), waiting,
                        recompute_limit > 0 and n.evals >= recompute_limit))
    key = (tuple(shape), tuple([pos[strip(n)] for n in stores]), tuple([pos[a] for a in accs]), isinstance(acc, (list, tuple)),
           recompute_limit, store_cost, tuple(sig))
    hit = _PROGRAM_CACHE.get(key)
    if hit is not None:
        if hit is _NOT_FUSABLE:
            raise NotFusable("not fusable (cached)")
        code, imm_src, leaf_plan, store_plan, n_requested = hit
        prog = Program(shape)
        prog.code = code                                     # shared, never modified
        prog.imm = [order[p].imm[j] for p, j in imm_src]
        prog.leaves = [(order[p].buf.handle, padded) for p, padded in leaf_plan]
        prog.n_stores = len(store_plan)
        prog.order = order
        return prog, [order[p] for p in store_plan], n_requested
    try:
        prog, store_nodes, n_requested = _compile(shape, stores, accs, recompute_limit, store_cost, sinks, order, uses, pos, full_volume)
    except NotFusable:
        if len(_PROGRAM_CACHE) < _PROGRAM_CACHE_MAX:
            _PROGRAM_CACHE[key] = _NOT_FUSABLE
        raise
    if len(_PROGRAM_CACHE) < _PROGRAM_CACHE_MAX:
        _PROGRAM_CACHE[key] = (prog.code, list(prog.imm_src), [(p, padded) for p, (_, padded) in zip(prog.leaf_src, prog.leaves)],
                               [pos[n] for n in store_nodes], n_requested)
    return prog, store_nodes, n_requested


_PROGRAM_CACHE: Dict[tuple, object] = {}
_PROGRAM_CACHE_MAX = 4096
_NOT_FUSABLE = object()


def _compile(shape, stores, accs, recompute_limit, store_cost, sinks, order, uses, pos, full_volume):
    """The uncached compilation: side-output choice, register allocation, emission."""
    prog = Program(shape)
    reg: Dict[Node, int] = {}
    store_nodes: List[Node] = [strip(n) for n in stores]
    n_requested = len(store_nodes)
    # Side outputs.  Recomputing a short chain from an operand that is read anyway costs no memory
    # traffic, so cheap values are recomputed (a bounded number of times); a value behind a
    # transcendental is stored the first time -- the kernel that computes it is issue-bound and the
    # store rides along -- and later programs load it.  Chosen bottom-up (a chosen value makes what
    # is built on it cheap), then pruned top-down: nothing reaches below a stored value any more.
    if recompute_limit > 0 or store_cost > 0:
        cost: Dict[Node, int] = {}
        chosen = set()
        for n in order:
            if n.stored() or n.kind in ("const", "leaf"):
                cost[n] = 0
                continue
            c = _weight(n) + sum(cost[strip(a)] for a in n.args)
            cell = n.owner() if n.owner is not None else None
            waiting = cell is not None and cell.store is None and cell.node is n
            if waiting and SF.to_store_size(n.shape) == full_volume and not any(n is s for s in store_nodes) \
                    and ((recompute_limit > 0 and n.evals >= recompute_limit) or (store_cost > 0 and c >= store_cost)):
                chosen.add(n)
                c = 0
            cost[n] = c
        seen, stack = set(), list(sinks)
        while stack:
            n = strip(stack.pop())
            if n in seen or n.stored():
                continue
            seen.add(n)
            if n in chosen and len(store_nodes) < L.EXPR_MAX_STORES:
                store_nodes.append(n)
                uses[n] += 1
                continue
            stack.extend(n.args)

    def release_use(n: Node):
        uses[n] -= 1
        if uses[n] == 0:
            prog.free.append(reg[n])

    for n in order:
        if n.stored():
            d = prog.alloc()
            prog.emit(L.X_LOAD, d, k=prog.leaf_index(n.buf.handle, n.shape, pos[n]))
        elif n.kind == "const":
            d = prog.alloc()
            prog.emit(L.X_CONST, d, k=prog.imm_index([n.imm[0]], pos[n]))
        else:
            children = [strip(a) for a in n.args]
            srcs = [reg[c] for c in children]
            for c in children:
                release_use(c)
            d = prog.alloc()                    # may reuse a source register: the kernel reads before it writes
            if n.kind == "bin":
                prog.emit(BIN_X[n.op], d, srcs[0], srcs[1])
            elif n.kind == "un":
                prog.emit(UN_X[n.op], d, srcs[0])
            elif n.kind == "square":
                prog.emit(L.X_SQUARE, d, srcs[0])
            elif n.kind == "clamp":
                prog.emit(L.X_CLAMP, d, srcs[0], k=prog.imm_index(list(n.imm), pos[n]))
            elif n.kind == "cmp":
                prog.emit(CMP_X[n.op], d, srcs[0], k=prog.imm_index([n.imm[0]], pos[n]))
            else:
                raise NotFusable(f"unknown node kind {n.kind}")
        reg[n] = d
        for k, sn in enumerate(store_nodes):
            if sn is n:
                prog.emit(L.X_STORE, a=d, k=k)
                release_use(n)
        for j, an in enumerate(accs):
            if an is n:
                prog.emit(L.X_ACC, a=d, k=j)
                release_use(n)
    prog.n_stores = len(store_nodes)
    prog.order = order
    return prog, store_nodes, n_requested


def run_program(ops, prog: Program, store_handles: Sequence[int], sink: int, sink_out: int, mean: bool) -> int:
    lib = ops.lib
    nd = len(prog.shape)
    code = (C.c_uint32 * len(prog.code))(*prog.code)
    imm = (C.c_float * max(1, len(prog.imm)))(*prog.imm)
    shape = (C.c_int64 * nd)(*prog.shape)
    nl = len(prog.leaves)
    leaves = (C.c_uint64 * max(1, nl))(*[h for h, _ in prog.leaves])
    lshapes = (C.c_int64 * max(1, nl * nd))(*[d for _, s in prog.leaves for d in s])
    stores = (C.c_uint64 * max(1, len(store_handles)))(*store_handles)
    return lib.ktc_expr_eval(code, len(prog.code), imm, len(prog.imm), shape, nd, leaves, lshapes, nl,
                             stores, len(store_handles), sink, sink_out, 1 if mean else 0)


def run_program_multi(ops, prog: Program, store_handles: Sequence[int], kinds: Sequence[int], outs: Sequence[int], means: Sequence[bool]) -> int:
    """ktc_expr_eval_multi: the ACC of sink j feeds a sum of kind kinds[j] written to outs[j]."""
    lib = ops.lib
    nd = len(prog.shape)
    code = (C.c_uint32 * len(prog.code))(*prog.code)
    imm = (C.c_float * max(1, len(prog.imm)))(*prog.imm)
    shape = (C.c_int64 * nd)(*prog.shape)
    nl = len(prog.leaves)
    leaves = (C.c_uint64 * max(1, nl))(*[h for h, _ in prog.leaves])
    lshapes = (C.c_int64 * max(1, nl * nd))(*[d for _, s in prog.leaves for d in s])
    stores = (C.c_uint64 * max(1, len(store_handles)))(*store_handles)
    ns = len(kinds)
    return lib.ktc_expr_eval_multi(code, len(prog.code), imm, len(prog.imm), shape, nd, leaves, lshapes, nl,
                                   stores, len(store_handles), (C.c_int * ns)(*kinds), (C.c_uint64 * ns)(*outs),
                                   (C.c_int * ns)(*[1 if m else 0 for m in means]), ns)


def has_pending_sum(roots: Sequence[Node]) -> bool:
    """True when an unevaluated `reduce` node is reachable from `roots` through unstored nodes."""
    seen, stack = set(), [r for r in roots if r.has_sum]
    while stack:
        n = stack.pop()
        if n in seen or n.buf is not None:
            continue
        seen.add(n)
        if n.kind == "reduce":
            return True
        stack.extend(a for a in n.args if a.has_sum)
    return False
