"""CUDATensorOperations -- the operations SPI of the kten-cuda backend.

Host-side mirror of `TensorOperations<RAW>` + `BasicTensorOperations`
(kten-api/.../tensor/operations/TensorOperations.kt:9-137,
BasicTensorOperations.kt:6-23) for the hot path: raw-tensor factories,
reference counting, the scoped garbage collector and the constant-base pow.
The GC scope follows the OpenCL backend (OCLTensorOperations.kt:72-94,
OCLEnvironment.kt:30-34): every raw tensor created while a scope is open is
released when it closes; survivors are those whose ref-count was raised
(Function.output, saveForBackward) or that were marked mustSurviveGC.
"""
from __future__ import annotations

import ctypes as C
import threading
import weakref
from typing import Callable, List, Optional, Sequence

import numpy as np

from . import _lib as L
from . import lazy as Z
from . import shape_functions as SF
from .raw_tensor import CUDARawTensor


class TensorOperationsGarbageCollector:
    """Closeable scope handle (TensorOperationsGarbageCollector.kt:9-33)."""

    def __init__(self, on_close: Callable[[], None]):
        self._on_close = on_close

    def mustKeep(self, *tensors) -> None:
        for t in tensors:
            raw = getattr(t, "raw", t)
            raw.mustSurviveGC = True

    def mayRelease(self, *tensors) -> None:
        for t in tensors:
            raw = getattr(t, "raw", t)
            raw.mustSurviveGC = False

    def close(self) -> None:
        self._on_close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


class CUDATensorOperations:
    """One instance per device (one platform per device, as OCLPlatformInitializer.kt:21-25)."""

    def __init__(self, device: int = 0):
        self.lib = L.load()
        n = C.c_int(0)
        L.check(self.lib.ktc_init(C.byref(n)))
        if device < 0 or device >= n.value:
            raise ValueError(f"CUDA device {device} not present ({n.value} visible)")
        self.device = device
        name = C.create_string_buffer(128)
        mem, sms = C.c_int64(0), C.c_int(0)
        L.check(self.lib.ktc_device_info(device, name, 128, C.byref(mem), C.byref(sms)))
        self.deviceName, self.totalMemory, self.smCount = name.value.decode(), mem.value, sms.value
        self.platformKey = f"CUDA - {device} - {self.deviceName}"
        self._tls = threading.local()
        self.epsilon = 1e-7                 # PlatformProvider.epsilon (PlatformProvider.kt:12): eq / neq tolerance
        # deferred elementwise expressions (kten_b200.lazy): off = every call runs at once, like kten-jvm
        self.lazy = False
        self._deps = {}                     # buffer handle -> weak references to the storage cells whose pending expressions read it
        self._deps_purge_at = 1024
        self.recomputeLimit = 2             # a pending value is recomputed at most this often before it is stored
        self.storeCost = 8                  # ... unless recomputing costs this much (a transcendental): stored at once
        self.deferSums = True               # with lazy: sums of deferred tensors wait too, and run several per pass
        self.deferInplace = True            # with lazy: an in-place call with a pending operand on a buffer nobody else holds waits too
        self._pending = []                  # [weak reference to a reduce node, the node itself once an update hangs on it, [target BufferRefs]]
        self._pending_targets = {}          # buffer handle -> number of pending `+= sum` updates
        self.multiSinkEvaluations = 0       # passes that produced more than one sum
        self.fusedEvaluations = 0           # programs run by ktc_expr_eval
        self.unfusedEvaluations = 0         # deferred expressions that fell back to separate calls

    # ---- GC scope ----------------------------------------------------------------
    def _collector(self) -> Optional[list]:
        return getattr(self._tls, "collector", None)

    def _instance_created(self, raw: CUDARawTensor) -> None:
        col = self._collector()
        if col is not None:
            col.append(raw)

    def garbageCollector(self) -> TensorOperationsGarbageCollector:
        if self._collector() is not None:           # nested scopes are no-ops (OCLTensorOperations.kt:73-74)
            return TensorOperationsGarbageCollector(lambda: None)
        self._tls.collector = []

        def close():
            col, self._tls.collector = self._tls.collector, None
            for raw in col:
                raw.release()

        return TensorOperationsGarbageCollector(close)

    # ---- factories ---------------------------------------------------------------
    def createRaw(self, shape: Sequence[int], init=None) -> CUDARawTensor:
        """createRaw(shape) / createRaw(shape, init) (TensorOperations.kt:11-16).  `init`
        may be a callable index -> float (as in the reference) or an array of the
        tensor's volume; either way the data is uploaded before the call returns."""
        shape = [int(d) for d in shape]
        n = SF.to_store_size(shape)
        h = C.c_uint64(0)
        L.check(self.lib.ktc_alloc(self.device, n, C.byref(h)))
        raw = CUDARawTensor(shape, h.value, self)
        if init is not None and n:
            if callable(init):
                host = np.fromiter((init(i) for i in range(n)), dtype=np.float32, count=n)
            else:
                host = np.ascontiguousarray(np.asarray(init, dtype=np.float32).reshape(-1))
                if host.size != n:
                    raise ValueError(f"init holds {host.size} values, shape {shape} needs {n}")
            L.check(self.lib.ktc_h2d(raw._store, 0, host.ctypes.data_as(C.c_void_p), n, 1))
        return raw

    def createRawFill(self, shape: Sequence[int], constant: float) -> CUDARawTensor:
        raw = self.createRaw(shape)
        raw.inplaceFill(constant)
        return raw

    def zerosLike(self, raw: CUDARawTensor) -> CUDARawTensor:
        return self.createRawFill(raw.shape, 0.0)

    def zeroOut(self, raw: CUDARawTensor) -> None:
        raw.inplaceFill(0.0)

    # ---- deferred expressions (kten_b200.lazy) ------------------------------------------------
    # A deferred tensor's cell holds an expression node instead of a buffer.  `_deps` maps a buffer
    # handle to the cells whose pending expressions read it, so that an in-place write to the buffer
    # can evaluate them first.
    def _register(self, cell, node) -> None:
        ref = node.owner = weakref.ref(cell)
        deps = self._deps
        for h in node.leaves:
            refs = deps.get(h)
            if refs is None:
                deps[h] = [ref]
            else:
                refs.append(ref)
                if len(refs) > 64 and (len(refs) & (len(refs) - 1)) == 0:      # at powers of two: drop the dead ones
                    deps[h] = [r for r in refs if r() is not None]
        if len(deps) > self._deps_purge_at:
            self._deps = {h: live for h, live in ((h, [r for r in refs if r() is not None]) for h, refs in deps.items()) if live}
            self._deps_purge_at = max(1024, 2 * len(self._deps))

    def _deferred(self, kind, shape, op, args, imm=()) -> CUDARawTensor:
        node = Z.Node(kind, shape, op, args, imm)
        t = CUDARawTensor(shape, None, self, node=node)
        self._register(t._cell, node)
        return t

    def _deferred_alias(self, src: CUDARawTensor) -> CUDARawTensor:
        """A new tensor with the same value and storage of its own (a deep copy that is not made yet)."""
        return self._deferred("bcast", src.shape, 0, (src._as_node(),))

    def _deferred_assign(self, target: CUDARawTensor, kind, op, args, imm=()) -> None:
        """target = f(target, ...) in place: a deferred target takes the new node; a stored target is
        evaluated now, into its own buffer."""
        node = Z.Node(kind, target.shape, op, args, imm)
        if target.isDeferred:
            target._node = node
            self._register(target._cell, node)
            return
        h = target._buf()
        self._flush_dependents(h)
        n = target.size
        other = Z.strip(args[1]) if kind == "bin" else None
        if node.has_sum and self._pending:
            if other is not None and op == L.PLUS and other.kind == "reduce" and not other.stored() and SF.to_store_size(other.shape) == n \
                    and Z.strip(args[0]).stored() and self._add_pending_update(other, h):
                return                                              # target += pending sum: applied when the sums run
            self._run_pending()
        if other is not None and (other.kind == "const" or (other.stored() and SF.to_store_size(other.shape) == n)):
            # nothing to fuse: the operand is already in memory (a gradient accumulated into a Variable, ...)
            if other.kind == "const":
                L.check(self.lib.ktc_scalar_inplace(op, h, other.imm[0], n))
            else:
                L.check(self.lib.ktc_binary_inplace(op, h, other.buf.handle, n))
            return
        if self.deferInplace and self._rebind_inplace(target, h, node):
            return
        if self._try_fused(target.shape, [node], [h], [False]):
            return
        self.unfusedEvaluations += 1
        if kind == "square":
            L.check(self.lib.ktc_scalar_inplace(L.POW, h, 2.0, n))
            return
        other = Z.strip(args[1])
        if other.kind == "const":
            L.check(self.lib.ktc_scalar_inplace(op, h, other.imm[0], n))
        else:
            hb, shp = self._force(other)
            if SF.to_store_size(shp) != n:                         # a broadcast marker over a smaller value
                tmp = self._alloc_handle(n)
                try:
                    self._eager_into(args[1], target.shape, tmp)
                    L.check(self.lib.ktc_binary_inplace(op, h, tmp, n))
                finally:
                    self.lib.ktc_release(tmp)
            else:
                L.check(self.lib.ktc_binary_inplace(op, h, hb, n))

    def _rebind_inplace(self, target: CUDARawTensor, h: int, node) -> bool:
        """target = f(target, pending expression) where nobody else holds target's buffer: instead of a pass that
        rewrites the buffer now, the tensor becomes deferred -- its node reads the old buffer as an operand -- so that
        the in-place calls that follow (SoftmaxCrossEntropy.kt:74-77: `+=`, `/=`, then the accumulation into the
        Variable) join one program.  Nobody can tell the difference: a buffer with a second holder (a view, a shallow
        copy, a pending expression that still reads it) is written in place as before."""
        cell = target._cell
        own = cell.node
        if own is None or not own.stored() or own.buf.handle != h or not any(a is own for a in node.args):
            return False
        cnt = C.c_int(0)
        L.check(self.lib.ktc_refcount(h, C.byref(cnt)))
        if cnt.value != 2:                                          # the cell's reference and its cached leaf's
            return False
        cell.store, cell.node = None, node
        L.check(self.lib.ktc_release(h))                            # the cell's reference; the leaf inside `node` keeps the buffer
        self._register(cell, node)
        return True

    def _flush_dependents(self, handle: int) -> None:
        if self._pending:
            if handle in self._pending_targets:
                self._run_pending()
            else:
                for ref, strong, _ in self._pending:
                    nd = strong if strong is not None else ref()
                    if nd is not None and handle in nd.leaves:
                        self._run_pending()
                        break
        refs = self._deps.pop(handle, None)
        if not refs:
            return
        for ref in refs:
            cell = ref()
            if cell is not None and cell.store is None and cell.node is not None and cell.share > 0 and handle in cell.node.leaves:
                self._materialize_cell(cell)

    def _alloc_handle(self, n: int) -> int:
        h = C.c_uint64(0)
        L.check(self.lib.ktc_alloc(self.device, n, C.byref(h)))
        return h.value

    def _adopt(self, node, handle: int) -> None:
        """`handle` (one owned reference) now holds node's value: the node keeps it, and the cell that
        owns the node -- if it is still waiting for exactly this value -- takes it as its storage."""
        cell = node.owner() if node.owner is not None else None
        if cell is not None and cell.store is None and cell.node is node and cell.share > 0:
            cell.store = handle                                                  # the cell takes the owned reference,
            node.set_stored(Z.BufferRef(self.lib, handle), self._deps)           # the node retains one of its own
        else:
            node.set_stored(Z.BufferRef(self.lib, handle, retain=False), self._deps)

    def _try_fused(self, shape, stores, handles, own, acc=None, sink=None, sink_out=0, mean=False, reshape=None) -> bool:
        """Compile `stores` (+ the summed node `acc`) and run them as one kernel.  handles[i] receives
        stores[i]; own[i]: the handle is a fresh buffer that node i adopts.  Nodes stored on the side
        get fresh buffers.  False: not fusable, nothing was run."""
        if self._pending and Z.has_pending_sum(list(stores) + ([acc] if acc is not None else [])):
            self._run_pending()
        try:
            prog, store_nodes, n_req = Z.compile_program(shape, stores, acc, self.recomputeLimit, self.storeCost)
            if reshape is not None and not reshape(prog):
                return False
        except Z.NotFusable:
            return False
        total = SF.to_store_size(shape)
        extra = [self._alloc_handle(total) for _ in store_nodes[n_req:]]
        rc = Z.run_program(self, prog, list(handles) + extra, L.EXPR_STORE_ONLY if sink is None else sink, sink_out, mean)
        if rc != L.KTC_OK:
            for h in extra:
                self.lib.ktc_release(h)
            if rc == L.KTC_ENOTSUP:
                return False
            L.check(rc)
        self.fusedEvaluations += 1
        for nd in prog.order:
            nd.evals += 1
        for nd, h, o in zip(store_nodes[:n_req], handles, own):
            if o:
                self._adopt(nd, h)
        for nd, h in zip(store_nodes[n_req:], extra):
            self._adopt(nd, h)
        return True

    def _force(self, node):
        """Make sure the value under `node` (looking through broadcast markers) is in memory; returns
        (handle, shape).  The handle stays valid while the node is alive."""
        nd = Z.strip(node)
        if nd.kind == "reduce" and not nd.stored():
            self._run_pending()
            if not nd.stored():
                raise RuntimeError("a pending sum was not evaluated")
        if not nd.stored():
            h = self._alloc_handle(SF.to_store_size(nd.shape))
            if not self._try_fused(nd.shape, [nd], [h], [True]):
                self.unfusedEvaluations += 1
                self._eager_into(nd, nd.shape, h)
                self._adopt(nd, h)
        return nd.buf.handle, nd.shape

    def _materialize(self, t: CUDARawTensor) -> None:
        """Give a deferred tensor storage."""
        self._materialize_cell(t._cell)

    def _materialize_cell(self, cell) -> None:
        node = cell.node
        if Z.strip(node) is node and not node.stored():
            self._force(node)                                       # adopted by the cell through node.owner
            if cell.store is None:
                raise RuntimeError("deferred tensor did not receive its storage")
            return
        # an alias of / a broadcast over another value: storage of its own
        h = self._alloc_handle(SF.to_store_size(node.shape))
        if not self._try_fused(node.shape, [node], [h], [False]):
            self.unfusedEvaluations += 1
            self._eager_into(node, node.shape, h)
        cell.store, cell.node = h, None

    def _sum_all(self, t: CUDARawTensor, mean: bool) -> Optional[CUDARawTensor]:
        """sum() / mean() of a deferred tensor fused with its expression; None: not fusable."""
        if self.deferSums:
            return self._defer_sum(t, L.EXPR_SUM_ALL, mean, [1])
        out = self.createRaw([1])
        if self._try_fused(t.shape, [], [], [], acc=t._node, sink=L.EXPR_SUM_ALL, sink_out=out._store, mean=mean):
            return out
        out.release()
        return None

    @staticmethod
    def _as_rows(shape):
        """The reshape hook that views the iteration space [A, ...] as [A, rest]: possible when every
        operand is either full or broadcast over the trailing dimensions."""
        rest = SF.to_store_size(shape[1:])
        full_tail = list(shape[1:])

        def as_rows(prog) -> bool:
            leaves2 = []
            for h, s in prog.leaves:
                if s[1:] == full_tail:
                    leaves2.append((h, [s[0], rest]))
                elif all(d == 1 for d in s[1:]):
                    leaves2.append((h, [s[0], 1]))
                else:
                    return False
            prog.shape, prog.leaves = [shape[0], rest], leaves2
            return True

        return as_rows

    def _sum_leading_axis(self, t: CUDARawTensor, res_shape=None) -> Optional[CUDARawTensor]:
        """sum over axis 0 of a deferred [A, ...] tensor fused with its expression (the leading-axis
        sums of mayUnexpand, Utils.kt:14-41): the iteration space is viewed as [A, rest]."""
        rest = SF.to_store_size(t.shape[1:])
        if self.deferSums and res_shape is not None:
            return self._defer_sum(t, L.EXPR_SUM_ROWS, False, res_shape)
        out = self.createRaw([rest])
        if self._try_fused(t.shape, [], [], [], acc=t._node, sink=L.EXPR_SUM_ROWS, sink_out=out._store, reshape=self._as_rows(t.shape)):
            return out
        out.release()
        return None

    # ---- pending sums --------------------------------------------------------------------------
    def _defer_sum(self, t: CUDARawTensor, kind: int, mean: bool, res_shape) -> CUDARawTensor:
        res = self._deferred("reduce", list(res_shape), kind, (t._node,), (1.0 if mean else 0.0,))
        self._pending.append([weakref.ref(res._node), None, []])
        return res

    def _add_pending_update(self, node, handle: int) -> bool:
        """Remember `buffer handle += node` (node: a pending sum).  The node is kept alive from here on."""
        for entry in self._pending:
            if entry[0]() is node:
                entry[1] = node
                entry[2].append(Z.BufferRef(self.lib, handle))
                self._pending_targets[handle] = self._pending_targets.get(handle, 0) + 1
                return True
        return False

    def _run_pending(self) -> None:
        """Evaluate every pending sum that is still wanted, then apply the pending updates in the order
        they were requested.  Sums over the same iteration space run as one multi-sink pass (up to
        KTC_EXPR_MAX_SINKS per pass); a sum whose expression contains another pending sum waits for it."""
        entries, self._pending, self._pending_targets = self._pending, [], {}
        todo = []
        for ref, strong, targets in entries:
            nd = strong if strong is not None else ref()
            if nd is not None and not nd.stored():
                todo.append((nd, targets))
        waiting = [nd for nd, _ in todo]
        while waiting:
            ready = [nd for nd in waiting if not Z.has_pending_sum([nd.args[0]])]
            if not ready:
                raise RuntimeError("pending sums depend on one another")
            waiting = [nd for nd in waiting if not any(nd is r for r in ready)]
            # one pass per iteration space; leading-axis sums view the space as [A, rest], last-axis sums need its
            # innermost dimension, so the two kinds do not share a pass (full sums join either)
            by_shape = {}
            for nd in ready:
                by_shape.setdefault(tuple(nd.args[0].shape), []).append(nd)
            groups = []
            for shape, nodes in by_shape.items():
                last = [nd for nd in nodes if nd.op == L.EXPR_SUM_LAST]
                rows = [nd for nd in nodes if nd.op == L.EXPR_SUM_ROWS]
                full = [nd for nd in nodes if nd.op == L.EXPR_SUM_ALL]
                if rows or not last:
                    groups.append((shape, rows + full))
                    full = []
                if last:
                    groups.append((shape, last + full))
            for shape, nodes in groups:
                for i in range(0, len(nodes), L.EXPR_MAX_SINKS):
                    chunk = nodes[i:i + L.EXPR_MAX_SINKS]
                    if len(chunk) > 1 and self._try_fused_sums(list(shape), chunk):
                        continue
                    for nd in chunk:
                        self._run_one_sum(nd)
        for nd, targets in todo:
            for ref in targets:
                L.check(self.lib.ktc_binary_inplace(L.PLUS, ref.handle, nd.buf.handle, SF.to_store_size(nd.shape)))

    def _try_fused_sums(self, shape, nodes) -> bool:
        """One pass over `shape` feeding every sum of `nodes`.  False: not fusable, nothing was run."""
        exprs = [nd.args[0] for nd in nodes]
        kinds = [nd.op for nd in nodes]
        try:
            # every consumer known so far sits in this pass: nothing is stored on the side for its cost alone
            prog, store_nodes, n_req = Z.compile_program(shape, [], list(exprs), self.recomputeLimit, 0)
            if any(k == L.EXPR_SUM_ROWS for k in kinds) and not self._as_rows(list(shape))(prog):
                return False
        except Z.NotFusable:
            return False
        total = SF.to_store_size(shape)
        outs = [self._alloc_handle(SF.to_store_size(nd.shape)) for nd in nodes]
        extra = [self._alloc_handle(total) for _ in store_nodes]
        rc = Z.run_program_multi(self, prog, extra, kinds, outs, [nd.imm[0] != 0 for nd in nodes])
        if rc != L.KTC_OK:
            for h in outs + extra:
                self.lib.ktc_release(h)
            if rc == L.KTC_ENOTSUP:
                return False
            L.check(rc)
        self.fusedEvaluations += 1
        self.multiSinkEvaluations += 1
        for nd in prog.order:
            nd.evals += 1
        for nd, h in zip(store_nodes, extra):
            self._adopt(nd, h)
        for nd, h in zip(nodes, outs):
            self._adopt(nd, h)
        return True

    def _run_one_sum(self, nd) -> None:
        """A single pending sum: fused with its expression, else the expression is evaluated and reduced
        by the library's reduction call."""
        expr = nd.args[0]
        shape = list(expr.shape)
        out = self._alloc_handle(SF.to_store_size(nd.shape))
        mean = nd.imm[0] != 0
        if nd.op == L.EXPR_SUM_ALL:
            ok = self._try_fused(shape, [], [], [], acc=expr, sink=L.EXPR_SUM_ALL, sink_out=out, mean=mean)
        elif nd.op == L.EXPR_SUM_LAST:
            ok = self._try_fused(shape, [], [], [], acc=expr, sink=L.EXPR_SUM_LAST, sink_out=out)
        else:
            ok = self._try_fused(shape, [], [], [], acc=expr, sink=L.EXPR_SUM_ROWS, sink_out=out, reshape=self._as_rows(shape))
        if not ok:
            self.unfusedEvaluations += 1
            h, shp = self._force(expr)
            n, tmp = SF.to_store_size(shape), None
            if SF.to_store_size(shp) != n:                          # a broadcast marker over a smaller value
                tmp = h = self._alloc_handle(n)
                self._eager_into(expr, shape, tmp)
            try:
                if nd.op == L.EXPR_SUM_ALL:
                    L.check(self.lib.ktc_reduce_all(L.MEAN if mean else L.SUM, out, h, n))
                elif nd.op == L.EXPR_SUM_LAST:
                    L.check(self.lib.ktc_reduce_axis(L.SUM, out, h, n // shape[-1], shape[-1], 1))
                else:
                    L.check(self.lib.ktc_reduce_axis(L.SUM, out, h, 1, shape[0], n // shape[0]))
            finally:
                if tmp is not None:
                    self.lib.ktc_release(tmp)
        self._adopt(nd, out)

    def _gather_deferred(self, t: CUDARawTensor, axis: int, index: CUDARawTensor) -> Optional[CUDARawTensor]:
        """gather(axis, index) of a deferred tensor when the index picks few of its elements (the one target per
        row of SoftmaxCrossEntropy.kt:53): elementwise operations commute with the pick, so the operands that are
        in memory are gathered and the expression is rebuilt over the index's shape -- the same operations with
        the same roundings on just the picked elements, and the full-size value is never written.  None: not
        applicable, gather the evaluated tensor as usual."""
        shape, ishape = list(t.shape), list(index.shape)
        nd = len(shape)
        if shape[axis] <= 1 or SF.to_store_size(ishape) * 8 > SF.to_store_size(shape):
            return None
        root = Z.strip(t._node)
        if root.stored():
            return None
        # children-first walk of the unstored part; pending sums underneath are evaluated first (they are operands in memory then)
        if self._pending and Z.has_pending_sum([root]):
            self._run_pending()
        order, _ = Z._toposort([root])
        plan = {}                                             # node -> ("same",) | ("gather", padded shape) for operands in memory
        for n in order:
            if n.kind == "const" or not n.stored():
                if n.kind == "reduce":
                    return None
                continue
            padded = [1] * (nd - len(n.shape)) + list(n.shape)
            if len(padded) != nd:
                return None
            if padded[axis] == 1:                             # broadcast along the axis: the pick does not touch it
                if any(p != 1 and p != i for k, (p, i) in enumerate(zip(padded, ishape)) if k != axis):
                    return None
                plan[n] = ("same",)
            elif padded[axis] == shape[axis] and all(p >= i for k, (p, i) in enumerate(zip(padded, ishape)) if k != axis):
                plan[n] = ("gather", padded)
            else:
                return None
        px, _ = L.shape_array(ishape)
        new = {}
        for n in order:
            if n.kind == "const":
                new[n] = n
            elif n.stored():
                if plan[n][0] == "same":
                    new[n] = n
                else:
                    h = self._alloc_handle(SF.to_store_size(ishape))
                    pi, _ = L.shape_array(plan[n][1])
                    rc = self.lib.ktc_gather_axis(h, n.buf.handle, pi, index._buf(), px, nd, axis)
                    if rc != L.KTC_OK:
                        self.lib.ktc_release(h)
                        L.check(rc)
                    new[n] = Z.Node("leaf", ishape, buf=Z.BufferRef(self.lib, h, retain=False))
            else:
                args = [new[Z.strip(a)] for a in n.args]
                out_shape = [1]
                for a in args:
                    if a.kind != "const":
                        out_shape = SF.infer_implicit_broadcast_shape(out_shape, a.shape)
                new[n] = Z.Node(n.kind, out_shape, n.op, args, n.imm)
        node = new[root]
        if list(node.shape) != ishape:
            node = Z.Node("bcast", ishape, 0, (node,))
        res = CUDARawTensor(ishape, None, self, node=node)
        self._register(res._cell, node)
        return res

    def _eager_into(self, node, shape, out_handle: int) -> None:
        """One step of the call-by-call evaluation: the operands of `node` are forced into memory
        (each as a fused program where possible), then the library call for `node` itself runs at the
        operation's natural shape -- the common shape of its operands with broadcast markers looked
        through -- and the result is spread to `shape` if that is larger."""
        lib = self.lib
        nd = Z.strip(node)
        n = SF.to_store_size(shape)

        def spread(h, shp):
            if SF.to_store_size(shp) == n:
                L.check(lib.ktc_d2d(out_handle, 0, h, 0, n))
            else:
                so, no = L.shape_array(shape)
                sa, na = L.shape_array(shp)
                L.check(lib.ktc_broadcast_to(out_handle, so, no, h, sa, na))

        if nd.stored():
            spread(nd.buf.handle, nd.shape)
            return
        kids = [Z.strip(c) for c in nd.args]
        tensors = [c for c in kids if c.kind != "const"]
        natural = list(tensors[0].shape)
        if len(tensors) == 2 and tensors[0].shape != tensors[1].shape:
            natural = SF.infer_implicit_broadcast_shape(tensors[0].shape, tensors[1].shape)
        m = SF.to_store_size(natural)
        if m == n:
            self._call_op(nd, kids, out_handle, m)
            return
        tmp = self._alloc_handle(m)
        try:
            self._call_op(nd, kids, tmp, m)
            spread(tmp, natural)
        finally:
            lib.ktc_release(tmp)

    def _call_op(self, nd, kids, out_handle: int, m: int) -> None:
        """The library call of one node; `m` elements at the natural shape."""
        lib = self.lib
        if nd.kind == "bin":
            a, b = kids
            if a.kind == "const" or b.kind == "const":
                first = a.kind == "const"
                h, _ = self._force(b if first else a)
                L.check(lib.ktc_scalar(nd.op, out_handle, h, (a if first else b).imm[0], m, 1 if first else 0))
                return
            (ha, sa_), (hb, sb_) = self._force(a), self._force(b)
            if sa_ == sb_:
                L.check(lib.ktc_binary(nd.op, out_handle, ha, hb, m))
            else:
                pa, na = L.shape_array(sa_)
                pb, nb = L.shape_array(sb_)
                L.check(lib.ktc_binary_bcast(nd.op, out_handle, ha, pa, na, hb, pb, nb))
            return
        h, _ = self._force(kids[0])
        if nd.kind == "un":
            L.check(lib.ktc_unary(nd.op, out_handle, h, m))
        elif nd.kind == "square":
            L.check(lib.ktc_scalar(L.POW, out_handle, h, 2.0, m, 0))
        elif nd.kind == "clamp":
            L.check(lib.ktc_clamp(out_handle, h, nd.imm[0], nd.imm[1], m))
        elif nd.kind == "cmp":
            L.check(lib.ktc_compare_scalar(nd.op, out_handle, h, nd.imm[0], m))
        else:
            raise RuntimeError(f"cannot evaluate expression node of kind {nd.kind}")

    # ---- reference counting --------------------------------------------------------
    def release(self, *raws: CUDARawTensor) -> None:
        for r in raws:
            r.release()

    def incrementRef(self, raw: CUDARawTensor) -> None:
        raw.incrementRef()

    def markSurviveGC(self, raw: CUDARawTensor) -> None:
        raw.mustSurviveGC = True

    def markReleasableInGC(self, raw: CUDARawTensor) -> None:
        raw.mustSurviveGC = False

    # ---- ops that live on the operations object ---------------------------------------
    def concat(self, axis: int, inputs: Sequence[CUDARawTensor]) -> CUDARawTensor:
        """concat (AbstractJVMTensorOperations.kt:106-120): each input is written into its range of the result."""
        shapes = [t.shape for t in inputs]
        res_shape = SF.concat_shapes(shapes, axis)
        a = SF.normalize_axis(shapes[0], axis)
        res = self.createRaw(res_shape)
        ranges = [(0, d - 1) for d in res_shape]
        last = 0
        for t in inputs:
            if t.shape[a] == 0:
                continue
            ranges[a] = (last, last + t.shape[a] - 1)
            res.set(ranges, t)
            last += t.shape[a]
        return res

    def pow(self, constant: float, raw: CUDARawTensor) -> CUDARawTensor:
        """pow(constant, raw) = constant ^ raw (TensorOperations.kt:39)."""
        return raw._scalar(L.POW, constant, scalar_first=True)

    def toSerializableData(self, raw: CUDARawTensor):
        return list(raw.shape), raw.toArray().reshape(-1)

    # ---- device plumbing ----------------------------------------------------------------
    def synchronize(self) -> None:
        L.check(self.lib.ktc_sync(self.device))

    def getMetrics(self) -> dict:
        """PlatformMetricsProvider.getMetrics (PlatformMetricsProvider.kt:3-6)."""
        live, cached, calls, hits = (C.c_int64(0) for _ in range(4))
        L.check(self.lib.ktc_pool_stats(self.device, C.byref(live), C.byref(cached), C.byref(calls), C.byref(hits)))
        return {"liveMB": live.value / 2**20, "pooledMB": cached.value / 2**20,
                "allocCalls": float(calls.value), "poolHits": float(hits.value),
                "kernelLaunches": float(self.lib.ktc_launch_count()),
                "fusedEvaluations": float(self.fusedEvaluations), "unfusedEvaluations": float(self.unfusedEvaluations),
                "multiSinkEvaluations": float(self.multiSinkEvaluations), "pendingSums": float(len(self._pending))}

    def setMemoryUsageScaleHint(self, fraction: float) -> None:
        """PlatformProvider.memoryUsageScaleHint (PlatformProvider.kt:12-40): cap the pool."""
        L.check(self.lib.ktc_pool_limit(self.device, int(self.totalMemory * fraction)))
