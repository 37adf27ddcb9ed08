"""Deferred elementwise expressions behind the RawTensor SPI: the client side.

kten's autograd issues one raw-tensor call per line of doForward / doBackward
(kten-api/.../autograd/functions/BasicFunctions.kt, PointwiseFunctions.kt,
AggregatingFunctions.kt); executed one by one, the sharded-graph step of the benchmark
moves 34 tensor volumes through HBM.  With `ops.lazy = True` a CUDARawTensor produced by
an elementwise call holds a CELL of the library's expression recorder (`ktc_lazy_*`,
kten_b200/csrc/ktc_lazy.cpp) instead of storage.  The recorder -- below the C ABI, so that
the Kotlin binding gets the same behaviour -- keeps the expression DAG, compiles it into a
program for the fused expression kernels when a value is needed (a host read, a sum, any call
outside the elementwise set, an in-place write to one of its operands), caches programs by DAG
structure, runs the sums of one iteration space as one pass, and falls back to the library's
separate calls for what the kernels decline.  Every instruction of a program is one reference
operation with its own rounding, so results equal the call-by-call execution bit for bit;
only the order of summation inside a fused sum differs.

What stays on this side is what belongs to the tensor object: which calls are elementwise,
the host copy of the shape, the tensor's own reference on its buffer, and telling the
recorder before a buffer it may have recorded is written by a call it does not see
(`flush`).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

from . import _lib as L

STATE_WRITTEN, STATE_PENDING, STATE_UPDATE_RECORDED, STATE_UPDATE_OF_ZEROED = 0, 1, 2, 3
OPTIONS = ("recompute_limit", "store_cost", "defer_sums", "defer_inplace")
STATS = ("fused", "unfused", "multi_sink", "pending_sums", "cache_hits", "compiled", "live_nodes", "live_cells", "folded_updates", "folded_exchanges")


class Recorder:
    """The `ktc_lazy_*` entry points of one library object, with Python-shaped arguments."""

    def __init__(self, lib):
        self.lib = lib

    def _cell(self, fn, *args) -> int:
        out = C.c_uint64(0)
        L.check(fn(*args, C.byref(out)))
        return out.value

    def leaf(self, handle: int, shape: Sequence[int]) -> int:
        arr, nd = L.shape_array(shape)
        return self._cell(self.lib.ktc_lazy_leaf, handle, arr, nd)

    def free(self, cell: int) -> None:
        self.lib.ktc_lazy_free(cell)

    def unary(self, op: int, a: int) -> int:
        return self._cell(self.lib.ktc_lazy_unary, op, a)

    def binary(self, op: int, a: int, b: int) -> int:
        return self._cell(self.lib.ktc_lazy_binary, op, a, b)

    def scalar(self, op: int, a: int, s: float, scalar_first: bool) -> int:
        return self._cell(self.lib.ktc_lazy_scalar, op, a, float(s), 1 if scalar_first else 0)

    def clamp(self, a: int, lo: float, hi: float) -> int:
        return self._cell(self.lib.ktc_lazy_clamp, a, float(lo), float(hi))

    def compare_scalar(self, op: int, a: int, value: float) -> int:
        return self._cell(self.lib.ktc_lazy_compare_scalar, op, a, float(value))

    def broadcast_to(self, a: int, shape: Sequence[int]) -> int:
        arr, nd = L.shape_array(shape)
        return self._cell(self.lib.ktc_lazy_broadcast_to, a, arr, nd)

    def assign_binary(self, op: int, target: int, other: int) -> int:
        state = C.c_int(0)
        L.check(self.lib.ktc_lazy_assign_binary(op, target, other, C.byref(state)))
        return state.value

    def assign_scalar(self, op: int, target: int, s: float) -> int:
        state = C.c_int(0)
        L.check(self.lib.ktc_lazy_assign_scalar(op, target, float(s), C.byref(state)))
        return state.value

    def full(self, device: int, shape: Sequence[int], value: float) -> int:
        """A cell whose pending value is `value` everywhere (createRawFill, zerosLike): no buffer until one is needed."""
        arr, nd = L.shape_array(shape)
        return self._cell(self.lib.ktc_lazy_full, device, arr, nd, float(value))

    def assign_fill(self, target: int, value: float) -> int:
        state = C.c_int(0)
        L.check(self.lib.ktc_lazy_assign_fill(target, float(value), C.byref(state)))
        return state.value

    def assign_scatter_const(self, target: int, index: int, value: float):
        """inplaceScatter(-1, index, constant) with one index per row, recorded; None: not recordable here."""
        state = C.c_int(0)
        rc = self.lib.ktc_lazy_assign_scatter_const(target, index, float(value), C.byref(state))
        if rc == L.KTC_ENOTSUP:
            return None
        L.check(rc)
        return state.value

    def softmax_xent_forward(self, logits: int, targets: int, lo: float, hi: float):
        """The forward of SoftmaxCrossEntropy, recorded: (softmax cell, nll cell), or None where the one-pass kernel does not
        apply (the caller issues the calls)."""
        fn = getattr(self.lib, "ktc_lazy_softmax_xent_forward", None)
        if fn is None:
            return None
        softmax, nll = C.c_uint64(0), C.c_uint64(0)
        rc = fn(logits, targets, float(lo), float(hi), C.byref(softmax), C.byref(nll))
        if rc == L.KTC_ENOTSUP:
            return None
        L.check(rc)
        return softmax.value, nll.value

    def sum(self, a: int, kind: int, mean: bool, res_shape: Sequence[int]) -> int:
        arr, nd = L.shape_array(res_shape)
        return self._cell(self.lib.ktc_lazy_sum, a, kind, 1 if mean else 0, arr, nd)

    def buffer(self, cell: int) -> int:
        """The buffer holding the cell's value (computed now if pending); the caller owns one reference."""
        out = C.c_uint64(0)
        L.check(self.lib.ktc_lazy_buffer(cell, C.byref(out)))
        return out.value

    def is_pending(self, cell: int) -> bool:
        pending = C.c_int(0)
        L.check(self.lib.ktc_lazy_info(cell, C.byref(pending), None, None, None))
        return bool(pending.value)

    def flush(self, handle: int) -> None:
        L.check(self.lib.ktc_lazy_flush(handle))

    def run_pending(self) -> None:
        L.check(self.lib.ktc_lazy_run_pending())

    def allreduce(self, comm: int, cells: Sequence[int]) -> None:
        """Sum the cells' values over the ranks of a peer-memory communicator, in place; pending work runs first
        and takes the exchange into its second-pass kernel where it can."""
        arr = (C.c_uint64 * len(cells))(*cells)
        L.check(self.lib.ktc_lazy_allreduce(comm, arr, len(cells)))

    def option(self, name: str, value: int) -> None:
        L.check(self.lib.ktc_lazy_option(name.encode(), int(value)))

    def stats(self) -> dict:
        out = (C.c_int64 * 10)()
        L.check(self.lib.ktc_lazy_stats(out))
        return dict(zip(STATS, (int(v) for v in out)))
