"""Batch-leading data parallelism for the hot path: one process per GPU, each owning a
contiguous block of rows of the leading dimension.

The reference has no multi-device execution (a tensor lives on exactly one platform,
kten-api/.../tensor/Tensor.kt:143); what shards here is the path itself:

  * elementwise ops whose small operand has leading extent 1 (or lower rank) and
    reductions over a non-leading axis need no communication: replicate the small
    operand, work on the local rows;
  * full reductions and sum-to-shape over the leading axis (the loss and the weight /
    bias gradients) leave one partial per rank; the partials are summed in place across
    the ranks -- by one kernel per rank over peer memory (PeerMemoryCollective), or
    packed into one buffer and passed to a single NCCL all-reduce (NcclCollective).

`ShardedSigmoidGraph` is the sharded autograd step of the benchmark configuration
"x[262144,1024], w[1,1024], b[1024]: loss = sum(sigmoid(x*w + b) pow 2)", issued as the
same raw-tensor call sequence kten's autograd issues (kten_b200.autograd), generic over
the backend so that it runs on the CUDA backend and, in tests, on a CPU backend.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence, Tuple

import numpy as np

from . import autograd as AG


def shard_rows(n_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """(first row, row count) of `rank`'s block: equal contiguous blocks, the first
    n_rows % world ranks take one extra row."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    base, extra = divmod(n_rows, world)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


class NcclCollective:
    """Sum small raw tensors across ranks: pack -> one in-place all-reduce on the
    device's compute stream -> unpack (ktc_allreduce_sum)."""

    def __init__(self, ops, comm: int):
        self.ops, self.comm = ops, comm
        self._packed = None

    def allreduce_sum(self, raws: Sequence) -> None:
        from . import _lib as L
        lib = self.ops.lib
        total = sum(r.size for r in raws)
        if self._packed is None or self._packed.size < total:
            if self._packed is not None:
                self._packed.release()
            self._packed = self.ops.createRaw([total])
            self._packed.mustSurviveGC = True
        off = 0
        for r in raws:
            L.check(lib.ktc_d2d(self._packed.storeReference, off, r.storeReference, 0, r.size)); off += r.size
        L.check(lib.ktc_allreduce_sum(self.comm, self._packed.storeReference, 0, total))
        off = 0
        for r in raws:
            L.check(lib.ktc_d2d(r.storeReference, 0, self._packed.storeReference, off, r.size)); off += r.size


class PeerMemoryCollective:
    """Sum small raw tensors across ranks with ONE kernel per rank over NVLink peer memory
    (ktc_p2p_allreduce_sum): values go straight from the tensors into every peer's mailbox, a bounded
    wait, then a rank-ordered sum written back in place -- no packing, no collective library.
    `exchange(my_bytes) -> list of every rank's bytes` carries the 64-byte IPC handles between the
    processes (e.g. torch.distributed.all_gather_object); `barrier()` is a host barrier."""

    def __init__(self, ops, world: int, rank: int, exchange, barrier):
        from . import _lib as L
        self.ops, self.world, self.rank, self._barrier = ops, world, rank, barrier
        self._L = L
        handle = C.create_string_buffer(L.P2P_HANDLE_BYTES)
        comm = C.c_uint64(0)
        L.check(ops.lib.ktc_p2p_create(ops.device, world, rank, C.byref(comm), handle))
        self.comm = comm.value
        everyone = exchange(bytes(handle.raw))
        if len(everyone) != world or any(len(h) != L.P2P_HANDLE_BYTES for h in everyone):
            raise RuntimeError("handle exchange returned a wrong number of handles")
        L.check(ops.lib.ktc_p2p_connect(self.comm, b"".join(everyone)))
        barrier()                                   # every mailbox is mapped everywhere before the first store

    def allreduce_sum(self, raws: Sequence) -> None:
        L = self._L
        if len(raws) <= L.P2P_MAX_TENSORS and all(hasattr(r, "_lz") for r in raws) and getattr(self.ops, "_recorder", None) is not None:
            # through the expression recorder: what is still pending is computed first, and where that is one pass with
            # several sums the exchange runs inside its second-pass kernel
            self.ops._recorder.allreduce(self.comm, [r._lz(apply_updates=False) for r in raws])
            return
        for i in range(0, len(raws), L.P2P_MAX_TENSORS):
            group = raws[i:i + L.P2P_MAX_TENSORS]
            bufs = (C.c_uint64 * len(group))(*[r.storeReference for r in group])
            counts = (C.c_int64 * len(group))(*[r.size for r in group])
            L.check(self.ops.lib.ktc_p2p_allreduce_sum(self.comm, bufs, counts, len(group)))

    def check(self) -> None:
        """Waits for the device; raises if a rank did not arrive within the limit."""
        st = C.c_int(0)
        self._L.check(self.ops.lib.ktc_p2p_status(self.comm, C.byref(st)))
        if st.value != self._L.KTC_OK:
            raise TimeoutError("peer-memory all-reduce: a rank did not arrive within the time limit")

    def close(self, barrier: bool = True) -> None:
        """`barrier=False` only where no all-reduce was ever issued (e.g. another rank failed to connect)."""
        if self.comm:
            self.ops.synchronize()
            if barrier:
                self._barrier()                     # nobody frees a mailbox a peer may still write
            self._L.check(self.ops.lib.ktc_p2p_destroy(self.comm))
            self.comm = 0


class LocalCollective:
    """World size 1: nothing to exchange.  The values are still looked up the way a collective looks
    them up (their buffer handles), so that whatever the backend deferred -- pending expressions,
    pending sums -- is computed inside the step, exactly as on a rank of a larger world."""

    def allreduce_sum(self, raws: Sequence) -> None:
        for r in raws:
            getattr(r, "storeReference", None)          # a backend without deferred values has nothing to look up


class ShardedSigmoidGraph:
    """loss = sum(sigmoid(x*w + b) pow 2) with x sharded by rows; backward gives the
    gradients of w ([1, C], via sum(0, keepDims)) and b ([C], via sum(0)); loss, gw
    and gb are then summed over the ranks.  `fused_unexpand` uses the backend's one-call
    sum-to-shape instead of the chain of axis sums."""

    def __init__(self, ops, x_raw, w_raw, b_raw, collective=None):
        self.ops = ops
        self.x = AG.NoGradVariable(ops, x_raw)
        self.w = AG.Variable(ops, w_raw)
        self.b = AG.Variable(ops, b_raw)
        self.collective = collective or LocalCollective()

    def step(self):
        """One forward + backward + exchange.  Returns raw tensors (loss [1], grad w
        [1, C], grad b [C]) holding the global sums; valid until the next step."""
        self.w.zeroGrad()
        self.b.zeroGrad()
        loss = ((self.x * self.w + self.b).sigmoid().pow(2.0)).sum()
        loss.forward()                                  # keeps the loss value across backward()
        loss.backward()
        out = [loss.getRawValue(), self.w.gradient, self.b.gradient]
        self.collective.allreduce_sum(out)
        self._last_loss_fn = loss
        return out

    def release_step(self):
        """Drop the graph of the last step (its retained loss value)."""
        fn = getattr(self, "_last_loss_fn", None)
        if fn is not None:
            fn.keepOutput = False
            fn.freeOutput = True
            fn.releaseUnusedInGraph()
            self._last_loss_fn = None
