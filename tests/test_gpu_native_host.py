"""The compiled host above the C ABI (kten_b200/csrc/host/kten_host.cpp, libkten_host.so): the raw tensor and the
autograd caller of the sharded benchmark step restated in C++.  It must issue the call sequence the Python
mirror issues -- itself pinned on the reference's test vectors -- so the two hosts have to agree bit for bit,
call by call and with everything deferred."""
import ctypes as C

import numpy as np
import pytest

from kten_b200 import _lib as L
from kten_b200 import datagen as D

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_ops():
    from kten_b200.tensor_operations import CUDATensorOperations
    return CUDATensorOperations(0)


def same_bits(a, b):
    a, b = np.asarray(a, np.float32).reshape(-1), np.asarray(b, np.float32).reshape(-1)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def read(lib, handle, n):
    out = np.empty(n, np.float32)
    L.check(lib.ktc_d2h(out.ctypes.data_as(C.c_void_p), handle, 0, n, 1))
    return out


@pytest.mark.parametrize("rows,cols", [(2048, 1024), (96, 64)])
def test_compiled_host_equals_the_python_host(cuda_ops, rows, cols):
    from kten_b200.native_host import NativeShardedStep
    from kten_b200.sharded import ShardedSigmoidGraph
    ops, lib = cuda_ops, cuda_ops.lib
    x = ops.createRaw([rows, cols], D.uniform(rows * cols, 0, -1.0, 1.0))
    w = ops.createRaw([1, cols], D.normal(cols, 0, 0.0, 0.02, stream=1))
    b = ops.createRawFill([cols], 0.0)
    try:
        for deferred in (False, True):
            ops.lazy = deferred
            graph = ShardedSigmoidGraph(ops, x, w, b)
            with ops.garbageCollector():
                for _ in range(2):                                      # the second step starts from accumulated state
                    out = graph.step()
                want = [r.toArray().reshape(-1).copy() for r in out]
                graph.release_step()
            ops.lazy = False
            launches0 = lib.ktc_launch_count()
            native = NativeShardedStep(ops, x, w, b, deferred)
            try:
                native.run(1)
                handles = native.run(1, results=True)
                got = [read(lib, handles[0], 1), read(lib, handles[1], cols), read(lib, handles[2], cols)]
            finally:
                native.close()
            assert lib.ktc_launch_count() > launches0
            for name, g, v in zip(("loss", "grad w", "grad b"), got, want):
                assert same_bits(g, v), (name, deferred)
            for r in (graph.w.gradient, graph.b.gradient):
                r.mustSurviveGC = False
                r.release()
        st = ops._recorder.stats()
        assert st["pending_sums"] == 0
    finally:
        ops.lazy = False
        for r in (x, w, b):
            r.release()


def test_compiled_host_gives_its_storage_back(cuda_ops):
    from kten_b200.native_host import NativeShardedStep
    ops, lib = cuda_ops, cuda_ops.lib
    rows, cols = 256, 128
    x = ops.createRaw([rows, cols], D.uniform(rows * cols, 3, -1.0, 1.0))
    w = ops.createRaw([1, cols], D.normal(cols, 3, 0.0, 0.02, stream=1))
    b = ops.createRawFill([cols], 0.0)
    ops.synchronize()
    live0 = ops.getMetrics()["liveMB"]
    nodes0 = ops._recorder.stats()["live_nodes"]
    for deferred in (False, True):
        native = NativeShardedStep(ops, x, w, b, deferred)
        native.run(5)
        native.run(1, results=True)
        native.close()
    assert ops.getMetrics()["liveMB"] == live0
    assert ops._recorder.stats()["live_nodes"] == nodes0
    for r in (x, w, b):
        r.release()


class _Exchange:
    """What PeerMemoryCollective.allreduce_sum does, over a communicator the test created itself."""

    def __init__(self, ops, comm):
        self.ops, self.comm = ops, comm

    def allreduce_sum(self, raws):
        self.ops._recorder.allreduce(self.comm, [r._lz(apply_updates=False) for r in raws])


def _communicator(lib, world, connect_self=False):
    handle = C.create_string_buffer(L.P2P_HANDLE_BYTES)
    comm = C.c_uint64(0)
    L.check(lib.ktc_p2p_create(0, world, 0, C.byref(comm), handle))
    if connect_self:
        L.check(lib.ktc_test_p2p_connect_self(comm.value))
    else:
        L.check(lib.ktc_p2p_connect(comm.value, handle.raw))
    return comm.value


def test_step_with_the_exchange_inside_its_second_pass(cuda_ops):
    """A world of one: the all-reduce of (loss, grad w, grad b) is the identity, so the step must give the bits of
    the step without a collective -- now with the accumulation into the gradients and the exchange performed by
    the second-pass kernel of the one pass: five launches (two gradient fills, the seed, the pass, its second
    pass).  Then a communicator whose second rank never arrives: the wait inside that kernel gives up, the status
    says so, the local values stand and the device stays usable."""
    from kten_b200.native_host import NativeShardedStep
    from kten_b200.sharded import ShardedSigmoidGraph
    ops, lib = cuda_ops, cuda_ops.lib
    rows, cols = 2048, 1024
    x = ops.createRaw([rows, cols], D.uniform(rows * cols, 0, -1.0, 1.0))
    w = ops.createRaw([1, cols], D.normal(cols, 0, 0.0, 0.02, stream=1))
    b = ops.createRawFill([cols], 0.0)
    comm = _communicator(lib, 1)
    st = C.c_int(-99)
    try:
        ops.lazy = True
        plain = ShardedSigmoidGraph(ops, x, w, b)
        with ops.garbageCollector():
            want = [r.toArray().reshape(-1).copy() for r in plain.step()]
            plain.release_step()
        fused = ShardedSigmoidGraph(ops, x, w, b, _Exchange(ops, comm))
        with ops.garbageCollector():
            fused.step(); fused.release_step()                          # compiles what there is to compile
        ops.synchronize()
        s0, n0 = ops._recorder.stats(), lib.ktc_launch_count()
        with ops.garbageCollector():
            out = fused.step()
            launches = lib.ktc_launch_count() - n0
            got = [r.toArray().reshape(-1).copy() for r in out]
            fused.release_step()
        s1 = ops._recorder.stats()
        assert s1["folded_exchanges"] - s0["folded_exchanges"] == 1 and s1["folded_updates"] - s0["folded_updates"] == 2
        assert launches <= 5, launches
        for name, g, v in zip(("loss", "grad w", "grad b"), got, want):
            assert same_bits(g, v), name
        L.check(lib.ktc_p2p_status(comm, C.byref(st)))
        assert st.value == L.KTC_OK
        ops.lazy = False
        native = NativeShardedStep(ops, x, w, b, True, comm)           # the compiled host takes the same route
        try:
            native.run(1)
            n0 = lib.ktc_launch_count()
            handles = native.run(1, results=True)
            assert lib.ktc_launch_count() - n0 <= 5
            for h, v in zip(handles, want):
                assert same_bits(read(lib, h, v.size), v)
        finally:
            native.close()
        # a rank that never arrives
        L.check(lib.ktc_p2p_destroy(comm))
        L.check(lib.ktc_tune_set(b"p2p_wait_ms", 50))
        comm = _communicator(lib, 2, connect_self=True)
        ops.lazy = True
        alone = ShardedSigmoidGraph(ops, x, w, b, _Exchange(ops, comm))
        with ops.garbageCollector():
            got = [r.toArray().reshape(-1).copy() for r in alone.step()]
            alone.release_step()
        L.check(lib.ktc_p2p_status(comm, C.byref(st)))
        assert st.value == L.KTC_ETIMEOUT
        for g, v in zip(got, want):
            assert same_bits(g, v)                                       # nothing was summed: the local values stand
        ops.lazy = False
        assert same_bits(w.plus(w).toArray(), 2 * w.toArray())          # the device still works
        for gr in (plain, fused, alone):
            for r in (gr.w.gradient, gr.b.gradient):
                r.mustSurviveGC = False
                r.release()
    finally:
        ops.lazy = False
        L.check(lib.ktc_tune_set(b"p2p_wait_ms", 10000))
        L.check(lib.ktc_p2p_destroy(comm))
        for r in (x, w, b):
            r.release()
