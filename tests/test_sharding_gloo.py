"""The N > 1 path on CPU: two gloo ranks shard the rows of the sharded-graph
configuration, run the same autograd call sequence on the CPU backend, all-reduce the
packed partials, and must reproduce the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kten_b200 import datagen as D
from kten_b200.sharded import ShardedSigmoidGraph, shard_rows
from oracle import oracle as O

ROWS, COLS = 512, 64


def test_shard_rows_partition():
    for n, world in ((262144, 8), (10, 4), (7, 2), (3, 5)):
        blocks = [shard_rows(n, world, r) for r in range(world)]
        assert blocks[0][0] == 0 and sum(c for _, c in blocks) == n
        for (f0, c0), (f1, _) in zip(blocks, blocks[1:]):
            assert f1 == f0 + c0
        assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


class GlooCollective:
    def allreduce_sum(self, raws):
        flat = torch.from_numpy(np.concatenate([r.data.reshape(-1) for r in raws]).astype(np.float32))
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        off = 0
        for r in raws:
            r.data[:] = flat[off:off + r.data.size].numpy(); off += r.data.size


def inputs():
    x = D.uniform(ROWS * COLS, 0, -1.0, 1.0, stream=0)
    w = D.normal(COLS, 0, 0.0, 0.02, stream=1)
    b = np.zeros(COLS, dtype=np.float32)
    return x, w, b


def run_graph(ops, x, rows, w, b, collective=None):
    g = ShardedSigmoidGraph(ops, ops.createRaw([rows, COLS], x), ops.createRaw([1, COLS], w), ops.createRaw([COLS], b), collective)
    loss, gw, gb = g.step()
    return loss.toArray().copy(), gw.toArray().copy(), gb.toArray().copy()


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, w, b = inputs()
        first, count = shard_rows(ROWS, world, rank)
        ops = O.OracleTensorOperations(mode=1)
        loss, gw, gb = run_graph(ops, x[first * COLS:(first + count) * COLS], count, w, b, GlooCollective())
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), loss=loss, gw=gw, gb=gb)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_gloo_ranks_match_the_unsharded_graph(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    x, w, b = inputs()
    loss, gw, gb = run_graph(O.OracleTensorOperations(mode=1), x, ROWS, w, b)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for key in ("loss", "gw", "gb"):
        assert np.array_equal(r0[key], r1[key])                     # every rank holds the same global sums
    assert gw.shape == (1, COLS) and gb.shape == (COLS,) and loss.shape == (1,)
    # partial sums are combined in a different order than the single pass: 1e-5 * sum|terms|
    s = 1.0 / (1.0 + np.exp(-(x.reshape(ROWS, COLS).astype(np.float64) * w + b)))
    assert abs(float(r0["loss"][0]) - float(loss[0])) <= 1e-5 * float((s * s).sum())
    g_terms = np.abs(2 * s * s * (1 - s))
    assert np.all(np.abs(r0["gb"].astype(np.float64) - gb) <= 1e-5 * g_terms.sum(axis=0) + 1e-12)
    assert np.all(np.abs(r0["gw"].reshape(-1).astype(np.float64) - gw.reshape(-1)) <=
                  1e-5 * (g_terms * np.abs(x.reshape(ROWS, COLS))).sum(axis=0) + 1e-12)
    # and against float64 ground truth
    assert abs(float(loss[0]) - float((s * s).sum())) <= 1e-5 * float((s * s).sum())


class GlooHandleCollective:
    """For the CUDA backend's host mirror over the stand-in library: looks the values up by buffer handle
    (which makes the backend run whatever it deferred), all-reduces them over gloo and writes them back in place."""

    def __init__(self, lib):
        self.lib = lib

    def allreduce_sum(self, raws):
        handles = [r.storeReference for r in raws]
        flat = torch.from_numpy(np.concatenate([self.lib._get(h)[:r.size] for h, r in zip(handles, raws)]).astype(np.float32))
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        off = 0
        for h, r in zip(handles, raws):
            r._before_inplace_write()
            self.lib._get(h)[:r.size] = flat[off:off + r.size].numpy(); off += r.size


def _deferred_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tests.fake_lib import make_ops
        x, w, b = inputs()
        first, count = shard_rows(ROWS, world, rank)
        ops = make_ops()
        ops.lazy = True                                        # elementwise calls, sums and gradient updates all wait
        with ops.garbageCollector():
            loss, gw, gb = run_graph(ops, x[first * COLS:(first + count) * COLS], count, w, b, GlooHandleCollective(ops.lib))
        np.savez(os.path.join(out_dir, f"deferred{rank}.npz"), loss=loss, gw=gw, gb=gb, multi=ops.lib.multi_calls)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_gloo_ranks_with_the_deferred_backend(tmp_path):
    """The sharded step with everything deferred on each rank: the exchange is what forces the one pass with three
    sinks, and the global sums equal the unsharded CPU result within the reduction tolerance."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_deferred_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    x, w, b = inputs()
    loss, gw, gb = run_graph(O.OracleTensorOperations(mode=1), x, ROWS, w, b)
    r0, r1 = np.load(tmp_path / "deferred0.npz"), np.load(tmp_path / "deferred1.npz")
    for key in ("loss", "gw", "gb"):
        assert np.array_equal(r0[key], r1[key])
    assert int(r0["multi"]) == 1 and int(r1["multi"]) == 1
    s = 1.0 / (1.0 + np.exp(-(x.reshape(ROWS, COLS).astype(np.float64) * w + b)))
    g_terms = np.abs(2 * s * s * (1 - s))
    assert abs(float(r0["loss"][0]) - float(loss[0])) <= 1e-5 * float((s * s).sum())
    assert np.all(np.abs(r0["gb"].astype(np.float64) - gb) <= 1e-5 * g_terms.sum(axis=0) + 1e-12)
    assert np.all(np.abs(r0["gw"].reshape(-1).astype(np.float64) - gw.reshape(-1)) <=
                  1e-5 * (g_terms * np.abs(x.reshape(ROWS, COLS))).sum(axis=0) + 1e-12)
