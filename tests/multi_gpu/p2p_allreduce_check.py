"""Run under torchrun on N >= 2 GPUs of one box (one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29531 \
        tests/multi_gpu/p2p_allreduce_check.py

Checks the peer-memory all-reduce (ktc_p2p_allreduce_sum) against the rank-ordered float sum computed on
the host and against NCCL within the reduction tolerance, over many calls and sizes, and times both; then
the exchange folded into the second-pass kernel of a deferred training step (ktc_lazy_allreduce) against the
rank-ordered host sum of the ranks' local results, bit for bit.  NVLS is not needed and is switched off for
the NCCL leg.  tests/test_gpu_multi.py runs this file when the box has at least two GPUs."""
import ctypes as C
import json
import os
import sys
import time

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import numpy as np
import torch
import torch.distributed as dist

from kten_b200 import _lib as L
from kten_b200 import datagen as D
from kten_b200.sharded import NcclCollective, PeerMemoryCollective
from kten_b200.tensor_operations import CUDATensorOperations


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    torch.cuda.set_device(local)
    dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    ops = CUDATensorOperations(local)
    lib = ops.lib

    def exchange(mine: bytes):
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        return everyone

    p2p = PeerMemoryCollective(ops, world, rank, exchange, dist.barrier)
    ident = C.create_string_buffer(L.COMM_ID_BYTES)
    if rank == 0:
        L.check(lib.ktc_comm_unique_id(ident))
    box = [bytes(ident.raw)]
    dist.broadcast_object_list(box, src=0)
    comm = C.c_uint64(0)
    L.check(lib.ktc_comm_init_rank(local, world, rank, box[0], C.byref(comm)))
    nccl = NcclCollective(ops, comm.value)

    sizes = [(1,), (1, 1024, 1024), (7, 3, 4099), (16384 - 8, 8), (5,) * 8]
    ok = True
    for rep in range(40):
        shapes = sizes[rep % len(sizes)]
        host = [[D.uniform(n, 100 + rep, -1.0, 1.0, stream=r * 16 + i) for i, n in enumerate(shapes)] for r in range(world)]
        mine = [ops.createRaw([v.size], v) for v in host[rank]]
        p2p.allreduce_sum(mine)
        p2p.check()
        for i, t in enumerate(mine):
            want = host[0][i].copy()
            for r in range(1, world):
                want = (want + host[r][i]).astype(np.float32)              # rank order, float32
            got = t.toArray()
            if not np.array_equal(got.view(np.uint32), want.view(np.uint32)):
                ok = False
                print(f"rank {rank}: rep {rep} tensor {i} differs from the rank-ordered sum", file=sys.stderr)
        again = [ops.createRaw([v.size], v) for v in host[rank]]
        nccl.allreduce_sum(again)
        for a, b in zip(mine, again):
            x, y = a.toArray().astype(np.float64), b.toArray().astype(np.float64)
            if not np.all(np.abs(x - y) <= 1e-5 * world):
                ok = False
                print(f"rank {rank}: rep {rep} differs from NCCL", file=sys.stderr)
        for t in mine + again:
            t.release()

    # the exchange inside the producing kernel: one deferred step of the sharded graph per rank
    from kten_b200.sharded import ShardedSigmoidGraph
    rows, cols = 4096, 1024
    xs = D.normal(rows * cols, 31, 0.0, 1.0, stream=rank)
    w, b = D.uniform(cols, 32, -0.5, 0.5), D.uniform(cols, 33, -0.5, 0.5)
    ops.lazy = True
    before = ops._recorder.stats()["folded_exchanges"]
    alone = ShardedSigmoidGraph(ops, ops.createRaw([rows, cols], xs), ops.createRaw([1, cols], w), ops.createRaw([cols], b))
    mine = [t.toArray().reshape(-1).copy() for t in alone.step()]                      # this rank's loss, gw, gb
    alone.release_step()
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    fused = ShardedSigmoidGraph(ops, ops.createRaw([rows, cols], xs), ops.createRaw([1, cols], w), ops.createRaw([cols], b), collective=p2p)
    for step in range(3):                                                               # the first step compiles, the others hit the cache
        launches0 = lib.ktc_launch_count()
        out = fused.step()
        launches = lib.ktc_launch_count() - launches0
        if step > 0 and launches != 2:                                                  # the pass and its second pass, nothing else
            ok = False
            print(f"rank {rank}: fused exchange, step {step}: {launches} launches", file=sys.stderr)
        got = [t.toArray().reshape(-1) for t in out]
        p2p.check()
        fused.release_step()
        for i in range(3):
            want = everyone[0][i].copy()
            for r in range(1, world):
                want = (want + everyone[r][i]).astype(np.float32)
            if not np.array_equal(got[i].view(np.uint32), want.view(np.uint32)):
                ok = False
                print(f"rank {rank}: fused exchange, step {step}, tensor {i} differs from the rank-ordered sum", file=sys.stderr)
    folded = ops._recorder.stats()["folded_exchanges"] - before
    if folded != 3:
        ok = False
        print(f"rank {rank}: {folded} of 3 exchanges ran inside the second-pass kernel", file=sys.stderr)
    ops.lazy = False

    # timing: loss [1] + gw [1, 1024] + gb [1024], as in the sharded graph
    ts = [ops.createRaw([n], D.uniform(n, 7, -1.0, 1.0, stream=rank)) for n in (1, 1024, 1024)]
    res = {}
    for name, coll in (("peer_memory", p2p), ("nccl", nccl)):
        for _ in range(10):
            coll.allreduce_sum(ts)
        ops.synchronize(); dist.barrier()
        ms = C.c_float(0)
        L.check(lib.ktc_timer_start(local))
        for _ in range(200):
            coll.allreduce_sum(ts)
        L.check(lib.ktc_timer_stop(local, C.byref(ms)))
        t = torch.tensor([ms.value / 200], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name + "_us_per_call"] = round(float(t[0]) * 1e3, 2)
    p2p.check()
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"world": world, "bit_exact_rank_ordered_sum": bool(flag.item()), **res}))
    p2p.close()
    lib.ktc_comm_destroy(comm.value)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if flag.item() else 1


if __name__ == "__main__":
    sys.exit(main())
