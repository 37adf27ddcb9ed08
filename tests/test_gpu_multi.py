"""Multi-GPU checks as collected tests: they start one process per GPU with torchrun and skip on a box with one GPU."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpu_count() -> int:
    from kten_b200 import _lib as L
    import ctypes as C
    n = C.c_int(0)
    L.check(L.load().ktc_init(C.byref(n)))
    return n.value


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_peer_memory_allreduce_and_fused_exchange_across_gpus():
    """tests/multi_gpu/p2p_allreduce_check.py on two GPUs (or four, where the box has them): the stand-alone exchange and the
    one folded into the second-pass kernel are bit-identical to the rank-ordered host sum on every rank."""
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 4 if n >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "multi_gpu", "p2p_allreduce_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    res = json.loads(line)
    assert res["world"] == world and res["bit_exact_rank_ordered_sum"] is True
