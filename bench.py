#!/usr/bin/env python
"""Benchmark of the kten float32 hot path on B200: HBM GB/s and fraction of peak for
contiguous elementwise ops, broadcast binary ops and axis / full reductions.

    python bench.py [--gpus N] [--steps K] [--warmup W]             # this library
    python bench.py --impl reference [--steps K] [--warmup W]        # kten-jvm's algorithm on the host cores

One step is one pass over the sweep below on synthetic, seeded inputs that are
already resident in HBM (every operand is >= 1 GiB, far larger than the 126 MB
L2, so nothing is served from cache between iterations):

  C2  contiguous, 2^28 elements ~ U(0.1, 2):   plus, times, div, pow;  exp, log, tanh, sigmoid
  C3  broadcast, a[1024,1024,256] ~ N(0,1):    a*b, (a*b)+c, a/b   with b[1,1024,1], c[1024,1,256]
  C4  reductions, N(0,1) rounded to 1/16:      sum, mean, max, argmax over the last axis of [65536,4096];
                                               sum, max over the middle axis of [512,4096,128]; full sum of 2^28

With N > 1 (one process per GPU, launched by torch.distributed.run) each rank
owns one leading-dimension shard of an N-times larger batch and runs the same
sweep on it (weak scaling); the only exchange on the path is the all-reduce of
the full-sum partial.  The value is whole-job algorithmic bytes / max-over-ranks
device time.

The JSON line also carries: `e2e` (the same sweep through the public API with
pinned HOST buffers, host<->device copies inside the timed region), `roofline`
for the kernel with the largest share of the step, `per_op` GB/s, `cpu_baseline`
(the CPU oracle in kten-jvm's structure, on a bounded sample) and the SM clocks
sampled during the timed region.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N28 = 1 << 28
GIB = 1 << 30
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


# ----------------------------------------------------------------------------------------------
# workload description (shared by both arms)
# ----------------------------------------------------------------------------------------------
def sweep_spec():
    """name, kernel family, algorithmic bytes (each distinct input element once at its
    un-broadcast size + each output element once), elements the throughput is quoted on."""
    ops = []
    for name in ("plus", "times", "div", "pow"):
        ops.append(dict(name=f"c2.{name}", family="map2", bytes=3 * GIB, elements=N28))
    for name in ("exp", "log", "tanh", "sigmoid"):
        ops.append(dict(name=f"c2.{name}", family="map1", bytes=2 * GIB, elements=N28))
    ops.append(dict(name="c3.a*b", family="bcast", bytes=2 * GIB + 4096, elements=N28))
    ops.append(dict(name="c3.(a*b)+c", family="bcast", bytes=2 * GIB + (1 << 20), elements=N28))
    ops.append(dict(name="c3.a/b", family="bcast", bytes=2 * GIB + 4096, elements=N28))
    for name in ("sum", "mean", "max", "argmax"):
        ops.append(dict(name=f"c4.last.{name}", family="reduce_rows", bytes=GIB + 65536 * 4, elements=N28))
    for name in ("sum", "max"):
        ops.append(dict(name=f"c4.mid.{name}", family="reduce_cols", bytes=GIB + 512 * 128 * 4, elements=N28))
    ops.append(dict(name="c4.full.sum", family="reduce_rows", bytes=GIB + 4, elements=N28))
    return ops


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi SM clock / throttle-reason samples (read only).  Sampling runs in the
    background; `stop(t0, t1)` keeps the samples whose timestamps fall inside [t0, t1]."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t0: float, t1: float):
        import datetime
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons, total = [], [], [], set(), 0
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                vals = (float(f[1]), float(f[2]), float(f[3]))
            except ValueError:
                continue
            total += 1
            if not (t0 - 0.02 <= ts <= t1 + 0.02):
                continue
            sm.append(vals[0]); smax.append(vals[1]); power.append(vals[2])
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"no samples inside the timed window ({total} outside)"]}
        return {"sm_mhz": float(np.median(sm)), "sm_min_mhz": float(min(sm)), "sm_max_mhz": float(max(smax)),
                "power_w_median": float(np.median(power)), "power_w_max": float(max(power)),
                "samples_in_window": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# CPU side: the oracle in kten-jvm's structure, on a bounded sample
# ----------------------------------------------------------------------------------------------
def cpu_sample_pass(sample_log2: int, tuned: bool = False):
    """One pass of the sweep on a 2^sample_log2-element sample with the CPU oracle:
    broadcast operands materialised, out-of-place maps single-threaded, in-place ops and
    axis aggregation on all host threads (what kten-jvm does).  `tuned`: every map on all
    host threads and no materialised broadcast operands -- the host's upper bound with the
    same arithmetic.  Returns (seconds, algorithmic bytes of the sample, per-op seconds)."""
    from kten_b200 import datagen as D
    from oracle import oracle as O
    n = 1 << sample_log2
    scale = n / N28
    a, b = D.uniform(n, 1, 0.1, 2.0), D.uniform(n, 2, 0.1, 2.0)
    rows3 = max(1, int(1024 * scale))
    a3 = D.normal(rows3 * 1024 * 256, 3, 0.0, 1.0)
    b3, c3 = D.uniform(1024, 4, 0.5, 2.0), D.uniform(rows3 * 256, 5, -1.0, 1.0)
    x4 = D.normal(n, 6, 0.0, 1.0, quantum=16.0)
    rows4, outer4 = n // 4096, max(1, n // (4096 * 128))
    per_op, total_bytes = {}, 0.0
    t_all = time.perf_counter()
    for spec in sweep_spec():
        name = spec["name"]
        t0 = time.perf_counter()
        if name.startswith("c2."):
            op = name[3:]
            if spec["family"] == "map2":
                O.binary_same({"plus": O.PLUS, "times": O.TIMES, "div": O.DIV, "pow": O.POW}[op], a, b, tuned=tuned)
            else:
                O.unary({"exp": O.EXP, "log": O.LOG, "tanh": O.TANH, "sigmoid": O.SIGMOID}[op], a, tuned=tuned)
        elif name == "c3.a*b":
            t3, _ = O.binary(O.TIMES, a3, [rows3, 1024, 256], b3, [1, 1024, 1], tuned=tuned)
        elif name == "c3.(a*b)+c":
            O.binary(O.PLUS, t3, [rows3, 1024, 256], c3, [rows3, 1, 256], tuned=tuned)
        elif name == "c3.a/b":
            O.binary(O.DIV, a3, [rows3, 1024, 256], b3, [1, 1024, 1], tuned=tuned)
        elif name.startswith("c4.last."):
            O.aggregate({"sum": O.SUM, "mean": O.MEAN, "max": O.MAX, "argmax": O.ARGMAX}[name[8:]], x4, rows4, 4096, 1, mode=0)
        elif name.startswith("c4.mid."):
            O.aggregate({"sum": O.SUM, "max": O.MAX}[name[7:]], x4[:outer4 * 4096 * 128], outer4, 4096, 128, mode=0)
        else:
            O.reduce_all(O.SUM, x4, mode=0)
        per_op[name] = time.perf_counter() - t0
        total_bytes += spec["bytes"] * scale
    return time.perf_counter() - t_all, total_bytes, per_op


def run_reference_arm(args):
    """`--impl reference`: the reference's own CPU algorithm (kten-jvm restated in C++, the
    JVM itself cannot run here) on the host cores, same metric and config."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle as O
    sample_log2 = args.cpu_sample_log2
    for _ in range(args.warmup):
        cpu_sample_pass(min(sample_log2, 20))
    secs, nbytes = 0.0, 0.0
    for _ in range(args.steps):
        s, b, _ = cpu_sample_pass(sample_log2)
        secs += s; nbytes += b
    gbs = nbytes / secs / 1e9
    line = {
        "impl": "reference", "metric": "HBM GB/s (algorithmic bytes / time), broadcast elementwise + axis reduce sweep",
        "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C2+C3+C4 sweep (contiguous elementwise, broadcast binary, axis/full reductions)",
                   "sample": f"2^{sample_log2} elements per operand (1/{N28 >> sample_log2} of the full size), same shapes ratio"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
                         "sample": f"each step = the sweep on 2^{sample_log2}-element operands; kten-jvm structure: broadcast operands "
                                   "materialised, out-of-place maps on one thread, in-place ops and axis aggregation on all threads"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "kten-jvm itself needs a JDK + Kotlin toolchain that is not in this image; this is its algorithm restated in C++ "
                "(oracle/kten_oracle.cpp), which is faster than the JVM original (no boxing, no per-element List allocation)",
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class GpuSweep:
    def __init__(self, device: int, rank: int, comm=None, collective=None):
        from kten_b200 import _lib as L
        from kten_b200 import datagen as D
        from kten_b200.tensor_operations import CUDATensorOperations
        self.L, self.D = L, D
        self.ops = CUDATensorOperations(device)
        self.lib, self.dev, self.rank, self.comm = self.ops.lib, device, rank, comm
        self.collective = collective             # object with allreduce_sum(raws), made once the ops exist (set_collective)
        first = rank * N28                       # this rank's shard of the N-times larger batch
        t0 = time.time()
        self.h_in = [self._pinned(N28), self._pinned(N28)]
        self.h_out = self._pinned(N28)
        mk = self.ops.createRaw
        # C2
        D.uniform(N28, 1, 0.1, 2.0, first=first, out=self.h_in[0]); self.a2 = mk([N28]); self._up(self.a2, self.h_in[0])
        D.uniform(N28, 2, 0.1, 2.0, first=first, out=self.h_in[1]); self.b2 = mk([N28]); self._up(self.b2, self.h_in[1])
        # C3
        D.normal(N28, 3, 0.0, 1.0, first=first, out=self.h_in[0]); self.a3 = mk([1024, 1024, 256]); self._up(self.a3, self.h_in[0])
        self.hb3 = D.uniform(1024, 4, 0.5, 2.0); self.b3 = mk([1, 1024, 1], self.hb3)
        self.hc3 = D.uniform(1024 * 256, 5, -1.0, 1.0, first=rank * 1024 * 256); self.c3 = mk([1024, 1, 256], self.hc3)
        self.t3 = mk([1024, 1024, 256])
        # C4
        D.normal(N28, 6, 0.0, 1.0, first=first, quantum=16.0, out=self.h_in[0]); self.x4 = mk([N28]); self._up(self.x4, self.h_in[0])
        self.out = mk([N28])
        self.small = mk([65536])
        self.full_sum_out = mk([1])                   # where the full sum lands (summed across the ranks in place)
        self.full_sum_e2e = mk([1])
        self.small_host = np.empty(65536, dtype=np.float32)
        self.ops.synchronize()
        self.setup_s = time.time() - t0
        self.h_state = None                       # which host data h_in currently holds

    def _pinned(self, n):
        p = C.POINTER(C.c_float)()
        self.L.check(self.lib.ktc_host_alloc(n, C.byref(p)))
        return np.ctypeslib.as_array(p, shape=(n,))

    def _up(self, raw, host, n=None):
        n = raw.size if n is None else n
        self.L.check(self.lib.ktc_h2d(raw.storeReference, 0, host.ctypes.data_as(C.c_void_p), n, 0))
        self.ops.synchronize()

    # ---- one op, inputs resident in HBM --------------------------------------------------------
    def launch(self, name):
        L, lib = self.L, self.lib
        ck = L.check
        a2, b2, out = self.a2.storeReference, self.b2.storeReference, self.out.storeReference
        if name.startswith("c2."):
            op = name[3:]
            if op in ("plus", "times", "div", "pow"):
                ck(lib.ktc_binary({"plus": L.PLUS, "times": L.TIMES, "div": L.DIV, "pow": L.POW}[op], out, a2, b2, N28))
            else:
                ck(lib.ktc_unary({"exp": L.EXP, "log": L.LOG, "tanh": L.TANH, "sigmoid": L.SIGMOID}[op], out, a2, N28))
        elif name.startswith("c3."):
            s3, n3 = L.shape_array([1024, 1024, 256]); sb, nb = L.shape_array([1, 1024, 1]); sc, nc = L.shape_array([1024, 1, 256])
            a3, b3, c3, t3 = self.a3.storeReference, self.b3.storeReference, self.c3.storeReference, self.t3.storeReference
            if name == "c3.a*b":
                ck(lib.ktc_binary_bcast(L.TIMES, t3, a3, s3, n3, b3, sb, nb))
            elif name == "c3.(a*b)+c":
                ck(lib.ktc_binary_bcast(L.PLUS, out, t3, s3, n3, c3, sc, nc))
            else:
                ck(lib.ktc_binary_bcast(L.DIV, out, a3, s3, n3, b3, sb, nb))
        elif name.startswith("c4.last."):
            ck(lib.ktc_reduce_axis({"sum": L.SUM, "mean": L.MEAN, "max": L.MAX, "argmax": L.ARGMAX}[name[8:]],
                                   self.small.storeReference, self.x4.storeReference, 65536, 4096, 1))
        elif name.startswith("c4.mid."):
            ck(lib.ktc_reduce_axis({"sum": L.SUM, "max": L.MAX}[name[7:]], self.small.storeReference, self.x4.storeReference, 512, 4096, 128))
        else:
            ck(lib.ktc_reduce_all(L.SUM, self.full_sum_out.storeReference, self.x4.storeReference, N28))
            if self.collective is not None:      # the one exchange step of the sharded path
                self.collective.allreduce_sum([self.full_sum_out])

    # ---- one op through the public API with HOST buffers (copies inside the timed region) -------
    CHUNK = 1 << 22          # 16 MiB pieces: upload of piece i+1, kernel of piece i and download of piece i-1 overlap

    def _views(self, raw, n_chunk, count):
        """Sub-range handles of `raw`, `count` pieces of `n_chunk` floats (created once, cached)."""
        key = (raw.storeReference, n_chunk)
        cache = self.__dict__.setdefault("_view_cache", {})
        if key not in cache:
            hs = []
            for i in range(count):
                h = C.c_uint64(0)
                self.L.check(self.lib.ktc_view(raw.storeReference, i * n_chunk, n_chunk, C.byref(h)))
                hs.append(h.value)
            cache[key] = hs
        return cache[key]

    def e2e_step(self, host_a, host_b):
        """One step of the sweep on pinned HOST operands through the C ABI.  Every distinct input of the step
        is uploaded once (a, b of the contiguous ops; the full-size operand and the small ones of the broadcast
        ops; the reduction input), in 16 MiB pieces; as a piece arrives every op that reads it runs on that piece
        and its result piece is downloaded, so upload, kernels and downloads of neighbouring pieces overlap
        (KTC_COPY_OVERLAP_UNFENCED: each device piece is written once per step, one fence per step).  Every
        op's result goes back to the host.  Returns (h2d bytes, d2h bytes)."""
        L, lib, ck = self.L, self.lib, self.L.check
        ck(lib.ktc_copy_fence(self.dev))
        OV = L.COPY_OVERLAP_UNFENCED
        CH = self.CHUNK
        nch = N28 // CH
        ptr = lambda h, off: C.c_void_p(h.ctypes.data + 4 * off)
        if not hasattr(self, "outs"):
            self.outs = [self.out] + [self.ops.createRaw([N28]) for _ in range(7)]      # one result buffer per op of a group
            self.smalls = [self.small] + [self.ops.createRaw([65536]) for _ in range(5)]
        h2d = d2h = 0
        # ---- contiguous elementwise: a, b -> plus times div pow (a, b), exp log tanh sigmoid (a) ----------------
        va, vb = self._views(self.a2, CH, nch), self._views(self.b2, CH, nch)
        vo = [self._views(o, CH, nch) for o in self.outs]
        bins, uns = (L.PLUS, L.TIMES, L.DIV, L.POW), (L.EXP, L.LOG, L.TANH, L.SIGMOID)
        for i in range(nch):
            ck(lib.ktc_h2d(va[i], 0, ptr(host_a, i * CH), CH, OV))
            ck(lib.ktc_h2d(vb[i], 0, ptr(host_b, i * CH), CH, OV))
            for k, code in enumerate(bins):
                ck(lib.ktc_binary(code, vo[k][i], va[i], vb[i], CH))
                ck(lib.ktc_d2h(ptr(self.h_out, i * CH), vo[k][i], 0, CH, OV))
            for k, code in enumerate(uns):
                ck(lib.ktc_unary(code, vo[4 + k][i], va[i], CH))
                ck(lib.ktc_d2h(ptr(self.h_out, i * CH), vo[4 + k][i], 0, CH, OV))
        h2d += 8 * N28; d2h += 8 * 4 * N28
        ck(lib.ktc_copy_fence(self.dev))                  # the next group reuses result buffers
        # ---- broadcast binary: a3 (+ b3, c3) -> a*b, (a*b)+c, a/b ----------------------------------------------
        rows = CH // (1024 * 256)                         # leading rows per piece
        s3, n3 = L.shape_array([rows, 1024, 256]); sb, nb = L.shape_array([1, 1024, 1]); sc, nc = L.shape_array([rows, 1, 256])
        v3, vt, vc = self._views(self.a3, CH, nch), self._views(self.t3, CH, nch), self._views(self.c3, rows * 256, nch)
        ck(lib.ktc_h2d(self.b3.storeReference, 0, ptr(self.hb3, 0), 1024, OV))
        b3 = self.b3.storeReference
        for i in range(nch):
            ck(lib.ktc_h2d(v3[i], 0, ptr(host_a, i * CH), CH, OV))
            ck(lib.ktc_h2d(vc[i], 0, ptr(self.hc3, i * rows * 256), rows * 256, OV))
            ck(lib.ktc_binary_bcast(L.TIMES, vt[i], v3[i], s3, n3, b3, sb, nb))
            ck(lib.ktc_d2h(ptr(self.h_out, i * CH), vt[i], 0, CH, OV))
            ck(lib.ktc_binary_bcast(L.PLUS, vo[0][i], vt[i], s3, n3, vc[i], sc, nc))
            ck(lib.ktc_d2h(ptr(self.h_out, i * CH), vo[0][i], 0, CH, OV))
            ck(lib.ktc_binary_bcast(L.DIV, vo[1][i], v3[i], s3, n3, b3, sb, nb))
            ck(lib.ktc_d2h(ptr(self.h_out, i * CH), vo[1][i], 0, CH, OV))
        h2d += 4 * N28 + 4096 + (1 << 20); d2h += 3 * 4 * N28
        # ---- reductions: x -> last-axis sum mean max argmax, middle-axis sum max, full sum ----------------------
        vx = self._views(self.x4, CH, nch)
        r, o = CH // 4096, CH // (4096 * 128)
        last = (L.SUM, L.MEAN, L.MAX, L.ARGMAX)
        vs_last = [self._views(self.smalls[k], r, nch) for k in range(4)]
        vs_mid = [self._views(self.smalls[4 + k], o * 128, nch) for k in range(2)]
        for i in range(nch):
            ck(lib.ktc_h2d(vx[i], 0, ptr(host_a, i * CH), CH, OV))
            for k, code in enumerate(last):
                ck(lib.ktc_reduce_axis(code, vs_last[k][i], vx[i], r, 4096, 1))
            for k, code in enumerate((L.SUM, L.MAX)):
                ck(lib.ktc_reduce_axis(code, vs_mid[k][i], vx[i], o, 4096, 128))
        ck(lib.ktc_reduce_all(L.SUM, self.full_sum_e2e.storeReference, self.x4.storeReference, N28))
        if self.collective is not None:
            self.collective.allreduce_sum([self.full_sum_e2e])
        for k in range(6):
            ck(lib.ktc_d2h(ptr(self.small_host, 0), self.smalls[k].storeReference, 0, 65536, OV))
        ck(lib.ktc_d2h(ptr(self.small_host, 0), self.full_sum_e2e.storeReference, 0, 1, OV))
        h2d += 4 * N28; d2h += 4 * (6 * 65536 + 1)
        ck(lib.ktc_copy_fence(self.dev))                  # the step ends when its last download has landed
        return h2d, d2h

    def timer_start(self):
        self.L.check(self.lib.ktc_timer_start(self.dev))

    def timer_stop(self) -> float:
        ms = C.c_float(0)
        self.L.check(self.lib.ktc_timer_stop(self.dev, C.byref(ms)))
        return float(ms.value)


def run_sharded_graph(ops, lib, L, D, rank, world, collective, steps, warmup, dist, gpu_index=0):
    """The sharded autograd configuration: x[262144,1024] ~ U(-1,1) split by rows over the ranks
    (strong scaling: the global tensor is fixed), w[1,1024] ~ N(0,0.02), b[1024] = 0;
    loss = sum(sigmoid(x*w + b) pow 2), backward for w and b, partials all-reduced."""
    from kten_b200.sharded import ShardedSigmoidGraph, shard_rows
    rows, cols = 262144, 1024
    first, count = shard_rows(rows, world, rank)
    hx = D.uniform(count * cols, 0, -1.0, 1.0, stream=0, first=first * cols)
    hw = D.normal(cols, 0, 0.0, 0.02, stream=1)
    x = ops.createRaw([count, cols], hx)
    w = ops.createRaw([1, cols], hw)
    b = ops.createRawFill([cols], 0.0)
    del hx
    graph = ShardedSigmoidGraph(ops, x, w, b, collective)

    def one_step():
        with ops.garbageCollector():
            out = graph.step()
            graph.release_step()
        return out

    def timed(deferred, defer_sums=True):
        """`steps` steps, call by call (every raw-tensor call one library call) or with the elementwise
        calls deferred and fused (kten_b200.lazy); with defer_sums the sums wait as well and the loss and
        both gradients come out of one pass."""
        ops.lazy, ops.deferSums = deferred, defer_sums
        passes0 = ops.multiSinkEvaluations
        rec0 = ops._recorder.stats()
        ms = C.c_float(0)
        for _ in range(max(warmup, 3)):
            one_step()
        ops.synchronize()
        if dist is not None:
            dist.barrier()
        launches0 = lib.ktc_launch_count()
        L.check(lib.ktc_timer_start(ops.device))
        for _ in range(steps):
            one_step()
        L.check(lib.ktc_timer_stop(ops.device, C.byref(ms)))
        launches = lib.ktc_launch_count() - launches0
        rec1 = ops._recorder.stats()
        ops.lazy, ops.deferSums = False, True
        # the loss tensor of the last step was released with its graph; gw / gb are the Variables' gradients
        gw, gb = graph.w.gradient.toArray().reshape(-1), graph.b.gradient.toArray()
        t = float(ms.value)
        if dist is not None:
            import torch
            tt = torch.tensor([t], dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt[0])
        return {"ms_per_step": t / steps, "gelem_per_s": rows * cols / (t / steps) / 1e6,
                "kernel_launches_per_step": launches / steps,
                "multi_sink_passes_per_step": (ops.multiSinkEvaluations - passes0) / (steps + max(warmup, 3)),
                "updates_in_second_pass_per_step": (rec1["folded_updates"] - rec0["folded_updates"]) / (steps + max(warmup, 3)),
                "exchanges_in_second_pass_per_step": (rec1["folded_exchanges"] - rec0["folded_exchanges"]) / (steps + max(warmup, 3)),
                "grad_w_abs_sum": float(np.abs(gw).sum()), "grad_b_abs_sum": float(np.abs(gb).sum())}

    def timed_native(deferred):
        """The same steps issued by the compiled host (kten_b200/csrc/host/kten_host.cpp): the raw tensor and the
        autograd caller restated in C++, as fast as the JVM host the reference would bring."""
        from kten_b200.native_host import NativeShardedStep
        comm_handle = getattr(collective, "comm", 0) if world > 1 else 0
        if world > 1 and not comm_handle:
            return {"unavailable": "the compiled host exchanges through the peer-memory collective only"}
        ops.lazy = False
        native = NativeShardedStep(ops, x, w, b, deferred, comm_handle)
        try:
            native.run(max(warmup, 3))
            ops.synchronize()
            if dist is not None:
                dist.barrier()
            ms = C.c_float(0)
            launches0 = lib.ktc_launch_count()
            stats0 = ops._recorder.stats()
            t0 = time.perf_counter()
            L.check(lib.ktc_timer_start(ops.device))
            native.run(steps)
            host_s = time.perf_counter() - t0                   # the host is back before the device has finished
            L.check(lib.ktc_timer_stop(ops.device, C.byref(ms)))
            launches = lib.ktc_launch_count() - launches0
            stats1 = ops._recorder.stats()
            handles = native.run(1, results=True)
            gw = np.empty(cols, np.float32); gb = np.empty(cols, np.float32)
            L.check(lib.ktc_d2h(gw.ctypes.data_as(C.c_void_p), handles[1], 0, cols, 1))
            L.check(lib.ktc_d2h(gb.ctypes.data_as(C.c_void_p), handles[2], 0, cols, 1))
        finally:
            native.close()
        t = float(ms.value)
        if dist is not None:
            import torch
            tt = torch.tensor([t], dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt[0])
        return {"ms_per_step": t / steps, "gelem_per_s": rows * cols / (t / steps) / 1e6, "host_us_per_step": host_s / steps * 1e6,
                "kernel_launches_per_step": launches / steps,
                "multi_sink_passes_per_step": (stats1["multi_sink"] - stats0["multi_sink"]) / steps,
                "programs_compiled_in_timed_region": stats1["compiled"] - stats0["compiled"],
                "updates_in_second_pass_per_step": (stats1["folded_updates"] - stats0["folded_updates"]) / steps,
                "exchanges_in_second_pass_per_step": (stats1["folded_exchanges"] - stats0["folded_exchanges"]) / steps,
                "grad_w_abs_sum": float(np.abs(gw).sum()), "grad_b_abs_sum": float(np.abs(gb).sum())}

    eager = timed(False)
    single = timed(True, defer_sums=False)
    sampler = ClockSampler(gpu_index)                       # clocks of this block's own window: the two deferred runs
    sampler.start()
    time.sleep(0.3)
    t_window0 = time.time()
    fused = timed(True)
    try:
        native_fused = timed_native(True)
        clocks = sampler.stop(t_window0, time.time())
        native_eager = timed_native(False)
    except Exception as exc:                                # the Python host's figures stand on their own
        clocks = sampler.stop(t_window0, time.time())
        native_fused = native_eager = {"unavailable": str(exc)}
    for r in (x, w, b):
        r.release()
    res = {"workload": "x[262144,1024] row-sharded, loss = sum(sigmoid(x*w+b) pow 2), backward + all-reduce of (loss, gw, gb)",
           "scaling": "strong", "rows_per_gpu": count, "n_gpus": world, "steps": steps}
    # the same raw-tensor call sequence of kten's autograd in the backend's two execution modes; the headline
    # figures are those of the faster one (the deferred mode is bound by this Python host side once a rank's
    # shard takes less device time than building and compiling the step's expressions)
    best = min((fused, single, eager), key=lambda r: r["ms_per_step"])
    res.update(best)
    res["execution"] = ("deferred elementwise calls and sums, one pass with three sinks per step (ops.lazy, ops.deferSums)" if best is fused
                        else "deferred elementwise calls fused into one sum each (ops.lazy)" if best is single
                        else "call by call (every raw-tensor call one library call)")
    res["deferred"] = fused
    res["deferred_one_sum_per_pass"] = single
    res["call_by_call"] = eager
    # the same two modes with the host side in C++ (what a JVM host would cost); when it ran, its deferred figure is the headline
    res["compiled_host"] = {"deferred": native_fused, "call_by_call": native_eager}
    if "ms_per_step" in native_fused and native_fused["ms_per_step"] < res["ms_per_step"]:
        res.update({k: native_fused[k] for k in ("ms_per_step", "gelem_per_s", "kernel_launches_per_step", "multi_sink_passes_per_step",
                                                 "updates_in_second_pass_per_step", "exchanges_in_second_pass_per_step",
                                                 "grad_w_abs_sum", "grad_b_abs_sum")})
        res["execution"] = "deferred elementwise calls and sums, one pass with three sinks per step, issued by the compiled host (libkten_host.so)"
        res["host_us_per_step"] = native_fused["host_us_per_step"]
    # roofline of the step: a rank has to read its shard of x once (the fused lower bound of the configuration); the
    # time is the max over ranks.  The kernel is bound by instruction issue, not by HBM -- sigmoid's exp costs about 40
    # issue slots per element, a double operation taking two -- which is what this fraction shows.
    peak, peak_src = measured_peak()
    shard_bytes = float(count * cols * 4)
    achieved = shard_bytes / res["ms_per_step"] / 1e6
    res["gelem_per_s_per_gpu"] = res["gelem_per_s"] / world
    res["roofline"] = {"bound": "hbm", "kernel": "ktc_jit_kernel (one pass with three sinks) + k_combine_multi", "achieved": achieved, "peak": peak,
                       "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "algorithmic_bytes_per_step_per_gpu": shard_bytes,
                       "hbm_floor_ms": shard_bytes / peak / 1e6, "traffic": None,
                       "note": "strong scaling: efficiency at N GPUs = ms_per_step(N=1) / (N * ms_per_step(N)), both from this block"}
    res["clocks"] = clocks
    return res


def release_loss(loss):
    """Drops what a finished SoftmaxCrossEntropy step still holds -- the retained [1] output of the root and the
    unsqueezed targets -- so that a loop of steps returns every buffer to the pool (on the JVM the tensors' owner does
    this; left alone each step would take two small device allocations)."""
    loss.keepOutput, loss.freeOutput = False, True
    loss.releaseUnusedInGraph()
    loss.targets.getRawValue().release()


def timed_in_batches(ops, lib, L, fn, reps, batches=5):
    """ms per call of `fn` (run inside a collector scope), timed in `batches` batches of `reps` calls with device events:
    returns (fastest batch, median batch, launches per call).  These steps are issued by the Python host, whose time per
    step (0.2-0.5 ms) is of the order of the device time: a batch in which the host is disturbed measures the host, so
    the fastest batch is the device figure and the median is printed beside it."""
    ms = C.c_float(0)
    per = []
    l0 = lib.ktc_launch_count()
    m0 = ops.getMetrics()
    for _ in range(batches):
        ops.synchronize()
        L.check(lib.ktc_timer_start(ops.device))
        for _ in range(reps):
            with ops.garbageCollector():
                fn()
        L.check(lib.ktc_timer_stop(ops.device, C.byref(ms)))
        per.append(ms.value / reps)
    per.sort()
    m1 = ops.getMetrics()
    timed_in_batches.last_device_mallocs = (m1["allocCalls"] - m1["poolHits"]) - (m0["allocCalls"] - m0["poolHits"])
    return per[0], per[len(per) // 2], (lib.ktc_launch_count() - l0) / (reps * batches)


def run_other_ops(ops, lib, L, D, steps):
    """The raw-tensor ops beside the sweep (slices, permutes, gather / scatter, the remaining maps), timed the same
    way on 2^28-element tensors: GB/s of algorithmic bytes (inputs read once + output written once)."""
    n = N28
    G = float(1 << 30)
    ms = C.c_float(0)
    out = []
    x = ops.createRaw([16384, 16384], D.uniform(n, 11, 0.1, 2.0))
    idx_h = np.floor(D.uniform(n, 12, 0.0, 16384.0)).astype(np.float32)
    np.minimum(idx_h, 16383.0, out=idx_h)
    idx = ops.createRaw([16384, 16384], idx_h)
    rows_h = np.floor(D.uniform(262144, 13, 0.0, 262144.0)).astype(np.float32)
    np.minimum(rows_h, 262143.0, out=rows_h)
    rows = ops.createRaw([262144], rows_h)
    mask = ops.createRaw([1, 1024, 1], (D.uniform(1024, 14, 0.0, 1.0) > 0.5).astype(np.float32))
    del idx_h, rows_h
    x3, xr, xm = x.view([64, 4096, 1024]), x.view([262144, 1024]), x.view([1024, 1024, 256])
    left, right = x.narrow(1, 0, 8192), x.narrow(1, 8192, 8192)
    acc = ops.createRawFill([262144, 1024], 0.0)
    cases = [
        ("transpose [16384,16384]", 2 * G, lambda: x.transpose(0, 1)),
        ("permute [64,4096,1024] -> (2,0,1)", 2 * G, lambda: x3.permute([2, 0, 1])),
        ("permute [64,4096,1024] -> (1,0,2)", 2 * G, lambda: x3.permute([1, 0, 2])),
        ("narrow [16384,16384] -> [16384,8192]", G, lambda: x.narrow(1, 4096, 8192)),
        ("concat 2 x [16384,8192] on axis 1", 2 * G, lambda: ops.concat(1, [left, right])),
        ("gather axis 1, index [16384,16384]", 3 * G, lambda: x.gather(1, idx)),
        ("indexSelect 262144 rows of [262144,1024]", 2 * G, lambda: xr.indexSelect(0, rows)),
        ("indexAdd 262144 rows into [262144,1024]", 3 * G, lambda: acc.indexAdd(0, rows, xr)),
        ("maskedFill [1024,1024,256], mask [1,1024,1]", 2 * G, lambda: xm.maskedFill(mask, 0.0)),
        ("sqrt", 2 * G, lambda: x.sqrt()),
        ("sin", 2 * G, lambda: x.sin()),
        ("eq (tensor, tensor)", 3 * G, lambda: x.eq(idx)),
        # tensor (op) scalar and the in-place forms (JVMRawTensor.kt:112-136): 8 B / element, and 12 B / element for a += b
        ("times (tensor, scalar)", 2 * G, lambda: x.times(1.5)),
        ("pow (scalar, tensor)", 2 * G, lambda: ops.pow(1.5, x)),
        ("timesAssign (scalar), in place", 2 * G, lambda: acc.timesAssign(0.999)),
        ("plusAssign (tensor), in place", 3 * G, lambda: acc.plusAssign(xr)),
        # the broadcast-gradient sum-to-shape (mayUnexpand, Utils.kt:14-41) in one call: the config-5 shapes, and the
        # two-axis shape of the plumbing graph scaled up ([32,64,128] -> [64,1] there)
        ("sumToShape [262144,1024] -> [1,1024]", G + 4096, lambda: xr.sumToShape([1, 1024])),
        ("sumToShape [262144,1024] -> [1024]", G + 4096, lambda: xr.sumToShape([1024])),
        ("sumToShape [1024,1024,256] -> [1024,1]", G + 4096, lambda: xm.sumToShape([1024, 1])),
    ]
    reps = max(2, min(steps, 10))
    for name, nbytes, fn in cases:
        with ops.garbageCollector():
            fn()
        ops.synchronize()
        L.check(lib.ktc_timer_start(ops.device))
        for _ in range(reps):
            with ops.garbageCollector():
                fn()
        L.check(lib.ktc_timer_stop(ops.device, C.byref(ms)))
        per = ms.value / reps
        out.append({"name": name, "ms": round(per, 4), "gbs": round(nbytes / per / 1e6, 1)})
    for r in (x3, xr, xm, left, right, acc, idx, rows, mask):
        r.release()
    # SoftmaxCrossEntropy forward + backward (functions/nn/SoftmaxCrossEntropy.kt) on [131072, 2048] logits through the
    # autograd caller, call by call and with elementwise calls and row sums deferred; algorithmic bytes: the logits
    # read once, their gradient written once
    from kten_b200 import autograd as AG
    logits = AG.Variable(ops, x.view([131072, 2048]))
    targets = AG.NoGradVariable(ops, ops.createRaw([131072], np.floor(D.uniform(131072, 15, 0.0, 2047.99)).astype(np.float32)))

    def xent():
        logits.zeroGrad()
        loss = logits.softmaxCrossEntropy(targets)
        loss.backward()
        logits.gradient.storeReference                      # gradient and loss in memory: nothing of the step is left pending
        loss.getRawValue().storeReference
        release_loss(loss)

    for mode, label in ((False, "call by call"), (True, "deferred")):
        ops.lazy = mode
        try:
            for _ in range(4):                              # the buffer pool settles over the first steps
                with ops.garbageCollector():
                    xent()
            per, med, launches = timed_in_batches(ops, lib, L, xent, max(2, reps // 2))
        finally:
            ops.lazy = False
        out.append({"name": f"softmaxCrossEntropy [131072,2048] forward + backward, {label}", "ms": round(per, 4), "ms_median_batch": round(med, 4),
                    "gbs": round(2 * G / per / 1e6, 1), "launches": launches})
    logits.gradient.release()
    logits.getRawValue().release()
    targets.getRawValue().release()
    x.release()

    # batch normalisation of [256, 64, 128, 128] along axis 1 (training: statistics, running averages, scale and shift) and
    # its backward, and nearest-neighbour upsampling by 2 with its gradient: compositions of recorded raw-tensor calls
    # (kten_b200/nn.py).  Bytes: what must cross HBM when every pass reads its operands once -- forward x three times + out,
    # backward x and gradOut twice + gradIn -- i.e. the passes the reference itself makes.
    shape, channels = [256, 64, 128, 128], 64
    n = 256 * 64 * 128 * 128
    bx = ops.createRaw(shape, D.normal(n, 21, 0.0, 1.0))
    bgo = ops.createRaw(shape, D.normal(n, 22, 0.0, 1.0))
    gam, bet = ops.createRaw([channels], D.uniform(channels, 23, 0.5, 1.5)), ops.createRaw([channels], D.uniform(channels, 24, -0.5, 0.5))
    rmean, rvar = ops.createRawFill([channels], 0.0), ops.createRawFill([channels], 1.0)
    bn = ops.batchNorm(1, 0.1, 1e-3, True)

    def bn_step():
        o, m, sd = bn.calculateOutput(bx, rmean, rvar, gam, bet)
        gi, gg, gb = bn.calculateGrads(bx, rmean, rvar, m, sd, gam, bgo, True, True, True)
        for t in (o, gi, gg, gb):
            t.storeReference

    up = ops.upsample("NEAREST", 2)
    ux = ops.createRaw([256, 64, 64, 64], D.normal(n // 4, 25, 0.0, 1.0))

    def up_step():
        o = up.upsample(ux)
        up.calculateGrad(o, [256, 64, 64, 64]).storeReference

    # spatial pooling of [256, 64, 128, 128] with its gradient (ktc_pool.cu).  Bytes: input read, result (and, for max, the
    # winners' positions) written; gradOut (and the positions) read, gradIn written
    from kten_b200.nn import PoolingOptions, PoolingType
    pools = {"max 2x2 / 2": ops.spatialPooling((2, 2), (0, 0), (2, 2), (1, 1), PoolingOptions(PoolingType.MAX)),
             "max 3x3 / 2 pad 1": ops.spatialPooling((3, 3), (1, 1), (2, 2), (1, 1), PoolingOptions(PoolingType.MAX)),
             "avg 2x2 / 2": ops.spatialPooling((2, 2), (0, 0), (2, 2), (1, 1), PoolingOptions(PoolingType.AVG))}

    def pool_step(op):
        def step():
            o, idx = op.updateOutput(bx)
            op.calculateGradInput(bx, o, idx).storeReference
        return step

    pool_lines = [(f"spatialPooling {k} of [256,64,128,128] + gradient", pool_step(op), (3.0 if k.startswith("max") else 2.5) * 4.0 * n) for k, op in pools.items()]
    for name, fn, nbytes in [("batchNorm [256,64,128,128] axis 1, training forward + backward", bn_step, 9 * 4.0 * n),
                             ("upsample2d nearest x2 of [256,64,64,64] + gradient", up_step, (0.25 + 1 + 1 + 0.25) * 4.0 * n)] + pool_lines:
        for _ in range(3):
            with ops.garbageCollector():
                fn()
        per, med, launches = timed_in_batches(ops, lib, L, fn, max(2, reps // 2))
        out.append({"name": name, "ms": round(per, 4), "ms_median_batch": round(med, 4), "gbs": round(nbytes / per / 1e6, 1), "launches": launches})
    for t in (bx, bgo, gam, bet, rmean, rvar, ux):
        t.release()
    return out


def init_distributed(n_gpus):
    """(rank, world, local_rank, dist module or None).  torch.distributed is plumbing only:
    rendezvous, the barrier and the max over ranks."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 0, 1, 0, None
    import torch
    import torch.distributed as dist
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    torch.cuda.set_device(local)
    dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    return rank, world, local, dist


def make_comm(lib, L, dist, rank, world, local):
    ident = C.create_string_buffer(L.COMM_ID_BYTES)
    if rank == 0:
        L.check(lib.ktc_comm_unique_id(ident))
    box = [bytes(ident.raw)]
    dist.broadcast_object_list(box, src=0)
    comm = C.c_uint64(0)
    L.check(lib.ktc_comm_init_rank(local, world, rank, box[0], C.byref(comm)))
    return comm.value


def run_gpu_arm(args):
    # Libraries underneath (NCCL's version banner, for one) write to stdout; the contract is ONE
    # JSON line there, so everything but that line goes to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    rank, world, local, dist = init_distributed(args.gpus)
    from kten_b200 import _lib as L
    lib = L.load()
    n = C.c_int(0)
    L.check(lib.ktc_init(C.byref(n)))
    comm = make_comm(lib, L, dist, rank, world, local) if dist is not None else None
    sweep = GpuSweep(local, rank, comm)
    collective, collective_name = None, "none (one rank)"
    if dist is not None:
        from kten_b200.sharded import NcclCollective, PeerMemoryCollective
        if args.collective == "p2p":
            def exchange(mine):
                everyone = [None] * world
                dist.all_gather_object(everyone, mine)
                return everyone
            try:
                collective = PeerMemoryCollective(sweep.ops, world, rank, exchange, dist.barrier)
                collective_name = "one kernel per rank over peer memory (ktc_p2p_allreduce_sum)"
            except Exception as exc:                      # e.g. CUDA IPC not permitted between these processes
                sys.stderr.write(f"peer-memory collective unavailable ({exc}); using NCCL\n")
        agree = [None] * world
        dist.all_gather_object(agree, collective is not None)
        if not all(agree):                                # every rank must take the same path
            if collective is not None:
                collective.close(barrier=False)           # nothing was exchanged yet; the ranks that failed are not waiting
            collective = None
        if collective is None:
            collective = NcclCollective(sweep.ops, comm)
            collective_name = "pack + NCCL all-reduce + unpack (ktc_allreduce_sum)"
    sweep.collective = collective
    spec = sweep_spec()
    names = [s["name"] for s in spec]
    step_bytes = float(sum(s["bytes"] for s in spec))

    def barrier():
        sweep.ops.synchronize()
        if dist is not None:
            dist.barrier()

    def run_step():
        for nm in names:
            sweep.launch(nm)

    for _ in range(max(args.warmup, 3)):
        run_step()
    barrier()
    if hasattr(collective, "check"):
        # the warm-up steps went through the peer-memory exchange: if any rank saw a wait run out, every rank
        # switches to the NCCL path before anything is timed
        try:
            collective.check()
            healthy = True
        except TimeoutError:
            healthy = False
        verdicts = [None] * world
        dist.all_gather_object(verdicts, healthy)
        if not all(verdicts):
            collective.close()
            collective = NcclCollective(sweep.ops, comm)
            collective_name = "pack + NCCL all-reduce + unpack (ktc_allreduce_sum); the peer-memory exchange timed out in warm-up"
            sweep.collective = collective
            barrier()

    # ---- timed region: exactly K steps, device-timed on the launching stream ----------------------
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.5)
    launches0 = lib.ktc_launch_count()
    barrier()
    t_window0 = time.time()
    sweep.timer_start()
    for _ in range(args.steps):
        run_step()
    step_ms_total = sweep.timer_stop()
    barrier()
    launches = lib.ktc_launch_count() - launches0

    # ---- per-op durations, same inputs, same clocks window (events around K launches of each op) --
    per_op = []
    for s in spec:
        sweep.launch(s["name"])
        sweep.timer_start()
        for _ in range(args.steps):
            sweep.launch(s["name"])
        ms = sweep.timer_stop() / args.steps
        per_op.append(dict(name=s["name"], family=s["family"], ms=ms, gbs=s["bytes"] / ms / 1e6,
                           gelem_s=s["elements"] / ms / 1e6))
    sweep.ops.synchronize()
    clocks = sampler.stop(t_window0, time.time())

    # ---- end to end: host buffers, copies inside the timed region ----------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    D = sweep.D
    first = rank * N28
    host_sets = {}
    D.uniform(N28, 1, 0.1, 2.0, first=first, out=sweep.h_in[0]); D.uniform(N28, 2, 0.1, 2.0, first=first, out=sweep.h_in[1])
    h2d = d2h = 0
    sweep.e2e_step(sweep.h_in[0], sweep.h_in[1])          # untimed: result buffers, piece handles, first-touch of the pinned ranges
    barrier()
    sweep.timer_start()
    t_wall = time.perf_counter()
    for _ in range(e2e_steps):
        bi, bo = sweep.e2e_step(sweep.h_in[0], sweep.h_in[1])
        h2d += bi; d2h += bo
    e2e_ms = sweep.timer_stop()
    e2e_wall = time.perf_counter() - t_wall
    barrier()

    # ---- the sharded autograd graph (strong scaling over the same ranks) ---------------------------
    sharded = None
    if args.sharded_graph:
        for r in [sweep.a2, sweep.b2, sweep.a3, sweep.t3, sweep.x4] + getattr(sweep, "outs", [sweep.out]):
            r.release()                               # hand the sweep's buffers back to the pool first
        L.check(lib.ktc_pool_trim(local))
        sharded = run_sharded_graph(sweep.ops, lib, L, D, rank, world, collective, max(args.steps, 20), args.warmup, dist, local)
        sharded["collective"] = collective_name

    other_ops = None
    if args.other_ops and rank == 0 and world == 1:
        if not args.sharded_graph:
            for r in [sweep.a2, sweep.b2, sweep.a3, sweep.t3, sweep.x4] + getattr(sweep, "outs", [sweep.out]):
                r.release()
        L.check(lib.ktc_pool_trim(local))
        other_ops = run_other_ops(sweep.ops, lib, L, D, args.steps)

    collective_error = None
    if hasattr(collective, "check"):
        try:
            collective.check()
        except TimeoutError as exc:
            collective_error = str(exc)

    # ---- max over ranks -----------------------------------------------------------------------------
    if dist is not None:
        import torch
        t = torch.tensor([step_ms_total, e2e_ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms_total, e2e_ms = float(t[0]), float(t[1])
    ms_per_step = step_ms_total / args.steps
    value = world * step_bytes / (ms_per_step * 1e6)
    e2e_value = world * step_bytes * e2e_steps / (e2e_ms * 1e6)

    peak, peak_src = measured_peak()
    fam_time = {}
    for p in per_op:
        fam_time[p["family"]] = fam_time.get(p["family"], 0.0) + p["ms"]
    top_family = max(fam_time, key=fam_time.get)
    fam_ops = [(p, s) for p, s in zip(per_op, spec) if p["family"] == top_family]
    fam_bytes = sum(s["bytes"] for _, s in fam_ops) / len(fam_ops)
    fam_ms = sum(p["ms"] for p, _ in fam_ops) / len(fam_ops)
    achieved = fam_bytes / fam_ms / 1e6
    kernel_names = {"map2": "k_map2_vec", "map1": "k_map1_vec", "bcast": "k_bcast3", "reduce_rows": "k_rows_warp", "reduce_cols": "k_cols_warp"}
    traffic, traffic_detail = load_traffic(kernel_names[top_family])

    line = {
        "metric": "HBM GB/s (algorithmic bytes / time), broadcast elementwise + axis reduce sweep",
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C2+C3+C4 sweep (contiguous elementwise, broadcast binary, axis/full reductions), one shard per GPU",
                   "elements_per_operand": N28, "ops_per_step": len(names), "algorithmic_bytes_per_step_per_gpu": step_bytes,
                   "l2": "inputs larger than L2 (every operand >= 1 GiB, L2 is 126 MB)", "parallelism": f"batch-sharded x{world}", "collective": collective_name},
        "frac_of_measured_peak": value / world / peak, "frac_of_nominal_8TBs": value / world / NOMINAL_HBM_GBS,
        "gelem_per_s": world * sum(s["elements"] for s in spec) / (ms_per_step * 1e6),
        "gpu_launches": int(launches),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d // e2e_steps, "d2h_bytes_per_step": d2h // e2e_steps,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "wall_ms_per_step": 1e3 * e2e_wall / e2e_steps,
                "h2d_gbs_per_gpu": h2d / (e2e_ms * 1e6), "d2h_gbs_per_gpu": d2h / (e2e_ms * 1e6),      # both directions run for the whole step
                "note": "pinned host operands: every distinct input of the step is uploaded once (ktc_h2d), every op's result is "
                        "downloaded (ktc_d2h), as a pipeline of 16 MiB pieces (KTC_COPY_OVERLAP_UNFENCED, one fence per step: "
                        "uploads, kernels and downloads of neighbouring pieces overlap); bound by the device-to-host link"},
        "roofline": {"bound": "hbm", "kernel": kernel_names[top_family], "ops": [p["name"] for p, _ in fam_ops],
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                     "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "traffic": traffic, "traffic_detail": traffic_detail,
                     "algorithmic_bytes_per_launch": fam_bytes, "ms_per_launch": fam_ms,
                     "share_of_step": fam_time[top_family] / sum(fam_time.values())},
        "per_op": [{"name": p["name"], "ms": round(p["ms"], 4), "gbs": round(p["gbs"], 1), "frac_measured": round(p["gbs"] / peak, 3),
                    "frac_nominal": round(p["gbs"] / NOMINAL_HBM_GBS, 3)} for p in per_op],
        "clocks": clocks,
        "setup_s": round(sweep.setup_s, 1),
    }
    if collective_error is not None:
        line["collective_error"] = collective_error
    if sharded is not None:
        line["sharded_graph"] = sharded
    if other_ops is not None:
        for o in other_ops:
            o["frac_measured"] = round(o["gbs"] / peak, 3)
        line["other_ops"] = other_ops
    if rank == 0:
        if args.cpu_baseline:
            secs, nbytes, _ = cpu_sample_pass(args.cpu_sample_log2)
            tuned_secs, tuned_bytes, _ = cpu_sample_pass(args.cpu_sample_log2, tuned=True)
            from oracle import oracle as O
            line["cpu_baseline"] = {"value": nbytes / secs / 1e9, "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
                                    "sample": f"the same sweep on 2^{args.cpu_sample_log2}-element operands ({secs:.1f} s), CPU oracle in "
                                              "kten-jvm's structure (broadcast operands materialised, out-of-place maps single-threaded, "
                                              "in-place ops and axis aggregation on all host threads)",
                                    "tuned": {"value": tuned_bytes / tuned_secs / 1e9, "unit": "GB/s", "cores": O.num_threads(),
                                              "sample": f"same sample ({tuned_secs:.1f} s), every elementwise map on all host threads: the "
                                                        "upper bound of what the host can do with the same algorithm"}}
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        if hasattr(collective, "close"):
            collective.close()
        if comm is not None:
            lib.ktc_comm_destroy(comm)
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_single_case(args):
    """`--case NAME --log2n L --reps R`: launch one op of the sweep R times on 2^L-element
    operands (same shapes ratio as the full sweep).  This is the small, self-terminating
    workload the ncu captures under profiles/ are taken on; it prints the op's GB/s."""
    from kten_b200 import _lib as L
    from kten_b200 import datagen as D
    from kten_b200.tensor_operations import CUDATensorOperations
    ops = CUDATensorOperations(0)
    lib = ops.lib
    n = 1 << args.log2n
    scale = n / N28
    name = args.case
    if name == "c5.graph_native":
        # the same step issued by the compiled host (libkten_host.so): deferred, one pass with three sinks
        from kten_b200.native_host import NativeShardedStep
        cols = 1024
        rows = max(1, n // cols)
        x = ops.createRaw([rows, cols], D.uniform(rows * cols, 0, -1.0, 1.0))
        w = ops.createRaw([1, cols], D.normal(cols, 0, 0.0, 0.02, stream=1))
        b = ops.createRawFill([cols], 0.0)
        host = NativeShardedStep(ops, x, w, b, lazy=True)
        host.run(3)
        ops.synchronize()
        l0 = lib.ktc_launch_count()
        L.check(lib.ktc_timer_start(0))
        host.run(args.reps)
        ms = C.c_float(0)
        L.check(lib.ktc_timer_stop(0, C.byref(ms)))
        print(json.dumps({"case": name, "elements": rows * cols, "ms": ms.value / args.reps,
                          "launches_per_step": (lib.ktc_launch_count() - l0) / args.reps}))
        host.close()
        return 0
    if name in ("c5.graph_eager", "c5.graph_deferred", "c5.graph_deferred_one_sum"):
        # the sharded-graph step on one device with n = rows * 1024 elements of x
        from kten_b200.sharded import ShardedSigmoidGraph
        cols = 1024
        rows = max(1, n // cols)
        x = ops.createRaw([rows, cols], D.uniform(rows * cols, 0, -1.0, 1.0))
        w = ops.createRaw([1, cols], D.normal(cols, 0, 0.0, 0.02, stream=1))
        b = ops.createRawFill([cols], 0.0)
        graph = ShardedSigmoidGraph(ops, x, w, b)
        ops.lazy = "deferred" in name
        ops.deferSums = not name.endswith("one_sum")         # one pass with three sinks, or one sum per pass

        def step():
            with ops.garbageCollector():
                graph.step()
                graph.release_step()

        for _ in range(3):
            step()
        ops.synchronize()
        l0 = lib.ktc_launch_count()
        L.check(lib.ktc_timer_start(0))
        for _ in range(args.reps):
            step()
        ms = C.c_float(0)
        L.check(lib.ktc_timer_stop(0, C.byref(ms)))
        print(json.dumps({"case": name, "elements": rows * cols, "ms": ms.value / args.reps,
                          "launches_per_step": (lib.ktc_launch_count() - l0) / args.reps}))
        return 0
    if name in ("x.softmax_eager", "x.softmax_deferred"):
        # SoftmaxCrossEntropy forward + backward on [n / 2048, 2048] logits through the autograd caller
        from kten_b200 import autograd as AG
        cols = args.cols
        rows = max(1, n // cols)
        logits = AG.Variable(ops, ops.createRaw([rows, cols], D.uniform(rows * cols, 11, 0.1, 2.0)))
        targets = AG.NoGradVariable(ops, ops.createRaw([rows], np.floor(D.uniform(rows, 15, 0.0, cols - 0.01)).astype(np.float32)))
        ops.lazy = name.endswith("deferred")

        def xent_unscoped():
            logits.zeroGrad()
            loss = logits.softmaxCrossEntropy(targets)
            loss.backward()
            logits.gradient.storeReference                  # gradient and loss in memory: nothing of the step is left pending
            loss.getRawValue().storeReference
            release_loss(loss)

        def xent():
            with ops.garbageCollector():
                xent_unscoped()

        for _ in range(4):                                  # the buffer pool settles over the first steps
            xent()
        per, med, launches = timed_in_batches(ops, lib, L, xent_unscoped, args.reps)
        print(json.dumps({"case": name, "elements": rows * cols, "ms": per, "ms_median_batch": med, "gbs": 2 * 4.0 * rows * cols / per / 1e6,
                          "launches_per_step": launches, "device_mallocs_in_timed_region": timed_in_batches.last_device_mallocs}))
        return 0
    if name in ("x.maxpool", "x.maxpool3", "x.avgpool"):
        # spatial pooling of [n / 2^20, 64, 128, 128] with its gradient
        from kten_b200.nn import PoolingOptions, PoolingType
        imgs = max(1, n >> 20)
        shape, vol = [imgs, 64, 128, 128], imgs << 20
        px = ops.createRaw(shape, D.normal(vol, 21, 0.0, 1.0))
        op = {"x.maxpool": ops.spatialPooling((2, 2), (0, 0), (2, 2), (1, 1), PoolingOptions(PoolingType.MAX)),
              "x.maxpool3": ops.spatialPooling((3, 3), (1, 1), (2, 2), (1, 1), PoolingOptions(PoolingType.MAX)),
              "x.avgpool": ops.spatialPooling((2, 2), (0, 0), (2, 2), (1, 1), PoolingOptions(PoolingType.AVG))}[name]

        def fn():
            o, idx = op.updateOutput(px)
            op.calculateGradInput(px, o, idx).storeReference
        nbytes = (2.5 if name == "x.avgpool" else 3.0) * 4.0 * vol
        for _ in range(3):
            with ops.garbageCollector():
                fn()
        per, med, launches = timed_in_batches(ops, lib, L, fn, args.reps)
        print(json.dumps({"case": name, "elements": vol, "ms": per, "ms_median_batch": med, "gbs": nbytes / per / 1e6, "launches_per_step": launches}))
        return 0
    if name in ("x.batchnorm", "x.upsample"):
        # batch norm (training forward + backward) of [n / 2^20, 64, 128, 128] along axis 1; upsampling by 2 with its gradient
        imgs = max(1, n >> 20)
        if name == "x.batchnorm":
            shape = [imgs, 64, 128, 128]
            vol = imgs << 20
            bx, bgo = ops.createRaw(shape, D.normal(vol, 21, 0.0, 1.0)), ops.createRaw(shape, D.normal(vol, 22, 0.0, 1.0))
            gam, bet = ops.createRaw([64], D.uniform(64, 23, 0.5, 1.5)), ops.createRaw([64], D.uniform(64, 24, -0.5, 0.5))
            rmean, rvar = ops.createRawFill([64], 0.0), ops.createRawFill([64], 1.0)
            bn = ops.batchNorm(1, 0.1, 1e-3, True)

            def fn():
                o, m, sd = bn.calculateOutput(bx, rmean, rvar, gam, bet)
                for t in (o,) + bn.calculateGrads(bx, rmean, rvar, m, sd, gam, bgo, True, True, True):
                    t.storeReference
            nbytes = 9 * 4.0 * vol
        else:
            shape = [imgs, 64, 64, 64]
            vol = imgs << 18
            ux = ops.createRaw(shape, D.normal(vol, 25, 0.0, 1.0))
            up = ops.upsample("NEAREST", 2)

            def fn():
                up.calculateGrad(up.upsample(ux), shape).storeReference
            nbytes = 10 * 4.0 * vol
        for _ in range(3):
            with ops.garbageCollector():
                fn()
        per, med, launches = timed_in_batches(ops, lib, L, fn, args.reps)
        print(json.dumps({"case": name, "elements": vol, "ms": per, "ms_median_batch": med, "gbs": nbytes / per / 1e6, "launches_per_step": launches}))
        return 0
    if name.startswith("x."):
        # data-movement ops beside the sweep, on a [rows, 4096] tensor of n elements
        cols = 4096
        rows = max(1, n // cols)
        x = ops.createRaw([rows, cols], D.uniform(rows * cols, 11, 0.1, 2.0))
        pick = np.minimum(np.floor(D.uniform(rows, 13, 0.0, float(rows))), rows - 1).astype(np.float32)
        ridx = ops.createRaw([rows], pick)
        acc = ops.createRawFill([rows, cols], 0.0)
        fns = {"x.transpose": (lambda: x.transpose(0, 1), 2), "x.permute_rows": (lambda: x.view([rows // 64, 64, cols]).permute([1, 0, 2]), 2),
               "x.narrow": (lambda: x.narrow(1, 1024, 2048), 1), "x.index_select": (lambda: x.indexSelect(0, ridx), 2),
               "x.index_add": (lambda: acc.indexAdd(0, ridx, x), 3)}
        if name == "x.gather":
            gidx = ops.createRaw([rows, cols], np.minimum(np.floor(D.uniform(rows * cols, 12, 0.0, float(cols))), cols - 1).astype(np.float32))
            fns[name] = (lambda: x.gather(1, gidx), 3)
        fn, volumes = fns[name]
        with ops.garbageCollector():
            fn()
        ops.synchronize()
        L.check(lib.ktc_timer_start(0))
        for _ in range(args.reps):
            with ops.garbageCollector():
                fn()
        ms = C.c_float(0)
        L.check(lib.ktc_timer_stop(0, C.byref(ms)))
        per = ms.value / args.reps
        print(json.dumps({"case": name, "elements": rows * cols, "ms": per, "gbs": volumes * 4.0 * rows * cols / per / 1e6}))
        return 0
    spec = {s_["name"]: s_ for s_ in sweep_spec()}[name]
    mk = ops.createRaw
    out = mk([n])
    small = mk([max(1, n // 4096)])
    if name.startswith("c2."):
        a, b = mk([n], D.uniform(n, 1, 0.1, 2.0)), mk([n], D.uniform(n, 2, 0.1, 2.0))
        op = name[3:]
        if op in ("plus", "times", "div", "pow"):
            code = {"plus": L.PLUS, "times": L.TIMES, "div": L.DIV, "pow": L.POW}[op]
            fn = lambda: L.check(lib.ktc_binary(code, out.storeReference, a.storeReference, b.storeReference, n))
        else:
            code = {"exp": L.EXP, "log": L.LOG, "tanh": L.TANH, "sigmoid": L.SIGMOID}[op]
            fn = lambda: L.check(lib.ktc_unary(code, out.storeReference, a.storeReference, n))
    elif name.startswith("c3."):
        rows = max(1, int(1024 * scale))
        a = mk([rows, 1024, 256], D.normal(n, 3, 0.0, 1.0))
        b = mk([1, 1024, 1], D.uniform(1024, 4, 0.5, 2.0))
        c = mk([rows, 1, 256], D.uniform(rows * 256, 5, -1.0, 1.0))
        s3, n3 = L.shape_array([rows, 1024, 256]); sb, nb = L.shape_array([1, 1024, 1]); sc, nc = L.shape_array([rows, 1, 256])
        if name == "c3.a*b":
            fn = lambda: L.check(lib.ktc_binary_bcast(L.TIMES, out.storeReference, a.storeReference, s3, n3, b.storeReference, sb, nb))
        elif name == "c3.(a*b)+c":
            fn = lambda: L.check(lib.ktc_binary_bcast(L.PLUS, out.storeReference, a.storeReference, s3, n3, c.storeReference, sc, nc))
        else:
            fn = lambda: L.check(lib.ktc_binary_bcast(L.DIV, out.storeReference, a.storeReference, s3, n3, b.storeReference, sb, nb))
    else:
        x = mk([n], D.normal(n, 6, 0.0, 1.0, quantum=16.0))
        if name.startswith("c4.last."):
            code = {"sum": L.SUM, "mean": L.MEAN, "max": L.MAX, "argmax": L.ARGMAX}[name[8:]]
            fn = lambda: L.check(lib.ktc_reduce_axis(code, small.storeReference, x.storeReference, n // 4096, 4096, 1))
        elif name.startswith("c4.mid."):
            code = {"sum": L.SUM, "max": L.MAX}[name[7:]]
            fn = lambda: L.check(lib.ktc_reduce_axis(code, small.storeReference, x.storeReference, max(1, n // (4096 * 128)), 4096, 128))
        else:
            fn = lambda: L.check(lib.ktc_reduce_all(L.SUM, small.storeReference, x.storeReference, n))
    fn()
    ops.synchronize()
    L.check(lib.ktc_timer_start(0))
    for _ in range(args.reps):
        fn()
    ms = C.c_float(0)
    L.check(lib.ktc_timer_stop(0, C.byref(ms)))
    per = ms.value / args.reps
    print(json.dumps({"case": name, "elements": n, "ms": per, "gbs": spec["bytes"] * scale / per / 1e6}))
    return 0


# dram__bytes_read.sum and dram__bytes_write.sum of one launch of each kernel family, from ncu captures of 2^26-element
# cases (a full-size launch is too large to replay for ~40 passes).  Traffic grows in proportion to the elements
# processed, so the figures are scaled x4 to the 2^28-element launch timed here.  Reads equal the operands exactly
# once.  The write counter stops at the end of the kernel while tens of MB of dirty lines are still in the 126 MB L2,
# so writes read low at the capture size, and the scaled total lands below the algorithmic bytes for kernels that
# write full-size results; the detail says so.
NCU_TRAFFIC_AT_2_26 = {
    "k_map2_vec": (536.9e6, 221.9e6, "c2.plus"),
    "k_map1_vec": (268.5e6, 213.9e6, "c2.exp"),
    "k_bcast3": (268.5e6, 212.8e6, "c3.a*b"),
    "k_rows_warp": (268.5e6, 3.5e6, "c4.last.sum"),
    "k_cols_warp": (268.4e6, 3.3e6, "c4.mid.sum"),
}


def load_traffic(kernel: str):
    """(traffic scaled to the full-size launch, what it is made of) or (None, None)."""
    rec = NCU_TRAFFIC_AT_2_26.get(kernel)
    if rec is None:
        return None, None
    scale = N28 / (1 << 26)
    read, write, case = rec
    return (read + write) * scale, {"dram_read_bytes": read * scale, "dram_write_bytes": write * scale, "measured_at_elements": 1 << 26,
                                    "scaled_by": scale, "case": case,
                                    "note": "ncu dram__bytes_read/write of one launch on 2^26-element operands, scaled by elements; reads = every "
                                            "operand exactly once; writes are under-counted at the capture size (dirty lines still in L2 when the "
                                            "kernel ends), so the total can read below the algorithmic bytes"}


def main():
    # torch.distributed.run exports OMP_NUM_THREADS=1; the host-side input generator and the CPU
    # baseline are OpenMP code and should use this rank's share of the cores
    world = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
    if world > 1 or "OMP_NUM_THREADS" not in os.environ:
        os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // world))
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="kten_b200", choices=["kten_b200", "reference"])
    ap.add_argument("--cols", type=int, default=2048, help="row length of the x.softmax_* cases (classes)")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--cpu-sample-log2", type=int, default=None, help="log2 of the CPU sample size per operand (default 26, for cpu_baseline and for --impl reference alike)")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--collective", choices=("p2p", "nccl"), default="p2p",
                    help="N > 1: sum of the partials across ranks by one kernel over peer memory (default) or through NCCL")
    ap.add_argument("--no-sharded-graph", dest="sharded_graph", action="store_false")
    ap.add_argument("--no-other-ops", dest="other_ops", action="store_false",
                    help="skip timing the raw-tensor ops beside the sweep (slices, permutes, gather / scatter)")
    ap.add_argument("--case", default=None, help="run one op of the sweep alone (profiling workload), e.g. c2.plus, c4.last.max")
    ap.add_argument("--log2n", type=int, default=26)
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    if args.cpu_sample_log2 is None:
        args.cpu_sample_log2 = 26                   # the reference arm and the in-line baseline time the same sample
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.case:
        return run_single_case(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
