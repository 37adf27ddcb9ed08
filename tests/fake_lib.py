"""A host stand-in for libkten_cuda.so, for CPU tests of the host logic only.

The deferred-expression layer is host code: which calls it makes, in which order, with which
buffers, decides whether aliases, in-place writes and side outputs keep the semantics of the eager
backend.  Its core -- the recorder behind `ktc_lazy_*` (kten_b200/csrc/ktc_lazy.cpp) -- is plain C++
that reaches the rest of the library through a table of C-ABI entry points, so it is compiled here
on its own (g++, no CUDA) and the table is filled with this module's implementations: buffers,
copies, the elementwise calls, the reductions and ktc_expr_eval (a numpy interpreter of the program
encoding), all with the CPU oracle's arithmetic.  The same script can then be run call by call and
deferred on a machine without a GPU and the two results compared.  It is test infrastructure:
nothing in the product imports it, and it says nothing about the CUDA kernels.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess
import tempfile

import numpy as np

from kten_b200 import _lib as L
from kten_b200.tensor_operations import CUDATensorOperations
from oracle import oracle as O

BIN = {L.PLUS: O.PLUS, L.MINUS: O.MINUS, L.TIMES: O.TIMES, L.DIV: O.DIV, L.POW: O.POW}


HERE = os.path.dirname(os.path.abspath(__file__))
RECORDER_SRC = os.path.join(HERE, "..", "kten_b200", "csrc", "ktc_lazy.cpp")
RECORDER_SO = os.path.join(HERE, "host_lazy", "libktc_lazy_host.so")

u64, i64, i32, f32 = C.c_uint64, C.c_int64, C.c_int, C.c_float
P = C.POINTER
# the recorder's backend table, in the order of `struct Backend` (ktc_lazy.cpp): name, C signature
BACKEND = [
    ("ktc_alloc", (i32, i32, i64, P(u64))),
    ("ktc_retain", (i32, u64)),
    ("ktc_release", (i32, u64)),
    ("ktc_refcount", (i32, u64, P(i32))),
    ("ktc_buf_info", (i32, u64, P(i32), P(i64), P(C.c_void_p))),
    ("ktc_d2d", (i32, u64, i64, u64, i64, i64)),
    ("ktc_fill", (i32, u64, i64, i64, f32)),
    ("ktc_binary", (i32, i32, u64, u64, u64, i64)),
    ("ktc_binary_bcast", (i32, i32, u64, u64, P(i64), i32, u64, P(i64), i32)),
    ("ktc_binary_inplace", (i32, i32, u64, u64, i64)),
    ("ktc_scalar", (i32, i32, u64, u64, f32, i64, i32)),
    ("ktc_scalar_inplace", (i32, i32, u64, f32, i64)),
    ("ktc_unary", (i32, i32, u64, u64, i64)),
    ("ktc_clamp", (i32, u64, u64, f32, f32, i64)),
    ("ktc_compare_scalar", (i32, i32, u64, u64, f32, i64)),
    ("ktc_broadcast_to", (i32, u64, P(i64), i32, u64, P(i64), i32)),
    ("ktc_reduce_axis", (i32, i32, u64, u64, i64, i64, i64)),
    ("ktc_reduce_all", (i32, i32, u64, u64, i64)),
    ("ktc_expr_eval", (i32, P(C.c_uint32), i32, P(f32), i32, P(i64), i32, P(u64), P(i64), i32, P(u64), i32, i32, u64, i32)),
    ("ktc_expr_eval_multi_fused", (i32, P(C.c_uint32), i32, P(f32), i32, P(i64), i32, P(u64), P(i64), i32, P(u64), i32, P(i32), P(u64), P(i32), i32,
                                   P(u64), P(i32), u64, P(u64), P(i64), i32)),
    ("ktc_p2p_allreduce_sum", (i32, u64, P(u64), P(i64), i32)),
    ("ktc_softmax_xent_forward", (i32, u64, u64, u64, u64, i64, i64, f32, f32)),
    ("ktc_softmax_xent_forward_expr", (i32, u64, u64, u64, u64, i64, i64, f32, f32, P(C.c_uint32), i32, P(f32), i32, P(u64), P(i64), i32, i32, P(u64), i32)),
]
RECORDER_CALLS = {
    "ktc_lazy_leaf": (i32, [u64, P(i64), i32, P(u64)]), "ktc_lazy_free": (i32, [u64]),
    "ktc_lazy_unary": (i32, [i32, u64, P(u64)]), "ktc_lazy_binary": (i32, [i32, u64, u64, P(u64)]),
    "ktc_lazy_scalar": (i32, [i32, u64, f32, i32, P(u64)]), "ktc_lazy_clamp": (i32, [u64, f32, f32, P(u64)]),
    "ktc_lazy_compare_scalar": (i32, [i32, u64, f32, P(u64)]), "ktc_lazy_broadcast_to": (i32, [u64, P(i64), i32, P(u64)]),
    "ktc_lazy_assign_binary": (i32, [i32, u64, u64, P(i32)]), "ktc_lazy_assign_scalar": (i32, [i32, u64, f32, P(i32)]),
    "ktc_lazy_sum": (i32, [u64, i32, i32, P(i64), i32, P(u64)]), "ktc_lazy_buffer": (i32, [u64, P(u64)]),
    "ktc_lazy_info": (i32, [u64, P(i32), P(i32), P(i64), P(i32)]), "ktc_lazy_flush": (i32, [u64]),
    "ktc_lazy_run_pending": (i32, []), "ktc_lazy_option": (i32, [C.c_char_p, i32]), "ktc_lazy_stats": (i32, [P(i64)]),
    "ktc_lazy_allreduce": (i32, [u64, P(u64), i32]),
    "ktc_lazy_full": (i32, [i32, P(i64), i32, f32, P(u64)]), "ktc_lazy_assign_fill": (i32, [u64, f32, P(i32)]),
    "ktc_lazy_assign_scatter_const": (i32, [u64, u64, f32, P(i32)]),
    "ktc_lazy_softmax_xent_forward": (i32, [u64, u64, f32, f32, P(u64), P(u64)]),
}


def build_recorder() -> str:
    """g++ build of the recorder alone (no CUDA); returns the path of the shared object."""
    if not os.path.exists(RECORDER_SO) or os.path.getmtime(RECORDER_SO) < os.path.getmtime(RECORDER_SRC):
        os.makedirs(os.path.dirname(RECORDER_SO), exist_ok=True)
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DKTC_LAZY_STANDALONE", "-o", RECORDER_SO, RECORDER_SRC], check=True)
    return RECORDER_SO


class _Out:
    """What the stand-in's methods expect of a ctypes.byref argument, over a pointer handed in by C."""

    def __init__(self, ptr):
        self._obj = self
        self._ptr = ptr

    @property
    def value(self):
        return self._ptr[0]

    @value.setter
    def value(self, v):
        self._ptr[0] = v


def _ints(ptr, n):
    return [int(ptr[i]) for i in range(n)]


class FakeLib:
    def __init__(self):
        self.bufs = {}          # handle -> [ndarray, refcount]
        self.next = 1
        self.launches = 0
        self.expr_calls = 0
        self.multi_calls = 0
        self.calls = []         # names of compute calls, in order
        self.programs = []      # every program handed to ktc_expr_eval / ktc_expr_eval_multi, as the recorder built it
        self.error = b""
        self._attach_recorder()

    # ---- the expression recorder, compiled alone, with this object as the library it drives ----------
    def _attach_recorder(self):
        # the recorder keeps one state per loaded object: every stand-in loads a copy of its own
        fd, path = tempfile.mkstemp(suffix=".so", prefix="ktc_lazy_host_")
        os.close(fd)
        shutil.copyfile(build_recorder(), path)
        self._recorder = C.CDLL(path)
        os.unlink(path)
        self._callbacks = []
        table = (C.c_void_p * len(BACKEND))()
        for i, (name, sig) in enumerate(BACKEND):
            cb = C.CFUNCTYPE(*sig)(self._adapter(name))
            self._callbacks.append(cb)
            table[i] = C.cast(cb, C.c_void_p).value
        self._recorder.ktc_lazy_test_set_backend.argtypes = [C.POINTER(C.c_void_p), i32]
        assert self._recorder.ktc_lazy_test_set_backend(table, len(BACKEND)) == 0
        for name, (res, args) in RECORDER_CALLS.items():
            fn = getattr(self._recorder, name)
            fn.restype, fn.argtypes = res, args
            setattr(self, name, fn)

    def _adapter(self, name):
        method = getattr(self, name)
        if name == "ktc_alloc":
            return lambda dev, n, out: method(dev, n, _Out(out))
        if name == "ktc_refcount":
            return lambda h, out: method(h, _Out(out))
        return method

    def ktc_buf_info(self, h, dev, n, ptr):
        if dev:
            dev[0] = 0
        if n:
            n[0] = self._get(h).size
        return 0

    # ---- buffers -----------------------------------------------------------------------------
    def _get(self, h):
        rec = self.bufs.get(int(h))
        if rec is None or rec[1] <= 0:
            raise AssertionError(f"use of a released or unknown buffer {h}")
        return rec[0]

    def ktc_alloc(self, dev, n, ref):
        h = self.next
        self.next += 1
        self.bufs[h] = [np.full(int(n), np.nan, dtype=np.float32), 1]      # fresh memory holds garbage
        ref._obj.value = h
        return 0

    def ktc_retain(self, h):
        self._get(h)
        self.bufs[int(h)][1] += 1
        return 0

    def ktc_release(self, h):
        self._get(h)
        self.bufs[int(h)][1] -= 1
        return 0

    def ktc_refcount(self, h, ref):
        self._get(h)
        ref._obj.value = self.bufs[int(h)][1]
        return 0

    def live_buffers(self):
        return sum(1 for a, c in self.bufs.values() if c > 0)

    def ktc_last_error(self):
        return self.error

    def ktc_launch_count(self):
        return self.launches

    def ktc_sync(self, dev):
        return 0

    def ktc_h2d(self, h, off, src, n, mode):
        addr = src.value if isinstance(src, C.c_void_p) else C.cast(src, C.c_void_p).value
        self._get(h)[off:off + n] = np.ctypeslib.as_array((C.c_float * n).from_address(addr))
        return 0

    def ktc_d2h(self, dst, h, off, n, mode):
        addr = dst.value if isinstance(dst, C.c_void_p) else C.addressof(dst)
        np.ctypeslib.as_array((C.c_float * n).from_address(addr))[:] = self._get(h)[off:off + n]
        return 0

    def ktc_d2d(self, dst, doff, src, soff, n):
        self._get(dst)[doff:doff + n] = self._get(src)[soff:soff + n]
        return 0

    def ktc_fill(self, h, off, n, v):
        self._get(h)[off:off + n] = np.float32(v)
        self.launches += 1
        return 0

    # ---- elementwise calls and the full reduction --------------------------------------------------
    def _note(self, name):
        self.calls.append(name)
        self.launches += 1

    def ktc_binary(self, op, out, a, b, n):
        self._note("binary")
        self._get(out)[:n] = O.binary_same(BIN[op], self._get(a)[:n].copy(), self._get(b)[:n].copy())
        return 0

    def ktc_binary_inplace(self, op, a, b, n):
        return self.ktc_binary(op, a, a, b, n)

    def ktc_binary_bcast(self, op, out, a, sa, na, b, sb, nb):
        self._note("binary_bcast")
        sha, shb = _ints(sa, na), _ints(sb, nb)
        res, cs = O.binary(BIN[op], self._get(a)[:int(np.prod(sha))], sha, self._get(b)[:int(np.prod(shb))], shb)
        self._get(out)[:res.size] = res
        return 0

    def ktc_scalar(self, op, out, a, s, n, scalar_first):
        self._note("scalar")
        self._get(out)[:n] = O.scalar(BIN[op], self._get(a)[:n].copy(), float(s), scalar_first=bool(scalar_first))
        return 0

    def ktc_scalar_inplace(self, op, a, s, n):
        return self.ktc_scalar(op, a, a, s, n, 0)

    def ktc_unary(self, op, out, a, n):
        self._note("unary")
        self._get(out)[:n] = O.unary(op, self._get(a)[:n].copy())
        return 0

    def ktc_clamp(self, out, a, lo, hi, n):
        self._note("clamp")
        self._get(out)[:n] = O.clamp(self._get(a)[:n].copy(), lo, hi)
        return 0

    def ktc_compare_scalar(self, op, out, a, v, n):
        self._note("compare")
        self._get(out)[:n] = O.compare(op, self._get(a)[:n].copy(), float(v))
        return 0

    def ktc_broadcast_to(self, out, so, no, a, sa, na):
        self._note("broadcast_to")
        sho, sha = _ints(so, no), _ints(sa, na)
        self._get(out)[:int(np.prod(sho))] = O.broadcast_to(self._get(a)[:int(np.prod(sha))], sha, sho)
        return 0

    def ktc_reduce_all(self, op, out, a, n):
        self._note("reduce_all")
        self._get(out)[0] = O.reduce_all(op, self._get(a)[:n].copy())
        return 0

    def ktc_reduce_axis(self, op, out, a, outer, length, inner):
        self._note("reduce_axis")
        self._get(out)[:outer * inner] = O.aggregate(op, self._get(a)[:outer * length * inner].copy(), outer, length, inner)
        return 0

    def ktc_sum_to_shape(self, out, out_shape, out_ndim, a, in_shape, in_ndim):
        self._note("sum_to_shape")
        ins, outs = _ints(in_shape, in_ndim), _ints(out_shape, out_ndim)
        n_in, n_out = int(np.prod(ins)), int(np.prod(outs))
        self._get(out)[:n_out] = O.sum_to_shape(self._get(a)[:n_in].copy(), ins, outs)
        return 0

    # ---- spatial pooling: the oracle's loops behind the library's entry points -------------------------------------------
    def _pool(self, geom, is_max, include_padding=False):
        H, W, OH, OW, kh, kw, ph, pw, sh, sw, dh, dw = (int(geom[i]) for i in range(12))
        opt = type("Options", (), {"type": "MAX" if is_max else "AVG", "useCeil": False, "includePadding": bool(include_padding)})()
        op = O.OracleSpatialPooling((kh, kw), (ph, pw), (sh, sw), (dh, dw), opt, None)
        op._geometry = lambda inp, g=None, i=None: (inp.shape[0], H, W, OH, OW, [inp.shape[0], OH, OW])      # the extents are the caller's
        return op, H, W, OH, OW

    def _plane_tensor(self, h, planes, rows, cols):
        return O.OracleRawTensor([planes, rows, cols], self._get(h)[:planes * rows * cols].copy(), None)

    def ktc_pool2d_max(self, out, indices, inp, planes, geom):
        self._note("pool2d_max")
        op, H, W, OH, OW = self._pool(geom, True)
        o, i = op.updateOutput(self._plane_tensor(inp, planes, H, W))
        self._get(out)[:planes * OH * OW], self._get(indices)[:planes * OH * OW] = o.data, i.data
        return 0

    def ktc_pool2d_max_grad(self, grad_in, grad_out, indices, planes, geom):
        self._note("pool2d_max_grad")
        op, H, W, OH, OW = self._pool(geom, True)
        x = O.OracleRawTensor([planes, H, W], np.zeros(planes * H * W, np.float32), None)
        g = op.calculateGradInput(x, self._plane_tensor(grad_out, planes, OH, OW), self._plane_tensor(indices, planes, OH, OW))
        self._get(grad_in)[:planes * H * W] = g.data
        return 0

    def ktc_pool2d_avg(self, out, inp, planes, geom, include_padding):
        self._note("pool2d_avg")
        op, H, W, OH, OW = self._pool(geom, False, include_padding)
        self._get(out)[:planes * OH * OW] = op.updateOutput(self._plane_tensor(inp, planes, H, W))[0].data
        return 0

    def ktc_pool2d_avg_grad(self, grad_in, grad_out, planes, geom, include_padding):
        self._note("pool2d_avg_grad")
        op, H, W, OH, OW = self._pool(geom, False, include_padding)
        x = O.OracleRawTensor([planes, H, W], np.zeros(planes * H * W, np.float32), None)
        self._get(grad_in)[:planes * H * W] = op.calculateGradInput(x, self._plane_tensor(grad_out, planes, OH, OW), None).data
        return 0

    def ktc_gather_axis(self, out, inp, in_shape, index, index_shape, ndim, axis):
        self._note("gather")
        ins, ixs = _ints(in_shape, ndim), _ints(index_shape, ndim)
        src = self._get(inp)[:int(np.prod(ins))].reshape(ins)
        idx = self._get(index)[:int(np.prod(ixs))].reshape(ixs).astype(np.int64)
        box = tuple(slice(None) if d == axis else slice(0, ixs[d]) for d in range(ndim))
        self._get(out)[:idx.size] = np.take_along_axis(src[box], idx, axis).reshape(-1)
        return 0

    def ktc_scatter_axis_nd(self, mode, target, target_shape, index, index_shape, src, src_shape, ndim, axis, constant):
        self._note("scatter")
        ts, ixs = _ints(target_shape, ndim), _ints(index_shape, ndim)
        tgt = self._get(target)[:int(np.prod(ts))].reshape(ts)
        idx = self._get(index)[:int(np.prod(ixs))].reshape(ixs).astype(np.int64)
        if mode != L.SCATTER_CONST:
            ss = _ints(src_shape, ndim)
            source = self._get(src)[:int(np.prod(ss))].reshape(ss)
        for pos in np.ndindex(*ixs):                       # the reference's order: row-major over the index
            dst = list(pos)
            dst[axis] = idx[pos]
            dst = tuple(dst)
            if mode == L.SCATTER_CONST:
                tgt[dst] = np.float32(constant)
            elif mode == L.SCATTER_ADD:
                tgt[dst] = np.float32(tgt[dst] + source[pos])
            else:
                tgt[dst] = source[pos]
        return 0

    def ktc_scatter_axis(self, target, index, src, outer, length, inner):
        self._note("scatter")
        tgt = self._get(target)[:outer * length * inner].reshape(outer, length, inner)
        idx = self._get(index)[:outer * inner].reshape(outer, inner).astype(np.int64)
        source = self._get(src)[:outer * inner].reshape(outer, inner)
        o, i = np.meshgrid(np.arange(outer), np.arange(inner), indexing="ij")
        tgt[o, idx, i] = source
        return 0

    # ---- a world of one: the exchange leaves the tensors as they are, and is counted -------------------
    def ktc_p2p_allreduce_sum(self, comm, bufs, counts, n):
        self._note("p2p_allreduce")
        for i in range(n):
            self._get(bufs[i])
        return 0

    # ---- SoftmaxCrossEntropy's forward: the call sequence of SoftmaxCrossEntropy.kt:40-59 with the oracle's arithmetic ----
    def _softmax_rows(self, logits, targets, rows, cols, lo, hi):
        x = self._get(logits)[:rows * cols].copy()
        t = self._get(targets)[:rows].astype(np.int64)
        rep = lambda v: np.repeat(v, cols)
        shifted = O.binary_same(O.MINUS, x, rep(O.aggregate(L.MAX, x, rows, cols, 1)))
        e = O.unary(O.EXP, shifted)
        p = O.binary_same(O.DIV, e, rep(O.aggregate(L.SUM, e, rows, cols, 1)))
        pn = O.binary_same(O.DIV, p, rep(O.aggregate(L.SUM, p, rows, cols, 1)))
        logp = O.unary(O.LOG, O.clamp(pn, lo, hi))
        nll = O.unary(O.NEG, logp.reshape(rows, cols)[np.arange(rows), t].copy())
        return p, nll

    def ktc_softmax_xent_forward(self, softmax, nll, logits, targets, rows, cols, lo, hi):
        if cols > 12288 or cols <= 64 or cols % 4:
            self.error = b"rows not handled in one pass"
            return L.KTC_ENOTSUP
        self._note("softmax_xent_forward")
        p, l = self._softmax_rows(logits, targets, rows, cols, lo, hi)
        if softmax:
            self._get(softmax)[:rows * cols] = p
        self._get(nll)[:rows] = l
        return 0

    def ktc_softmax_xent_forward_expr(self, softmax, nll, logits, targets, rows, cols, lo, hi, code, n_code, imm, n_imm, leaves, lshapes, n_leaves, soft_leaf,
                                      stores, n_stores):
        if cols > 12288 or cols <= 64 or cols % 4 or getattr(self, "no_softmax_epilogue", False):
            self.error = b"rows not handled in one pass"
            return L.KTC_ENOTSUP
        self._note("softmax_xent_forward_expr")
        self.launches -= 1                                   # one kernel: the program below counts it
        p, l = self._softmax_rows(logits, targets, rows, cols, lo, hi)
        if softmax:
            self._get(softmax)[:rows * cols] = p
        self._get(nll)[:rows] = l
        # the program sees the row's softmax as its leaf `soft_leaf`: a scratch buffer here, registers in the kernel
        ref = _Out([0])
        self.ktc_alloc(0, rows * cols, ref)
        tmp = ref.value
        self._get(tmp)[:] = p
        hs = (u64 * n_leaves)(*[tmp if i == soft_leaf else int(leaves[i]) for i in range(n_leaves)])
        shapes = []
        for i in range(n_leaves):
            shapes += [rows, cols] if i == soft_leaf else [int(lshapes[2 * i]), int(lshapes[2 * i + 1])]
        rc = self.ktc_expr_eval(code, n_code, imm, n_imm, (i64 * 2)(rows, cols), 2, hs, (i64 * len(shapes))(*shapes), n_leaves, stores, n_stores,
                                L.EXPR_STORE_ONLY, 0, 0)
        self.ktc_release(tmp)
        return rc

    def ktc_expr_eval_multi_fused(self, code, n_code, imm, n_imm, shape, ndim, leaves, lshapes, n_leaves, stores, n_stores, kinds, outs, means, n_sinks,
                                  add_to, add_mode, comm, x_bufs, x_counts, n_x):
        rc = self.ktc_expr_eval_multi(code, n_code, imm, n_imm, shape, ndim, leaves, lshapes, n_leaves, stores, n_stores, kinds, outs, means, n_sinks)
        if rc != 0:
            return rc
        shp = _ints(shape, ndim)
        total = int(np.prod(shp))
        folded = 0
        for j in range(n_sinks):
            if add_to and add_to[j]:
                n = 1 if kinds[j] == L.EXPR_SUM_ALL else shp[-1] if kinds[j] == L.EXPR_SUM_ROWS else total // shp[-1]
                t = self._get(add_to[j])
                old = np.zeros(n, np.float32) if add_mode and add_mode[j] == 2 else t[:n]
                t[:n] = (old + self._get(outs[j])[:n]).astype(np.float32)
                folded += 1
        self.programs[-1]["folded_updates"] = folded
        self.programs[-1]["exchange"] = [int(x_bufs[i]) for i in range(n_x)] if comm else None
        return 0

    # ---- the fused expression call: the program encoding interpreted with the oracle's arithmetic ----
    def ktc_expr_eval_multi(self, code, n_code, imm, n_imm, shape, ndim, leaves, lshapes, n_leaves, stores, n_stores, kinds, outs, means, n_sinks):
        self.multi_calls += 1
        return self.ktc_expr_eval(code, n_code, imm, n_imm, shape, ndim, leaves, lshapes, n_leaves, stores, n_stores,
                                  L.EXPR_MULTI, 0, 0, sinks=[(int(kinds[j]), int(outs[j]), int(means[j])) for j in range(n_sinks)])

    def ktc_expr_eval(self, code, n_code, imm, n_imm, shape, ndim, leaves, lshapes, n_leaves, stores, n_stores, sink, sink_out, mean, sinks=None):
        shp = _ints(shape, ndim)
        if shp[-1] % 4 != 0 or len([d for d in shp if d != 1]) > 3:
            self.error = b"not fusable (stand-in rule: innermost extent must be a multiple of 4, at most 3 non-unit dims)"
            return L.KTC_ENOTSUP
        self.expr_calls += 1
        self._note("expr_eval")
        total = int(np.prod(shp))
        self.programs.append({"code": [int(code[i]) for i in range(n_code)], "imm": [float(imm[i]) for i in range(n_imm)], "shape": shp,
                              "leaves": [int(leaves[i]) for i in range(n_leaves)],
                              "leaf_shapes": [_ints(lshapes, (i + 1) * ndim)[i * ndim:] for i in range(n_leaves)],
                              "n_stores": int(n_stores), "sink": int(sink), "sinks": sinks})
        regs = [None] * L.EXPR_REGS
        acc = None
        accs = {}
        flat = lambda v: np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
        for pc in range(n_code):
            w = int(code[pc])
            op, d, a, b, k = w & 0xFF, (w >> 8) & 0xF, (w >> 12) & 0xF, (w >> 16) & 0xF, w >> 20
            if op == L.X_LOAD:
                ls = _ints(lshapes, (k + 1) * ndim)[k * ndim:]
                src = self._get(leaves[k])[:int(np.prod(ls))]
                regs[d] = flat(np.broadcast_to(src.reshape(ls), shp))
            elif op == L.X_CONST:
                regs[d] = np.full(total, imm[k], np.float32)
            elif op in (L.X_ADD, L.X_SUB, L.X_MUL, L.X_DIV, L.X_POW):
                o = {L.X_ADD: O.PLUS, L.X_SUB: O.MINUS, L.X_MUL: O.TIMES, L.X_DIV: O.DIV, L.X_POW: O.POW}[op]
                regs[d] = O.binary_same(o, regs[a], regs[b])
            elif op in (L.X_NEG, L.X_RCP, L.X_EXP, L.X_LOG, L.X_TANH, L.X_SIGMOID, L.X_SQRT, L.X_RSQRT, L.X_ABS):
                o = {L.X_NEG: O.NEG, L.X_RCP: O.RECIPROCAL, L.X_EXP: O.EXP, L.X_LOG: O.LOG, L.X_TANH: O.TANH, L.X_SIGMOID: O.SIGMOID,
                     L.X_SQRT: O.SQRT, L.X_RSQRT: O.RSQRT, L.X_ABS: O.ABS}[op]
                regs[d] = O.unary(o, regs[a])
            elif op == L.X_SQUARE:
                regs[d] = O.binary_same(O.TIMES, regs[a], regs[a])
            elif op == L.X_CLAMP:
                regs[d] = O.clamp(regs[a], imm[k], imm[k + 1])
            elif L.X_CMP_LT <= op <= L.X_CMP_GTE:
                regs[d] = O.compare(op - L.X_CMP_LT, regs[a], float(imm[k]))
            elif op == L.X_SCATC:
                cols = np.broadcast_to(np.arange(shp[-1]), shp).reshape(-1)
                regs[d] = np.where(cols == regs[b].astype(np.int64), np.float32(imm[k]), regs[a]).astype(np.float32)
            elif op == L.X_STORE:
                self._get(stores[k])[:total] = regs[a]
            elif op == L.X_ACC:
                acc = regs[a].astype(np.float64)
                accs[k] = acc
            else:
                raise AssertionError(f"bad opcode {op}")
        if sinks is None:
            sinks = [(sink, sink_out, mean)] if sink != L.EXPR_STORE_ONLY else []
            accs = {0: acc}
        for j, (kind, out, mean_j) in enumerate(sinks):
            if kind == L.EXPR_SUM_ALL:
                self._get(out)[0] = np.float32(accs[j].sum() / (total if mean_j else 1))
            elif kind == L.EXPR_SUM_LAST:
                self._get(out)[:total // shp[-1]] = accs[j].reshape(-1, shp[-1]).sum(axis=1).astype(np.float32)
            else:
                self._get(out)[:shp[-1]] = accs[j].reshape(-1, shp[-1]).sum(axis=0).astype(np.float32)
        return 0


def make_ops() -> CUDATensorOperations:
    """A CUDATensorOperations whose library is the stand-in above (no device, no CUDA library)."""
    import threading
    ops = object.__new__(CUDATensorOperations)
    ops.lib = FakeLib()
    ops.device, ops.deviceName, ops.totalMemory, ops.smCount = 0, "host stand-in", 0, 0
    ops.platformKey = "CUDA - host stand-in"
    ops._tls = threading.local()
    ops.epsilon = 1e-7
    ops._init_deferred()
    return ops
