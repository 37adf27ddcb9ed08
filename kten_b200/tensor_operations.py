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
        self._init_deferred()

    # ---- deferred elementwise expressions (kten_b200.lazy, ktc_lazy_*) ----------------------------------------
    # `lazy` off: every call runs at once, like kten-jvm.  On: elementwise calls are recorded below the C ABI
    # and run fused when a value is needed.  The recorder is one per process; its options are set through
    # these attributes.
    def _init_deferred(self) -> None:
        import os
        self.lazy = os.environ.get("KTEN_CUDA_LAZY", "0") == "1"    # the process-wide default; the attribute can be set at any time
        self._recorder = Z.Recorder(self.lib)
        self._pending_targets = set()       # buffers with a recorded `+= pending sum` update (may hold stale entries)
        self._options = {"recompute_limit": 2, "store_cost": 8, "defer_sums": 1, "defer_inplace": 1}
        for name, value in self._options.items():
            self._recorder.option(name, value)

    def _option(name):
        def get(self):
            return self._options[name]

        def put(self, value):
            self._options[name] = int(value)
            self._recorder.option(name, int(value))
        return property(get, put)

    recomputeLimit = _option("recompute_limit")     # a pending value is recomputed at most this often before it is stored
    storeCost = _option("store_cost")               # ... unless recomputing costs this much (a transcendental): stored at once
    deferSums = _option("defer_sums")               # sums of deferred tensors wait too, and run several per pass
    deferInplace = _option("defer_inplace")         # an in-place call with a pending operand on a buffer nobody else holds waits too
    del _option

    @property
    def fusedEvaluations(self) -> int:              # programs run by ktc_expr_eval
        return self._recorder.stats()["fused"]

    @property
    def unfusedEvaluations(self) -> int:            # deferred expressions that fell back to separate calls
        return self._recorder.stats()["unfused"]

    @property
    def multiSinkEvaluations(self) -> int:          # passes that produced more than one sum
        return self._recorder.stats()["multi_sink"]

    def _run_pending(self) -> None:
        self._pending_targets.clear()
        self._recorder.run_pending()

    def _flush_dependents(self, handle: int) -> None:
        """Before `handle` is written in place by a call the recorder does not see."""
        self._pending_targets.discard(handle)
        self._recorder.flush(handle)

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
        if self.lazy:                       # a pending constant: no buffer and no fill until somebody needs one
            shape = [int(d) for d in shape]
            return CUDARawTensor(shape, None, self, lz=self._recorder.full(self.device, shape, constant))
        raw = self.createRaw(shape)
        raw.inplaceFill(constant)
        return raw

    def zerosLike(self, raw: CUDARawTensor) -> CUDARawTensor:
        return self.createRawFill(raw.shape, 0.0)

    # ---- nn operations built on the path's kernels (TensorOperations.kt:127-131) ------------------------------
    def batchNorm(self, axis: int, momentum: float, epsilon: float, training: bool):
        from .nn import CUDABatchNorm
        return CUDABatchNorm(axis, momentum, epsilon, training, self)

    def upsample(self, upsampleType: str, scale: int):
        from .nn import CUDAUpsample2DNearest
        if upsampleType != "NEAREST":                      # UpsampleType has this one member
            raise ValueError(f"unknown upsample type {upsampleType}")
        return CUDAUpsample2DNearest(scale, self)

    def spatialPooling(self, kernel, padding, stride, dilation, options):
        """TensorOperations.spatialPooling (TensorOperations.kt:127): options is a PoolingOptions (kten_b200.nn)."""
        from .nn import CUDASpatialPooling
        return CUDASpatialPooling(kernel, padding, stride, dilation, options, self)

    def zeroOut(self, raw: CUDARawTensor) -> None:
        raw.inplaceFill(0.0)

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
                **{("recorder." + k): float(v) for k, v in self._recorder.stats().items()}}

    def setMemoryUsageScaleHint(self, fraction: float) -> None:
        """PlatformProvider.memoryUsageScaleHint (PlatformProvider.kt:12-40): cap the pool."""
        L.check(self.lib.ktc_pool_limit(self.device, int(self.totalMemory * fraction)))
