"""`CudaBackend`: the host-side mirror of Kandle's backend contract for device name "cuda".

The reference defines a backend as `IBackend { name, createTensorHandle, operators }`
(packages/types/src/backend/index.ts:33-55) whose `operators` registry maps dispatch keys to
kernel functions (packages/types/src/backend/register.ts:128-144,
packages/utils/src/registry/index.ts:3-17).  Its only implementation is the WebGPU backend
(packages/backend-webgpu/src/index.ts:15-87, kernels/index.ts:36-90).  This module provides the
same three members on top of the C ABI: same keys, same argument meaning, same error behaviour
(exceptions thrown synchronously; operators only enqueue work; `dataAsync()` is the only
synchronisation point).
"""
from __future__ import annotations

import ctypes
import itertools
import math
from typing import Callable, Sequence

import numpy as np

from . import lib
from .lib import DTYPES, KandleCudaError, kd_matmul_cfg, kd_tensor

_ids = itertools.count(1)


def contiguous_strides(shape: Sequence[int]) -> tuple[int, ...]:
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(st))


class CudaStorage:
    """Refcounted device buffer (IStorage, packages/types/src/storage.ts:5-25; the WebGPU
    counterpart is packages/backend-webgpu/src/base/storage.ts:60-143)."""

    def __init__(self, nbytes: int, zero: bool = True):
        h = ctypes.c_uint64(0)
        lib.call("kd_storage_alloc", ctypes.c_uint64(int(nbytes)), int(zero), ctypes.byref(h))
        self.handle = h.value
        self.nbytes = int(nbytes)
        self.id = next(_ids)
        self._refs = 1

    def incRef(self) -> None:
        if self._refs <= 0:
            raise RuntimeError("storage already released")
        self._refs += 1

    def decRef(self) -> None:
        if self._refs <= 0:
            return
        self._refs -= 1
        if self._refs == 0:
            lib.call("kd_storage_release", ctypes.c_uint64(self.handle))
            self.handle = 0

    @property
    def isDisposed(self) -> bool:
        return self._refs <= 0

    def device_ptr(self) -> int:
        p = ctypes.c_void_p()
        lib.call("kd_storage_device_ptr", ctypes.c_uint64(self.handle), ctypes.byref(p))
        return p.value or 0

    def __del__(self):  # GC fallback, like the reference's FinalizationRegistry
        try:
            if self._refs > 0 and self.handle:
                self._refs = 0
                lib.raw().kd_storage_release(ctypes.c_uint64(self.handle))
        except Exception:
            pass


class CudaTensorHandle:
    """ITensorHandle (packages/types/src/tensor.ts:6-55): metadata + a share of a storage.
    Strides and offset are in elements."""

    device = "cuda"

    def __init__(self, storage: CudaStorage, shape, dtype: str, strides=None, offset: int = 0,
                 memoryFormat: str = "contiguous"):
        self.storage = storage
        self.shape = tuple(int(s) for s in shape)
        if len(self.shape) > lib.KD_MAX_DIMS:
            raise ValueError(f"rank {len(self.shape)} exceeds {lib.KD_MAX_DIMS}")
        if dtype not in DTYPES:
            raise ValueError(f"unsupported dtype {dtype!r}")
        self.dtype = dtype
        self.strides = tuple(int(s) for s in strides) if strides is not None else contiguous_strides(self.shape)
        self.offset = int(offset)
        self.memoryFormat = memoryFormat
        self.id = next(_ids)
        self._disposed = False

    # --- metadata
    @property
    def numel(self) -> int:
        return int(math.prod(self.shape))

    @property
    def storageId(self) -> int:
        return self.storage.id

    @property
    def buffer(self) -> int:
        return self.storage.handle

    @property
    def isDisposed(self) -> bool:
        return self._disposed

    def isContiguous(self) -> bool:
        expect = 1
        for s, st in zip(reversed(self.shape), reversed(self.strides)):
            if s != 1 and st != expect:
                return False
            expect *= s
        return True

    def dispose(self) -> None:
        if not self._disposed:
            self._disposed = True
            self.storage.decRef()

    def view(self, shape, strides, offset) -> "CudaTensorHandle":
        """New handle sharing this storage (refcount++), as createTensorHandle({storage,...})."""
        self.storage.incRef()
        return CudaTensorHandle(self.storage, shape, self.dtype, strides, offset)

    def c(self) -> kd_tensor:
        if self._disposed or self.storage.isDisposed:
            raise RuntimeError("tensor handle used after dispose()")
        t = kd_tensor()
        t.storage = self.storage.handle
        t.offset = self.offset
        t.dtype = DTYPES[self.dtype][0]
        t.ndim = len(self.shape)
        for i, (s, st) in enumerate(zip(self.shape, self.strides)):
            t.shape[i] = s
            t.strides[i] = st
        return t

    # --- readback
    def dataAsync(self) -> np.ndarray:
        """De-strides on the device when needed, downloads (stream-synchronising) and converts
        physical -> logical dtype like packages/backend-webgpu/src/base/tensor.ts:120-156
        (bfloat16 is widened to float32 on the host)."""
        h = self
        tmp = None
        if not (self.isContiguous()):
            tmp = CudaBackend.instance().createTensorHandle(self.shape, self.dtype)
            lib.call("kd_copy", ctypes.byref(tmp.c()), ctypes.byref(self.c()))
            h = tmp
        code, esz, npdt = DTYPES[self.dtype]
        out = np.empty(self.shape, dtype=npdt)
        if out.size:
            lib.call("kd_download", ctypes.c_uint64(h.storage.handle), ctypes.c_uint64(h.offset * esz),
                     out.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(out.nbytes))
        else:
            lib.call("kd_synchronize")
        if tmp is not None:
            tmp.dispose()
        if self.dtype == "bfloat16":
            return lib.bf16_bits_to_f32(out).reshape(self.shape)
        return out


class OperatorRegistry:
    """IBackendOpsRegister {register, find, has} (packages/types/src/backend/register.ts:128-144)."""

    def __init__(self):
        self._ops: dict[str, Callable] = {}

    def register(self, key: str, fn: Callable) -> None:
        self._ops[key] = fn

    def find(self, key: str):
        return self._ops.get(key)

    def has(self, key: str) -> bool:
        return key in self._ops

    def keys(self):
        return sorted(self._ops)


class CudaBackend:
    """IBackend for device "cuda"."""

    name = "cuda"
    _instance: "CudaBackend | None" = None

    def __init__(self, device_ordinal: int = 0):
        lib.call("kd_init", int(device_ordinal), 0)
        self.device_ordinal = device_ordinal
        self.operators = OperatorRegistry()
        from .kernels import register_cuda_kernels
        register_cuda_kernels(self.operators)

    @classmethod
    def create(cls, device_ordinal: int = 0) -> "CudaBackend":
        """Counterpart of WebGPUBackend.create() (packages/backend-webgpu/src/index.ts:73-85)."""
        if cls._instance is None:
            cls._instance = cls(device_ordinal)
        elif cls._instance.device_ordinal != device_ordinal:
            raise KandleCudaError(1, f"backend already created on device {cls._instance.device_ordinal}")
        return cls._instance

    @classmethod
    def instance(cls) -> "CudaBackend":
        if cls._instance is None:
            raise KandleCudaError(4, "CudaBackend.create() has not been called")
        return cls._instance

    # createTensorHandle(shape, dtype, data?)  |  createTensorHandle({shape,dtype,storage?,...})
    def createTensorHandle(self, shape, dtype: str | None = None, data=None, *, storage: CudaStorage | None = None,
                           strides=None, offset: int = 0, memoryFormat: str = "contiguous") -> CudaTensorHandle:
        if isinstance(shape, dict):
            o = shape
            return self.createTensorHandle(o["shape"], o["dtype"], o.get("data"), storage=o.get("storage"),
                                           strides=o.get("strides"), offset=o.get("offset", 0),
                                           memoryFormat=o.get("memoryFormat", "contiguous"))
        if dtype not in DTYPES:
            raise ValueError(f"unsupported dtype {dtype!r}")
        shape = tuple(int(s) for s in shape)
        if storage is not None:
            storage.incRef()
            return CudaTensorHandle(storage, shape, dtype, strides, offset, memoryFormat)
        code, esz, npdt = DTYPES[dtype]
        n = int(math.prod(shape))
        st = CudaStorage(max(n * esz, 1), zero=(data is None))  # new storage is zero-initialised
        h = CudaTensorHandle(st, shape, dtype, None, 0, memoryFormat)
        if data is not None:
            self.upload(h, data)
        return h

    def upload(self, h: CudaTensorHandle, data) -> None:
        """Host -> device with logical -> physical conversion (the reference converts on upload in
        DTypeResolver, packages/backend-webgpu/src/base/DTypeResolver.ts:52-99)."""
        code, esz, npdt = DTYPES[h.dtype]
        arr = np.asarray(data)
        if h.dtype == "bfloat16":
            arr = arr if arr.dtype == np.uint16 else lib.f32_to_bf16_bits(arr.astype(np.float32, copy=False))
        else:
            arr = np.ascontiguousarray(arr, dtype=npdt)
        arr = np.ascontiguousarray(arr)
        if arr.size != h.numel:
            raise ValueError(f"data has {arr.size} elements, tensor has {h.numel}")
        if not h.isContiguous():
            raise ValueError("upload target must be contiguous")
        if arr.size:
            lib.call("kd_upload", ctypes.c_uint64(h.storage.handle), ctypes.c_uint64(h.offset * esz),
                     arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(arr.nbytes))

    def synchronize(self) -> None:
        lib.call("kd_synchronize")

    def launch_count(self, reset: bool = False) -> int:
        n = ctypes.c_uint64(0)
        lib.call("kd_launch_count", ctypes.byref(n), int(reset))
        return n.value

    def memory_stats(self) -> dict:
        a, b, c = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_uint64(0)
        lib.call("kd_memory_stats", ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        return {"in_use": a.value, "cached": b.value, "reserved": c.value}


class CudaEvent:
    """CUDA event on the library's stream, for device-side timing."""

    def __init__(self):
        h = ctypes.c_uint64(0)
        lib.call("kd_event_create", ctypes.byref(h))
        self.handle = h.value

    def record(self) -> "CudaEvent":
        lib.call("kd_event_record", ctypes.c_uint64(self.handle))
        return self

    def elapsed_ms(self, stop: "CudaEvent") -> float:
        ms = ctypes.c_float(0)
        lib.call("kd_event_elapsed_ms", ctypes.c_uint64(self.handle), ctypes.c_uint64(stop.handle), ctypes.byref(ms))
        return float(ms.value)
