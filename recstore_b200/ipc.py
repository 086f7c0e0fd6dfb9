"""Named tensors and barriers shared by the processes of one box.

API-compatible stand-ins for the torch custom classes the reference registers in
``librecstore_pytorch`` (src/framework/pytorch/IPCTensor.cc:62-88, IPC_barrier.cc:4-12):
``IPCTensorFactory``, ``SlicedTensor``, ``MultiProcessBarrierFactory`` and ``Mfence``.  Host
tensors live in POSIX shared memory (one object per name, see ``csrc/runtime/ipc.cpp``); GPU
tensors are ``cudaMalloc`` allocations whose CUDA IPC handle is published in the shared header, so
any process of the box can map them by name.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import i32, i64, u64, vp, cstr

_lib.register_signatures({
    "rs_shm_set_namespace": (i32, [cstr]),
    "rs_shm_create": (i32, [cstr, i32, i32, C.POINTER(i64), u64, i32, i32, C.POINTER(vp), C.POINTER(i32)]),
    "rs_shm_open": (i32, [cstr, C.POINTER(vp)]),
    "rs_shm_data": (vp, [vp]),
    "rs_shm_blob": (vp, [vp]),
    "rs_shm_meta": (i32, [vp, C.POINTER(i32), C.POINTER(i32), C.POINTER(i64), C.POINTER(u64), C.POINTER(i32), C.POINTER(i32)]),
    "rs_shm_get_sliced_end": (i64, [vp]),
    "rs_shm_set_sliced_end": (None, [vp, i64]),
    "rs_shm_close": (i32, [vp]),
    "rs_shm_unlink": (i32, [cstr]),
    "rs_shm_list": (i32, [C.c_char_p, i32]),
    "rs_shm_clear_all": (i32, []),
    "rs_barrier_create": (i32, [cstr, i32, C.POINTER(vp)]),
    "rs_barrier_wait": (i32, [vp, i32]),
    "rs_barrier_close": (i32, [vp]),
    "rs_barrier_unlink": (i32, [cstr]),
    "rs_mfence": (None, []),
    "rs_lfence": (None, []),
    "rs_sfence": (None, []),
})

_DTYPES = [torch.float32, torch.int64, torch.int32, torch.float16, torch.bfloat16, torch.uint8, torch.float64, torch.bool]
_NP = {torch.float32: np.float32, torch.int64: np.int64, torch.int32: np.int32, torch.float16: np.float16,
       torch.uint8: np.uint8, torch.float64: np.float64, torch.bool: np.bool_, torch.bfloat16: np.uint16}


def _code(dtype: torch.dtype) -> int:
    return _DTYPES.index(dtype)


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def set_namespace(ns: str) -> None:
    """Separates the shared objects of concurrent jobs of one user (default namespace: "default")."""
    _lib.lib()
    _lib.call("rs_shm_set_namespace", ns.encode())


class _Mapped:
    """Keeps a shared-memory mapping alive for as long as tensors built on it exist."""

    def __init__(self, handle: int, name: str):
        self.handle, self.name = handle, name

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().rs_shm_close(self.handle)
        except Exception:
            pass


_handles: Dict[str, _Mapped] = {}
_tensors: Dict[str, torch.Tensor] = {}
_gpu_local: Dict[str, int] = {}


def _meta(handle):
    dt, nd, dev, pid = i32(), i32(), i32(), i32()
    shape = (i64 * 8)()
    nbytes = u64()
    _lib.call("rs_shm_meta", handle, C.byref(dt), C.byref(nd), shape, C.byref(nbytes), C.byref(dev), C.byref(pid))
    return _DTYPES[dt.value], tuple(shape[i] for i in range(nd.value)), nbytes.value, dev.value, pid.value


def _host_tensor(m: _Mapped) -> torch.Tensor:
    dtype, shape, nbytes, dev, _ = _meta(m.handle)
    n = int(np.prod(shape)) if shape else 1
    addr = _lib.lib().rs_shm_data(m.handle)
    buf = (C.c_char * max(nbytes, 1)).from_address(addr)
    arr = np.frombuffer(buf, dtype=_NP[dtype], count=n).reshape(shape)
    t = torch.from_numpy(arr)
    if dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    t._rs_keepalive = m  # type: ignore[attr-defined]
    return t


def _gpu_tensor(m: _Mapped, name: str) -> torch.Tensor:
    from .parallel.peer import tensor_from_ptr
    dtype, shape, nbytes, dev, pid = _meta(m.handle)
    if name in _gpu_local:
        ptr = _gpu_local[name]
    else:
        blob = _lib.lib().rs_shm_blob(m.handle)
        h = (C.c_ubyte * 64).from_address(blob)
        q = vp()
        with torch.cuda.device(dev):
            _lib.call("rs_ipc_open", h, C.byref(q))
        ptr = q.value
        _gpu_local[name] = ptr
    t = tensor_from_ptr(ptr, nbytes, torch.device(f"cuda:{dev}")).view(dtype).view(*shape)
    t._rs_keepalive = m  # type: ignore[attr-defined]
    return t


class SlicedTensor:
    """Variable-length view of a named tensor: the logical length lives in the shared header, so a
    producer process can publish "the first n rows are valid" atomically (reference:
    src/framework/pytorch/IPCTensor.h:556-602)."""

    def __init__(self, name: str, full: torch.Tensor, m: _Mapped):
        self._name, self._full, self._m = name, full, m

    def GetSlicedTensor(self) -> torch.Tensor:
        return self._full[: _lib.lib().rs_shm_get_sliced_end(self._m.handle)]

    def Copy_(self, right: torch.Tensor, non_blocking: bool = False) -> None:
        n = right.shape[0]
        assert n <= self._full.shape[0], "SlicedTensor overflow"
        self._full[:n].copy_(right, non_blocking=non_blocking)
        _lib.lib().rs_sfence()
        _lib.lib().rs_shm_set_sliced_end(self._m.handle, n)

    def SetSameShape4Debug(self, other: "SlicedTensor") -> None:
        _lib.lib().rs_shm_set_sliced_end(self._m.handle, _lib.lib().rs_shm_get_sliced_end(other._m.handle))

    def __len__(self):
        return int(_lib.lib().rs_shm_get_sliced_end(self._m.handle))


class IPCTensorFactory:
    """Creates / finds named tensors shared across processes."""

    @staticmethod
    def ClearIPCMemory() -> int:
        _lib.lib()
        _handles.clear()
        _tensors.clear()
        _gpu_local.clear()
        return _lib.lib().rs_shm_clear_all()

    @staticmethod
    def _create(name: str, shape: Sequence[int], dtype: torch.dtype, device: int, exclusive: bool):
        _lib.lib()
        shape = tuple(int(s) for s in shape)
        n = int(np.prod(shape)) if shape else 1
        arr = (i64 * 8)(*shape)
        h, created = vp(), i32()
        _lib.call("rs_shm_create", name.encode(), _code(dtype), len(shape), arr, n * _itemsize(dtype), device,
                  1 if exclusive else 0, C.byref(h), C.byref(created))
        m = _Mapped(h.value, name)
        _handles[name] = m
        return m, bool(created.value)

    @staticmethod
    def NewIPCTensor(name: str, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> Optional[torch.Tensor]:
        """New zero-filled host tensor; ``None`` when the name already exists (reference semantics)."""
        try:
            m, _ = IPCTensorFactory._create(name, shape, dtype, -1, True)
        except _lib.RecStoreError as e:
            if e.code == _lib.ERR_STATE:
                return None
            raise
        t = _host_tensor(m)
        _tensors[name] = t
        return t

    @staticmethod
    def NewOrGetIPCTensor(name: str, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        m, _ = IPCTensorFactory._create(name, shape, dtype, -1, False)
        t = _host_tensor(m)
        assert tuple(t.shape) == tuple(shape) and t.dtype == dtype, "existing shared tensor has another shape/dtype"
        _tensors[name] = t
        return t

    @staticmethod
    def NewIPCGPUTensor(name: str, shape: Sequence[int], dtype: torch.dtype, dev_id: int) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        nbytes = int(np.prod(shape)) * _itemsize(dtype)
        m, created = IPCTensorFactory._create(name, shape, dtype, dev_id, True)
        p = vp()
        with torch.cuda.device(dev_id):
            _lib.call("rs_peer_alloc", max(nbytes, 256), C.byref(p))
            blob = _lib.lib().rs_shm_blob(m.handle)
            _lib.call("rs_ipc_get_handle", p.value, blob)
        _gpu_local[name] = p.value
        t = _gpu_tensor(m, name)
        _tensors[name] = t
        return t

    @staticmethod
    def FindIPCTensorFromName(name: str) -> torch.Tensor:
        if name in _tensors:
            return _tensors[name]
        _lib.lib()
        h = vp()
        _lib.call("rs_shm_open", name.encode(), C.byref(h))
        m = _Mapped(h.value, name)
        _handles[name] = m
        dev = _meta(m.handle)[3]
        t = _host_tensor(m) if dev < 0 else _gpu_tensor(m, name)
        _tensors[name] = t
        return t

    @staticmethod
    def ListIPCTensors() -> List[str]:
        _lib.lib()
        n = _lib.lib().rs_shm_list(None, 0)
        buf = C.create_string_buffer(n + 1)
        _lib.lib().rs_shm_list(buf, n + 1)
        return [x for x in buf.value.decode().split("\n") if x and not x.startswith("barrier.")]

    @staticmethod
    def NewSlicedIPCTensor(name: str, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> SlicedTensor:
        t = IPCTensorFactory.NewIPCTensor(name, shape, dtype)
        if t is None:
            raise _lib.RecStoreError(_lib.ERR_STATE, f"shared tensor {name} already exists")
        s = SlicedTensor(name, t, _handles[name])
        _lib.lib().rs_shm_set_sliced_end(_handles[name].handle, 0)
        return s

    @staticmethod
    def NewSlicedIPCGPUTensor(name: str, shape: Sequence[int], dtype: torch.dtype, dev_id: int) -> SlicedTensor:
        t = IPCTensorFactory.NewIPCGPUTensor(name, shape, dtype, dev_id)
        _lib.lib().rs_shm_set_sliced_end(_handles[name].handle, 0)
        return SlicedTensor(name, t, _handles[name])

    @staticmethod
    def GetSlicedIPCTensorFromName(name: str) -> SlicedTensor:
        t = IPCTensorFactory.FindIPCTensorFromName(name)
        return SlicedTensor(name, t, _handles[name])

    @staticmethod
    def Delete(name: str) -> None:
        _lib.lib()
        _tensors.pop(name, None)
        _handles.pop(name, None)
        _lib.call("rs_shm_unlink", name.encode())


class MultiProcessBarrier:
    def __init__(self, handle: int, name: str, parties: int, timeout_ms: int):
        self._h, self.name, self.parties, self.timeout_ms = handle, name, parties, timeout_ms

    def Wait(self, timeout_ms: Optional[int] = None) -> None:
        """Blocks until all parties arrived; raises ``RecStoreError(ERR_TIMEOUT)`` if one never does."""
        _lib.call("rs_barrier_wait", self._h, self.timeout_ms if timeout_ms is None else timeout_ms)


class MultiProcessBarrierFactory:
    @staticmethod
    def Create(name: str, count: int, timeout_ms: int = 100_000) -> MultiProcessBarrier:
        _lib.lib()
        h = vp()
        _lib.call("rs_barrier_create", name.encode(), count, C.byref(h))
        return MultiProcessBarrier(h.value, name, count, timeout_ms)

    @staticmethod
    def ClearIPCMemory() -> None:
        n = _lib.lib().rs_shm_list(None, 0)
        buf = C.create_string_buffer(n + 1)
        _lib.lib().rs_shm_list(buf, n + 1)
        for x in buf.value.decode().split("\n"):
            if x.startswith("barrier."):
                _lib.call("rs_barrier_unlink", x[len("barrier."):].encode())


class Mfence:
    @staticmethod
    def mfence():
        _lib.lib().rs_mfence()

    @staticmethod
    def lfence():
        _lib.lib().rs_lfence()

    @staticmethod
    def sfence():
        _lib.lib().rs_sfence()
