"""Sub-allocators over slabs of device or host memory (native: ``csrc/runtime/device_pool.cpp``).

``DevicePool("pool" | "binning" | "fixed", ...)`` hands out 256-byte aligned addresses without calling ``cudaMalloc``
on the hot path; ``tensor()`` wraps an allocation as a torch tensor that returns its block when it is garbage
collected.  Plays the part of the reference's RMM pool / binning / fixed-length resources
(src/gpu_memory/memory_pool.h:23-81).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from .. import _lib
from .._lib import i32, sz, vp

_lib.register_signatures({
    "rs_devpool_create": (i32, [i32, i32, sz, sz, sz, C.POINTER(vp)]),
    "rs_devpool_destroy": (i32, [vp]),
    "rs_devpool_alloc": (i32, [vp, sz, C.POINTER(vp)]),
    "rs_devpool_free": (i32, [vp, vp]),
    "rs_devpool_stats": (i32, [vp, C.POINTER(C.c_ulonglong)]),
})

_KIND = {"pool": 0, "binning": 1, "fixed": 2}
_BACKING = {"device": 0, "pinned": 1, "host": 2}
_TYPESTR = {torch.float32: "<f4", torch.float16: "<f2", torch.int64: "<i8", torch.int32: "<i4", torch.uint8: "|u1",
            torch.float64: "<f8", torch.int16: "<i2", torch.int8: "|i1", torch.bool: "|b1"}


class _Block:
    """Array-interface view of one allocation; frees the block when the last tensor over it dies."""

    def __init__(self, pool: "DevicePool", ptr: int, shape, dtype: torch.dtype, cuda: bool):
        self._pool, self._ptr = pool, ptr
        iface = {"shape": tuple(shape), "typestr": _TYPESTR[torch.uint8 if dtype == torch.bfloat16 else dtype],
                 "data": (ptr, False), "version": 3 if not cuda else 2}
        if cuda:
            self.__cuda_array_interface__ = iface
        else:
            self.__array_interface__ = iface

    def __del__(self):
        try:
            self._pool.free(self._ptr)
        except Exception:
            pass


class DevicePool:
    def __init__(self, kind: str = "pool", backing: str = "device", initial_bytes: int = 64 << 20, max_bytes: int = 1 << 30,
                 block_bytes: int = 0, max_bin_bytes: int = 4 << 20):
        self.kind, self.backing = kind, backing
        h = vp()
        param = block_bytes if kind == "fixed" else (max_bin_bytes if kind == "binning" else 0)
        _lib.call("rs_devpool_create", _KIND[kind], _BACKING[backing], int(initial_bytes), int(max_bytes), int(param), C.byref(h))
        self._h = h.value

    def alloc(self, nbytes: int) -> int:
        p = vp()
        _lib.call("rs_devpool_alloc", self._h, int(nbytes), C.byref(p))
        return int(p.value)

    def free(self, ptr: int) -> None:
        if self._h:
            _lib.call("rs_devpool_free", self._h, int(ptr))

    def tensor(self, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(1, n * torch.empty((), dtype=dtype).element_size())
        ptr = self.alloc(nbytes)
        cuda = self.backing == "device"
        if dtype == torch.bfloat16:    # no array-interface code for bf16: view bytes
            blk = _Block(self, ptr, (nbytes,), torch.uint8, cuda)
            t = torch.as_tensor(blk, device="cuda" if cuda else "cpu")
            return t.view(torch.bfloat16).view(*shape)
        blk = _Block(self, ptr, shape, dtype, cuda)
        if cuda:
            return torch.as_tensor(blk, device="cuda")
        import numpy as np
        return torch.from_numpy(np.asarray(blk))

    def stats(self) -> dict:
        o = (C.c_ulonglong * 6)()
        _lib.call("rs_devpool_stats", self._h, o)
        return dict(zip(("reserved_bytes", "in_use_bytes", "live_blocks", "slabs", "peak_in_use_bytes", "failures"), map(int, o)))

    def close(self) -> None:
        if self._h:
            _lib.lib().rs_devpool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
