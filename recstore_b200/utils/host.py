"""Host-side helpers of the native runtime that have no other home: thread pinning, the ring of free indices and the
coarse clock (``csrc/runtime/base.{h,cpp}``; roles of src/base/bind_core.cc:14-70, src/base/lf_list.h and
src/base/async_time.h of the reference)."""
from __future__ import annotations

import ctypes as C
from typing import List

import numpy as np

from .. import _lib
from .._lib import i32, u64, vp

_lib.register_signatures({
    "rs_bind_core": (i32, [i32]),
    "rs_numa_node_cores": (i32, [i32, C.POINTER(i32), i32]),
    "rs_coarse_now_ns": (u64, []),
    "rs_steady_now_ns": (u64, []),
    "rs_ring_new": (i32, [C.c_uint, C.POINTER(vp)]),
    "rs_ring_delete": (i32, [vp]),
    "rs_ring_push": (i32, [vp, vp, C.c_uint]),
    "rs_ring_pop": (C.c_uint, [vp, vp, C.c_uint]),
    "rs_ring_size": (C.c_uint, [vp]),
    "rs_ring_clear": (None, [vp]),
})


def bind_core(core: int) -> None:
    """Pins the calling thread to one core."""
    _lib.call("rs_bind_core", int(core))


def numa_node_cores(node: int) -> List[int]:
    """Cores of a NUMA node as the operating system reports them (empty when unknown)."""
    l = _lib.lib()
    n = l.rs_numa_node_cores(int(node), None, 0)
    out = (i32 * max(n, 1))()
    l.rs_numa_node_cores(int(node), out, n)
    return [int(out[i]) for i in range(n)]


def coarse_now_ns() -> int:
    """A monotonic clock that costs one load: a background thread refreshes it every 10 ms."""
    return int(_lib.lib().rs_coarse_now_ns())


def steady_now_ns() -> int:
    return int(_lib.lib().rs_steady_now_ns())


class IndexRing:
    """Bounded ring of free indices (int32): ``push`` appends a batch or refuses it whole, ``pop(n)`` takes up to ``n``
    entries in ring order; any number of threads may pop at once."""

    def __init__(self, capacity: int):
        self._l = _lib.lib()
        h = vp()
        _lib.call("rs_ring_new", int(capacity), C.byref(h))
        self._h = h.value
        self.capacity = int(capacity)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._l.rs_ring_delete(self._h)
            self._h = None

    __del__ = close

    def push(self, values) -> bool:
        v = np.ascontiguousarray(np.asarray(values, dtype=np.int32).reshape(-1))
        return bool(self._l.rs_ring_push(self._h, v.ctypes.data, v.size))

    def pop(self, want: int) -> np.ndarray:
        out = np.empty(int(want), dtype=np.int32)
        n = int(self._l.rs_ring_pop(self._h, out.ctypes.data, int(want)))
        return out[:n]

    def __len__(self) -> int:
        return int(self._l.rs_ring_size(self._h))

    def clear(self) -> None:
        self._l.rs_ring_clear(self._h)
