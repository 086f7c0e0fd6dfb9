"""GPU-resident caches and the HBM hash-table shard.

``GpuCache`` keeps the reference's torch class contract
(src/framework/pytorch/recstore_gpu_cache.h:31-106): ``Query(keys, values) -> CacheQueryResult
{values, missing_index, missing_keys}``, ``Replace(keys, values)``; plus ``Update`` and ``Dump``
of the underlying cache API (src/storage/gpu_cache/gpu_cache_api.hpp:27-50).  ``GpuHashTable`` is
the key -> row index of an HBM shard (insert / lookup / erase / dump / check); ``unique_keys``
deduplicates a key batch on the device.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _lib
from .._lib import HashTableView, i32, i64, u64, vp, ptr, stream_ptr

_lib.register_signatures({
    "rs_cache_create": (i32, [u64, i32, C.POINTER(vp)]),
    "rs_cache_destroy": (i32, [vp]),
    "rs_cache_capacity": (u64, [vp]),
    "rs_cache_num_sets": (u64, [vp]),
    "rs_cache_query": (i32, [vp, vp, i64, vp, vp, vp, vp, vp]),
    "rs_cache_replace": (i32, [vp, vp, i64, vp, vp, vp]),
    "rs_cache_update": (i32, [vp, vp, i64, vp, vp, vp]),
    "rs_cache_dump": (i32, [vp, u64, u64, vp, vp, vp]),
    "rs_merge_rows": (i32, [vp, vp, vp, i64, i32, vp]),
    "rs_range_cache_query": (i32, [vp, vp, i64, i32, vp, vp, i64, i64, i64, vp, vp]),
    "rs_ht_create": (i32, [u64, i32, C.POINTER(vp), C.POINTER(HashTableView)]),
    "rs_ht_destroy": (i32, [vp]),
    "rs_ht_clear": (i32, [vp, vp]),
    "rs_ht_insert": (i32, [C.POINTER(HashTableView), vp, i64, vp, vp, vp]),
    "rs_ht_lookup": (i32, [C.POINTER(HashTableView), vp, i64, vp, vp]),
    "rs_ht_erase": (i32, [C.POINTER(HashTableView), vp, i64, vp, vp]),
    "rs_ht_erase_checked": (i32, [C.POINTER(HashTableView), vp, i64, vp, vp, vp]),
    "rs_ht_dump": (i32, [C.POINTER(HashTableView), vp, vp, vp, u64, vp]),
    "rs_ht_check": (i32, [C.POINTER(HashTableView), C.POINTER(u64), C.POINTER(i64), C.POINTER(u64)]),
    "rs_unique_keys": (i32, [vp, i64, vp, vp, u64, vp, vp, vp, vp, vp]),
})


@dataclass
class CacheQueryResult:
    values: torch.Tensor          # [n, dim]; hit rows filled, miss rows untouched
    missing_index: torch.Tensor   # [n_miss] positions of the misses in the query
    missing_keys: torch.Tensor    # [n_miss]


class GpuCache:
    def __init__(self, num_items: int, emb_dim: int, device=None):
        _lib.lib()
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.dim = emb_dim
        h = vp()
        with torch.cuda.device(self.device):
            _lib.call("rs_cache_create", int(num_items), int(emb_dim), C.byref(h))
        self._h = h.value
        self.capacity = int(_lib.lib().rs_cache_capacity(self._h))
        self.num_sets = int(_lib.lib().rs_cache_num_sets(self._h))
        self.status = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._miss_count = torch.zeros(1, dtype=torch.int32, device=self.device)

    def __del__(self):
        try:
            if self._h:
                _lib.lib().rs_cache_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def Query(self, keys: torch.Tensor, values: Optional[torch.Tensor] = None, sync: bool = True) -> CacheQueryResult:
        """With ``sync=False`` the miss lists keep their full length and ``miss_count()`` tells how many
        entries are valid (no device -> host read on the hot path)."""
        keys = keys.to(self.device, torch.int64).contiguous()
        n = keys.numel()
        if values is None:
            values = torch.empty(n, self.dim, device=self.device)
        mi = torch.empty(max(n, 1), dtype=torch.int64, device=self.device)
        mk = torch.empty(max(n, 1), dtype=torch.int64, device=self.device)
        _lib.call("rs_cache_query", self._h, ptr(keys), n, ptr(values), ptr(mi), ptr(mk), ptr(self._miss_count), stream_ptr())
        if sync:
            m = int(self._miss_count.item())
            mi, mk = mi[:m], mk[:m]
        return CacheQueryResult(values, mi, mk)

    def miss_count(self) -> torch.Tensor:
        return self._miss_count

    def Replace(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        keys = keys.to(self.device, torch.int64).contiguous()
        values = values.to(self.device, torch.float32).contiguous()
        _lib.call("rs_cache_replace", self._h, ptr(keys), keys.numel(), ptr(values), ptr(self.status), stream_ptr())

    def Update(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        keys = keys.to(self.device, torch.int64).contiguous()
        values = values.to(self.device, torch.float32).contiguous()
        _lib.call("rs_cache_update", self._h, ptr(keys), keys.numel(), ptr(values), ptr(self.status), stream_ptr())

    def Dump(self, set_begin: int = 0, set_end: Optional[int] = None) -> torch.Tensor:
        set_end = self.num_sets if set_end is None else set_end
        out = torch.empty(max((set_end - set_begin) * 32, 1), dtype=torch.int64, device=self.device)
        cnt = torch.zeros(1, dtype=torch.int64, device=self.device)
        _lib.call("rs_cache_dump", self._h, set_begin, set_end, ptr(out), ptr(cnt), stream_ptr())
        return out[: int(cnt.item())]


def merge_op(dst: torch.Tensor, retrieved: torch.Tensor, missing_index: torch.Tensor) -> torch.Tensor:
    """``dst[missing_index[i]] = retrieved[i]`` (rows fetched for cache misses scattered into place)."""
    n = missing_index.numel()
    _lib.call("rs_merge_rows", ptr(dst), ptr(retrieved.contiguous()), ptr(missing_index.contiguous()), n, dst.shape[1], stream_ptr())
    return dst


def uva_cache_query_op(dst: torch.Tensor, ids: torch.Tensor, hbm_cache: torch.Tensor, host_table: torch.Tensor,
                       start: int, end: int, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per id: row ``id - start`` of the HBM range cache when ``start <= id < end``, else row ``id`` of the
    page-locked host table read in place over the interconnect."""
    from ..kvstore import get_kvstore
    if not host_table.is_cuda and not host_table.is_pinned():
        kv = get_kvstore()
        if kv is None:
            from ..kvstore import kvinit
            kv = kvinit()
        rc = kv.GetUVAMap(host_table)
        if rc not in (0, 712):  # 712 = already registered
            raise _lib.RecStoreError(_lib.ERR_CUDA, f"cudaHostRegister failed with code {rc}")
    _lib.call("rs_range_cache_query", ptr(dst), ptr(ids.contiguous()), ids.numel(), dst.shape[1], ptr(hbm_cache),
              host_table.data_ptr(), int(start), int(end), host_table.shape[0], ptr(status), stream_ptr())
    return dst


class GpuHashTable:
    """64-bit key -> row index (dense, reusable) in HBM."""

    def __init__(self, capacity: int, max_rows: Optional[int] = None, device=None):
        _lib.lib()
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.view = HashTableView()
        h = vp()
        max_rows = int(max_rows if max_rows is not None else capacity)
        with torch.cuda.device(self.device):
            _lib.call("rs_ht_create", int(capacity), max_rows, C.byref(h), C.byref(self.view))
        self._h = h.value
        self.max_rows = max_rows
        self.status = torch.zeros(1, dtype=torch.int64, device=self.device)

    def __del__(self):
        try:
            if self._h:
                _lib.lib().rs_ht_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def _k(self, keys):
        return keys.to(self.device, torch.int64).contiguous()

    def insert(self, keys: torch.Tensor) -> torch.Tensor:
        keys = self._k(keys)
        rows = torch.empty(keys.numel(), dtype=torch.int64, device=self.device)
        _lib.call("rs_ht_insert", C.byref(self.view), ptr(keys), keys.numel(), ptr(rows), ptr(self.status), stream_ptr())
        return rows

    def lookup(self, keys: torch.Tensor) -> torch.Tensor:
        keys = self._k(keys)
        rows = torch.empty(keys.numel(), dtype=torch.int64, device=self.device)
        _lib.call("rs_ht_lookup", C.byref(self.view), ptr(keys), keys.numel(), ptr(rows), stream_ptr())
        return rows

    def erase(self, keys: torch.Tensor) -> torch.Tensor:
        keys = self._k(keys)
        rows = torch.empty(keys.numel(), dtype=torch.int64, device=self.device)
        _lib.call("rs_ht_erase_checked", C.byref(self.view), ptr(keys), keys.numel(), ptr(rows), ptr(self.status), stream_ptr())
        return rows

    def clear(self) -> None:
        _lib.call("rs_ht_clear", self._h, stream_ptr())

    def dump(self) -> Tuple[torch.Tensor, torch.Tensor]:
        cap = int(self.view.mask) + 1
        k = torch.empty(cap, dtype=torch.int64, device=self.device)
        r = torch.empty(cap, dtype=torch.int64, device=self.device)
        c = torch.zeros(1, dtype=torch.int64, device=self.device)
        _lib.call("rs_ht_dump", C.byref(self.view), ptr(k), ptr(r), ptr(c), cap, stream_ptr())
        n = int(c.item())
        return k[:n], r[:n]

    def check(self) -> Tuple[int, int, int]:
        """(live slots, size counter, inconsistent slots); synchronises."""
        live, size, bad = u64(), i64(), u64()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            _lib.call("rs_ht_check", C.byref(self.view), C.byref(live), C.byref(size), C.byref(bad))
        return int(live.value), int(size.value), int(bad.value)

    def __len__(self):
        return self.check()[1]


def unique_keys(keys: torch.Tensor, status: Optional[torch.Tensor] = None):
    """Device-side unique: returns (unique keys [u] in arbitrary order, inverse [n] with
    ``unique[inverse] == keys``).  Allocates its scratch (2 n slots rounded up to a power of two).
    The reserved keys -1 and -2 are not deduplicated: their inverse is -1 and ``status`` gets ``DEV_BAD_ARG``."""
    keys = keys.contiguous()
    n = keys.numel()
    nslots = 2
    while nslots < 2 * max(n, 1):
        nslots <<= 1
    dev = keys.device
    sk = torch.empty(nslots, dtype=torch.int64, device=dev)
    si = torch.empty(nslots, dtype=torch.int32, device=dev)
    uniq = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    inv = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=dev)
    _lib.call("rs_unique_keys", ptr(keys), n, ptr(sk), ptr(si), nslots, ptr(uniq), ptr(inv), ptr(cnt), ptr(status), stream_ptr())
    u = int(cnt.item())
    return uniq[:u], inv[:n].long()
