"""Host KV engines behind the ``BaseKV`` interface (native, see ``csrc/runtime/kv_engine.h``).

``BaseKV(engine, config)`` with ``config = {"path", "capacity", "value_size", ...}`` mirrors
``base::Factory<BaseKV, const BaseKVConfig&>::NewInstance`` of the reference
(src/storage/kv_engine/base_kv.h:14-56, engine_map.h:129).  Values are float32 vectors of
``value_size // 4`` elements.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import List, Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import cstr, i32, i64, u64, vp

_lib.register_signatures({
    "rs_kv_create": (i32, [cstr, cstr, C.POINTER(vp)]),
    "rs_kv_destroy": (i32, [vp]),
    "rs_kv_value_size": (i32, [vp]),
    "rs_kv_put": (i32, [vp, u64, vp]),
    "rs_kv_get": (i32, [vp, u64, vp, C.POINTER(i32)]),
    "rs_kv_erase": (i32, [vp, u64, C.POINTER(i32)]),
    "rs_kv_batch_get": (i32, [vp, vp, i64, vp, vp]),
    "rs_kv_batch_put": (i32, [vp, vp, i64, vp, C.POINTER(i64)]),
    "rs_kv_bulk_load": (i32, [vp, u64]),
    "rs_kv_clear": (i32, [vp]),
    "rs_kv_size": (u64, [vp]),
    "rs_kv_flush": (i32, [vp]),
    "rs_kv_keys": (i64, [vp, vp, i64]),
    "rs_kv_debug_info": (i32, [vp, C.c_char_p, i32]),
    "rs_kv_check_consistency": (i32, [vp, C.POINTER(i32)]),
    "rs_kv_migrate_hot": (i32, [vp, vp, i64, C.POINTER(i64)]),
    "rs_kv_recovery_state": (i32, [vp, C.POINTER(i32), C.POINTER(i32)]),
    "rs_kv_list_engines": (i32, [C.c_char_p, i32]),
    "rs_kv_preload": (i32, [vp, i32, i32, u64, i32, i32, C.POINTER(u64)]),
    "rs_kv_check_preload": (i32, [vp, i32, i32, u64, i32, C.POINTER(u64), C.POINTER(u64)]),
})


def list_engines() -> List[str]:
    l = _lib.lib()
    n = l.rs_kv_list_engines(None, 0)
    buf = C.create_string_buffer(n + 1)
    l.rs_kv_list_engines(buf, n + 1)
    return [x for x in buf.value.decode().split("\n") if x]


class BaseKV:
    def __init__(self, engine: str = "KVEngineMap", config: Optional[dict] = None):
        self._l = _lib.lib()
        cfg = dict(config or {})
        h = vp()
        _lib.call("rs_kv_create", engine.encode(), json.dumps(cfg).encode(), C.byref(h))
        self._h = h.value
        self.engine = engine
        self.value_size = self._l.rs_kv_value_size(self._h)
        self.dim = self.value_size // 4

    def close(self):
        if getattr(self, "_h", None):
            self._l.rs_kv_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _keys(keys) -> torch.Tensor:
        return torch.as_tensor(keys, dtype=torch.int64).contiguous()

    def Put(self, key: int, value) -> None:
        v = torch.as_tensor(value, dtype=torch.float32).contiguous()
        assert v.numel() == self.dim
        _lib.call("rs_kv_put", self._h, int(key), v.data_ptr())

    def Get(self, key: int) -> Optional[torch.Tensor]:
        out = torch.empty(self.dim, dtype=torch.float32)
        found = i32()
        _lib.call("rs_kv_get", self._h, int(key), out.data_ptr(), C.byref(found))
        return out if found.value else None

    def Erase(self, key: int) -> bool:
        e = i32()
        _lib.call("rs_kv_erase", self._h, int(key), C.byref(e))
        return bool(e.value)

    def BatchGet(self, keys) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (values [n, dim] with zero rows for absent keys, found [n] bool)."""
        k = self._keys(keys)
        out = torch.empty(k.numel(), self.dim, dtype=torch.float32)
        found = torch.empty(k.numel(), dtype=torch.uint8)
        _lib.call("rs_kv_batch_get", self._h, k.data_ptr(), k.numel(), out.data_ptr(), found.data_ptr())
        return out, found.bool()

    def BatchPut(self, keys, values) -> None:
        k = self._keys(keys)
        v = torch.as_tensor(values, dtype=torch.float32).contiguous()
        assert v.shape == (k.numel(), self.dim)
        stored = i64()
        _lib.call("rs_kv_batch_put", self._h, k.data_ptr(), k.numel(), v.data_ptr(), C.byref(stored))

    def BulkLoad(self, n: int) -> None:
        _lib.call("rs_kv_bulk_load", self._h, int(n))

    def clear(self) -> None:
        _lib.call("rs_kv_clear", self._h)

    def Flush(self) -> None:
        _lib.call("rs_kv_flush", self._h)

    def __len__(self) -> int:
        return int(self._l.rs_kv_size(self._h))

    def keys(self) -> torch.Tensor:
        n = len(self)
        out = torch.empty(max(n, 1), dtype=torch.int64)
        m = self._l.rs_kv_keys(self._h, out.data_ptr(), n)
        return out[:m]

    def DebugInfo(self) -> str:
        n = self._l.rs_kv_debug_info(self._h, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._l.rs_kv_debug_info(self._h, buf, n + 1)
        return buf.value.decode()

    def check_consistency(self) -> bool:
        ok = i32()
        _lib.call("rs_kv_check_consistency", self._h, C.byref(ok))
        return bool(ok.value)

    def migrate_hot(self, keys) -> int:
        k = self._keys(keys)
        moved = i64()
        _lib.call("rs_kv_migrate_hot", self._h, k.data_ptr(), k.numel(), C.byref(moved))
        return int(moved.value)

    def recovery_state(self) -> Tuple[bool, bool]:
        r, c = i32(), i32()
        _lib.call("rs_kv_recovery_state", self._h, C.byref(r), C.byref(c))
        return bool(r.value), bool(c.value)


_lib.register_signatures({
    "rs_ppool_open": (i32, [cstr, u64, u64, C.POINTER(vp), C.POINTER(i32)]),
    "rs_ppool_close": (i32, [vp]),
    "rs_ppool_malloc": (u64, [vp, u64]),
    "rs_ppool_free": (i32, [vp, u64]),
    "rs_ppool_slab_size": (u64, [vp, u64]),
    "rs_ppool_class_size": (u64, [u64]),
    "rs_ppool_write": (i32, [vp, u64, vp, u64]),
    "rs_ppool_read": (i32, [vp, u64, vp, u64]),
    "rs_ppool_stats": (i32, [vp, vp]),
    "rs_ppool_allocated": (i64, [vp, vp, i64]),
    "rs_ppool_sync": (i32, [vp]),
    "rs_epoch_new": (i32, [C.POINTER(vp)]),
    "rs_epoch_delete": (i32, [vp]),
    "rs_epoch_protect": (i32, [vp]),
    "rs_epoch_unprotect": (i32, [vp]),
    "rs_epoch_current": (u64, [vp]),
    "rs_epoch_bump": (u64, [vp]),
    "rs_epoch_safe": (i32, [vp, u64]),
    "rs_epoch_retire_slab": (i32, [vp, vp, u64]),
    "rs_epoch_collect": (i64, [vp]),
    "rs_epoch_drain": (i64, [vp]),
    "rs_epoch_pending": (i64, [vp]),
    "rs_recycler_new": (i32, [vp, i32, u64, vp, C.c_uint, C.POINTER(vp)]),
    "rs_recycler_delete": (i32, [vp]),
    "rs_recycler_recycle": (i64, [vp, u64]),
    "rs_recycler_clear": (i64, [vp]),
    "rs_recycler_pending": (i64, [vp]),
    "rs_recycler_set_delay_ns": (i32, [vp, u64]),
})


class PersistSlabPool:
    """Crash-recoverable slab allocator over one file (``path=None``: anonymous memory).  Allocations are byte offsets
    into the mapping; after a reopen the bitmaps of the chunks say which slabs are live (``recovered`` is then True).
    Native, see ``csrc/runtime/persist_pool.h``; role of the reference's PersistMemoryPool
    (src/memory/persist_malloc.h:126-420)."""

    def __init__(self, path: Optional[str], nbytes: int, chunk_bytes: int = 2 << 20):
        self._l = _lib.lib()
        h, rec = vp(), i32(0)
        _lib.call("rs_ppool_open", (path or "").encode(), int(nbytes), int(chunk_bytes), C.byref(h), C.byref(rec))
        self._h = h.value
        self.recovered = bool(rec.value)

    def _depends_on_me(self, obj) -> None:
        """Recyclers and epoch managers hold slabs of this pool that they will free later: they are settled before the
        mapping goes away."""
        import weakref
        if not hasattr(self, "_dependents"):
            self._dependents = []
        if not any(r() is obj for r in self._dependents):
            self._dependents.append(weakref.ref(obj))

    def close(self):
        for ref in getattr(self, "_dependents", []):
            dep = ref()
            if dep is not None and getattr(dep, "_h", None):
                dep._settle()
        self._dependents = []
        if getattr(self, "_h", None):
            self._l.rs_ppool_close(self._h)
            self._h = None

    __del__ = close

    def malloc(self, size: int) -> int:
        """Offset of a slab of at least ``size`` bytes; 0 when the pool is exhausted."""
        return int(self._l.rs_ppool_malloc(self._h, int(size)))

    def free(self, off: int) -> None:
        self._l.rs_ppool_free(self._h, int(off))

    def slab_size(self, off: int) -> int:
        return int(self._l.rs_ppool_slab_size(self._h, int(off)))

    @staticmethod
    def class_size(size: int) -> int:
        return int(_lib.lib().rs_ppool_class_size(int(size)))

    def write(self, off: int, data: bytes) -> None:
        _lib.call("rs_ppool_write", self._h, int(off), C.c_char_p(data), len(data))

    def read(self, off: int, n: int) -> bytes:
        buf = C.create_string_buffer(n)
        _lib.call("rs_ppool_read", self._h, int(off), buf, n)
        return buf.raw

    def allocated(self) -> List[int]:
        n = int(self._l.rs_ppool_allocated(self._h, None, 0))
        a = np.zeros(max(n, 1), dtype=np.uint64)
        self._l.rs_ppool_allocated(self._h, a.ctypes.data, n)
        return a[:n].tolist()

    def stats(self) -> dict:
        a = np.zeros(6, dtype=np.uint64)
        self._l.rs_ppool_stats(self._h, a.ctypes.data)
        names = ("chunk_bytes", "chunks_total", "chunks_in_use", "slabs_in_use", "bytes_in_use", "bytes_reserved")
        return dict(zip(names, (int(x) for x in a)))

    def sync(self) -> None:
        self._l.rs_ppool_sync(self._h)


class EpochManager:
    """Epoch-based reclamation (``csrc/runtime/persist_pool.h``; role of src/memory/epoch_manager.h): readers bracket
    their accesses with ``protect`` / ``unprotect`` (or ``with em:``), writers ``retire`` what they unlinked and it is
    freed once no protected region that could still see it is left."""

    def __init__(self):
        self._l = _lib.lib()
        h = vp()
        _lib.call("rs_epoch_new", C.byref(h))
        self._h = h.value

    def close(self):
        for ref in getattr(self, "_recyclers", []):          # recyclers with the epoch policy consult this manager
            rec = ref()
            if rec is not None and getattr(rec, "_h", None):
                rec.close()
        self._recyclers = []
        if getattr(self, "_h", None):
            self._l.rs_epoch_delete(self._h)
            self._h = None

    __del__ = close

    def protect(self) -> None:
        self._l.rs_epoch_protect(self._h)

    def unprotect(self) -> None:
        self._l.rs_epoch_unprotect(self._h)

    def __enter__(self):
        self.protect()
        return self

    def __exit__(self, *exc):
        self.unprotect()

    def current(self) -> int:
        return int(self._l.rs_epoch_current(self._h))

    def bump(self) -> int:
        return int(self._l.rs_epoch_bump(self._h))

    def safe_to_reclaim(self, epoch: int) -> bool:
        return bool(self._l.rs_epoch_safe(self._h, int(epoch)))

    def retire_slab(self, pool: PersistSlabPool, off: int) -> None:
        pool._depends_on_me(self)
        _lib.call("rs_epoch_retire_slab", self._h, pool._h, int(off))

    def drain(self) -> int:
        """Frees everything that waits, whatever its epoch: for shutdown, when no reader is left."""
        return int(self._l.rs_epoch_drain(self._h))

    _settle = drain

    def collect(self) -> int:
        return int(self._l.rs_epoch_collect(self._h))

    def pending(self) -> int:
        return int(self._l.rs_epoch_pending(self._h))


class SlabRecycler:
    """When a freed slab goes back to its pool: ``"direct"`` (at once), ``"delayed"`` (after ``delay_s``) or
    ``"epoch"`` (once every region protected before the call has ended; needs ``epochs``).  Every ``recycle`` also
    frees what has become due.  Role of DirectRecycle / DelayedRecycle / ShmEpochRecycle, src/memory/malloc.h:34-152."""

    POLICIES = {"direct": 0, "delayed": 1, "epoch": 2}

    def __init__(self, pool: PersistSlabPool, policy: str = "direct", delay_s: float = 1.0,
                 epochs: Optional[EpochManager] = None, bump_every: int = 1000):
        if policy not in self.POLICIES:
            raise ValueError(f"unknown recycle policy {policy!r}; known: {sorted(self.POLICIES)}")
        self._l = _lib.lib()
        self._pool, self._epochs = pool, epochs       # keep both alive for as long as the recycler
        h = vp()
        _lib.call("rs_recycler_new", pool._h, self.POLICIES[policy], int(delay_s * 1e9),
                  epochs._h if epochs is not None else None, int(bump_every), C.byref(h))
        self._h = h.value
        pool._depends_on_me(self)
        if epochs is not None:
            import weakref
            if not hasattr(epochs, "_recyclers"):
                epochs._recyclers = []
            epochs._recyclers.append(weakref.ref(self))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._l.rs_recycler_delete(self._h)
            self._h = None

    __del__ = close

    def recycle(self, off: int = 0) -> int:
        """Hands over the slab at ``off`` (0: nothing, just free what is due); returns how many slabs were freed."""
        return int(self._l.rs_recycler_recycle(self._h, int(off)))

    def clear(self) -> int:
        return int(self._l.rs_recycler_clear(self._h))

    _settle = close

    def pending(self) -> int:
        return int(self._l.rs_recycler_pending(self._h))

    def set_delay(self, delay_s: float) -> None:
        self._l.rs_recycler_set_delay_ns(self._h, int(delay_s * 1e9))


class LoadDBHelper:
    """Warm-up of one PS shard's engine and its check: of the keys ``1 ... warm_capacity`` those that
    ``ShardManager.KeyPartition`` gives to ``server_id`` are stored with the value ``float(key)`` repeated, by
    ``warm_thread_count`` native threads (``shuffle_load``: one thread, scattered key order).  Role of LoadDBHelper,
    src/storage/kv_engine/load_db.h:13-165."""

    def __init__(self, kv: "BaseKV", server_id: int = 0, num_servers: int = 1, warm_thread_count: int = 8,
                 warm_capacity: int = 0):
        self.kv, self.server_id, self.num_servers = kv, int(server_id), int(num_servers)
        self.warm_thread_count, self.warm_capacity = int(warm_thread_count), int(warm_capacity)
        self.inserted = 0

    def PreLoadDB(self, shuffle_load: bool = False) -> int:
        n = u64()
        _lib.call("rs_kv_preload", self.kv._h, self.server_id, self.num_servers, self.warm_capacity,
                  1 if shuffle_load else self.warm_thread_count, int(shuffle_load), C.byref(n))
        self.inserted = int(n.value)
        return self.inserted

    def CheckDBLoad(self) -> Tuple[int, int]:
        """(keys of this shard that hold their warm-up value, keys of this shard): equal after a complete warm-up."""
        right, expected = u64(), u64()
        _lib.call("rs_kv_check_preload", self.kv._h, self.server_id, self.num_servers, self.warm_capacity,
                  self.warm_thread_count, C.byref(right), C.byref(expected))
        return int(right.value), int(expected.value)


class HashAPI:
    """``find / insert / update / remove`` over any engine: the call surface that hash-table evaluation harnesses expect
    (the reference adapts its chunked hash to one in src/storage/nvm/pet_kv/PiBenchWrapper.cc).  ``insert`` refuses a key
    that is present, ``update`` one that is absent; both return whether they stored the value."""

    def __init__(self, engine: str = "KVEngineChunkHash", config: Optional[dict] = None):
        self.kv = BaseKV(engine, config)

    def find(self, key: int) -> Optional[torch.Tensor]:
        return self.kv.Get(key)

    def insert(self, key: int, value) -> bool:
        if self.kv.Get(key) is not None:
            return False
        self.kv.Put(key, value)
        return True

    def update(self, key: int, value) -> bool:
        if self.kv.Get(key) is None:
            return False
        self.kv.Put(key, value)
        return True

    def remove(self, key: int) -> bool:
        return bool(self.kv.Erase(key))

    def __len__(self) -> int:
        return len(self.kv)

    def close(self) -> None:
        self.kv.close()


def reinit(path: str) -> List[str]:
    """Removes the files that the persistent engines keep in ``path`` (``values.slab``, ``shard_*.dict``,
    ``poolmap.slabs``), so the next engine opened there starts empty; other files are left alone.  Returns the names
    removed.  The reference's tool for this wipes its persistent-memory mount points (src/memory/pm_command.cc:9-21)."""
    import glob
    import os
    gone = []
    for pat in ("values.slab", "shard_*.dict", "poolmap.slabs"):
        for f in sorted(glob.glob(os.path.join(path, pat))):
            os.remove(f)
            gone.append(os.path.basename(f))
    return gone


def _main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="python -m recstore_b200.storage",
                                 description="maintenance of the persistent engines' directories")
    ap.add_argument("--command", required=True, choices=["reinit", "engines"])
    ap.add_argument("--path", default=None, help="directory of a persistent engine (reinit)")
    a = ap.parse_args(argv)
    if a.command == "engines":
        print("\n".join(list_engines()))
        return 0
    if not a.path:
        ap.error("--command reinit needs --path")
    for f in reinit(a.path):
        print("removed", f)
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
