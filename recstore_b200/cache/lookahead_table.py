"""Embedding table whose rows live in pinned host memory, with a write-back cache in HBM fed by the lookahead window.

Storage.  ``host`` is one pinned array ``[num_rows, dim + 4]``: the weights of a row, its row-wise Adagrad state in
column ``dim``, padding.  The HBM tier is the 32-way set-associative :class:`~recstore_b200.cache.gpu_cache.GpuCache`
with rows of the same layout; a cached row is the authoritative copy (updates are applied to it in place and mark it
dirty) until it is evicted, at which point it is written back.

Pipeline (the reference's lookahead controller + GPU cache + UvmTable staging, src/python/pytorch/recstore/
controller_process.py:24-132, src/framework/pytorch/recstore_gpu_cache.h:31-106, src/storage/gpu_cache/
uvm_table.cu:421-497, and the read-your-updates contract of grad_async_v2.h:189-212):

* ``prefetch(ids, step)`` -- called by the sampler for a batch ``lookahead`` steps before it is used.  On a side
  stream the batch is deduplicated and PROBED against the cache (hits get a fresh stamp, which protects them from
  eviction until they are used); the miss keys go to pinned memory; a host worker thread gathers those rows from
  ``host`` into a pinned staging buffer with every core and issues ONE ``cudaMemcpyAsync`` of the staged block to the
  device on the side stream.  Nothing here waits on the training stream.
* ``lookup(ids, step)`` -- on the training stream: waits for the staged block (a stream wait on its event), inserts the
  staged rows (evicting least-recently stamped rows that are not protected; dirty evicted rows are copied out and
  handed to the worker, which writes them back before it serves any later gather), then reads the batch from the cache.
* ``update(grads)`` -- folds duplicate ids and applies SGD / row-wise Adagrad to the cached rows in place.

Read-your-updates.  Every mutation of the cache happens on the training stream, in step order.  A row that step s
needs is either already cached (then its staged copy, if any, is ignored by the insert) or it was written back before
the worker gathered it: the worker is one FIFO, write-backs are queued at the step that evicts, gathers of later
announcements come after them.  A gather that was queued BEFORE a write-back of the same row can only happen for a
row that was evicted after it had been announced, which the protection window (stamps of the last ``lookahead + 1``
steps are never evicted) rules out; a set that is full of protected rows refuses the insert instead, which is reported
through the device status word (``DEV_TABLE_FULL``): size the cache at several times ``(lookahead + 2) * max_keys``.

Hashed host tier.  With ``host_engine`` (the name of a host KV engine, e.g. ``"KVEngineExtendibleHash"``) the rows live
in that engine instead of a dense array, so keys are arbitrary non-negative 64-bit ids and ``num_rows`` is only the
engine's capacity: this is the two-level table of the reference (device hash block over a host hash block,
src/storage/gpu_cache/uvm_table.h, uvm_table.cu:421-497) with the lookahead staging in front.  A key that the engine
has never seen reads as its initial value, a pure function of the key, and enters the engine when it is first written
back.

The host side never spins on the device and the device never waits for the host: the only blocking wait is the
training thread waiting (bounded) for the worker to have QUEUED the copy of a batch that was announced too late.
"""
from __future__ import annotations

import ctypes as C
import math
import queue
import threading
from typing import Optional

import torch

from .. import _lib
from .._lib import f32, i32, i64, ptr, stream_ptr, u32, u64, vp
from .gpu_cache import GpuCache

_lib.register_signatures({
    "rs_cache_replace_evict": (i32, [vp, vp, vp, i64, vp, u32, vp, vp, vp, vp, vp, vp, vp]),
    "rs_cache_apply": (i32, [vp, vp, vp, i64, vp, vp, i32, f32, f32, i32, vp, vp, vp]),
    "rs_cache_set_clock": (i32, [vp, u32, vp]),
    "rs_cache_flush_dirty": (i32, [vp, vp, vp, vp, vp]),
    "rs_cache_query_noclock": (i32, [vp, vp, i64, vp, vp, vp, vp, vp]),
    "rs_host_gather_rows": (i32, [vp, i64, i64, vp, i64, vp]),
    "rs_host_scatter_rows": (i32, [vp, i64, i64, vp, i64, vp]),
    "rs_unique_keys": (i32, [vp, i64, vp, vp, u64, vp, vp, vp, vp, vp]),
    "rs_segment_sum": (i32, [vp, vp, i64, i32, vp, vp, vp]),
    "rs_expand_rows": (i32, [vp, vp, i64, i32, vp, vp]),
})


class _Slot:
    """Buffers of one announced batch."""

    def __init__(self, cap: int, dv: int, dev: torch.device):
        i64d = dict(dtype=torch.int64, device=dev)
        self.step = -1
        self.n = 0
        self.ids = torch.empty(cap, **i64d)
        ns = 2
        while ns < 2 * cap:
            ns <<= 1
        self.nslots = ns
        self.sk = torch.empty(ns, **i64d)
        self.si = torch.empty(ns, dtype=torch.int32, device=dev)
        self.uniq = torch.empty(cap, **i64d)
        self.inv = torch.empty(cap, dtype=torch.int32, device=dev)
        self.ucount = torch.zeros(1, dtype=torch.int32, device=dev)
        self.miss_index = torch.empty(cap, **i64d)
        self.miss_keys = torch.empty(cap, **i64d)
        self.miss_count = torch.zeros(1, dtype=torch.int32, device=dev)
        self.miss_keys_host = torch.empty(cap, dtype=torch.int64).pin_memory()
        self.miss_count_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.rows_host = torch.empty(cap, dv).pin_memory()
        self.rows_dev = torch.empty(cap, dv, device=dev)
        self.evict_keys = torch.empty(cap, **i64d)
        self.evict_rows = torch.empty(cap, dv, device=dev)
        self.evict_count = torch.zeros(1, dtype=torch.int32, device=dev)
        self.evict_keys_host = torch.empty(cap, dtype=torch.int64).pin_memory()
        self.evict_rows_host = torch.empty(cap, dv).pin_memory()
        self.evict_count_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.probed = torch.cuda.Event()
        self.staged = torch.cuda.Event()
        self.evicted = torch.cuda.Event()
        self.staged_queued = threading.Event()       # the worker has issued the H2D copy (the CUDA event is recorded)
        self.writeback_done = threading.Event()
        self.writeback_done.set()
        self.staged_bytes = 0


class LookaheadCachedTable:
    def __init__(self, num_rows: int, dim: int, cache_rows: int, max_keys: int, *, lr: float = 0.01, eps: float = 1e-10,
                 optimizer: str = "rowwise_adagrad", device: Optional[torch.device] = None, lookahead: int = 2,
                 init: str = "uniform", seed: int = 0, wait_timeout_s: float = 20.0, host_engine: Optional[str] = None,
                 host_engine_config: Optional[dict] = None):
        assert dim % 4 == 0 and lookahead >= 1
        self.N, self.D, self.Dv, self.cap, self.L = int(num_rows), int(dim), int(dim) + 4, int(max_keys), int(lookahead)
        self.dev = dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.lr, self.eps, self.optimizer = lr, eps, optimizer
        self.timeout = wait_timeout_s
        self._init, self._seed = init, int(seed)
        if init not in ("uniform", "row_index", "zeros"):
            raise ValueError(init)
        self.kv = None
        if host_engine is not None:
            from ..storage import BaseKV
            cfg = {"capacity": self.N, "value_size": self.Dv * 4}
            cfg.update(host_engine_config or {})
            self.kv = BaseKV(host_engine, cfg)
            self.host = None
        else:
            self.host = torch.zeros(self.N, self.Dv).pin_memory()
            if init == "uniform":
                b = math.sqrt(1.0 / self.N)
                self.host[:, :self.D].uniform_(-b, b, generator=torch.Generator().manual_seed(seed))
            elif init == "row_index":
                self.host[:, :self.D] = torch.arange(self.N, dtype=torch.float32).unsqueeze(1)
        self.cache = GpuCache(cache_rows, self.Dv, dev)
        self.status = self.cache.status
        self.side = torch.cuda.Stream(device=dev)
        self.slots = [_Slot(self.cap, self.Dv, dev) for _ in range(self.L + 1)]
        self._ugrad = torch.empty(self.cap, self.D, device=dev)
        self._unorm = torch.empty(self.cap, device=dev)
        self._vals = torch.empty(self.cap, self.Dv, device=dev)
        self._refused = torch.zeros(1, dtype=torch.int32, device=dev)
        self._refused_keys = torch.empty(self.cap, dtype=torch.int64, device=dev)
        self._apply_missing = torch.zeros(1, dtype=torch.int32, device=dev)
        self._cur: Optional[_Slot] = None
        self.stats = {"lookups": 0, "unique": 0, "staged_rows": 0, "staged_bytes": 0, "written_back_rows": 0, "late_announcements": 0}
        self._q: "queue.Queue" = queue.Queue()
        self._worker_error: Optional[BaseException] = None
        self._hold = threading.Event()                # tests: set() makes the worker hold the staging of the next batch
        self._worker = threading.Thread(target=self._work, daemon=True)
        self._worker.start()

    # ------------------------------------------------------------------ host worker (one FIFO)
    def _work(self):
        torch.cuda.set_device(self.dev)
        while True:
            task = self._q.get()
            if task is None:
                return
            try:
                task()
            except BaseException as e:     # noqa: BLE001 - surfaced by the next call on the training thread
                self._worker_error = e

    def _check_worker(self):
        if self._worker_error is not None:
            e, self._worker_error = self._worker_error, None
            raise e

    def close(self):
        self._q.put(None)
        self._worker.join(timeout=5)
        if self.kv is not None and not self._worker.is_alive():
            self.kv.close()
            self.kv = None

    # ------------------------------------------------------------------ announce a future batch
    def prefetch(self, ids: torch.Tensor, step: int) -> None:
        """Announces that ``ids`` (device or host, int64) will be looked up at ``step``."""
        self._check_worker()
        n = ids.numel()
        assert n <= self.cap
        s = self.slots[step % len(self.slots)]
        if not s.writeback_done.wait(self.timeout):
            raise _lib.RecStoreError(_lib.ERR_TIMEOUT, "the write-back of the batch that used these buffers has not finished")
        s.step, s.n = step, n
        s.staged_queued.clear()
        cur = torch.cuda.current_stream(self.dev)
        self.side.wait_stream(cur)
        with torch.cuda.stream(self.side):
            s.ids[:n].copy_(ids, non_blocking=True)
            s.uniq.fill_(-1)
            _lib.call("rs_unique_keys", ptr(s.ids), n, ptr(s.sk), ptr(s.si), s.nslots, ptr(s.uniq), ptr(s.inv), ptr(s.ucount),
                      ptr(self.status), stream_ptr())
            # probe: hits get a fresh stamp (= protected until they are used), misses are listed
            _lib.call("rs_cache_query_noclock", self.cache._h, ptr(s.uniq), n, None, ptr(s.miss_index), ptr(s.miss_keys),
                      ptr(s.miss_count), stream_ptr())
            s.miss_keys_host[:n].copy_(s.miss_keys[:n], non_blocking=True)
            s.miss_count_host.copy_(s.miss_count, non_blocking=True)
            s.probed.record(self.side)

        def stage():
            if self._hold.is_set():               # (tests) the staging signal is withheld
                return
            s.probed.synchronize()
            m = int(s.miss_count_host.item())
            if m:
                self._host_gather(s.miss_keys_host, m, s.rows_host)
            with torch.cuda.stream(self.side):
                if m:
                    s.rows_dev[:m].copy_(s.rows_host[:m], non_blocking=True)      # one cudaMemcpyAsync for the staged block
                s.staged.record(self.side)
            s.staged_bytes = m * self.Dv * 4
            self.stats["staged_rows"] += m
            self.stats["staged_bytes"] += s.staged_bytes
            s.staged_queued.set()
        self._q.put(stage)

    # ------------------------------------------------------------------ forward
    def lookup(self, ids: torch.Tensor, step: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Rows of ``ids`` at ``step``; ``ids`` is the batch that was announced for ``step`` (announced now if it was not)."""
        self._check_worker()
        s = self.slots[step % len(self.slots)]
        if s.step != step:
            self.stats["late_announcements"] += 1
            self.prefetch(ids, step)
        n = s.n
        assert ids.numel() == n
        if not s.staged_queued.wait(self.timeout):
            raise _lib.RecStoreError(_lib.ERR_TIMEOUT, f"the staged rows of step {step} were not delivered within {self.timeout} s")
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_event(s.staged)
        sp = stream_ptr()
        _lib.call("rs_cache_set_clock", self.cache._h, step + 1, sp)
        s.evict_count.zero_()
        # insert the staged rows; rows stamped since the announcement of THIS batch (L steps ago) stay; dirty victims are
        # copied out
        _lib.call("rs_cache_replace_evict", self.cache._h, ptr(s.miss_keys), ptr(s.miss_count), n, ptr(s.rows_dev),
                  max(step - self.L, 0), ptr(s.evict_keys), ptr(s.evict_rows), ptr(s.evict_count), ptr(self._refused_keys),
                  ptr(self._refused), ptr(self.status), sp)
        s.evict_keys_host[:n].copy_(s.evict_keys[:n], non_blocking=True)
        s.evict_count_host.copy_(s.evict_count, non_blocking=True)
        s.evicted.record(cur)
        s.writeback_done.clear()

        def write_back():
            s.evicted.synchronize()
            m = int(s.evict_count_host.item())
            if m:
                s.evict_rows_host[:m].copy_(s.evict_rows[:m])          # D2H of the evicted block (worker thread, blocking)
                self._host_scatter(s.evict_keys_host, m, s.evict_rows_host)
                self.stats["written_back_rows"] += m
            s.writeback_done.set()
        self._q.put(write_back)
        # read the batch from the cache; an id whose set refused the insert is reported in the status word
        _lib.call("rs_cache_query_noclock", self.cache._h, ptr(s.uniq), n, ptr(self._vals), ptr(s.miss_index), ptr(s.miss_keys),
                  ptr(s.miss_count), sp)
        if out is None:
            out = torch.empty(n, self.D, device=self.dev)
        vals = self._vals[:, :self.D]
        # expand: out[i] = vals[inv[i]] (strided source: through a gather on the weights view)
        out.copy_(vals[s.inv[:n].long()])
        self._mark_refusals()
        self._cur = s
        self.stats["lookups"] += n
        return out

    def _mark_refusals(self):
        # refused inserts -> DEV_TABLE_FULL in the status word, without a host read (one tiny kernel via torch)
        self.status.bitwise_or_((self._refused > 0).to(torch.int64) * _lib.DEV_TABLE_FULL)

    # ------------------------------------------------------------------ backward
    def update(self, grads: torch.Tensor) -> None:
        """Applies the optimizer to the rows of the last lookup (``grads`` [n, D] fp32, one row per looked-up id)."""
        s = self._cur
        assert s is not None and grads.shape == (s.n, self.D) and grads.dtype == torch.float32
        n, sp = s.n, stream_ptr()
        grads = grads.contiguous()
        self._ugrad[:n].zero_()
        self._unorm[:n].zero_()
        _lib.call("rs_segment_sum", ptr(grads), ptr(s.inv), n, self.D, ptr(self._ugrad), ptr(self._unorm), sp)
        _lib.call("rs_cache_apply", self.cache._h, ptr(s.uniq), ptr(s.ucount), n, ptr(self._ugrad), ptr(self._unorm), self.D, self.lr,
                  self.eps, 1 if self.optimizer == "rowwise_adagrad" else 0, ptr(s.miss_index), ptr(self._apply_missing), sp)
        self.status.bitwise_or_((self._apply_missing > 0).to(torch.int64) * _lib.DEV_TABLE_FULL)

    # ------------------------------------------------------------------ whole-table access
    def flush(self) -> None:
        """Writes every dirty cached row back to ``host`` (synchronous): before a checkpoint or a comparison."""
        self._check_worker()
        done = threading.Event()
        self._q.put(done.set)
        if not done.wait(self.timeout):
            raise _lib.RecStoreError(_lib.ERR_TIMEOUT, "the host worker did not drain")
        cap = self.cache.capacity
        keys = torch.empty(cap, dtype=torch.int64, device=self.dev)
        rows = torch.empty(cap, self.Dv, device=self.dev)
        cnt = torch.zeros(1, dtype=torch.int32, device=self.dev)
        _lib.call("rs_cache_flush_dirty", self.cache._h, ptr(keys), ptr(rows), ptr(cnt), stream_ptr())
        m = int(cnt.item())
        if m:
            k, r = keys[:m].cpu(), rows[:m].cpu()
            self._host_scatter(k.contiguous(), m, r.contiguous())

    # ------------------------------------------------------------------ host tier (dense array or KV engine)
    def _initial_rows(self, keys: torch.Tensor) -> torch.Tensor:
        """Rows of keys the engine has never stored: a pure function of (seed, key, column)."""
        n = keys.numel()
        out = torch.zeros(n, self.Dv)
        if self._init == "row_index":
            out[:, :self.D] = keys.to(torch.float32).unsqueeze(1)
        elif self._init == "uniform":
            # splitmix64 of (key * D + column + seed), top 24 bits -> U(-b, b); int64 arithmetic wraps like uint64
            x = keys.view(-1, 1) * self.D + torch.arange(self.D, dtype=torch.int64) + (self._seed * 0x632BE59B + 0x9E3779B9)
            x = (x ^ (x >> 30).bitwise_and(0x3FFFFFFFF)) * -0x40A7B892E31B1A47
            x = (x ^ (x >> 27).bitwise_and(0x1FFFFFFFFF)) * -0x6B2FB644ECCEEE15
            x = x ^ (x >> 31).bitwise_and(0x1FFFFFFFF)
            u = ((x >> 40).bitwise_and(0xFFFFFF)).to(torch.float32) / float(1 << 24)
            out[:, :self.D] = (u * 2 - 1) * math.sqrt(1.0 / self.N)
        return out

    def _host_gather(self, keys_host: torch.Tensor, m: int, rows_host: torch.Tensor) -> None:
        if self.kv is None:
            _lib.call("rs_host_gather_rows", self.host.data_ptr(), self.N, self.Dv, keys_host.data_ptr(), m, rows_host.data_ptr())
            return
        k = keys_host[:m]
        rows, found = self.kv.BatchGet(k)
        if not bool(found.all()):
            miss = ~found
            rows[miss] = self._initial_rows(k[miss])
        rows_host[:m].copy_(rows)

    def _host_scatter(self, keys: torch.Tensor, m: int, rows: torch.Tensor) -> None:
        if self.kv is None:
            _lib.call("rs_host_scatter_rows", self.host.data_ptr(), self.N, self.Dv, keys.data_ptr(), m, rows.data_ptr())
        else:
            self.kv.BatchPut(keys[:m], rows[:m])

    def host_rows(self, keys) -> torch.Tensor:
        """``[n, dim + 1]``: weights and Adagrad state of ``keys`` as the host tier holds them (call :meth:`flush` first)."""
        k = torch.as_tensor(keys, dtype=torch.int64).cpu().contiguous()
        buf = torch.empty(k.numel(), self.Dv)
        self._host_gather(k, k.numel(), buf)
        return buf[:, : self.D + 1]

    def check(self) -> None:
        self._check_worker()
        word = int(self.status.item()) & 0xFFFFFFFFFFFFFFFF
        if word:
            self.status.zero_()
            self._refused.zero_()
            self._apply_missing.zero_()
            raise _lib.DeviceStatusError(_lib.ERR_CAPACITY if word & _lib.DEV_TABLE_FULL else _lib.ERR_INVALID,
                                         "device status: " + _lib.decode_status(word) +
                                         (" (a cache set was full of protected rows: enlarge the cache)" if word & _lib.DEV_TABLE_FULL else ""))

    def weights(self) -> torch.Tensor:
        """Host view of the weights (call :meth:`flush` first); dense host tier only, see :meth:`host_rows`."""
        assert self.host is not None, "a hashed host tier has no dense view: use host_rows(keys)"
        return self.host[:, :self.D]

    def state(self) -> torch.Tensor:
        assert self.host is not None, "a hashed host tier has no dense view: use host_rows(keys)"
        return self.host[:, self.D]
