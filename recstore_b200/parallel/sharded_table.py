"""Row-sharded embedding table over the GPUs of one box (owner(id) = id % world).

``lookup(ids)`` returns the rows of arbitrary global ids on the calling rank; ``update(grads)`` sends
the gradients of the last lookup back to the owners, which segment-reduce duplicates and apply SGD
or row-wise Adagrad in place.  Keys, rows and gradients move with peer stores into NVLink-mapped
windows (``csrc/comm/shard_exchange.cu``); every kernel publishes its own flag when its grid is
done and the consumer waits inside its own prologue, so a lookup is five launches (clear + unique,
bucket-and-push keys, owner-side gather-and-push rows, unbucket-and-expand) and an update four
(segment sum, push, optimizer state, apply).  Nothing is staged through the host and no collective is
called.  Duplicate ids are folded before they travel (``unique_keys`` + ``segment_sum``), which
matters for Zipf / power-law id streams.

Storage of a shard: a dense array indexed by ``id // world`` (ids are row numbers 0..N-1), or, with
``hashed=True``, an HBM hash table (``csrc/kv/hash_table.cuh``) from arbitrary 64-bit keys to rows of
a row store: a key is inserted when it is first looked up and its row starts from values derived
from the key, so a table does not depend on the order in which keys arrive.  ``hbm_ratio < 1`` (dense
storage only) keeps the cold part of every shard in pinned host memory.

This is the storage behind the knowledge-graph entity table (86 M x 400 spread over 8 x HBM) and the
parameter-server micro-benchmark, and the native counterpart of the reference's
``KnownShardedCachedEmbedding`` exchange (src/python/pytorch/recstore/cache/sharded_cache.py:181-345).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _lib
from .._lib import HashTableView, i32, i64, vp, f32, ptr, stream_ptr
from ..ops import functional as F_
from .peer import PeerContext

_lib.register_signatures({
    "rs_shard_push_keys": (i32, [vp, i64, i32, i32, i64, vp, vp, vp, vp, vp, vp, vp]),
    "rs_shard_gather_push_rows": (i32, [vp, i64, vp, vp, vp, vp, i32, i32, i32, i64, C.POINTER(HashTableView), vp, vp]),
    "rs_shard_gather_push_rows_tiered": (i32, [vp, vp, i64, i64, vp, vp, vp, vp, i32, i32, i32, i64, vp, vp]),
    "rs_tiered_apply": (i32, [vp, vp, vp, vp, i64, i64, vp, i64, i32, vp, vp, f32, f32, i32, vp]),
    "rs_rows_gather_checked": (i32, [vp, i64, vp, i64, i32, vp, vp, vp]),
    "rs_shard_unbucket_rows": (i32, [vp, vp, i64, i32, vp, i32, vp]),
    "rs_shard_push_grads": (i32, [vp, vp, i64, i32, i32, i64, vp, vp, vp, vp]),
    "rs_segment_sum": (i32, [vp, vp, i64, i32, vp, vp, vp]),
    "rs_segment_sum_ex": (i32, [vp, vp, i64, i32, vp, vp, vp, vp]),
    "rs_expand_rows": (i32, [vp, vp, i64, i32, vp, vp]),
    "rs_unique_keys": (i32, [vp, i64, vp, vp, _lib.u64, vp, vp, vp, vp, vp]),
    "rs_shard_keys_fused": (i32, [vp, vp, i64, i32, i32, i64, vp, vp, vp, vp, vp, i64, vp, vp, vp, i32, vp]),
    "rs_shard_gather_fused": (i32, [vp, vp, i64, i64, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, C.POINTER(HashTableView), f32, vp,
                                    i64, i32, i32, vp, vp, vp, vp, vp, _lib.u64, i32, i32, vp]),
    "rs_shard_scatter_rows": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i64, vp, vp, _lib.u64, i32, i32, vp, vp]),
    "rs_ht_clear": (i32, [vp, vp]),
    "rs_shard_unbucket_fused": (i32, [vp, vp, vp, i64, i32, vp, i32, vp, vp, vp, vp, vp, i64, vp, vp, _lib.u64, i32, i32, vp, vp]),
    "rs_shard_grads_fused": (i32, [vp, vp, vp, i64, i32, i32, i64, vp, vp, vp, vp, vp, vp, i32, i32, vp]),
    "rs_ht_create": (i32, [_lib.u64, i32, C.POINTER(vp), C.POINTER(HashTableView)]),
    "rs_ht_destroy": (i32, [vp]),
    "rs_ht_dump": (i32, [C.POINTER(HashTableView), vp, vp, vp, _lib.u64, vp]),
})

CH_KEYS, CH_ROWS, CH_GRADS = 8, 9, 10


class ShardedEmbeddingTable:
    def __init__(self, ctx: PeerContext, name: str, num_rows: int, dim: int, max_keys: int, *, lr: float = 0.01,
                 eps: float = 1e-10, optimizer: str = "rowwise_adagrad", dedup: bool = True, init: str = "uniform",
                 init_scale: Optional[float] = None, seed: int = 0, hbm_ratio: float = 1.0, hashed: bool = False,
                 fused: bool = True, range_rows: int = 0, host_table: Optional[torch.Tensor] = None):
        """``range_rows = c > 0`` switches from cyclic to RANGE ownership: rank r holds ids ``[r*c, (r+1)*c)`` in HBM (a
        range-sharded device cache) and ids ``>= world*c`` are rows of ``host_table`` (device-visible host memory), read in
        place by ``lookup`` and left alone by ``update`` (their gradients are the caller's to deliver).  ``init`` is then the
        tensor holding this rank's ``c`` rows."""
        assert dim % 4 == 0
        assert not (hashed and hbm_ratio < 1.0), "the hash-table shard lives in HBM"
        self.range_c = int(range_rows)
        self.host_table = host_table
        assert not (self.range_c and (hashed or hbm_ratio < 1.0)), "range ownership: dense HBM rows only"
        self.ctx, self.name, self.N, self.D = ctx, name, int(num_rows), int(dim)
        self.rank, self.world = ctx.rank, ctx.world
        self.cap = int(max_keys)
        self.lr, self.eps, self.optimizer, self.dedup = lr, eps, optimizer, dedup
        dev = self.dev = ctx.device
        self.hashed, self.fused = bool(hashed), bool(fused) or bool(hashed)
        # dense storage: rows of ids me, me + world, ...; hashed storage: room for this shard's share of N distinct keys
        self.local_rows = (self.N + self.world - 1) // self.world
        if self.range_c:
            self.local_rows = self.range_c
        if self.hashed:
            self.local_rows = int(self.local_rows * 1.25) + 1024        # keys hash unevenly over the owners
        # Two tiers per shard when hbm_ratio < 1: local rows [0, hot_rows) in HBM, the rest in pinned host memory that
        # the kernels address in place.  Local row = id // world, so with ids in popularity order the hot ids of every
        # shard are its first rows.
        self.hot_rows = self.local_rows if hbm_ratio >= 1.0 else max(1, int(math.ceil(self.local_rows * hbm_ratio)))
        self.tiered = self.hot_rows < self.local_rows
        self.cold = torch.empty(self.local_rows - self.hot_rows, self.D, pin_memory=True) if self.tiered else None
        self.weight = torch.empty(self.hot_rows, self.D, device=dev)
        g = torch.Generator(device=dev).manual_seed(seed * 131 + self.rank)
        if isinstance(init, torch.Tensor):
            assert init.shape == (self.hot_rows, self.D)
            self.weight.copy_(init)
        elif init == "uniform":
            b = init_scale if init_scale is not None else math.sqrt(1.0 / self.N)
            self.weight.uniform_(-b, b, generator=g)
            if self.tiered:
                self.cold.uniform_(-b, b, generator=torch.Generator().manual_seed(seed * 131 + self.rank + 7))
        elif init == "zeros":
            self.weight.zero_()
            if self.tiered:
                self.cold.zero_()
        elif init == "row_index":                          # row of global id i holds the value i (tests)
            ids = torch.arange(self.local_rows, dtype=torch.float32) * self.world + self.rank
            full = ids.unsqueeze(1).expand(-1, self.D)
            self.weight.copy_(full[:self.hot_rows])
            if self.tiered:
                self.cold.copy_(full[self.hot_rows:])
        else:
            raise ValueError(init)
        self.init_scale = float(init_scale if init_scale is not None else math.sqrt(1.0 / self.N))
        self._ht = self._ht_view = None
        if self.hashed:
            self._ht, self._ht_view = vp(), HashTableView()
            with torch.cuda.device(dev):
                _lib.call("rs_ht_create", 2 * self.local_rows, self.local_rows, C.byref(self._ht), C.byref(self._ht_view))
            self.row_init = torch.zeros(self.local_rows, dtype=torch.uint8, device=dev)
        adagrad = optimizer == "rowwise_adagrad"
        self.state = torch.zeros(self.hot_rows, device=dev) if adagrad else None
        self.cold_state = torch.zeros(self.local_rows - self.hot_rows, pin_memory=True) if adagrad and self.tiered else None
        W, cap, D = self.world, self.cap, self.D
        self.key_win = ctx.alloc(f"{name}.keys", W * cap * 8)
        self.count_win = ctx.alloc(f"{name}.counts", W * 4)
        self.row_win = ctx.alloc(f"{name}.rows", W * cap * D * 4)
        self.grad_win = ctx.alloc(f"{name}.grads", W * cap * D * 4)
        self.norm_win = ctx.alloc(f"{name}.norms", W * cap * 4)
        self._unorm = torch.empty(W * cap, device=dev)
        self.rowidx = torch.full((W * cap,), -1, dtype=torch.int64, device=dev)
        self._counts = torch.zeros(W, dtype=torch.int32, device=dev)
        self._cursor = torch.zeros(W, dtype=torch.int32, device=dev)
        n = W * cap
        self._slot = torch.empty(n, dtype=torch.int64, device=dev)
        nslots = 2
        while nslots < 2 * n:
            nslots <<= 1
        self._nslots = nslots
        self._sk = torch.empty(nslots, dtype=torch.int64, device=dev)
        self._si = torch.empty(nslots, dtype=torch.int32, device=dev)
        self._uniq = torch.empty(n, dtype=torch.int64, device=dev)
        self._inv = torch.empty(n, dtype=torch.int32, device=dev)
        self._ucount = torch.zeros(1, dtype=torch.int32, device=dev)
        self._urows = torch.empty(n, D, device=dev)
        self._ugrad = torch.empty(n, D, device=dev)
        # compact (row, slot) occurrence list written by the owner-side gather of the fused path, and the "grid done"
        # counters of the kernels that publish their own flag
        self._occ_row = torch.empty(n, dtype=torch.int64, device=dev)
        self._occ_slot = torch.empty(n, dtype=torch.int32, device=dev)
        self._occ_cursor = torch.zeros(1, dtype=torch.int32, device=dev)
        self._grid_done = torch.zeros(4, dtype=torch.int32, device=dev)
        self._n = 0
        self.launches = 0

    def close(self) -> None:
        """Collective: gives the five exchange windows back to the context (with a symmetric heap their bytes are reused
        by the next table; otherwise they are unmapped and freed).  The table must not be used afterwards."""
        for w in ("key_win", "count_win", "row_win", "grad_win", "norm_win"):
            win = getattr(self, w, None)
            if win is not None and win.name in self.ctx.windows:
                self.ctx.free(win.name)
            setattr(self, w, None)

    def __del__(self):
        try:
            if self._ht:
                _lib.lib().rs_ht_destroy(self._ht)
                self._ht = None
        except Exception:
            pass

    # ------------------------------------------------------------------ forward
    def lookup(self, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Rows of ``ids`` ([n] int64 on this device, n <= world * max_keys and at most ``max_keys`` per owner)."""
        ids = ids.contiguous()
        n = ids.numel()
        assert n <= self.world * self.cap
        st, sp = self.ctx.status, stream_ptr()
        self._n = n
        self.launches = 0
        if self.dedup:
            self._uniq[:n].fill_(-1)
            _lib.call("rs_unique_keys", ptr(ids), n, ptr(self._sk), ptr(self._si), self._nslots, ptr(self._uniq), ptr(self._inv),
                      ptr(self._ucount), ptr(st), sp)
            keys = self._uniq
            self.launches += 3
        else:
            keys = ids
        if self.world == 1 and not self.tiered and not self.hashed and not self.range_c:
            # One rank: every row is local (local row = id), so nothing is bucketed or exchanged.
            src_keys = keys[:n]
            if out is None:
                out = torch.empty(n, self.D, device=self.dev)
            dst = self._urows if self.dedup else out
            _lib.call("rs_rows_gather_checked", ptr(self.weight), self.N, ptr(src_keys), n, self.D, ptr(dst), ptr(st), sp)
            if self.dedup:
                _lib.call("rs_expand_rows", ptr(self._urows), ptr(self._inv), n, self.D, ptr(out), sp)
            self._local_rows = src_keys
            self.launches += 2
            return out
        if self.fused:
            return self._lookup_fused(keys, n, out, st, sp)
        _lib.call("rs_shard_push_keys", ptr(keys), n, self.world, self.rank, self.cap, ptr(self._counts), ptr(self._cursor),
                  ptr(self.key_win.table), ptr(self.count_win.table), ptr(self._slot), ptr(st), sp)
        self.ctx.signal(CH_KEYS); self.ctx.wait_own(CH_KEYS)
        if self.tiered:
            _lib.call("rs_shard_gather_push_rows_tiered", ptr(self.weight), ptr(self.cold), self.hot_rows, self.local_rows,
                      self.key_win.local_ptr, self.count_win.local_ptr, ptr(self.row_win.table), ptr(self.rowidx), self.world,
                      self.rank, self.D, self.cap, ptr(st), sp)
        else:
            _lib.call("rs_shard_gather_push_rows", ptr(self.weight), self.local_rows, self.key_win.local_ptr, self.count_win.local_ptr,
                      ptr(self.row_win.table), ptr(self.rowidx), self.world, self.rank, self.D, self.cap, None, ptr(st), sp)
        self.ctx.signal(CH_ROWS); self.ctx.wait_own(CH_ROWS)
        if out is None:
            out = torch.empty(n, self.D, device=self.dev)
        if self.dedup:
            _lib.call("rs_shard_unbucket_rows", self.row_win.local_ptr, ptr(self._slot), n, self.D, ptr(self._urows), 0, sp)
            _lib.call("rs_expand_rows", ptr(self._urows), ptr(self._inv), n, self.D, ptr(out), sp)
            self.launches += 1
        else:
            _lib.call("rs_shard_unbucket_rows", self.row_win.local_ptr, ptr(self._slot), n, self.D, ptr(out), 0, sp)
        self.launches += 9
        return out

    def _lookup_fused(self, keys, n, out, st, sp):
        c = self.ctx
        self._exchange_keys(keys, n, st, sp, push_rows=True)
        if out is None:
            out = torch.empty(n, self.D, device=self.dev)
        ht = self.host_table
        _lib.call("rs_shard_unbucket_fused", self.row_win.local_ptr, ptr(self._slot), ptr(self._inv) if self.dedup else None, n, self.D,
                  ptr(out), 0, ptr(self._ugrad) if self.dedup else None, ptr(self._unorm) if self.dedup else None,
                  ptr(self._ucount) if self.dedup else None, ptr(keys), ht.data_ptr() if ht is not None else None,
                  ht.shape[0] if ht is not None else 0, c.my_flags_ptr, c.counters_ptr, c.wait_timeout_ns, CH_ROWS, self.world,
                  ptr(st), sp)
        self.launches += 4
        return out

    def _exchange_keys(self, keys, n, st, sp, push_rows: bool, find_only: bool = False, folded: Optional[bool] = None):
        """Keys to their owners (+ CH_KEYS), owner-side resolution into the compact occurrence list and, for a lookup, the
        rows back to the askers (+ CH_ROWS)."""
        c, gd = self.ctx, self._grid_done
        folded = self.dedup if folded is None else folded
        self._occ_cursor.zero_()
        _lib.call("rs_shard_keys_fused", ptr(keys), ptr(self._ucount) if folded else None, n, self.world, self.rank, self.cap,
                  ptr(self._cursor), ptr(self.key_win.table), ptr(self.count_win.table), ptr(self._slot), ptr(st), self.range_c,
                  c.flags_table_ptr, c.counters_ptr, ptr(gd[0:1]), CH_KEYS, sp)
        _lib.call("rs_shard_gather_fused", ptr(self.weight), ptr(self.cold), self.hot_rows, self.local_rows, self.key_win.local_ptr,
                  self.count_win.local_ptr, ptr(self.row_win.table), ptr(self.rowidx) if self.tiered else None, ptr(self._occ_row),
                  ptr(self._occ_slot), ptr(self._occ_cursor), self.world, self.rank, self.D, self.cap,
                  C.byref(self._ht_view) if self.hashed else None, self.init_scale, ptr(self.row_init) if self.hashed else None,
                  self.range_c, 1 if push_rows else 0, 1 if find_only else 0, ptr(st), c.my_flags_ptr, c.flags_table_ptr,
                  c.counters_ptr, ptr(gd[1:2]),
                  c.wait_timeout_ns, CH_KEYS, CH_ROWS, sp)

    # ------------------------------------------------------------------ parameter-server verbs (hashed shards)
    def get(self, ids: torch.Tensor):
        """Rows of ``ids`` WITHOUT inserting: ``(rows, found)``; a key that was never put or looked up gives a zero row and
        ``found = False``.  (The owner marks such a row with a NaN in column 0 on the wire.)"""
        assert self.fused and not self.tiered
        ids = ids.contiguous()
        n = ids.numel()
        assert n <= self.world * self.cap
        st, sp = self.ctx.status, stream_ptr()
        self._exchange_keys(ids, n, st, sp, push_rows=True, find_only=self.hashed, folded=False)
        out = torch.empty(n, self.D, device=self.dev)
        c = self.ctx
        _lib.call("rs_shard_unbucket_fused", self.row_win.local_ptr, ptr(self._slot), None, n, self.D, ptr(out), 0, None, None, None,
                  ptr(ids), None, 0, c.my_flags_ptr, c.counters_ptr, c.wait_timeout_ns, CH_ROWS, self.world, ptr(st), sp)
        found = ~torch.isnan(out[:, 0])
        out[~found] = 0
        return out, found

    def put(self, ids: torch.Tensor, values: torch.Tensor) -> None:
        """Stores ``values[i]`` as the row of ``ids[i]`` on its owner (inserting the key if the shard is hashed); the row's
        optimizer state starts over.  Keys of one call should be distinct (of two equal keys one wins)."""
        assert self.fused and not self.tiered
        ids, values = ids.contiguous(), values.contiguous()
        n = ids.numel()
        assert n <= self.world * self.cap and values.shape == (n, self.D) and values.dtype == torch.float32
        st, sp, c = self.ctx.status, stream_ptr(), self.ctx
        self._exchange_keys(ids, n, st, sp, push_rows=False, folded=False)
        _lib.call("rs_shard_grads_fused", ptr(values), ptr(self._slot), None, n, self.D, self.rank, self.cap, ptr(self.grad_win.table),
                  None, None, c.flags_table_ptr, c.counters_ptr, ptr(self._grid_done[2:3]), CH_GRADS, self.world, sp)
        _lib.call("rs_shard_scatter_rows", ptr(self.weight), ptr(self._occ_row), ptr(self._occ_slot), ptr(self._occ_cursor),
                  self.grad_win.local_ptr, ptr(self.state), ptr(self.row_init) if self.hashed else None, self.D, self.world * self.cap,
                  c.my_flags_ptr, c.counters_ptr, c.wait_timeout_ns, CH_GRADS, self.world, ptr(st), sp)

    def clear(self) -> None:
        """Forgets every key of a hashed shard (rows and optimizer state start over)."""
        assert self.hashed
        _lib.call("rs_ht_clear", self._ht, stream_ptr())
        self.row_init.zero_()
        if self.state is not None:
            self.state.zero_()

    def push_update(self, ids: torch.Tensor, grads: torch.Tensor) -> None:
        """A gradient exchange WITHOUT a preceding lookup: ``grads[i]`` is delivered to the owner of ``ids[i]`` and applied
        there (duplicates folded first); ids that belong to the host table are skipped.  This is how a replicated-read cache
        (every rank reads its own hot range and the host table, nobody asks a peer) still gets every rank's updates to the
        rank that holds the row."""
        assert self.fused and not self.tiered
        ids, grads = ids.contiguous(), grads.contiguous()
        n = ids.numel()
        assert n <= self.world * self.cap and grads.shape == (n, self.D) and grads.dtype == torch.float32
        st, sp = self.ctx.status, stream_ptr()
        self._n = n
        self.launches = 0
        if self.dedup:
            _lib.call("rs_unique_keys", ptr(ids), n, ptr(self._sk), ptr(self._si), self._nslots, ptr(self._uniq), ptr(self._inv),
                      ptr(self._ucount), ptr(st), sp)
            keys = self._uniq
            self._ugrad[:n].zero_()
            self._unorm[:n].zero_()
            self.launches += 4
        else:
            keys = ids
        self._exchange_keys(keys, n, st, sp, push_rows=False)
        self.launches += 3
        self._update_fused(grads, n, st, sp)

    def _fold(self, grads, n, sp, norms=None):
        """ugrad / unorm of the unique keys: sums over the occurrences (``norms``: per-occurrence squared norms that
        replace |grad row|^2 in the Adagrad state)."""
        if norms is None:
            _lib.call("rs_segment_sum", ptr(grads), ptr(self._inv), n, self.D, ptr(self._ugrad), ptr(self._unorm), sp)
        else:
            assert norms.numel() == n and norms.dtype == torch.float32 and norms.is_contiguous()
            _lib.call("rs_segment_sum_ex", ptr(grads), ptr(self._inv), n, self.D, ptr(self._ugrad), ptr(self._unorm), ptr(norms), sp)

    def _update_fused(self, grads, n, st, sp, norms=None):
        c = self.ctx
        if self.dedup:      # the accumulators were cleared by the lookup's last kernel
            self._fold(grads, n, sp, norms)
            g, gn, nd = self._ugrad, self._unorm, self._ucount
            self.launches += 1
        else:
            g, gn, nd = grads, None, None
        _lib.call("rs_shard_grads_fused", ptr(g), ptr(self._slot), ptr(nd), n, self.D, self.rank, self.cap, ptr(self.grad_win.table),
                  ptr(gn), ptr(self.norm_win.table) if gn is not None else None, c.flags_table_ptr, c.counters_ptr,
                  ptr(self._grid_done[2:3]), CH_GRADS, self.world, sp)
        nnz = self.world * self.cap
        if self.tiered:
            c.wait_own(CH_GRADS)
            gnorm = self.norm_win.view(torch.float32, (nnz,)) if gn is not None else None
            self._apply_tiered(nnz, gnorm, st, sp)
            self.launches += 11
            return
        F_.emb_backward_ex(self.weight, self.state, self._occ_row, self._occ_slot, nnz, self.grad_win.local, grad_row_stride=self.D,
                           B=nnz, D=self.D, grad_bf16=False, lr=self.lr, eps=self.eps, optimizer=self.optimizer, status=st,
                           gnorm=self.norm_win.local if gn is not None else None, gnorm_stride=1, nnz_dev=self._occ_cursor,
                           ctx=c, wait_channel=CH_GRADS)
        self.launches += 3 if self.optimizer == "rowwise_adagrad" else 2

    # ------------------------------------------------------------------ backward
    def update(self, grads: torch.Tensor, norms: Optional[torch.Tensor] = None) -> None:
        """Applies the optimizer to the rows of the LAST lookup; ``grads`` [n, D] fp32, one row per looked-up id.
        ``norms`` [n] (deduplicating tables only): the squared norm that row-wise Adagrad accounts for each occurrence
        instead of the row's own; rows that are slices of one wider parameter (the D rows of a D x D relation matrix)
        pass the whole parameter's norm / D here and so share ONE accumulator value."""
        n = self._n
        assert grads.shape == (n, self.D) and grads.dtype == torch.float32
        assert norms is None or self.dedup, "per-occurrence norms need a deduplicating table"
        grads = grads.contiguous()
        st, sp = self.ctx.status, stream_ptr()
        if self.world == 1 and not self.tiered and not self.hashed and not self.range_c:
            if self.dedup:
                self._ugrad[:n].zero_()
                self._unorm[:n].zero_()
                self._fold(grads, n, sp, norms)
                g, gn = self._ugrad, self._unorm
            else:
                g, gn = grads, None
            F_.emb_backward(self.weight, self.state, self._local_rows, None, n, g, grad_row_stride=self.D, B=n, D=self.D,
                            grad_bf16=False, lr=self.lr, eps=self.eps, optimizer=self.optimizer, status=st, gnorm=gn, gnorm_stride=1)
            self.launches += 5
            return
        if self.fused:
            return self._update_fused(grads, n, st, sp, norms)
        gnorm = None
        if self.dedup:
            self._ugrad[:n].zero_()
            self._unorm[:n].zero_()
            self._fold(grads, n, sp, norms)
            _lib.call("rs_shard_push_grads", ptr(self._ugrad), ptr(self._slot), n, self.D, self.rank, self.cap,
                      ptr(self.grad_win.table), ptr(self._unorm), ptr(self.norm_win.table), sp)
            gnorm = self.norm_win.view(torch.float32, (self.world * self.cap,))
        else:
            _lib.call("rs_shard_push_grads", ptr(grads), ptr(self._slot), n, self.D, self.rank, self.cap,
                      ptr(self.grad_win.table), None, None, sp)
        self.ctx.signal(CH_GRADS); self.ctx.wait_own(CH_GRADS)
        nnz = self.world * self.cap
        if self.tiered:
            self._apply_tiered(nnz, gnorm, st, sp)
            self.launches += 10
            return
        F_.emb_backward(self.weight, self.state, self.rowidx, None, nnz, self.grad_win.view(torch.float32, (nnz, self.D)),
                        grad_row_stride=self.D, B=nnz, D=self.D, grad_bf16=False, lr=self.lr, eps=self.eps,
                        optimizer=self.optimizer, status=st, gnorm=gnorm, gnorm_stride=1)
        self.launches += 7

    def _apply_tiered(self, nnz: int, gnorm, st, sp) -> None:
        """Owner side of the tiered update: the received (row, gradient) pairs still hold duplicates across source ranks,
        so they are folded once more here (unique + segment sum); every distinct row is then updated by exactly one
        warp with plain loads and stores, which is what makes the host tier safe (no atomics over PCIe)."""
        if not hasattr(self, "_own_uniq"):
            n, dev = nnz, self.dev
            ns = 2
            while ns < 2 * n:
                ns <<= 1
            self._own_ns = ns
            self._own_sk = torch.empty(ns, dtype=torch.int64, device=dev)
            self._own_si = torch.empty(ns, dtype=torch.int32, device=dev)
            self._own_uniq = torch.empty(n, dtype=torch.int64, device=dev)
            self._own_inv = torch.empty(n, dtype=torch.int32, device=dev)
            self._own_cnt = torch.zeros(1, dtype=torch.int32, device=dev)
            self._own_grad = torch.empty(n, self.D, device=dev)
            self._own_norm = torch.empty(n, device=dev)
            self._own_nbuf = torch.empty(n, device=dev)
        rows = torch.where(self.rowidx < 0, torch.full_like(self.rowidx, self.local_rows), self.rowidx)   # empty slots -> a row past the shard (skipped)
        grads = self.grad_win.view(torch.float32, (nnz, self.D))
        self._own_uniq.fill_(-1)
        _lib.call("rs_unique_keys", ptr(rows), nnz, ptr(self._own_sk), ptr(self._own_si), self._own_ns, ptr(self._own_uniq),
                  ptr(self._own_inv), ptr(self._own_cnt), ptr(st), sp)
        self._own_grad.zero_()
        self._own_norm.zero_()
        self._own_nbuf.zero_()
        _lib.call("rs_segment_sum", ptr(grads), ptr(self._own_inv), nnz, self.D, ptr(self._own_grad), ptr(self._own_nbuf), sp)
        if gnorm is not None:      # per-key squared norms travelled with the gradients: add them up per distinct row
            self._own_norm.index_add_(0, self._own_inv.long().clamp_min(0), gnorm.view(-1)[:nnz] * (self.rowidx >= 0))
            norm = self._own_norm
        else:
            norm = self._own_nbuf  # segment_sum's own sum of squares (rows were not folded at the source)
        _lib.call("rs_tiered_apply", ptr(self.weight), ptr(self.state), ptr(self.cold), ptr(self.cold_state), self.hot_rows,
                  self.local_rows, ptr(self._own_uniq), nnz, self.D, ptr(self._own_grad), ptr(norm), self.lr, self.eps,
                  1 if self.optimizer == "rowwise_adagrad" else 0, sp)

    # ------------------------------------------------------------------ whole-table access (tests, checkpoints)
    def local_global_ids(self) -> torch.Tensor:
        return torch.arange(self.local_rows, device=self.dev) * self.world + self.rank

    def dump(self):
        """(keys, rows) of this rank's shard: every key of a hashed shard with its row values, for checkpoints and tests;
        for dense storage the ids ``rank, rank + world, ...`` below ``num_rows`` with theirs."""
        if not self.hashed:
            ids = self.local_global_ids()
            ids = ids[ids < self.N]
            return ids, self.weight[:ids.numel()].clone()
        cap = int(self._ht_view.mask) + 1
        k = torch.empty(cap, dtype=torch.int64, device=self.dev)
        r = torch.empty(cap, dtype=torch.int64, device=self.dev)
        cnt = torch.zeros(1, dtype=torch.int64, device=self.dev)
        _lib.call("rs_ht_dump", C.byref(self._ht_view), ptr(k), ptr(r), ptr(cnt), cap, stream_ptr())
        m = int(cnt.item())
        return k[:m], self.weight[r[:m]]

    def nvlink_bytes_per_lookup(self, n_unique_remote: int) -> int:
        return n_unique_remote * (8 + self.D * 4)
