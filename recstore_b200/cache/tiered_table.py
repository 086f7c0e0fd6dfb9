"""Two-tier embedding table of one GPU: hot id range in HBM, the rest in pinned host memory read in place.

``TieredEmbeddingTable(num_rows, dim, hbm_ratio)`` keeps rows ``[0, hot_rows)`` (ids in popularity order: hot ids
first, which is what the renumbering step produces) in an HBM tensor and rows ``[hot_rows, num_rows)`` in a pinned
host tensor that the kernels address directly.  ``lookup(ids)`` folds duplicate ids, gathers every distinct row once
from its tier and expands; ``update(grads)`` segment-sums the gradients of the last lookup and applies SGD or
row-wise Adagrad on both tiers in one kernel.  ``hit_stats()`` reports how many distinct rows came from HBM.

**Lookahead prefetch.**  ``prefetch(next_ids)`` runs the duplicate folding and the gather of the NEXT step's rows on a
side stream while the current step is still computing (the host-tier reads are the slow part; BagPipe-style lookahead
hides them); ``update()`` of the current step then re-reads, from the staged rows, exactly those that it has just
changed (membership in its own folding hash), so the staged copy is what a fresh gather would return; the next
``lookup(next_ids)`` only expands the staged rows.

This is the storage of the PS / cache micro-benchmark (HBM cache of 10 % over a host-DRAM tier) and the native
counterpart of the reference's known-range cache over a UVA-mapped host table
(src/python/pytorch/recstore/cache/local_cache.py:357-467, src/framework/pytorch/recstore_pytorch.cu:12-64).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _lib
from .._lib import f32, i32, i64, ptr, stream_ptr, u64, vp

_lib.register_signatures({
    "rs_tiered_gather": (i32, [vp, vp, i64, i64, vp, i64, i32, vp, vp, vp, vp]),
    "rs_tiered_apply": (i32, [vp, vp, vp, vp, i64, i64, vp, i64, i32, vp, vp, f32, f32, i32, vp]),
    "rs_tiered_refresh": (i32, [vp, vp, i64, i64, vp, i64, i32, vp, vp, u64, vp, vp]),
    "rs_unique_keys": (i32, [vp, i64, vp, vp, u64, vp, vp, vp, vp, vp]),
    "rs_segment_sum": (i32, [vp, vp, i64, i32, vp, vp, vp]),
    "rs_expand_rows": (i32, [vp, vp, i64, i32, vp, vp]),
})


class TieredEmbeddingTable:
    def __init__(self, num_rows: int, dim: int, hbm_ratio: float = 0.1, max_keys: int = 1 << 18, *, lr: float = 0.01,
                 eps: float = 1e-10, optimizer: str = "rowwise_adagrad", device: Optional[torch.device] = None,
                 init: str = "uniform", seed: int = 0, status: Optional[torch.Tensor] = None):
        assert dim % 4 == 0 and 0.0 <= hbm_ratio <= 1.0
        self.N, self.D, self.cap = int(num_rows), int(dim), int(max_keys)
        self.dev = dev = torch.device(device if device is not None else "cuda")
        self.hot_rows = min(self.N, int(math.ceil(self.N * hbm_ratio)))
        self.cold_rows = self.N - self.hot_rows
        self.lr, self.eps, self.optimizer = lr, eps, optimizer
        b = math.sqrt(1.0 / self.N)
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.hot = torch.empty(self.hot_rows, self.D, device=dev)
        self.cold = torch.empty(self.cold_rows, self.D, pin_memory=True) if self.cold_rows else None
        if init == "uniform":
            self.hot.uniform_(-b, b)
            if self.cold is not None:
                self.cold.uniform_(-b, b, generator=g)
        elif init == "row_index":                    # row i holds the value i (tests)
            self.hot.copy_(torch.arange(self.hot_rows, dtype=torch.float32).unsqueeze(1).expand(-1, self.D))
            if self.cold is not None:
                self.cold.copy_(torch.arange(self.hot_rows, self.N, dtype=torch.float32).unsqueeze(1).expand(-1, self.D))
        else:
            raise ValueError(init)
        adagrad = optimizer == "rowwise_adagrad"
        self.hot_state = torch.zeros(self.hot_rows, device=dev) if adagrad else None
        self.cold_state = torch.zeros(self.cold_rows, pin_memory=True) if adagrad and self.cold_rows else None
        n = self.cap
        nslots = 2
        while nslots < 2 * n:
            nslots <<= 1
        self._nslots = nslots

        class _Scratch:
            pass
        self._sc = []
        for _ in range(2):          # two sets: the step whose update is pending, and the step prefetched behind it
            sc = _Scratch()
            sc.sk = torch.empty(nslots, dtype=torch.int64, device=dev)
            sc.si = torch.empty(nslots, dtype=torch.int32, device=dev)
            sc.uniq = torch.empty(n, dtype=torch.int64, device=dev)
            sc.inv = torch.empty(n, dtype=torch.int32, device=dev)
            sc.ucount = torch.zeros(1, dtype=torch.int32, device=dev)
            sc.urows = torch.empty(n, self.D, device=dev)
            sc.n, sc.ids, sc.ev = 0, None, torch.cuda.Event()
            self._sc.append(sc)
        self._cur = 0                # scratch of the last lookup (its update may still come)
        self._pf: Optional[int] = None
        self.s_pf = torch.cuda.Stream(device=dev)
        self._ugrad = torch.empty(n, self.D, device=dev)
        self._unorm = torch.empty(n, device=dev)
        self._counters = torch.zeros(3, dtype=torch.int64, device=dev)     # HBM rows, host rows, staged rows read again
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int64, device=dev)
        self.prefetched_lookups = 0

    # ------------------------------------------------------------------
    def _fold_and_gather(self, sc, ids: torch.Tensor, sp) -> None:
        n = ids.numel()
        sc.n = n
        sc.uniq[:n].fill_(-1)
        _lib.call("rs_unique_keys", ptr(ids), n, ptr(sc.sk), ptr(sc.si), self._nslots, ptr(sc.uniq), ptr(sc.inv),
                  ptr(sc.ucount), ptr(self.status), sp)
        _lib.call("rs_tiered_gather", ptr(self.hot), ptr(self.cold), self.hot_rows, self.N, ptr(sc.uniq), n, self.D,
                  ptr(sc.urows), ptr(self._counters), ptr(self.status), sp)

    def prefetch(self, next_ids: torch.Tensor) -> None:
        """Stages the rows of the NEXT lookup on a side stream.  Pass the same tensor object to ``lookup`` afterwards;
        at most one ``update`` (of the current step) may lie in between."""
        next_ids = next_ids.contiguous()
        assert next_ids.numel() <= self.cap and next_ids.is_cuda and next_ids.dtype == torch.int64
        j = 1 - self._cur
        sc = self._sc[j]
        self.s_pf.wait_stream(torch.cuda.current_stream(self.dev))     # the ids exist; earlier users of this scratch are done
        with torch.cuda.stream(self.s_pf):
            self._fold_and_gather(sc, next_ids, stream_ptr())
            sc.ev.record()
        sc.ids = next_ids
        self._pf = j

    def lookup(self, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = ids.numel()
        assert n <= self.cap and ids.is_cuda and ids.dtype == torch.int64
        sp = stream_ptr()
        if self._pf is not None and self._sc[self._pf].ids is ids:
            sc = self._sc[self._pf]
            torch.cuda.current_stream(self.dev).wait_event(sc.ev)      # staged (and refreshed, which ran on this stream)
            self._cur, self._pf = self._pf, None
            self.prefetched_lookups += 1
        else:
            ids = ids.contiguous()
            self._pf = None                                            # a pending prefetch was for other ids: drop it
            sc = self._sc[self._cur]
            self._fold_and_gather(sc, ids, sp)
        sc.ids = None
        if out is None:
            out = torch.empty(n, self.D, device=self.dev)
        _lib.call("rs_expand_rows", ptr(sc.urows), ptr(sc.inv), n, self.D, ptr(out), sp)
        return out

    def update(self, grads: torch.Tensor) -> None:
        """Optimizer step on the rows of the LAST lookup; ``grads`` [n, D] fp32, one row per looked-up id."""
        sc = self._sc[self._cur]
        n = sc.n
        assert grads.shape == (n, self.D) and grads.dtype == torch.float32 and grads.is_cuda
        sp = stream_ptr()
        self._ugrad[:n].zero_()
        self._unorm[:n].zero_()
        _lib.call("rs_segment_sum", ptr(grads.contiguous()), ptr(sc.inv), n, self.D, ptr(self._ugrad), ptr(self._unorm), sp)
        _lib.call("rs_tiered_apply", ptr(self.hot), ptr(self.hot_state), ptr(self.cold), ptr(self.cold_state), self.hot_rows, self.N,
                  ptr(sc.uniq), n, self.D, ptr(self._ugrad), ptr(self._unorm), self.lr, self.eps,
                  1 if self.optimizer == "rowwise_adagrad" else 0, sp)
        if self._pf is not None:
            # Rows staged for the next step that this update has just changed (or that were read while it ran) are
            # read again, after the gather and after the apply: the staged copy equals a fresh gather.
            pf = self._sc[self._pf]
            torch.cuda.current_stream(self.dev).wait_event(pf.ev)
            _lib.call("rs_tiered_refresh", ptr(self.hot), ptr(self.cold), self.hot_rows, self.N, ptr(pf.uniq), pf.n, self.D,
                      ptr(pf.urows), ptr(sc.sk), self._nslots, ptr(self._counters), sp)
            pf.ev.record()

    def hit_stats(self, reset: bool = True) -> dict:
        """Distinct rows served from HBM / from the host tier since the last reset (synchronises)."""
        c = self._counters.cpu().tolist()
        if reset:
            self._counters.zero_()
        tot = max(1, c[0] + c[1])
        return {"hbm_rows": c[0], "host_rows": c[1], "hit_ratio": c[0] / tot, "staged_rows_refreshed": c[2],
                "prefetched_lookups": self.prefetched_lookups}

    def row(self, i: int) -> torch.Tensor:
        torch.cuda.synchronize(self.dev)
        return self.hot[i].cpu() if i < self.hot_rows else self.cold[i - self.hot_rows].clone()

    def nbytes(self) -> dict:
        return {"hbm": self.hot.numel() * 4, "host": (self.cold.numel() * 4 if self.cold is not None else 0)}
