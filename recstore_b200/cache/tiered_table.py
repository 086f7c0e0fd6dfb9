"""Two-tier embedding table of one GPU: hot id range in HBM, the rest in pinned host memory read in place.

``TieredEmbeddingTable(num_rows, dim, hbm_ratio)`` keeps rows ``[0, hot_rows)`` (ids in popularity order: hot ids
first, which is what the renumbering step produces) in an HBM tensor and rows ``[hot_rows, num_rows)`` in a pinned
host tensor that the kernels address directly.  ``lookup(ids)`` folds duplicate ids, gathers every distinct row once
from its tier and expands; ``update(grads)`` segment-sums the gradients of the last lookup and applies SGD or
row-wise Adagrad on both tiers in one kernel.  ``hit_stats()`` reports how many distinct rows came from HBM.

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
        self._sk = torch.empty(nslots, dtype=torch.int64, device=dev)
        self._si = torch.empty(nslots, dtype=torch.int32, device=dev)
        self._uniq = torch.empty(n, dtype=torch.int64, device=dev)
        self._inv = torch.empty(n, dtype=torch.int32, device=dev)
        self._ucount = torch.zeros(1, dtype=torch.int32, device=dev)
        self._urows = torch.empty(n, self.D, device=dev)
        self._ugrad = torch.empty(n, self.D, device=dev)
        self._unorm = torch.empty(n, device=dev)
        self._counters = torch.zeros(2, dtype=torch.int64, device=dev)
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int64, device=dev)
        self._n = 0

    # ------------------------------------------------------------------
    def lookup(self, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        ids = ids.contiguous()
        n = ids.numel()
        assert n <= self.cap and ids.is_cuda and ids.dtype == torch.int64
        sp = stream_ptr()
        self._n = n
        self._uniq[:n].fill_(-1)
        _lib.call("rs_unique_keys", ptr(ids), n, ptr(self._sk), ptr(self._si), self._nslots, ptr(self._uniq), ptr(self._inv),
                  ptr(self._ucount), ptr(self.status), sp)
        _lib.call("rs_tiered_gather", ptr(self.hot), ptr(self.cold), self.hot_rows, self.N, ptr(self._uniq), n, self.D,
                  ptr(self._urows), ptr(self._counters), ptr(self.status), sp)
        if out is None:
            out = torch.empty(n, self.D, device=self.dev)
        _lib.call("rs_expand_rows", ptr(self._urows), ptr(self._inv), n, self.D, ptr(out), sp)
        return out

    def update(self, grads: torch.Tensor) -> None:
        """Optimizer step on the rows of the LAST lookup; ``grads`` [n, D] fp32, one row per looked-up id."""
        n = self._n
        assert grads.shape == (n, self.D) and grads.dtype == torch.float32 and grads.is_cuda
        sp = stream_ptr()
        self._ugrad[:n].zero_()
        self._unorm[:n].zero_()
        _lib.call("rs_segment_sum", ptr(grads.contiguous()), ptr(self._inv), n, self.D, ptr(self._ugrad), ptr(self._unorm), sp)
        _lib.call("rs_tiered_apply", ptr(self.hot), ptr(self.hot_state), ptr(self.cold), ptr(self.cold_state), self.hot_rows, self.N,
                  ptr(self._uniq), n, self.D, ptr(self._ugrad), ptr(self._unorm), self.lr, self.eps,
                  1 if self.optimizer == "rowwise_adagrad" else 0, sp)

    def hit_stats(self, reset: bool = True) -> dict:
        """Distinct rows served from HBM / from the host tier since the last reset (synchronises)."""
        c = self._counters.cpu().tolist()
        if reset:
            self._counters.zero_()
        tot = max(1, c[0] + c[1])
        return {"hbm_rows": c[0], "host_rows": c[1], "hit_ratio": c[0] / tot}

    def row(self, i: int) -> torch.Tensor:
        torch.cuda.synchronize(self.dev)
        return self.hot[i].cpu() if i < self.hot_rows else self.cold[i - self.hot_rows].clone()

    def nbytes(self) -> dict:
        return {"hbm": self.hot.numel() * 4, "host": (self.cold.numel() * 4 if self.cold is not None else 0)}
