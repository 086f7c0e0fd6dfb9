"""``EmbeddingBag`` semantics over parameter-server rows, in plain tensor code.

Same options as ``torch.nn.EmbeddingBag`` and as the reference's pure-python bag over its PS client
(src/grpc_ps/python_client/EmbBag.py:8-185): ``mode`` sum / mean / max, ``offsets`` (with or without the trailing end
offset), ``per_sample_weights`` (sum only) and ``padding_idx`` (rows that neither contribute nor receive gradient).
``PSEmbeddingBagModule`` fetches the rows from a client, pools them and hands the row gradients back on ``step()``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch


def pool_rows(rows: torch.Tensor, indices: torch.Tensor, offsets: Optional[torch.Tensor] = None, mode: str = "sum",
              per_sample_weights: Optional[torch.Tensor] = None, padding_idx: Optional[int] = None,
              include_last_offset: bool = False) -> torch.Tensor:
    """Pools ``rows[i]`` (the embedding of ``indices[i]``) into bags; differentiable w.r.t. ``rows``."""
    assert mode in ("sum", "mean", "max")
    n = indices.numel()
    if indices.dim() == 2:                       # fixed-length bags given as a matrix
        assert offsets is None
        nb, L = indices.shape
        offsets = torch.arange(0, nb * L, L)
        indices = indices.reshape(-1)
    elif offsets is None:
        offsets = torch.arange(n)
    offsets = offsets.to(torch.int64)
    if include_last_offset:
        ends, offsets = offsets[1:], offsets[:-1]
    else:
        ends = torch.cat([offsets[1:], torch.tensor([n], dtype=torch.int64)])
    nb = offsets.numel()
    lens = ends - offsets
    bag = torch.repeat_interleave(torch.arange(nb), lens)
    keep = torch.ones(n, dtype=torch.bool) if padding_idx is None else indices != padding_idx
    x = rows
    if per_sample_weights is not None:
        assert mode == "sum", "per_sample_weights only with mode='sum'"
        x = x * per_sample_weights.reshape(-1, 1)
    x = x * keep.unsqueeze(1).to(x.dtype)
    dim = rows.shape[1]
    if mode in ("sum", "mean"):
        out = torch.zeros(nb, dim, dtype=rows.dtype).index_add(0, bag, x)
        if mode == "mean":
            cnt = torch.zeros(nb, dtype=rows.dtype).index_add(0, bag, keep.to(rows.dtype))
            out = out / cnt.clamp(min=1).unsqueeze(1)
        return out
    neg = torch.finfo(rows.dtype).min
    xm = torch.where(keep.unsqueeze(1), rows, torch.full_like(rows, neg))
    out = torch.full((nb, dim), neg, dtype=rows.dtype).scatter_reduce(0, bag.unsqueeze(1).expand(-1, dim), xm, reduce="amax")
    empty = torch.zeros(nb, dtype=torch.bool).index_put((bag[keep],), torch.ones(int(keep.sum()), dtype=torch.bool)).logical_not()
    return torch.where(empty.unsqueeze(1), torch.zeros_like(out), out)


class PSEmbeddingBagModule:
    """Bags of one table whose rows live behind ``client`` (``GetParameter`` / ``UpdateParameter``)."""

    def __init__(self, client, num_embeddings: int, dim: int, mode: str = "sum", padding_idx: Optional[int] = None,
                 key_offset: int = 0, include_last_offset: bool = False):
        self.client, self.N, self.dim, self.mode = client, num_embeddings, dim, mode
        self.padding_idx, self.key_offset, self.include_last_offset = padding_idx, key_offset, include_last_offset
        self._trace: List[Tuple[torch.Tensor, torch.Tensor]] = []

    def __call__(self, indices: torch.Tensor, offsets: Optional[torch.Tensor] = None, per_sample_weights=None) -> torch.Tensor:
        flat = indices.to(torch.int64).reshape(-1)
        rows = self.client.GetParameter(flat + self.key_offset).requires_grad_(True)
        self._trace.append((flat, rows))
        return pool_rows(rows, indices.to(torch.int64), offsets, self.mode, per_sample_weights, self.padding_idx,
                         self.include_last_offset)

    def step(self) -> int:
        n = 0
        for idx, rows in self._trace:
            if rows.grad is None:
                continue
            keep = torch.ones_like(idx, dtype=torch.bool) if self.padding_idx is None else idx != self.padding_idx
            if keep.any():
                n += self.client.UpdateParameter(idx[keep] + self.key_offset, rows.grad[keep])
        self._trace = []
        return n
