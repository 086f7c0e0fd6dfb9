"""DLRM whose embedding tables live on sharded parameter servers (runs without a GPU).

Every rank hosts one PS shard and serves it on a loopback port; tables are addressed as
``key = table_prefix + id`` and routed with ``hash(key) % shards``.  ``PSEmbeddingBag`` pulls the rows
of a batch (``GetParameter``), pools them, and pushes the row gradients back with ``UpdateParameter``
(server-side SGD or row-wise Adagrad) when ``step()`` is called.  The MLPs are ordinary torch modules,
averaged across ranks by ``DistributedDataParallel``.  This is the CPU/gloo configuration of the
reference's PS-backed DLRM (src/grpc_ps/python_client/EmbBag.py:8-185 bags over the PS client;
src/executable/dlrm/dlrm_model.py:316-351 dot interaction).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ps import AllShardsParameterClient


class PSEmbeddingBag:
    """Sum / mean pooled bags of one table stored on the parameter servers."""

    def __init__(self, client: AllShardsParameterClient, table_id: int, num_embeddings: int, dim: int, mode: str = "sum",
                 key_prefix_bits: int = 40):
        assert mode in ("sum", "mean")
        self.client, self.table_id, self.N, self.dim, self.mode = client, table_id, num_embeddings, dim, mode
        self.prefix = table_id << key_prefix_bits
        self._trace: List = []

    def init_uniform(self, rank: int, world: int, seed: int = 0, chunk: int = 1 << 16) -> None:
        """U(+-sqrt(1/n)) as in the reference DLRM; rank r uploads ids r, r+world, ..."""
        g = torch.Generator().manual_seed(seed * 7919 + self.table_id)
        b = (1.0 / self.N) ** 0.5
        w = (torch.rand(self.N, self.dim, generator=g) * 2 - 1) * b
        ids = torch.arange(rank, self.N, world)
        for s in range(0, ids.numel(), chunk):
            i = ids[s:s + chunk]
            self.client.PutParameter(i + self.prefix, w[i])

    def __call__(self, indices: torch.Tensor, offsets: Optional[torch.Tensor] = None, per_sample_weights=None) -> torch.Tensor:
        indices = indices.to(torch.int64).reshape(-1)
        rows = self.client.GetParameter(indices + self.prefix).requires_grad_(True)
        if offsets is None:
            offsets = torch.arange(indices.numel())
        nb = offsets.numel()
        lens = torch.diff(torch.cat([offsets, torch.tensor([indices.numel()])]))
        bag = torch.repeat_interleave(torch.arange(nb), lens)
        x = rows if per_sample_weights is None else rows * per_sample_weights.unsqueeze(1)
        out = torch.zeros(nb, self.dim).index_add(0, bag, x)
        if self.mode == "mean":
            out = out / lens.clamp(min=1).unsqueeze(1)
        self._trace.append((indices, rows))
        return out

    def step(self) -> int:
        """Pushes the gradients of every traced lookup to the servers; returns the number of rows updated."""
        n = 0
        for idx, rows in self._trace:
            if rows.grad is not None:
                n += self.client.UpdateParameter(idx + self.prefix, rows.grad)
        self._trace = []
        return n


class PSDLRM(nn.Module):
    """Bottom MLP, PS-backed embedding bags, pairwise dot interaction, top MLP, one logit."""

    def __init__(self, bags: Sequence[PSEmbeddingBag], num_dense: int = 13, bottom=(64, 16), top=(64, 1)):
        super().__init__()
        self.bags = list(bags)
        d = bags[0].dim
        assert bottom[-1] == d
        dims = [num_dense] + list(bottom)
        self.bot = nn.Sequential(*[m for i in range(len(bottom)) for m in (nn.Linear(dims[i], dims[i + 1]), nn.ReLU())])
        F_ = len(bags) + 1
        n_inter = d + F_ * (F_ - 1) // 2
        dims = [n_inter] + list(top)
        layers = []
        for i in range(len(top)):
            layers.append(nn.Linear(dims[i], dims[i + 1]))
            if i < len(top) - 1:
                layers.append(nn.ReLU())
        self.top = nn.Sequential(*layers)
        li, lj = torch.tril_indices(F_, F_, offset=-1)
        self.register_buffer("li", li); self.register_buffer("lj", lj)

    def forward(self, dense: torch.Tensor, emb: torch.Tensor) -> torch.Tensor:
        """``emb`` [B, T, D]: the pooled rows (kept outside the module so that DDP only sees the MLPs)."""
        x = self.bot(dense)
        T = torch.cat([x.unsqueeze(1), emb], 1)
        Z = torch.bmm(T, T.transpose(1, 2))
        return self.top(torch.cat([x, Z[:, self.li, self.lj]], 1)).squeeze(1)

    def lookup(self, ids: Sequence[torch.Tensor]) -> torch.Tensor:
        return torch.stack([bag(i) for bag, i in zip(self.bags, ids)], 1)

    def sparse_step(self) -> int:
        return sum(b.step() for b in self.bags)
