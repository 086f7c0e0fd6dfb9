"""Parameter-server client whose shards are HBM hash tables reached over NVLink.

The reference's client talks gRPC to server processes that keep the rows in CPU / SSD engines
(src/grpc_ps/grpc_ps_client.h:33-77, cache_ps_impl.h:34-143).  Inside one box the same verbs -- ``GetParameter``,
``PutParameter``, ``UpdateParameter``, ``ClearPS``, ``SaveCkpt`` / ``LoadCkpt``, ``Stats`` -- are served here by the GPUs
themselves: every rank of the job owns one shard (``csrc/kv/hash_table.cuh`` key -> row, rows and optimizer state in
HBM, owner of a key = key % world), and a request is the fused peer-window exchange of
:class:`~recstore_b200.parallel.sharded_table.ShardedEmbeddingTable` (keys pushed to the owners, rows pushed back,
gradients folded and applied on the owner), without a socket, a server thread or a host copy in between.  The TCP client
(:mod:`recstore_b200.ps.client`) remains the transport for CPU-only deployments.

All verbs are collective over the ranks of the ``PeerContext`` (every rank calls them with its own keys, possibly none).
Semantics follow the TCP server: a key that was never put reads as zeros (``GetParameterWithMask`` tells), ``Put``
overwrites, ``Update`` applies the shard's optimizer (SGD by default, as ``UpdateParameter`` of the reference;
``optimizer="rowwise_adagrad"`` keeps one accumulator per row).
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..parallel.peer import PeerContext
from ..parallel.sharded_table import ShardedEmbeddingTable


class NvlinkParameterClient:
    def __init__(self, ctx: PeerContext, emb_dim: int = 32, capacity: int = 1 << 22, max_batch: int = 1 << 16, *, lr: float = 0.01,
                 optimizer: str = "sgd", name: str = "ps"):
        self.ctx, self.dim = ctx, int(emb_dim)
        self.table = ShardedEmbeddingTable(ctx, name, capacity, emb_dim, max_keys=max_batch, lr=lr, optimizer=optimizer, dedup=True,
                                           init="zeros", init_scale=0.0, hashed=True)
        self.requests = self.keys_served = 0

    def shard(self) -> int:
        return self.ctx.rank

    def _keys(self, keys) -> torch.Tensor:
        return torch.as_tensor(keys, dtype=torch.int64).to(self.ctx.device).reshape(-1)

    def GetParameter(self, keys, perf: bool = True) -> torch.Tensor:
        return self.GetParameterWithMask(keys)[0]

    def GetParameterWithMask(self, keys) -> Tuple[torch.Tensor, torch.Tensor]:
        k = self._keys(keys)
        self.requests += 1
        self.keys_served += k.numel()
        return self.table.get(k)

    def PutParameter(self, keys, values) -> bool:
        k = self._keys(keys)
        v = torch.as_tensor(values, dtype=torch.float32).to(self.ctx.device).reshape(k.numel(), self.dim)
        self.requests += 1
        self.table.put(k, v)
        return True

    def UpdateParameter(self, keys, grads) -> int:
        k = self._keys(keys)
        g = torch.as_tensor(grads, dtype=torch.float32).to(self.ctx.device).reshape(k.numel(), self.dim)
        self.requests += 1
        self.table.push_update(k, g)
        return k.numel()

    def ClearPS(self) -> bool:
        self.table.clear()
        self.ctx.barrier()
        return True

    def LoadFakeData(self, n: int) -> bool:
        """Keys ``0..n-1`` with row value = key (the reference's fake data), this rank loading the keys it owns."""
        mine = torch.arange(self.ctx.rank, n, self.ctx.world, device=self.ctx.device)
        step = self.table.cap
        rounds = (max(n // self.ctx.world + 1, 1) + step - 1) // step
        for i in range(rounds):                       # every rank runs the same number of (collective) puts
            k = mine[i * step:(i + 1) * step]
            self.table.put(k, k.to(torch.float32).unsqueeze(1).expand(-1, self.dim).contiguous())
        return True

    def Stats(self) -> dict:
        keys, _ = self.table.dump()
        n = torch.tensor([keys.numel()], dtype=torch.int64, device=self.ctx.device)
        if self.ctx.world > 1:
            import torch.distributed as dist
            dist.all_reduce(n, group=self.ctx.group)
        return {"keys_stored": int(n.item()), "requests": self.requests, "keys_served": self.keys_served}

    def SaveCkpt(self, path: str) -> bool:
        """One file per shard: ``<path>.shard<r>of<w>`` with the keys and rows this rank holds."""
        keys, rows = self.table.dump()
        torch.save({"keys": keys.cpu(), "rows": rows.cpu(), "dim": self.dim}, f"{path}.shard{self.ctx.rank}of{self.ctx.world}")
        self.ctx.barrier()
        return True

    def LoadCkpt(self, model_config_path=None, emb_file_path=None) -> bool:
        """Loads the shard files of a save made with ANY number of ranks (keys are re-distributed by the put)."""
        import glob
        path = emb_file_path or model_config_path
        files = sorted(glob.glob(f"{path}.shard*of*"))
        if not files:
            raise FileNotFoundError(f"no shard files for {path}")
        step = self.table.cap
        parts = [torch.load(f, map_location="cpu") for i, f in enumerate(files) if i % self.ctx.world == self.ctx.rank]
        k = torch.cat([p["keys"] for p in parts]) if parts else torch.empty(0, dtype=torch.int64)
        v = torch.cat([p["rows"] for p in parts]) if parts else torch.empty(0, self.dim)
        rounds = torch.tensor([(k.numel() + step - 1) // step], dtype=torch.int64, device=self.ctx.device)
        if self.ctx.world > 1:
            import torch.distributed as dist
            dist.all_reduce(rounds, op=dist.ReduceOp.MAX, group=self.ctx.group)
        for i in range(int(rounds.item())):
            self.PutParameter(k[i * step:(i + 1) * step], v[i * step:(i + 1) * step])
        return True
