"""Cached-embedding front ends: one ``forward(keys)`` / ``reg_opt(opt)`` interface over several placements.

Types (``CacheEmbFactory.New``), as in src/python/pytorch/recstore/cache/cache_emb_factory.py:7-67:

* ``TorchNativeStdEmb`` / ``TorchNativeStdEmbDDP``  golden baselines: ``nn.Embedding`` (sparse) on one
  device / replicated under DDP (cache_common.py:60-159).
* ``KnownLocalCachedEmbedding`` (+ ``...Software``)  the "Frugal" placement (local_cache.py:357-471): the full
  table lives in host shared memory, rank r keeps the hot range ``[r*c, (r+1)*c)`` in device memory;
  forward reads the range from the device copy and everything else from the host table (one kernel
  over device-mapped host memory on a GPU); no communication in forward; after backward every rank's
  (keys, grads/world) reach the cache owners and the lookahead controller, which updates the host table
  now or lazily under the read-your-updates contract.
* ``KnownShardedCachedEmbedding``  row-range-sharded device cache (sharded_cache.py:181-345): keys are
  bucketed by owner, exchanged, gathered on the owner, rows exchanged back, misses come from the host
  table; backward sends (keys, grads) to the owners and the miss gradients to the host table.
* ``KGExternelEmbedding``  host table updated directly in backward (cache_common.py:162-220).
* ``LocalCachedEmbedding`` / ``ShardedCachedEmbedding``  the hash-cache forms (local_cache.py:17-110,
  sharded_cache.py:13-178): a set-associative ``GpuCache`` filled on demand instead of a known hot range, per rank
  or sharded by row range; cached copies are updated in backward.

On CUDA devices the two cached placements run on the native data plane: the per-rank hot ranges are the shards of a
range-owned :class:`~recstore_b200.parallel.sharded_table.ShardedEmbeddingTable` (peer windows over NVLink, fused
exchange kernels with in-kernel flags, no NCCL call and no ``torch`` masking on the path); the sharded variant asks
the owners for rows (``lookup``), both deliver every rank's gradients to the owning rank with ``push_update`` (dedup,
key / gradient push, segment-reduce + SGD on the owner), and rows outside the cached ranges are read from the
device-mapped host table inside the same kernels.  The CPU path (gloo) keeps the ``torch`` implementation below.

``args``: ``max_batch_keys`` (native path: most ids one rank looks up or updates per step, default 65,536),
``cache_ratio`` (per-rank fraction c = int(N * ratio)), ``backwardMode`` in {PySync, CppSync, CppAsync,
CppAsyncV2}, ``kForwardItersPerStep``, ``backgrad_init`` (accepted, unused: gradients stay on their device), ``clr``.
Semantics of the update on the cached paths: plain SGD with ``clr`` on the sum over duplicates, gradients pre-divided
by the world size (grad_base.h:456-457, local_cache.py:342-349).
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..dist_tensor import DistEmbedding
from ..utils import comm


def _rank_world() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class CacheShardingPolicy:
    _presampling: Optional[List[int]] = None

    @staticmethod
    def generate_cached_range(num_embeddings: int, cache_ratio: float, world: Optional[int] = None) -> List[Tuple[int, int]]:
        """Rank r caches ids ``[r*c, (r+1)*c)`` with ``c = int(N * ratio)`` (total cached fraction = world * ratio)."""
        world = world if world is not None else _rank_world()[1]
        c = int(num_embeddings * cache_ratio)
        return [(r * c, (r + 1) * c) for r in range(world)]

    @classmethod
    def set_presampling(cls, cache_sizes_all_rank: List[int]) -> None:
        cls._presampling = list(cache_sizes_all_rank)

    @classmethod
    def generate_cached_range_from_presampling(cls) -> List[Tuple[int, int]]:
        assert cls._presampling is not None, "call set_presampling first"
        out, s = [], 0
        for n in cls._presampling:
            out.append((s, s + n))
            s += n
        return out


class AbsEmb(ABC):
    @abstractmethod
    def forward(self, keys: torch.Tensor, trace: bool = True) -> torch.Tensor: ...

    @abstractmethod
    def reg_opt(self, opt) -> None: ...

    def __call__(self, keys, trace: bool = True):
        return self.forward(keys, trace)


class TorchNativeStdEmb(AbsEmb):
    def __init__(self, emb: DistEmbedding, device="cpu"):
        self.device = torch.device(device)
        self.std_emb = nn.Embedding.from_pretrained(emb.weight.clone(), freeze=False, sparse=True).to(self.device)

    def forward(self, keys, trace=True):
        return self.std_emb(keys.to(self.device))

    def reg_opt(self, opt):
        opt.add_param_group({"params": self.std_emb.parameters()})

    @property
    def weight(self):
        return self.std_emb.weight


class TorchNativeStdEmbDDP(AbsEmb):
    """Replicated table; gradients are summed over ranks (dense all-reduce) so every replica stays identical."""

    def __init__(self, emb: DistEmbedding, device="cpu"):
        self.device = torch.device(device)
        self.std_emb = nn.Embedding.from_pretrained(emb.weight.clone(), freeze=False, sparse=False).to(self.device)
        self.world = _rank_world()[1]
        if self.world > 1:
            for p in self.std_emb.parameters():
                p.register_hook(self._allreduce)

    def _allreduce(self, g):
        g = g.clone()
        dist.all_reduce(g)
        return g / self.world

    def forward(self, keys, trace=True):
        return self.std_emb(keys.to(self.device))

    def reg_opt(self, opt):
        opt.add_param_group({"params": self.std_emb.parameters()})

    @property
    def weight(self):
        return self.std_emb.weight


class _CachedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, owner: "_CachedBase", keys, dummy):
        ctx.owner, ctx.keys = owner, keys
        return owner._lookup(keys)

    @staticmethod
    def backward(ctx, grad):
        ctx.owner._push_grad(ctx.keys, grad)
        return None, None, None


class _CachedBase(AbsEmb):
    def __init__(self, emb: DistEmbedding, args: dict, device="cpu"):
        self.emb = emb
        self.device = torch.device(device)
        self.rank, self.world = _rank_world()
        self.N, self.D = emb.shape
        self.ratio = float(args.get("cache_ratio", 0.1))
        self.mode = args.get("backwardMode", "CppSync")
        self.clr = float(args.get("clr", 0.01))
        self.ranges = CacheShardingPolicy.generate_cached_range(self.N, self.ratio, self.world)
        self.start, self.end = self.ranges[self.rank]
        self.full = emb.get_shm_tensor()
        self.cache = self.full[self.start:self.end].to(self.device).clone()
        self._dummy = torch.zeros(1, requires_grad=True, device=self.device)
        self.controller = args.get("controller")          # KGCacheControllerWrapper or None
        self.native = None
        if self.device.type == "cuda" and self.end > self.start:
            self._init_native(int(args.get("max_batch_keys", 65536)))
        self._step_keys: List[torch.Tensor] = []
        self._step_grads: List[torch.Tensor] = []
        self.hits = self.lookups = 0

    _native_count = 0

    def _init_native(self, max_keys: int) -> None:
        """The hot ranges become the shards of a range-owned table on the peer-window transport (collective: every rank
        constructs its embedding at the same point)."""
        from ..kvstore import get_kvstore, kvinit
        from ..parallel.peer import PeerContext
        from ..parallel.sharded_table import ShardedEmbeddingTable
        if not self.full.is_pinned():                      # the kernels read host rows in place
            kv = get_kvstore() or kvinit()
            rc = kv.GetUVAMap(self.full)
            if rc not in (0, 712):
                raise RuntimeError(f"cudaHostRegister of the host table failed with code {rc}")
        _CachedBase._native_count += 1
        self._ctx = PeerContext(self.rank, self.world, device=self.device)
        self.native = ShardedEmbeddingTable(self._ctx, f"cached_emb{_CachedBase._native_count}", self.N, self.D, max_keys=max_keys,
                                            lr=self.clr, optimizer="sgd", dedup=True, init=self.cache,
                                            range_rows=self.end - self.start, host_table=self.full)
        self.cache = self.native.weight                    # one copy: the shard IS the cache

    def forward(self, keys, trace=True):
        keys = keys.to(self.device)
        return _CachedFn.apply(self, keys, self._dummy)

    def reg_opt(self, opt):
        pass                                               # the cache is updated by after_backward()

    # -------------------------------------------------------------- to be provided
    def _lookup(self, keys): raise NotImplementedError

    def _push_grad(self, keys, grad):
        self._step_keys.append(keys.detach())
        self._step_grads.append(grad.detach() / self.world)

    def _apply_cache(self, keys, grads):
        """cache[keys - start] -= clr * grads, duplicates summed, keys already restricted to my range."""
        if keys.numel() == 0:
            return
        if self.cache.is_cuda:
            from ..ops import functional as F_
            rows = (keys - self.start).contiguous()
            F_.emb_backward(self.cache, None, rows, None, rows.numel(), grads.float().contiguous(), grad_row_stride=self.D,
                            B=max(rows.numel(), 1), D=self.D, grad_bf16=False, lr=self.clr, optimizer="sgd")
        else:
            self.cache.index_add_(0, keys - self.start, -self.clr * grads.float())

    def _host_update(self, keys, grads):
        """Sends every rank's (keys, grads) to the controller on rank 0 (or applies them directly without one)."""
        ks = comm.gather_variable_shape_tensor(keys.cpu(), 0)
        gs = comm.gather_variable_shape_tensor(grads.float().cpu(), 0)
        if self.rank != 0:
            return
        ctrl = getattr(self.controller, "controller", None)
        if ctrl is not None:
            for r, (k, g) in enumerate(zip(ks, gs)):
                ctrl.SetStepInput(r, k, g)
        else:
            for k, g in zip(ks, gs):
                self.full.index_add_(0, k, -self.clr * g)

    def after_backward(self):
        raise NotImplementedError


class KnownLocalCachedEmbedding(_CachedBase):
    software = False

    def _lookup(self, keys):
        self.lookups += keys.numel()
        if self.cache.is_cuda and not self.software:
            from .gpu_cache import uva_cache_query_op
            out = torch.empty(keys.numel(), self.D, device=self.device)
            uva_cache_query_op(out, keys, self.cache, self.full, self.start, self.end)
            return out
        in_cache = (keys >= self.start) & (keys < self.end)
        self.hits += int(in_cache.sum())
        out = torch.empty(keys.numel(), self.D, device=self.device)
        out[in_cache] = self.cache[keys[in_cache] - self.start]
        miss = ~in_cache
        if miss.any():
            out[miss] = self.full[keys[miss].cpu()].to(self.device)
        return out

    def after_backward(self):
        """Every rank's gradients update (a) the cache replica of whichever rank holds the key, (b) the host table
        (through the controller: immediately, or lazily ordered by the published future reads)."""
        keys = torch.cat(self._step_keys) if self._step_keys else torch.empty(0, dtype=torch.int64, device=self.device)
        grads = torch.cat(self._step_grads) if self._step_grads else torch.empty(0, self.D, device=self.device)
        self._step_keys, self._step_grads = [], []
        if self.native is not None:
            self.native.push_update(keys, grads.float())    # (a) on the native plane: owners fold duplicates and apply SGD
            self._host_update(keys, grads)
            if self.controller is not None:
                self.controller.AfterBackward()
            return
        owner = torch.full_like(keys, -1)
        for r, (s, e) in enumerate(self.ranges):
            owner[(keys >= s) & (keys < e)] = r
        kb = [keys[owner == r] for r in range(self.world)]
        gb = [grads[owner == r] for r in range(self.world)]
        if self.world > 1:
            kr, gr = comm.all2all_data_transfer(kb), comm.all2all_data_transfer(gb)
            mk, mg = torch.cat(kr), torch.cat(gr)
        else:
            mk, mg = kb[0], gb[0]
        self._apply_cache(mk, mg)
        self._host_update(keys, grads)
        if self.controller is not None:
            self.controller.AfterBackward()


class KnownLocalCachedEmbeddingSoftware(KnownLocalCachedEmbedding):
    software = True


class KnownShardedCachedEmbedding(_CachedBase):
    def _lookup(self, keys):
        self.lookups += keys.numel()
        if self.native is not None:
            return self.native.lookup(keys)       # keys to the owners, rows back, host rows read in place: three fused kernels
        owner = torch.full_like(keys, -1)
        for r, (s, e) in enumerate(self.ranges):
            owner[(keys >= s) & (keys < e)] = r
        out = torch.empty(keys.numel(), self.D, device=self.device)
        pos = [torch.nonzero(owner == r).flatten() for r in range(self.world)]
        if self.world > 1:
            asked = comm.all2all_data_transfer([keys[p] for p in pos])                      # keys other ranks want from me
            rows = comm.all2all_data_transfer([self.cache[k - self.start] for k in asked])  # rows back to the askers
            for p, r in zip(pos, rows):
                out[p] = r
        else:
            out[pos[0]] = self.cache[keys[pos[0]] - self.start]
        miss = owner < 0
        self.hits += int((~miss).sum())
        if miss.any():
            out[miss] = self.full[keys[miss].cpu()].to(self.device)
        return out

    def after_backward(self):
        keys = torch.cat(self._step_keys) if self._step_keys else torch.empty(0, dtype=torch.int64, device=self.device)
        grads = torch.cat(self._step_grads) if self._step_grads else torch.empty(0, self.D, device=self.device)
        self._step_keys, self._step_grads = [], []
        if self.native is not None:
            self.native.push_update(keys, grads.float())
            miss = keys >= self.world * (self.end - self.start)
            self._host_update(keys[miss], grads[miss])
            if self.controller is not None:
                self.controller.AfterBackward()
            return
        owner = torch.full_like(keys, -1)
        for r, (s, e) in enumerate(self.ranges):
            owner[(keys >= s) & (keys < e)] = r
        if self.world > 1:
            mk, mg = comm.all2all_sparse_tensor([keys[owner == r] for r in range(self.world)],
                                                [grads[owner == r] for r in range(self.world)])
        else:
            mk, mg = comm.sum_sparse_tensor([keys[owner == 0]], [grads[owner == 0]])
        self._apply_cache(mk, mg)
        miss = owner < 0
        self._host_update(keys[miss], grads[miss])          # the sharded cache is authoritative for its rows
        if self.controller is not None:
            self.controller.AfterBackward()


class _HostRowCache:
    """Stand-in for :class:`GpuCache` on a CPU device (same Query / Replace / Update surface, LRU over a dict) so that the
    hash-cache placements run under gloo as well."""

    def __init__(self, capacity: int, dim: int):
        from collections import OrderedDict
        self.capacity, self.dim = max(1, capacity), dim
        self.rows: "OrderedDict[int, torch.Tensor]" = OrderedDict()

    def Query(self, keys, values=None, sync=True):
        from .gpu_cache import CacheQueryResult
        n = keys.numel()
        values = torch.zeros(n, self.dim) if values is None else values
        mi, mk = [], []
        for i, k in enumerate(keys.tolist()):
            r = self.rows.get(k)
            if r is None:
                mi.append(i)
                mk.append(k)
            else:
                self.rows.move_to_end(k)
                values[i] = r
        return CacheQueryResult(values, torch.tensor(mi, dtype=torch.int64), torch.tensor(mk, dtype=torch.int64))

    def Replace(self, keys, values):
        for k, v in zip(keys.tolist(), values):
            if k in self.rows:
                self.rows.move_to_end(k)
                continue
            if len(self.rows) >= self.capacity:
                self.rows.popitem(last=False)
            self.rows[k] = v.clone()

    def Update(self, keys, values):
        for k, v in zip(keys.tolist(), values):
            if k in self.rows:
                self.rows[k] = v.clone()


class _HashCachedBase(_CachedBase):
    """Placements whose device cache is a hash cache filled on demand (no key range known in advance).  The reference
    sketches both (local_cache.py:17-110 ``LocalCachedEmbedding``, whose constructor still raises "TODO: update cache in
    backward", and sharded_cache.py:13-178 ``ShardedCachedEmbedding``); here the cached copies ARE updated in backward,
    with the same SGD rule as the host table, so a cached row never goes stale."""

    def __init__(self, emb, args, device="cpu"):
        ratio = float(dict(args).get("cache_ratio", 0.1))
        a = dict(args)
        a["cache_ratio"] = 0.0                                 # no range-owned slice: the base only sets up the host side
        super().__init__(emb, a, device)
        self.ratio = ratio
        cap = max(32, int(self.N * ratio))
        if self.device.type == "cuda":
            from .gpu_cache import GpuCache
            self.gpu_cache = GpuCache(cap, self.D, self.device)
        else:
            self.gpu_cache = _HostRowCache(cap, self.D)

    def _host_rows(self, keys: torch.Tensor) -> torch.Tensor:
        return self.full[keys.cpu()].to(self.device)

    def _query_fill(self, keys: torch.Tensor) -> torch.Tensor:
        """Rows of ``keys``: hits from the cache, misses from the host table (and into the cache for next time)."""
        out = torch.zeros(keys.numel(), self.D, device=self.device)
        if keys.numel() == 0:
            return out
        res = self.gpu_cache.Query(keys, out)
        self.lookups += keys.numel()
        self.hits += keys.numel() - res.missing_keys.numel()
        if res.missing_keys.numel():
            rows = self._host_rows(res.missing_keys)
            out[res.missing_index] = rows
            mk, first = _first_occurrence(res.missing_keys)
            self.gpu_cache.Replace(mk, rows[first])
        return out

    def _update_cached(self, keys: torch.Tensor, grads: torch.Tensor) -> None:
        """Applies row -= clr * (sum of the key's gradients) to the rows of ``keys`` that this rank's cache holds."""
        if keys.numel() == 0:
            return
        uk, inv = torch.unique(keys, return_inverse=True)
        g = torch.zeros(uk.numel(), self.D, device=grads.device, dtype=torch.float32).index_add_(0, inv, grads.float())
        cur = torch.zeros(uk.numel(), self.D, device=self.device)
        res = self.gpu_cache.Query(uk, cur)
        present = torch.ones(uk.numel(), dtype=torch.bool, device=self.device)
        present[res.missing_index] = False
        if present.any():
            self.gpu_cache.Update(uk[present], cur[present] - self.clr * g[present])


def _first_occurrence(keys: torch.Tensor):
    """(unique keys, index of one occurrence of each) so that a batch inserts every missing key once."""
    uk, inv = torch.unique(keys, return_inverse=True)
    first = torch.empty(uk.numel(), dtype=torch.int64, device=keys.device)
    first[inv] = torch.arange(keys.numel(), device=keys.device)
    return uk, first


class LocalCachedEmbedding(_HashCachedBase):
    """Every rank keeps its own hash cache (``cache_ratio`` x table rows) over the shared host table: no communication
    in forward; after backward every rank learns every rank's (keys, gradients), refreshes its cached copies, and the
    host table is updated through the controller."""

    def _lookup(self, keys):
        return self._query_fill(keys)

    def after_backward(self):
        keys = torch.cat(self._step_keys) if self._step_keys else torch.empty(0, dtype=torch.int64, device=self.device)
        grads = torch.cat(self._step_grads) if self._step_grads else torch.empty(0, self.D, device=self.device)
        self._step_keys, self._step_grads = [], []
        if self.world > 1:                                      # any rank may cache any key
            ak = comm.all2all_data_transfer([keys] * self.world)
            ag = comm.all2all_data_transfer([grads] * self.world)
            self._update_cached(torch.cat(ak), torch.cat(ag))
        else:
            self._update_cached(keys, grads)
        self._host_update(keys, grads)
        if self.controller is not None:
            self.controller.AfterBackward()


class ShardedCachedEmbedding(_HashCachedBase):
    """Keys are owned by row range (``linspace(0, N, world + 1)``); the owner answers from its hash cache and fills it
    from the host table on a miss; keys travel to the owners and rows back (two all-to-alls), gradients travel to the
    owners after backward."""

    def __init__(self, emb, args, device="cpu"):
        super().__init__(emb, args, device)
        self.shard_range = [int(x) for x in torch.linspace(0, self.N, self.world + 1).long().tolist()]
        self.shard_range[-1] = self.N

    def _owner(self, keys):
        bounds = torch.tensor(self.shard_range[1:-1], device=keys.device, dtype=keys.dtype)
        return torch.bucketize(keys, bounds, right=True)

    def _lookup(self, keys):
        if self.world == 1:
            return self._query_fill(keys)
        owner = self._owner(keys)
        pos = [torch.nonzero(owner == r).flatten() for r in range(self.world)]
        asked = comm.all2all_data_transfer([keys[p] for p in pos])
        rows = comm.all2all_data_transfer([self._query_fill(k) for k in asked])
        out = torch.empty(keys.numel(), self.D, device=self.device)
        for p, r in zip(pos, rows):
            out[p] = r
        return out

    def after_backward(self):
        keys = torch.cat(self._step_keys) if self._step_keys else torch.empty(0, dtype=torch.int64, device=self.device)
        grads = torch.cat(self._step_grads) if self._step_grads else torch.empty(0, self.D, device=self.device)
        self._step_keys, self._step_grads = [], []
        if self.world > 1:
            owner = self._owner(keys)
            mk = comm.all2all_data_transfer([keys[owner == r] for r in range(self.world)])
            mg = comm.all2all_data_transfer([grads[owner == r] for r in range(self.world)])
            self._update_cached(torch.cat(mk), torch.cat(mg))
        else:
            self._update_cached(keys, grads)
        self._host_update(keys, grads)
        if self.controller is not None:
            self.controller.AfterBackward()


class KGExternelEmbedding(_CachedBase):
    """No device cache: rows come from the host table and the update is applied to it right after backward."""

    def __init__(self, emb, args, device="cpu"):
        args = dict(args); args["cache_ratio"] = 0.0
        super().__init__(emb, args, device)

    def _lookup(self, keys):
        return self.full[keys.cpu()].to(self.device)

    def after_backward(self):
        keys = torch.cat(self._step_keys) if self._step_keys else torch.empty(0, dtype=torch.int64)
        grads = torch.cat(self._step_grads) if self._step_grads else torch.empty(0, self.D)
        self._step_keys, self._step_grads = [], []
        self._host_update(keys, grads)
        if self.controller is not None:
            self.controller.AfterBackward()


class ShmTensorStore:
    """Process-wide registry of named zero-filled tensors in shared memory, so that forked workers see one copy
    (src/python/pytorch/recstore/cache/cache_common.py:244-260)."""

    _tensor_store: dict = {}

    @classmethod
    def GetTensor(cls, name: str):
        return cls._tensor_store.get(name)

    @classmethod
    def RegTensor(cls, name: str, shape, dtype=torch.float32):
        cls._tensor_store[name] = torch.zeros(shape, dtype=dtype).share_memory_()
        return cls._tensor_store[name]


class NVGPUCache:
    """Thin wrapper with the reference's name (cache_common.py:223-241) over :class:`GpuCache`."""

    def __init__(self, capacity: int, feature_dim: int, device=None):
        from .gpu_cache import GpuCache
        self.gpu_cache = GpuCache(capacity, feature_dim, device)

    def Query(self, keys, values):
        return self.gpu_cache.Query(keys, values)

    def Replace(self, keys, values):
        return self.gpu_cache.Replace(keys, values)


class CacheEmbFactory:
    _types = {
        "KnownShardedCachedEmbedding": KnownShardedCachedEmbedding,
        "KnownLocalCachedEmbedding": KnownLocalCachedEmbedding,
        "KnownLocalCachedEmbeddingSoftware": KnownLocalCachedEmbeddingSoftware,
        "KGExternelEmbedding": KGExternelEmbedding,
        "LocalCachedEmbedding": LocalCachedEmbedding,
        "ShardedCachedEmbedding": ShardedCachedEmbedding,
    }

    @staticmethod
    def SupportedCacheType() -> List[str]:
        return list(CacheEmbFactory._types) + ["TorchNativeStdEmb", "TorchNativeStdEmbDDP"]

    @staticmethod
    def New(cache_type: str, emb: DistEmbedding, args: Optional[dict] = None, device="cpu") -> AbsEmb:
        args = dict(args or {})
        if cache_type == "TorchNativeStdEmb":
            return TorchNativeStdEmb(emb, device)
        if cache_type == "TorchNativeStdEmbDDP":
            return TorchNativeStdEmbDDP(emb, device)
        if cache_type not in CacheEmbFactory._types:
            raise ValueError(f"unknown cache type {cache_type!r}; supported: {CacheEmbFactory.SupportedCacheType()}")
        return CacheEmbFactory._types[cache_type](emb, args, device)
