"""``DistTensor`` and ``DistEmbedding``: named tensors / embedding tables visible to every worker.

Public surface as in the reference (src/python/pytorch/recstore/DistTensor.py:18-185,
DistEmb.py:11-240): create-or-attach by name, ``t[idx]`` / ``t[idx] = v`` on the shared storage,
``init_func(tensor, shape, dtype)`` fills in place, non-persistent tensors are deleted by their
creator; ``DistEmbedding(idx, device)`` gathers rows, attaches a gradient and records the
(ids, rows) trace that the sparse optimizers consume, ``record_grad`` feeds hand-computed
gradients (the cached-embedding paths use it).
"""
from __future__ import annotations

import math
from typing import Iterator, List, Optional, Tuple

import torch

from .kvstore import get_kvstore


class PartitionPolicy:
    """Which ids a rank is responsible for when optimizer state is saved: ``id % world == rank``
    (the split used by the reference's ``local_state_dict``, DistOpt.py:84-96)."""

    def __init__(self, num_ids: int):
        self.num_ids = num_ids

    def local_ids(self, rank: int, world: int) -> torch.Tensor:
        return torch.arange(rank, self.num_ids, world, dtype=torch.int64)


def _default_init(tensor, shape, dtype):
    tensor.zero_()


def uniform_init(tensor, shape, dtype):
    """U(+-sqrt(1/n)), the embedding init of the reference DLRM (dlrm_model.py:121-126)."""
    b = math.sqrt(1.0 / shape[0])
    tensor.uniform_(-b, b)


class DistTensor:
    def __init__(self, shape, dtype, name=None, init_func=None, part_policy=None, persistent=False, is_gdata=True,
                 attach=True):
        if not isinstance(shape, tuple):
            raise TypeError("shape must be a tuple")
        if name is None:
            raise NotImplementedError("anonymous DistTensor is not supported: pass a name")
        self.kvstore = get_kvstore()
        if self.kvstore is None:
            raise RuntimeError("the KV store is not initialised: call recstore_b200.kvinit() first")
        self._shape, self._dtype, self._name = shape, dtype, name
        self._part_policy = part_policy if part_policy is not None else PartitionPolicy(shape[0])
        self._persistent, self._is_gdata, self._attach = persistent, is_gdata, attach
        if name not in self.kvstore.data_name_list():
            self._owner = True
            self.kvstore.init_data(name, shape, dtype, part_policy, init_func or _default_init, is_gdata)
        else:
            self._owner = False
            dtype1, shape1, _ = self.kvstore.get_data_meta(name)
            if dtype1 != dtype or tuple(shape1) != tuple(shape):
                raise ValueError(f"DistTensor {name!r} exists with {shape1}/{dtype1}, asked for {shape}/{dtype}")
        self._weight = self.kvstore.GetRowTensor(name)

    def __del__(self):
        try:
            if not self._persistent and self._owner:
                self.kvstore.Delete(self._name)
        except Exception:
            pass

    def __getitem__(self, idx):
        return self._weight[idx]

    def __setitem__(self, idx, val):
        self._weight[idx] = val

    def __len__(self):
        return self._shape[0]

    def dim(self):
        return len(self._shape)

    def get_shm_tensor(self) -> torch.Tensor:
        return self.kvstore.GetRowTensor(self._name)

    def to_dense_tensor(self) -> torch.Tensor:
        assert self.dim() == 2
        return self.kvstore.GetRowTensor(self._name)

    shape = property(lambda self: self._shape)
    dtype = property(lambda self: self._dtype)
    name = property(lambda self: self._name)
    tensor_name = property(lambda self: self._name)
    kvstore_key = property(lambda self: self._name)
    part_policy = property(lambda self: self._part_policy)


class DistEmbedding:
    def __init__(self, num_embeddings: int, embedding_dim: int, name: Optional[str] = None, init_func=None,
                 part_policy=None):
        self._tensor = DistTensor((num_embeddings, embedding_dim), torch.float32, name, init_func=init_func,
                                  part_policy=part_policy, persistent=True)
        self._trace: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self._hand_grad: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self._name = name
        self._num_embeddings, self._embedding_dim = num_embeddings, embedding_dim
        self._optm_state = None
        self._part_policy = self._tensor.part_policy

    def __call__(self, idx, device=torch.device("cpu"), record_trace: bool = True) -> torch.Tensor:
        idx = torch.as_tensor(idx, dtype=torch.int64)
        emb = self._tensor[idx.cpu()].to(device, non_blocking=True)
        emb.requires_grad_(True)
        if record_trace:
            self._trace.append((idx.to(device, non_blocking=True), emb))
        return emb

    def record_grad(self, idx: torch.Tensor, grad: torch.Tensor) -> None:
        assert len(idx) == len(grad)
        self._hand_grad.append((idx, grad))

    def reset_trace(self) -> None:
        self._trace = []
        self._hand_grad = []

    def get_grad(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        for idx, emb in self._trace:
            if emb.grad is not None:
                yield idx, emb.grad.data
        for idx, grad in self._hand_grad:
            if grad is not None:
                yield idx, grad

    def set_data(self, data: torch.Tensor) -> None:
        assert tuple(data.shape) == self.shape, "shape does not match"
        self.weight.copy_(data)

    def get_shm_tensor(self) -> torch.Tensor:
        return self._tensor.get_shm_tensor()

    name = property(lambda self: self._tensor.tensor_name)
    data_name = property(lambda self: self._tensor.name)
    kvstore = property(lambda self: self._tensor.kvstore)
    num_embeddings = property(lambda self: self._num_embeddings)
    embedding_dim = property(lambda self: self._embedding_dim)
    shape = property(lambda self: (self._num_embeddings, self._embedding_dim))
    optm_state = property(lambda self: self._optm_state)
    weight = property(lambda self: self._tensor.get_shm_tensor())
    part_policy = property(lambda self: self._part_policy)


class HbmDistEmbedding:
    """``DistEmbedding`` whose rows live in the GPUs' HBM instead of host shared memory.

    Same surface as :class:`DistEmbedding` (``emb(idx, device)`` -> rows that record their gradient, ``record_grad``,
    ``get_grad``, ``reset_trace``, ``weight``, ``set_data``, ``name``, ``shape``), so a training loop written against
    the reference API (src/python/pytorch/recstore/DistEmb.py:10-108) runs unchanged, but the table is a row-sharded
    :class:`~recstore_b200.parallel.sharded_table.ShardedEmbeddingTable` over the NVLink peer windows: a lookup sends the
    keys to their owning GPUs and brings the rows back with the fused exchange kernels, and the sparse optimizers of
    ``dist_opt`` deliver the traced gradients to the owners (``push_update``), where duplicates are folded and the
    update is applied in place.  Lookups and optimizer steps are collective: every rank calls them the same number of
    times per step (with any ids, up to ``max_keys`` per call).

    ``optimizer`` ("rowwise_adagrad" or "sgd") is fixed at construction because the state lives beside the rows; the
    ``dist_opt`` optimizer that is given this embedding must be the matching one (it sets the learning rate).
    """

    def __init__(self, ctx, num_embeddings: int, embedding_dim: int, name: str, init_func=None, max_keys: int = 65536,
                 optimizer: str = "rowwise_adagrad", eps: float = 1e-10):
        from .parallel.sharded_table import ShardedEmbeddingTable
        self._ctx = ctx
        self._name = name
        self._num_embeddings, self._embedding_dim = int(num_embeddings), int(embedding_dim)
        self._table = ShardedEmbeddingTable(ctx, "distemb_" + name, num_embeddings, embedding_dim, max_keys=max_keys, lr=0.0, eps=eps,
                                            optimizer=optimizer, dedup=True, init="zeros")
        self.optimizer_kind = optimizer
        if init_func is not None:            # the reference's init_func(tensor, shape, dtype) fills the whole table
            full = torch.empty(num_embeddings, embedding_dim)
            init_func(full, (num_embeddings, embedding_dim), torch.float32)
            self.set_data(full)
        self._trace: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self._hand_grad: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self._optm_state = None

    # ---- DistEmbedding surface
    def __call__(self, idx, device=None, record_trace: bool = True) -> torch.Tensor:
        dev = self._table.dev
        idx = torch.as_tensor(idx, dtype=torch.int64).to(dev)
        emb = self._table.lookup(idx).clone()
        if device is not None and torch.device(device) != dev:
            emb = emb.to(device)
        emb.requires_grad_(True)
        if record_trace:
            self._trace.append((idx, emb))
        return emb

    def record_grad(self, idx: torch.Tensor, grad: torch.Tensor) -> None:
        assert len(idx) == len(grad)
        self._hand_grad.append((idx, grad))

    def reset_trace(self) -> None:
        self._trace = []
        self._hand_grad = []

    def get_grad(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        for idx, emb in self._trace:
            if emb.grad is not None:
                yield idx, emb.grad.data
        for idx, grad in self._hand_grad:
            if grad is not None:
                yield idx, grad

    def apply_grad(self, idx: torch.Tensor, grad: torch.Tensor, lr: float) -> None:
        """One gradient batch to the owners (collective).  Called by the ``dist_opt`` optimizers."""
        t = self._table
        t.lr = float(lr)
        t.push_update(torch.as_tensor(idx, dtype=torch.int64).to(t.dev), grad.detach().to(t.dev, torch.float32))

    def set_data(self, data: torch.Tensor) -> None:
        assert tuple(data.shape) == self.shape, "shape does not match"
        t = self._table
        mine = data[t.rank::t.world].to(t.dev, torch.float32)
        t.weight[: mine.shape[0]].copy_(mine)

    def to_dense_tensor(self) -> Optional[torch.Tensor]:
        """Collective: the whole table on rank 0's host (``None`` elsewhere)."""
        t = self._table
        torch.cuda.synchronize(t.dev)
        local = t.weight.cpu()
        if t.world == 1:
            return local[: self._num_embeddings]
        import torch.distributed as dist
        parts = [None] * t.world if t.rank == 0 else None
        dist.gather_object(local, parts, dst=0, group=self._ctx.group)
        if t.rank != 0:
            return None
        full = torch.empty(t.local_rows * t.world, t.D)
        for r, p in enumerate(parts):
            full[r::t.world] = p
        return full[: self._num_embeddings]

    name = property(lambda self: self._name)
    data_name = property(lambda self: self._name)
    num_embeddings = property(lambda self: self._num_embeddings)
    embedding_dim = property(lambda self: self._embedding_dim)
    shape = property(lambda self: (self._num_embeddings, self._embedding_dim))
    optm_state = property(lambda self: self._table.state)
    weight = property(lambda self: self._table.weight)          # this rank's shard: rows of ids rank, rank + world, ...
    table = property(lambda self: self._table)
    part_policy = property(lambda self: None)
