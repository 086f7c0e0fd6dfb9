"""Sparse optimizers over ``DistEmbedding`` tables: ``SparseSGD``, ``SparseAdagrad`` and
``SparseRowWiseAdaGrad``.

Numerics follow the reference (src/python/pytorch/recstore/DistOpt.py): the effective learning
rate is ``lr / world_size`` (:373, :451, :535); ``SparseSGD`` and the element-wise ``SparseAdagrad``
average the gradients of duplicate ids (:384-391, :468-475); ``SparseRowWiseAdaGrad`` keeps one
accumulator per row, adds ``mean(g^2)`` of EVERY occurrence and then applies every occurrence with
the post-step accumulator (:511-557).  The element-wise Adagrad, which the reference disables with
``assert False``, works here.

Checkpoints keep the reference format (:54-116, 164-235): rank r writes ``"{f}_{r}"`` =
``torch.save({"params": {"world_size", "_lr", "_eps"}, "emb_states": {emb: {"ids", "states": {name: tensor}}}})``;
``load`` tolerates another world size (missing file -> warning; fewer ranks -> every rank also loads
the files of the ranks it replaces).
"""
from __future__ import annotations

import os
import warnings
from abc import ABC, abstractmethod
from typing import Dict, List

import torch
import torch.distributed as dist

from .dist_tensor import DistEmbedding, DistTensor, HbmDistEmbedding

EMB_STATES, PARAMS, WORLD_SIZE, IDS, STATES = "emb_states", "params", "world_size", "ids", "states"


def _zero_init(tensor, shape, dtype):
    tensor.zero_()


class DistSparseGradOptimizer(ABC):
    def __init__(self, params: List[DistEmbedding], lr: float):
        self._params = list(params)
        self._lr = lr
        self._state: Dict[str, object] = {}
        self._defaults: Dict[str, float] = {}
        if dist.is_available() and dist.is_initialized():
            self._rank, self._world_size = dist.get_rank(), dist.get_world_size()
        else:
            self._rank, self._world_size = 0, 1

    # ------------------------------------------------------------------ state dicts
    def _states_of(self, emb_name: str) -> List[DistTensor]:
        s = self._state[emb_name]
        return list(s) if isinstance(s, tuple) else [s]

    def local_state_dict(self) -> dict:
        out = {EMB_STATES: {}, PARAMS: {WORLD_SIZE: self._world_size}}
        for emb in self._params:
            if isinstance(emb, HbmDistEmbedding):       # the accumulator is the table's own: this rank's rows of it
                t = emb.table
                idx = t.local_global_ids()
                keep = idx < emb.num_embeddings
                out[EMB_STATES][emb.name] = {IDS: idx[keep].cpu(), STATES: {emb.name + "_hbm_state": t.state[: int(keep.sum())].cpu()}}
                continue
            idx = emb.part_policy.local_ids(self._rank, self._world_size)
            out[EMB_STATES][emb.name] = {IDS: idx, STATES: {st.name: st[idx].clone() for st in self._states_of(emb.name)}}
        out[PARAMS].update(self._defaults)
        return out

    def load_local_state_dict(self, sd: dict) -> None:
        hbm = {e.name: e for e in self._params if isinstance(e, HbmDistEmbedding)}
        for emb_name, emb_state in sd[EMB_STATES].items():
            if emb_name in hbm:       # rows owned by this rank (id % world == rank) take their accumulator values
                t = hbm[emb_name].table
                idx = emb_state[IDS].to(torch.int64)
                val = next(iter(emb_state[STATES].values())).to(torch.float32)
                own = (idx % t.world) == t.rank
                t.state[(idx[own] // t.world).to(t.dev)] = val[own].to(t.dev)
                continue
            if emb_name not in self._state:
                raise ValueError(f"loaded state refers to embedding {emb_name!r} unknown to this optimizer")
            states = {st.name: st for st in self._states_of(emb_name)}
            if len(emb_state[STATES]) != len(states):
                raise ValueError(f"loaded state dict has a different number of states for embedding {emb_name}")
            idx = emb_state[IDS]
            for name, value in emb_state[STATES].items():
                if name not in states:
                    raise ValueError(f"loaded state {name!r} cannot be found in the optimizer states")
                states[name][idx] = value.to("cpu", states[name].dtype)
        p = {k: v for k, v in sd[PARAMS].items() if k != WORLD_SIZE}
        self._defaults.update(p)
        self.__dict__.update(p)

    def save(self, f) -> None:
        """Every rank writes its part to ``f"{f}_{rank}"`` (call on all ranks)."""
        if self._world_size > 1:
            dist.barrier()
        f = os.fsdecode(f)
        torch.save(self.local_state_dict(), f"{f}_{self._rank}")
        if self._world_size > 1:
            dist.barrier()

    def _load_from(self, path: str) -> int:
        sd = torch.load(path, weights_only=False)
        world = sd[PARAMS].get(WORLD_SIZE, 1)
        self.load_local_state_dict(sd)
        return world

    def load(self, f) -> None:
        if self._world_size > 1:
            dist.barrier()
        f = os.fsdecode(f)
        mine = f"{f}_{self._rank}"
        if not os.path.exists(mine):
            warnings.warn(f"File {mine} can't be found, load nothing.")
        else:
            old_world = self._load_from(mine)
            for r in range(self._rank + self._world_size, old_world, self._world_size):
                self._load_from(f"{f}_{r}")
        if self._world_size > 1:
            dist.barrier()

    # ------------------------------------------------------------------ stepping
    @property
    def lr(self) -> float:
        return self._lr

    _hbm_kind = None     # the table optimizer of an HbmDistEmbedding that this class corresponds to

    def step(self) -> None:
        with torch.no_grad():
            for emb in self._params:
                for idx, grad in emb.get_grad():
                    if isinstance(emb, HbmDistEmbedding):
                        # rows and state live in HBM beside each other: the gradients go to the owning GPUs, which fold
                        # duplicates and apply the same rule there (lr / world_size as on the host path)
                        if emb.optimizer_kind != self._hbm_kind:
                            raise TypeError(f"{type(self).__name__} cannot drive an HBM embedding built with optimizer="
                                            f"{emb.optimizer_kind!r}")
                        emb.apply_grad(idx, grad, self._lr / self._world_size)
                    else:
                        self.update(idx, grad, emb)

    def zero_grad(self) -> None:
        for emb in self._params:
            emb.reset_trace()

    @abstractmethod
    def update(self, idx: torch.Tensor, grad: torch.Tensor, emb: DistEmbedding) -> None: ...


def _mean_over_duplicates(idx: torch.Tensor, grad: torch.Tensor):
    uniq, inv, cnt = torch.unique(idx, return_inverse=True, return_counts=True)
    g = torch.zeros(uniq.shape[0], grad.shape[1], dtype=grad.dtype, device=grad.device)
    g.index_add_(0, inv, grad)
    return uniq, g / cnt.unsqueeze(1).to(grad.dtype)


class SparseSGD(DistSparseGradOptimizer):
    _hbm_kind = "sgd"        # on an HBM embedding duplicates are SUMMED (the cached-embedding convention), not averaged

    def __init__(self, params, lr):
        super().__init__(params, lr)
        self._defaults = {"_lr": lr}

    def update(self, idx, grad, emb):
        clr = self._lr / self._world_size
        uniq, g = _mean_over_duplicates(idx.cpu(), grad.detach().cpu().float())
        w = emb.weight
        w[uniq] = w[uniq] - clr * g


class SparseAdagrad(DistSparseGradOptimizer):
    """Element-wise Adagrad: state has the shape of the table."""

    def __init__(self, params, lr, eps=1e-10):
        super().__init__(params, lr)
        self._eps = eps
        self._defaults = {"_lr": lr, "_eps": eps}
        for emb in params:
            assert isinstance(emb, DistEmbedding), "SparseAdagrad only supports DistEmbedding"
            assert emb.name not in self._state, f"{emb.name} already registered in the optimizer"
            self._state[emb.name] = DistTensor((emb.num_embeddings, emb.embedding_dim), torch.float32, emb.name + "_sum",
                                               init_func=_zero_init, part_policy=emb.part_policy, persistent=True,
                                               is_gdata=False)

    def update(self, idx, grad, emb):
        clr = self._lr / self._world_size
        uniq, g = _mean_over_duplicates(idx.cpu(), grad.detach().cpu().float())
        st = self._state[emb.name]
        s = st[uniq] + g * g
        st[uniq] = s
        w = emb.weight
        w[uniq] = w[uniq] - clr * g / (s.sqrt() + self._eps)


class SparseRowWiseAdaGrad(DistSparseGradOptimizer):
    """One accumulator per row; state tensor ``{emb}_SparseRowWiseAdaGrad_sum`` of shape ``(N,)``.  For an
    ``HbmDistEmbedding`` the accumulator is the table's own (``emb.optm_state``) and the update runs on the owning GPU."""
    _hbm_kind = "rowwise_adagrad"

    def __init__(self, params, lr, eps=1e-10):
        super().__init__(params, lr)
        self._eps = eps
        self._defaults = {"_lr": lr, "_eps": eps}
        for emb in params:
            if isinstance(emb, HbmDistEmbedding):
                emb.table.eps = eps
                continue
            assert isinstance(emb, DistEmbedding), "SparseRowWiseAdaGrad only supports DistEmbedding"
            assert emb.name not in self._state, f"{emb.name} already registered in the optimizer"
            self._state[emb.name] = DistTensor((emb.num_embeddings,), torch.float32,
                                               emb.name + "_SparseRowWiseAdaGrad_sum", init_func=_zero_init,
                                               part_policy=emb.part_policy, persistent=True, is_gdata=False)

    def update(self, idx, grad, emb):
        clr = self._lr / self._world_size
        idx = idx.cpu()
        g = grad.detach().cpu().float()
        st = self._state[emb.name].get_shm_tensor()
        st.index_add_(0, idx, g.pow(2).mean(1))
        std = st[idx].sqrt().add_(self._eps)
        emb.weight.index_add_(0, idx, -clr * g / std.unsqueeze(1))
