"""The two embedding-table objects of the knowledge-graph trainer.

* ``ExternalEmbedding``: a table on one device with its own row-wise Adagrad state, updated from a trace of the rows
  that a step looked up: ``emb(idx)`` returns detached rows that require grad and remembers them, ``update()`` applies
  the gradients that backward left on them.  Optional asynchronous update (a worker applies the updates behind the
  trainer), cross-partition relations kept in a shared global table, ``.npy`` save / load.  Role of
  src/kg/kg/dgl-ke/python/dglke/models/pytorch/tensor_models.py:217-476.
* ``CustomExternalEmbedding``: the same surface over a ``DistEmbedding`` in shared memory, looked up through one of the
  cached embeddings of ``recstore_b200.cache`` and updated by it after backward (role of cus_external_emb.py:20-215;
  unlike there, ``save`` / ``load`` work).
"""
from __future__ import annotations

import os
import queue
import threading
from typing import List, Optional, Tuple

import numpy as np
import torch

from ..baseline.kge_torch import rowwise_adagrad_


class ExternalEmbedding:
    def __init__(self, num: int, dim: int, device="cpu", lr: float = 0.1, eps: float = 1e-10):
        self.num, self.dim, self.lr, self.eps = int(num), int(dim), float(lr), float(eps)
        self.emb = torch.empty(num, dim, dtype=torch.float32, device=device)
        self.state_sum = torch.zeros(num, dtype=torch.float32, device=device)
        self.state_step = 0
        self.trace: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.has_cross_rel = False
        self._async_q: Optional[queue.Queue] = None
        self._async_t: Optional[threading.Thread] = None
        self._async_err: Optional[BaseException] = None

    def init(self, emb_init: float) -> None:
        """Rows uniform in ``[-emb_init, emb_init]``, optimizer state zero."""
        torch.nn.init.uniform_(self.emb, -emb_init, emb_init)
        self.state_sum.zero_()

    def share_memory(self) -> None:
        """Lets forked workers update one copy (Hogwild-style)."""
        self.emb.share_memory_()
        self.state_sum.share_memory_()

    def prepare_per_worker_process(self) -> None:
        pass

    # Relations that occur in more than one worker's partition live in a global table that every worker updates; a
    # worker's own copy of such a row is refreshed from there before it is read (tensor_models.py:259-297).
    def setup_cross_rels(self, cross_rels, global_emb: "ExternalEmbedding") -> None:
        self.cpu_bitmap = torch.zeros(self.num, dtype=torch.bool)
        self.cpu_bitmap[torch.as_tensor(cross_rels, dtype=torch.int64)] = True
        self.global_emb = global_emb
        self.has_cross_rel = True

    def get_noncross_idx(self, idx: torch.Tensor) -> torch.Tensor:
        return idx[~self.cpu_bitmap[idx.cpu()]]

    def __call__(self, idx: torch.Tensor, gpu_id: int = -1, trace: bool = True) -> torch.Tensor:
        idx = torch.as_tensor(idx, dtype=torch.int64)
        if self.has_cross_rel:
            cross = torch.unique(idx.cpu()[self.cpu_bitmap[idx.cpu()]])
            if cross.numel():
                self.emb[cross.to(self.emb.device)] = self.global_emb.emb[cross].to(self.emb.device)
        s = self.emb[idx.to(self.emb.device)]
        if gpu_id >= 0:
            s = s.cuda(gpu_id)
        if not trace:
            return s
        data = s.clone().detach().requires_grad_(True)
        self.trace.append((idx, data))
        return data

    def _apply(self, idx: torch.Tensor, grad: torch.Tensor) -> None:
        dev = self.emb.device
        idx, grad = idx.to(dev), grad.to(dev)
        if self.has_cross_rel:                      # the shared rows take their update in the global table
            mask = self.cpu_bitmap[idx.cpu()].to(dev)
            if bool(mask.any()):
                g = self.global_emb
                rowwise_adagrad_(g.emb, g.state_sum, idx[mask].to(g.emb.device), grad[mask].to(g.emb.device), self.lr, self.eps)
        rowwise_adagrad_(self.emb, self.state_sum, idx, grad, self.lr, self.eps)

    @torch.no_grad()
    def update(self, gpu_id: int = -1) -> None:
        """Row-wise Adagrad over the traced rows, duplicates allowed (state first, then every occurrence's step with
        the new state)."""
        self.state_step += 1
        for idx, data in self.trace:
            if data.grad is None:
                continue
            if self._async_q is not None:
                if self._async_err is not None:
                    raise RuntimeError("asynchronous embedding update failed") from self._async_err
                self._async_q.put((idx, data.grad.detach()))
            else:
                self._apply(idx, data.grad)
        self.trace = []

    # The asynchronous form: updates are handed to a worker and applied while the next step computes, so a step may
    # read rows whose last update is still queued (tensor_models.py:144-182, 433-447; a process there, a thread here:
    # the table is shared either way, and the bounded queue keeps the trainer at most `max_pending` steps ahead).
    def create_async_update(self, max_pending: int = 1) -> None:
        if self._async_t is not None:
            return
        self._async_q = queue.Queue(maxsize=max_pending)

        def run():
            while True:
                item = self._async_q.get()
                try:
                    if item is None:
                        return
                    with torch.no_grad():
                        self._apply(*item)
                except BaseException as e:          # noqa: BLE001 - reported by the trainer's next update / at finish
                    self._async_err = e
                    return
                finally:
                    self._async_q.task_done()
        self._async_t = threading.Thread(target=run, name="external-emb-async-update", daemon=True)
        self._async_t.start()

    def wait_async_update(self) -> None:
        if self._async_t is not None and self._async_err is None:
            self._async_q.join()
        if self._async_err is not None:
            raise RuntimeError("asynchronous embedding update failed") from self._async_err

    def finish_async_update(self) -> None:
        if self._async_t is None:
            return
        if self._async_err is None:
            self._async_q.put(None)
        self._async_t.join()
        self._async_q = self._async_t = None
        if self._async_err is not None:
            raise RuntimeError("asynchronous embedding update failed") from self._async_err

    def curr_emb(self) -> torch.Tensor:
        """The rows in the trace, in lookup order."""
        return torch.cat([d for _, d in self.trace], 0)

    def save(self, path: str, name: str) -> None:
        np.save(os.path.join(path, name + ".npy"), self.emb.detach().cpu().numpy())

    def load(self, path: str, name: str) -> None:
        w = torch.from_numpy(np.load(os.path.join(path, name + ".npy"))).float()
        assert tuple(w.shape) == (self.num, self.dim), f"{name}.npy holds {tuple(w.shape)}, expected {(self.num, self.dim)}"
        self.emb.copy_(w)


class CustomExternalEmbedding:
    """``ExternalEmbedding``'s surface over the shared-memory ``DistEmbedding`` named ``emb_name`` and a cached
    embedding in front of it.  ``cache_args``: ``cache_ratio``, ``backwardMode``, ``clr``, ``controller`` (what
    ``CacheEmbFactory.New`` takes); with ``TorchNativeStdEmb`` / ``TorchNativeStdEmbDDP`` the rows are updated by a
    torch SGD optimizer instead."""

    def __init__(self, num: int, dim: int, emb_name: str, lr: float = 0.1, cached_emb_type: str = "KGExternelEmbedding",
                 cache_args: Optional[dict] = None, device="cpu"):
        from ..dist_tensor import DistEmbedding
        self.num, self.dim, self.lr, self.device = int(num), int(dim), float(lr), device
        self.emb = DistEmbedding(num, dim, name=emb_name)
        self.cached_emb_type = cached_emb_type
        self.cache_args = dict(cache_args or {})
        self.cache_args.setdefault("clr", lr)
        self.cached_emb = None
        self._torch_opt = None
        self.trace: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.has_cross_rel = False

    def init(self, emb_init: float) -> None:
        """Uniform rows; ``emb_init == 0`` zero-fills (what the reference's driver does for the entity table)."""
        w = self.emb.weight
        w.zero_() if emb_init == 0 else torch.nn.init.uniform_(w, -emb_init, emb_init)

    def share_memory(self) -> None:
        pass                                        # the table lives in named shared memory already

    def prepare_per_worker_process(self) -> None:
        """Builds this worker's cached embedding (collective where the cache type is: every worker calls it)."""
        from ..cache import CacheEmbFactory
        self.cached_emb = CacheEmbFactory.New(self.cached_emb_type, self.emb, self.cache_args, self.device)
        if not hasattr(self.cached_emb, "after_backward"):
            self._torch_opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=self.lr)
            self.cached_emb.reg_opt(self._torch_opt)

    def __call__(self, idx: torch.Tensor, gpu_id: int = -1, trace: bool = True) -> torch.Tensor:
        assert self.cached_emb is not None, "call prepare_per_worker_process() in the worker first"
        idx = torch.as_tensor(idx, dtype=torch.int64)
        s = self.cached_emb.forward(idx, trace)
        if gpu_id >= 0:
            s = s.cuda(gpu_id)
        if trace:
            self.trace.append((idx, s))
        return s

    def update(self, gpu_id: int = -1) -> None:
        if self._torch_opt is not None:
            self._torch_opt.step()
            self._torch_opt.zero_grad()
        else:
            self.cached_emb.after_backward()
        self.trace.clear()

    def curr_emb(self) -> torch.Tensor:
        return torch.cat([d for _, d in self.trace], 0)

    def save(self, path: str, name: str) -> None:
        np.save(os.path.join(path, name + ".npy"), self.emb.weight.detach().cpu().numpy())

    def load(self, path: str, name: str) -> None:
        w = torch.from_numpy(np.load(os.path.join(path, name + ".npy"))).float()
        assert tuple(w.shape) == (self.num, self.dim), f"{name}.npy holds {tuple(w.shape)}, expected {(self.num, self.dim)}"
        self.emb.weight.copy_(w)
