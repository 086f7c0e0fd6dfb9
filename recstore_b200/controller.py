"""Lookahead cache controller and samplers (Python side).

``KGCacheController`` wraps the native controller (``csrc/runtime/controller.cpp``) with the method
names of the reference's torch class (src/framework/pytorch/kg_controller.h:36-116):
``Init(json)``, ``RegTensorsPerProcess``, ``ProcessOneStep(step)``, ``BlockToStepN(step)``,
``StopThreads``, ``PrintPq``.  ``CircleBuffer`` / ``BasePerfSampler`` / ``TestPerfSampler`` publish the
ids of the next ``L`` batches (lookahead) as in src/python/pytorch/recstore/controller_process.py:
24-132; ``KGCacheControllerWrapper`` gives the training loop the ``AfterBackward()`` hook
(:376-405): barrier -> rank 0 ``ProcessOneStep`` -> ``BlockToStepN(step + 1)`` -> barrier.

JSON keys understood: ``num_gpus, L, clr, dim, backwardMode (PySync|CppSync|CppAsync|CppAsyncV2),
nr_background_threads, kUpdatePqWorkerNum, full_emb_capacity, cache_ratio``.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Dict, List, Optional

import torch

from . import _lib
from ._lib import cstr, i32, i64, vp

_lib.register_signatures({
    "rs_heap_create": (vp, []),
    "rs_heap_destroy": (None, [vp]),
    "rs_heap_upsert": (None, [vp, i64, i64]),
    "rs_heap_erase": (i32, [vp, i64]),
    "rs_heap_pop": (i32, [vp, C.POINTER(i64), C.POINTER(i64)]),
    "rs_heap_top": (i32, [vp, C.POINTER(i64), C.POINTER(i64)]),
    "rs_heap_size": (i64, [vp]),
    "rs_heap_check": (i32, [vp]),
    "rs_ctrl_create": (i32, [cstr, C.POINTER(vp)]),
    "rs_ctrl_destroy": (i32, [vp]),
    "rs_ctrl_register_table": (i32, [vp, vp, i64]),
    "rs_ctrl_register_cache": (i32, [vp, i32, vp]),
    "rs_ctrl_start": (i32, [vp]),
    "rs_ctrl_stop": (i32, [vp]),
    "rs_ctrl_drain": (i32, [vp]),
    "rs_ctrl_publish_reads": (i32, [vp, i32, i64, vp, i64]),
    "rs_ctrl_set_step_input": (i32, [vp, i32, vp, i64, vp]),
    "rs_ctrl_process_one_step": (i32, [vp, i64]),
    "rs_ctrl_block_to_step": (i32, [vp, i64, i32]),
    "rs_ctrl_pending": (i64, [vp]),
    "rs_ctrl_min_priority": (i64, [vp]),
    "rs_ctrl_print_pq": (i32, [vp, C.c_char_p, i32]),
    "rs_ctrl_stats": (i32, [vp, vp]),
})


class IndexedPriorityQueue:
    """Binary heap with an id -> position index (push / adjust / erase in O(log n)) and an invariant checker."""

    def __init__(self):
        self._l = _lib.lib()
        self._h = self._l.rs_heap_create()

    def __del__(self):
        try:
            self._l.rs_heap_destroy(self._h)
        except Exception:
            pass

    def upsert(self, id_: int, prio: int):
        self._l.rs_heap_upsert(self._h, id_, prio)

    def erase(self, id_: int) -> bool:
        return bool(self._l.rs_heap_erase(self._h, id_))

    def pop(self):
        a, b = i64(), i64()
        return (a.value, b.value) if self._l.rs_heap_pop(self._h, C.byref(a), C.byref(b)) else None

    def top(self):
        a, b = i64(), i64()
        return (a.value, b.value) if self._l.rs_heap_top(self._h, C.byref(a), C.byref(b)) else None

    def __len__(self):
        return int(self._l.rs_heap_size(self._h))

    def CheckConsistency(self) -> bool:
        return bool(self._l.rs_heap_check(self._h))


class KGCacheController:
    _instance: Optional["KGCacheController"] = None

    def __init__(self, json_str: str):
        self._l = _lib.lib()
        self.cfg = json.loads(json_str)
        h = vp()
        _lib.call("rs_ctrl_create", json_str.encode(), C.byref(h))
        self._h = h.value
        self._keep: Dict[str, torch.Tensor] = {}

    @classmethod
    def Init(cls, json_str: str) -> "KGCacheController":
        cls._instance = cls(json_str)
        return cls._instance

    @classmethod
    def GetInstance(cls) -> Optional["KGCacheController"]:
        return cls._instance

    def RegTensorsPerProcess(self, full_emb: torch.Tensor, caches: Optional[List[Optional[torch.Tensor]]] = None) -> None:
        """Binds the host table (and, on the CPU path, the per-rank cache tensors) and starts the flusher threads."""
        assert full_emb.dtype == torch.float32 and full_emb.is_contiguous() and not full_emb.is_cuda
        self._keep["full"] = full_emb
        _lib.call("rs_ctrl_register_table", self._h, full_emb.data_ptr(), full_emb.shape[0])
        for r, c in enumerate(caches or []):
            if c is not None and not c.is_cuda:
                self._keep[f"cache{r}"] = c
                _lib.call("rs_ctrl_register_cache", self._h, r, c.data_ptr())
        _lib.call("rs_ctrl_start", self._h)

    def PublishReads(self, rank: int, step: int, ids: torch.Tensor) -> None:
        ids = ids.to(torch.int64).contiguous().cpu()
        _lib.call("rs_ctrl_publish_reads", self._h, rank, step, ids.data_ptr(), ids.numel())

    def SetStepInput(self, rank: int, keys: torch.Tensor, grads: torch.Tensor) -> None:
        keys = keys.to(torch.int64).contiguous().cpu()
        grads = grads.to(torch.float32).contiguous().cpu()
        self._keep[f"k{rank}"], self._keep[f"g{rank}"] = keys, grads
        _lib.call("rs_ctrl_set_step_input", self._h, rank, keys.data_ptr(), keys.numel(), grads.data_ptr())

    def ProcessOneStep(self, step: int) -> None:
        _lib.call("rs_ctrl_process_one_step", self._h, step)

    def BlockToStepN(self, step: int, timeout_ms: int = 60_000) -> None:
        _lib.call("rs_ctrl_block_to_step", self._h, step, timeout_ms)

    def Drain(self) -> None:
        _lib.call("rs_ctrl_drain", self._h)

    def StopThreads(self) -> None:
        _lib.call("rs_ctrl_stop", self._h)

    def PendingCount(self) -> int:
        return int(self._l.rs_ctrl_pending(self._h))

    def Stats(self) -> dict:
        """Counters that tell the strategies apart: rows written back, whole-bucket swaps (CppAsyncV2), announcements
        that went through a mailbox and the detect thread (CppAsync), and how the steps' keys were upserted."""
        out = (C.c_longlong * 6)()
        _lib.call("rs_ctrl_stats", self._h, out)
        return {"flushed": out[0], "bucket_swaps": out[1], "mailed_announcements": out[2], "upsert_serial": out[3],
                "upsert_per_rank": out[4], "upsert_per_shard_group": out[5]}

    def PrintPq(self) -> str:
        n = self._l.rs_ctrl_print_pq(self._h, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._l.rs_ctrl_print_pq(self._h, buf, n + 1)
        return buf.value.decode()

    def __del__(self):
        try:
            if self._h:
                self._l.rs_ctrl_destroy(self._h)
                self._h = None
        except Exception:
            pass


class CircleBuffer:
    """Ring of the next ``L`` id batches of one rank; ``push`` publishes the batch for ``step`` to the controller."""

    def __init__(self, L: int, rank: int, controller: Optional[KGCacheController] = None):
        self.L, self.rank, self.controller = L, rank, controller
        # L batches wait in the ring and a push comes before the matching pop, so L + 1 slots: with only L the push of
        # batch t + L would overwrite batch t before it is popped and every batch would be read L steps before the
        # step it was announced for.
        self.slots: List[Optional[torch.Tensor]] = [None] * (max(L, 1) + 1)
        self.start = self.end = 0
        self.step_of_next_push = 0

    def push(self, ids: torch.Tensor, sync: bool = False) -> None:
        self.slots[self.end % len(self.slots)] = ids
        self.end += 1
        if self.controller is not None:
            self.controller.PublishReads(self.rank, self.step_of_next_push, ids)
        self.step_of_next_push += 1

    def pop(self) -> Optional[torch.Tensor]:
        if self.start == self.end:
            return None
        t = self.slots[self.start % len(self.slots)]
        self.start += 1
        return t

    def __len__(self):
        return self.end - self.start


class BasePerfSampler:
    """Prefills ``L`` future batches, then every ``next()`` pushes batch t+L and pops batch t."""

    def __init__(self, rank: int, L: int, num_ids_per_step: int, full_emb_capacity: int, backmode: str = "CppAsyncV2",
                 controller: Optional[KGCacheController] = None, seed: int = 0):
        self.rank, self.L, self.n, self.capacity = rank, L, num_ids_per_step, full_emb_capacity
        self.ring = CircleBuffer(L, rank, controller if backmode in ("CppAsync", "CppAsyncV2") else None)
        self.gen = torch.Generator().manual_seed(seed * 1000 + rank)

    def gen_next_sample(self) -> torch.Tensor:
        return torch.randint(0, self.capacity, (self.n,), generator=self.gen)

    def Prefill(self) -> None:
        for _ in range(self.L):
            self.ring.push(self.gen_next_sample(), sync=True)

    def __next__(self) -> torch.Tensor:
        self.ring.push(self.gen_next_sample())
        return self.ring.pop()

    def __iter__(self):
        return self


class TestPerfSampler(BasePerfSampler):
    """Deterministic ids: rank r reads ``[r, r+1, ...]`` shifted by the step (for exact expectations in tests)."""
    __test__ = False

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self._i = 0

    def gen_next_sample(self) -> torch.Tensor:
        base = (self._i * 7 + self.rank) % self.capacity
        self._i += 1
        return (torch.arange(self.n) * 3 + base) % self.capacity


class ZipfPerfSampler(BasePerfSampler):
    def __init__(self, *a, alpha: float = 0.99, **k):
        super().__init__(*a, **k)
        self.alpha = alpha

    def gen_next_sample(self) -> torch.Tensor:
        from .utils.data import zipf_ids_torch
        return zipf_ids_torch(self.n, self.capacity, self.alpha, self.gen)


class GraphCachedSampler:
    """Lookahead wrapper of a knowledge-graph sampler: keeps the next ``L`` batches, and publishes the entity ids a
    batch will touch (``cat(head, tail, negatives)``) when it enters the window, so that pending host-tier updates of
    those rows are flushed before the step that reads them.  ``sampler`` yields ``(h, r, t, neg, corrupt_head)`` (e.g.
    ``utils.kg_data.ChunkedNegativeSampler``).  Counterpart of the reference's wrapper around the DGL sampler
    (src/python/pytorch/recstore/controller_process.py:160-242)."""

    def __init__(self, sampler, rank: int, L: int, backmode: str = "CppAsyncV2", controller: Optional[KGCacheController] = None):
        self.sampler, self.rank, self.L = sampler, rank, L
        self.ring = CircleBuffer(L, rank, controller if backmode in ("CppAsync", "CppAsyncV2") else None)
        self._batches: List = []

    @staticmethod
    def entity_ids(batch) -> torch.Tensor:
        h, _, t, neg = batch[0], batch[1], batch[2], batch[3]
        return torch.cat([h.reshape(-1), t.reshape(-1), neg.reshape(-1)]).cpu()

    def _push(self) -> None:
        b = next(self.sampler)
        self._batches.append(b)
        self.ring.push(self.entity_ids(b))

    def Prefill(self) -> None:
        for _ in range(self.L):
            self._push()

    def __next__(self):
        self._push()
        self.ring.pop()
        return self._batches.pop(0)

    def __iter__(self):
        return self

    @staticmethod
    def BatchCreateCachedSamplers(L: int, samplers, backmode: str = "CppAsyncV2", controller: Optional[KGCacheController] = None):
        """One cached sampler per rank-local sampler, all prefilled (rank = position in the list)."""
        out = [GraphCachedSampler(s, r, L, backmode, controller) for r, s in enumerate(samplers)]
        for c in out:
            c.Prefill()
        return out


class KGCacheControllerWrapperBase:
    @staticmethod
    def BeforeDDPInit() -> None:
        from .ipc import IPCTensorFactory, MultiProcessBarrierFactory
        IPCTensorFactory.ClearIPCMemory()
        MultiProcessBarrierFactory.ClearIPCMemory()

    @staticmethod
    def FactoryNew(kind: str, json_str: str, rank: int = 0, world: int = 1):
        if kind == "Dummy":
            return KGCacheControllerWrapperDummy(json_str, rank, world)
        if kind == "RecStore":
            return KGCacheControllerWrapper(json_str, rank, world)
        raise ValueError(f"unknown controller kind {kind!r}")


class KGCacheControllerWrapperDummy(KGCacheControllerWrapperBase):
    def __init__(self, json_str: str, rank: int = 0, world: int = 1):
        self.rank, self.world, self.step = rank, world, 0

    def init(self, *a, **k): pass

    def AfterBackward(self):
        self.step += 1

    def StopThreads(self): pass

    def GraceFullyStopThreads(self): pass


class KGCacheControllerWrapper(KGCacheControllerWrapperBase):
    """Per-rank handle.  Rank 0 owns the native controller; the other ranks reach it through the shared
    barrier only (their keys / gradients travel in shared tensors that rank 0 registers)."""

    def __init__(self, json_str: str, rank: int = 0, world: int = 1, barrier_timeout_ms: int = 100_000):
        from .ipc import MultiProcessBarrierFactory
        self.rank, self.world, self.step = rank, world, 0
        self.controller = KGCacheController.Init(json_str) if rank == 0 else None
        self.barrier = MultiProcessBarrierFactory.Create("kg_cache_controller", world, barrier_timeout_ms) if world > 1 else None

    def init(self, full_emb: Optional[torch.Tensor] = None, caches=None) -> None:
        if self.controller is not None and full_emb is not None:
            self.controller.RegTensorsPerProcess(full_emb, caches)

    def AfterBackward(self) -> None:
        if self.barrier:
            self.barrier.Wait()
        if self.controller is not None:
            self.controller.ProcessOneStep(self.step)
        self.step += 1
        if self.controller is not None:
            self.controller.BlockToStepN(self.step)
        if self.barrier:
            self.barrier.Wait()

    def StopThreads(self) -> None:
        if self.controller is not None:
            self.controller.StopThreads()

    def GraceFullyStopThreads(self) -> None:
        if self.controller is not None:
            self.controller.Drain()
            self.controller.StopThreads()
