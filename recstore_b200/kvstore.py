"""Name -> tensor store that backs ``DistTensor`` / ``DistEmbedding``.

``ShmKVStore`` keeps every named tensor in POSIX shared memory (``ipc.IPCTensorFactory``), so all
worker processes of one box see the same full embedding table, as in the reference
(src/python/pytorch/recstore/PsKvstore.py:11-116).  ``kvinit()`` creates the process-wide
singleton, ``get_kvstore()`` returns it.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from .ipc import IPCTensorFactory


class AbsKVStore(ABC):
    @abstractmethod
    def init_data(self, name, shape, dtype, part_policy=None, init_func=None, is_gdata=None): ...

    @abstractmethod
    def data_name_list(self): ...

    @abstractmethod
    def get_data_meta(self, name): ...

    @abstractmethod
    def Get(self, name, id_tensor): ...

    @abstractmethod
    def Put(self, name, id_tensor, data_tensor): ...

    @abstractmethod
    def Delete(self, name): ...


class ShmKVStore(AbsKVStore):
    """Tensors shared through /dev/shm; attach-or-create by name."""

    def __init__(self):
        self.tensor_store: Dict[str, torch.Tensor] = {}
        self._registered = set()

    def init_data(self, name: str, shape: Tuple[int, ...], dtype=torch.float32, part_policy=None,
                  init_func: Optional[Callable] = None, is_gdata=None) -> None:
        if name in self.tensor_store:
            raise KeyError(f"tensor {name!r} is already registered in this process")
        t = IPCTensorFactory.NewIPCTensor(name, shape, dtype)
        if t is None:                      # another process created it first: attach
            t = IPCTensorFactory.FindIPCTensorFromName(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise ValueError(f"shared tensor {name!r} exists with shape {tuple(t.shape)} / {t.dtype}")
        elif init_func is not None:
            init_func(t, shape, dtype)
        self.tensor_store[name] = t

    def attach(self, name: str) -> torch.Tensor:
        t = IPCTensorFactory.FindIPCTensorFromName(name)
        self.tensor_store[name] = t
        return t

    def data_name_list(self):
        return self.tensor_store.keys()

    def get_data_meta(self, name):
        t = self.tensor_store[name]
        return t.dtype, tuple(t.shape), None

    def Get(self, name, id_tensor):
        if isinstance(id_tensor, (list, tuple)):
            id_tensor = torch.tensor(id_tensor, dtype=torch.int64)
        if id_tensor.dtype not in (torch.int64, torch.int32):
            raise TypeError("ids must be int32 or int64")
        t = self.tensor_store[name]
        return F.embedding(id_tensor, t) if t.dim() == 2 else t[id_tensor.long()]

    def Put(self, name, id_tensor, data_tensor):
        self.tensor_store[name][id_tensor] = data_tensor

    def Delete(self, name):
        if name in self.tensor_store:
            del self.tensor_store[name]
            IPCTensorFactory.Delete(name)

    def GetRowTensor(self, name) -> torch.Tensor:
        return self.tensor_store[name]

    def GetUVAMap(self, tensor: torch.Tensor) -> int:
        """Page-locks and maps the host tensor into the CUDA address space so that kernels can read it
        in place (cudaHostRegister); returns the CUDA error code (0 = success)."""
        key = tensor.data_ptr()
        if key in self._registered:
            return 0
        rc = torch.cuda.cudart().cudaHostRegister(tensor.data_ptr(), tensor.numel() * tensor.element_size(), 0)
        if int(rc) == 0:
            self._registered.add(key)
        return int(rc)


KVSTORE: Optional[ShmKVStore] = None


def kvinit() -> ShmKVStore:
    global KVSTORE
    if KVSTORE is None:
        KVSTORE = ShmKVStore()
    return KVSTORE


def get_kvstore() -> Optional[ShmKVStore]:
    return KVSTORE


def kvreset() -> None:
    """Drops the singleton (tests)."""
    global KVSTORE
    KVSTORE = None
