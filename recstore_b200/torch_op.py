"""Operator aliases with the names the reference exports from ``librecstore_pytorch``
(src/python/pytorch/recstore/torch_op.py:4-26, src/framework/pytorch/recstore_pytorch.cc:113-142).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

import torch

from . import _lib
from ._lib import i32, i64, u64, vp, f64
from .cache.gpu_cache import GpuCache, merge_op, uva_cache_query_op  # noqa: F401
from .ipc import IPCTensorFactory, Mfence, MultiProcessBarrierFactory, SlicedTensor  # noqa: F401
from .controller import KGCacheController  # noqa: F401

_lib.register_signatures({
    "rs_construct_renumbering_dict": (i32, [vp, i64, i32, vp, vp]),
    "rs_zipf_fill": (i32, [vp, i64, u64, f64, u64, i32]),
})


def construct_renumbering_dict_op(renumbering_dict: torch.Tensor, nr_world: int, hotsets: Sequence[torch.Tensor]) -> torch.Tensor:
    """Fills ``renumbering_dict[old_id] = new_id`` so that rank r's hot ids become the contiguous range that
    follows the previous ranks' hot sets; cold ids follow in increasing order."""
    assert renumbering_dict.dtype == torch.int64 and renumbering_dict.is_contiguous() and not renumbering_dict.is_cuda
    hs = [h.to(torch.int64).contiguous().cpu() for h in hotsets[:nr_world]]
    ptrs = (vp * max(nr_world, 1))(*[h.data_ptr() for h in hs])
    lens = (i64 * max(nr_world, 1))(*[h.numel() for h in hs])
    _lib.lib()
    _lib.call("rs_construct_renumbering_dict", renumbering_dict.data_ptr(), renumbering_dict.numel(), nr_world, ptrs, lens)
    return renumbering_dict


def NarrowShapeTensor_op(buffer: torch.Tensor, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
    """Reinterprets the head of a big (e.g. pinned staging) buffer as a smaller tensor of another shape / dtype,
    without copying."""
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    flat = buffer.reshape(-1).view(torch.uint8)
    assert nbytes <= flat.numel(), "NarrowShapeTensor: the buffer is too small"
    return flat[:nbytes].view(dtype).view(*shape)


def init_folly() -> None:
    """Kept for source compatibility: starts the periodic timer report like the reference's start-up hook."""
    from .utils.timer import Reporter
    Reporter.StartReportThread(5000)


class ZipfianTorchFiller:
    """``ZipfianTorchFiller(capacity, theta).fillArrayTorch(t)``: fills an int64 tensor with 1-based Zipf ids
    (the reference's ids are 1-based too, recstore_pytorch.cc:77-82); any theta >= 0 is accepted."""

    def __init__(self, capacity: int, theta: float, seed: int = 1):
        self.capacity, self.theta, self.seed = int(capacity), float(theta), int(seed)
        self._calls = 0

    def fillArrayTorch(self, t: torch.Tensor) -> torch.Tensor:
        assert t.dtype == torch.int64 and t.is_contiguous() and not t.is_cuda
        _lib.lib()
        self._calls += 1
        _lib.call("rs_zipf_fill", t.data_ptr(), t.numel(), self.capacity, self.theta, self.seed * 7919 + self._calls, 1)
        return t
