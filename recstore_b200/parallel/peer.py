"""Peer-window manager: named device allocations that every rank of one box can address.

One process drives one GPU.  ``PeerContext.alloc(name, nbytes)`` is a collective: each rank
allocates its window with ``cudaMalloc``, the CUDA IPC handles travel through the host
process group (``torch.distributed`` object all-gather, any backend), every rank opens the
others' windows and gets a device-resident table of base pointers that kernels index by
rank.  With ``world_size == 1`` nothing is exchanged and the table has one entry.

Cross-rank ordering uses flag channels (``signal`` / ``wait``) implemented by two tiny kernels
whose epochs are device counters, so they can be captured in a CUDA graph and replayed.  Waits
are bounded; when one runs out the device status word gets ``DEV_WAIT_TIMEOUT`` and
:meth:`PeerContext.check_status` raises on the host while the CUDA context stays usable.

``PeerContext(heap_bytes=N)`` adds a symmetric heap: ONE window of N bytes is allocated and exchanged at start-up, and
``alloc`` then carves named windows out of it with an allocator that every rank runs identically (same calls in the same
order give the same offsets on every rank), so a window costs no ``cudaMalloc``, no handle exchange and no peer
mapping, and ``free(name)`` returns its bytes for reuse.  Requests that do not fit fall back to a window of their own.

Takes the place of ``IPCTensorFactory`` GPU tensors and the shm barrier of the reference
(src/framework/pytorch/IPCTensor.h:281-317, IPC_barrier.h:20-51).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .. import _lib

_DTYPE_STR = {torch.float32: "<f4", torch.bfloat16: "<u2", torch.int64: "<i8", torch.int32: "<i4",
              torch.uint8: "|u1", torch.float16: "<f2"}


class _RawCudaBuffer:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """uint8 tensor aliasing ``nbytes`` of device memory at ``ptr`` (no ownership)."""
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)


class SymmetricAllocator:
    """Offsets inside a heap of ``nbytes``: first fit at the lowest address, neighbours merged on free.  Pure host logic
    with no randomness, so ranks that make the same calls in the same order hold the same layout without talking."""

    def __init__(self, nbytes: int, align: int = 256):
        assert align > 0 and align & (align - 1) == 0, "alignment must be a power of two"
        self.nbytes, self.align = int(nbytes) // align * align, align
        self._free: List[List[int]] = [[0, self.nbytes]] if self.nbytes else []     # [offset, size], sorted by offset
        self._used: Dict[int, int] = {}

    def alloc(self, nbytes: int) -> Optional[int]:
        """Offset of a block of at least ``nbytes`` (rounded up to the alignment), ``None`` when nothing fits."""
        need = max(self.align, (int(nbytes) + self.align - 1) // self.align * self.align)
        for i, (off, size) in enumerate(self._free):
            if size >= need:
                if size == need:
                    self._free.pop(i)
                else:
                    self._free[i] = [off + need, size - need]
                self._used[off] = need
                return off
        return None

    def free(self, off: int) -> None:
        size = self._used.pop(off, None)
        if size is None:
            raise ValueError(f"offset {off} is not an allocated block")
        import bisect
        i = bisect.bisect_left(self._free, [off, 0])
        self._free.insert(i, [off, size])
        if i + 1 < len(self._free) and self._free[i][0] + self._free[i][1] == self._free[i + 1][0]:
            self._free[i][1] += self._free.pop(i + 1)[1]
        if i > 0 and self._free[i - 1][0] + self._free[i - 1][1] == self._free[i][0]:
            self._free[i - 1][1] += self._free.pop(i)[1]

    @property
    def bytes_in_use(self) -> int:
        return sum(self._used.values())

    @property
    def largest_free(self) -> int:
        return max((s for _, s in self._free), default=0)

    def layout(self) -> List[tuple]:
        """``[(offset, size, "used" | "free"), ...]`` in address order (tests and debugging)."""
        return sorted([(o, s, "used") for o, s in self._used.items()] + [(o, s, "free") for o, s in self._free])


@dataclass
class PeerWindow:
    name: str
    nbytes: int
    rank: int
    ptrs: List[int]                      # base address of the window of every rank, as mapped here
    table: torch.Tensor                  # int64 [world] on device: the same pointers
    local: torch.Tensor                  # uint8 view of this rank's window
    _opened: List[int] = field(default_factory=list)
    heap_offset: Optional[int] = None    # set for windows carved out of the symmetric heap (they own no allocation)

    @property
    def local_ptr(self) -> int:
        return self.ptrs[self.rank]

    def view(self, dtype: torch.dtype, shape, byte_offset: int = 0) -> torch.Tensor:
        """Typed view of the local window."""
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.local[byte_offset:byte_offset + nb].view(dtype).view(*shape)

    def peer_view(self, rank: int, dtype: torch.dtype, shape, byte_offset: int = 0) -> torch.Tensor:
        """Typed view of rank ``rank``'s window through the peer mapping (debug / tests)."""
        t = tensor_from_ptr(self.ptrs[rank], self.nbytes, self.local.device)
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        return t[byte_offset:byte_offset + nb].view(dtype).view(*shape)


class PeerContext:
    """Per-process handle on the in-box transport (rank, world, windows, flags, status word)."""

    NUM_CHANNELS = 16

    def __init__(self, rank: int = 0, world: int = 1, device: Optional[torch.device] = None, group=None,
                 wait_timeout_s: float = 2.0, heap_bytes: int = 0):
        self.rank, self.world = int(rank), int(world)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.group = group
        self.wait_timeout_ns = int(wait_timeout_s * 1e9)
        self.windows: Dict[str, PeerWindow] = {}
        self.status = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._counters = torch.zeros(2 * self.NUM_CHANNELS, dtype=torch.int32, device=self.device)
        self._heap: Optional[PeerWindow] = None
        self._heap_alloc: Optional[SymmetricAllocator] = None
        self._flags = self.alloc("__flags__", 4 * self.NUM_CHANNELS * max(self.world, 1))
        if heap_bytes > 0:
            self._heap = self.alloc("__heap__", heap_bytes)
            self._heap_alloc = SymmetricAllocator(self._heap.nbytes)

    # ------------------------------------------------------------------ windows
    def alloc(self, name: str, nbytes: int) -> PeerWindow:
        """Collective: allocates ``nbytes`` (rounded up to 256) on every rank and maps all peers."""
        if name in self.windows:
            raise ValueError(f"peer window {name!r} already exists")
        nbytes = (int(nbytes) + 255) // 256 * 256
        if self._heap_alloc is not None:
            off = self._heap_alloc.alloc(nbytes)
            if off is not None:              # a slice of the heap: the peers' addresses follow from the heap's own
                ptrs = [p + off for p in self._heap.ptrs]
                table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
                local = self._heap.local[off:off + nbytes]
                w = PeerWindow(name, nbytes, self.rank, ptrs, table, local, [], heap_offset=off)
                self.windows[name] = w
                return w
        with torch.cuda.device(self.device):
            p = C.c_void_p()
            _lib.call("rs_peer_alloc", nbytes, C.byref(p))
            local_ptr = p.value
            ptrs = [0] * self.world
            ptrs[self.rank] = local_ptr
            opened = []
            if self.world > 1:
                import torch.distributed as dist
                h = (C.c_ubyte * 64)()
                _lib.call("rs_ipc_get_handle", local_ptr, h)
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(h), group=self.group)
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                    q = C.c_void_p()
                    _lib.call("rs_ipc_open", buf, C.byref(q))
                    ptrs[r] = q.value
                    opened.append(q.value)
            table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
            local = tensor_from_ptr(local_ptr, nbytes, self.device)
        w = PeerWindow(name, nbytes, self.rank, ptrs, table, local, opened)
        self.windows[name] = w
        return w

    def free(self, name: str) -> None:
        """Collective: gives one window back.  A slice of the symmetric heap returns to the heap's allocator for reuse;
        a window of its own is unmapped and freed.  Every rank must have finished with the window (no kernel of any
        rank may still address it): the call synchronises this device and meets the others at a host barrier first."""
        w = self.windows.get(name)
        if w is None:
            raise KeyError(f"no peer window named {name!r}")
        if name in ("__flags__", "__heap__"):
            raise ValueError(f"{name} lives as long as the context")
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                import torch.distributed as dist
                dist.barrier(group=self.group)
            if w.heap_offset is not None:
                self._heap_alloc.free(w.heap_offset)
            else:
                for q in w._opened:
                    _lib.call("rs_ipc_close", q)
                if self.world > 1:
                    dist.barrier(group=self.group)
                _lib.call("rs_peer_free", w.local_ptr)
        del self.windows[name]

    def heap_stats(self) -> Dict[str, int]:
        a = self._heap_alloc
        return {"heap_bytes": a.nbytes if a else 0, "in_use": a.bytes_in_use if a else 0, "largest_free": a.largest_free if a else 0,
                "windows_in_heap": sum(1 for w in self.windows.values() if w.heap_offset is not None)}

    def free_all(self) -> None:
        """Unmaps peers and frees local windows.  Collective in spirit: call on every rank after a barrier."""
        own = [w for w in self.windows.values() if w.heap_offset is None]       # heap slices own no allocation
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for w in own:
                for q in w._opened:
                    _lib.call("rs_ipc_close", q)
            if self.world > 1:
                import torch.distributed as dist
                dist.barrier(group=self.group)
            for w in own:
                _lib.call("rs_peer_free", w.local_ptr)
        self.windows.clear()
        self._heap = self._heap_alloc = None

    # ------------------------------------------------------------------ flags
    def signal(self, channel: int, stream=None) -> None:
        """Tells every rank that this rank's writes issued so far on the stream are complete."""
        _lib.call("rs_peer_signal", self._flags.table.data_ptr(), self.world, self.rank, channel,
                  self._counters.data_ptr(), _lib.stream_ptr(stream))

    def wait(self, channel: int, stream=None) -> None:
        """Orders the stream after the matching ``signal`` of every rank (bounded)."""
        _lib.call("rs_peer_wait", self._flags.local_ptr, self.world, channel,
                  self._counters.data_ptr() + 4 * self.NUM_CHANNELS, self.wait_timeout_ns,
                  self.status.data_ptr(), _lib.stream_ptr(stream))

    def wait_own(self, channel: int, stream=None) -> None:
        """Orders the stream after every rank's flag on ``channel`` has reached THIS rank's own signal count there: for
        channels whose signals come from inside producing kernels (one per rank and round)."""
        _lib.call("rs_peer_wait_own", self._flags.local_ptr, self.world, channel, self._counters.data_ptr(),
                  self.wait_timeout_ns, self.status.data_ptr(), _lib.stream_ptr(stream))

    # what a kernel with a fused signal / an in-kernel wait needs
    @property
    def flags_table_ptr(self) -> int:
        return self._flags.table.data_ptr()

    @property
    def my_flags_ptr(self) -> int:
        return self._flags.local_ptr

    @property
    def counters_ptr(self) -> int:
        return self._counters.data_ptr()

    def sync(self, channel: int, stream=None) -> None:
        """``signal`` + ``wait`` on one channel in a single launch (a barrier of the ranks on that channel)."""
        _lib.call("rs_peer_sync", self._flags.table.data_ptr(), self._flags.local_ptr, self.world, self.rank, channel,
                  self._counters.data_ptr(), self._counters.data_ptr() + 4 * self.NUM_CHANNELS, self.wait_timeout_ns,
                  self.status.data_ptr(), _lib.stream_ptr(stream))

    def barrier(self, channel: int = NUM_CHANNELS - 1, stream=None) -> None:
        self.sync(channel, stream)

    # ------------------------------------------------------------------ status
    def check_status(self, reset: bool = True) -> None:
        """Reads the device status word (synchronises) and raises if any kernel recorded an error."""
        word = int(self.status.item()) & 0xFFFFFFFFFFFFFFFF
        if word:
            if reset:
                self.status.zero_()
            raise _lib.DeviceStatusError(_lib.ERR_TIMEOUT if word & _lib.DEV_WAIT_TIMEOUT else _lib.ERR_INVALID,
                                         "device status: " + _lib.decode_status(word))
