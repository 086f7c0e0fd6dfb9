"""Parameter-server front end.

* ``ParameterServer``: one shard ("CachePS": KV engine + Put/Get/Update/LoadFakeData/Clear +
  checkpoints) that can be used in-process or served on a loopback port.
* ``ParameterClient(host, port, shard)``: the client API of the reference
  (src/grpc_ps/grpc_ps_client.h:33-77): ``GetParameter``, ``PutParameter``, ``ClearPS``,
  ``LoadFakeData``, ``LoadCkpt`` (+ ``SaveCkpt`` and ``UpdateParameter``, the gradient verb).  Requests
  are cut into sub-requests of ``MAX_PARAMETER_BATCH`` keys that are pipelined on the connection.
  A missing key yields a zero row, not an error.
* ``PythonParameterClient(host, port, shard, emb_dim)``: the torch-facing variant
  (src/grpc_ps/grpc_ps_client_pytorch.cpp:5-73) returning ``Tensor[n, dim]``.
* Asynchronous form of ``BaseParameterClient`` (src/rdma_ps/base_client.h:6-47):
  ``GetParameterAsync -> rpc_id``, ``QueryRPCFinished``, ``WaitRPCFinish``, ``RevokeRPCResource``,
  ``GetReceiveBuffer``.
* ``AllShardsParameterClient``: partitions keys with ``ShardManager.KeyPartition`` (hash(key) %
  servers, src/ps_common/shard_manager.h:5-9) and fans out (src/rdma_ps/allshards_ps_client.h:46-95).
"""
from __future__ import annotations

import ctypes as C
import json
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _lib
from .._lib import cstr, i32, i64, u64, vp

_lib.register_signatures({
    "rs_wire_packed_size": (i64, [i64, i32]),
    "rs_wire_pack": (i32, [vp, i64, i32, vp, vp, vp, i64, C.POINTER(i64)]),
    "rs_wire_count": (i32, [vp, i64]),
    "rs_wire_unpack": (i32, [vp, i64, i32, vp, vp, vp]),
    "rs_ps_create": (i32, [cstr, cstr, C.POINTER(vp)]),
    "rs_ps_destroy": (i32, [vp]),
    "rs_ps_dim": (i32, [vp]),
    "rs_ps_size": (u64, [vp]),
    "rs_ps_put": (i32, [vp, vp, i64, vp]),
    "rs_ps_get": (i32, [vp, vp, i64, vp, vp]),
    "rs_ps_update": (i32, [vp, vp, i64, vp, C.POINTER(i64)]),
    "rs_ps_load_fake": (i32, [vp, u64]),
    "rs_ps_clear": (i32, [vp]),
    "rs_ps_save": (i32, [vp, cstr]),
    "rs_ps_load": (i32, [vp, cstr]),
    "rs_ps_server_start": (i32, [vp, i32, C.POINTER(vp), C.POINTER(i32)]),
    "rs_ps_server_start_pool": (i32, [vp, i32, i32, cstr, i32, C.POINTER(vp), C.POINTER(i32)]),
    "rs_ps_server_start_on": (i32, [vp, cstr, i32, i32, cstr, i32, C.POINTER(vp), C.POINTER(i32)]),
    "rs_ps_server_stop": (i32, [vp]),
    "rs_ps_server_monitor_start": (i32, [vp, i32, i32]),
    "rs_ps_server_monitor_stop": (i32, [vp]),
    "rs_ps_server_monitor_last": (u64, [vp, C.POINTER(C.c_double)]),
    "rs_ps_client_connect": (i32, [cstr, i32, C.POINTER(vp)]),
    "rs_ps_client_close": (i32, [vp]),
    "rs_ps_client_get": (i32, [vp, vp, i64, i32, vp, vp, i32]),
    "rs_ps_client_put": (i32, [vp, vp, i64, i32, vp, i32]),
    "rs_ps_client_update": (i32, [vp, vp, i64, i32, vp, i32, C.POINTER(u64)]),
    "rs_ps_client_command": (i32, [vp, i32, vp, i64, C.POINTER(u64)]),
})

_lib.register_signatures({
    "rs_provider_new": (i32, [cstr, i32, u64, C.POINTER(vp)]),
    "rs_provider_delete": (i32, [vp]),
    "rs_provider_put": (i32, [vp, i64, u64]),
    "rs_provider_try_get": (i64, [vp]),
    "rs_provider_left": (i64, [vp]),
    "rs_provider_improve": (i32, [vp, u64]),
    "rs_provider_level": (i32, [vp, u64]),
})

MAX_PARAMETER_BATCH = 2000
OP_CLEAR, OP_FAKE, OP_SAVE, OP_LOAD, OP_STATS, OP_PRIORITY = 4, 5, 6, 7, 8, 10


def _keys(keys) -> torch.Tensor:
    return torch.as_tensor(keys, dtype=torch.int64).contiguous()


def pack_records(keys, values: torch.Tensor, dims: Optional[Sequence[int]] = None) -> bytes:
    """[int32 n][int32 end_offset[n]]{u64 key; int32 dim; float emb[dim]} x n"""
    _lib.lib()
    k = _keys(keys)
    v = torch.as_tensor(values, dtype=torch.float32).contiguous()
    n, dim = v.shape
    cap = _lib.lib().rs_wire_packed_size(n, dim)
    buf = C.create_string_buffer(cap)
    d = torch.as_tensor(dims, dtype=torch.int32).contiguous() if dims is not None else None
    w = i64()
    _lib.call("rs_wire_pack", k.data_ptr(), n, dim, v.data_ptr(), d.data_ptr() if d is not None else None, buf, cap, C.byref(w))
    return buf.raw[: w.value]


def unpack_records(buf: bytes, dim: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (keys [n], dims [n], values [n, dim]; records of another dim give zero rows)."""
    _lib.lib()
    n = _lib.lib().rs_wire_count(buf, len(buf))
    if n < 0:
        raise _lib.RecStoreError(_lib.ERR_INVALID, "malformed record buffer")
    k = torch.empty(n, dtype=torch.int64)
    d = torch.empty(n, dtype=torch.int32)
    v = torch.empty(n, dim, dtype=torch.float32)
    _lib.call("rs_wire_unpack", buf, len(buf), dim, k.data_ptr(), d.data_ptr(), v.data_ptr())
    return k, d, v


class TaskProvider:
    """The server's task schedulers on their own (``csrc/runtime/task_provider.h``): ``"fifo"``, or ``"priority"``
    with ``levels`` lists where the next task comes from level i with probability proportional to i x (tasks waiting
    at level i) and ``ImprovePriority(klass)`` raises a class by one level (src/grpc_ps/provider.h:13-201)."""

    def __init__(self, kind: str = "fifo", levels: int = 7, seed: int = 1):
        self._l = _lib.lib()
        h = vp()
        _lib.call("rs_provider_new", kind.encode(), int(levels), int(seed), C.byref(h))
        self._h = h.value

    def PutTask(self, task: int, klass: int = 0) -> None:
        _lib.call("rs_provider_put", self._h, int(task), int(klass))

    def GetTask(self) -> Optional[int]:
        t = int(self._l.rs_provider_try_get(self._h))
        return None if t < 0 else t

    def ExistTask(self) -> bool:
        return self.LeftTask() > 0

    def LeftTask(self) -> int:
        return int(self._l.rs_provider_left(self._h))

    def ImprovePriority(self, klass: int) -> None:
        _lib.call("rs_provider_improve", self._h, int(klass))

    def LevelOf(self, klass: int) -> int:
        return int(self._l.rs_provider_level(self._h, int(klass)))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._l.rs_provider_delete(self._h)
            self._h = None

    __del__ = close


class ShardManager:
    @staticmethod
    def KeyPartition(keys, num_shards: int) -> torch.Tensor:
        """Owner shard of every key: a 64-bit mix of the key modulo the shard count."""
        k = _keys(keys).numpy().astype(np.uint64)
        with np.errstate(over="ignore"):
            k ^= k >> np.uint64(33); k *= np.uint64(0xff51afd7ed558ccd)
            k ^= k >> np.uint64(33); k *= np.uint64(0xc4ceb9fe1a85ec53)
            k ^= k >> np.uint64(33)
        return torch.from_numpy((k % np.uint64(num_shards)).astype(np.int64))


class ParameterServer:
    """One PS shard.  ``config``: ``dim`` (floats per key), ``capacity``, ``engine``-specific keys, and the
    server-side optimizer: ``optimizer`` ("rowwise_adagrad" | "sgd"), ``lr``, ``eps``."""

    def __init__(self, engine: str = "KVEngineMap", config: Optional[dict] = None):
        self._l = _lib.lib()
        cfg = {"dim": 32, "capacity": 1 << 20}
        cfg.update(config or {})
        h = vp()
        _lib.call("rs_ps_create", engine.encode(), json.dumps(cfg).encode(), C.byref(h))
        self._h = h.value
        self.dim = self._l.rs_ps_dim(self._h)
        self._server = None
        self.port = None

    # in-process verbs -------------------------------------------------
    def PutParameter(self, keys, values) -> None:
        k = _keys(keys); v = torch.as_tensor(values, dtype=torch.float32).contiguous()
        assert v.shape == (k.numel(), self.dim)
        _lib.call("rs_ps_put", self._h, k.data_ptr(), k.numel(), v.data_ptr())

    def GetParameter(self, keys) -> torch.Tensor:
        k = _keys(keys)
        out = torch.empty(k.numel(), self.dim)
        _lib.call("rs_ps_get", self._h, k.data_ptr(), k.numel(), out.data_ptr(), None)
        return out

    def GetParameterWithMask(self, keys) -> Tuple[torch.Tensor, torch.Tensor]:
        k = _keys(keys)
        out = torch.empty(k.numel(), self.dim)
        found = torch.empty(k.numel(), dtype=torch.uint8)
        _lib.call("rs_ps_get", self._h, k.data_ptr(), k.numel(), out.data_ptr(), found.data_ptr())
        return out, found.bool()

    def UpdateParameter(self, keys, grads) -> int:
        k = _keys(keys); g = torch.as_tensor(grads, dtype=torch.float32).contiguous()
        a = i64()
        _lib.call("rs_ps_update", self._h, k.data_ptr(), k.numel(), g.data_ptr(), C.byref(a))
        return int(a.value)

    def LoadFakeData(self, n: int) -> None:
        _lib.call("rs_ps_load_fake", self._h, int(n))

    def ClearPS(self) -> None:
        _lib.call("rs_ps_clear", self._h)

    def SaveCkpt(self, path: str) -> None:
        _lib.call("rs_ps_save", self._h, path.encode())

    def LoadCkpt(self, path: str) -> None:
        _lib.call("rs_ps_load", self._h, path.encode())

    def __len__(self):
        return int(self._l.rs_ps_size(self._h))

    # serving ----------------------------------------------------------
    def serve(self, port: int = 0, workers: int = 0, scheduler: str = "fifo", levels: int = 7, host: str = "127.0.0.1") -> int:
        """Starts the loopback server; returns the bound port (``port=0`` picks a free one).  ``workers=0``: each
        connection's thread executes its requests (the reference's synchronous server); ``workers>0``: connection
        threads hand requests to a pool of worker threads through a ``"fifo"`` or ``"priority"`` task provider
        (the asynchronous server and the schedulers of src/grpc_ps/provider.h); answers keep request order per
        connection.  ``host``: the IPv4 address to listen on (loopback by default; ``"0.0.0.0"`` for every interface,
        which is what the reference's server does)."""
        s, p = vp(), i32()
        if host not in ("127.0.0.1", "localhost"):
            _lib.call("rs_ps_server_start_on", self._h, host.encode(), int(port), int(workers), scheduler.encode(), int(levels),
                      C.byref(s), C.byref(p))
        elif workers > 0:
            _lib.call("rs_ps_server_start_pool", self._h, int(port), int(workers), scheduler.encode(), int(levels), C.byref(s), C.byref(p))
        else:
            _lib.call("rs_ps_server_start", self._h, int(port), C.byref(s), C.byref(p))
        self._server, self.port = s.value, p.value
        return self.port

    def start_monitor(self, period_s: float = 1.0, print_lines: bool = True) -> None:
        """A server thread measures requests, keys and payload served per period and (``print_lines``) writes
        ``PS throughput: ... Kreq/s ... Mkeys/s ... MB/s`` to stderr while there is traffic (the once-a-second line of
        the reference's asynchronous server, src/grpc_ps/grpc_ps_server_async.cpp:109-117)."""
        assert self._server, "serve() first"
        _lib.call("rs_ps_server_monitor_start", self._server, max(1, int(period_s * 1000)), int(print_lines))

    def stop_monitor(self) -> None:
        if self._server:
            self._l.rs_ps_server_monitor_stop(self._server)

    def monitor_last(self) -> dict:
        """The last period's reading: ``{"periods", "kreq_per_s", "mkeys_per_s", "mb_per_s"}``."""
        out = (C.c_double * 3)()
        n = int(self._l.rs_ps_server_monitor_last(self._server, out))
        return {"periods": n, "kreq_per_s": out[0], "mkeys_per_s": out[1], "mb_per_s": out[2]}

    def stop(self) -> None:
        if self._server:
            self._l.rs_ps_server_stop(self._server)
            self._server = None

    def close(self) -> None:
        self.stop()
        if self._h:
            self._l.rs_ps_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ParameterClient:
    def __init__(self, host: str, port: int, shard: int = 0, emb_dim: int = 32):
        self._l = _lib.lib()
        h = vp()
        _lib.call("rs_ps_client_connect", host.encode(), int(port), C.byref(h))
        self._h = h.value
        self._shard = shard
        self.dim = emb_dim
        self._pool: Optional[ThreadPoolExecutor] = None
        self._rpcs: Dict[int, Tuple[Future, torch.Tensor]] = {}
        self._next_rpc = 0

    def shard(self) -> int:
        return self._shard

    def GetParameter(self, keys, perf: bool = True) -> torch.Tensor:
        k = _keys(keys)
        out = torch.empty(k.numel(), self.dim)
        _lib.call("rs_ps_client_get", self._h, k.data_ptr(), k.numel(), self.dim, out.data_ptr(), None, MAX_PARAMETER_BATCH)
        return out

    def GetParameterWithMask(self, keys) -> Tuple[torch.Tensor, torch.Tensor]:
        k = _keys(keys)
        out = torch.empty(k.numel(), self.dim)
        found = torch.empty(k.numel(), dtype=torch.uint8)
        _lib.call("rs_ps_client_get", self._h, k.data_ptr(), k.numel(), self.dim, out.data_ptr(), found.data_ptr(), MAX_PARAMETER_BATCH)
        return out, found.bool()

    def PutParameter(self, keys, values) -> bool:
        k = _keys(keys); v = torch.as_tensor(values, dtype=torch.float32).contiguous()
        assert v.shape == (k.numel(), self.dim)
        _lib.call("rs_ps_client_put", self._h, k.data_ptr(), k.numel(), self.dim, v.data_ptr(), MAX_PARAMETER_BATCH)
        return True

    def UpdateParameter(self, keys, grads) -> int:
        k = _keys(keys); g = torch.as_tensor(grads, dtype=torch.float32).contiguous()
        a = u64()
        _lib.call("rs_ps_client_update", self._h, k.data_ptr(), k.numel(), self.dim, g.data_ptr(), MAX_PARAMETER_BATCH, C.byref(a))
        return int(a.value)

    def _cmd(self, op: int, payload: bytes = b"") -> Tuple[int, int, int, int]:
        r = (u64 * 4)()
        _lib.call("rs_ps_client_command", self._h, op, payload, len(payload), r)
        return int(r[0]), int(r[1]), int(r[2]), int(r[3])

    def ClearPS(self) -> bool:
        self._cmd(OP_CLEAR)
        return True

    def LoadFakeData(self, n: int) -> bool:
        self._cmd(OP_FAKE, int(n).to_bytes(8, "little"))
        return True

    def LoadCkpt(self, model_config_path=None, emb_file_path=None) -> bool:
        """Loads a checkpoint written by ``SaveCkpt``; ``emb_file_path`` may be a path or a list of paths."""
        paths = emb_file_path if isinstance(emb_file_path, (list, tuple)) else [emb_file_path or model_config_path]
        for p in paths:
            rc = self._cmd(OP_LOAD, str(p).encode())[0]
            if rc != 0:
                raise _lib.RecStoreError(_lib.ERR_IO, f"server could not load {p}")
        return True

    def SaveCkpt(self, path: str) -> bool:
        if self._cmd(OP_SAVE, str(path).encode())[0] != 0:
            raise _lib.RecStoreError(_lib.ERR_IO, f"server could not write {path}")
        return True

    def Stats(self) -> dict:
        s = self._cmd(OP_STATS)
        return {"keys_stored": s[0], "requests": s[1], "keys_served": s[2], "pooled_requests": s[3]}

    def ImprovePriority(self) -> int:
        """Raises this connection's class by one level at a server with the priority scheduler; returns the new level
        (always 1 at a FIFO or synchronous server).  Role of Provider::ImporvePriority, src/grpc_ps/provider.h."""
        return self._cmd(OP_PRIORITY)[0]

    # asynchronous form ------------------------------------------------------------------
    def InitThread(self, n: int = 1) -> None:
        self._pool = ThreadPoolExecutor(max_workers=max(1, n))

    def GetParameterAsync(self, keys) -> int:
        if self._pool is None:
            self.InitThread()
        k = _keys(keys)
        out = torch.empty(k.numel(), self.dim)
        fut = self._pool.submit(lambda: _lib.call("rs_ps_client_get", self._h, k.data_ptr(), k.numel(), self.dim,
                                                  out.data_ptr(), None, MAX_PARAMETER_BATCH))
        rid = self._next_rpc
        self._next_rpc += 1
        self._rpcs[rid] = (fut, out)
        return rid

    def PutParameterAsync(self, keys, values) -> int:
        """Issues the put and returns at once with an rpc id for ``QueryRPCFinished`` / ``WaitRPCFinish``; the rows are
        copied first, so the caller may reuse its buffer."""
        if self._pool is None:
            self.InitThread()
        k = _keys(keys).clone()
        v = torch.as_tensor(values, dtype=torch.float32).contiguous().clone()
        assert v.shape == (k.numel(), self.dim)
        fut = self._pool.submit(lambda: _lib.call("rs_ps_client_put", self._h, k.data_ptr(), k.numel(), self.dim, v.data_ptr(),
                                                  MAX_PARAMETER_BATCH))
        rid = self._next_rpc
        self._next_rpc += 1
        self._rpcs[rid] = (fut, v)
        return rid

    # The asynchronous put of the reference's client interface (src/rdma_ps/base_client.h:37-40,
    # src/rdma_ps/petps_client.cc:147-174: the request names the keys and the caller's value buffer, the id is polled).
    FakePutParameter = PutParameterAsync

    def Barrier(self, name: str, count: int, postoffice=None) -> None:
        """Waits until ``count`` participants have called it with this name (src/rdma_ps/base_client.h:17-19).  The
        rendezvous is the process group's store: pass the ``Postoffice`` that the participants share."""
        if postoffice is None:
            raise ValueError("Barrier needs the Postoffice that the participants share")
        assert count == postoffice.num_members, "every member of the postoffice takes part in its barriers"
        postoffice.barrier(name)

    def QueryRPCFinished(self, rpc_id: int) -> bool:
        return self._rpcs[rpc_id][0].done()

    def WaitRPCFinish(self, rpc_id: int) -> None:
        self._rpcs[rpc_id][0].result()

    def GetReceiveBuffer(self, rpc_id: int) -> torch.Tensor:
        return self._rpcs[rpc_id][1]

    def RevokeRPCResource(self, rpc_id: int) -> None:
        self._rpcs.pop(rpc_id, None)

    def close(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None
        if self._h:
            self._l.rs_ps_client_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PythonParameterClient(ParameterClient):
    """``PythonParameterClient(host, port, shard, emb_dim)``: argument order of the torch custom class."""

    def __init__(self, host: str, port: int, shard: int, emb_dim: int):
        super().__init__(host, port, shard, emb_dim)


class AllShardsParameterClient:
    """Fans a request out to every shard's client and reassembles the rows in request order."""

    def __init__(self, clients: List[ParameterClient]):
        self.clients = clients
        self.dim = clients[0].dim
        self._pool = ThreadPoolExecutor(max_workers=len(clients))

    def _split(self, keys):
        k = _keys(keys)
        owner = ShardManager.KeyPartition(k, len(self.clients))
        return k, [torch.nonzero(owner == s).flatten() for s in range(len(self.clients))]

    def GetParameter(self, keys) -> torch.Tensor:
        k, parts = self._split(keys)
        out = torch.empty(k.numel(), self.dim)
        futs = [self._pool.submit(c.GetParameter, k[p]) if p.numel() else None for c, p in zip(self.clients, parts)]
        for f, p in zip(futs, parts):
            if f is not None:
                out[p] = f.result()
        return out

    def PutParameter(self, keys, values) -> bool:
        k, parts = self._split(keys)
        v = torch.as_tensor(values, dtype=torch.float32)
        futs = [self._pool.submit(c.PutParameter, k[p], v[p]) for c, p in zip(self.clients, parts) if p.numel()]
        for f in futs:
            f.result()
        return True

    def UpdateParameter(self, keys, grads) -> int:
        k, parts = self._split(keys)
        g = torch.as_tensor(grads, dtype=torch.float32)
        futs = [self._pool.submit(c.UpdateParameter, k[p], g[p]) for c, p in zip(self.clients, parts) if p.numel()]
        return sum(f.result() for f in futs)

    def ClearPS(self) -> bool:
        for c in self.clients:
            c.ClearPS()
        return True
