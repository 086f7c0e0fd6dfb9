"""Stand-alone parameter-server shard.

    python -m recstore_b200.ps.server --port 15000 --host 0.0.0.0 --engine KVEngineMap --dim 32 --capacity 40000000 \\
        --workers 8 --scheduler priority --monitor 1

One process serves one shard until it is told to stop (SIGINT / SIGTERM), like the reference's server binaries
(src/grpc_ps/grpc_ps_server.cpp:120-150: listens on 0.0.0.0:15000, health + reflection; grpc_ps_server_async.cpp:42-48
for the worker flags).  ``--transport tcp`` is the native framed-socket server (``csrc/runtime/ps.cpp``; ``--workers 0``
= synchronous mode, ``> 0`` = worker pool behind the FIFO or priority task provider), ``--transport grpc`` the
``xmhps.ParameterService`` of ``ps/grpc_transport.py``.  ``--path DIR`` gives a persistent engine its directory,
``--load_ckpt`` / ``--save_on_exit`` restore and keep the rows and optimizer state, ``--warm N`` preloads the keys
``1 ... N`` that the partition function gives ``--shard_id`` of ``--num_shards`` (value = key repeated: the reference's
warm-up, src/storage/kv_engine/load_db.h).  The line ``listening on HOST:PORT`` is printed when the shard accepts
requests (scripts and the experiment harness wait for it).
"""
from __future__ import annotations

import argparse
import json
import signal
import sys
import threading


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="python -m recstore_b200.ps.server", description=__doc__.split("\n")[0])
    p.add_argument("--host", default="127.0.0.1", help="IPv4 address to listen on (0.0.0.0: every interface)")
    p.add_argument("--port", type=int, default=15000, help="0 picks a free port (printed)")
    p.add_argument("--transport", choices=["tcp", "grpc"], default="tcp")
    p.add_argument("--engine", default="KVEngineMap")
    p.add_argument("--dim", type=int, default=32, help="floats per key (value_size / 4)")
    p.add_argument("--capacity", type=int, default=1 << 20)
    p.add_argument("--path", default=None, help="directory of a persistent engine")
    p.add_argument("--optimizer", choices=["rowwise_adagrad", "sgd"], default="rowwise_adagrad", help="server-side optimizer of UpdateParameter")
    p.add_argument("--lr", type=float, default=0.01)
    p.add_argument("--eps", type=float, default=1e-10)
    p.add_argument("--workers", type=int, default=0, help="tcp: worker threads behind the task provider (0: synchronous); grpc: handler threads")
    p.add_argument("--scheduler", choices=["fifo", "priority"], default="fifo")
    p.add_argument("--levels", type=int, default=7, help="priority levels of the priority scheduler")
    p.add_argument("--monitor", type=float, default=0.0, metavar="SECONDS", help="tcp: print a throughput line every SECONDS while there is traffic")
    p.add_argument("--load_fake", type=int, default=0, help="store keys 0 ... N-1 with value = key repeated")
    p.add_argument("--warm", type=int, default=0, help="store this shard's keys of 1 ... N with value = key repeated")
    p.add_argument("--shard_id", type=int, default=0)
    p.add_argument("--num_shards", type=int, default=1)
    p.add_argument("--load_ckpt", default=None)
    p.add_argument("--save_on_exit", default=None)
    return p


def main(argv=None, stop_event: "threading.Event | None" = None, on_ready=None) -> int:
    """As a process: serves until SIGINT / SIGTERM.  Embedded (a thread of another program): pass ``stop_event`` to end
    it and ``on_ready(port)`` to learn the bound port."""
    a = build_parser().parse_args(argv)
    from .client import ParameterServer
    cfg = {"dim": a.dim, "capacity": a.capacity, "optimizer": a.optimizer, "lr": a.lr, "eps": a.eps}
    if a.path:
        cfg["path"] = a.path
    ps = ParameterServer(a.engine, cfg)
    if a.load_ckpt:
        ps.LoadCkpt(a.load_ckpt)
    if a.load_fake:
        ps.LoadFakeData(a.load_fake)
    if a.warm:
        import torch
        from .client import ShardManager
        stored = 0
        for lo in range(1, a.warm + 1, 1 << 18):
            k = torch.arange(lo, min(a.warm + 1, lo + (1 << 18)), dtype=torch.int64)
            k = k[ShardManager.KeyPartition(k, a.num_shards) == a.shard_id]
            if k.numel():
                ps.PutParameter(k, k.to(torch.float32).unsqueeze(1).expand(-1, a.dim).contiguous())
                stored += k.numel()
        print(f"warmed {stored} keys of shard {a.shard_id}/{a.num_shards}", flush=True)
    gsrv = None
    if a.transport == "grpc":
        from .grpc_transport import GrpcParameterServer
        gsrv = GrpcParameterServer(ps, a.port, a.host, workers=max(1, a.workers or 8))
        port = gsrv.port
    else:
        port = ps.serve(a.port, workers=a.workers, scheduler=a.scheduler, levels=a.levels, host=a.host)
        if a.monitor > 0:
            ps.start_monitor(a.monitor)
    stop = stop_event or threading.Event()
    if stop_event is None:                       # as a process: leave on SIGINT / SIGTERM
        for sig in (signal.SIGINT, signal.SIGTERM):
            signal.signal(sig, lambda *_: stop.set())
    print(f"listening on {a.host}:{port} ({a.transport}, engine {a.engine}, {len(ps)} keys)", flush=True)
    if on_ready is not None:
        on_ready(port)
    while not stop.wait(0.2):
        pass
    if gsrv is not None:
        gsrv.stop()
    else:
        ps.stop()
    summary = {"keys_stored": len(ps)}
    if a.save_on_exit:
        ps.SaveCkpt(a.save_on_exit)
        summary["saved"] = a.save_on_exit
    print(json.dumps({"stopped": summary}), flush=True)
    ps.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
