"""Parameter-server client benchmark: closed loop with a window of requests in flight, or open loop (Poisson).

    python -m recstore_b200.bench.ps_client --threads 4 --window 4 --batch 500 --alpha 0.99 --seconds 3
    python -m recstore_b200.bench.ps_client --poisson-rate 2000 --seconds 3
    python -m recstore_b200.bench.ps_client --processes 8 --threads 2 --seconds 3

Starts an in-process server shard on a loopback port unless ``--host/--port`` point at a running one.  Prints the
throughput once per second and a JSON summary, like the reference's closed-loop client benchmark
(src/benchmark/benchmark_client_common.h:16-292: async window, zipf or dataset keys, per-second print).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

from ..ps import ParameterClient, ParameterServer
from ..ps.load_generator import DatasetReplay, PoissonLoadGenerator, zipf_key_source


def make_client(host, port, dim, transport="tcp"):
    """``tcp``: the native framed-socket client; ``grpc``: the reference's transport (``ps/grpc_transport.py``)."""
    if transport == "grpc":
        from ..ps.grpc_transport import GrpcParameterClient
        return GrpcParameterClient(host, port, 0, dim)
    return ParameterClient(host, port, 0, dim)


def _latency(hists, quiet) -> dict:
    """The threads' latency histograms merged: percentiles for the JSON line, the bucket table on stderr."""
    total = hists[0]
    for h in hists[1:]:
        total.Merge(h)
    if not quiet and os.environ.get("RECSTORE_PS_CLIENT_HISTOGRAM"):
        print(total.ToString(), file=sys.stderr)
    s = total.summary()
    return {"lat_us_mean": s["mean"], "lat_us_p50": total.Percentile(50), "lat_us_p99": total.Percentile(99), "lat_us_max": s["max"]}


def closed_loop(host, port, dim, threads, window, batch, alpha, key_space, seconds, dataset=None, quiet=False, transport="tcp",
                cut_off_period=0.0, cut_off_stride=2):
    """``cut_off_period > 0``: the thread cut-off mode of the reference's client benchmark
    (src/benchmark/benchmark_client_common.h:156-184): every period ``cut_off_stride`` sender threads are stopped, the
    run ends when none is left (``seconds`` is ignored), and the result lists the throughput seen at every thread
    count -- one run gives the whole load curve."""
    done = [0] * threads
    stop = threading.Event()
    stop_one = [threading.Event() for _ in range(threads)]
    from ..utils.timer import Histogram
    hists = [Histogram() for _ in range(threads)]        # request latency in microseconds, issue to completion

    def worker(t):
        c = make_client(host, port, dim, transport)
        c.InitThread(window)
        src = iter(DatasetReplay(dataset)) if dataset else zipf_key_source(key_space, batch, alpha, seed=t + 1)
        inflight = []
        while not stop.is_set() and not stop_one[t].is_set():
            while len(inflight) < window:
                k = next(src)
                inflight.append((c.GetParameterAsync(k), k.numel(), time.perf_counter()))
            rid, n, t_issue = inflight.pop(0)
            c.WaitRPCFinish(rid)
            hists[t].Add((time.perf_counter() - t_issue) * 1e6)
            c.RevokeRPCResource(rid)
            done[t] += n
        for rid, _, _ in inflight:
            c.WaitRPCFinish(rid)
        c.close()

    ths = [threading.Thread(target=worker, args=(t,)) for t in range(threads)]
    t0 = time.perf_counter()
    for th in ths:
        th.start()
    last, last_t = 0, t0
    per_sec = []
    if cut_off_period > 0:
        curve, alive = [], threads
        while alive > 0:
            a0, n0 = time.perf_counter(), sum(done)
            time.sleep(cut_off_period)
            rate = (sum(done) - n0) / (time.perf_counter() - a0)
            curve.append({"threads": alive, "keys_per_s": rate})
            if not quiet:
                print(f"[ps_client] {alive:3d} threads {rate / 1e6:8.3f} M keys/s", flush=True)
            for _ in range(min(cut_off_stride, alive)):
                alive -= 1
                stop_one[alive].set()
                ths[alive].join()
        el = time.perf_counter() - t0
        return {"mode": "closed_cut_off", "threads": threads, "window": window, "batch": batch, "keys_per_s": sum(done) / el,
                "by_threads": curve, "seconds": el, **_latency(hists, quiet)}
    while time.perf_counter() - t0 < seconds:
        time.sleep(min(1.0, max(0.05, seconds - (time.perf_counter() - t0))))
        now, tot = time.perf_counter(), sum(done)
        rate = (tot - last) / (now - last_t)
        per_sec.append(rate)
        if not quiet:
            print(f"[ps_client] {rate / 1e6:8.3f} M keys/s", flush=True)
        last, last_t = tot, now
    stop.set()
    for th in ths:
        th.join()
    el = time.perf_counter() - t0
    return {"mode": "closed", "threads": threads, "window": window, "batch": batch, "keys_per_s": sum(done) / el,
            "per_second": per_sec, "seconds": el, **_latency(hists, quiet)}


def _process_entry(args, q):
    q.put(closed_loop(*args))          # args end with (dataset, quiet, transport)


def multi_process(host, port, dim, processes, threads, window, batch, alpha, key_space, seconds, dataset=None, transport="tcp"):
    """``processes`` load-generator processes (each with ``threads`` closed-loop senders) against one server: the Python
    interpreter of a single process is the limit long before the server is, as the reference's multi_client.py (8
    processes) works around (src/grpc_ps/python_client/multi_client.py)."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_process_entry, args=((host, port, dim, threads, window, batch, alpha, key_space, seconds, dataset, True, transport), q))
          for _ in range(processes)]
    for p in ps:
        p.start()
    res = [q.get(timeout=seconds + 120) for _ in ps]
    for p in ps:
        p.join(30)
    return {"mode": "closed", "processes": processes, "threads": threads, "window": window, "batch": batch,
            "keys_per_s": sum(r["keys_per_s"] for r in res), "per_process": [r["keys_per_s"] for r in res],
            "seconds": max(r["seconds"] for r in res),
            "lat_us_p50": float(np.median([r["lat_us_p50"] for r in res])), "lat_us_p99": max(r["lat_us_p99"] for r in res),
            "lat_us_max": max(r["lat_us_max"] for r in res)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--host", default=None)
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--dim", type=int, default=32)
    ap.add_argument("--threads", type=int, default=2)
    ap.add_argument("--window", type=int, default=4, help="requests in flight per thread")
    ap.add_argument("--batch", type=int, default=500)
    ap.add_argument("--alpha", type=float, default=0.99)
    ap.add_argument("--key-space", type=int, default=1_000_000)
    ap.add_argument("--seconds", type=float, default=3.0)
    ap.add_argument("--dataset", default=None, help="replay key batches from this file instead of Zipf keys")
    ap.add_argument("--poisson-rate", type=float, default=0.0, help="open loop: requests per second (0 = closed loop)")
    ap.add_argument("--engine", default="KVEngineMap")
    ap.add_argument("--processes", type=int, default=1, help="closed loop: load-generator processes, each with --threads senders")
    ap.add_argument("--transport", choices=["tcp", "grpc"], default="tcp", help="framed loopback sockets or gRPC (closed loop / poisson)")
    ap.add_argument("--thread-cut-off", type=float, default=0.0, metavar="SECONDS",
                    help="closed loop: stop --cut-off-stride sender threads every SECONDS and report the throughput per thread count")
    ap.add_argument("--cut-off-stride", type=int, default=2)
    ap.add_argument("--histogram", action="store_true", help="closed loop: print the request-latency histogram (microseconds) to stderr")
    a = ap.parse_args(argv)
    if a.histogram:
        os.environ["RECSTORE_PS_CLIENT_HISTOGRAM"] = "1"
    srv = None
    host, port = a.host, a.port
    if host is None:
        srv = ParameterServer(a.engine, {"capacity": int(a.key_space * 1.5), "dim": a.dim})
        srv.LoadFakeData(a.key_space)
        if a.transport == "grpc":
            from ..ps.grpc_transport import GrpcParameterServer
            gsrv = GrpcParameterServer(srv, 0, workers=max(8, a.threads * 2))
            host, port = "127.0.0.1", gsrv.port
        else:
            host, port = "127.0.0.1", srv.serve(0)
    try:
        if a.poisson_rate > 0:
            src = iter(DatasetReplay(a.dataset)) if a.dataset else zipf_key_source(a.key_space, a.batch, a.alpha)
            gen = PoissonLoadGenerator(lambda: make_client(host, port, a.dim, a.transport), src, a.poisson_rate, senders=a.threads)
            out = {"mode": "poisson", "rate": a.poisson_rate, **gen.run(a.seconds).summary()}
        elif a.processes > 1:
            out = multi_process(host, port, a.dim, a.processes, a.threads, a.window, a.batch, a.alpha, a.key_space, a.seconds, a.dataset,
                                transport=a.transport)
        else:
            out = closed_loop(host, port, a.dim, a.threads, a.window, a.batch, a.alpha, a.key_space, a.seconds, a.dataset,
                              transport=a.transport, cut_off_period=a.thread_cut_off, cut_off_stride=a.cut_off_stride)
        out["transport"] = a.transport
        print(json.dumps(out), flush=True)
    finally:
        if srv is not None:
            srv.close()


if __name__ == "__main__":
    main()
