"""Open-loop load generation for a parameter server: Poisson arrivals, Zipf or replayed keys.

``PoissonLoadGenerator`` issues ``GetParameter`` requests at exponentially distributed intervals of a given rate from
a pool of sender threads and records each request's latency (queueing included), as the reference's load generator
does against its PS (src/grpc_ps/python_client/loadGenerator.py:16-79).  ``DatasetReplay`` iterates key batches of a
recorded trace: a text file with one request per line (ids separated by spaces or commas), or a ``.npy`` pair of ids
and offsets (src/grpc_ps/python_client/dataset.py:5-29).
"""
from __future__ import annotations

import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Callable, Iterator, List, Optional

import numpy as np
import torch

from ..utils.data import zipf_ids


def write_binary_trace(path: str, requests, dim: int = 32) -> None:
    """Writes key batches as the reference's binary trace: ``int32 nreq``, then per request ``int32 nkeys`` followed by
    ``nkeys`` records of ``{uint64 key, int32 dim}`` (src/benchmark/parse_dataset.h:19-148)."""
    with open(path, "wb") as f:
        f.write(np.int32(len(requests)).tobytes())
        for keys in requests:
            k = np.asarray(keys, dtype=np.uint64)
            f.write(np.int32(k.size).tobytes())
            rec = np.zeros(k.size, dtype=np.dtype([("key", "<u8"), ("dim", "<i4")]))
            rec["key"], rec["dim"] = k, dim
            f.write(rec.tobytes())


def read_binary_trace(path: str) -> List[np.ndarray]:
    return [r["key"].astype(np.int64) for r in _read_trace_records(path)]


VALID_TRACE_DIMS = (4, 8, 16, 32, 64)


def _read_trace_records(path: str):
    """Requests of a binary trace as structured arrays with ``key`` and ``dim`` fields; a truncated or over-long file
    is a ``ValueError`` that says where it stops making sense."""
    raw = np.fromfile(path, dtype=np.uint8)
    rec = np.dtype([("key", "<u8"), ("dim", "<i4")])

    def i32(o, what):
        if o + 4 > raw.size:
            raise ValueError(f"{path}: truncated at byte {o} (expected {what})")
        return int(raw[o:o + 4].view("<i4")[0])

    nreq = i32(0, "the request count")
    if nreq < 0:
        raise ValueError(f"{path}: negative request count {nreq}")
    o, out = 4, []
    for q in range(nreq):
        n = i32(o, f"the key count of request {q}"); o += 4
        if n < 0 or o + n * rec.itemsize > raw.size:
            raise ValueError(f"{path}: request {q} announces {n} keys but only {raw.size - o} bytes follow")
        out.append(raw[o:o + n * rec.itemsize].view(rec).copy()); o += n * rec.itemsize
    if o != raw.size:
        raise ValueError(f"{path}: {raw.size - o} trailing bytes after {nreq} requests")
    return out


def renumber_trace(in_path: str, out_path: str) -> int:
    """Rewrites a binary trace with dense keys ``0..n_unique-1`` in order of first appearance and returns ``n_unique``;
    every record's dim must be one of 4, 8, 16, 32, 64 (the reference's tool: src/benchmark/dataset_renumbering.cc:24-80)."""
    reqs = _read_trace_records(in_path)
    if not reqs:
        write_binary_trace(out_path, [])
        return 0
    allrec = np.concatenate(reqs)
    bad = ~np.isin(allrec["dim"], VALID_TRACE_DIMS)
    if bad.any():
        raise ValueError(f"{in_path}: record {int(np.nonzero(bad)[0][0])} has dim {int(allrec['dim'][bad][0])}, expected one of {VALID_TRACE_DIMS}")
    uniq, first, inv = np.unique(allrec["key"], return_index=True, return_inverse=True)
    rank = np.empty(uniq.size, dtype=np.uint64)
    rank[np.argsort(first, kind="stable")] = np.arange(uniq.size, dtype=np.uint64)      # order of first appearance
    new = rank[inv]
    with open(out_path, "wb") as f:
        f.write(np.int32(len(reqs)).tobytes())
        o = 0
        for r in reqs:
            f.write(np.int32(r.size).tobytes())
            out = r.copy()
            out["key"] = new[o:o + r.size]
            o += r.size
            f.write(out.tobytes())
    return int(uniq.size)


def trace_wordcount(path: str):
    """Keys of a binary trace with how often each is requested, most frequent first (dataset_wordcount.cc of the reference)."""
    reqs = _read_trace_records(path)
    if not reqs:
        return np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.int64)
    keys, counts = np.unique(np.concatenate(reqs)["key"], return_counts=True)
    order = np.argsort(-counts, kind="stable")
    return keys[order].astype(np.int64), counts[order].astype(np.int64)


class DatasetReplay:
    def __init__(self, path: str, offsets_path: Optional[str] = None, loop: bool = True):
        self.loop = loop
        if path.endswith(".bin"):
            self.batches = read_binary_trace(path)
        elif path.endswith(".npy"):
            ids = np.load(path).astype(np.int64).reshape(-1)
            if offsets_path:
                off = np.load(offsets_path).astype(np.int64).reshape(-1)
                if off[-1] != ids.size:
                    off = np.concatenate([off, [ids.size]])
            else:
                off = np.arange(0, ids.size + 1, 26 if ids.size % 26 == 0 else 1)
            self.batches = [ids[off[i]:off[i + 1]] for i in range(off.size - 1)]
        else:
            self.batches = []
            with open(path) as f:
                for line in f:
                    toks = line.replace(",", " ").split()
                    if toks:
                        self.batches.append(np.array([int(t) for t in toks], dtype=np.int64))
        if not self.batches:
            raise ValueError(f"no requests in {path}")

    def __len__(self):
        return len(self.batches)

    def __iter__(self) -> Iterator[torch.Tensor]:
        while True:
            for b in self.batches:
                yield torch.from_numpy(b)
            if not self.loop:
                return


def zipf_key_source(key_space: int, batch: int, alpha: float, seed: int = 0) -> Iterator[torch.Tensor]:
    rng = np.random.default_rng(seed)
    while True:
        yield torch.from_numpy(zipf_ids(batch, key_space, alpha, rng))


@dataclass
class LoadReport:
    sent: int = 0
    completed: int = 0
    keys: int = 0
    seconds: float = 0.0
    latencies_ms: List[float] = field(default_factory=list)

    def summary(self) -> dict:
        lat = np.array(self.latencies_ms) if self.latencies_ms else np.zeros(1)
        return {"sent": self.sent, "completed": self.completed, "offered_rps": self.sent / max(self.seconds, 1e-9),
                "achieved_rps": self.completed / max(self.seconds, 1e-9), "keys_per_s": self.keys / max(self.seconds, 1e-9),
                "lat_ms_mean": float(lat.mean()), "lat_ms_p50": float(np.percentile(lat, 50)),
                "lat_ms_p99": float(np.percentile(lat, 99)), "lat_ms_max": float(lat.max())}


class PoissonLoadGenerator:
    """``run(seconds)`` sends requests with exponential inter-arrival times of mean ``1 / rate`` (requests / s)."""

    def __init__(self, make_client: Callable[[], object], keys: Iterator[torch.Tensor], rate: float, senders: int = 4,
                 seed: int = 0):
        self.make_client, self.keys, self.rate, self.senders = make_client, keys, float(rate), senders
        self.rng = np.random.default_rng(seed)
        self._local = threading.local()
        self._clients: List[object] = []
        self._lock = threading.Lock()

    def _client(self):
        c = getattr(self._local, "c", None)
        if c is None:
            c = self._local.c = self.make_client()
            with self._lock:
                self._clients.append(c)
        return c

    def _one(self, k: torch.Tensor, t_arrival: float, rep: LoadReport):
        self._client().GetParameter(k)
        dt = (time.perf_counter() - t_arrival) * 1e3
        with self._lock:
            rep.completed += 1
            rep.keys += k.numel()
            rep.latencies_ms.append(dt)

    def run(self, seconds: float) -> LoadReport:
        rep = LoadReport()
        t0 = time.perf_counter()
        nxt = t0
        with ThreadPoolExecutor(max_workers=self.senders) as pool:
            while True:
                nxt += self.rng.exponential(1.0 / self.rate)
                if nxt - t0 > seconds:
                    break
                d = nxt - time.perf_counter()
                if d > 0:
                    time.sleep(d)
                pool.submit(self._one, next(self.keys), nxt, rep)   # latency counts from the scheduled arrival
                rep.sent += 1
        rep.seconds = time.perf_counter() - t0
        for c in self._clients:
            close = getattr(c, "close", None)
            if close:
                close()
        self._clients = []
        return rep


def _main(argv=None):
    """``python -m recstore_b200.ps.load_generator renumber IN OUT`` / ``wordcount IN [TOP]``."""
    import argparse
    import json
    p = argparse.ArgumentParser(description="binary PS trace tools")
    sub = p.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("renumber"); r.add_argument("src"); r.add_argument("dst")
    w = sub.add_parser("wordcount"); w.add_argument("src"); w.add_argument("top", nargs="?", type=int, default=20)
    a = p.parse_args(argv)
    if a.cmd == "renumber":
        print(json.dumps({"unique_keys": renumber_trace(a.src, a.dst)}))
    else:
        k, c = trace_wordcount(a.src)
        print(json.dumps({"unique_keys": int(k.size), "requests_keys": int(c.sum()), "top": [[int(x), int(y)] for x, y in zip(k[:a.top], c[:a.top])]}))


if __name__ == "__main__":
    _main()
