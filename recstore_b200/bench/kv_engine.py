"""Throughput of the host KV engines (closed loop, Zipf keys), in millions of key-values per second.

    python -m recstore_b200.bench.kv_engine --engine KVEngineChunkHash --threads 8 --batch 128 --alpha 0.99

The measuring loop is native (``csrc/runtime/kv_bench.cpp``); this module builds the engine, pre-loads it and prints
one JSON line per engine.  Same knobs as the reference's benchmark_kv_engine (thread count, batch size, Zipf theta,
read ratio; src/storage/kv_engine/benchmark_kv_engine.cc:50-186).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import tempfile
from typing import Optional

from .. import _lib
from .._lib import f64, i32, i64, u64, vp
from ..storage import BaseKV, list_engines

_lib.register_signatures({
    "rs_kv_benchmark": (i32, [vp, i32, f64, i32, f64, f64, u64, u64, C.POINTER(f64)]),
    "rs_zipf_check": (i32, [u64, f64, u64, i64, i64, C.POINTER(f64), C.POINTER(f64)]),
})


def run_engine(engine: str, *, threads: int = 4, seconds: float = 1.0, batch: int = 128, alpha: float = 0.99,
               read_ratio: float = 1.0, key_space: int = 1_000_000, value_size: int = 128, path: Optional[str] = None,
               seed: int = 1, preload: bool = True) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        kv = BaseKV(engine, {"path": path or tmp, "capacity": int(key_space * 1.5), "value_size": value_size})
        try:
            if preload:
                kv.BulkLoad(key_space)
            out = (f64 * 8)()
            _lib.call("rs_kv_benchmark", kv._h, threads, float(seconds), batch, float(alpha), float(read_ratio),
                      int(key_space), int(seed), out)
            return {"engine": engine, "threads": threads, "batch": batch, "zipf_alpha": alpha, "read_ratio": read_ratio,
                    "key_space": key_space, "value_size": value_size, "get_mkvs": round(out[0], 3),
                    "put_mkvs": round(out[1], 3), "hit_ratio": round(out[2], 4), "batches_per_s": round(out[3], 1),
                    "mean_batch_us": round(out[4], 2), "max_batch_us": round(out[5], 1), "seconds": round(out[6], 3)}
        finally:
            kv.close()


def zipf_check(key_space: int, alpha: float, n: int = 1_000_000, top: int = 100, seed: int = 7) -> dict:
    """Empirical mass of the ``top`` hottest ids against the analytic value of the bounded Zipf density."""
    mass, rate = f64(), f64()
    _lib.call("rs_zipf_check", int(key_space), float(alpha), int(seed), int(n), int(top), C.byref(mass), C.byref(rate))
    n1 = key_space + 1.0
    if abs(alpha - 1.0) < 1e-9:
        import math
        expect = math.log(top + 1.0) / math.log(n1)
    else:
        e = 1.0 - alpha
        expect = ((top + 1.0) ** e - 1.0) / (n1 ** e - 1.0)
    return {"alpha": alpha, "top": top, "mass": mass.value, "expected": expect, "draws_per_s": rate.value}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--engine", default="all", help="engine name or 'all' (%s)" % ", ".join(list_engines()))
    ap.add_argument("--threads", type=int, default=4)
    ap.add_argument("--seconds", type=float, default=2.0)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--alpha", type=float, default=0.99, help="Zipf exponent (0 = uniform)")
    ap.add_argument("--read-ratio", type=float, default=1.0)
    ap.add_argument("--key-space", type=int, default=1_000_000)
    ap.add_argument("--value-size", type=int, default=128, help="bytes per value")
    ap.add_argument("--zipf-check", action="store_true", help="only check the key generator against its analytic CDF")
    a = ap.parse_args(argv)
    if a.zipf_check:
        print(json.dumps(zipf_check(a.key_space, a.alpha)))
        return
    for e in (list_engines() if a.engine == "all" else [a.engine]):
        print(json.dumps(run_engine(e, threads=a.threads, seconds=a.seconds, batch=a.batch, alpha=a.alpha,
                                    read_ratio=a.read_ratio, key_space=a.key_space, value_size=a.value_size)), flush=True)


if __name__ == "__main__":
    main()
