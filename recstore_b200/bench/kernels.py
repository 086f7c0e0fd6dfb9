"""Per-kernel micro-benchmarks with roofline fractions.

    python -m recstore_b200.bench.kernels --kernel all
    python -m recstore_b200.bench.kernels --kernel gemm --m 65536 --n 1024 --k 1024
    python -m recstore_b200.bench.kernels --kernel gemm --small          # sizes suited to an ncu capture

Timing: CUDA events on the launching stream, >= 3 warm-up launches, an L2 flush (a 256 MB write) between
timed launches, median of the timed launches.  Fractions are against the measured copy bandwidth and
cuBLAS bf16 throughput in ``MEASURED_PEAKS.json`` at the repository root (fallback 6.65 TB/s and
1.59 PFLOP/s when the file is absent; the output says which).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
from typing import Callable, Dict

import torch

from ..ops import functional as F_


def peaks() -> Dict[str, float]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


class Timer:
    def __init__(self, dev):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def run(self, fn: Callable[[], None], iters: int = 10, warmup: int = 3) -> float:
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            self.flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)


def _report(name, ms, flops=None, bytes_=None, extra=""):
    pk = peaks()
    out = {"kernel": name, "ms": round(ms, 4)}
    if flops:
        tf = flops / ms / 1e9
        out["tflops"] = round(tf, 1)
        out[f"frac_of_{pk['kind']}_bf16"] = round(tf / pk["bf16_tflops"], 3)
    if bytes_:
        gb = bytes_ / ms / 1e6
        out["gbs"] = round(gb, 1)
        out[f"frac_of_{pk['kind']}_hbm"] = round(gb / pk["hbm_gbs"], 3)
    if extra:
        out["note"] = extra
    print(json.dumps(out), flush=True)
    return out


def bench_gemm(tm, dev, M, N, K, mode=0, epi=F_.EPI_RELU):
    g = torch.Generator(device=dev).manual_seed(0)
    st = torch.zeros(1, dtype=torch.int64, device=dev)
    if mode == 0:
        a = torch.randn(M, K, device=dev, generator=g).bfloat16()
        b = torch.randn(N, K, device=dev, generator=g).bfloat16()
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        bias = torch.zeros(N, device=dev)
        aux = torch.randn(M, N, device=dev, generator=g).bfloat16() if epi == F_.EPI_RELU_MASK else None
        fn = lambda: F_.gemm_bf16(a, b, out, mode=0, epi=epi, bias=bias if epi != F_.EPI_RELU_MASK else None, aux=aux, status=st)
        bytes_ = 2 * (M * K + N * K + M * N) + (2 * M * N if aux is not None else 0)
        name = f"gemm_tn M={M} N={N} K={K} epi={epi}"
    else:
        a = torch.randn(K, M, device=dev, generator=g).bfloat16()
        b = torch.randn(K, N, device=dev, generator=g).bfloat16()
        out = torch.zeros(M, N, device=dev)
        fn = lambda: F_.gemm_bf16(a, b, out, mode=1, epi=F_.EPI_ATOMIC_F32, status=st)
        bytes_ = 2 * (M * K + N * K) + 4 * M * N
        name = f"gemm_nt(wgrad) M={M} N={N} R={K}"
    ms = tm.run(fn)
    assert st.item() == 0
    return _report(name, ms, flops=2.0 * M * N * K, bytes_=bytes_)


def bench_embedding(tm, dev, B, T, D, rows, alpha=1.2):
    from ..utils.data import zipf_ids_torch
    i64 = dict(dtype=torch.int64, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    weight = torch.randn(rows * T, D, device=dev)
    state = torch.zeros(rows * T, device=dev)
    ids = torch.cat([zipf_ids_torch(B, rows, alpha, device=dev) for _ in range(T)])
    out = torch.empty(B, T * D, device=dev, dtype=torch.bfloat16)
    row_idx = torch.empty(B * T, **i64)
    occ2bag = torch.empty(B * T, **i32)
    st = torch.zeros(1, dtype=torch.int64, device=dev)
    tb = torch.arange(T, **i64) * rows
    tr = torch.full((T,), rows, **i64)
    hot = torch.ones(T, **i32)
    hb = torch.arange(T, **i64) * B
    dst = torch.tensor([out.data_ptr()], **i64)
    col = (torch.arange(T, **i32) * D).to(torch.int32)
    fwd = lambda: F_.emb_forward(weight, tb, tr, ids, hotness=hot, hot_base=hb, T=T, B=B, D=D, B_local=B, dst_table=dst,
                                 dst_row_stride=T * D, dst_col=col, out_bf16=True, row_idx=row_idx, occ2bag=occ2bag, status=st)
    ms = tm.run(fwd)
    _report(f"emb_fwd B={B} T={T} D={D} rows/table={rows} zipf={alpha}", ms, bytes_=B * T * (D * 4 + D * 2 + 8 + 12),
            extra="bytes = fp32 row read + bf16 row write + id + row_idx/occ2bag per bag (duplicates served by L2 count as read)")
    grad = torch.randn(B, T * D, device=dev).bfloat16()
    gnorm = grad.float().view(B, T, D).pow(2).sum(-1).contiguous()
    bwd = lambda: F_.emb_backward(weight, state, row_idx, occ2bag, B * T, grad, grad_col=col, grad_row_stride=T * D, B=B, D=D,
                                  grad_bf16=True, lr=0.01, optimizer="rowwise_adagrad", status=st, gnorm=gnorm, gnorm_stride=T)
    ms = tm.run(bwd)
    _report(f"emb_bwd(rowwise adagrad) B={B} T={T} D={D} zipf={alpha}", ms, bytes_=B * T * (D * 2 + 16 + 4) + 2 * B * T * D * 4 // 4,
            extra="bytes = bf16 grad read + indices + norm; unique-row RMW estimated at 1/4 of occurrences")


def bench_cache(tm, dev, n_keys, D, items, alpha=1.1):
    """32-way set-associative HBM cache: Query of a Zipf batch (hits copy a row, misses are listed), Replace of the missed
    keys, Update of resident rows.  Bytes counted: 8 B key + one 256 B tag line per probe + the rows moved."""
    from ..cache.gpu_cache import GpuCache
    from ..utils.data import zipf_ids_torch
    cache = GpuCache(items, D, dev)
    space = items * 4
    perm = torch.randperm(space, device=dev)                 # popular ids are spread over the sets
    warm = perm[: items * 3 // 4]                             # the cache holds the most popular keys, as a warmed-up cache would
    cache.Replace(warm, torch.randn(warm.numel(), D, device=dev))
    keys = perm[zipf_ids_torch(n_keys, space, alpha, device=dev)]
    vals = torch.empty(n_keys, D, device=dev)
    r = cache.Query(keys, vals)
    hit = 1.0 - r.missing_keys.numel() / n_keys
    ms = tm.run(lambda: cache.Query(keys, vals, sync=False))
    _report(f"cache_query n={n_keys} D={D} items={items} zipf={alpha} hit={hit:.2f}", ms,
            bytes_=n_keys * (8 + 256) + int(n_keys * hit) * D * 4 * 2,
            extra="bytes = key + 256-B tag line per probe, row read + row write per hit")
    resident = keys[torch.isin(keys, r.missing_keys, invert=True)]
    upd = torch.unique(resident)
    uv = torch.randn(upd.numel(), D, device=dev)
    ms = tm.run(lambda: cache.Update(upd, uv))
    _report(f"cache_update n={upd.numel()} D={D}", ms, bytes_=upd.numel() * (8 + 256 + D * 4 * 2),
            extra="bytes = key + tag line + value read + row write")
    fresh = torch.arange(space, space + n_keys, device=dev)   # all absent: every key evicts the LRU way of its set
    fv = torch.randn(n_keys, D, device=dev)
    ms = tm.run(lambda: cache.Replace(fresh, fv), iters=5)
    _report(f"cache_replace n={n_keys} D={D} (all new keys)", ms, bytes_=n_keys * (8 + 512 + D * 4 * 2),
            extra="bytes = key + tag and stamp lines + value read + row write")
    cache.status.zero_()


def bench_hash(tm, dev, n_keys, capacity):
    """GPU hash table (open addressing, 64-bit CAS): insert of new keys, lookup of resident keys, device-side unique."""
    from ..cache.gpu_cache import GpuHashTable, unique_keys
    from ..utils.data import zipf_ids_torch
    ht = GpuHashTable(capacity, device=dev)
    base = torch.randperm(capacity * 2, device=dev)[: capacity // 2]
    ht.insert(base)                                           # load factor 0.5 before the timed calls
    look = base[torch.randint(0, base.numel(), (n_keys,), device=dev)]
    ms = tm.run(lambda: ht.lookup(look))
    _report(f"hash_lookup n={n_keys} capacity={capacity} load=0.5", ms, bytes_=n_keys * (8 + 32 + 8),
            extra="bytes = key + one 32-B sector of the slot array per probe + row index out")
    ms = tm.run(lambda: ht.lookup(look + capacity * 4))
    _report(f"hash_lookup (all absent) n={n_keys}", ms, bytes_=n_keys * (8 + 32 + 8))
    dup = zipf_ids_torch(n_keys, capacity, 1.1, device=dev)
    ms = tm.run(lambda: unique_keys(dup))
    _report(f"unique_keys n={n_keys} zipf=1.1", ms, bytes_=n_keys * (8 + 32 + 8 + 8),
            extra="includes the scratch-table clear; bytes = key + slot sector + inverse + unique list")


def bench_interaction(tm, dev, B, F, D):
    T = torch.randn(B, F, D, device=dev).bfloat16()
    n = D + F * (F - 1) // 2
    ld = (n + 63) // 64 * 64
    out = torch.empty(B, ld, device=dev, dtype=torch.bfloat16)
    ms = tm.run(lambda: F_.interaction_forward(T, B, F, D, out))
    _report(f"interaction_fwd B={B} F={F} D={D}", ms, bytes_=B * (F * D * 2 + ld * 2), flops=2.0 * B * F * F * D)
    dout = torch.randn(B, ld, device=dev).bfloat16()
    dx = torch.empty(B, D, device=dev, dtype=torch.bfloat16)
    G = torch.empty(B, (F - 1) * D, device=dev, dtype=torch.bfloat16)
    nrm = torch.empty(B, F - 1, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    own = torch.zeros(F - 1, **i32)
    gcol = (torch.arange(F - 1, **i32) * D).to(torch.int32)
    gt = torch.tensor([G.data_ptr()], dtype=torch.int64, device=dev)
    nt = torch.tensor([nrm.data_ptr()], dtype=torch.int64, device=dev)
    ms = tm.run(lambda: F_.interaction_backward(T, dout, B, F, D, dx, gt, own, gcol, G.stride(0), 0, True, nt, F - 1))
    _report(f"interaction_bwd B={B} F={F} D={D}", ms, bytes_=B * (2 * F * D * 2 + ld * 2 + (F - 1) * 4), flops=2.0 * B * 32 * 32 * D)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", choices=["all", "gemm", "wgrad", "embedding", "interaction", "cache", "hash"])
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--epi", type=int, default=F_.EPI_RELU)
    ap.add_argument("--batch", type=int, default=65536)
    ap.add_argument("--alpha", type=float, default=1.2, help="Zipf exponent of the embedding ids (0 = uniform)")
    ap.add_argument("--small", action="store_true", help="a few hundred MB on the device: suited to an ncu capture")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    tm = Timer(dev)
    print(json.dumps({"peaks": peaks()}), flush=True)
    B = 16384 if a.small else a.batch
    if a.kernel in ("all", "gemm"):
        if a.kernel == "gemm":
            bench_gemm(tm, dev, 16384 if a.small else a.m, a.n, a.k, 0, a.epi)
        else:
            for (n, k) in [(1024, 1024), (1024, 512), (512, 1024), (256, 512), (512, 64), (128, 256)]:
                bench_gemm(tm, dev, B, n, k, 0, F_.EPI_RELU)
            bench_gemm(tm, dev, B, 1024, 512, 0, F_.EPI_RELU_MASK)
    if a.kernel in ("all", "wgrad"):
        for (m, n) in [(1024, 1024), (1024, 512), (256, 512)]:
            bench_gemm(tm, dev, m, n, B, 1)
    if a.kernel in ("all", "embedding"):
        bench_embedding(tm, dev, B, 26 if not a.small else 8, 128, 1_000_000, alpha=a.alpha)
    if a.kernel in ("all", "interaction"):
        bench_interaction(tm, dev, B, 27, 128)
    if a.kernel in ("all", "cache"):
        bench_cache(tm, dev, 262144 if a.small else 1 << 20, 128, (1 << 20) if a.small else (1 << 22), a.alpha)
    if a.kernel in ("all", "hash"):
        bench_hash(tm, dev, 1 << 20 if a.small else 1 << 22, 1 << 24)


if __name__ == "__main__":
    main()
