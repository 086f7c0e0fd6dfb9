"""PS / cache micro-benchmark: lookup + row-wise Adagrad update batches on a tiered or a sharded table.

    python -m recstore_b200.bench.ps_microbench --rows 100000000 --dim 32 --hbm-ratio 0.1            # 1 GPU, HBM + host tier
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m recstore_b200.bench.ps_microbench --sharded

One GPU: ``TieredEmbeddingTable`` (hot id range in HBM, the rest in pinned host memory read in place); reports
Mkeys/s and the HBM hit ratio for every (Zipf alpha, batch) pair.  ``--sharded`` (any number of ranks): the table is
row-sharded over the GPUs' HBM (``ShardedEmbeddingTable``, owner = id % world), keys / rows / gradients travel by
peer stores; reports Mkeys/s summed over ranks and the NVLink GB/s of the exchange.  Device-timed with CUDA events,
warm-up first, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--rows", type=int, default=20_000_000, help="table rows (the headline config has 1e9: 128 GB at dim 32)")
    ap.add_argument("--dim", type=int, default=32)
    ap.add_argument("--hbm-ratio", type=float, default=0.1)
    ap.add_argument("--alphas", type=float, nargs="+", default=[0.9, 1.1, 1.3])
    ap.add_argument("--batches", type=int, nargs="+", default=[4096, 32768, 262144])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--prefetch", action="store_true", help="tiered table: stage the next batch's rows one step ahead (lookahead prefetch)")
    ap.add_argument("--sharded-tiered", action="store_true",
                    help="with --sharded / several ranks: every shard keeps only --hbm-ratio of its rows in HBM, the rest in pinned host memory")
    ap.add_argument("--sharded", action="store_true", help="all-HBM table sharded over the ranks instead of the tiered table")
    a = ap.parse_args(argv)
    from recstore_b200.utils.data import zipf_ids_torch
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    maxb = max(a.batches)
    if a.sharded or world > 1:
        from recstore_b200.parallel.peer import PeerContext
        from recstore_b200.parallel.sharded_table import ShardedEmbeddingTable
        ctx = PeerContext(rank, world, device=dev)
        tab = ShardedEmbeddingTable(ctx, "psbench", a.rows, a.dim, max_keys=maxb, lr=0.01,
                                    hbm_ratio=a.hbm_ratio if a.sharded_tiered else 1.0)
    else:
        from recstore_b200.cache.tiered_table import TieredEmbeddingTable
        tab = TieredEmbeddingTable(a.rows, a.dim, a.hbm_ratio, max_keys=maxb, lr=0.01, device=dev)
    for alpha in a.alphas:
        for B in a.batches:
            g = torch.Generator(device=dev).manual_seed(17 + rank)
            pool = [zipf_ids_torch(B, a.rows, alpha, generator=g, device=dev) for _ in range(4)]
            grads = torch.randn(B, a.dim, device=dev) * 0.01
            it = [0]

            def step():
                ids = pool[it[0] & 3]
                it[0] += 1
                tab.lookup(ids)
                if a.prefetch and hasattr(tab, "prefetch"):
                    tab.prefetch(pool[it[0] & 3])        # next step's rows are staged while this step updates
                tab.update(grads)
            if hasattr(tab, "hit_stats"):
                tab.hit_stats()
            ms = _time(step, a.iters)
            uniq = float(torch.stack([torch.unique(p).numel() * torch.ones((), device=dev) for p in pool]).mean().item())
            rec = {"alpha": alpha, "batch_per_gpu": B, "ms": round(ms, 4), "mkeys_per_s_per_gpu": round(B / ms / 1e3, 2),
                   "unique_fraction": round(uniq / B, 4)}
            if world > 1:
                import torch.distributed as dist
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = t.item()
                remote = uniq * (world - 1) / world
                rec.update({"ms": round(ms, 4), "mkeys_per_s_total": round(B * world / ms / 1e3, 2),
                            "nvlink_gbs_per_gpu": round(2 * tab.nvlink_bytes_per_lookup(int(remote)) / ms / 1e6, 2),
                            "mode": f"sharded x{world}" + (f" tiered hbm_ratio={a.hbm_ratio}" if a.sharded_tiered else "")})
            elif a.sharded:
                rec["mode"] = "sharded x1"
            else:
                rec.update({"mode": f"tiered hbm_ratio={a.hbm_ratio}", **tab.hit_stats()})
            if rank == 0:
                print(json.dumps(rec), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
