"""PS / cache micro-benchmark: lookup + row-wise Adagrad update batches on a tiered or a sharded table.

    python -m recstore_b200.bench.ps_microbench --rows 100000000 --dim 32 --hbm-ratio 0.1            # 1 GPU, HBM + host tier
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m recstore_b200.bench.ps_microbench --sharded

One GPU: ``TieredEmbeddingTable`` (hot id range in HBM, the rest in pinned host memory read in place); reports
Mkeys/s and the HBM hit ratio for every (Zipf alpha, batch) pair.  ``--sharded`` (any number of ranks): the table is
row-sharded over the GPUs' HBM (``ShardedEmbeddingTable``, owner = id % world), keys / rows / gradients travel by
peer stores; reports Mkeys/s summed over ranks and the NVLink GB/s of the exchange.  Device-timed with CUDA events,
warm-up first, max over ranks.  ``--graph`` replays each lookup + update pair from a CUDA graph (what a training loop
does); ``--impl torch`` runs the same work as PyTorch ops + NCCL ``all_to_all_single`` (bucket by owner, exchange
counts / keys / rows, ``index_select``; gradients back, ``unique`` + ``index_add_`` + row-wise Adagrad on the owner): the
path of the reference's sharded cached embedding (src/python/pytorch/recstore/cache/sharded_cache.py:181-345).
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


class TorchShardedTable:
    """The comparison arm: the same row-sharded table on PyTorch ops and NCCL collectives."""

    def __init__(self, rows, dim, rank, world, dev, lr=0.01, eps=1e-10):
        self.rank, self.world, self.dev, self.D, self.lr, self.eps = rank, world, dev, dim, lr, eps
        self.local_rows = (rows + world - 1) // world
        self.weight = torch.empty(self.local_rows, dim, device=dev).uniform_(-0.01, 0.01)
        self.state = torch.zeros(self.local_rows, device=dev)

    def _a2a(self, send, send_counts, recv_counts, width=None):
        import torch.distributed as dist
        shape = (int(sum(recv_counts)),) + (() if width is None else (width,))
        recv = torch.empty(shape, dtype=send.dtype, device=self.dev)
        if self.world == 1:
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=send_counts)
        return recv

    def lookup(self, ids):
        import torch.distributed as dist
        uniq, self._inv = torch.unique(ids, return_inverse=True)
        owner = uniq % self.world
        order = torch.argsort(owner, stable=True)
        self._order = order
        keys = uniq[order]
        sc = torch.bincount(owner, minlength=self.world)
        rc = torch.empty_like(sc)
        if self.world == 1:
            rc.copy_(sc)
        else:
            dist.all_to_all_single(rc, sc)
        self._sc, self._rc = sc.tolist(), rc.tolist()                   # host sync, as in the reference's shape exchange
        got = self._a2a(keys, self._sc, self._rc)
        self._local = got // self.world
        rows = self._a2a(self.weight.index_select(0, self._local), self._rc, self._sc, self.D)
        out = torch.empty(uniq.numel(), self.D, device=self.dev)
        out[order] = rows
        return out[self._inv]

    def update(self, grads):
        n_u = self._order.numel()
        ug = torch.zeros(n_u, self.D, device=self.dev).index_add_(0, self._inv, grads)
        un = torch.zeros(n_u, device=self.dev).index_add_(0, self._inv, grads.pow(2).sum(1))
        g = self._a2a(ug[self._order], self._sc, self._rc, self.D)
        nrm = self._a2a(un[self._order], self._sc, self._rc)
        rows, inv = torch.unique(self._local, return_inverse=True)
        gs = torch.zeros(rows.numel(), self.D, device=self.dev).index_add_(0, inv, g)
        ns = torch.zeros(rows.numel(), device=self.dev).index_add_(0, inv, nrm)
        st = self.state[rows] + ns / self.D
        self.state[rows] = st
        self.weight[rows] -= self.lr * gs / (st.sqrt() + self.eps).unsqueeze(1)

    def nvlink_bytes_per_lookup(self, n_unique_remote):
        return n_unique_remote * (8 + self.D * 4)


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
    ap.add_argument("--lookahead", type=int, default=0,
                    help="one GPU: host-resident table behind a write-back HBM cache of --hbm-ratio of the rows, batches announced this "
                         "many steps ahead (LookaheadCachedTable) instead of the static hot range")
    ap.add_argument("--graph", action="store_true", help="sharded table: replay lookup + update from a CUDA graph")
    ap.add_argument("--legacy", action="store_true", help="sharded table: separate count / signal / wait launches instead of the fused kernels")
    ap.add_argument("--hashed", action="store_true", help="sharded table: hash-table shards (keys inserted on first touch)")
    ap.add_argument("--impl", default="native", choices=["native", "torch"], help="torch: PyTorch ops + NCCL all_to_all_single (sharded table only)")
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
        if a.impl == "torch":
            tab = TorchShardedTable(a.rows, a.dim, rank, world, dev)
        else:
            ctx = PeerContext(rank, world, device=dev)
            tab = ShardedEmbeddingTable(ctx, "psbench", a.rows, a.dim, max_keys=maxb, lr=0.01,
                                        hbm_ratio=a.hbm_ratio if a.sharded_tiered else 1.0, fused=not a.legacy, hashed=a.hashed)
    elif a.lookahead > 0:
        from recstore_b200.cache import LookaheadCachedTable
        tab = LookaheadCachedTable(a.rows, a.dim, int(a.rows * a.hbm_ratio), maxb, lr=0.01, device=dev, lookahead=a.lookahead)
    else:
        from recstore_b200.cache.tiered_table import TieredEmbeddingTable
        tab = TieredEmbeddingTable(a.rows, a.dim, a.hbm_ratio, max_keys=maxb, lr=0.01, device=dev)
    for alpha in a.alphas:
        for B in a.batches:
            g = torch.Generator(device=dev).manual_seed(17 + rank)
            pool = [zipf_ids_torch(B, a.rows, alpha, generator=g, device=dev) for _ in range(4)]
            grads = torch.randn(B, a.dim, device=dev) * 0.01
            it = [0]

            graphs = {}
            out_buf = torch.empty(B, a.dim, device=dev)
            if a.lookahead > 0:
                # the sampler runs `lookahead` batches ahead of the trainer (fresh ids every step, as in training)
                L = a.lookahead
                nsteps = a.iters + 5 + 2 * L + 2
                stream_ids = [zipf_ids_torch(B, a.rows, alpha, generator=g, device=dev) for _ in range(nsteps)]
                base = getattr(tab, "_bench_step", 0)
                for t in range(L):
                    tab.prefetch(stream_ids[t], base + t)
                it[0] = 0
                st0 = dict(tab.stats)

                def step():
                    t = it[0]
                    it[0] += 1
                    tab.prefetch(stream_ids[t + L], base + t + L)
                    tab.lookup(stream_ids[t], base + t, out=out_buf)
                    tab.update(grads)
                ms = _time(step, a.iters, warmup=5)
                # announced but unused batches are consumed so that the next configuration starts clean
                for t in range(it[0], it[0] + L):
                    tab.lookup(stream_ids[t], base + t, out=out_buf)
                tab._bench_step = base + it[0] + L
                tab.check()
                d = {k: tab.stats[k] - st0[k] for k in st0}
                nst = it[0] + L
                uniq = float(torch.stack([torch.unique(p).numel() * torch.ones((), device=dev) for p in stream_ids[:8]]).mean().item())
                rec = {"alpha": alpha, "batch_per_gpu": B, "ms": round(ms, 4), "mkeys_per_s_per_gpu": round(B / ms / 1e3, 2),
                       "unique_fraction": round(uniq / B, 4), "mode": f"lookahead cache hbm_ratio={a.hbm_ratio} L={L}",
                       "hit_ratio_unique": round(1.0 - d["staged_rows"] / max(uniq * nst, 1.0), 4),
                       "staged_mb_per_step": round(d["staged_bytes"] / nst / 1e6, 3),
                       "written_back_rows_per_step": round(d["written_back_rows"] / nst, 1), "late_announcements": d["late_announcements"],
                       "rows": a.rows, "host_table_gb": round(a.rows * (a.dim + 4) * 4 / 1e9, 1)}
                if rank == 0:
                    print(json.dumps(rec), flush=True)
                continue

            def step():
                ids = pool[it[0] & 3]
                it[0] += 1
                if a.graph and a.impl == "native" and (a.sharded or world > 1):
                    k = (it[0] - 1) & 3
                    if k not in graphs:                  # one graph per resident id batch, captured on first use
                        s_ = torch.cuda.Stream()
                        s_.wait_stream(torch.cuda.current_stream())
                        with torch.cuda.stream(s_):
                            gr = torch.cuda.CUDAGraph()
                            with torch.cuda.graph(gr, stream=s_, capture_error_mode="relaxed"):
                                tab.lookup(ids, out=out_buf)
                                tab.update(grads)
                        torch.cuda.current_stream().wait_stream(s_)
                        graphs[k] = gr
                    graphs[k].replay()
                    return
                tab.lookup(ids)
                if a.prefetch and hasattr(tab, "prefetch"):
                    tab.prefetch(pool[it[0] & 3])        # next step's rows are staged while this step updates
                tab.update(grads)
            if hasattr(tab, "hit_stats"):
                tab.hit_stats()
            ms = _time(step, a.iters, warmup=5)
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
                            "nvlink_fraction_of_770gbs": round(2 * tab.nvlink_bytes_per_lookup(int(remote)) / ms / 1e6 / 770.0, 3),
                            "mode": f"sharded x{world}" + (f" tiered hbm_ratio={a.hbm_ratio}" if a.sharded_tiered else "")})
            elif a.sharded:
                rec["mode"] = "sharded x1"
            if a.sharded or world > 1:
                rec.update({"impl": a.impl, "graph": bool(a.graph), "fused": not a.legacy, "hashed": bool(a.hashed)})
                if a.impl == "native":
                    rec["launches_per_lookup_update"] = tab.launches
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
