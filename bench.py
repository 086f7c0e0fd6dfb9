#!/usr/bin/env python
"""Headline benchmark: DLRM (dot interaction) training throughput, samples/s.

Config (fixed; the one the baseline names): 26 fp32 embedding tables x dim 128, row counts
log-uniform in [10, 10M] from the seed, rescaled to ~34M rows in total; one id per table per
sample, Zipf(alpha=1.2); 13 dense features log(1+Exp(1)); labels Bernoulli(0.25); bottom MLP
13-512-256-128, top MLP 479-1024-1024-512-256-1, bf16 MLPs; GLOBAL batch 65,536 at every N
(strong scaling); row-wise Adagrad on the embeddings, SGD on the MLPs; table-wise
model-parallel embeddings + data-parallel MLPs.  Synthetic data, random-init weights.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events around exactly K steps,
max over ranks) with the inputs already staged on the device; ``e2e`` is the same metric through
the public API (``DLRM.submit``), including every step's pinned-host -> device input copies and
the device -> host read of the loss.  ``--impl torch_baseline`` runs the PyTorch+NCCL+cuBLAS
restatement of the reference algorithm on the same data; ``--impl reference`` runs the
unmodified reference when it is installed under baseline/_ref.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

TABLES, DIM, BATCH, ALPHA = 26, 128, 65536, 1.2
METRIC = "dlrm_train_samples_per_s"


def table_rows(seed: int = 0):
    from recstore_b200.utils.data import loguniform_table_rows
    return loguniform_table_rows(TABLES, 10, 10_000_000, 34_000_000, seed)


# Second workload (not the headline): DLRM-DCNv2, multi-hot, ~200 M rows, largest table 40 M rows, low-rank (512) cross
# network of 3 layers, top MLP 1024-1024-512-256-1, ids Zipf(1.1); tables are placed table-wise on the GPUs.
DCN_HOTNESS = [3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1]


def dcn_table_rows(seed: int = 0):
    """Row counts drawn as for the headline config, then handed out so that tables with more ids per sample are the
    larger ones (as in click logs: the long multi-hot features are the high-cardinality ones).  With U(+-sqrt(1/n))
    rows, a 100-hot sum over a 75-row table would start at magnitude ~10 and the cubic cross network overflows bf16."""
    from recstore_b200.utils.data import loguniform_table_rows
    rows = sorted(loguniform_table_rows(TABLES, 10, 40_000_000, 200_000_000, seed, pin_largest=40_000_000), reverse=True)
    order = sorted(range(TABLES), key=lambda t: -DCN_HOTNESS[t])
    out = [0] * TABLES
    for k, t in enumerate(order):
        out[t] = rows[k]
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.p = None
        self.idx = gpu_index

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                      stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out, _ = self.p.communicate()
        sm, mx, reasons, pw = [], [], set(), []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load = upper half by power draw
        thr = statistics.median(pw)
        load = [s for s, p in zip(sm, pw) if p >= thr] or sm
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(pw)}


def dist_setup(n):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n}")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def run_native(args):
    from recstore_b200.models.dlrm import DLRM, DLRMConfig
    from recstore_b200.parallel.peer import PeerContext
    from recstore_b200.utils.data import DLRMBatchSource
    rank, world, local = dist_setup(args.gpus)
    dcn = args.workload == "dcnv2"
    B = args.batch
    rows = dcn_table_rows(args.seed) if dcn else table_rows(args.seed)
    hot = DCN_HOTNESS if dcn else [1] * TABLES
    ctx = PeerContext(rank, world, device=torch.device(f"cuda:{local}"))
    # dcnv2: the heavy multi-hot tables are spread row-wise over the ranks (--row-split none keeps every table whole on
    # one rank), the others are placed by a greedy on their ids per sample.
    extra = dict(interaction="dcn", dcn_layers=3, dcn_rank=512, hotness=hot, top_mlp=(1024, 1024, 512, 256, 1),
                 row_split=(None if args.row_split == "none" else "auto" if args.row_split == "auto" else
                            [int(t) for t in args.row_split.split(",")]), placement="balanced") if dcn else {}
    # dcnv2: with sum-of-squares row-wise Adagrad a row that occurs n times in a batch moves by ~lr * sqrt(n); the
    # 100-hot Zipf feature repeats its hottest rows ~10^5 times per batch, so the embedding step is kept small.
    cfg = DLRMConfig(table_rows=rows, batch=B, emb_dim=DIM, emb_lr=0.01 if not dcn else 1e-4, mlp_lr=0.01 if not dcn else 0.001, seed=args.seed,
                     use_cuda_graph=not args.no_graph, trace_phases=args.trace_phases, pipeline_lookup=bool(args.pipeline),
                     **extra)
    eng = DLRM(cfg, ctx)
    src = DLRMBatchSource(rows, hot, B, alpha=1.1 if dcn else ALPHA, seed=args.seed + 1)
    nb = 4
    batches = []
    for _ in range(nb):
        b = src.next()
        batches.append(eng.make_pinned_batch(b.dense, b.ids, b.labels))
    # ---- warm-up through the public API (also captures the CUDA graphs)
    last = None
    for i in range(max(args.warmup, 3)):
        last = eng.train_step(batches[i % nb])
    eng.check()
    # ---- device-timed region: exactly K steps, inputs resident on the device
    # The K-step region is timed `repeats` times (each bracketed by barrier + synchronize, max over ranks); the median
    # is the value, the spread is reported beside it.
    sampler = ClockSampler(local)
    barrier(world)
    if rank == 0:
        sampler.start()
    samples = []
    for _ in range(max(1, args.repeats)):
        barrier(world)
        samples.append(max_over_ranks(eng.time_steps_on_device(args.steps), world))
    barrier(world)
    clocks = sampler.stop() if rank == 0 else None
    ms_dev = statistics.median(samples)
    # ---- end to end: pinned host -> device copies and the loss read back, every step
    barrier(world)
    t0 = time.perf_counter()
    prev = None
    for i in range(args.steps):
        h = eng.submit(batches[i % nb])
        if prev is not None:
            last = prev.result()
        prev = h
    last = prev.result()
    torch.cuda.synchronize()
    ms_e2e = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    eng.check()
    if args.trace_phases:   # per-rank phase timeline of the last step (stamps cost one tiny launch each)
        ph = eng.phase_times()
        allph = [ph]
        if world > 1:
            import torch.distributed as dist
            allph = [None] * world
            dist.all_gather_object(allph, ph)
        if rank == 0:
            for k in ph:
                print(f"[phases] {k:42s} " + " ".join(f"{p[k]:8.1f}" for p in allph) + "  us per rank", file=sys.stderr)
    h2d = batches[0].nbytes
    if rank == 0:
        out = {
            "metric": METRIC if not dcn else "dlrm_dcnv2_train_samples_per_s", "value": B * args.steps / (ms_dev * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": f"synthetic (Zipf {1.1 if dcn else 1.2} ids, random-init weights)", "impl": "native",
            "config": {"model": "DLRM dot, 26 tables x dim 128, ~34M rows, bot 13-512-256-128, top 479-1024-1024-512-256-1" if not dcn else
                       "DLRM-DCNv2 multi-hot (sum of hotness 214), 26 tables x dim 128, ~200M rows (largest 40M), bot 13-512-256-128, "
                       "3-layer rank-512 cross network, top 3456-1024-1024-512-256-1",
                       "global_batch": B, "seq_len": None,
                       "parallelism": (f"table-wise MP embeddings x{world} + DP MLP x{world}" if not eng.K else
                                       f"row-wise sharded tables {eng.split_tables} + table-wise MP for the rest x{world} + DP MLP x{world}"),
                       "l2": "working set per step (>=450 MB of windows + ~17 GB of tables) exceeds the 126 MB L2",
                       "optimizer": "row-wise Adagrad (embeddings) + SGD (MLP)", "total_rows": sum(rows),
                       "pipeline_lookup": bool(eng._pipe)},
            "clocks": clocks,
            "e2e": {"value": B * args.steps / (ms_e2e * 1e-3), "unit": "samples/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "timed_regions": {"repeats": len(samples), "ms_per_step_min": min(samples) / args.steps,
                              "ms_per_step_max": max(samples) / args.steps, "value_is": "median"},
            "gpu_launches": eng.launches_per_step * args.steps,
            "launches_per_step": eng.launches_per_step,
            "last_loss_rank0": last,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_kge(args):
    """Knowledge-graph embedding training at the shape of the fourth benchmark config: 86 M entities x dim 400 fp32 (138 GB)
    spread over the GPUs' HBM, 14,824 relations, 1,024 positives per GPU with 256 chunk-shared uniform negatives, log-sigmoid
    loss, gamma 10, sparse row-wise Adagrad lr 0.1; synthetic triples (head / tail power law alpha 1.3, relations uniform)
    drawn on the device.  Weak scaling: the per-GPU batch is fixed.  --kge-entities scales the table down for small runs."""
    from recstore_b200.models.kge import KGEConfig, KGEModel
    from recstore_b200.parallel.peer import PeerContext
    from recstore_b200.utils.data import device_uniform_ids, device_zipf_ids
    rank, world, local = dist_setup(args.gpus)
    dev = torch.device(f"cuda:{local}")
    ctx = PeerContext(rank, world, device=dev)
    NE, NR, D, bs, ns = args.kge_entities, 14824, 400, 1024, 256
    cfg = KGEConfig(NE, NR, dim=D, model=args.kge_model, gamma=10.0, batch=bs, neg_sample_size=ns, neg_chunk_size=ns, lr=0.1,
                    seed=args.seed, use_cuda_graph=(not args.no_graph) and args.kge_model != "TransR",   # TransR scores through autograd
                    tf32_scoring=args.kge_model == "TransR")
    model = KGEModel(cfg, ctx)
    nneg = bs // ns * ns
    nb = 8

    def draw(k):   # one step's ids, on the device, from counter-based streams
        c = (k * world + rank) * 4 * bs
        return (device_zipf_ids(bs, NE, 1.3, args.seed + 11, c, device=dev, spread=True),
                device_uniform_ids(bs, NR, args.seed + 12, c, device=dev),
                device_zipf_ids(bs, NE, 1.3, args.seed + 13, c, device=dev, spread=True),
                device_uniform_ids(nneg, NE, args.seed + 14, c, device=dev))
    dev_batches = [draw(k) for k in range(nb)]
    host_batches = [tuple(t.cpu().pin_memory() for t in b) for b in dev_batches]
    for i in range(max(args.warmup, 3) + 2):          # both corruption sides get captured
        loss = model.train_step(*dev_batches[i % nb])
    ctx.check_status()
    sampler = ClockSampler(local)
    barrier(world)
    if rank == 0:
        sampler.start()
    samples = []
    for _ in range(max(1, args.repeats)):
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            loss = model.train_step(*dev_batches[i % nb])
        e1.record()
        e1.synchronize()
        samples.append(max_over_ranks(e0.elapsed_time(e1), world))
    barrier(world)
    clocks = sampler.stop() if rank == 0 else None
    ms_dev = statistics.median(samples)
    # end to end: ids from pinned host memory every step, loss read back every step
    bufs = [tuple(torch.empty_like(t, device=dev) for t in host_batches[0]) for _ in range(2)]
    barrier(world)
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        hb, db = host_batches[i % nb], bufs[i & 1]
        for d, h in zip(db, hb):
            d.copy_(h, non_blocking=True)
        last = model.train_step(*db).item()
    torch.cuda.synchronize()
    ms_e2e = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    ctx.check_status()
    if rank == 0:
        h2d = sum(t.numel() * 8 for t in host_batches[0])
        out = {
            "metric": "kge_train_triples_per_s", "value": bs * world * args.steps / (ms_dev * 1e-3), "unit": "triples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": ("fp32 tables, tf32 batched score GEMMs (cuBLAS, autograd)" if args.kge_model == "TransR" else
                      "fp32 tables, fp32 pair kernels" if args.kge_model in ("TransE_l1", "RotatE") else "fp32 tables, bf16 score GEMMs"),
            "impl": "native",
            "data": "synthetic (power-law alpha 1.3 head / tail entities, uniform relations and negatives, drawn on the device)",
            "config": {"model": f"{args.kge_model}, {NE} entities x dim {D} fp32 ({NE * D * 4 / 1e9:.0f} GB) sharded over {world} GPU(s), {NR} relations",
                       "global_batch": bs * world, "negatives": f"{ns} chunk-shared uniform per {ns} positives", "gamma": 10.0,
                       "optimizer": "sparse row-wise Adagrad lr 0.1", "parallelism": f"row-sharded entity / relation tables x{world}",
                       "l2": "the entity shard (17-138 GB) exceeds the 126 MB L2; ids differ every step"},
            "clocks": clocks,
            "e2e": {"value": bs * world * args.steps / (ms_e2e * 1e-3), "unit": "triples/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "timed_regions": {"repeats": len(samples), "ms_per_step_min": min(samples) / args.steps,
                              "ms_per_step_max": max(samples) / args.steps, "value_is": "median"},
            "gpu_launches": model.launches_per_step * args.steps, "launches_per_step": model.launches_per_step, "last_loss_rank0": last,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_kge_torch(args):
    """The KG workload on the PyTorch path (`baseline/kge_torch.py`: dense tables on one device, autograd scoring with
    the bmm-style chunked negatives, sparse row-wise Adagrad through index_add_), same ids and shapes as `run_kge`.
    One GPU; --kge-entities sizes the table (the PyTorch path builds it on the host first)."""
    from recstore_b200.baseline.kge_torch import TorchKGE
    from recstore_b200.utils.data import device_uniform_ids, device_zipf_ids
    rank, world, local = dist_setup(args.gpus)
    assert world == 1, "the PyTorch KG arm is single-GPU"
    dev = torch.device(f"cuda:{local}")
    NE, NR, D, bs, ns = args.kge_entities, 14824, 400, 1024, 256
    m = TorchKGE(NE, NR, D, args.kge_model, gamma=10.0, lr=0.1, device=dev, seed=args.seed)
    nneg, nb = bs // ns * ns, 8

    def draw(k):
        c = k * 4 * bs
        return (device_zipf_ids(bs, NE, 1.3, args.seed + 11, c, device=dev, spread=True),
                device_uniform_ids(bs, NR, args.seed + 12, c, device=dev),
                device_zipf_ids(bs, NE, 1.3, args.seed + 13, c, device=dev, spread=True),
                device_uniform_ids(nneg, NE, args.seed + 14, c, device=dev))
    dev_batches = [draw(k) for k in range(nb)]
    host_batches = [tuple(t.cpu().pin_memory() for t in b) for b in dev_batches]
    for i in range(max(args.warmup, 3)):
        m.train_step(*dev_batches[i % nb], ns)
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(args.steps):
        m.train_step(*dev_batches[i % nb], ns)
    e1.record()
    e1.synchronize()
    clocks = sampler.stop()
    ms_dev = e0.elapsed_time(e1)
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        last = m.train_step(*(t.to(dev, non_blocking=True) for t in host_batches[i % nb]), ns)
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) * 1e3
    h2d = sum(t.numel() * t.element_size() for t in host_batches[0])
    print(json.dumps({
        "metric": "kge_train_triples_per_s", "value": bs * args.steps / (ms_dev * 1e-3), "unit": "triples/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "impl": "torch_baseline",
        "data": "synthetic (same device-drawn ids as the native arm)",
        "config": {"model": f"{args.kge_model}, {NE} entities x dim {D} fp32 on one GPU (PyTorch tables, autograd scoring)",
                   "global_batch": bs, "negatives": f"{ns} chunk-shared uniform per {ns} positives", "gamma": 10.0,
                   "optimizer": "sparse row-wise Adagrad lr 0.1 (index_add_)"},
        "clocks": clocks,
        "e2e": {"value": bs * args.steps / (ms_e2e * 1e-3), "unit": "triples/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": 0, "last_loss": last}), flush=True)


def run_torch_baseline(args):
    """PyTorch + NCCL + cuBLAS restatement of the reference algorithm on the same data."""
    from recstore_b200.baseline.dlrm_torch import TorchDLRM
    from recstore_b200.utils.data import DLRMBatchSource
    rank, world, local = dist_setup(args.gpus)
    dcn = args.workload == "dcnv2"
    rows = dcn_table_rows(args.seed) if dcn else table_rows(args.seed)
    hot = DCN_HOTNESS if dcn else [1] * TABLES
    dev = torch.device(f"cuda:{local}")
    extra = dict(interaction="dcn", dcn_layers=3, dcn_rank=512, hotness=hot, top_mlp=(1024, 1024, 512, 256, 1), emb_lr=1e-4,
                 mlp_lr=0.001) if dcn else {}
    m = TorchDLRM(rows, BATCH, emb_dim=DIM, device=dev, rank=rank, world=world, autocast_bf16=True, seed=args.seed, **extra)
    src = DLRMBatchSource(rows, hot, BATCH, alpha=1.1 if dcn else ALPHA, seed=args.seed + 1)
    nb = 4
    host = []
    for _ in range(nb):
        b = src.next()
        host.append((b.dense.pin_memory(), [i.pin_memory() for i in b.ids], b.labels.pin_memory()))
    devb = [(d.to(dev), [i.to(dev) for i in ids], l.to(dev)) for d, ids, l in host]
    for i in range(max(args.warmup, 3)):
        m.train_step(*devb[i % nb])
    sampler = ClockSampler(local)
    barrier(world)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        m.train_step(*devb[i % nb])
    e1.record()
    barrier(world)
    clocks = sampler.stop() if rank == 0 else None
    ms_dev = max_over_ranks(e0.elapsed_time(e1), world)
    barrier(world)
    t0 = time.perf_counter()
    for i in range(args.steps):
        d, ids, l = host[i % nb]
        loss = m.train_step(d.to(dev, non_blocking=True), [x.to(dev, non_blocking=True) for x in ids],
                            l.to(dev, non_blocking=True))
        last = loss.item()
    torch.cuda.synchronize()
    ms_e2e = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    if rank == 0:
        print(json.dumps({
            "metric": "dlrm_dcnv2_train_samples_per_s" if dcn else METRIC, "value": BATCH * args.steps / (ms_dev * 1e-3),
            "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "torch_baseline", "config": {"model": ("DLRM-DCNv2 multi-hot" if dcn else "DLRM dot") +
                                                          " (PyTorch+NCCL+cuBLAS restatement of the reference algorithm)",
                                                 "global_batch": BATCH, "parallelism": f"table-wise MP x{world} + DP"},
            "clocks": clocks,
            "e2e": {"value": BATCH * args.steps / (ms_e2e * 1e-3), "unit": "samples/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in [host[0][0], host[0][2]] + host[0][1]),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "last_loss": last}), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    try:
        from recstore_b200.baseline import reference_arm
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"reference arm not importable: {e}"}))
        return
    reference_arm.main(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "torch_baseline"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true", help="launch kernels eagerly instead of replaying a CUDA graph")
    ap.add_argument("--workload", default="dlrm", choices=["dlrm", "dcnv2", "kge"],
                    help="dlrm: the headline config; dcnv2: the multi-hot DLRM-DCNv2 config; kge: knowledge-graph embedding training "
                         "(native arm only for the last two)")
    ap.add_argument("--kge-model", default="TransE_l2", choices=["TransE_l2", "DistMult", "ComplEx", "SimplE", "TransE_l1", "RotatE", "RESCAL", "TransR"])
    ap.add_argument("--kge-entities", type=int, default=86_054_151, help="entities of the kge workload (the config's Freebase count)")
    ap.add_argument("--row-split", default="auto",
                    help="dcnv2 workload: tables spread row-wise over the GPUs: auto (those with more than 1/N of the ids per sample), "
                         "none (every table whole on one GPU) or a comma-separated list of table indices")
    ap.add_argument("--pipeline", type=int, choices=[0, 1], default=int(os.environ.get("RECSTORE_PIPELINE_LOOKUP", "0")),
                    help="dlrm workload: 1 = the lookup + forward all-to-all of batch t + 1 runs at the end of step t's graph")
    ap.add_argument("--repeats", type=int, default=5, help="how many times the K-step timed region is measured (median reported)")
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="global batch; the headline config is 65,536 (other values are for profiling, e.g. 8,192 on one GPU "
                         "has the per-GPU dense shapes of the 8-GPU run)")
    ap.add_argument("--trace-phases", action="store_true",
                    help="stamp the GPU timer at phase boundaries of the step and print the timeline of every rank to stderr")
    args = ap.parse_args()
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "torch_baseline" and args.workload == "kge":
        run_kge_torch(args)
    elif args.impl == "torch_baseline":
        run_torch_baseline(args)
    elif args.workload == "kge":
        run_kge(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
