"""Recommendation-model step on the cached-embedding path: ids from a click-log dataset, embeddings through
``CacheEmbFactory``, sum pooling over the features, a small MLP, MSE against random labels, SGD.

Flags follow the reference's ``perf_rec_model.py`` (src/executable/dlrm/perf_rec_model.py:86-131): ``--num_workers
--emb_dim --L --batch_size --cache_ratio --log_interval --run_steps --emb_choice --backwardMode --backgrad_init
--kForwardItersPerStep --nr_background_threads --dataset criteo|avazu|criteoTB --with_nn "512,256,1"``, plus
``--device``, ``--data_root`` and ``--diff_test`` (compare every step's pooled embeddings with a replicated
``nn.Embedding``; the reference's DIFF_TEST switch, :452-466).

    python -m recstore_b200.cli.perf_rec_model --num_workers 2 --device cpu --run_steps 30 --dataset avazu --diff_test
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import time


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--num_workers", type=int, default=2)
    p.add_argument("--emb_dim", type=int, default=32)
    p.add_argument("--L", type=int, default=10)
    p.add_argument("--with_perf", action="store_true")
    p.add_argument("--profile_dir", default=None,
                   help="record three steps (after three warm-up steps) with torch.profiler: trace_rank{r}.json + ops_rank{r}.txt")
    p.add_argument("--batch_size", type=int, default=1024)
    p.add_argument("--cache_ratio", type=float, default=0.1)
    p.add_argument("--log_interval", type=int, default=50)
    p.add_argument("--run_steps", type=int, default=200)
    p.add_argument("--emb_choice", default="KnownLocalCachedEmbedding")
    p.add_argument("--backwardMode", choices=["CppSync", "CppAsync", "CppAsyncV2", "PySync"], default="CppAsyncV2")
    p.add_argument("--backgrad_init", choices=["cpu", "gpu", "both"], default="both")
    p.add_argument("--kForwardItersPerStep", type=int, default=1)
    p.add_argument("--nr_background_threads", type=int, default=4)
    p.add_argument("--dataset", choices=["criteo", "avazu", "criteoTB"], default="criteo")
    p.add_argument("--with_nn", type=str, default="512,256,1", help="MLP widths after the pooled embedding ('' = no MLP)")
    p.add_argument("--data_root", default=None, help="directory with <dataset>.npy / <dataset>_offsets.npy (else synthetic)")
    p.add_argument("--num_embs", type=int, default=200_000, help="total rows of the synthetic stream")
    p.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    p.add_argument("--clr", type=float, default=0.05)
    p.add_argument("--nn_lr", type=float, default=0.01)
    p.add_argument("--diff_test", action="store_true")
    p.add_argument("--max_seconds", type=float, default=90.0)
    return p.parse_args(argv)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def build_mlp(widths, in_dim):
    """``SimpleDLRM`` of the reference (:53-83): Linear+ReLU stack ending in a linear output."""
    import torch.nn as nn
    layers, d = [], in_dim
    for i, w in enumerate(widths):
        layers.append(nn.Linear(d, w))
        if i < len(widths) - 1:
            layers.append(nn.ReLU())
        d = w
    return nn.Sequential(*layers)


def routine(rank: int, args, port: int, ns: str, out=None):
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    if args.device == "cuda":
        torch.cuda.set_device(rank)
    dist.init_process_group("nccl" if args.device == "cuda" else "gloo", rank=rank, world_size=args.num_workers)
    import recstore_b200 as rs
    from recstore_b200 import ipc
    from recstore_b200.cache import CacheEmbFactory
    from recstore_b200.controller import KGCacheControllerWrapperBase
    from recstore_b200.utils import comm
    from recstore_b200.utils.rec_dataset import RecDatasetLoader
    from recstore_b200.utils.timer import Reporter, Timer
    ipc.set_namespace(ns)
    if rank == 0:
        KGCacheControllerWrapperBase.BeforeDDPInit()
    dist.barrier()
    rs.kvinit()
    dev = torch.device(f"cuda:{rank}") if args.device == "cuda" else torch.device("cpu")
    loader = RecDatasetLoader(args.dataset, args.batch_size, root=args.data_root, rank=rank, world=args.num_workers,
                              synthetic_total=args.num_embs, seed=3)
    N, D, F = loader.num_embeddings, args.emb_dim, loader.F

    def init(t, shape, dtype):
        t.copy_(((torch.arange(shape[0], dtype=dtype) % 997) - 498).unsqueeze(1).expand(shape) * 1e-3)
    if rank == 0:
        emb = rs.DistEmbedding(N, D, name="full_emb", init_func=init)
    dist.barrier()
    if rank != 0:
        emb = rs.DistEmbedding(N, D, name="full_emb", init_func=init)
    cfg = json.dumps({"num_gpus": args.num_workers, "L": args.L, "clr": args.clr, "dim": D, "backwardMode": args.backwardMode,
                      "nr_background_threads": args.nr_background_threads, "full_emb_capacity": N, "cache_ratio": args.cache_ratio,
                      "kForwardItersPerStep": args.kForwardItersPerStep})
    ctrl = KGCacheControllerWrapperBase.FactoryNew("RecStore", cfg, rank, args.num_workers)
    ctrl.init(emb.get_shm_tensor() if rank == 0 else None)
    abs_emb = CacheEmbFactory.New(args.emb_choice, emb, {"cache_ratio": args.cache_ratio, "backwardMode": args.backwardMode,
                                                           "clr": args.clr, "controller": ctrl,
                                                           "kForwardItersPerStep": args.kForwardItersPerStep,
                                                           "backgrad_init": args.backgrad_init}, device=dev)
    golden = gopt = None
    if args.diff_test:
        golden = CacheEmbFactory.New("TorchNativeStdEmbDDP", emb, device=dev)
        gopt = torch.optim.SGD(golden.std_emb.parameters(), lr=args.clr)
    widths = [int(x) for x in args.with_nn.split(",") if x.strip()]
    torch.manual_seed(11)
    mlp = opt = None
    if widths:
        mlp = DDP(build_mlp(widths, D).to(dev), device_ids=[rank] if args.device == "cuda" else None)
        opt = torch.optim.SGD(mlp.parameters(), lr=args.nn_lr)
    gmlp = gopt_nn = None
    if golden is not None and widths:
        torch.manual_seed(11)
        gmlp = build_mlp(widths, D).to(dev)
        gmlp.load_state_dict(mlp.module.state_dict())
        gmlp = DDP(gmlp, device_ids=[rank] if args.device == "cuda" else None)
        gopt_nn = torch.optim.SGD(gmlp.parameters(), lr=args.nn_lr)
    label_gen = torch.Generator().manual_seed(100 + rank)

    def publish(step, ids):
        allids = comm.gather_variable_shape_tensor(ids, 0)
        if rank == 0 and ctrl.controller is not None:
            for r, t in enumerate(allids):
                ctrl.controller.PublishReads(r, step, t)
    future = [loader.next_batch() for _ in range(args.L)]
    for s, b in enumerate(future):
        publish(s, b.reshape(-1))
    t_step = Timer("OneStep")
    from recstore_b200.utils.profiling import StepProfiler
    prof = StepProfiler(args.profile_dir, rank)
    t0 = time.time()
    worst = 0.0
    last_loss = float("nan")
    steps_done = 0
    for step in range(args.run_steps):
        with t_step:
            nxt = loader.next_batch()
            publish(step + args.L, nxt.reshape(-1))
            future.append(nxt)
            ids = future.pop(0).to(dev)                                   # [B, F] global ids
            B = ids.shape[0]
            labels = torch.rand(B, widths[-1] if widths else D, generator=label_gen).to(dev)
            for _ in range(args.kForwardItersPerStep):
                rows = abs_emb.forward(ids.reshape(-1))                   # [B * F, D]
                pooled = rows.view(B, F, D).sum(1)
                pred = mlp(pooled) if mlp is not None else pooled
                loss = torch.nn.functional.mse_loss(pred, labels)
                if opt is not None:
                    opt.zero_grad()
                loss.backward()
                if opt is not None:
                    opt.step()
                last_loss = loss.item()
                if golden is not None:
                    gr = golden.forward(ids.reshape(-1))
                    gp = gr.view(B, F, D).sum(1)
                    worst = max(worst, (pooled.detach() - gp.detach()).abs().max().item())
                    gpred = gmlp(gp) if gmlp is not None else gp
                    gopt.zero_grad()
                    if gopt_nn is not None:
                        gopt_nn.zero_grad()
                    torch.nn.functional.mse_loss(gpred, labels).backward()
                    gopt.step()
                    if gopt_nn is not None:
                        gopt_nn.step()
            abs_emb.after_backward()
        prof.step()
        steps_done += 1
        if rank == 0 and (step + 1) % args.log_interval == 0:
            el = time.time() - t0
            print(f"step {step + 1}: loss {last_loss:.5f}, {el / (step + 1) * 1e3:.2f} ms/step, "
                  f"{args.batch_size * args.num_workers * (step + 1) / el:.0f} samples/s", flush=True)
        stop = torch.tensor([1 if time.time() - t0 > args.max_seconds else 0])
        if args.device == "cuda":
            stop = stop.to(dev)
        dist.all_reduce(stop)
        if int(stop.item()) > 0:
            break
    prof.finish()
    ctrl.GraceFullyStopThreads()
    dist.barrier()
    if rank == 0:
        if args.with_perf:
            print(Reporter.Report())
        if args.diff_test:
            print(f"diff_test: worst |pooled - golden| = {worst:.3e}")
        print("Successfully xmh", flush=True)
    if out is not None:
        out[rank] = (steps_done, worst, last_loss)
    dist.barrier()                       # nobody opens a shared object by name after this point
    if rank == 0:
        ipc.IPCTensorFactory.ClearIPCMemory()        # the run's shared-memory objects do not outlive it
    dist.destroy_process_group()


def main(argv=None):
    args = parse_args(argv)
    import torch.multiprocessing as mp
    port, ns = _free_port(), f"perf_rec_{os.getpid()}"
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(routine, args=(args, port, ns, out), nprocs=args.num_workers, join=True)
    return dict(out)


if __name__ == "__main__":
    main()
