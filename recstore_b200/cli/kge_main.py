"""Knowledge-graph embedding training driver (the counterpart of the reference's ``dgl-ke-main.py``).

    python -m recstore_b200.cli.kge_main --model_name TransE_l2 --dataset synthetic --n_entities 100000 --n_triples 2000000 \
        --hidden_dim 400 --gamma 10 --batch_size 1024 --neg_sample_size 256 --max_step 1000 --num_proc 2 --device cuda --test

Pipeline (src/executable/kg/dgl-ke-main.py:168-552): load or synthesise the dataset -> partition the training triples
over the workers (``--rel_part`` balanced, ``--soft_rel_part``, ``--graph_part`` edge-cut, else random) -> per-worker chunked negative samplers ->
optional pre-sampling of ``--presample_steps`` steps, hot sets of ``--cache_ratio`` x entities per worker, renumbering so
that each worker's hot entities are contiguous -> one training process per worker -> save -> sampled-negative test
(MRR / MR / HITS@k).

Engines: on ``--device cuda`` TransE (L1 / L2), DistMult, ComplEx, SimplE and RotatE run on the native path (entity and
relation tables row-sharded over the GPUs' HBM; tcgen05 scoring where the negative scores are cross products, fp32 pair
kernels for the L1 / modulus distances; RESCAL with a row-blocked matrix table; TransR with the same tables and its
scoring as autograd over batched cuBLAS GEMMs); ``--device cpu`` runs the PyTorch implementation on
tables shared between the worker processes (lock-free updates, as the reference's stock path does).  Prints
``Successfully xmh`` when done.

The command line mirrors the reference's (utils.py:199-304, dgl-ke-main.py:84-152).  Loss options (``--loss_genre``,
``-adv``, ``-rc``), degree-based negatives and edge importance run on the PyTorch tables; ``--mix_cpu_gpu`` keeps only the
``--cache_ratio`` share of every entity shard in HBM and the rest in pinned host memory that the kernels address in
place; ``--gpu`` / ``--nr_gpus`` select the CUDA path with one worker per GPU; ``--valid --eval_interval N`` scores the
validation split during training; ``--force_sync_interval N`` puts a barrier between the workers every N steps.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import time

import numpy as np
import torch

NATIVE_MODELS = ("TransE", "TransE_l1", "TransE_l2", "DistMult", "ComplEx", "SimplE", "RotatE", "RESCAL", "TransR")


def parse_args(argv=None):
    from recstore_b200.baseline.kge_torch import MODEL_NAMES
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--model_name", default="TransE_l2", choices=MODEL_NAMES)
    p.add_argument("--dataset", default="synthetic")
    p.add_argument("--data_path", default=None)
    p.add_argument("--data_files", nargs="+", default=None)
    p.add_argument("--format", default="raw_udd_hrt")
    p.add_argument("--n_entities", type=int, default=20000)
    p.add_argument("--n_relations", type=int, default=50)
    p.add_argument("--n_triples", type=int, default=200000)
    p.add_argument("--hidden_dim", type=int, default=64)
    p.add_argument("--gamma", type=float, default=12.0)
    p.add_argument("--lr", type=float, default=0.1)
    p.add_argument("--batch_size", type=int, default=256)
    p.add_argument("--neg_sample_size", type=int, default=64)
    p.add_argument("--neg_chunk_size", type=int, default=None)
    p.add_argument("--max_step", type=int, default=200)
    p.add_argument("--log_interval", type=int, default=100)
    p.add_argument("--num_proc", type=int, default=1)
    p.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    p.add_argument("--rel_part", action="store_true")
    p.add_argument("--soft_rel_part", action="store_true")
    p.add_argument("--graph_part", action="store_true", help="balanced edge-cut partition of the entity graph (the METIS role)")
    p.add_argument("--cache_ratio", type=float, default=0.0)
    p.add_argument("--presample_steps", type=int, default=0)
    p.add_argument("--test", action="store_true")
    p.add_argument("--batch_size_eval", type=int, default=256)
    p.add_argument("--neg_sample_size_eval", type=int, default=256, help="-1: rank against all entities (filtered unless --no_eval_filter)")
    p.add_argument("--save_path", default=None)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--no_graph", action="store_true", help="native path: launch the step eagerly instead of replaying a CUDA graph")
    # ---- the rest of the reference's surface (utils.py:199-304 CommonArgParser, dgl-ke-main.py:84-152)
    p.add_argument("--delimiter", default="\t", help="field separator of the triple files")
    p.add_argument("--double_ent", action="store_true", help="entity embeddings are 2 x hidden_dim wide (RotatE, ComplEx)")
    p.add_argument("--double_rel", action="store_true", help="relation embeddings are 2 x hidden_dim wide (ComplEx)")
    p.add_argument("--loss_genre", "-lg", default="Logsigmoid", choices=["Hinge", "Logistic", "Logsigmoid", "BCE"])
    p.add_argument("--margin", "-m", type=float, default=1.0, help="margin of the hinge loss")
    p.add_argument("--pairwise", "-pw", action="store_true", help="pairwise loss (closed in the reference: loss.py asserts)")
    p.add_argument("--neg_adversarial_sampling", "-adv", action="store_true")
    p.add_argument("--adversarial_temperature", "-a", type=float, default=1.0)
    p.add_argument("--regularization_coef", "-rc", type=float, default=0.0)
    p.add_argument("--regularization_norm", "-rn", type=int, default=3)
    p.add_argument("--neg_deg_sample", action="store_true", help="draw negatives proportionally to entity degree")
    p.add_argument("--neg_deg_sample_eval", action="store_true", help="PyTorch path: evaluation negatives in proportion to entity degree")
    p.add_argument("--valid", action="store_true", help="evaluate on the validation split every --eval_interval steps")
    p.add_argument("--eval_interval", type=int, default=10000)
    p.add_argument("--eval_percent", type=float, default=1.0, help="share of the evaluation split that is scored")
    p.add_argument("--no_eval_filter", action="store_true", help="full ranking (--neg_sample_size_eval -1) without removing other true triples")
    p.add_argument("--no_save_emb", action="store_true")
    p.add_argument("--num_thread", type=int, default=0, help="host threads per worker (0: share the cores evenly)")
    p.add_argument("--force_sync_interval", type=int, default=-1, help="barrier between the workers every N steps")
    p.add_argument("--shuffle", action="store_true", help="accepted: batches are drawn uniformly at random already")
    p.add_argument("--has_edge_importance", action="store_true", help="a fourth column of the triple files weighs each triple")
    p.add_argument("--gpu", type=int, nargs="+", default=None, help="GPU ids: selects --device cuda and one worker per GPU")
    p.add_argument("--nr_gpus", type=int, default=None)
    p.add_argument("--mix_cpu_gpu", action="store_true", help="keep only the hot share (--cache_ratio) of the entity table in HBM")
    p.add_argument("--async_update", action="store_true", help="PyTorch path: a worker thread applies the entity updates behind the trainer; no effect on the native path (its update is a few kernels inside the step)")
    p.add_argument("--use_my_emb", type=lambda v: str(v).lower() in ("1", "true", "yes"), default=True,
                   help="RecStore embedding path (here: the native sharded tables); false = the PyTorch tables")
    p.add_argument("--cached_emb_type", default="KnownShardedCachedEmbedding")
    p.add_argument("--backwardMode", default="CppAsyncV2", choices=["PySync", "CppSync", "CppAsync", "CppAsyncV2"])
    p.add_argument("--L", type=int, default=10, help="lookahead window of the cached sampler, in steps")
    p.add_argument("--nr_background_threads", type=int, default=4)
    p.add_argument("--update_cache_use_omp", type=int, default=1)
    p.add_argument("--update_pq_use_omp", type=int, default=1)
    p.add_argument("--determinism_dir", default=os.environ.get("RECSTORE_DETERMINISM_DIR"),
                   help="record the sampled batches of the first --determinism_steps steps there; later runs must reproduce them")
    p.add_argument("--determinism_steps", type=int, default=20)
    p.add_argument("--profile_dir", default=None,
                   help="record three steps (after three warm-up steps) with torch.profiler: trace_rank{r}.json + ops_rank{r}.txt")
    p.add_argument("--heartbeat_timeout", type=float, default=0.0,
                   help="seconds without a sign of life after which a worker counts as lost (0: no liveness check); the "
                        "others then stop before their next step instead of waiting inside a collective")
    a = p.parse_args(argv)
    if a.pairwise:
        p.error("--pairwise is closed in the reference (its loss generator asserts) and is not offered here")
    if a.gpu is not None or a.nr_gpus is not None:
        a.device = "cuda"
        a.num_proc = a.nr_gpus if a.nr_gpus is not None else len(a.gpu)
    if a.double_rel and not a.double_ent:
        p.error("--double_rel without --double_ent: entity and relation widths must match for every model but RotatE")
    a.dim = a.hidden_dim * (2 if a.double_ent else 1)          # width of an entity row
    if a.neg_chunk_size is None:
        a.neg_chunk_size = min(a.neg_sample_size, a.batch_size)
    a.batch_size = -(-a.batch_size // a.neg_chunk_size) * a.neg_chunk_size      # whole chunks, like the reference (utils.py:27-33)
    return a


def _native(args) -> bool:
    """The sharded-HBM engine takes the default loss only; every other combination runs on the PyTorch tables."""
    plain = (args.loss_genre == "Logsigmoid" and not args.neg_adversarial_sampling and args.regularization_coef == 0.0
             and not args.neg_deg_sample and not args.has_edge_importance)
    return args.device == "cuda" and args.use_my_emb and plain and args.model_name in NATIVE_MODELS


def _loss_kwargs(args) -> dict:
    return dict(loss_genre=args.loss_genre, margin=args.margin, neg_adversarial_sampling=args.neg_adversarial_sampling,
                adversarial_temperature=args.adversarial_temperature, regularization_coef=args.regularization_coef,
                regularization_norm=args.regularization_norm)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def prepare(args):
    """Dataset -> partitions (-> renumbering).  Returns (dataset, parts, info)."""
    from recstore_b200.utils import kg_data as K
    if args.dataset == "planted_grid":            # a small graph with structure to find: quality is visible on it
        ds = K.KGDataset.planted_grid(seed=args.seed)
    elif args.dataset == "synthetic" or args.data_path is None:
        ds = K.KGDataset.synthetic(args.n_entities, args.n_relations, args.n_triples, seed=args.seed)
    else:
        ds = K.KGDataset.load(args.data_path, args.data_files or ["train.tsv"], args.format, name=args.dataset,
                              delimiter=args.delimiter, has_edge_importance=args.has_edge_importance)
    W = args.num_proc
    info = {"n_entities": ds.n_entities, "n_relations": ds.n_relations, "n_train": int(ds.train[0].size)}
    if args.rel_part:
        parts, cross = K.balanced_relation_partition(ds.train[1], W, args.seed)
        info["cross_relations"] = int(cross.sum())
    elif args.soft_rel_part:
        parts, cross = K.soft_relation_partition(ds.train[1], W, seed=args.seed)
        info["cross_relations"] = int(cross.sum())
    elif args.graph_part:
        parts, node_part, st = K.graph_partition(ds.train[0], ds.train[2], ds.n_entities, W, seed=args.seed)
        info["edge_cut"] = st["edge_cut"]
        if args.device == "cuda" and W > 1:      # the sharded tables place row id on GPU id % W: make that the entity's part
            ds, new_id = K.renumber_by_partition(ds, node_part, W)
            info["entities_on_their_workers_gpu"] = float(np.mean(new_id % W == node_part))
    else:
        parts = K.random_partition(ds.train[0].size, W, args.seed)
    if args.cache_ratio > 0 and args.presample_steps > 0:
        cache = max(1, int(ds.n_entities * args.cache_ratio / W))
        smp = [K.ChunkedNegativeSampler(tuple(x[p] for x in ds.train), ds.n_entities, args.batch_size, args.neg_sample_size,
                                        args.neg_chunk_size, seed=args.seed * 100 + r) for r, p in enumerate(parts)]
        counts = K.presample(smp, ds.n_entities, args.presample_steps)
        hot = K.hot_sets(counts, cache)
        covered = sum(int(c[h].sum()) for c, h in zip(counts, hot)) / max(1, sum(int(c.sum()) for c in counts))
        ds, _ = K.renumber_graph(ds, hot, cache)
        info.update({"cache_rows_per_worker": cache, "presampled_hit_ratio": covered})
    return ds, parts, info


def worker(rank: int, args, ds, parts, port: int, shared, out):
    from recstore_b200.utils.kg_data import ChunkedNegativeSampler
    W = args.num_proc
    dev = torch.device(f"cuda:{rank}") if args.device == "cuda" else torch.device("cpu")
    native = _native(args)
    if args.num_thread > 0:
        torch.set_num_threads(args.num_thread)
    elif args.device == "cpu" and W > 1:
        torch.set_num_threads(max(1, (os.cpu_count() or W) // W))       # the workers share the host's cores
    if W > 1 or native:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
        if args.device == "cuda":
            torch.cuda.set_device(rank)
        dist.init_process_group("nccl" if args.device == "cuda" else "gloo", rank=rank, world_size=W)
    hb = None
    if W > 1 and args.heartbeat_timeout > 0:
        from recstore_b200.utils.liveness import Heartbeat
        hb = Heartbeat(rank, W, name=f"kge_heartbeat_{port}", period_s=min(0.2, args.heartbeat_timeout / 5)).start()
        hb.wait_all_alive(max(60.0, args.heartbeat_timeout))
    mine = tuple(x[parts[rank]] for x in ds.train)
    w_mine = ds.train_weight[parts[rank]] if (args.has_edge_importance and ds.train_weight is not None) else None
    smp = ChunkedNegativeSampler(mine, ds.n_entities, args.batch_size, args.neg_sample_size, args.neg_chunk_size,
                                 seed=args.seed * 100 + rank, device=dev, neg_deg_sample=args.neg_deg_sample, weight=w_mine)
    if native:
        from recstore_b200.models.kge import KGEConfig, KGEModel
        from recstore_b200.parallel.peer import PeerContext
        ctx = PeerContext(rank, W, device=dev)
        hbm = (args.cache_ratio if args.cache_ratio > 0 else 0.25) if args.mix_cpu_gpu else 1.0
        model = KGEModel(KGEConfig(ds.n_entities, ds.n_relations, dim=args.dim, model=args.model_name, gamma=args.gamma,
                                   batch=args.batch_size, neg_sample_size=args.neg_sample_size, neg_chunk_size=args.neg_chunk_size,
                                   lr=args.lr, seed=args.seed, dataset=ds.name, use_cuda_graph=(not args.no_graph) and args.model_name != "TransR",
                                   entity_hbm_ratio=hbm), ctx)
        step_fn = lambda h, r, t, n, ch: model.train_step(h, r, t, n, ch)
    else:
        from recstore_b200.baseline.kge_torch import TorchKGE
        model = TorchKGE(ds.n_entities, ds.n_relations, args.dim, args.model_name, args.gamma, args.lr, device=dev, seed=args.seed,
                         **_loss_kwargs(args))
        if shared is not None:           # one table for all CPU workers
            model.entity, model.relation, model.proj, model.state = shared["entity"], shared["relation"], shared.get("proj"), shared["state"]
        if args.async_update:            # entity updates applied by a worker thread behind the trainer (train_pytorch.py:134-135)
            model.create_async_update()
        step_fn = lambda h, r, t, n, ch: model.train_step(h, r, t, n, args.neg_chunk_size, ch, edge_weight=smp.last_weight)
    def run_eval(split, percent: float = 1.0):
        """Sampled-negative ranking metrics of (a share of) a split; native: every rank scores, else rank 0 only."""
        if not native and args.async_update:
            model.wait_async_update()
        n_eval = max(args.batch_size, int(min(split[0].size, args.batch_size_eval * 4) * percent))
        th, tr, tt = (torch.as_tensor(x[:n_eval]).to(dev) for x in split)
        g = torch.Generator(device=dev if native else "cpu").manual_seed(5)
        if args.neg_sample_size_eval < 0:           # rank against every entity, filtered unless --no_eval_filter
            from recstore_b200.baseline.kge_torch import TorchKGE, known_triple_index
            known = None if args.no_eval_filter else known_triple_index(ds.train, ds.valid, ds.test)
            if native:                               # the sharded tables come to rank 0 (collective), scored there on the host
                ent, rel = model._gather_table(model.entity), model._gather_table(model.relation)
                if rank != 0:
                    return None
                scorer = TorchKGE(2, 2, args.dim, args.model_name, args.gamma, args.lr)
                scorer.entity, scorer.relation = torch.from_numpy(ent), torch.from_numpy(rel)
                return scorer.evaluate_full(th.cpu(), tr.cpu(), tt.cpu(), known)
            return model.evaluate_full(th, tr, tt, known) if rank == 0 else None
        if native:
            ms = []
            for s0 in range(0, th.numel() - args.batch_size + 1, args.batch_size):
                ms.append(model.evaluate(th[s0:s0 + args.batch_size], tr[s0:s0 + args.batch_size], tt[s0:s0 + args.batch_size], g))
            return {k: float(np.mean([m[k] for m in ms])) for k in ms[0]} if ms else None
        if rank == 0:
            prob = None
            if args.neg_deg_sample_eval:                 # corruptions drawn in proportion to 1 + degree in the training graph
                deg = torch.bincount(torch.as_tensor(np.concatenate([ds.train[0], ds.train[2]])), minlength=ds.n_entities).float() + 1.0
                prob = deg / deg.sum()
            return model.evaluate(th, tr, tt, args.neg_sample_size_eval, g, neg_prob=prob)
        return None

    t0 = time.time()
    losses = []
    valid_log = []
    from recstore_b200.utils.determinism import RunRecorder
    recorder = RunRecorder(args.determinism_dir)
    from recstore_b200.utils.profiling import StepProfiler
    prof = StepProfiler(args.profile_dir, rank)
    for step in range(args.max_step):
        h, r, t, n, ch = next(smp)
        if hb is not None:
            hb.check(args.heartbeat_timeout)
        if step < args.determinism_steps:
            recorder.diff_presampling(h, r, t, n, rank, step, ch)
        losses.append(step_fn(h, r, t, n, ch))
        prof.step()
        if args.force_sync_interval > 0 and W > 1 and (step + 1) % args.force_sync_interval == 0:
            import torch.distributed as dist
            dist.barrier()                   # keeps the workers within one interval of each other (train_pytorch.py:292-294)
        if args.valid and (step + 1) % args.eval_interval == 0 and (ds.valid is not None or ds.test is not None):
            m = run_eval(ds.valid if ds.valid is not None else ds.test, args.eval_percent)
            if m is not None:
                valid_log.append({"step": step + 1, **m})
                if rank == 0:
                    print(f"[{rank}] valid @ {step + 1}: " + ", ".join(f"{k} {v:.4f}" for k, v in m.items()), flush=True)
        if native and (step + 1) % args.log_interval == 0:
            model.ctx.check_status()         # an id out of range or a peer wait that ran out must not train on silently
        if rank == 0 and (step + 1) % args.log_interval == 0:
            recent = [float(x) for x in losses[-args.log_interval:]]
            print(f"[{rank}] step {step + 1}: loss {np.mean(recent):.5f}, {(time.time() - t0) / (step + 1) * 1e3:.2f} ms/step", flush=True)
    if not native and args.async_update:
        model.finish_async_update()          # train_pytorch.py:338-339
    prof.finish()
    if args.device == "cuda":
        torch.cuda.synchronize()
    el = time.time() - t0
    res = {"steps": args.max_step, "first_loss": float(losses[0]), "last_loss": float(np.mean([float(x) for x in losses[-10:]])),
           "triples_per_s": args.batch_size * args.max_step / el}
    if W > 1 or native:
        import torch.distributed as dist
        dist.barrier()
    if valid_log:
        res["valid"] = valid_log
    if args.test and ds.test is not None:
        res["test"] = run_eval(ds.test)
    if args.save_path and not args.no_save_emb:
        if native:
            model.save(args.save_path)
        elif rank == 0:
            os.makedirs(args.save_path, exist_ok=True)
            np.save(os.path.join(args.save_path, f"{ds.name}_{args.model_name}_entity.npy"), model.entity.cpu().numpy())
            np.save(os.path.join(args.save_path, f"{ds.name}_{args.model_name}_relation.npy"), model.relation.cpu().numpy())
            if getattr(model, "proj", None) is not None:      # TransR / RESCAL: the per-relation matrices (tensor_models.py:452-476)
                np.save(os.path.join(args.save_path, f"{ds.name}_{args.model_name}projection.npy"), model.proj.cpu().numpy())
            with open(os.path.join(args.save_path, "config.json"), "w") as f:
                json.dump({"dataset": ds.name, "model_name": args.model_name, "hidden_dim": args.dim, "gamma": args.gamma,
                           "emp_file": f"{ds.name}_{args.model_name}_entity.npy", "rmap_file": f"{ds.name}_{args.model_name}_relation.npy"}, f, indent=2)
    if out is not None:
        out[rank] = res
    if W > 1 or native:
        import torch.distributed as dist
        dist.barrier()
        if hb is not None:
            hb.stop(leaving=True)            # only now: a worker that finishes early keeps beating until all are done
            dist.barrier()
            if rank == 0:
                from recstore_b200.ipc import IPCTensorFactory
                IPCTensorFactory.Delete(hb.name)
        dist.destroy_process_group()


def main(argv=None):
    args = parse_args(argv)
    ds, parts, info = prepare(args)
    print(json.dumps({"prepared": info}), flush=True)
    shared = None
    native = _native(args)
    if not native and args.num_proc > 1 and args.device == "cpu":
        from recstore_b200.baseline.kge_torch import TorchKGE
        m = TorchKGE(ds.n_entities, ds.n_relations, args.dim, args.model_name, args.gamma, args.lr, seed=args.seed)
        shared = {"entity": m.entity.share_memory_(), "relation": m.relation.share_memory_(),
                  "state": {k: v.share_memory_() for k, v in m.state.items()}}
        if m.proj is not None:
            shared["proj"] = m.proj.share_memory_()
    if args.num_proc == 1 and not native:
        out = {}
        worker(0, args, ds, parts, 0, shared, out)
    else:
        import torch.multiprocessing as mp
        out = mp.Manager().dict()
        mp.spawn(worker, args=(args, ds, parts, _free_port(), shared, out), nprocs=args.num_proc, join=True)
        out = dict(out)
    print(json.dumps({"result": out.get(0)}), flush=True)
    print("Successfully xmh", flush=True)
    return dict(out), info


if __name__ == "__main__":
    main()
