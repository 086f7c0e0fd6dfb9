"""Distributed knowledge-graph training against parameter-server shards: the KVStore mode of the reference's DGL-KE.

Servers hold the entity and relation embeddings (key-sharded, row-wise Adagrad applied on the server by the
``UpdateParameter`` verb: ``state += mean(g^2); emb -= lr * g / (sqrt(state) + eps)``, the push handler of
kvserver.py:38-57); every trainer owns one partition of the triples (kvclient.py:119-215), pulls the rows of its batch
with ``GetParameter``, scores and differentiates locally, and pushes one summed gradient per distinct row.  The
launcher (the role of dist_train.py:121-211, here for the processes of one box) partitions the graph, optionally
writes the per-part dataset directories, starts the servers, spawns the trainers and saves the usual checkpoint.

    python -m recstore_b200.cli.kge_dist --model_name TransE_l2 --num_servers 2 --num_clients 2 --max_step 200 \
        --n_entities 20000 --n_triples 200000 --hidden_dim 64 --graph_part --test --save_path out/

Models: those whose relation row is as wide as the entity row and that have no per-relation matrix (TransE l1 / l2,
DistMult, ComplEx, SimplE).
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import time
from typing import List, Sequence

import numpy as np
import torch

REL_BASE = 1 << 40          # relation r is key REL_BASE + r: one key space for both tables
PROJ_BASE = 1 << 41         # TransR / RESCAL: row i of relation r's hidden_dim x hidden_dim matrix is key PROJ_BASE + r * hidden_dim + i
                            # (a matrix is hidden_dim shard rows; the server keeps one Adagrad state per ROW of it, where the
                            # single-box trainers keep one per matrix)
DIST_MODELS = ("TransE", "TransE_l1", "TransE_l2", "DistMult", "ComplEx", "SimplE", "RotatE", "TransR", "RESCAL")


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--model_name", default="TransE_l2", choices=DIST_MODELS)
    p.add_argument("--num_servers", type=int, default=2)
    p.add_argument("--num_clients", type=int, default=2)
    p.add_argument("--n_entities", type=int, default=20000)
    p.add_argument("--n_relations", type=int, default=50)
    p.add_argument("--n_triples", type=int, default=200000)
    p.add_argument("--data_path", default=None)
    p.add_argument("--data_files", nargs="+", default=None)
    p.add_argument("--format", default="raw_udd_hrt")
    p.add_argument("--dataset", default="synthetic")
    p.add_argument("--hidden_dim", type=int, default=64)
    p.add_argument("--gamma", type=float, default=12.0)
    p.add_argument("--lr", type=float, default=0.1)
    p.add_argument("--batch_size", type=int, default=256)
    p.add_argument("--neg_sample_size", type=int, default=64)
    p.add_argument("--neg_chunk_size", type=int, default=None)
    p.add_argument("--max_step", type=int, default=100)
    p.add_argument("--graph_part", action="store_true", help="edge-cut partition of the entities (else random triples)")
    p.add_argument("--partition_dir", default=None, help="also write the per-part dataset directories there")
    p.add_argument("--from_partition_dir", default=None,
                   help="train on existing per-part directories (part_<i>/train.txt in global ids, meta.json), one trainer per part")
    p.add_argument("--loss_genre", "-lg", default="Logsigmoid", choices=["Hinge", "Logistic", "Logsigmoid", "BCE"])
    p.add_argument("--margin", "-m", type=float, default=1.0, help="margin of the hinge loss")
    p.add_argument("--neg_adversarial_sampling", "-adv", action="store_true", help="weigh a positive's negatives by softmax(score * temperature)")
    p.add_argument("--adversarial_temperature", "-a", type=float, default=1.0)
    p.add_argument("--regularization_coef", "-rc", type=float, default=0.0, help="Lp penalty on the rows a step touches")
    p.add_argument("--regularization_norm", "-rn", type=int, default=3)
    p.add_argument("--engine", default="KVEngineMap", help="KV engine of the server shards")
    p.add_argument("--servers", nargs="+", default=None, metavar="HOST:PORT",
                   help="shards that are running already (python -m recstore_b200.ps.server, possibly on other machines; they must "
                        "have been started with --dim = --hidden_dim, --optimizer rowwise_adagrad and the --lr of this run): "
                        "none is started here and --num_servers is their count")
    p.add_argument("--test", action="store_true")
    p.add_argument("--save_path", default=None)
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args(argv)
    if a.neg_chunk_size is None:
        a.neg_chunk_size = min(a.neg_sample_size, a.batch_size)
    a.batch_size = -(-a.batch_size // a.neg_chunk_size) * a.neg_chunk_size
    return a


class ShardedClient:
    """The trainers' view of the servers: keys are routed by ``ShardManager.KeyPartition`` and answers put back in order."""

    def __init__(self, ports: Sequence, dim: int):
        """``ports``: one entry per shard, a port on this machine or a ``(host, port)`` pair."""
        from recstore_b200.ps.client import ParameterClient
        addrs = [("127.0.0.1", p) if isinstance(p, int) else (p[0], int(p[1])) for p in ports]
        self.clients = [ParameterClient(h, p, shard=i, emb_dim=dim) for i, (h, p) in enumerate(addrs)]
        self.dim = dim

    def _route(self, keys: torch.Tensor) -> List[torch.Tensor]:
        from recstore_b200.ps.client import ShardManager
        shard = ShardManager.KeyPartition(keys, len(self.clients))
        return [torch.nonzero(shard == s).reshape(-1) for s in range(len(self.clients))]

    def pull(self, keys: torch.Tensor) -> torch.Tensor:
        out = torch.empty(keys.numel(), self.dim)
        for c, idx in zip(self.clients, self._route(keys)):
            if idx.numel():
                out[idx] = c.GetParameter(keys[idx])
        return out

    def push(self, keys: torch.Tensor, values: torch.Tensor, update: bool) -> None:
        for c, idx in zip(self.clients, self._route(keys)):
            if idx.numel():
                (c.UpdateParameter if update else c.PutParameter)(keys[idx], values[idx])

    def close(self) -> None:
        for c in self.clients:
            c.close()


def trainer(rank: int, args, triples, ports, queue) -> None:
    """One trainer process: sample -> pull -> score -> push."""
    from recstore_b200.baseline.kge_torch import chunk_neg_score, edge_score, kg_loss
    from recstore_b200.utils.kg_data import ChunkedNegativeSampler
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // max(1, args.num_clients)))
    ps = ShardedClient(ports, args.hidden_dim)
    smp = ChunkedNegativeSampler(triples, args.n_entities, args.batch_size, args.neg_sample_size, args.neg_chunk_size,
                                 seed=args.seed * 100 + rank)
    emb_init = (args.gamma + 2.0) / args.hidden_dim
    from recstore_b200.baseline.kge_torch import relation_dim
    rel_dim = relation_dim(args.model_name, args.hidden_dim)
    matrix_model = args.model_name in ("TransR", "RESCAL")
    losses, t0 = [], time.time()
    for step in range(args.max_step):
        h, r, t, neg, corrupt_head = next(smp)
        ent_ids, ent_inv = torch.unique(torch.cat([h, t, neg]), return_inverse=True)
        rel_ids, rel_inv = torch.unique(r, return_inverse=True)
        ent = ps.pull(ent_ids).requires_grad_(True)                     # one row per distinct id: duplicates sum in autograd
        rel = ps.pull(rel_ids + REL_BASE).requires_grad_(True)
        bs = h.numel()
        he, te, ne = ent[ent_inv[:bs]], ent[ent_inv[bs:2 * bs]], ent[ent_inv[2 * bs:]]
        re = rel[rel_inv][:, :rel_dim]               # RotatE: a relation is hidden_dim / 2 phases; the shard's rows are hidden_dim wide
        proj = mat = None
        if matrix_model:
            D = args.hidden_dim
            mat_keys = (rel_ids.unsqueeze(1) * D + torch.arange(D)).reshape(-1) + PROJ_BASE
            mat = ps.pull(mat_keys).requires_grad_(True)            # [distinct relations * D, D]
            proj = mat.view(rel_ids.numel(), D * D)[rel_inv]
        pos = edge_score(args.model_name, he, re, te, args.gamma, proj, emb_init)
        negs = chunk_neg_score(args.model_name, he, re, te, ne, corrupt_head, args.neg_chunk_size, args.gamma, proj, emb_init)
        loss = kg_loss(pos, negs, args.loss_genre, args.margin, args.neg_adversarial_sampling, args.adversarial_temperature)
        if args.regularization_coef > 0:         # on the distinct rows of the step (general_models.py:623-629)
            loss = loss + args.regularization_coef * (ent.norm(p=args.regularization_norm) ** args.regularization_norm +
                                                      rel.norm(p=args.regularization_norm) ** args.regularization_norm)
        loss.backward()
        ps.push(ent_ids, ent.grad, update=True)
        if rel.grad is not None:                     # RESCAL scores with the matrix only
            ps.push(rel_ids + REL_BASE, rel.grad, update=True)
        if mat is not None:
            ps.push(mat_keys, mat.grad, update=True)
        losses.append(loss.item())
    el = time.time() - t0
    ps.close()
    queue.put((rank, {"first_loss": losses[0], "last_loss": float(np.mean(losses[-10:])),
                      "triples_per_s": args.batch_size * args.max_step / max(el, 1e-9)}))


def _load_partition_dirs(root: str, name: str):
    """Dataset and per-part triple index lists from ``part_<i>`` directories (``utils.kg_data.write_partition_files``)."""
    from recstore_b200.utils import kg_data as K
    dirs = sorted((d for d in os.listdir(root) if d.startswith("part_")), key=lambda d: int(d.split("_")[1]))
    if not dirs:
        raise FileNotFoundError(f"{root} holds no part_<i> directories")
    hs, rs, ts, parts, o = [], [], [], [], 0
    meta = {}
    for d in dirs:
        with open(os.path.join(root, d, "meta.json")) as f:
            meta = json.load(f)
        tri = np.loadtxt(os.path.join(root, d, "train.txt"), dtype=np.int64, ndmin=2)
        hs.append(tri[:, 0]); rs.append(tri[:, 1]); ts.append(tri[:, 2])
        parts.append(np.arange(o, o + tri.shape[0], dtype=np.int64))
        o += tri.shape[0]
    assert meta.get("n_parts", len(dirs)) == len(dirs), "a part directory is missing"
    train = (np.concatenate(hs), np.concatenate(rs), np.concatenate(ts))
    return K.KGDataset(name, int(meta["n_entities"]), int(meta["n_relations"]), train), parts


def main(argv=None) -> dict:
    args = parse_args(argv)
    from recstore_b200.baseline.kge_torch import TorchKGE
    from recstore_b200.ps.client import ParameterServer
    from recstore_b200.utils import kg_data as K
    if args.from_partition_dir:
        ds, parts = _load_partition_dirs(args.from_partition_dir, args.dataset)
        args.num_clients = len(parts)
    elif args.dataset == "planted_grid":
        ds = K.KGDataset.planted_grid(seed=args.seed)
    elif args.data_path:
        ds = K.KGDataset.load(args.data_path, args.data_files or ["train.tsv"], args.format, name=args.dataset)
    else:
        ds = K.KGDataset.synthetic(args.n_entities, args.n_relations, args.n_triples, seed=args.seed)
    args.n_entities, args.n_relations = ds.n_entities, ds.n_relations
    info = {"n_entities": ds.n_entities, "n_relations": ds.n_relations, "n_train": int(ds.train[0].size)}
    node_part = None
    if args.from_partition_dir:
        pass                                         # the directories are the partition
    elif args.graph_part:
        parts, node_part, st = K.graph_partition(ds.train[0], ds.train[2], ds.n_entities, args.num_clients, seed=args.seed)
        info["edge_cut"] = st["edge_cut"]
    else:
        parts = K.random_partition(ds.train[0].size, args.num_clients, args.seed)
    if args.partition_dir:
        info["partition_dirs"] = K.write_partition_files(args.partition_dir, ds, parts, node_part)
    # ---- servers: one shard each, server-side row-wise Adagrad (started here, or running already)
    servers = []
    if args.servers:
        ports = [(a.rsplit(":", 1)[0], int(a.rsplit(":", 1)[1])) for a in args.servers]
        args.num_servers = len(ports)
    else:
        n_keys = ds.n_entities + ds.n_relations * (1 + (args.hidden_dim if args.model_name in ("TransR", "RESCAL") else 0))
        cap = 1 << max(16, int(np.ceil(np.log2(n_keys * 2 / args.num_servers + 1))))
        servers = [ParameterServer(args.engine, {"dim": args.hidden_dim, "capacity": cap, "optimizer": "rowwise_adagrad", "lr": args.lr})
                   for _ in range(args.num_servers)]
        ports = [s.serve(0) for s in servers]
    boot = ShardedClient(ports, args.hidden_dim)
    g = torch.Generator().manual_seed(args.seed)
    emb_init = (args.gamma + 2.0) / args.hidden_dim
    tables = [(0, ds.n_entities), (REL_BASE, ds.n_relations)]
    if args.model_name in ("TransR", "RESCAL"):
        tables.append((PROJ_BASE, ds.n_relations * args.hidden_dim))
    for base, n in tables:                                                # U(+-emb_init), as the single-box trainers start
        for lo in range(0, n, 65536):
            k = torch.arange(lo, min(n, lo + 65536), dtype=torch.int64)
            boot.push(k + base, (torch.rand(k.numel(), args.hidden_dim, generator=g) * 2 - 1) * emb_init, update=False)
    # ---- trainers
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=trainer, args=(r, args, tuple(x[parts[r]] for x in ds.train), ports, queue))
             for r in range(args.num_clients)]
    t0 = time.time()
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=3600) for _ in procs)
    for p in procs:
        p.join(60)
    out = {"prepared": info, "seconds": time.time() - t0, "workers": [results[r] for r in range(args.num_clients)],
           "triples_per_s": sum(results[r]["triples_per_s"] for r in results),
           "server_keys": [len(s) for s in servers] if servers else [c.Stats()["keys_stored"] for c in boot.clients]}
    # ---- the trained tables come back for evaluation and the checkpoint
    if args.test or args.save_path:
        ent = boot.pull(torch.arange(ds.n_entities, dtype=torch.int64))
        from recstore_b200.baseline.kge_torch import relation_dim
        rel = boot.pull(torch.arange(ds.n_relations, dtype=torch.int64) + REL_BASE)[:, :relation_dim(args.model_name, args.hidden_dim)].contiguous()
        if args.test and ds.test is not None:
            m = TorchKGE(ds.n_entities, ds.n_relations, args.hidden_dim, args.model_name, args.gamma, args.lr, seed=args.seed)
            m.entity, m.relation = ent, rel
            if args.model_name in ("TransR", "RESCAL"):
                m.proj = boot.pull(torch.arange(ds.n_relations * args.hidden_dim, dtype=torch.int64) + PROJ_BASE).view(ds.n_relations, -1)
            th, tr, tt = (torch.as_tensor(x[:1024]) for x in ds.test)
            out["test"] = m.evaluate(th, tr, tt, 256, torch.Generator().manual_seed(5))
        if args.save_path:
            os.makedirs(args.save_path, exist_ok=True)
            np.save(os.path.join(args.save_path, f"{ds.name}_{args.model_name}_entity.npy"), ent.numpy())
            np.save(os.path.join(args.save_path, f"{ds.name}_{args.model_name}_relation.npy"), rel.numpy())
            if args.model_name in ("TransR", "RESCAL"):
                prj = boot.pull(torch.arange(ds.n_relations * args.hidden_dim, dtype=torch.int64) + PROJ_BASE)
                np.save(os.path.join(args.save_path, f"{ds.name}_{args.model_name}projection.npy"), prj.view(ds.n_relations, -1).numpy())
            with open(os.path.join(args.save_path, "config.json"), "w") as f:
                json.dump({"dataset": ds.name, "model_name": args.model_name, "hidden_dim": args.hidden_dim, "gamma": args.gamma,
                           "emp_file": f"{ds.name}_{args.model_name}_entity.npy",
                           "rmap_file": f"{ds.name}_{args.model_name}_relation.npy"}, f, indent=2)
    boot.close()
    for s in servers:
        s.stop()
        s.close()
    print(json.dumps({"result": {k: v for k, v in out.items() if k != "prepared"}}), flush=True)
    return out


if __name__ == "__main__":
    main()
