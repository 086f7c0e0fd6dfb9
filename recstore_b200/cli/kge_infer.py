"""Tools around trained knowledge-graph embeddings: ranking triples, embedding similarity, evaluation of a saved
model, and dataset conversion.

``python -m recstore_b200.cli.kge_infer <command> ...`` with the commands and flags of the reference's four scripts
(src/kg/kg/dgl-ke/python/dglke):

* ``score`` (infer_score.py:28-234): ``--model_path DIR --format h_r_t|h_r_*|h_*_t|*_r_t|h_*_*|*_r_*|*_*_t
  --data_files ... [--raw_data --entity_mfile F --rel_mfile F] --exec_mode all|triplet_wise|batch_head|batch_rel|
  batch_tail --topK K --score_func none|logsigmoid --output result.tsv [--gpu N]`` writes ``head rel tail score``
  lines.  ``--exclude_mode mask|exclude --known_files F...`` (triples as integer ids, one ``h<TAB>r<TAB>t`` per line)
  adds the treatment of triples that are already known.
* ``emb_sim`` (infer_emb_sim.py:28-150): ``--emb_file F.npy --format l_r|l_*|*_r|* --data_files ... [--raw_data
  --mfile F] --exec_mode all|pairwise|batch_left --topK K --sim_func cosine|l2|l1|dot|ext_jaccard --output result.tsv``.
* ``eval`` (eval.py:107-229): ranks the test triples of a dataset with a saved model: ``--model_path DIR`` plus the
  dataset flags of the trainer; ``--neg_sample_size_eval -1`` (default) ranks against every entity, filtered unless
  ``--no_eval_filter``; ``--num_proc N`` splits the test triples over N processes and averages.
* ``convert`` (convert.py:24-75): ``--data_path DIR --data_files train [valid] [test] --input_format raw_udd_{hrt}
  --output_format udd_{hrt} --output_path DIR`` rewrites name triples as id triples plus the two dictionaries.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------------- id lists
def _read_map(path: str) -> Tuple[Dict[str, int], Dict[int, str]]:
    """A dictionary file ``id<TAB>name`` per line, as the trainers write beside the data."""
    n2i, i2n = {}, {}
    with open(path) as f:
        for line in f:
            p = line.rstrip("\n").split("\t")
            if len(p) >= 2:
                n2i[p[1]] = int(p[0])
                i2n[int(p[0])] = p[1]
    return n2i, i2n


def _read_list(path: Optional[str], n2i: Optional[Dict[str, int]] = None) -> Optional[np.ndarray]:
    """One id (or, with a dictionary, one name) per line; ``None`` stands for "all of them"."""
    if path is None:
        return None
    out = []
    with open(path) as f:
        for ln, line in enumerate(f):
            s = line.rstrip("\n")
            if not s:
                continue
            if n2i is not None:
                if s not in n2i:
                    raise SystemExit(f"{path}:{ln + 1}: {s!r} is not in the id mapping file")
                out.append(n2i[s])
            else:
                out.append(int(s))
    return np.asarray(out, dtype=np.int64)


def _device(gpu: int) -> str:
    return f"cuda:{gpu}" if gpu >= 0 and torch.cuda.is_available() else "cpu"


# ---------------------------------------------------------------------------------------------------- score
def cmd_score(a) -> int:
    from recstore_b200.models.kge_infer import ScoreInfer
    slots = a.format.split("_")
    if len(slots) != 3 or any(s not in (x, "*") for s, x in zip(slots, "hrt")) or slots == ["*", "*", "*"]:
        raise SystemExit(f"unsupported --format {a.format}")
    given = [s != "*" for s in slots]
    files = list(a.data_files or [])
    if len(files) != sum(given):
        raise SystemExit(f"--format {a.format} wants {sum(given)} data file(s), got {len(files)}")
    e2i = r2i = i2e = i2r = None
    if a.raw_data:
        if (given[0] or given[2]) and not a.entity_mfile or given[1] and not a.rel_mfile:
            raise SystemExit("--raw_data needs --entity_mfile (and --rel_mfile when relations are listed)")
        if a.entity_mfile:
            e2i, i2e = _read_map(a.entity_mfile)
        if a.rel_mfile:
            r2i, i2r = _read_map(a.rel_mfile)
    it = iter(files)
    head = _read_list(next(it), e2i) if given[0] else None
    rel = _read_list(next(it), r2i) if given[1] else None
    tail = _read_list(next(it), e2i) if given[2] else None
    inf = ScoreInfer.load(a.model_path, _device(a.gpu), a.score_func)
    if a.exclude_mode:
        if not a.known_files:
            raise SystemExit("--exclude_mode needs --known_files")
        known = np.concatenate([np.loadtxt(f, dtype=np.int64, delimiter="\t", ndmin=2)[:, :3] for f in a.known_files])
        inf.attach_graph(known[:, 0], known[:, 1], known[:, 2])
    result = inf.topk(head, rel, tail, a.topK, a.exec_mode, a.exclude_mode)
    with open(a.output, "w") as f:
        f.write("head\trel\ttail\tscore" + ("\texists\n" if a.exclude_mode == "mask" else "\n"))
        for res in result:
            cols = [x.tolist() for x in res]
            for row in zip(*cols):
                h, r, t, s = row[:4]
                if a.raw_data:
                    h, t = (i2e[h], i2e[t]) if i2e else (h, t)
                    r = i2r[r] if i2r else r
                f.write(f"{h}\t{r}\t{t}\t{s}" + (f"\t{int(row[4])}\n" if len(row) > 4 else "\n"))
    print(f"Inference Done\nThe result is saved in {a.output}")
    return 0


# ---------------------------------------------------------------------------------------------------- emb_sim
def cmd_emb_sim(a) -> int:
    from recstore_b200.models.kge_infer import EmbSimInfer
    want = {"l_r": 2, "l_*": 1, "*_r": 1, "*": 0}
    if a.format not in want:
        raise SystemExit(f"unsupported --format {a.format}")
    files = list(a.data_files or [])
    if len(files) != want[a.format]:
        raise SystemExit(f"--format {a.format} wants {want[a.format]} data file(s), got {len(files)}")
    n2i = i2n = None
    if a.raw_data:
        if not a.mfile:
            raise SystemExit("--raw_data needs --mfile")
        n2i, i2n = _read_map(a.mfile)
    left = _read_list(files[0], n2i) if a.format in ("l_r", "l_*") else None
    right = _read_list(files[-1], n2i) if a.format in ("l_r", "*_r") else None
    modes = {"all": (False, False), "pairwise": (True, False), "batch_left": (False, True)}
    if a.exec_mode not in modes:
        raise SystemExit(f"unknown --exec_mode {a.exec_mode}")
    pair_ws, bcast = modes[a.exec_mode]
    emb = torch.from_numpy(np.load(a.emb_file))
    result = EmbSimInfer(emb, a.sim_func, _device(a.gpu)).topk(left, right, a.topK, pair_ws=pair_ws, bcast=bcast)
    with open(a.output, "w") as f:
        f.write("left\tright\tscore\n")
        for l, r, s in result:
            for x, y, v in zip(l.tolist(), r.tolist(), s.tolist()):
                if i2n:
                    x, y = i2n[x], i2n[y]
                f.write(f"{x}\t{y}\t{v}\n")
    print(f"Inference Done\nThe result is saved in {a.output}")
    return 0


# ---------------------------------------------------------------------------------------------------- eval
def _load_scorer(model_path: str, device: str):
    """A ``TorchKGE`` whose tables are the saved ones."""
    from recstore_b200.baseline.kge_torch import TorchKGE
    with open(os.path.join(model_path, "config.json")) as f:
        c = json.load(f)
    ent = torch.from_numpy(np.load(os.path.join(model_path, c["emp_file"]))).float()
    rel = torch.from_numpy(np.load(os.path.join(model_path, c["rmap_file"]))).float()
    name = c.get("model_name", c.get("model"))
    m = TorchKGE(2, 2, ent.shape[1], name, float(c.get("gamma", 12.0)), device=device)
    m.entity, m.relation = ent.to(device), rel.to(device)
    pf = os.path.join(model_path, c["emp_file"].replace("_entity.npy", "projection.npy"))
    if os.path.exists(pf):
        m.proj = torch.from_numpy(np.load(pf)).float().to(device)
    elif name == "RESCAL" and rel.shape[1] == ent.shape[1] ** 2:      # the matrices are the relation file
        m.proj = m.relation
    elif m.proj is not None:
        raise SystemExit(f"{name} needs its projection file next to {c['emp_file']}")
    m.emb_init = (m.gamma + 2.0) / ent.shape[1]
    return m, c


def _eval_shard(model_path: str, device: str, split, known, neg_size: int, seed: int, threads: int):
    if threads > 0:
        torch.set_num_threads(threads)
    m, _ = _load_scorer(model_path, device)
    h, r, t = (torch.as_tensor(x).to(device) for x in split)
    if neg_size < 0:
        res = m.evaluate_full(h, r, t, known)
    else:
        res = m.evaluate(h, r, t, neg_size, torch.Generator().manual_seed(seed))
    res["triples"] = int(h.numel())
    return res


def _eval_worker(i, model_path, device, shards, known, neg_size, seed, threads, q):
    q.put((i, _eval_shard(model_path, device, shards[i], known, neg_size, seed + i, threads)))


def cmd_eval(a) -> int:
    from recstore_b200.baseline.kge_torch import known_triple_index
    from recstore_b200.utils import kg_data as K
    if not os.path.exists(os.path.join(a.model_path, "config.json")):
        raise SystemExit(f"no saved model in {a.model_path}")
    if a.neg_deg_sample_eval and not a.no_eval_filter and a.neg_sample_size_eval < 0:
        raise SystemExit("degree-based evaluation negatives cannot be combined with the filtered full ranking")
    if a.dataset == "planted_grid":
        ds = K.KGDataset.planted_grid(seed=a.seed)
    elif a.dataset == "synthetic" or a.data_path is None:
        ds = K.KGDataset.synthetic(a.n_entities, a.n_relations, a.n_triples, seed=a.seed)
    else:
        ds = K.KGDataset.load(a.data_path, a.data_files or ["train.tsv"], a.format, name=a.dataset, delimiter=a.delimiter)
    split = ds.test if ds.test is not None else ds.valid
    if split is None:
        raise SystemExit("the dataset has no test (or validation) triples")
    device = _device(a.gpu[0] if a.gpu else -1)
    _, conf = _load_scorer(a.model_path, "cpu")
    known = None
    if a.neg_sample_size_eval < 0 and not a.no_eval_filter:
        known = known_triple_index(ds.train, ds.valid, ds.test)
    n = int(split[0].size)
    W = max(1, min(a.num_proc, n))
    t0 = time.time()
    if W == 1:
        logs = [_eval_shard(a.model_path, device, split, known, a.neg_sample_size_eval, a.seed, a.num_thread)]
    else:
        import torch.multiprocessing as mp
        ctx = mp.get_context("spawn")
        bounds = np.linspace(0, n, W + 1).astype(np.int64)
        shards = [tuple(x[bounds[i]:bounds[i + 1]] for x in split) for i in range(W)]
        q = ctx.Queue()
        threads = a.num_thread or max(1, (os.cpu_count() or W) // W)
        procs = [ctx.Process(target=_eval_worker, args=(i, a.model_path, device if len(a.gpu or []) <= 1 else _device(a.gpu[i % len(a.gpu)]),
                                                         shards, known, a.neg_sample_size_eval, a.seed, threads, q)) for i in range(W)]
        for p in procs:
            p.start()
        got = {}
        while len(got) < W:
            try:
                i, res = q.get(timeout=5)
                got[i] = res
            except Exception:
                dead = [p for p in procs if p.exitcode not in (None, 0)]
                if dead:
                    for p in procs:
                        if p.is_alive():
                            p.terminate()
                    raise SystemExit(f"an evaluation process ended with exit code {dead[0].exitcode}")
        for p in procs:
            p.join()
        logs = [got[i] for i in range(W)]
    tot = sum(l["triples"] for l in logs)
    metrics = {k: sum(l[k] * l["triples"] for l in logs) / tot for k in ("MRR", "MR", "HITS@1", "HITS@3", "HITS@10")}
    print("-------------- Test result --------------")
    for k, v in metrics.items():
        print(f"Test average {k}: {v}")
    print("-----------------------------------------")
    print(f"Test takes {time.time() - t0:.3f} seconds")
    out = {"model": conf.get("model_name", conf.get("model")), "triples": tot, "processes": W,
           "filtered": known is not None, **metrics}
    if a.json_out:
        with open(a.json_out, "w") as f:
            json.dump(out, f, indent=2)
    return out if a._return else 0


# ---------------------------------------------------------------------------------------------------- convert
def cmd_convert(a) -> int:
    from recstore_b200.utils import kg_data as K
    if not a.input_format.startswith("raw_udd_") or not a.output_format.startswith("udd_"):
        raise SystemExit("convert rewrites raw_udd_{hrt} (names) as udd_{hrt} (ids)")
    order = a.output_format.split("_")[-1]
    if sorted(order) != ["h", "r", "t"]:
        raise SystemExit(f"bad --output_format {a.output_format}")
    ds = K.KGDataset.load(a.data_path, a.data_files, a.input_format, delimiter=a.delimiter)
    os.makedirs(a.output_path, exist_ok=True)
    K._write_dict(os.path.join(a.output_path, "entities.tsv"), ds.entity2id, a.delimiter)
    K._write_dict(os.path.join(a.output_path, "relations.tsv"), ds.relation2id, a.delimiter)
    written = ["entities.tsv", "relations.tsv"]
    for name, split in (("train_output.txt", ds.train), ("valid_output.txt", ds.valid), ("test_output.txt", ds.test)):
        if split is None:
            continue
        cols = {"h": split[0], "r": split[1], "t": split[2]}
        with open(os.path.join(a.output_path, name), "w") as f:
            for row in zip(*(cols[c].tolist() for c in order)):
                f.write(a.delimiter.join(str(x) for x in row) + "\n")
        written.append(name)
    print("wrote " + ", ".join(written) + f" to {a.output_path}")
    return 0


# ---------------------------------------------------------------------------------------------------- main
def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="python -m recstore_b200.cli.kge_infer", description=__doc__.split("\n")[0])
    sub = p.add_subparsers(dest="command", required=True)

    s = sub.add_parser("score", help="top-k triples by model score")
    s.add_argument("--model_path", default="ckpts")
    s.add_argument("--format", required=True)
    s.add_argument("--data_files", nargs="+", default=None)
    s.add_argument("--raw_data", action="store_true", help="the lists hold names; translate through the mapping files")
    s.add_argument("--exec_mode", default="all", choices=["all", "triplet_wise", "batch_head", "batch_rel", "batch_tail"])
    s.add_argument("--topK", type=int, default=10)
    s.add_argument("--score_func", default="none", choices=["none", "logsigmoid"])
    s.add_argument("--output", default="result.tsv")
    s.add_argument("--entity_mfile", default=None)
    s.add_argument("--rel_mfile", default=None)
    s.add_argument("--gpu", type=int, default=-1)
    s.add_argument("--exclude_mode", default=None, choices=["mask", "exclude"])
    s.add_argument("--known_files", nargs="+", default=None, help="id triples (h, r, t per line) that count as existing")
    s.set_defaults(fn=cmd_score)

    s = sub.add_parser("emb_sim", help="top-k pairs by embedding similarity")
    s.add_argument("--mfile", default=None)
    s.add_argument("--emb_file", required=True)
    s.add_argument("--format", required=True)
    s.add_argument("--data_files", nargs="+", default=None)
    s.add_argument("--raw_data", action="store_true")
    s.add_argument("--exec_mode", default="all")
    s.add_argument("--topK", type=int, default=10)
    s.add_argument("--sim_func", default="cosine", choices=["cosine", "l2", "l1", "dot", "ext_jaccard"])
    s.add_argument("--output", default="result.tsv")
    s.add_argument("--gpu", type=int, default=-1)
    s.set_defaults(fn=cmd_emb_sim)

    s = sub.add_parser("eval", help="ranking metrics of a saved model on the test triples")
    s.add_argument("--model_path", default="ckpts")
    s.add_argument("--dataset", default="synthetic")
    s.add_argument("--data_path", default=None)
    s.add_argument("--data_files", nargs="+", default=None)
    s.add_argument("--format", default="raw_udd_hrt")
    s.add_argument("--delimiter", default="\t")
    s.add_argument("--n_entities", type=int, default=20000)
    s.add_argument("--n_relations", type=int, default=50)
    s.add_argument("--n_triples", type=int, default=200000)
    s.add_argument("--seed", type=int, default=0)
    s.add_argument("--neg_sample_size_eval", type=int, default=-1)
    s.add_argument("--no_eval_filter", action="store_true")
    s.add_argument("--neg_deg_sample_eval", action="store_true")
    s.add_argument("--num_proc", type=int, default=1)
    s.add_argument("--num_thread", type=int, default=0)
    s.add_argument("--gpu", type=int, nargs="+", default=None)
    s.add_argument("--json_out", default=None, help="also write the metrics there as JSON")
    s.set_defaults(fn=cmd_eval)

    s = sub.add_parser("convert", help="name triples -> id triples + dictionaries")
    s.add_argument("--data_path", default="data")
    s.add_argument("--data_files", nargs="+", required=True)
    s.add_argument("--delimiter", default="\t")
    s.add_argument("--input_format", default="raw_udd_hrt")
    s.add_argument("--output_format", default="udd_hrt")
    s.add_argument("--output_path", default="data")
    s.set_defaults(fn=cmd_convert)
    return p


def main(argv=None, return_result: bool = False):
    a = build_parser().parse_args(argv)
    a._return = return_result
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
