"""Knowledge-graph datasets, triple partitioning, pre-sampling and hot-id renumbering.

* ``KGDataset``: user-defined datasets in the reference's ``raw_udd_{hrt|htr|...}`` form (tab separated triples of
  names, dictionaries built on the fly and written as ``entities.tsv`` / ``relations.tsv``) or ``udd_*`` (triples of
  integer ids plus the two dictionary files), and synthetic power-law graphs for boxes without data
  (src/kg/kg/dgl-ke/python/dglke/dataloader/KGDataset.py: ``KGDatasetUDDRaw`` / ``KGDatasetUDD``).
* Partitioning of the training triples over the workers: ``random_partition``, ``balanced_relation_partition`` (every
  relation on as few workers as its size allows, equal shares) and ``soft_relation_partition`` (large relations spread,
  small ones pinned) -- sampler.py:45-313 of the reference -- and ``graph_partition``: a balanced edge-cut partition of
  the entity graph (the role METIS plays in sampler.py:408-429) by the native multilevel partitioner
  (``csrc/runtime/graph_partition.cpp``); a triple goes to the part of its tail.
* ``presample``: run the sampler ahead for some steps and count how often each entity is touched per worker
  (sampler.py:512-600) -> per-worker hot sets.
* ``renumber_graph``: give the hot entities of worker r the ids ``[start_r, start_r + len_r)`` and everything else the
  ids after them, rewrite the triples (sampler.py:600-634; the dictionary is built by the native
  ``construct_renumbering_dict_op``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class KGDataset:
    name: str
    n_entities: int
    n_relations: int
    train: Tuple[np.ndarray, np.ndarray, np.ndarray]          # (head, rel, tail) int64
    valid: Optional[Tuple[np.ndarray, np.ndarray, np.ndarray]] = None
    test: Optional[Tuple[np.ndarray, np.ndarray, np.ndarray]] = None
    entity2id: Optional[Dict[str, int]] = None
    relation2id: Optional[Dict[str, int]] = None
    train_weight: Optional[np.ndarray] = None                 # importance of every training triple (a fourth column), float32

    @staticmethod
    def synthetic(n_entities: int, n_relations: int, n_triples: int, alpha: float = 1.3, seed: int = 0, test_frac: float = 0.02):
        from .data import powerlaw_triples
        h, r, t = powerlaw_triples(n_triples, n_entities, n_relations, alpha, seed)
        n_test = max(1, int(n_triples * test_frac))
        cut = lambda a, b: (h[a:b], r[a:b], t[a:b])
        return KGDataset("synthetic", n_entities, n_relations, cut(2 * n_test, n_triples), cut(0, n_test), cut(n_test, 2 * n_test))

    @staticmethod
    def planted_grid(width: int = 20, height: int = 15, shifts: Sequence[Tuple[int, int]] = ((1, 0), (0, 1), (2, 1), (-1, 3)),
                     test_frac: float = 0.1, seed: int = 0) -> "KGDataset":
        """A graph with structure to find: the entities are the cells of a ``width x height`` grid, relation k links a
        cell to the cell ``shifts[k]`` away (where that is still on the grid).  A share of the triples is held out:
        a model that has learnt the geometry ranks them high without having seen them, one that memorises does not."""
        trip = [(x * height + y, k, (x + dx) * height + (y + dy)) for x in range(width) for y in range(height)
                for k, (dx, dy) in enumerate(shifts) if 0 <= x + dx < width and 0 <= y + dy < height]
        trip = np.array(trip, dtype=np.int64)
        np.random.default_rng(seed).shuffle(trip)
        n_test = max(1, int(len(trip) * test_frac))
        cut = lambda a, b: tuple(np.ascontiguousarray(trip[a:b, i]) for i in range(3))
        return KGDataset("planted_grid", width * height, len(shifts), cut(n_test, len(trip)), None, cut(0, n_test))

    BUILT_IN = ("FB15k", "FB15k-237", "wn18", "wn18rr", "wikikg2", "biokg", "Freebase")

    @staticmethod
    def load_built_in(data_path: str, name: str, delimiter: str = "\t") -> "KGDataset":
        """The directory layouts of the reference's named datasets (``--format built_in``; KGDataset.py:186-470), read
        from ``data_path/name``; nothing is downloaded.  FB15k, FB15k-237, wn18, wn18rr, wikikg2, biokg:
        ``entities.dict`` / ``relations.dict`` (``id<TAB>name``) and ``train.txt`` / ``valid.txt`` / ``test.txt`` with
        ``head<TAB>relation<TAB>tail`` names.  Freebase: ``entity2id.txt`` / ``relation2id.txt`` whose first line is
        the count, and triple files of integer ids in the order ``head<TAB>tail<TAB>relation``."""
        if name not in KGDataset.BUILT_IN:
            raise ValueError(f"unknown built-in dataset {name!r}; known: {', '.join(KGDataset.BUILT_IN)}")
        d = os.path.join(data_path, name)
        if not os.path.isdir(d):
            raise FileNotFoundError(f"{d} does not exist: put the extracted dataset there (this build downloads nothing)")

        def triples(fn, parse):
            path = os.path.join(d, fn)
            if not os.path.exists(path):
                return None
            hs, rs, ts = [], [], []
            with open(path) as f:
                for ln, line in enumerate(f):
                    p = line.strip().split(delimiter)
                    if len(p) < 3:
                        if line.strip():
                            raise ValueError(f"{path}:{ln + 1}: expected 3 columns")
                        continue
                    try:
                        h, r, t = parse(p)
                    except KeyError as e:
                        raise ValueError(f"{path}:{ln + 1}: {e.args[0]!r} is not in the dictionaries") from None
                    hs.append(h); rs.append(r); ts.append(t)
            return (np.array(hs, dtype=np.int64), np.array(rs, dtype=np.int64), np.array(ts, dtype=np.int64))
        if name == "Freebase":
            with open(os.path.join(d, "entity2id.txt")) as f:
                ne = int(f.readline())
            with open(os.path.join(d, "relation2id.txt")) as f:
                nr = int(f.readline())
            e2i = r2i = None
            parse = lambda p: (int(p[0]), int(p[2]), int(p[1]))
        else:
            e2i = _read_dict(os.path.join(d, "entities.dict"), delimiter)
            r2i = _read_dict(os.path.join(d, "relations.dict"), delimiter)
            ne, nr = len(e2i), len(r2i)
            parse = lambda p: (e2i[p[0]], r2i[p[1]], e2i[p[2]])
        train = triples("train.txt", parse)
        if train is None:
            raise FileNotFoundError(f"{d} has no train.txt")
        valid, test = triples("valid.txt", parse), triples("test.txt", parse)
        for sp in (train, valid, test):
            if sp is not None and sp[0].size and (max(sp[0].max(), sp[2].max()) >= ne or sp[1].max() >= nr or min(sp[0].min(), sp[1].min(), sp[2].min()) < 0):
                raise ValueError(f"{d}: a triple id lies outside the {ne} entities / {nr} relations")
        return KGDataset(name, ne, nr, train, valid, test, e2i, r2i)

    @staticmethod
    def load(path: str, files: Sequence[str], fmt: str = "raw_udd_hrt", name: Optional[str] = None, delimiter: str = "\t",
             has_edge_importance: bool = False):
        """``files``: train [valid test] for ``raw_udd_*``; entities, relations, train [valid test] for ``udd_*``.
        With ``has_edge_importance`` the training file has a fourth column, the weight of the triple in the loss
        (KGDataset.py of the reference: ``has_importance``)."""
        if fmt == "built_in":
            return KGDataset.load_built_in(path, name or "FB15k", delimiter)
        raw = fmt.startswith("raw_udd_")
        order = fmt.split("_")[-1]
        assert sorted(order) == ["h", "r", "t"], f"bad format {fmt}"
        col = {c: i for i, c in enumerate(order)}
        files = list(files)
        if raw:
            e2i: Dict[str, int] = {}
            r2i: Dict[str, int] = {}
            tfiles = files
        else:
            e2i = _read_dict(os.path.join(path, files[0]), delimiter)
            r2i = _read_dict(os.path.join(path, files[1]), delimiter)
            tfiles = files[2:]
        assert 1 <= len(tfiles) <= 3, "expected train [valid test]"
        splits = []
        weights: List[float] = []
        for fi, fn in enumerate(tfiles):
            hs, rs, ts = [], [], []
            with open(os.path.join(path, fn)) as f:
                for ln, line in enumerate(f):
                    p = line.rstrip("\n").split(delimiter)
                    if len(p) < 3:
                        if line.strip():
                            raise ValueError(f"{fn}:{ln + 1}: expected 3 columns")
                        continue
                    hn, rn, tn = p[col["h"]], p[col["r"]], p[col["t"]]
                    if has_edge_importance and fi == 0:
                        if len(p) < 4:
                            raise ValueError(f"{fn}:{ln + 1}: expected a fourth column with the triple's importance")
                        weights.append(float(p[3]))
                    if raw:
                        hs.append(e2i.setdefault(hn, len(e2i))); ts.append(e2i.setdefault(tn, len(e2i)))
                        rs.append(r2i.setdefault(rn, len(r2i)))
                    else:
                        hs.append(int(hn)); rs.append(int(rn)); ts.append(int(tn))
            splits.append((np.array(hs, dtype=np.int64), np.array(rs, dtype=np.int64), np.array(ts, dtype=np.int64)))
        if raw:   # the dictionaries the run used, as the reference writes them beside the data
            _write_dict(os.path.join(path, "entities.tsv"), e2i, delimiter)
            _write_dict(os.path.join(path, "relations.tsv"), r2i, delimiter)
        ne, nr = (len(e2i), len(r2i))
        for h, r, t in splits:
            if h.size and (max(h.max(), t.max()) >= ne or r.max() >= nr):
                raise ValueError("triple id outside the dictionaries")
        return KGDataset(name or os.path.basename(os.path.normpath(path)), ne, nr, splits[0], splits[1] if len(splits) > 1 else None,
                         splits[2] if len(splits) > 2 else None, e2i, r2i,
                         np.array(weights, dtype=np.float32) if has_edge_importance else None)


def _read_dict(path: str, delimiter: str) -> Dict[str, int]:
    d = {}
    with open(path) as f:
        for line in f:
            p = line.rstrip("\n").split(delimiter)
            if len(p) >= 2:
                d[p[1]] = int(p[0])
    return d


def _write_dict(path: str, d: Dict[str, int], delimiter: str) -> None:
    with open(path, "w") as f:
        for k, v in sorted(d.items(), key=lambda kv: kv[1]):
            f.write(f"{v}{delimiter}{k}\n")


# ------------------------------------------------------------------------------------------------ partitioning
def random_partition(n_triples: int, n_parts: int, seed: int = 0) -> List[np.ndarray]:
    perm = np.random.default_rng(seed).permutation(n_triples)
    return [np.sort(p) for p in np.array_split(perm, n_parts)]


def balanced_relation_partition(rel: np.ndarray, n_parts: int, seed: int = 0) -> Tuple[List[np.ndarray], np.ndarray]:
    """Equal-sized parts with every relation on as few parts as possible.  Relations are placed largest first on the
    emptiest part; a relation that does not fit is cut.  Returns the parts and ``cross[r]`` (relation spans parts)."""
    n = rel.size
    cap = -(-n // n_parts)
    cnt = np.bincount(rel)
    order = np.argsort(-cnt, kind="stable")
    fill = np.zeros(n_parts, dtype=np.int64)
    take: List[List[Tuple[int, int]]] = [[] for _ in range(n_parts)]     # (relation, how many) per part
    cross = np.zeros(cnt.size, dtype=bool)
    for r in order:
        left = int(cnt[r])
        first = True
        while left > 0:
            p = int(np.argmin(fill))
            room = cap - int(fill[p])
            k = min(left, room) if room > 0 else left
            take[p].append((int(r), k)); fill[p] += k; left -= k
            if not first or left > 0:
                cross[r] = True
            first = False
    rng = np.random.default_rng(seed)
    by_rel = {int(r): rng.permutation(np.nonzero(rel == r)[0]) for r in np.nonzero(cnt)[0]}
    cur = {r: 0 for r in by_rel}
    parts = []
    for p in range(n_parts):
        idx = []
        for r, k in take[p]:
            idx.append(by_rel[r][cur[r]:cur[r] + k]); cur[r] += k
        parts.append(np.sort(np.concatenate(idx)) if idx else np.zeros(0, dtype=np.int64))
    return parts, cross


def soft_relation_partition(rel: np.ndarray, n_parts: int, threshold: float = 0.05, seed: int = 0) -> Tuple[List[np.ndarray], np.ndarray]:
    """Relations with more than ``threshold`` of the triples are spread evenly over all parts; the others go whole to
    the emptiest part."""
    n = rel.size
    cnt = np.bincount(rel)
    rng = np.random.default_rng(seed)
    fill = np.zeros(n_parts, dtype=np.int64)
    buckets: List[List[np.ndarray]] = [[] for _ in range(n_parts)]
    cross = np.zeros(cnt.size, dtype=bool)
    for r in np.argsort(-cnt, kind="stable"):
        if cnt[r] == 0:
            continue
        idx = rng.permutation(np.nonzero(rel == r)[0])
        if cnt[r] > threshold * n and n_parts > 1:
            cross[r] = True
            for p, piece in enumerate(np.array_split(idx, n_parts)):
                buckets[p].append(piece); fill[p] += piece.size
        else:
            p = int(np.argmin(fill))
            buckets[p].append(idx); fill[p] += idx.size
    return [np.sort(np.concatenate(b)) if b else np.zeros(0, dtype=np.int64) for b in buckets], cross


def graph_partition(head: np.ndarray, tail: np.ndarray, n_entities: int, n_parts: int, imbalance: float = 0.03, seed: int = 0,
                    refine_sweeps: int = 8, balance: str = "triples") -> Tuple[List[np.ndarray], np.ndarray, Dict[str, float]]:
    """Balanced edge-cut partition of the entities (multilevel: heavy-edge matching, greedy growing, boundary
    refinement).  ``balance="triples"`` weighs an entity by the triples it brings to its part (1 + its count as a tail),
    so that the workers get equal shares of the training set; ``"nodes"`` gives equal entity counts.  Returns the triple
    indices per part (a triple belongs to the part of its tail), the part of every entity, and ``{"edge_cut": fraction
    of triples whose ends lie in different parts, "max_part": heaviest part / ideal weight, "levels": ...}``."""
    import ctypes as C
    from .. import _lib
    from .._lib import i32, i64, u64, vp, f64
    _lib.register_signatures({"rs_graph_partition": (i32, [i64, i64, vp, vp, vp, i32, f64, u64, i32, vp, vp])})
    assert balance in ("triples", "nodes")
    h = np.ascontiguousarray(head, dtype=np.int64)
    t = np.ascontiguousarray(tail, dtype=np.int64)
    part = np.empty(n_entities, dtype=np.int32)
    stats = np.zeros(4, dtype=np.int64)
    nw = (1 + np.bincount(t, minlength=n_entities)).astype(np.int64) if balance == "triples" else None
    _lib.call("rs_graph_partition", int(n_entities), int(h.size), h.ctypes.data, t.ctypes.data,
              nw.ctypes.data if nw is not None else None, int(n_parts), float(imbalance),
              int(seed), int(refine_sweeps), part.ctypes.data, stats.ctypes.data)
    owner = part[t]
    parts = [np.nonzero(owner == p)[0].astype(np.int64) for p in range(n_parts)]
    return parts, part, {"edge_cut": float(stats[0]) / max(1, h.size), "max_part": float(stats[1]) * n_parts / max(1, int(stats[3])),
                         "levels": int(stats[2])}


def renumber_by_partition(ds: "KGDataset", node_part: np.ndarray, n_parts: int) -> Tuple["KGDataset", np.ndarray]:
    """New entity ids such that ``new_id % n_parts`` is the entity's part wherever the part sizes allow: a table that is
    sharded cyclically over ``n_parts`` GPUs (row ``id`` on GPU ``id % n_parts``) then keeps every part's entities on
    the GPU of the worker that trains the part, and only the cut edges and the negatives cross NVLink.  Parts larger
    than ``ceil(n / n_parts)`` spill their last entities into the free ids of smaller parts.  Returns the rewritten
    dataset and ``new_id[old_id]``."""
    n = ds.n_entities
    new_id = np.full(n, -1, dtype=np.int64)
    slots = [np.arange(p, n, n_parts, dtype=np.int64) for p in range(n_parts)]       # ids with residue p
    spill: List[np.ndarray] = []
    free: List[np.ndarray] = []
    for p in range(n_parts):
        mine = np.nonzero(node_part == p)[0]
        k = min(mine.size, slots[p].size)
        new_id[mine[:k]] = slots[p][:k]
        if mine.size > k:
            spill.append(mine[k:])
        elif slots[p].size > k:
            free.append(slots[p][k:])
    if spill:
        sp, fr = np.concatenate(spill), np.concatenate(free)
        assert sp.size == fr.size
        new_id[sp] = fr
    assert (new_id >= 0).all()
    f = lambda tr: None if tr is None else (new_id[tr[0]], tr[1], new_id[tr[2]])
    e2i = {k: int(new_id[v]) for k, v in ds.entity2id.items()} if ds.entity2id else None
    return KGDataset(ds.name, n, ds.n_relations, f(ds.train), f(ds.valid), f(ds.test), e2i, ds.relation2id, ds.train_weight), new_id


def write_partition_files(out_dir: str, ds: "KGDataset", parts: Sequence[np.ndarray], node_part: Optional[np.ndarray] = None) -> List[str]:
    """One directory per part (``part_<i>``) for a multi-machine run, as the reference's partition tool lays them out
    (partition.py:35-160): ``train.txt`` with the part's triples as ``head<TAB>rel<TAB>tail`` in GLOBAL ids,
    ``local_to_global.txt`` (line i = global id of the part's i-th entity: those the part owns first, then the remote
    ends of its triples), ``partition_book.txt`` (owner part of every local entity) and ``meta.json``."""
    import json
    h, r, t = ds.train
    if node_part is None:                                     # no node partition given: an entity belongs to the part with most of its triples
        votes = np.zeros((len(parts), ds.n_entities), dtype=np.int64)
        for p, idx in enumerate(parts):
            np.add.at(votes[p], h[idx], 1); np.add.at(votes[p], t[idx], 1)
        node_part = votes.argmax(0).astype(np.int32)
    dirs = []
    for p, idx in enumerate(parts):
        d = os.path.join(out_dir, f"part_{p}")
        os.makedirs(d, exist_ok=True)
        ends = np.unique(np.concatenate([h[idx], t[idx]])) if idx.size else np.zeros(0, dtype=np.int64)
        own = np.nonzero(node_part == p)[0]
        halo = ends[node_part[ends] != p]
        l2g = np.concatenate([own, halo]).astype(np.int64)
        np.savetxt(os.path.join(d, "train.txt"), np.stack([h[idx], r[idx], t[idx]], 1), fmt="%d", delimiter="\t")
        np.savetxt(os.path.join(d, "local_to_global.txt"), l2g, fmt="%d")
        np.savetxt(os.path.join(d, "partition_book.txt"), node_part[l2g], fmt="%d")
        with open(os.path.join(d, "meta.json"), "w") as f:
            json.dump({"part": p, "n_parts": len(parts), "n_triples": int(idx.size), "n_owned_entities": int(own.size),
                       "n_halo_entities": int(halo.size), "n_entities": ds.n_entities, "n_relations": ds.n_relations}, f)
        dirs.append(d)
    return dirs


# ------------------------------------------------------------------------------------------------ sampling
class ChunkedNegativeSampler:
    """Positive batches from one worker's triples plus ``batch / chunk * neg_sample_size`` uniform negative entities;
    head / tail corruption alternates (sampler.py:703-818 of the reference).  ``neg_deg_sample`` draws the negatives in
    proportion to ``1 + degree`` over this worker's triples instead of uniformly; ``weight`` (one float per triple)
    makes ``last_weight`` hold the importance of the batch's positives after every ``next()``."""

    def __init__(self, triples, n_entities: int, batch: int, neg_sample_size: int, neg_chunk_size: int, seed: int = 0, device="cpu",
                 neg_deg_sample: bool = False, weight=None):
        self.h, self.r, self.t = (torch.as_tensor(x, dtype=torch.int64, device=device) for x in triples)
        self.weight = torch.as_tensor(weight, dtype=torch.float32, device=device) if weight is not None else None
        self.last_weight: Optional[torch.Tensor] = None
        self.neg_prob = None
        if neg_deg_sample:
            deg = torch.bincount(torch.cat([self.h, self.t]), minlength=n_entities).float() + 1.0
            self.neg_prob = deg / deg.sum()
        assert batch % neg_chunk_size == 0
        self.n, self.ne, self.batch = self.h.numel(), n_entities, batch
        self.nneg = batch // neg_chunk_size * neg_sample_size
        self.chunk = neg_chunk_size
        self.gen = torch.Generator(device=device).manual_seed(seed)
        self.dev = device
        self.step = 0

    def __next__(self):
        idx = torch.randint(0, self.n, (self.batch,), generator=self.gen, device=self.dev)
        if self.neg_prob is None:
            neg = torch.randint(0, self.ne, (self.nneg,), generator=self.gen, device=self.dev)
        else:
            neg = torch.multinomial(self.neg_prob, self.nneg, replacement=True, generator=self.gen)
        if self.weight is not None:
            self.last_weight = self.weight[idx]
        corrupt_head = bool(self.step & 1)
        self.step += 1
        return self.h[idx], self.r[idx], self.t[idx], neg, corrupt_head

    def __iter__(self):
        return self


def presample(samplers: Sequence[ChunkedNegativeSampler], n_entities: int, steps: int) -> List[torch.Tensor]:
    """Access counts ``[n_entities]`` per worker over ``steps`` sampled batches (positives and negatives).  The
    samplers are advanced; build fresh ones (same seeds) for training if the streams must match."""
    out = []
    for s in samplers:
        c = torch.zeros(n_entities, dtype=torch.int64)
        for _ in range(steps):
            h, _, t, neg, _ = next(s)
            ids = torch.cat([h, t, neg]).cpu()
            c += torch.bincount(ids, minlength=n_entities)
        out.append(c)
    return out


def hot_sets(counts: Sequence[torch.Tensor], cache_size: int) -> List[torch.Tensor]:
    """Disjoint per-worker hot sets: every entity goes to the worker that touches it most; each keeps its top
    ``cache_size`` by count."""
    C = torch.stack(list(counts))                     # [W, N]
    owner = C.argmax(0)
    best = C.max(0).values
    out = []
    for w in range(C.shape[0]):
        mine = torch.nonzero((owner == w) & (best > 0)).view(-1)
        if mine.numel() > cache_size:
            top = torch.topk(best[mine], cache_size).indices
            mine = mine[top]
        out.append(mine.sort().values)
    return out


def renumber_graph(ds: KGDataset, hot: Sequence[torch.Tensor], cache_size: int) -> Tuple[KGDataset, torch.Tensor]:
    """New ids: hot set of worker r -> ``[r * cache_size, r * cache_size + len)``, the rest after them in old order.
    Returns the rewritten dataset and ``new_id[old_id]``."""
    from ..torch_op import construct_renumbering_dict_op
    W = len(hot)
    padded = []
    used = torch.zeros(ds.n_entities, dtype=torch.bool)
    for hs in hot:
        assert hs.numel() <= cache_size
        used[hs] = True
        padded.append(hs)
    # pad every hot set to cache_size with cold ids so that worker r's range starts at r * cache_size
    cold = torch.nonzero(~used).view(-1)
    need = [cache_size - p.numel() for p in padded]
    assert sum(need) <= cold.numel(), "cache_size * workers exceeds the number of entities"
    o = 0
    full = []
    for p, k in zip(padded, need):
        full.append(torch.cat([p, cold[o:o + k]]))
        o += k
    d = torch.full((ds.n_entities,), -1, dtype=torch.int64)
    construct_renumbering_dict_op(d, W, full)
    m = d.numpy()
    f = lambda tr: None if tr is None else (m[tr[0]], tr[1], m[tr[2]])
    e2i = {k: int(m[v]) for k, v in ds.entity2id.items()} if ds.entity2id else None
    return KGDataset(ds.name, ds.n_entities, ds.n_relations, f(ds.train), f(ds.valid), f(ds.test), e2i, ds.relation2id,
                     ds.train_weight), d


def _main(argv=None):
    """``python -m recstore_b200.utils.kg_data -k 4 --out parts/ [--data_path D --data_files train.tsv --format raw_udd_hrt]``:
    edge-cut partition of a dataset into per-part directories (the reference's ``dglke_partition`` command,
    partition.py:35-160); without ``--data_path`` a synthetic power-law graph is partitioned."""
    import argparse
    import json
    p = argparse.ArgumentParser(description="partition a knowledge graph for multi-worker training")
    p.add_argument("-k", "--num-parts", type=int, required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--data_path", default=None)
    p.add_argument("--data_files", nargs="+", default=None)
    p.add_argument("--format", default="raw_udd_hrt")
    p.add_argument("--dataset", default="synthetic")
    p.add_argument("--delimiter", default="\t")
    p.add_argument("--n_entities", type=int, default=20000)
    p.add_argument("--n_relations", type=int, default=50)
    p.add_argument("--n_triples", type=int, default=200000)
    p.add_argument("--balance", choices=["triples", "nodes"], default="triples")
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args(argv)
    if a.data_path:
        ds = KGDataset.load(a.data_path, a.data_files or ["train.tsv"], a.format, name=a.dataset, delimiter=a.delimiter)
    else:
        ds = KGDataset.synthetic(a.n_entities, a.n_relations, a.n_triples, seed=a.seed)
    parts, node_part, st = graph_partition(ds.train[0], ds.train[2], ds.n_entities, a.num_parts, seed=a.seed, balance=a.balance)
    dirs = write_partition_files(a.out, ds, parts, node_part)
    out = {"parts": dirs, "triples_per_part": [int(x.size) for x in parts], **st}
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    _main()
