"""Inference over trained knowledge-graph embeddings: top-k triple scoring, link prediction and embedding similarity.

* ``ScoreInfer.topk(head, rel, tail, k, exec_mode)`` ranks candidate triples by a model's score function
  (``all``: every head x rel x tail combination; ``triplet_wise``: aligned lists; ``batch_head`` / ``batch_rel`` /
  ``batch_tail``: one top-k list per element of that argument) -- the modes of the reference's ``ScoreInfer``
  (src/kg/kg/dgl-ke/python/dglke/models/infer.py:52-214).  Candidates are scored in blocks and merged into a running
  top-k, so memory is bounded by the block, not by ``len(head) * len(rel) * len(tail)``.
* ``EmbSimInfer.topk(left, right, k, pair_ws, bcast)`` ranks entity pairs by ``cosine`` / ``l2`` / ``l1`` / ``dot`` /
  ``ext_jaccard`` similarity (infer.py:216-344).
* ``KGEModel``: the model-object surface (``load``, ``attach_graph``, ``link_predict`` with the ``none`` /
  ``logsigmoid`` output functions and the ``mask`` / ``exclude`` treatment of triples that are already in the graph,
  ``embed_sim`` over entity or relation embeddings; ke_model.py:56-853 ``BasicGEModel``), with one subclass per
  score function as there (``TransEModel`` ... ``SimplEModel``).

All of them load the ``.npy`` + ``config.json`` checkpoints written by the trainers, or take tensors directly.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Tuple

import numpy as np
import torch

from ..baseline.kge_torch import edge_score

DEFAULT_INFER_BATCH = 1 << 16          # candidate triples scored at a time


def _ids(x, n: int, dev) -> torch.Tensor:
    if x is None:
        return torch.arange(n, device=dev)
    return torch.as_tensor(x, dtype=torch.int64, device=dev).reshape(-1)


class _TripleIndex:
    """Membership test for (head, rel, tail) against the triples of a graph: pairs (head, tail) packed into one sorted
    int64 array, the relations of equal pairs beside them."""

    def __init__(self, head, rel, tail, n_entities: int):
        h, r, t = (np.asarray(x, dtype=np.int64).reshape(-1) for x in (head, rel, tail))
        self.n = int(n_entities)
        key = h * self.n + t
        order = np.lexsort((r, key))
        self.key, self.rel = key[order], r[order]

    def contains(self, head, rel, tail) -> np.ndarray:
        h, r, t = (np.asarray(x, dtype=np.int64).reshape(-1) for x in (head, rel, tail))
        key = h * self.n + t
        lo, hi = np.searchsorted(self.key, key, "left"), np.searchsorted(self.key, key, "right")
        out = np.zeros(key.shape[0], dtype=bool)
        for i in np.nonzero(hi > lo)[0]:
            out[i] = bool((self.rel[lo[i]:hi[i]] == r[i]).any())
        return out


class ScoreInfer:
    def __init__(self, model_name: str, entity: torch.Tensor, relation: torch.Tensor, gamma: float = 12.0, device="cpu",
                 projection: Optional[torch.Tensor] = None, sfunc: str = "none"):
        assert sfunc in ("none", "logsigmoid"), sfunc
        self.model, self.gamma, self.dev, self.sfunc = model_name, gamma, torch.device(device), sfunc
        self.entity, self.relation = entity.to(self.dev), relation.to(self.dev)
        # TransR / RESCAL: one matrix per relation, stored flat (tensor_models.py:188-199 reads the same file)
        self.projection = projection.to(self.dev) if projection is not None else None
        assert self.projection is not None or model_name not in ("TransR",), f"{model_name} needs its projection matrices"
        self.emb_init = (gamma + 2.0) / entity.shape[1]
        self.known: Optional[_TripleIndex] = None

    @staticmethod
    def load(path: str, device="cpu", sfunc: str = "none") -> "ScoreInfer":
        with open(os.path.join(path, "config.json")) as f:
            c = json.load(f)
        ent = torch.from_numpy(np.load(os.path.join(path, c["emp_file"])))
        rel = torch.from_numpy(np.load(os.path.join(path, c["rmap_file"])))
        name = c.get("model_name", c.get("model"))
        pfile = os.path.join(path, c["emp_file"].replace("_entity.npy", "projection.npy"))
        proj = torch.from_numpy(np.load(pfile)) if os.path.exists(pfile) else None
        return ScoreInfer(name, ent, rel, float(c.get("gamma", 12.0)), device, projection=proj, sfunc=sfunc)

    def attach_graph(self, head, rel, tail) -> None:
        """The triples that count as existing for ``exclude_mode``."""
        self.known = _TripleIndex(head, rel, tail, self.entity.shape[0])

    @torch.no_grad()
    def _score(self, h, r, t) -> torch.Tensor:
        proj = self.projection[r] if self.projection is not None else None
        if proj is None and self.model == "RESCAL":          # checkpoints that keep the matrices in the relation file
            assert self.relation.shape[1] == self.entity.shape[1] ** 2, "RESCAL needs one dim x dim matrix per relation"
            proj = self.relation[r]
        s = edge_score(self.model, self.entity[h], self.relation[r], self.entity[t], self.gamma, proj, self.emb_init)
        return torch.nn.functional.logsigmoid(s) if self.sfunc == "logsigmoid" else s

    def _grid_topk(self, h, r, t, k: int, batch: int):
        """Top k of score(h_i, r_j, t_l) over the whole grid: (flat positions into the grid, scores), best first."""
        nh, nr, nt = h.numel(), r.numel(), t.numel()
        total = nh * nr * nt
        best_s = torch.empty(0, device=self.dev)
        best_i = torch.empty(0, dtype=torch.int64, device=self.dev)
        for lo in range(0, total, batch):
            flat = torch.arange(lo, min(total, lo + batch), device=self.dev)
            s = self._score(h[flat // (nr * nt)], r[(flat // nt) % nr], t[flat % nt])
            best_s, best_i = torch.cat([best_s, s]), torch.cat([best_i, flat])
            if best_s.numel() > k:
                top = torch.topk(best_s, k)
                best_s, best_i = top.values, best_i[top.indices]
        order = torch.argsort(best_s, descending=True, stable=True)
        return best_i[order], best_s[order]

    def _one_list(self, h, r, t, k: int, exclude_mode: Optional[str], batch: int, triplet_wise: bool = False):
        nh, nr, nt = h.numel(), r.numel(), t.numel()
        total = nh if triplet_wise else nh * nr * nt
        want = min(k, total)
        take = want if exclude_mode != "exclude" else min(total, 2 * want + 16)
        while True:
            if triplet_wise:
                s = torch.cat([self._score(h[lo:lo + batch], r[lo:lo + batch], t[lo:lo + batch]) for lo in range(0, total, batch)]) \
                    if total else torch.empty(0, device=self.dev)
                top = torch.topk(s, take)
                H, R, T, S = h[top.indices], r[top.indices], t[top.indices], top.values
            else:
                flat, S = self._grid_topk(h, r, t, take, batch)
                H, R, T = h[flat // (nr * nt)], r[(flat // nt) % nr], t[flat % nt]
            if exclude_mode is None:
                return H, R, T, S
            assert self.known is not None, "exclude_mode needs the graph: call attach_graph(head, rel, tail) first"
            exists = torch.from_numpy(self.known.contains(H.cpu().numpy(), R.cpu().numpy(), T.cpu().numpy())).to(self.dev)
            if exclude_mode == "mask":
                return H, R, T, S, exists
            keep = ~exists
            if int(keep.sum()) >= want or take >= total:
                sel = torch.nonzero(keep).reshape(-1)[:want]
                return H[sel], R[sel], T[sel], S[sel]
            take = min(total, take * 2)          # too many of the best candidates exist already: look further down

    def topk(self, head=None, rel=None, tail=None, k: int = 10, exec_mode: str = "all", exclude_mode: Optional[str] = None,
             batch_size: int = DEFAULT_INFER_BATCH) -> List[Tuple[torch.Tensor, ...]]:
        """Each result is ``(head_ids, rel_ids, tail_ids, scores)`` sorted by decreasing score (``exclude_mode="mask"``
        adds a fifth tensor: True where the triple is in the attached graph; ``"exclude"`` leaves such triples out).
        ``None`` for an argument = all ids."""
        assert exclude_mode in (None, "mask", "exclude"), exclude_mode
        head, rel, tail = (_ids(head, self.entity.shape[0], self.dev), _ids(rel, self.relation.shape[0], self.dev),
                           _ids(tail, self.entity.shape[0], self.dev))
        if exec_mode == "triplet_wise":
            assert head.numel() == rel.numel() == tail.numel(), "triplet_wise wants three lists of one length"
            return [self._one_list(head, rel, tail, k, exclude_mode, batch_size, triplet_wise=True)]
        if exec_mode == "all":
            return [self._one_list(head, rel, tail, k, exclude_mode, batch_size)]
        if exec_mode == "batch_head":
            return [self._one_list(head[i:i + 1], rel, tail, k, exclude_mode, batch_size) for i in range(head.numel())]
        if exec_mode == "batch_rel":
            return [self._one_list(head, rel[i:i + 1], tail, k, exclude_mode, batch_size) for i in range(rel.numel())]
        if exec_mode == "batch_tail":
            return [self._one_list(head, rel, tail[i:i + 1], k, exclude_mode, batch_size) for i in range(tail.numel())]
        raise ValueError(f"unknown exec_mode {exec_mode!r}")

    topK = topk


def _pair_sim(a: torch.Tensor, b: torch.Tensor, fn: str) -> torch.Tensor:
    """Similarity matrix ``[len(a), len(b)]`` (larger = more similar)."""
    if fn == "cosine":
        return torch.nn.functional.normalize(a, dim=1) @ torch.nn.functional.normalize(b, dim=1).t()
    if fn == "dot":
        return a @ b.t()
    if fn == "l2":
        return -torch.cdist(a, b, p=2)
    if fn == "l1":
        return -torch.cdist(a, b, p=1)
    if fn == "ext_jaccard":
        ab = a @ b.t()
        return ab / ((a * a).sum(1, keepdim=True) + (b * b).sum(1).unsqueeze(0) - ab)
    raise ValueError(fn)


def _row_sim(a: torch.Tensor, b: torch.Tensor, fn: str) -> torch.Tensor:
    """Similarity of aligned rows ``[n]``."""
    if fn == "cosine":
        return (torch.nn.functional.normalize(a, dim=1) * torch.nn.functional.normalize(b, dim=1)).sum(1)
    if fn == "dot":
        return (a * b).sum(1)
    if fn == "l2":
        return -(a - b).norm(p=2, dim=1)
    if fn == "l1":
        return -(a - b).norm(p=1, dim=1)
    if fn == "ext_jaccard":
        ab = (a * b).sum(1)
        return ab / ((a * a).sum(1) + (b * b).sum(1) - ab)
    raise ValueError(fn)


class EmbSimInfer:
    def __init__(self, emb: torch.Tensor, sfunc: str = "cosine", device="cpu"):
        self.emb, self.sfunc = emb.to(device), sfunc

    @torch.no_grad()
    def topk(self, left=None, right=None, k: int = 10, pair_ws: bool = False, bcast: bool = False, batch_size: int = 1024):
        n, dev = self.emb.shape[0], self.emb.device
        left, right = _ids(left, n, dev), _ids(right, n, dev)
        if pair_ws:                                    # aligned pairs
            assert left.numel() == right.numel(), "pair_ws wants two lists of one length"
            s = torch.cat([_row_sim(self.emb[left[lo:lo + batch_size]], self.emb[right[lo:lo + batch_size]], self.sfunc)
                           for lo in range(0, left.numel(), batch_size)]) if left.numel() else torch.empty(0, device=dev)
            top = torch.topk(s, min(k, s.numel()))
            return [(left[top.indices], right[top.indices], top.values)]
        if bcast:                                      # one list per left id
            out = []
            kk = min(k, right.numel())
            for lo in range(0, left.numel(), batch_size):
                S = _pair_sim(self.emb[left[lo:lo + batch_size]], self.emb[right], self.sfunc)
                top = torch.topk(S, kk, dim=1)
                out += [(left[lo + i].expand(kk), right[top.indices[i]], top.values[i]) for i in range(S.shape[0])]
            return out
        best_s = torch.empty(0, device=dev)
        best_i = torch.empty(0, dtype=torch.int64, device=dev)
        for lo in range(0, left.numel(), batch_size):   # running top-k over blocks of left rows
            S = _pair_sim(self.emb[left[lo:lo + batch_size]], self.emb[right], self.sfunc).reshape(-1)
            best_s = torch.cat([best_s, S])
            best_i = torch.cat([best_i, torch.arange(S.numel(), device=dev) + lo * right.numel()])
            if best_s.numel() > k:
                top = torch.topk(best_s, k)
                best_s, best_i = top.values, best_i[top.indices]
        order = torch.argsort(best_s, descending=True, stable=True)
        best_s, best_i = best_s[order], best_i[order]
        return [(left[best_i // right.numel()], right[best_i % right.numel()], best_s)]

    topK = topk


class KGEModel:
    """A trained model as an object: embeddings, optional graph, ``link_predict`` and ``embed_sim``."""

    def __init__(self, device="cpu", model_name: str = "TransE_l2", gamma: float = 12.0):
        self._device, self._model_name, self._gamma = torch.device(device), model_name, gamma
        self._entity: Optional[torch.Tensor] = None
        self._relation: Optional[torch.Tensor] = None
        self._projection: Optional[torch.Tensor] = None
        self._graph: Optional[Tuple[np.ndarray, np.ndarray, np.ndarray]] = None

    # ------------------------------------------------------------------ state
    def load(self, model_path: str, entity_file: Optional[str] = None, relation_file: Optional[str] = None) -> "KGEModel":
        """Reads the embeddings of ``model_path``: the files ``config.json`` names when it is there (the trainers write
        it), else ``entity.npy`` / ``relation.npy``, or the names given."""
        cfg_file = os.path.join(model_path, "config.json")
        c = json.load(open(cfg_file)) if os.path.exists(cfg_file) else {}
        ef = entity_file or c.get("emp_file", "entity.npy")
        rf = relation_file or c.get("rmap_file", "relation.npy")
        self._entity = torch.from_numpy(np.load(os.path.join(model_path, ef)))
        self._relation = torch.from_numpy(np.load(os.path.join(model_path, rf)))
        pf = os.path.join(model_path, ef.replace("_entity.npy", "projection.npy"))
        self._projection = torch.from_numpy(np.load(pf)) if pf != os.path.join(model_path, ef) and os.path.exists(pf) else None
        if "gamma" in c:
            self._gamma = float(c["gamma"])
        name = c.get("model_name", c.get("model"))
        if name:
            self._model_name = name
        return self

    def set_embeddings(self, entity: torch.Tensor, relation: torch.Tensor, projection: Optional[torch.Tensor] = None) -> "KGEModel":
        self._entity, self._relation, self._projection = entity, relation, projection
        return self

    def attach_graph(self, head, rel, tail) -> None:
        """The known triples, needed by ``link_predict(exclude_mode=...)``."""
        self._graph = tuple(np.asarray(x, dtype=np.int64).reshape(-1) for x in (head, rel, tail))

    def save(self, model_path: str) -> None:
        raise NotImplementedError("a model object is for inference; the trainers write the checkpoints")

    model_name = property(lambda self: self._model_name)
    entity_embed = property(lambda self: self._entity)
    relation_embed = property(lambda self: self._relation)
    num_entity = property(lambda self: -1 if self._entity is None else self._entity.shape[0])
    num_rel = property(lambda self: -1 if self._relation is None else self._relation.shape[0])
    graph = property(lambda self: self._graph)

    # ------------------------------------------------------------------ queries
    def link_predict(self, head=None, rel=None, tail=None, exec_mode: str = "all", sfunc: str = "none", topk: int = 10,
                     exclude_mode: Optional[str] = None, batch_size: int = DEFAULT_INFER_BATCH):
        """A list of ``(head, rel, tail, score)`` (``exclude_mode="mask"``: plus the mask of existing triples), best
        first; one entry for ``all`` / ``triplet_wise``, one per element for the ``batch_*`` modes."""
        assert self._entity is not None, "load() or set_embeddings() first"
        assert exclude_mode is None or self._graph is not None, "exclude_mode needs attach_graph(head, rel, tail)"
        inf = ScoreInfer(self._model_name, self._entity, self._relation, self._gamma, self._device, self._projection, sfunc)
        if exclude_mode is not None:
            inf.attach_graph(*self._graph)
        return inf.topk(head, rel, tail, topk, exec_mode, exclude_mode, batch_size)

    def embed_sim(self, left=None, right=None, embed_type: str = "entity", sfunc: str = "cosine", bcast: bool = False,
                  pair_ws: bool = False, topk: int = 10):
        assert embed_type in ("entity", "relation"), embed_type
        emb = self._entity if embed_type == "entity" else self._relation
        assert emb is not None, "load() or set_embeddings() first"
        return EmbSimInfer(emb, sfunc, self._device).topk(left, right, topk, pair_ws, bcast)


def _model_class(name: str, model_name: str):
    def __init__(self, device="cpu", gamma: float = 12.0):
        KGEModel.__init__(self, device, model_name, gamma)
    return type(name, (KGEModel,), {"__init__": __init__, "__doc__": f"``KGEModel`` with the {model_name} score function."})


TransEModel = _model_class("TransEModel", "TransE")
TransE_l2Model = _model_class("TransE_l2Model", "TransE_l2")
TransE_l1Model = _model_class("TransE_l1Model", "TransE_l1")
TransRModel = _model_class("TransRModel", "TransR")
DistMultModel = _model_class("DistMultModel", "DistMult")
ComplExModel = _model_class("ComplExModel", "ComplEx")
RESCALModel = _model_class("RESCALModel", "RESCAL")
RotatEModel = _model_class("RotatEModel", "RotatE")
SimplEModel = _model_class("SimplEModel", "SimplE")
