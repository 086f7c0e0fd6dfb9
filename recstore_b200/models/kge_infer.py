"""Inference over trained knowledge-graph embeddings: top-k triple scoring and embedding similarity.

* ``ScoreInfer.topk(head, rel, tail, k, exec_mode)`` ranks candidate triples by a model's score function
  (``all``: every head x rel x tail combination; ``triplet_wise``: aligned lists; ``batch_head`` / ``batch_rel`` /
  ``batch_tail``: one top-k list per element of that argument) -- the modes of the reference's ``ScoreInfer``
  (src/kg/kg/dgl-ke/python/dglke/models/infer.py:24-252).
* ``EmbSimInfer.topk(left, right, k, pair_ws, bcast)`` ranks entity pairs by ``cosine`` / ``l2`` / ``l1`` / ``dot`` /
  ``ext_jaccard`` similarity (infer.py:254-402).

Both load the ``.npy`` + ``config.json`` checkpoints written by the trainers, or take tensors directly.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Tuple

import numpy as np
import torch

from ..baseline.kge_torch import edge_score


class ScoreInfer:
    def __init__(self, model_name: str, entity: torch.Tensor, relation: torch.Tensor, gamma: float = 12.0, device="cpu",
                 projection: Optional[torch.Tensor] = None):
        self.model, self.gamma, self.dev = model_name, gamma, torch.device(device)
        self.entity, self.relation = entity.to(self.dev), relation.to(self.dev)
        # TransR / RESCAL: one matrix per relation, stored flat (tensor_models.py:188-199 reads the same file)
        self.projection = projection.to(self.dev) if projection is not None else None
        assert self.projection is not None or model_name not in ("TransR", "RESCAL"), f"{model_name} needs its projection matrices"
        self.emb_init = (gamma + 2.0) / entity.shape[1]

    @staticmethod
    def load(path: str, device="cpu") -> "ScoreInfer":
        with open(os.path.join(path, "config.json")) as f:
            c = json.load(f)
        ent = torch.from_numpy(np.load(os.path.join(path, c["emp_file"])))
        rel = torch.from_numpy(np.load(os.path.join(path, c["rmap_file"])))
        name = c.get("model_name", c.get("model"))
        pfile = os.path.join(path, c["emp_file"].replace("_entity.npy", "projection.npy"))
        proj = torch.from_numpy(np.load(pfile)) if os.path.exists(pfile) else None
        return ScoreInfer(name, ent, rel, float(c.get("gamma", 12.0)), device, projection=proj)

    def _score(self, h, r, t) -> torch.Tensor:
        proj = self.projection[r] if self.projection is not None else None
        return edge_score(self.model, self.entity[h], self.relation[r], self.entity[t], self.gamma, proj, self.emb_init)

    def topk(self, head=None, rel=None, tail=None, k: int = 10, exec_mode: str = "all") -> List[Tuple[torch.Tensor, ...]]:
        """Each result is ``(head_ids, rel_ids, tail_ids, scores)`` sorted by decreasing score.  ``None`` = all ids."""
        ar = lambda x, n: torch.arange(n, device=self.dev) if x is None else torch.as_tensor(x, dtype=torch.int64, device=self.dev)
        head, rel, tail = ar(head, self.entity.shape[0]), ar(rel, self.relation.shape[0]), ar(tail, self.entity.shape[0])
        if exec_mode == "triplet_wise":
            assert head.numel() == rel.numel() == tail.numel()
            s = self._score(head, rel, tail)
            top = torch.topk(s, min(k, s.numel()))
            i = top.indices
            return [(head[i], rel[i], tail[i], top.values)]

        def grid(h, r, t):
            H, R, T = torch.meshgrid(h, r, t, indexing="ij")
            H, R, T = H.reshape(-1), R.reshape(-1), T.reshape(-1)
            s = self._score(H, R, T)
            top = torch.topk(s, min(k, s.numel()))
            i = top.indices
            return H[i], R[i], T[i], top.values
        if exec_mode == "all":
            return [grid(head, rel, tail)]
        if exec_mode == "batch_head":
            return [grid(head[i:i + 1], rel, tail) for i in range(head.numel())]
        if exec_mode == "batch_rel":
            return [grid(head, rel[i:i + 1], tail) for i in range(rel.numel())]
        if exec_mode == "batch_tail":
            return [grid(head, rel, tail[i:i + 1]) for i in range(tail.numel())]
        raise ValueError(exec_mode)


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


class EmbSimInfer:
    def __init__(self, emb: torch.Tensor, sfunc: str = "cosine", device="cpu"):
        self.emb, self.sfunc = emb.to(device), sfunc

    def topk(self, left=None, right=None, k: int = 10, pair_ws: bool = False, bcast: bool = False):
        n = self.emb.shape[0]
        ar = lambda x: torch.arange(n, device=self.emb.device) if x is None else torch.as_tensor(x, dtype=torch.int64, device=self.emb.device)
        left, right = ar(left), ar(right)
        if pair_ws:                                    # aligned pairs
            assert left.numel() == right.numel()
            s = torch.stack([_pair_sim(self.emb[l:l + 1], self.emb[r:r + 1], self.sfunc)[0, 0] for l, r in zip(left.tolist(), right.tolist())])
            top = torch.topk(s, min(k, s.numel()))
            return [(left[top.indices], right[top.indices], top.values)]
        S = _pair_sim(self.emb[left], self.emb[right], self.sfunc)
        if bcast:                                      # one list per left id
            top = torch.topk(S, min(k, S.shape[1]), dim=1)
            return [(left[i].expand(top.indices.shape[1]), right[top.indices[i]], top.values[i]) for i in range(left.numel())]
        top = torch.topk(S.reshape(-1), min(k, S.numel()))
        return [(left[top.indices // right.numel()], right[top.indices % right.numel()], top.values)]
