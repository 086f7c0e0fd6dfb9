"""Knowledge-graph embedding models in plain PyTorch: every score function, chunked negatives, trainer.

This is the oracle for the native KG kernels and the CPU path of the KG driver.  Score functions and their
chunked-negative forms follow the reference's DGL-KE (src/kg/kg/dgl-ke/python/dglke/models/pytorch/score_fun.py:
TransE l1/l2 :40-108, TransR :110-220, DistMult :222-286, ComplEx :288-368, RESCAL :370-438, RotatE :440-538,
SimplE :540-641); loss = log-sigmoid (loss.py:69-99); embeddings trained with row-wise sparse Adagrad
(tensor_models.py:366-436); init U(+-(gamma + 2) / dim) (general_models.py:223-224).

Layouts: ComplEx and RotatE entities are ``[re | im]`` halves; RotatE relations are ``dim / 2`` phases scaled by
``pi / emb_init``; SimplE entities are ``[head role | tail role]`` and relations ``[r | r_inv]``; TransR / RESCAL
relations carry a ``dim x rel_dim`` (``dim x dim``) matrix in a second table.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

MODEL_NAMES = ("TransE", "TransE_l1", "TransE_l2", "TransR", "DistMult", "ComplEx", "RESCAL", "RotatE", "SimplE")


def relation_dim(model: str, dim: int) -> int:
    return dim // 2 if model == "RotatE" else dim


def projection_dim(model: str, dim: int, rel_dim: Optional[int] = None) -> int:
    """Floats per relation in the second (matrix) table; 0 if the model has none."""
    if model == "TransR":
        return dim * (rel_dim or dim)
    if model == "RESCAL":
        return dim * dim
    return 0


def _rotate_rel(r: torch.Tensor, emb_init: float) -> Tuple[torch.Tensor, torch.Tensor]:
    phase = r / (emb_init / math.pi)
    return torch.cos(phase), torch.sin(phase)


def edge_score(model: str, h: torch.Tensor, r: torch.Tensor, t: torch.Tensor, gamma: float, proj: Optional[torch.Tensor] = None,
               emb_init: float = 1.0) -> torch.Tensor:
    """Score of aligned triples: ``h, t`` ``[n, dim]``, ``r`` ``[n, rel_dim]`` -> ``[n]``."""
    if model in ("TransE", "TransE_l2"):
        return gamma - torch.sqrt(((h + r - t) ** 2).sum(-1).clamp_min(1e-30))
    if model == "TransE_l1":
        return gamma - (h + r - t).abs().sum(-1)
    if model == "DistMult":
        return (h * r * t).sum(-1)
    if model == "ComplEx":
        hr, hi = h.chunk(2, -1); tr, ti = t.chunk(2, -1); rr, ri = r.chunk(2, -1)
        return (hr * tr * rr + hi * ti * rr + hr * ti * ri - hi * tr * ri).sum(-1)
    if model == "RotatE":
        hr, hi = h.chunk(2, -1); tr, ti = t.chunk(2, -1)
        c, s = _rotate_rel(r, emb_init)
        dr, di = hr * c - hi * s - tr, hr * s + hi * c - ti
        return gamma - torch.sqrt(dr * dr + di * di).sum(-1)
    if model == "SimplE":
        h_i, h_j = h.chunk(2, -1); t_i, t_j = t.chunk(2, -1); rel, rinv = r.chunk(2, -1)
        return (((h_i * rel * t_j).sum(-1) + (t_i * rinv * h_j).sum(-1)) / 2).clamp(-20, 20)
    if model == "TransR":
        d = h.shape[-1]
        M = proj.view(h.shape[0], d, -1)
        hp, tp = torch.einsum("nd,ndk->nk", h, M), torch.einsum("nd,ndk->nk", t, M)
        return gamma - (hp + r - tp).abs().sum(-1)
    if model == "RESCAL":
        d = h.shape[-1]
        M = proj.view(h.shape[0], d, d)
        return (h * torch.einsum("nij,nj->ni", M, t)).sum(-1)
    raise ValueError(model)


def chunk_neg_score(model: str, h, r, t, neg, corrupt_head: bool, chunk: int, gamma: float, proj=None, emb_init: float = 1.0):
    """Scores of every positive against the ``ns`` negatives shared by its chunk: ``h, r, t`` ``[bs, .]``, ``neg``
    ``[bs / chunk * ns, dim]`` -> ``[bs, ns]``.  Written as the per-pair definition (broadcast), which is what the
    bmm forms of the reference compute."""
    bs, d = h.shape
    C = bs // chunk
    ns = neg.shape[0] // C
    # The two models of the headline benchmarks in the batched-GEMM form the reference uses for them
    # (score_fun.py:61-108 TransE create_neg with baddbmm / cdist, :268-286 DistMult create_neg with bmm); the per-pair
    # form below is their definition and the oracle of the tests.
    if model == "DistMult" and proj is None:
        a = (t * r) if corrupt_head else (h * r)
        return torch.bmm(a.view(C, chunk, d), neg.view(C, ns, d).transpose(1, 2)).reshape(bs, ns)
    if model in ("TransE", "TransE_l2") and proj is None:
        a = (t - r) if corrupt_head else (h + r)
        return (gamma - torch.cdist(a.view(C, chunk, d), neg.view(C, ns, d), p=2.0)).reshape(bs, ns)
    n = neg.view(C, 1, ns, d).expand(C, chunk, ns, d).reshape(bs * ns, d)
    rep = lambda x: None if x is None else x.unsqueeze(1).expand(bs, ns, x.shape[-1]).reshape(bs * ns, -1)
    hh, tt = (n, rep(t)) if corrupt_head else (rep(h), n)
    return edge_score(model, hh, rep(r), tt, gamma, rep(proj), emb_init).view(bs, ns)


def logsigmoid_loss(pos: torch.Tensor, neg: torch.Tensor) -> torch.Tensor:
    return (-F.logsigmoid(pos).mean() - F.logsigmoid(-neg).mean()) / 2


LOSS_GENRES = ("Logsigmoid", "Logistic", "Hinge", "BCE")


def kg_loss(pos: torch.Tensor, neg: torch.Tensor, genre: str = "Logsigmoid", margin: float = 1.0, adversarial: bool = False,
            temperature: float = 1.0, edge_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Loss over positive scores ``[bs]`` and negative scores ``[bs, ns]`` (loss.py:10-99 of the reference): a criterion
    applied with label +1 to positives and -1 (0 for BCE) to negatives, negatives averaged per positive -- or weighted by
    ``softmax(neg * temperature)`` (self-adversarial sampling, weights not differentiated) -- then
    ``(mean(pos part) + mean(neg part)) / 2``.  ``edge_weight`` ``[bs]`` scales both parts per positive."""
    if genre == "Logsigmoid":
        crit = lambda x, y: -F.logsigmoid(y * x)
        neg_label = -1.0
    elif genre == "Logistic":
        crit = lambda x, y: F.softplus(-y * x)
        neg_label = -1.0
    elif genre == "Hinge":
        crit = lambda x, y: (margin - y * x).clamp_min(0)
        neg_label = -1.0
    elif genre == "BCE":
        crit = lambda x, y: -(y * F.logsigmoid(x) + (1 - y) * F.logsigmoid(-x))     # log(1 - sigmoid(x)) = logsigmoid(-x)
        neg_label = 0.0
    else:
        raise ValueError(f"loss genre {genre!r} is not supported; one of {LOSS_GENRES}")
    pl, nl = crit(pos, 1.0), crit(neg, neg_label)
    if edge_weight is not None:
        pl, nl = pl * edge_weight, nl * edge_weight.view(-1, 1)
    if adversarial:
        nl = (torch.softmax(neg * temperature, dim=-1).detach() * nl).sum(-1)
    else:
        nl = nl.mean(-1)
    return (pl.mean() + nl.mean()) / 2


def rowwise_adagrad_(weight: torch.Tensor, state: torch.Tensor, ids: torch.Tensor, grad: torch.Tensor, lr: float, eps: float = 1e-10):
    """The reference's sparse row-wise Adagrad (tensor_models.py:398-430 ``ExternalEmbedding.update``), duplicates
    allowed: ``state[id] += mean_d(g^2)`` for every occurrence, then every occurrence moves its row by
    ``-lr * g / (sqrt(state[id]) + eps)`` with the state AFTER all of the step's occurrences were added."""
    state.index_add_(0, ids, (grad * grad).mean(1))
    std = state[ids].sqrt().add_(eps).unsqueeze(1)
    weight.index_add_(0, ids, -lr * grad / std)


class TorchKGE:
    """Dense entity / relation tables on one device, trained like the reference's stock path."""

    def __init__(self, n_entities: int, n_relations: int, dim: int, model: str = "TransE_l2", gamma: float = 12.0,
                 lr: float = 0.1, device="cpu", seed: int = 0, rel_dim: Optional[int] = None, neg_chunk_size: int = 0,
                 loss_genre: str = "Logsigmoid", margin: float = 1.0, neg_adversarial_sampling: bool = False,
                 adversarial_temperature: float = 1.0, regularization_coef: float = 0.0, regularization_norm: int = 3):
        assert model in MODEL_NAMES, model
        assert loss_genre in LOSS_GENRES, loss_genre
        self.loss_cfg = dict(genre=loss_genre, margin=margin, adversarial=neg_adversarial_sampling, temperature=adversarial_temperature)
        self.reg_coef, self.reg_norm = regularization_coef, regularization_norm
        self.model, self.dim, self.gamma, self.lr, self.device = model, dim, gamma, lr, torch.device(device)
        self.emb_init = (gamma + 2.0) / dim
        g = torch.Generator().manual_seed(seed)
        u = lambda n, d: ((torch.rand(n, d, generator=g) * 2 - 1) * self.emb_init).to(self.device)
        self.rel_dim = relation_dim(model, rel_dim or dim)
        self.entity, self.relation = u(n_entities, dim), u(n_relations, self.rel_dim)
        pd = projection_dim(model, dim, rel_dim)
        self.proj = u(n_relations, pd) if pd else None
        self.state: Dict[str, torch.Tensor] = {"entity": torch.zeros(n_entities, device=self.device),
                                               "relation": torch.zeros(n_relations, device=self.device)}
        if self.proj is not None:
            self.state["proj"] = torch.zeros(n_relations, device=self.device)
        self.step_no = 0
        self._async_q = None
        self._async_thread = None
        self._async_error: Optional[BaseException] = None

    # Asynchronous entity update: the trainer hands (ids, gradients) of a step to a worker that applies the sparse
    # Adagrad update while the next step already computes, so a step may read rows whose last update is still queued
    # (the reference's --async_update: tensor_models.py:144-182 async_update, 433-447 create / finish).  Relations
    # stay synchronous, as there.  The queue is bounded: a trainer that runs ahead of the updater blocks.
    def create_async_update(self, max_pending: int = 4) -> None:
        import queue
        import threading
        if self._async_thread is not None:
            return
        self._async_q = queue.Queue(maxsize=max_pending)

        def run():
            while True:
                item = self._async_q.get()
                if item is None:
                    return
                try:
                    with torch.no_grad():
                        ids, grads = item
                        rowwise_adagrad_(self.entity, self.state["entity"], ids.to(self.device), grads.to(self.device), self.lr)
                except BaseException as e:      # noqa: BLE001 - surfaces in the trainer at its next step / at finish
                    self._async_error = e
                    return
                finally:
                    self._async_q.task_done()
        self._async_thread = threading.Thread(target=run, name="kge-async-update", daemon=True)
        self._async_thread.start()

    def wait_async_update(self) -> None:
        """Blocks until every queued update has been applied (before evaluation or a checkpoint)."""
        if self._async_thread is not None and self._async_error is None:
            self._async_q.join()
        if self._async_error is not None:
            raise RuntimeError("asynchronous entity update failed") from self._async_error

    def finish_async_update(self) -> None:
        if self._async_thread is None:
            return
        try:
            self.wait_async_update()
        finally:
            if self._async_thread.is_alive():
                self._async_q.put(None)
            self._async_thread.join(timeout=30)
            self._async_thread, self._async_q = None, None

    def _rows(self, h_ids, r_ids, t_ids, neg_ids):
        rows = [self.entity[h_ids].clone().requires_grad_(True), self.relation[r_ids].clone().requires_grad_(True),
                self.entity[t_ids].clone().requires_grad_(True), self.entity[neg_ids].clone().requires_grad_(True)]
        p = self.proj[r_ids].clone().requires_grad_(True) if self.proj is not None else None
        return rows, p

    def scores(self, h_ids, r_ids, t_ids, neg_ids, corrupt_head: bool, chunk: int):
        (h, r, t, n), p = self._rows(h_ids, r_ids, t_ids, neg_ids)
        pos = edge_score(self.model, h, r, t, self.gamma, p, self.emb_init)
        neg = chunk_neg_score(self.model, h, r, t, n, corrupt_head, chunk, self.gamma, p, self.emb_init)
        return pos, neg, (h, r, t, n, p)

    def train_step(self, h_ids, r_ids, t_ids, neg_ids, chunk: int, corrupt_head: Optional[bool] = None,
                   edge_weight: Optional[torch.Tensor] = None) -> float:
        if corrupt_head is None:
            corrupt_head = bool(self.step_no & 1)
        self.step_no += 1
        pos, neg, (h, r, t, n, p) = self.scores(h_ids, r_ids, t_ids, neg_ids, corrupt_head, chunk)
        loss = kg_loss(pos, neg, edge_weight=edge_weight, **self.loss_cfg)
        if self.reg_coef > 0.0 and self.reg_norm > 0:          # on the rows of this batch (general_models.py:623-629)
            loss = loss + self.reg_coef * (torch.cat([h, t, n]).norm(p=self.reg_norm) + r.norm(p=self.reg_norm))
        loss.backward()
        with torch.no_grad():
            ids = torch.cat([h_ids, t_ids, neg_ids])
            if self._async_thread is not None:
                if self._async_error is not None:
                    raise RuntimeError("asynchronous entity update failed") from self._async_error
                self._async_q.put((ids.clone(), torch.cat([h.grad, t.grad, n.grad])))
            else:
                rowwise_adagrad_(self.entity, self.state["entity"], ids, torch.cat([h.grad, t.grad, n.grad]), self.lr)
            if r.grad is not None:      # RESCAL scores with the relation matrix only
                rowwise_adagrad_(self.relation, self.state["relation"], r_ids, r.grad, self.lr)
            if p is not None:
                rowwise_adagrad_(self.proj, self.state["proj"], r_ids, p.grad, self.lr)
        return loss.item()

    @torch.no_grad()
    def evaluate(self, h_ids, r_ids, t_ids, n_neg: int = 256, generator: Optional[torch.Generator] = None,
                 neg_prob: Optional[torch.Tensor] = None) -> Dict[str, float]:
        """Rank of each positive among ``n_neg`` sampled corruptions of its head and of its tail; ``neg_prob``
        (``[n_entities]``, e.g. proportional to degree: ``--neg_deg_sample_eval``) replaces the uniform draw."""
        bs = h_ids.numel()
        ranks = []
        for corrupt_head in (False, True):
            if neg_prob is None:
                neg_ids = torch.randint(0, self.entity.shape[0], (n_neg,), generator=generator).to(self.device)
            else:
                neg_ids = torch.multinomial(neg_prob.cpu(), n_neg, replacement=True, generator=generator).to(self.device)
            p = self.proj[r_ids] if self.proj is not None else None
            pos = edge_score(self.model, self.entity[h_ids], self.relation[r_ids], self.entity[t_ids], self.gamma, p, self.emb_init)
            neg = chunk_neg_score(self.model, self.entity[h_ids], self.relation[r_ids], self.entity[t_ids], self.entity[neg_ids],
                                  corrupt_head, bs, self.gamma, p, self.emb_init)
            ranks.append(1 + (neg >= pos.unsqueeze(1)).sum(1))
        r = torch.cat(ranks).float()
        return {"MRR": (1.0 / r).mean().item(), "MR": r.mean().item(), "HITS@1": (r <= 1).float().mean().item(),
                "HITS@3": (r <= 3).float().mean().item(), "HITS@10": (r <= 10).float().mean().item()}

    @torch.no_grad()
    def evaluate_full(self, h_ids, r_ids, t_ids, known: Optional[Dict[str, Dict[tuple, torch.Tensor]]] = None,
                      batch: int = 64) -> Dict[str, float]:
        """Ranks every test triple against ALL entities as corrupted tails and as corrupted heads (the reference's full
        evaluation, ``neg_sample_size_eval = -1``).  ``known`` = :func:`known_triple_index` of every true triple turns on
        the filtered setting: other true answers are taken out of the candidate list (the default of the reference;
        ``--no_eval_filter`` switches it off)."""
        n_ent = self.entity.shape[0]
        allent = self.entity
        ranks = []
        for lo in range(0, h_ids.numel(), batch):
            h, r, t = h_ids[lo:lo + batch], r_ids[lo:lo + batch], t_ids[lo:lo + batch]
            bs = h.numel()
            p = self.proj[r] if self.proj is not None else None
            he, re, te = self.entity[h], self.relation[r], self.entity[t]
            pos = edge_score(self.model, he, re, te, self.gamma, p, self.emb_init)
            for corrupt_head in (False, True):
                sc = chunk_neg_score(self.model, he, re, te, allent, corrupt_head, bs, self.gamma, p, self.emb_init)   # [bs, n_ent]
                if known is not None:
                    table = known["heads" if corrupt_head else "tails"]
                    for i in range(bs):
                        key = (int(r[i]), int(t[i])) if corrupt_head else (int(h[i]), int(r[i]))
                        others = table.get(key)
                        if others is not None:
                            sc[i, others.to(sc.device)] = float("-inf")
                truth = h if corrupt_head else t
                sc[torch.arange(bs), truth] = float("-inf")              # the positive itself is compared through `pos`
                ranks.append(1 + (sc > pos.unsqueeze(1)).sum(1))
        r_ = torch.cat(ranks).float()
        return {"MRR": (1.0 / r_).mean().item(), "MR": r_.mean().item(), "HITS@1": (r_ <= 1).float().mean().item(),
                "HITS@3": (r_ <= 3).float().mean().item(), "HITS@10": (r_ <= 10).float().mean().item(), "candidates": n_ent}


def known_triple_index(*splits) -> Dict[str, Dict[tuple, torch.Tensor]]:
    """``{"tails": {(h, r): tensor of true tails}, "heads": {(r, t): tensor of true heads}}`` over the given
    ``(head, rel, tail)`` splits (train, valid, test): the filter of the filtered ranking metrics."""
    tails: Dict[tuple, list] = {}
    heads: Dict[tuple, list] = {}
    for sp in splits:
        if sp is None:
            continue
        h, r, t = (torch.as_tensor(x).tolist() for x in sp)
        for a, b, c in zip(h, r, t):
            tails.setdefault((a, b), []).append(c)
            heads.setdefault((b, c), []).append(a)
    return {"tails": {k: torch.tensor(sorted(set(v)), dtype=torch.int64) for k, v in tails.items()},
            "heads": {k: torch.tensor(sorted(set(v)), dtype=torch.int64) for k, v in heads.items()}}
