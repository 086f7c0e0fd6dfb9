"""Knowledge-graph embedding training (TransE L2 / L1, DistMult, ComplEx, SimplE, RotatE, RESCAL) on row-sharded HBM tables.

Model, negative sampling and loss follow the reference's patched DGL-KE
(src/kg/kg/dgl-ke/python/dglke/models/general_models.py:568-631, score_fun.py, loss.py:69-99,
sampler.py:703-818): a batch of ``batch`` positives per GPU is cut into chunks of ``neg_chunk_size``, each
chunk shares ``neg_sample_size`` uniformly drawn negative entities, corrupt-head and corrupt-tail
batches alternate, the loss is the log-sigmoid loss, and embeddings are trained with row-wise sparse
Adagrad (tensor_models.py:366-436).  Init is ``U(+-(gamma + 2) / dim)`` (general_models.py:223-224).

What is different: the entity table (86 M x 400 fp32 = 138 GB in the headline config) does not live in
host memory behind a cache; it is spread cyclically over the GPUs' HBM
(``parallel.sharded_table.ShardedEmbeddingTable``), rows and gradients move by peer stores, and the
scoring is three element-wise kernels around tcgen05 GEMMs for the models whose negative scores are cross
products (TransE-L2, DistMult, ComplEx, SimplE) and three pair-walking fp32 kernels for TransE-L1 and RotatE
(``csrc/ops/kge.cu``).  RESCAL (score h^T M_r t, score_fun.py:378-449) is in the GEMM family too: a = M_r^T h or M_r t is
a matrix-vector product per positive, the negatives' scores are a . e'.  Its relation table is ROW-BLOCKED: relation r
owns the D table rows r*D .. r*D+D-1 (the rows of its D x D matrix), and every row is updated with the squared norm of
the whole matrix gradient / D, so that all D rows carry the same Adagrad accumulator: one state per relation, as the
reference's [n_relations, D*D] embedding has.  TransR (score gamma - |h M_r + r - t M_r|_1, score_fun.py:110-220) projects
every negative with the matrix of every positive of its chunk, a batched [ns x D] x [D x D] product per positive: its
tables live on the same sharded HBM plane (entities, relation vectors, a row-blocked projection table), and the scoring
between lookup and update is PyTorch autograd over ``torch.einsum`` / cuBLAS batched GEMMs (plain library GEMMs; there is
no fused kernel for it).

Checkpoints keep the reference layout (tensor_models.py:452-476, general_models.py:316-346):
``{dataset}_{model}_entity.npy``, ``{dataset}_{model}_relation.npy`` and ``config.json``.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .. import _lib
from .._lib import f32, i32, ptr, stream_ptr, vp
from ..ops import functional as F_
from ..parallel.peer import PeerContext
from ..parallel.sharded_table import ShardedEmbeddingTable

_lib.register_signatures({
    "rs_kge_stage": (i32, [i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp,
                           vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
})

MODELS = {"TransE": 0, "TransE_l2": 0, "DistMult": 1, "ComplEx": 2, "SimplE": 3, "TransE_l1": 4, "RotatE": 5, "RESCAL": 6,
          "TransR": 7}                # 7: tables on the HBM plane, scoring by autograd over batched library GEMMs
PAIRWISE = (4, 5)                     # no cross-product form: scored pair by pair in fp32


@dataclass
class KGEConfig:
    n_entities: int
    n_relations: int
    dim: int = 400
    model: str = "TransE_l2"
    gamma: float = 10.0
    batch: int = 1024                 # positives per GPU and step
    neg_sample_size: int = 256
    neg_chunk_size: int = 256
    lr: float = 0.1
    eps: float = 1e-10
    seed: int = 0
    dataset: str = "synthetic"
    entity_hbm_ratio: float = 1.0     # < 1: that share of every entity shard stays in HBM (low ids), the rest in pinned host memory
    use_cuda_graph: bool = False      # capture the step (one graph per corruption side) and replay it: ~40 launches per step
    tf32_scoring: bool = False        # TransR: run its batched fp32 GEMMs with TF32 tensor-core math (10-bit mantissa products)


class KGEModel:
    def __init__(self, cfg: KGEConfig, ctx: Optional[PeerContext] = None):
        if cfg.model not in MODELS:
            raise ValueError(f"unsupported model {cfg.model!r}; available: {sorted(MODELS)}")
        assert cfg.batch % cfg.neg_chunk_size == 0, "the batch is cut into whole chunks (reference rounds it up, utils.py:27-33)"
        assert cfg.dim % 4 == 0
        self.cfg = cfg
        self.ctx = ctx if ctx is not None else PeerContext(0, 1)
        dev = self.dev = self.ctx.device
        self.bs, self.cs, self.ns, self.D = cfg.batch, cfg.neg_chunk_size, cfg.neg_sample_size, cfg.dim
        self.C = self.bs // self.cs
        self.nneg = self.C * self.ns
        self.Dp = (self.D + 63) // 64 * 64
        self.model_id = MODELS[cfg.model]
        self.pairwise = self.model_id in PAIRWISE
        self.rescal = cfg.model == "RESCAL"
        self.transr = cfg.model == "TransR"
        if self.transr:
            assert not cfg.use_cuda_graph, "TransR scores through autograd: no graph replay"
        self.Dr = self.D // 2 if cfg.model == "RotatE" else self.D      # RotatE relations are phases
        if self.rescal:
            assert self.D <= 512, "RESCAL: dim <= 512"
            self.Dr = self.D * self.D                                    # a row-major D x D matrix per relation
        if self.pairwise:
            assert self.cs % 8 == 0 and self.ns % 8 == 0, "TransE_l1 / RotatE: chunk and negative counts are multiples of 8"
        scale = self.emb_init = (cfg.gamma + 2.0) / cfg.dim
        n_ids = 2 * self.bs + self.nneg
        self.entity = ShardedEmbeddingTable(self.ctx, "kge_entity", cfg.n_entities, self.D, max_keys=n_ids, lr=cfg.lr, eps=cfg.eps,
                                            init="uniform", init_scale=scale, seed=cfg.seed, hbm_ratio=cfg.entity_hbm_ratio)
        if self.rescal:   # row-blocked: D table rows of D floats per relation
            self.relation = ShardedEmbeddingTable(self.ctx, "kge_relation", cfg.n_relations * self.D, self.D, max_keys=self.bs * self.D,
                                                  lr=cfg.lr, eps=cfg.eps, init="uniform", init_scale=scale, seed=cfg.seed + 1)
            self._row_of_block = torch.arange(self.D, dtype=torch.int64, device=dev)
        elif self.transr:  # relation vectors, and a row-blocked table of D x D projection matrices (D rows per relation)
            self.relation = ShardedEmbeddingTable(self.ctx, "kge_relation", cfg.n_relations, self.Dr, max_keys=self.bs, lr=cfg.lr,
                                                  eps=cfg.eps, init="uniform", init_scale=scale, seed=cfg.seed + 1)
            self.proj = ShardedEmbeddingTable(self.ctx, "kge_proj", cfg.n_relations * self.D, self.Dr, max_keys=self.bs * self.D,
                                              lr=cfg.lr, eps=cfg.eps, init="uniform", init_scale=scale, seed=cfg.seed + 2)
            self._row_of_block = torch.arange(self.D, dtype=torch.int64, device=dev)
        else:
            self.relation = ShardedEmbeddingTable(self.ctx, "kge_relation", cfg.n_relations, self.Dr, max_keys=self.bs, lr=cfg.lr,
                                                  eps=cfg.eps, init="uniform", init_scale=scale, seed=cfg.seed + 1)
        f = dict(dtype=torch.float32, device=dev)
        b = dict(dtype=torch.bfloat16, device=dev)
        self.ent_rows = torch.empty(n_ids, self.D, **f)
        self.rel_rows = torch.empty(self.bs, self.Dr, **f)
        self.ent_grad = torch.empty(n_ids, self.D, **f)
        self.rel_grad = torch.empty(self.bs, self.Dr, **f)
        if self.rescal or self.transr:
            self._rel_keys = torch.empty(self.bs * self.D, dtype=torch.int64, device=dev)
            self._rel_norm = torch.empty(self.bs * self.D, **f)
        if self.transr:
            self.proj_rows = torch.empty(self.bs * self.D, self.Dr, **f)
            self.proj_grad = torch.empty(self.bs * self.D, self.Dr, **f)
        self.A = torch.zeros(self.bs, self.Dp, **b)
        self.Bn = torch.zeros(self.nneg, self.Dp, **b)
        self.a2 = torch.empty(self.bs, **f)
        self.b2 = torch.empty(self.nneg, **f)
        self.S = torch.empty(self.bs, self.nneg, **f)
        self.W = torch.empty(self.bs, self.nneg, **b)
        self.rowsum = torch.empty(self.bs, **f)
        self.colsum = torch.empty(self.nneg, **f)
        self.GA = torch.empty(self.bs, self.Dp, **f)
        self.GB = torch.empty(self.nneg, self.Dp, **f)
        self.loss = torch.zeros(2, **f)
        self.pos_score = torch.empty(self.bs, **f)
        self.neg_score = torch.empty(self.bs, self.ns, **f)
        self.ids = torch.empty(n_ids, dtype=torch.int64, device=dev)
        self.step_no = 0
        self.heartbeat = None                # utils/liveness.Heartbeat: checked on the host before every step when set
        self.heartbeat_timeout_s = 2.0
        self.launches_per_step = 0
        self._graphs: Dict[bool, torch.cuda.CUDAGraph] = {}
        self._g_ids = (torch.zeros(self.bs, dtype=torch.int64, device=dev), torch.zeros(self.bs, dtype=torch.int64, device=dev),
                       torch.zeros(self.bs, dtype=torch.int64, device=dev), torch.zeros(self.nneg, dtype=torch.int64, device=dev))
        self._g_loss = torch.zeros((), **f)
        self._cap_stream: Optional[torch.cuda.Stream] = None

    # ------------------------------------------------------------------ kernels
    def _stage(self, stage: int, corrupt_head: bool, want_scores: bool):
        bs = self.bs
        h, t, neg = self.ent_rows[:bs], self.ent_rows[bs:2 * bs], self.ent_rows[2 * bs:]
        gh, gt, gneg = self.ent_grad[:bs], self.ent_grad[bs:2 * bs], self.ent_grad[2 * bs:]
        _lib.call("rs_kge_stage", stage, ptr(h), ptr(self.rel_rows), ptr(t), ptr(neg), bs, self.cs, self.ns, self.D, self.Dp,
                  self.Dr, self.model_id, 1 if corrupt_head else 0, self.cfg.gamma, self.emb_init, ptr(self.A), ptr(self.Bn), ptr(self.a2), ptr(self.b2),
                  ptr(self.loss), ptr(gh), ptr(self.rel_grad), ptr(gt), ptr(gneg), ptr(self.S), ptr(self.W), ptr(self.rowsum),
                  ptr(self.colsum), ptr(self.GA), ptr(self.GB), ptr(self.pos_score) if want_scores else None,
                  ptr(self.neg_score) if want_scores else None, stream_ptr())

    def _forward(self, corrupt_head: bool, want_scores: bool):
        st = self.ctx.status
        self.loss.zero_(); self.rowsum.zero_(); self.colsum.zero_()
        self._stage(0, corrupt_head, want_scores)
        if not self.pairwise:
            F_.gemm_bf16(self.A, self.Bn, self.S, mode=0, epi=F_.EPI_F32, status=st)
        self._stage(1, corrupt_head, want_scores)

    def _fetch(self, h_ids, r_ids, t_ids, neg_ids):
        bs = self.bs
        self.ids[:bs].copy_(h_ids); self.ids[bs:2 * bs].copy_(t_ids); self.ids[2 * bs:].copy_(neg_ids)
        self.entity.lookup(self.ids, out=self.ent_rows)
        if self.rescal:
            self._rel_keys.copy_((r_ids.view(-1, 1) * self.D + self._row_of_block).view(-1))
            self.relation.lookup(self._rel_keys, out=self.rel_rows.view(self.bs * self.D, self.D))
        else:
            self.relation.lookup(r_ids.contiguous(), out=self.rel_rows)
        if self.transr:
            self._rel_keys.copy_((r_ids.view(-1, 1) * self.D + self._row_of_block).view(-1))
            self.proj.lookup(self._rel_keys, out=self.proj_rows)

    # ------------------------------------------------------------------ TransR: autograd over batched library GEMMs
    def _transr_scores(self, h, r, t, neg, M, corrupt_head: bool):
        """pos [bs], neg [bs, ns]: gamma - |x M + r - y M|_1 with the negatives of a chunk projected by every positive's
        own matrix (one batched [ns x D] x [D x Dr] product per positive)."""
        bs, C, cs, ns, D, Dr = self.bs, self.C, self.cs, self.ns, self.D, self.Dr
        hp = torch.einsum("nd,ndk->nk", h, M)
        tp = torch.einsum("nd,ndk->nk", t, M)
        pos = self.cfg.gamma - (hp + r - tp).abs().sum(-1)
        P = torch.einsum("cjd,cidk->cijk", neg.view(C, ns, D), M.view(C, cs, D, Dr))        # projected negatives
        if corrupt_head:
            diff = P + (r - tp).view(C, cs, 1, Dr)
        else:
            diff = (hp + r).view(C, cs, 1, Dr) - P
        return pos, (self.cfg.gamma - diff.abs().sum(-1)).view(bs, ns)

    def _transr_step(self, corrupt_head: bool) -> torch.Tensor:
        bs, D = self.bs, self.D
        leaf = lambda x: x.detach().requires_grad_(True)
        h, t, neg = leaf(self.ent_rows[:bs]), leaf(self.ent_rows[bs:2 * bs]), leaf(self.ent_rows[2 * bs:])
        r, M = leaf(self.rel_rows), leaf(self.proj_rows.view(bs, D, self.Dr))
        old_tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = bool(self.cfg.tf32_scoring)
        try:
            with torch.enable_grad():
                pos, negs = self._transr_scores(h, r, t, neg, M, corrupt_head)
                loss = (-torch.nn.functional.logsigmoid(pos).mean() - torch.nn.functional.logsigmoid(-negs).mean()) / 2
                loss.backward()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = old_tf32
        self.ent_grad[:bs].copy_(h.grad); self.ent_grad[bs:2 * bs].copy_(t.grad); self.ent_grad[2 * bs:].copy_(neg.grad)
        self.rel_grad.copy_(r.grad)
        self.proj_grad.copy_(M.grad.view(bs * D, self.Dr))
        self.entity.update(self.ent_grad)
        self.relation.update(self.rel_grad)
        # one Adagrad state per relation: every row of a matrix is accounted the whole matrix's squared norm / D
        self._rel_norm.copy_((M.grad.pow(2).sum((1, 2)) / D).view(-1, 1).expand(bs, D).reshape(-1))
        self.proj.update(self.proj_grad, norms=self._rel_norm)
        self.launches_per_step = self.entity.launches + self.relation.launches + self.proj.launches
        return loss.detach()

    def train_step(self, h_ids: torch.Tensor, r_ids: torch.Tensor, t_ids: torch.Tensor, neg_ids: torch.Tensor,
                   corrupt_head: Optional[bool] = None) -> torch.Tensor:
        """One step on device id tensors (``neg_ids``: ``[batch / chunk * neg_sample_size]`` entity ids); returns the
        loss as a 0-d device tensor (no host synchronisation).  With ``use_cuda_graph`` the ids are copied into fixed
        buffers and the captured launch sequence of that corruption side is replayed."""
        if self.heartbeat is not None:
            self.heartbeat.check(self.heartbeat_timeout_s)
        if corrupt_head is None:
            corrupt_head = bool(self.step_no & 1)            # head / tail corruption alternate
        self.step_no += 1
        if not self.cfg.use_cuda_graph:
            return self._step(h_ids, r_ids, t_ids, neg_ids, corrupt_head)
        for dst, src in zip(self._g_ids, (h_ids, r_ids, t_ids, neg_ids)):
            dst.copy_(src, non_blocking=True)
        if corrupt_head not in self._graphs:
            self._g_loss.copy_(self._step(*self._g_ids, corrupt_head))   # eager once (this step's update): one-time set-up happens here
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            cur = torch.cuda.current_stream()
            if cur == torch.cuda.default_stream():           # capture needs a non-default stream; replay runs on any
                if self._cap_stream is None:
                    self._cap_stream = torch.cuda.Stream()
                self._cap_stream.wait_stream(cur)
                cur = self._cap_stream
            with torch.cuda.graph(g, stream=cur, capture_error_mode="relaxed"):
                self._g_loss.copy_(self._step(*self._g_ids, corrupt_head))
            self._graphs[corrupt_head] = g
            return self._g_loss.clone()                       # the eager pass above already did this step's update
        self._graphs[corrupt_head].replay()
        return self._g_loss.clone()

    def _step(self, h_ids, r_ids, t_ids, neg_ids, corrupt_head: bool) -> torch.Tensor:
        st = self.ctx.status
        self._fetch(h_ids, r_ids, t_ids, neg_ids)
        if self.transr:
            return self._transr_step(corrupt_head)
        self._forward(corrupt_head, False)
        if not self.pairwise:
            F_.gemm_bf16(self.W, self.Bn, self.GA, mode=2, epi=F_.EPI_F32, status=st)
            F_.gemm_bf16(self.W, self.A, self.GB, mode=1, epi=F_.EPI_F32, status=st)
        self._stage(2, corrupt_head, False)
        self.entity.update(self.ent_grad)
        if self.rescal:   # rowsum holds |dM|^2 of every positive: / D makes the table's mean over a row the mean over the matrix
            self._rel_norm.copy_((self.rowsum / self.D).view(-1, 1).expand(self.bs, self.D).reshape(-1))
            self.relation.update(self.rel_grad.view(self.bs * self.D, self.D), norms=self._rel_norm)
        else:
            self.relation.update(self.rel_grad)
        self.launches_per_step = (7 if self.pairwise else 9) + self.entity.launches + self.relation.launches
        return self.loss.sum()

    @torch.no_grad()
    def score_batch(self, h_ids, r_ids, t_ids, neg_ids, corrupt_head: bool) -> Tuple[torch.Tensor, torch.Tensor]:
        """Scores of the positives ``[batch]`` and of every (positive, chunk negative) pair ``[batch, neg_sample_size]``."""
        self._fetch(h_ids, r_ids, t_ids, neg_ids)
        if self.transr:
            bs = self.bs
            return self._transr_scores(self.ent_rows[:bs], self.rel_rows, self.ent_rows[bs:2 * bs], self.ent_rows[2 * bs:],
                                       self.proj_rows.view(bs, self.D, self.Dr), corrupt_head)
        self._forward(corrupt_head, True)
        return self.pos_score.clone(), self.neg_score.clone()

    @torch.no_grad()
    def evaluate(self, h_ids, r_ids, t_ids, generator: Optional[torch.Generator] = None) -> Dict[str, float]:
        """Link-prediction metrics of one batch of test triples against sampled negatives, both corruptions
        (rank of the positive among its chunk's negatives; general_models.py:464-513): MRR, MR, HITS@1/3/10."""
        ranks = []
        for corrupt_head in (False, True):
            if generator is not None:
                neg = torch.randint(0, self.cfg.n_entities, (self.nneg,), device=self.dev, generator=generator)
            else:
                from ..utils.data import device_uniform_ids
                self._eval_draws = getattr(self, "_eval_draws", 0) + 1
                neg = device_uniform_ids(self.nneg, self.cfg.n_entities, 0x5EED + self.cfg.seed, self._eval_draws * self.nneg, device=self.dev)
            pos, negs = self.score_batch(h_ids, r_ids, t_ids, neg, corrupt_head)
            ranks.append(1 + (negs >= pos.unsqueeze(1)).sum(1))
        r = torch.cat(ranks).float()
        return {"MRR": (1.0 / r).mean().item(), "MR": r.mean().item(), "HITS@1": (r <= 1).float().mean().item(),
                "HITS@3": (r <= 3).float().mean().item(), "HITS@10": (r <= 10).float().mean().item()}

    # ------------------------------------------------------------------ checkpoints
    def _gather_table(self, tab: ShardedEmbeddingTable) -> Optional[np.ndarray]:
        """Full table on rank 0 (host), ``None`` elsewhere.  Meant for tables that fit in host memory."""
        world, rank = self.ctx.world, self.ctx.rank
        local = tab.weight.cpu()
        if tab.tiered:                       # hot rows in HBM, then the host tier
            local = torch.cat([local, tab.cold])
        if world == 1:
            return local[: tab.N].numpy()
        import torch.distributed as dist
        parts = [None] * world if rank == 0 else None
        dist.gather_object(local, parts, dst=0, group=self.ctx.group)
        if rank != 0:
            return None
        full = torch.empty(tab.local_rows * world, tab.D)
        for r, p in enumerate(parts):
            full[r::world] = p
        return full[: tab.N].numpy()

    def save(self, path: str) -> None:
        self.ctx.check_status()              # tables written after a device-side error would be a wrong checkpoint
        os.makedirs(path, exist_ok=True)
        ent = self._gather_table(self.entity)
        rel = self._gather_table(self.relation)
        prj = self._gather_table(self.proj) if self.transr else None
        if self.ctx.rank == 0:
            c = self.cfg
            if self.rescal:
                rel = rel.reshape(c.n_relations, self.D * self.D)
            if prj is not None:      # the reference's name for the TransR matrices (score_fun.py TransRScore.save)
                np.save(os.path.join(path, f"{c.dataset}_{c.model}projection.npy"), prj.reshape(c.n_relations, self.D * self.Dr))
            np.save(os.path.join(path, f"{c.dataset}_{c.model}_entity.npy"), ent)
            np.save(os.path.join(path, f"{c.dataset}_{c.model}_relation.npy"), rel)
            conf = asdict(c)
            conf.update({"emp_file": f"{c.dataset}_{c.model}_entity.npy", "rmap_file": f"{c.dataset}_{c.model}_relation.npy",
                         "hidden_dim": c.dim, "model_name": c.model})
            with open(os.path.join(path, "config.json"), "w") as f:
                json.dump(conf, f, indent=2)

    def load(self, path: str) -> None:
        c = self.cfg
        tabs = [(self.entity, "_entity"), (self.relation, "_relation")] + ([(self.proj, "projection")] if self.transr else [])
        for tab, kind in tabs:
            full = torch.from_numpy(np.load(os.path.join(path, f"{c.dataset}_{c.model}{kind}.npy")))
            if (self.rescal and kind == "_relation") or kind == "projection":
                full = full.reshape(c.n_relations * self.D, -1)
            mine = full[self.ctx.rank::self.ctx.world]
            hot = min(mine.shape[0], tab.weight.shape[0])
            tab.weight[:hot].copy_(mine[:hot])
            if tab.tiered and mine.shape[0] > hot:
                tab.cold[: mine.shape[0] - hot].copy_(mine[hot:])


class KGSampler:
    """Synthetic triples with power-law entity degrees; every ``next()`` yields device id tensors of one step."""

    def __init__(self, cfg: KGEConfig, n_triples: int, alpha: float = 1.3, device="cuda", rank: int = 0, seed: int = 0):
        from ..utils.data import powerlaw_triples
        h, r, t = powerlaw_triples(n_triples, cfg.n_entities, cfg.n_relations, alpha, seed * 97 + rank)
        self.h, self.r, self.t = (torch.from_numpy(x).to(device) for x in (h, r, t))
        self.cfg, self.dev, self.n = cfg, device, n_triples
        self.gen = torch.Generator(device=device).manual_seed(seed * 31 + rank)
        self._seed = (seed * 31 + rank) * 2 + 1000003
        self.nneg = cfg.batch // cfg.neg_chunk_size * cfg.neg_sample_size
        self.step = 0

    def __next__(self):
        # positives and negatives are drawn on the device from counter-based streams (csrc/ops/sampling.cu): no host
        # generator state, the same stream whatever the launch shape
        from ..utils.data import device_uniform_ids
        c = self.step * (self.cfg.batch + self.nneg)
        idx = device_uniform_ids(self.cfg.batch, self.n, self._seed, c, device=self.dev)
        neg = device_uniform_ids(self.nneg, self.cfg.n_entities, self._seed + 1, c, device=self.dev)
        self.step += 1
        return self.h[idx], self.r[idx], self.t[idx], neg

    def __iter__(self):
        return self
