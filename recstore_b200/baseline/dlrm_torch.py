"""PyTorch (+NCCL, +cuBLAS) restatement of the reference's distributed DLRM step.

This is the measured same-box baseline and the numerical oracle, not the product path: it
follows the reference algorithm with stock PyTorch ops only --
``nn.EmbeddingBag(mode="sum")`` per local table over the full batch, ``all_to_all_single`` of
the pooled rows (src/executable/dlrm/dlrm_model.py:364-405, extend_distributed.py:389-486),
cuBLAS MLPs, ``bmm`` + lower-triangle interaction (dlrm_model.py:316-340), gradient
all-reduce of the replicated MLPs, SGD on the MLPs and row-wise Adagrad on the embedding rows
with the duplicate handling of ``SparseRowWiseAdaGrad`` (src/python/pytorch/recstore/
DistOpt.py:511-557: state += sum over occurrences of mean(g^2); W -= lr * g / (sqrt(state)+eps)
per occurrence with the post-step state).

It runs on CPU (fp32, gloo or single process) for tests and on GPUs (bf16 autocast MLPs) as the
baseline arm of the benchmarks.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn.functional as F


def rowwise_adagrad_update(weight: torch.Tensor, state: torch.Tensor, idx: torch.Tensor, grad: torch.Tensor,
                           lr: float, eps: float) -> None:
    """In-place reference update for one table (idx [n], grad [n, D]); duplicates allowed."""
    g2 = grad.float().pow(2).mean(1)
    state.index_add_(0, idx, g2)
    std = state[idx].sqrt().add_(eps)
    weight.index_add_(0, idx, (-lr * grad.float() / std.unsqueeze(1)).to(weight.dtype))


def sgd_update(weight: torch.Tensor, idx: torch.Tensor, grad: torch.Tensor, lr: float) -> None:
    weight.index_add_(0, idx, (-lr * grad.float()).to(weight.dtype))


class TorchDLRM:
    """Explicit-parameter DLRM with manual sparse optimizers; world-size aware."""

    def __init__(self, table_rows: Sequence[int], batch: int, emb_dim: int = 128, hotness: Optional[Sequence[int]] = None,
                 num_dense: int = 13, bottom_mlp=(512, 256, 128), top_mlp=(1024, 1024, 512, 256, 1),
                 emb_lr: float = 0.01, emb_eps: float = 1e-10, emb_optimizer: str = "rowwise_adagrad",
                 mlp_lr: float = 0.01, device="cpu", rank: int = 0, world: int = 1, autocast_bf16: bool = False,
                 seed: int = 0, group=None, interaction: str = "dot", dcn_layers: int = 3, dcn_rank: int = 512,
                 projection_sizes: Sequence[int] = (4, 4), projection_hidden: Sequence[Sequence[int]] = ((), ())):
        self.table_rows = list(table_rows)
        self.T = len(self.table_rows)
        self.D = emb_dim
        self.hotness = list(hotness) if hotness is not None else [1] * self.T
        self.B, self.Bl = batch, batch // world
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device)
        self.emb_lr, self.emb_eps, self.emb_optimizer, self.mlp_lr = emb_lr, emb_eps, emb_optimizer, mlp_lr
        self.loss_function, self.loss_weights = "bce", (1.0, 1.0)     # "bce" | "mse" | "wbce"; set by the driver
        self.autocast = autocast_bf16
        self.owner = [t % world for t in range(self.T)]
        self.local_tables = [t for t in range(self.T) if self.owner[t] == rank]
        self.tables: Dict[int, torch.Tensor] = {}
        self.states: Dict[int, torch.Tensor] = {}
        for t in self.local_tables:
            n = self.table_rows[t]
            w = torch.empty(n, emb_dim, device=self.device)
            w.uniform_(-math.sqrt(1.0 / n), math.sqrt(1.0 / n))
            self.tables[t] = w
            self.states[t] = torch.zeros(n, device=self.device)
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.params: Dict[str, torch.Tensor] = {}
        self.interaction = interaction
        self._num_dense, self._bottom_mlp, self._top_mlp = num_dense, list(bottom_mlp), list(top_mlp)
        self._dcn_layers, self._dcn_rank = dcn_layers, dcn_rank
        assert interaction in ("dot", "dcn", "projection")
        self.I1, self.I2 = projection_sizes
        self.proj_hidden = (tuple(projection_hidden[0]), tuple(projection_hidden[1]))    # hidden widths of the two branch MLPs
        n_inter = (self.T + 1) * emb_dim if interaction == "dcn" else emb_dim + (self.T + 1) * self.T // 2
        if interaction == "projection":          # DLRM_Projection: two learned projections of the features, then their product
            n_inter = emb_dim + self.I1 * self.I2
        kb = [num_dense] + list(bottom_mlp[:-1])
        for i, (k, n) in enumerate(zip(kb, bottom_mlp)):
            self.params[f"bot.{i}.weight"] = (torch.randn(n, k, generator=g) * math.sqrt(2.0 / (n + k))).to(self.device)
            self.params[f"bot.{i}.bias"] = (torch.randn(n, generator=g) * math.sqrt(1.0 / n)).to(self.device)
        kt = [n_inter] + list(top_mlp[:-2])
        for i, (k, n) in enumerate(zip(kt, top_mlp[:-1])):
            self.params[f"top.{i}.weight"] = (torch.randn(n, k, generator=g) * math.sqrt(2.0 / (n + k))).to(self.device)
            self.params[f"top.{i}.bias"] = (torch.randn(n, generator=g) * math.sqrt(1.0 / n)).to(self.device)
        self.n_cross = dcn_layers if interaction == "dcn" else 0
        for l in range(self.n_cross):
            # low-rank cross layer of DCNv2 (torchrec LowRankCrossNet as used by model_zoo/dlrm.py:261-286)
            self.params[f"crossV.{l}.weight"] = (torch.randn(dcn_rank, n_inter, generator=g) * math.sqrt(2.0 / (dcn_rank + n_inter))).to(self.device)
            self.params[f"crossV.{l}.bias"] = torch.zeros(dcn_rank, device=self.device)       # unused, kept for a uniform layout
            self.params[f"crossW.{l}.weight"] = (torch.randn(n_inter, dcn_rank, generator=g) * math.sqrt(2.0 / (dcn_rank + n_inter))).to(self.device)
            self.params[f"crossW.{l}.bias"] = torch.zeros(n_inter, device=self.device)
        if interaction == "projection":
            # InteractionProjectionArch of the reference (model_zoo/dlrm.py:289-404): Linear((F*D) -> I*D) branches
            fd = (self.T + 1) * emb_dim
            for name, I, hid in (("proj1", self.I1, self.proj_hidden[0]), ("proj2", self.I2, self.proj_hidden[1])):
                widths = [fd] + list(hid) + [I * emb_dim]
                for li, (k, n) in enumerate(zip(widths[:-1], widths[1:])):
                    self.params[f"{name}.{li}.weight"] = (torch.randn(n, k, generator=g) * math.sqrt(2.0 / (n + k))).to(self.device)
                    self.params[f"{name}.{li}.bias"] = torch.zeros(n, device=self.device)
        hk = top_mlp[-2]
        self.params["head.weight"] = (torch.randn(hk, generator=g) * math.sqrt(2.0 / (1 + hk))).to(self.device)
        self.params["head.bias"] = torch.randn(1, generator=g).to(self.device)
        self.n_bot, self.n_top = len(bottom_mlp), len(top_mlp) - 1
        for p in self.params.values():
            p.requires_grad_(True)
        li, lj = torch.tril_indices(self.T + 1, self.T + 1, offset=-1)
        self.li, self.lj = li.to(self.device), lj.to(self.device)

    # -------------------------------------------------------------- pieces
    def _mlp(self, x, prefix, n, last_relu=True):
        for i in range(n):
            x = F.linear(x, self.params[f"{prefix}.{i}.weight"].to(x.dtype), self.params[f"{prefix}.{i}.bias"].to(x.dtype))
            if i < n - 1 or last_relu:
                x = F.relu(x)
        return x

    def _pooled(self, ids: Dict[int, torch.Tensor]) -> List[torch.Tensor]:
        outs = []
        for t in self.local_tables:
            h = self.hotness[t]
            idx = ids[t].to(self.device).view(self.B, h)
            outs.append(self.tables[t][idx].sum(1))            # [B, D]
        return outs

    def _a2a_fwd(self, pooled: List[torch.Tensor]) -> torch.Tensor:
        """[B, Tl*D] on the owner -> [Bl, T, D] on every rank (global table order)."""
        if self.world == 1:
            return torch.stack(pooled, 1)
        send = torch.stack(pooled, 1) if pooled else torch.zeros(self.B, 0, self.D, device=self.device)  # [B,Tl,D]
        Tl = [sum(1 for t in range(self.T) if self.owner[t] == r) for r in range(self.world)]
        recv = torch.empty(sum(Tl) * self.Bl * self.D, device=self.device, dtype=send.dtype)
        dist.all_to_all_single(recv, send.contiguous().view(-1), output_split_sizes=[n * self.Bl * self.D for n in Tl],
                               input_split_sizes=[self.Bl * send.shape[1] * self.D] * self.world, group=self.group)
        parts = torch.split(recv, [n * self.Bl * self.D for n in Tl])
        out = torch.empty(self.Bl, self.T, self.D, device=self.device, dtype=send.dtype)
        for r, p in enumerate(parts):
            cols = [t for t in range(self.T) if self.owner[t] == r]
            if cols:
                out[:, cols] = p.view(self.Bl, len(cols), self.D)
        return out

    def _a2a_bwd(self, g: torch.Tensor) -> torch.Tensor:
        """[Bl, T, D] gradients -> [B, Tl, D] on the owners."""
        if self.world == 1:
            return g
        Tl = [sum(1 for t in range(self.T) if self.owner[t] == r) for r in range(self.world)]
        send = torch.cat([g[:, [t for t in range(self.T) if self.owner[t] == r]].reshape(-1) for r in range(self.world)])
        mine = Tl[self.rank]
        recv = torch.empty(self.world * self.Bl * mine * self.D, device=self.device, dtype=g.dtype)
        dist.all_to_all_single(recv, send, output_split_sizes=[self.Bl * mine * self.D] * self.world,
                               input_split_sizes=[n * self.Bl * self.D for n in Tl], group=self.group)
        return recv.view(self.B, mine, self.D)

    def forward_logits(self, dense_local: torch.Tensor, emb: torch.Tensor) -> torch.Tensor:
        with torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.autocast):
            x = self._mlp(dense_local, "bot", self.n_bot)
            Tm = torch.cat([x.unsqueeze(1), emb.to(x.dtype)], 1)                 # [Bl, F, D]
            if self.interaction == "dcn":
                x0 = Tm.reshape(Tm.shape[0], -1)
                z = x0
                for l in range(self.n_cross):
                    tl = F.linear(z, self.params[f"crossV.{l}.weight"].to(z.dtype))
                    u = F.linear(tl, self.params[f"crossW.{l}.weight"].to(z.dtype), self.params[f"crossW.{l}.bias"].to(z.dtype))
                    z = x0 * u + z
            elif self.interaction == "projection":
                flat = Tm.reshape(Tm.shape[0], -1)
                b1 = self._mlp(flat, "proj1", len(self.proj_hidden[0]) + 1)       # ReLU after every layer of a branch
                b2 = self._mlp(flat, "proj2", len(self.proj_hidden[1]) + 1)
                inter = torch.bmm(b1.view(-1, self.I1, self.D), b2.view(-1, self.I2, self.D).transpose(1, 2))   # [B, I1, I2]
                z = torch.cat([x, inter.reshape(inter.shape[0], -1)], 1)
            else:
                Z = torch.bmm(Tm, Tm.transpose(1, 2))
                z = torch.cat([x, Z[:, self.li, self.lj]], 1)
            y = self._mlp(z, "top", self.n_top)
            logit = F.linear(y, self.params["head.weight"].to(y.dtype).unsqueeze(0), self.params["head.bias"].to(y.dtype))
        return logit.float().squeeze(1)

    # -------------------------------------------------------------- one training step
    # ---- state access shared with the GPU engine (checkpoints move between the two)
    def describe(self) -> dict:
        return {"table_rows": list(self.table_rows), "emb_dim": self.D, "hotness": list(self.hotness),
                "num_dense": self._num_dense, "bottom_mlp": list(self._bottom_mlp), "top_mlp": list(self._top_mlp),
                "interaction": self.interaction, "dcn_layers": self._dcn_layers, "dcn_rank": self._dcn_rank,
                "projection_sizes": [self.I1, self.I2], "projection_hidden": [list(h) for h in self.proj_hidden]}

    def dense_state(self) -> Dict[str, torch.Tensor]:
        return {k: v.detach().clone() for k, v in self.params.items()}

    def load_dense_state(self, sd: Dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            for k, v in self.params.items():
                v.copy_(sd[k].view_as(v))

    def table_weight(self, t: int) -> torch.Tensor:
        return self.tables[t]

    def table_state(self, t: int) -> torch.Tensor:
        return self.states[t]

    def train_step(self, dense: torch.Tensor, ids: Sequence[torch.Tensor], labels: torch.Tensor) -> torch.Tensor:
        """``dense`` [B, nd], ``ids`` per table [B*hot], ``labels`` [B]: the GLOBAL batch."""
        lo, hi = self.rank * self.Bl, (self.rank + 1) * self.Bl
        ids_local = {t: ids[t] for t in self.local_tables}
        with torch.no_grad():
            pooled = self._pooled(ids_local)
            emb = self._a2a_fwd(pooled)
        emb.requires_grad_(True)
        for p in self.params.values():
            p.grad = None
        logit = self.forward_logits(dense[lo:hi].to(self.device), emb)
        y = labels[lo:hi].to(self.device)
        if self.loss_function == "bce":
            loss = F.binary_cross_entropy_with_logits(logit, y, reduction="sum") / self.B
        elif self.loss_function == "mse":                    # on the click probability (dlrm_model.py: loss_fn = MSELoss on sigmoid output)
            loss = ((torch.sigmoid(logit) - y) ** 2).sum() / self.B
        else:                                                # "wbce": per-class weights w[0] for label 0, w[1] for label 1
            w = self.loss_weights[1] * y + self.loss_weights[0] * (1 - y)
            loss = (w * F.binary_cross_entropy_with_logits(logit, y, reduction="none")).sum() / self.B
        loss.backward()
        with torch.no_grad():
            gemb = self._a2a_bwd(emb.grad)                                           # [B, Tl, D]
            for j, t in enumerate(self.local_tables):
                h = self.hotness[t]
                idx = ids[t].to(self.device).view(-1)
                g = gemb[:, j].repeat_interleave(h, 0) if h > 1 else gemb[:, j]
                if self.emb_optimizer == "rowwise_adagrad":
                    rowwise_adagrad_update(self.tables[t], self.states[t], idx, g, self.emb_lr, self.emb_eps)
                else:
                    sgd_update(self.tables[t], idx, g, self.emb_lr)
            if self.world > 1:
                for p in self.params.values():
                    if p.grad is None:
                        p.grad = torch.zeros_like(p)
                flat = torch.cat([p.grad.reshape(-1) for p in self.params.values()])
                dist.all_reduce(flat, group=self.group)
                o = 0
                for p in self.params.values():
                    p.grad.copy_(flat[o:o + p.numel()].view_as(p))
                    o += p.numel()
            for p in self.params.values():
                if p.grad is not None:
                    p.add_(p.grad, alpha=-self.mlp_lr)
        return loss.detach()

    @torch.no_grad()
    def predict(self, dense, ids) -> torch.Tensor:
        lo, hi = self.rank * self.Bl, (self.rank + 1) * self.Bl
        emb = self._a2a_fwd(self._pooled({t: ids[t] for t in self.local_tables}))
        return torch.sigmoid(self.forward_logits(dense[lo:hi].to(self.device), emb))
