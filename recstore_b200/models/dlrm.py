"""DLRM (dot interaction) training / inference engine on the native sm_100a kernels.

Model: the Facebook DLRM as forked by the reference (``DLRM_Net``,
src/executable/dlrm/dlrm_model.py:72-110 MLPs, :255-314 embedding bags, :316-351 dot
interaction, :364-423 distributed forward): bottom MLP on the dense features, one sum-pooled
embedding bag per table, pairwise dot interaction, top MLP, sigmoid + BCE.

Parallelisation (one process per GPU): embedding tables are placed table-wise on the ranks
(model parallel), the MLPs are replicated (data parallel).  The "butterfly" all-to-all of the
reference is not a collective here: the embedding gather kernel stores each pooled row straight
into the destination rank's interaction buffer over NVLink, the interaction backward kernel
stores each embedding gradient straight into the owning rank's gradient window, and flag
channels order the steps.  The dense gradient all-reduce is a two-shot push kernel followed by
the SGD kernels (``parallel.peer``).  There is no autograd graph: the backward pass is written
out as a fixed sequence of kernel launches, captured once into a CUDA graph and replayed.

Inputs are double buffered: ``submit`` enqueues the host-to-device copies of the next batch on a
copy stream while the previous step still computes.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _lib
from .._lib import call, stream_ptr
from ..ops import functional as F_
from ..parallel.peer import PeerContext

CH_FWD, CH_BWD, CH_GRADS, CH_REDUCED, CH_MISC, CH_GRADS_TOP, CH_KEYS, CH_PART = 0, 1, 2, 3, 4, 5, 6, 7


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class DLRMConfig:
    table_rows: Sequence[int]
    batch: int                                   # global batch size
    emb_dim: int = 128
    hotness: Optional[Sequence[int]] = None      # ids per bag for every table (default 1)
    num_dense: int = 13
    bottom_mlp: Sequence[int] = (512, 256, 128)  # output widths; the last equals emb_dim
    top_mlp: Sequence[int] = (1024, 1024, 512, 256, 1)
    emb_lr: float = 0.01
    emb_eps: float = 1e-10
    emb_optimizer: str = "rowwise_adagrad"       # or "sgd"
    mlp_lr: float = 0.01
    seed: int = 0
    use_cuda_graph: bool = True
    emb_init: str = "uniform"                    # U(+-sqrt(1/n)) as in the reference, or "normal"
    interaction: str = "dot"                     # "dot" (DLRM), "dcn" (DLRM-DCNv2: low-rank cross network) or "projection"
    projection_sizes: Tuple[int, int] = (4, 4)   # DLRM_Projection: rows of the two projected branches
    projection_hidden: Tuple[Sequence[int], Sequence[int]] = ((), ())   # hidden widths of the two branch MLPs (multiples of 64)
    dcn_layers: int = 3
    dcn_rank: int = 512
    placement: str = "round_robin"               # tables on ranks: "round_robin" (t % world) or "balanced" (greedy by ids per sample)
    trace_phases: bool = False                   # stamp the GPU timer at phase boundaries (see DLRM.phase_times)
    # Tables spread ROW-WISE over all ranks (owner of id = id % world) instead of living whole on one rank: a list of
    # table indices, or "auto" = every table whose share of the ids per sample exceeds 1 / world (one rank could
    # never keep up with it).  Ignored on one GPU.
    row_split: object = None
    # Cross-step pipelining of the sparse forward (dot interaction, tables whole on their ranks): the lookup + forward
    # all-to-all of batch t + 1 runs at the END of step t's graph, beside the dense all-reduce and SGD, instead of at the
    # start of step t + 1 (role of TrainPipelineSparseDist, model_zoo/golden_train.py:146-159).  `submit` then launches
    # step t when batch t + 1 is submitted (or when the result of step t is asked for).
    pipeline_lookup: bool = False

    def __post_init__(self):
        if self.hotness is None:
            self.hotness = [1] * len(self.table_rows)
        assert len(self.hotness) == len(self.table_rows)
        assert self.bottom_mlp[-1] == self.emb_dim, "bottom MLP must end at the embedding width"
        assert self.top_mlp[-1] == 1, "top MLP ends in one logit"


class _Layer:
    """One Linear(K -> N): fp32 master slices of the flat buffers plus bf16 copies W and W^T."""

    def __init__(self, N: int, K: int, Kp: int):
        self.N, self.K, self.Kp = N, K, Kp
        self.w = self.b = self.gw = self.gb = self.rw = self.rb = None
        self.wb = self.wt = None


@dataclass
class PinnedBatch:
    """One rank's share of a global batch in pinned host memory."""
    dense: torch.Tensor     # [B_local, num_dense] fp32
    ids: torch.Tensor       # [nnz_local] int64: for each whole local table, B * hotness ids, sample-major
    labels: torch.Tensor    # [B_local] fp32
    ids_rw: Optional[torch.Tensor] = None   # row-sharded tables: for each of them, this rank's B_local * hotness ids

    @property
    def nbytes(self) -> int:
        return (self.dense.numel() * 4 + self.ids.numel() * 8 + self.labels.numel() * 4 +
                (self.ids_rw.numel() * 8 if self.ids_rw is not None else 0))


class StepHandle:
    """Result of an asynchronously submitted step."""

    def __init__(self, engine: "DLRM", slot: int, event: torch.cuda.Event, step: int = 0):
        self._e, self._slot, self._ev, self._step = engine, slot, event, step

    def result(self) -> float:
        """Waits for the step and returns this rank's share of the mean BCE loss (sum over ranks = loss)."""
        e = self._e
        if self._step >= e._launched:                # pipelined mode: the step still waits for its successor
            e.flush()
        self._ev.synchronize()
        word = int(e._status_host[self._slot].item()) & 0xFFFFFFFFFFFFFFFF
        if word:
            # A kernel of this step (or an earlier one) gave up a bounded wait, met an id outside its table or a full
            # window: what the step computed from that point on is not to be trusted.
            e.ctx.status.zero_()
            raise _lib.DeviceStatusError(_lib.ERR_TIMEOUT if word & _lib.DEV_WAIT_TIMEOUT else _lib.ERR_INVALID,
                                         "device status after the step: " + _lib.decode_status(word))
        return float(e._loss_host[self._slot].item())


class DLRM:
    def __init__(self, cfg: DLRMConfig, ctx: Optional[PeerContext] = None):
        if not torch.cuda.is_available():
            raise _lib.RecStoreError(_lib.ERR_STATE, "models.DLRM needs a CUDA device (sm_100a)")
        _lib.lib()
        self.cfg = cfg
        self.ctx = ctx if ctx is not None else PeerContext(0, 1)
        self.rank, self.world = self.ctx.rank, self.ctx.world
        dev = self.dev = self.ctx.device
        assert cfg.batch % self.world == 0
        self.B = cfg.batch
        self.Bl = cfg.batch // self.world
        self.T = len(cfg.table_rows)
        self.D = cfg.emb_dim
        self.F = self.T + 1
        self.dcn = cfg.interaction == "dcn"
        self.proj = cfg.interaction == "projection"
        assert cfg.interaction in ("dot", "dcn", "projection")
        assert self.dcn or self.proj or self.F <= 32, "dot interaction kernel handles up to 31 embedding features"
        # ---- table placement.  Row-sharded tables (if any) are local tables 0..K-1 of EVERY rank; the others live whole
        # on one rank: round robin unless the config asks for the load-balanced greedy.
        split: List[int] = []
        if self.world > 1 and cfg.row_split:
            if cfg.row_split == "auto":
                tot = float(sum(cfg.hotness))
                split = [t for t in range(self.T) if cfg.hotness[t] / tot > 1.0 / self.world]
            else:
                split = sorted(set(int(t) for t in cfg.row_split))
        self.split_tables, self.K = split, len(split)
        K = self.K
        whole = [t for t in range(self.T) if t not in split]
        if cfg.placement == "round_robin":
            own = {t: (t if not split else i) % self.world for i, t in enumerate(whole)}
        else:
            from ..parallel.placement import place_tables
            placed = place_tables([cfg.hotness[t] for t in whole], [cfg.table_rows[t] for t in whole], self.world, cfg.placement)
            own = {t: placed[i] for i, t in enumerate(whole)}
        self.owner = [-1 if t in split else own[t] for t in range(self.T)]
        self.whole_local = [t for t in whole if self.owner[t] == self.rank]
        self.local_tables = split + self.whole_local
        self.Tl, self.Tw = len(self.local_tables), len(self.whole_local)
        self.Tmax = K + max(sum(1 for t in whole if self.owner[t] == r) for r in range(self.world))
        local_idx = {t: k for k, t in enumerate(split)}
        cnt = [K] * self.world
        for t in whole:
            local_idx[t] = cnt[self.owner[t]]
            cnt[self.owner[t]] += 1
        self.local_idx = local_idx

        g = torch.Generator(device="cpu").manual_seed(cfg.seed)
        i32 = dict(dtype=torch.int32, device=dev)
        i64 = dict(dtype=torch.int64, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)

        # ---- embedding shard: [rows of the row-sharded tables with id % world == rank | rows of the whole local tables]
        def local_rows(t):
            n = cfg.table_rows[t]
            return (n - self.rank + self.world - 1) // self.world if t in split else n
        rows = [local_rows(t) for t in self.local_tables]
        base = [0]
        for r in rows:
            base.append(base[-1] + r)
        self.total_rows = base[-1]
        self.table_base = torch.tensor(base[:-1] or [0], **i64)
        self.table_rows = torch.tensor(rows or [0], **i64)
        self.weight = torch.empty(max(self.total_rows, 1), self.D, **f32)
        for j, t in enumerate(self.local_tables):
            n = cfg.table_rows[t]
            gt = torch.Generator(device=dev).manual_seed(cfg.seed * 1000 + t)
            w = self.weight[base[j]:base[j + 1]]
            if t in split:
                # the same values as the whole table would get, of which this rank keeps every world-th row
                full = torch.empty(n, self.D, **f32)
                if cfg.emb_init == "uniform":
                    full.uniform_(-math.sqrt(1.0 / n), math.sqrt(1.0 / n), generator=gt)
                else:
                    full.normal_(0.0, 0.01, generator=gt)
                w.copy_(full[self.rank::self.world])
                del full
            elif cfg.emb_init == "uniform":
                w.uniform_(-math.sqrt(1.0 / n), math.sqrt(1.0 / n), generator=gt)
            else:
                w.normal_(0.0, 0.01, generator=gt)
        self.state = torch.zeros(max(self.total_rows, 1), **f32)
        # whole local tables: the ids of the GLOBAL batch, table after table
        hot = [cfg.hotness[t] for t in self.whole_local]
        hb = [0]
        for h in hot:
            hb.append(hb[-1] + self.B * h)
        self.nnz = hb[-1]
        self.hotness = torch.tensor(hot or [1], **i32)
        self.hot_base = torch.tensor(hb[:-1] or [0], **i64)
        self.dst_col = torch.tensor([(1 + t) * self.D for t in self.whole_local] or [0], **i32)
        self.grad_col = torch.tensor([(K + j) * self.D for j in range(self.Tw)] or [0], **i32)
        self.row_idx = torch.empty(max(self.nnz, 1), **i64)
        self.occ2bag = torch.empty(max(self.nnz, 1), **i32)
        self.owner_dev = torch.tensor(self.owner, **i32)
        self.gcol_dev = torch.tensor([local_idx[t] * self.D for t in range(self.T)], **i32)
        self.table_base_w, self.table_rows_w = self.table_base[K:], self.table_rows[K:]
        if self.Tw == 0:
            self.table_base_w = self.table_rows_w = torch.zeros(1, **i64)
        # row-sharded tables: this rank's B_local samples send their ids to the owners (key windows), the owners pool
        # their share of every bag and send the partial sums back (partial windows)
        if K:
            hk = [cfg.hotness[t] for t in split]
            self.hot_rw = torch.tensor(hk, **i32)
            idb, kb = [0], [0]
            for h in hk:
                idb.append(idb[-1] + self.Bl * h)
                kb.append(kb[-1] + self.B * h)
            self.nnz_rw_local = idb[-1]                    # ids of this rank's samples
            self.nnz_rw_cap = kb[-1]                       # key slots per owner (worst case: every id lives here)
            self.id_base_rw = torch.tensor(idb[:-1], **i64)
            self.key_base_rw = torch.tensor(kb[:-1], **i64)
            self.key_win = self.ctx.alloc("dlrm_rw_keys", self.nnz_rw_cap * 8)
            self.cnt_win = self.ctx.alloc("dlrm_rw_counts", K * self.B * 4)
            self.part_win = self.ctx.alloc("dlrm_rw_partials", self.Bl * K * self.world * self.D * 2)
            self.part_col = torch.tensor([(k * self.world + self.rank) * self.D for k in range(K)], **i32)
            self.red_col = torch.tensor([(1 + t) * self.D for t in split], **i32)
            self.grad_col_rw = torch.tensor([k * self.D for k in range(K)], **i32)
            self.row_idx_rw = torch.empty(self.nnz_rw_cap, **i64)
            self.occ2bag_rw = torch.empty(self.nnz_rw_cap, **i32)
            self.occ_cursor = torch.zeros(1, **i32)
        self._grid_done = torch.zeros(8, **i32)            # "grid done" counters of the kernels that publish their own flag

        # ---- peer windows
        self.grow_stride = self.Tmax * self.D
        # Two forward windows, used alternately by the two input slots: a peer that is one step ahead writes the rows of
        # batch t + 1 into the other window while this rank may still read those of batch t.
        self._T = []
        for i in range(2):
            w = self.ctx.alloc("dlrm_T" if i == 0 else "dlrm_T1", self.Bl * self.F * self.D * 2)
            self._T.append((w, w.view(torch.bfloat16, (self.Bl, self.F * self.D))))
        self.Twin = self._T[0][0]
        # gradient window: [B, Tmax*D] bf16 rows pushed by the peers, then [B, Tmax] fp32 squared norms
        self.gn_off = _round_up(self.B * self.grow_stride * 2, 256)
        self.Gwin = self.ctx.alloc("dlrm_G", self.gn_off + self.B * self.Tmax * 4)
        self.gnorm = self.Gwin.view(torch.float32, (self.B, self.Tmax), byte_offset=self.gn_off)
        self.ndst_table = torch.tensor([p + self.gn_off for p in self.Gwin.ptrs], dtype=torch.int64, device=dev)
        self.Tbuf = self._T[0][1]
        if self.world > 1 and not self.dcn and not self.proj and (self.K or os.environ.get("RECSTORE_GRAD_PUSH", "") == "staged"):
            # Backward all-to-all with row-sharded tables under the dot interaction: its backward leaves the per-(sample,
            # table) gradient rows in this local staging buffer; a thin copy kernel then fans them out to their owners.
            self.gstage = torch.empty(self.Bl, self.T * self.D, **bf)
            self.stage_table = torch.tensor([self.gstage.data_ptr()] * self.world, **i64)
            self.stage_owner = torch.zeros(self.T, **i32)
            self.stage_col = torch.tensor([t * self.D for t in range(self.T)], **i32)

        # ---- dense parameters (flat fp32 master / grad / reduced buffers)
        self.Kin0 = _round_up(cfg.num_dense, 64)
        self.n_inter = self.F * self.D if self.dcn else self.D + self.F * (self.F - 1) // 2
        if self.proj:
            self.I1, self.I2 = cfg.projection_sizes
            assert 1 <= self.I1 <= 8 and 1 <= self.I2 <= 8, "projection branches have 1..8 rows"
            assert (self.F * self.D) % 64 == 0, "projection needs (1 + tables) * dim to be a multiple of 64"
            self.n_inter = self.D + self.I1 * self.I2
        self.Kz = _round_up(self.n_inter, 64)
        assert not self.dcn or self.Kz == self.n_inter, "DCN needs (1 + tables) * dim to be a multiple of 64"
        dims_b = [(cfg.num_dense, self.Kin0)] + [(n, n) for n in cfg.bottom_mlp[:-1]]
        self.bot: List[_Layer] = [_Layer(n, k, kp) for (k, kp), n in zip(dims_b, cfg.bottom_mlp)]
        dims_t = [(self.n_inter, self.Kz)] + [(n, n) for n in cfg.top_mlp[:-2]]
        self.top: List[_Layer] = [_Layer(n, k, kp) for (k, kp), n in zip(dims_t, cfg.top_mlp[:-1])]
        self.head_K = cfg.top_mlp[-2]
        # DCNv2 low-rank cross layers: x_{l+1} = x0 * (W_l (V_l x_l) + b_l) + x_l, V_l [rank, in], W_l [in, rank]
        self.crossV: List[_Layer] = []
        self.crossW: List[_Layer] = []
        if self.dcn:
            r = cfg.dcn_rank
            assert r % 64 == 0
            self.crossV = [_Layer(r, self.n_inter, self.n_inter) for _ in range(cfg.dcn_layers)]
            self.crossW = [_Layer(self.n_inter, r, r) for _ in range(cfg.dcn_layers)]
        # DLRM_Projection: two branch MLPs over the flattened features, F * D -> hidden... -> I * D, ReLU after every layer
        self.projB: List[List[_Layer]] = [[], []]
        if self.proj:
            for b, (I, hid) in enumerate(zip((self.I1, self.I2), cfg.projection_hidden)):
                widths = [self.F * self.D] + list(hid) + [I * self.D]
                assert all(w % 64 == 0 for w in widths[:-1]), "projection branch widths are multiples of 64"
                self.projB[b] = [_Layer(n, k, k) for k, n in zip(widths[:-1], widths[1:])]
        self.projL: List[_Layer] = self.projB[0] + self.projB[1]
        layers = self.bot + self.top + self.crossV + self.crossW + self.projL
        self.layers = layers
        off = 0
        w_off = []
        for L in layers:
            w_off.append(off)
            off += L.N * L.Kp
        self.n_w = off
        self.top_w_off = w_off[len(self.bot)]              # weights of the top MLP (and cross layers) start here
        b_off = []
        for L in layers:
            b_off.append(off)
            off += _round_up(L.N, 4)
        head_w_off = off
        off += _round_up(self.head_K, 4)
        head_b_off = off
        off += 4
        self.n_params = off
        self.tail_off, self.tail_n = self.n_w, off - self.n_w
        self.master = torch.zeros(self.n_params, **f32)
        self.Gflat = self.ctx.alloc("dlrm_dense_grad", self.n_params * 4)
        self.grads = self.Gflat.view(torch.float32, (self.n_params,))
        if self.world > 1:
            self.Rflat = self.ctx.alloc("dlrm_dense_reduced", self.n_params * 4)
            self.reduced = self.Rflat.view(torch.float32, (self.n_params,))
        else:
            self.reduced = self.grads
        for L, wo, bo in zip(layers, w_off, b_off):
            L.w = self.master[wo:wo + L.N * L.Kp].view(L.N, L.Kp)
            L.b = self.master[bo:bo + L.N]
            L.gw = self.grads[wo:wo + L.N * L.Kp].view(L.N, L.Kp)
            L.gb = self.grads[bo:bo + L.N]
            L.rw = self.reduced[wo:wo + L.N * L.Kp].view(L.N, L.Kp)
            L.wb = torch.zeros(L.N, L.Kp, **bf)
            L.wt = torch.zeros(L.Kp, L.N, **bf)
            w0 = torch.randn(L.N, L.K, generator=g) * math.sqrt(2.0 / (L.N + L.K))
            b0 = torch.randn(L.N, generator=g) * math.sqrt(1.0 / L.N)
            if L in self.crossV:
                b0.zero_()                       # V has no bias
            if L in self.crossW or L in self.projL:
                b0.zero_()                       # cross / projection biases start at zero
            L.w[:, :L.K].copy_(w0)
            L.b.copy_(b0)
        self.head_w = self.master[head_w_off:head_w_off + self.head_K]
        self.head_b = self.master[head_b_off:head_b_off + 1]
        self.g_head_w = self.grads[head_w_off:head_w_off + self.head_K]
        self.g_head_b = self.grads[head_b_off:head_b_off + 1]
        self.head_w.copy_(torch.randn(self.head_K, generator=g) * math.sqrt(2.0 / (1 + self.head_K)))
        self.head_b.copy_(torch.randn(1, generator=g))
        self._refresh_bf16()
        # descriptor of the one-launch SGD step over all layers (8 int64 per layer) and its tile prefix
        desc, prefix = [], [0]
        for L in layers:
            desc += [L.w.data_ptr(), L.rw.data_ptr(), L.wb.data_ptr(), L.wt.data_ptr(), L.N, L.Kp, L.wb.stride(0), L.wt.stride(0)]
            prefix.append(prefix[-1] + ((L.Kp + 31) // 32) * ((L.N + 31) // 32))
        self._sgd_desc = torch.tensor(desc, dtype=torch.int64, device=dev)
        self._sgd_prefix = torch.tensor(prefix, dtype=torch.int32, device=dev)
        self._sgd_tiles = prefix[-1]

        # ---- activations and their gradients
        Bl = self.Bl
        self.x0p = torch.zeros(Bl, self.Kin0, **bf)
        self.act_b = [torch.empty(Bl, L.N, **bf) for L in self.bot[:-1]]          # h1, h2 (h3 lives in Tbuf)
        self.z = torch.empty(Bl, self.Kz, **bf)
        self.act_t = [torch.empty(Bl, L.N, **bf) for L in self.top]               # t1..t4
        self.d_act_t = [torch.empty(Bl, L.N, **bf) for L in self.top]
        self.d_z = torch.empty(Bl, self.Kz, **bf)
        self.d_act_b = [torch.empty(Bl, L.N, **bf) for L in self.bot]             # d_h1, d_h2, d_h3
        if self.dcn:
            nl, r = cfg.dcn_layers, cfg.dcn_rank
            self.cx = [self.Tbuf] + [torch.empty(Bl, self.n_inter, **bf) for _ in range(nl - 1)] + [self.z]   # x_0 .. x_L
            self.ct = [torch.empty(Bl, r, **bf) for _ in range(nl)]                    # V_l x_l
            self.cu = [torch.empty(Bl, self.n_inter, **bf) for _ in range(nl)]         # W_l t_l + b_l
            self.c_du = torch.empty(Bl, self.n_inter, **bf)
            self.c_dt = torch.empty(Bl, r, **bf)
            self.c_dx = [self.d_z, torch.empty(Bl, self.n_inter, **bf)]                # ping-pong dX_l
            self.c_dx0 = torch.empty(Bl, self.n_inter, **f32)
        if self.proj:
            self.pb = [[torch.empty(Bl, L.N, **bf) for L in Ls] for Ls in self.projB]   # activations of the branch layers
            self.pdb = [[torch.empty(Bl, L.N, **bf) for L in Ls] for Ls in self.projB]  # and their gradients
            self.p_dx = [torch.empty(Bl, self.F * self.D, **bf) for _ in range(2)]
        self.prob = torch.empty(Bl, **f32)

        # ---- double-buffered inputs, loss
        self.in_dense = [torch.empty(Bl, cfg.num_dense, **f32) for _ in range(2)]
        self.in_ids = [torch.empty(max(self.nnz, 1), **i64) for _ in range(2)]
        self.in_ids_rw = [torch.empty(self.nnz_rw_local, **i64) for _ in range(2)] if self.K else [None, None]
        self.in_labels = [torch.empty(Bl, **f32) for _ in range(2)]
        self._loss_dev = [torch.zeros(1, **f32) for _ in range(2)]
        self._loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
        self._status_host = [torch.zeros(1, dtype=torch.int64).pin_memory() for _ in range(2)]   # the device status word, read back with the loss
        # Dot interaction without row-sharded tables: the interaction backward pushes the embedding gradients itself.  With
        # row-sharded tables (a gradient row then goes to every rank) they are staged and a thin copy kernel fans them out.
        # (RECSTORE_GRAD_PUSH=staged forces the staged form for measurements.)
        self._fused_push = not self.K and not self.dcn and not self.proj and os.environ.get("RECSTORE_GRAD_PUSH", "") != "staged"
        # Stream priorities (RECSTORE_STREAM_PRIORITIES: 0 = none, 1 = main stream first, 2 = communication stream first).
        prio = os.environ.get("RECSTORE_STREAM_PRIORITIES", "0")
        p_main, p_comm, p_col, p_wgrad = {"1": (-3, -2, -1, 0), "2": (-2, -3, -1, 0)}.get(prio, (0, 0, 0, 0))
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.compute_stream = torch.cuda.Stream(device=dev, priority=p_main)
        self._copied = [torch.cuda.Event() for _ in range(2)]
        self._consumed = [torch.cuda.Event() for _ in range(2)]
        self._done = [torch.cuda.Event() for _ in range(2)]
        self._graphs: Dict[object, torch.cuda.CUDAGraph] = {}
        self._step_no = 0
        # Optional liveness check before every launch (utils/liveness.Heartbeat): set both to have `submit` raise
        # RankLostError when another rank has died or left, instead of launching a step whose peers never answer.
        self.heartbeat = None
        self.heartbeat_timeout_s = 2.0
        self.launches_per_step = 0
        # Pipelined lookup: supported where the forward exchange is the one lookup kernel (dot interaction, no row-sharded
        # tables).  `_pending` is the submitted step whose graph has not been launched yet (its lookup has been).
        self._pipe = bool(cfg.pipeline_lookup) and not self.dcn and not self.proj and not self.K
        self._pending: Optional[int] = None           # slot of the pending step
        self._launched = 0                            # steps whose graph has been launched
        self.s_wgrad = torch.cuda.Stream(device=dev, priority=p_wgrad)   # weight/bias gradients, then the dense all-reduce and SGD
        self.s_comm = torch.cuda.Stream(device=dev, priority=p_comm)     # embedding lookup / gradient push: the NVLink-bound kernels
        self.s_wgrad2 = torch.cuda.Stream(device=dev, priority=p_wgrad)  # weight gradients of the bottom MLP
        self.s_col = torch.cuda.Stream(device=dev, priority=p_col)       # bias gradients (column sums): bandwidth-bound, beside the wgrad GEMMs
        self._phase_names: List[str] = []
        self._no_stamp = False
        self._phase_buf = torch.zeros(64, dtype=torch.int64, device=dev)
        self._warm_native()
        torch.cuda.synchronize(dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.ctx.group)

    # ------------------------------------------------------------------ helpers
    def _warm_native(self):
        """Runs both GEMM variants once on scratch data so that one-time function attributes are set
        before any stream capture (the model state is untouched)."""
        a = torch.zeros(128, 64, dtype=torch.bfloat16, device=self.dev)
        o = torch.zeros(128, 128, dtype=torch.bfloat16, device=self.dev)
        o32 = torch.zeros(64, 64, dtype=torch.float32, device=self.dev)
        F_.gemm_bf16(a, a, o, mode=0, epi=F_.EPI_NONE, status=self.ctx.status)
        F_.gemm_bf16(a, a, o32, mode=1, epi=F_.EPI_ATOMIC_F32, status=self.ctx.status)

    def _refresh_bf16(self):
        for L in self.layers:
            L.wb.copy_(L.w)
            L.wt.copy_(L.w.t())

    def make_pinned_batch(self, dense: torch.Tensor, ids: Sequence[torch.Tensor], labels: torch.Tensor) -> PinnedBatch:
        """Cuts this rank's share out of a GLOBAL batch (dense [B,nd], per-table ids [B*hot], labels [B])."""
        lo, hi = self.rank * self.Bl, (self.rank + 1) * self.Bl
        d = dense[lo:hi].contiguous().pin_memory()
        l = labels[lo:hi].contiguous().pin_memory()
        if self.whole_local:
            i = torch.cat([ids[t].reshape(-1) for t in self.whole_local]).to(torch.int64).pin_memory()
        else:
            i = torch.zeros(1, dtype=torch.int64).pin_memory()
        assert i.numel() == max(self.nnz, 1)
        irw = None
        if self.K:     # row-sharded tables: the ids of this rank's own samples; the owners get them over NVLink
            irw = torch.cat([ids[t].reshape(self.B, -1)[lo:hi].reshape(-1) for t in self.split_tables]).to(torch.int64).pin_memory()
            assert irw.numel() == self.nnz_rw_local
        return PinnedBatch(d, i, l, irw)

    def _count(self, n=1):
        self.launches_per_step += n

    def _stamp(self, name: str):
        """Phase boundary: with ``trace_phases`` a one-thread kernel stores the GPU timer here (also inside the graph)."""
        if not self.cfg.trace_phases or self._no_stamp:
            return
        if name not in self._phase_names:
            self._phase_names.append(name)
        call("rs_stamp_time", self._phase_buf.data_ptr() + 8 * self._phase_names.index(name), stream_ptr())
        self._count()

    def phase_times(self) -> Dict[str, float]:
        """Microseconds spent between consecutive phase stamps of the last completed step on this rank."""
        assert self.cfg.trace_phases, "construct the engine with trace_phases=True"
        torch.cuda.synchronize(self.dev)
        t = self._phase_buf[:len(self._phase_names)].cpu().tolist()
        return {f"{a}->{b}": (t[i + 1] - t[i]) / 1e3
                for i, (a, b) in enumerate(zip(self._phase_names[:-1], self._phase_names[1:]))}

    # ------------------------------------------------------------------ the step as a launch sequence
    def _bind_slot(self, slot: int):
        """The forward window of this input slot becomes the one the launch sequence below refers to."""
        self.Twin, self.Tbuf = self._T[slot]
        if self.dcn:
            self.cx[0] = self.Tbuf

    def _lookup(self, slot: int):
        """Embedding lookup + forward all-to-all of the batch in input slot ``slot`` (current stream: communication)."""
        st = self.ctx.status
        twin = self._T[slot][0]
        if self.world == 1:
            if self.Tl:
                F_.emb_forward(self.weight, self.table_base, self.table_rows, self.in_ids[slot], hotness=self.hotness,
                               hot_base=self.hot_base, T=self.Tl, B=self.B, D=self.D, B_local=self.Bl,
                               dst_table=twin.table, dst_row_stride=self.F * self.D, dst_col=self.dst_col,
                               out_bf16=True, row_idx=self.row_idx, occ2bag=self.occ2bag, status=st)
                self._count()
            return
        gd = self._grid_done
        if self.K:
            # row-sharded tables, step 1: the ids of my samples go to their owners (+ CH_KEYS)
            F_.rw_push_keys(self.in_ids_rw[slot], self.id_base_rw, self.hot_rw, self.key_base_rw, self.K, self.Bl,
                            self.B, self.key_win.table, self.cnt_win.table, self.occ_cursor, ctx=self.ctx,
                            sig_channel=CH_KEYS, sig_done=gd[0:1], status=st)
            self._count()
        if self.Tw:
            # whole tables: pooled rows go straight into the samples' ranks; the kernel publishes CH_FWD itself
            F_.emb_forward_ex(self.weight, self.table_base_w, self.table_rows_w, self.in_ids[slot], self.hotness,
                              self.hot_base, T=self.Tw, B=self.B, D=self.D, B_local=self.Bl, dst_table=twin.table,
                              dst_row_stride=self.F * self.D, dst_col=self.dst_col, row_idx=self.row_idx,
                              occ2bag=self.occ2bag, status=st, ctx=self.ctx, sig_channel=CH_FWD, sig_done=gd[1:2])
        else:
            self.ctx.signal(CH_FWD)
        self._count()
        if self.K:
            # step 2 (owner side): wait for each source rank's keys, pool my share of every bag, push the partial
            # sums into the samples' ranks (+ CH_PART); step 3: add the partials up into the feature slots
            F_.emb_forward_ex(self.weight, self.table_base, self.table_rows, self.key_win.local_ptr, self.hot_rw,
                              self.key_base_rw, T=self.K, B=self.B, D=self.D, B_local=self.Bl,
                              dst_table=self.part_win.table, dst_row_stride=self.K * self.world * self.D,
                              dst_col=self.part_col, row_idx=self.row_idx_rw, occ2bag=self.occ2bag_rw, status=st,
                              counts=self.cnt_win.local_ptr, id_div=self.world, id_rem=self.rank,
                              occ_cursor=self.occ_cursor, ctx=self.ctx, wait_channel=CH_KEYS, sig_channel=CH_PART,
                              sig_done=gd[2:3])
            F_.rw_reduce_partials(self.part_win.local_ptr, self._T[slot][1], self.red_col, self.Bl, self.K, self.D,
                                  ctx=self.ctx, wait_channel=CH_PART, status=st)
            self._count(2)

    def _forward(self, slot: int, lookup: bool = True):
        c, st = self.cfg, self.ctx.status
        self._bind_slot(slot)
        self._stamp("start")
        F_.pad_cast_bf16(self.in_dense[slot], self.x0p); self._count()
        main = torch.cuda.current_stream(self.dev)
        if lookup:
            # the lookup (bound by HBM, and by NVLink when multi-GPU) runs beside the bottom MLP (bound by the tensor pipe)
            self.s_comm.wait_stream(main)
            with torch.cuda.stream(self.s_comm):
                self._lookup(slot)
        self._stamp("emb_fwd_done")
        x = self.x0p
        for i, L in enumerate(self.bot):
            out = self.act_b[i] if i < len(self.bot) - 1 else self.Tbuf[:, :self.D]
            F_.gemm_bf16(x, L.wb, out, mode=0, epi=F_.EPI_RELU, bias=L.b, status=st, n=L.N); self._count()
            x = out
        self._stamp("bot_fwd_done")
        if lookup:
            main.wait_stream(self.s_comm)         # (without a lookup of its own the step started after the one it relies on)
        if self.world > 1 and (self.dcn or self.proj):
            self.ctx.wait_own(CH_FWD); self._count()     # the consumer is a GEMM fed by TMA: it cannot wait in its own prologue
        self._stamp("a2a_fwd_arrived")
        if self.dcn:
            for l in range(len(self.crossV)):
                V, W = self.crossV[l], self.crossW[l]
                F_.gemm_bf16(self.cx[l], V.wb, self.ct[l], mode=0, epi=F_.EPI_NONE, status=st)
                F_.gemm_bf16(self.ct[l], W.wb, self.cu[l], mode=0, epi=F_.EPI_NONE, bias=W.b, status=st)
                F_.cross_fwd(self.Tbuf, self.cu[l], self.cx[l], self.cx[l + 1])
                self._count(3)
        elif self.proj:
            for Ls, outs in zip(self.projB, self.pb):
                x = self.Tbuf
                for L, out in zip(Ls, outs):
                    F_.gemm_bf16(x, L.wb, out, mode=0, epi=F_.EPI_RELU, bias=L.b, status=st); self._count()
                    x = out
            F_.proj_inter_forward(self.Tbuf, self.pb[0][-1], self.pb[1][-1], self.I1, self.I2, self.D, self.z)
            self._count()
        elif self.world > 1:
            F_.interaction_forward_ex(self.Tbuf, self.Bl, self.F, self.D, self.z, ctx=self.ctx, wait_channel=CH_FWD, status=st)
            self._count()
        else:
            F_.interaction_forward(self.Tbuf, self.Bl, self.F, self.D, self.z); self._count()
        self._stamp("interaction_fwd_done")
        x = self.z
        for i, L in enumerate(self.top):
            F_.gemm_bf16(x, L.wb, self.act_t[i], mode=0, epi=F_.EPI_RELU, bias=L.b, status=st); self._count()
            x = self.act_t[i]
        return x

    def _run_step(self, slot: int, mode: str = "self"):
        """One training step on input slot ``slot``.  ``mode``: "self" = with its own lookup at the start; "none" = the
        rows of this batch are already on their way (a previous graph looked them up); "next" = like "none", and the
        lookup of the OTHER slot's batch runs at the end of this step, behind the sparse optimizer."""
        c, st = self.cfg, self.ctx.status
        self.launches_per_step = 0
        x = self._forward(slot, lookup=(mode == "self"))
        self._stamp("top_fwd_done")
        self._loss_dev[slot].zero_(); self._count()
        F_.head_bce(x, self.head_w, self.head_b, self.in_labels[slot], 1.0 / self.B, prob=self.prob,
                    loss_sum=self._loss_dev[slot], dx=self.d_act_t[-1], dw=self.g_head_w, db=self.g_head_b)
        self._count()
        self._stamp("head_done")
        main = torch.cuda.current_stream(self.dev)
        side = self.s_wgrad
        # ---- top MLP backward.  The dgrad chain is the critical path; bias and weight gradients of a layer only need
        # that layer's dY, so they run beside it on a second stream and fill the gaps and tails of the chain.
        for i in range(len(self.top) - 1, -1, -1):
            L = self.top[i]
            dy = self.d_act_t[i]
            xin = self.act_t[i - 1] if i > 0 else self.z
            side.wait_stream(main)
            self.s_col.wait_stream(main)
            with torch.cuda.stream(self.s_col):
                # Bias gradient as a pass of its own: summing columns inside the dgrad epilogue was measured slower
                # (every CTA adds into the same N addresses) than this bandwidth-bound kernel.
                F_.colsum_bf16(dy, L.gb); self._count()
            with torch.cuda.stream(side):
                F_.gemm_bf16(dy, xin, L.gw, mode=1, epi=F_.EPI_ATOMIC_F32, status=st); self._count()
            if i > 0:
                F_.gemm_bf16(dy, L.wt, self.d_act_t[i - 1], mode=0, epi=F_.EPI_RELU_MASK, aux=xin, status=st)
            else:
                F_.gemm_bf16(dy, L.wt, self.d_z, mode=0, epi=F_.EPI_NONE, status=st)
            self._count()
        # First all-reduce bucket: the top MLP's weight gradients (most of the dense parameters) are complete once the
        # wgrad stream has drained, long before the bottom MLP's; reducing them now hides the transfer behind the rest
        # of the backward.  (With the cross network its layers' gradients come later, so everything goes at the end.)
        early_bucket = self.world > 1 and not self.dcn and not self.proj
        if early_bucket:
            with torch.cuda.stream(side):
                self.ctx.sync(CH_GRADS_TOP)
                F_.allreduce_push(self.Gflat.table, self.Rflat.table, self.world, self.rank, self.n_w - self.top_w_off,
                                  offset=self.top_w_off)
                self._count(2)
        self._stamp("top_bwd_done")
        # ---- interaction backward: dense part stays, embedding gradients go to their owners
        if self.dcn:
            main.wait_stream(side)                                # the scratch buffers below are shared with nothing on `side`
            dx = self.c_dx[0]                                     # dX_L from the over-arch
            for l in range(len(self.crossV) - 1, -1, -1):
                V, W = self.crossV[l], self.crossW[l]
                nxt = self.c_dx[(len(self.crossV) - l) & 1]
                F_.cross_bwd(dx, self.Tbuf, self.cu[l], self.c_du, self.c_dx0, accumulate=(l != len(self.crossV) - 1))
                F_.colsum_bf16(self.c_du, W.gb)
                F_.gemm_bf16(self.c_du, self.ct[l], W.gw, mode=1, epi=F_.EPI_ATOMIC_F32, status=st)
                F_.gemm_bf16(self.c_du, W.wt, self.c_dt, mode=0, epi=F_.EPI_NONE, status=st)
                F_.gemm_bf16(self.c_dt, self.cx[l], V.gw, mode=1, epi=F_.EPI_ATOMIC_F32, status=st)
                F_.gemm_bf16(self.c_dt, V.wt, nxt, mode=0, epi=F_.EPI_ADD, aux=dx, status=st)
                dx = nxt
                self._count(6)
            F_.push_feature_grads(self.c_dx0, dx, self.Tbuf, self.Bl, self.F, self.D, self.d_act_b[-1], self.Gwin.table,
                                  self.owner_dev, self.gcol_dev, self.grow_stride, self.rank * self.Bl, relu_mask_dx=True,
                                  ndst_table=self.ndst_table, nstride=self.Tmax, world=self.world)
            self._count()
            if self.world > 1:
                self.ctx.signal(CH_BWD); self._count()
        elif self.proj:
            F_.proj_inter_backward(self.d_z, self.pb[0][-1], self.pb[1][-1], self.I1, self.I2, self.D,
                                   self.pdb[0][-1], self.pdb[1][-1])
            self._count()
            for b, Ls in enumerate(self.projB):
                for li in range(len(Ls) - 1, -1, -1):
                    L, dy = Ls[li], self.pdb[b][li]
                    xin = self.pb[b][li - 1] if li > 0 else self.Tbuf
                    side.wait_stream(main)
                    self.s_col.wait_stream(main)
                    with torch.cuda.stream(self.s_col):
                        F_.colsum_bf16(dy, L.gb)
                    with torch.cuda.stream(side):
                        F_.gemm_bf16(dy, xin, L.gw, mode=1, epi=F_.EPI_ATOMIC_F32, status=st)
                    if li > 0:
                        F_.gemm_bf16(dy, L.wt, self.pdb[b][li - 1], mode=0, epi=F_.EPI_RELU_MASK, aux=xin, status=st)
                    elif b == 0:
                        F_.gemm_bf16(dy, L.wt, self.p_dx[0], mode=0, epi=F_.EPI_NONE, status=st)
                    else:
                        F_.gemm_bf16(dy, L.wt, self.p_dx[1], mode=0, epi=F_.EPI_ADD, aux=self.p_dx[0], status=st)
                    self._count(3)
            # features: both branches' input gradients; the dense feature also feeds the over-arch directly
            F_.push_feature_grads(None, self.p_dx[1], self.Tbuf, self.Bl, self.F, self.D, self.d_act_b[-1], self.Gwin.table,
                                  self.owner_dev, self.gcol_dev, self.grow_stride, self.rank * self.Bl, relu_mask_dx=True,
                                  ndst_table=self.ndst_table, nstride=self.Tmax, dense_extra=self.d_z, world=self.world)
            self._count()
            if self.world > 1:
                self.ctx.signal(CH_BWD); self._count()
        elif self.world > 1 and self._fused_push:
            # The gradient all-to-all is done by the interaction backward itself (peer stores from the kernel that computes
            # the rows, bound by NVLink) on the communication stream; it leads to the sparse optimizer, the longest chain
            # of the backward, so it starts as soon as the top MLP's input gradient exists.  A small kernel of its own
            # produces only the bottom MLP's input gradient (a matrix-vector product per sample) on the main stream.
            self.s_comm.wait_stream(main)
            F_.interaction_dx(self.Tbuf, self.d_z, self.Bl, self.F, self.D, self.d_act_b[-1], relu_mask_dx=True)
            with torch.cuda.stream(self.s_comm):
                F_.interaction_backward(self.Tbuf, self.d_z, self.Bl, self.F, self.D, self.d_act_b[-1], self.Gwin.table,
                                        self.owner_dev, self.gcol_dev, self.grow_stride, self.rank * self.Bl,
                                        relu_mask_dx=True, ndst_table=self.ndst_table, nstride=self.Tmax, rows=2)
                self.ctx.signal(CH_BWD)
            self._count(3)
        elif self.world > 1:
            # Dot interaction with row-sharded tables: one pass leaves dx (the bottom MLP's input gradient) and every
            # embedding gradient row in a local staging buffer; the thin push below fans them out.
            F_.interaction_backward(self.Tbuf, self.d_z, self.Bl, self.F, self.D, self.d_act_b[-1], self.stage_table,
                                    self.stage_owner, self.stage_col, self.T * self.D, 0, relu_mask_dx=True)
            self._count()
        else:
            F_.interaction_backward(self.Tbuf, self.d_z, self.Bl, self.F, self.D, self.d_act_b[-1], self.Gwin.table,
                                    self.owner_dev, self.gcol_dev, self.grow_stride, self.rank * self.Bl,
                                    relu_mask_dx=True, ndst_table=self.ndst_table, nstride=self.Tmax)
            self._count()
        # ---- sparse optimizer on the owned rows (after the staged gradient rows, if any, have been fanned out): bound by
        # HBM and by the peers' pushes, so it runs on the communication stream beside the bottom MLP's backward, the dense
        # all-reduce and the SGD step.  Its first kernel waits for the peers' flags itself.
        self.s_comm.wait_stream(main)
        with torch.cuda.stream(self.s_comm):
            if self.world > 1:
                if not (self._fused_push or self.dcn or self.proj):
                    F_.push_rows(self.gstage, self.Bl, self.T, self.D, self.Gwin.table, self.owner_dev, self.gcol_dev,
                                 self.grow_stride, self.rank * self.Bl, ndst_table=self.ndst_table, nstride=self.Tmax,
                                 ctx=self.ctx, sig_channel=CH_BWD, sig_done=self._grid_done[3:4])
                    self._count()
                nl = 2 if c.emb_optimizer == "rowwise_adagrad" else 1
                if self.Tw:
                    F_.emb_backward_ex(self.weight, self.state, self.row_idx, self.occ2bag, self.nnz, self.Gwin.local,
                                       grad_col=self.grad_col, grad_row_stride=self.grow_stride, B=self.B, D=self.D,
                                       lr=c.emb_lr, eps=c.emb_eps, optimizer=c.emb_optimizer, status=st,
                                       gnorm=self.gnorm.data_ptr() + 4 * self.K, gnorm_stride=self.Tmax,
                                       ctx=self.ctx, wait_channel=CH_BWD)
                    self._count(nl)
                if self.K:
                    F_.emb_backward_ex(self.weight, self.state, self.row_idx_rw, self.occ2bag_rw, self.nnz_rw_cap,
                                       self.Gwin.local, grad_col=self.grad_col_rw, grad_row_stride=self.grow_stride, B=self.B,
                                       D=self.D, lr=c.emb_lr, eps=c.emb_eps, optimizer=c.emb_optimizer, status=st,
                                       gnorm=self.gnorm, gnorm_stride=self.Tmax, nnz_dev=self.occ_cursor,
                                       ctx=self.ctx, wait_channel=CH_BWD)
                    self._count(nl)
                if not self.Tl:
                    self.ctx.wait_own(CH_BWD); self._count()       # nothing to update here, but the step ends after the peers' pushes
            elif self.Tl:
                F_.emb_backward(self.weight, self.state, self.row_idx, self.occ2bag, self.nnz, self.Gwin.local,
                                grad_col=self.grad_col, grad_row_stride=self.grow_stride, B=self.B, D=self.D,
                                grad_bf16=True, lr=c.emb_lr, eps=c.emb_eps, optimizer=c.emb_optimizer, status=st,
                                gnorm=self.gnorm, gnorm_stride=self.Tmax)
                self._count(2 if c.emb_optimizer == "rowwise_adagrad" else 1)
            if mode == "next":
                # The tables now hold this step's update: the next batch's lookup + forward all-to-all can go, beside the
                # bottom MLP's backward, the dense all-reduce and the SGD step that are still to come.
                self._lookup(1 - slot)
        self._stamp("interaction_bwd_done")
        # ---- bottom MLP backward
        for i in range(len(self.bot) - 1, -1, -1):
            L = self.bot[i]
            dy = self.d_act_b[i]
            xin = self.act_b[i - 1] if i > 0 else self.x0p
            self.s_wgrad2.wait_stream(main)                       # bottom-MLP weight gradients do not queue behind the top MLP's
            self.s_col.wait_stream(main)
            with torch.cuda.stream(self.s_col):
                F_.colsum_bf16(dy, L.gb); self._count()
            with torch.cuda.stream(self.s_wgrad2):
                F_.gemm_bf16(dy, xin, L.gw, mode=1, epi=F_.EPI_ATOMIC_F32, status=st); self._count()
            if i > 0:
                F_.gemm_bf16(dy, L.wt, self.d_act_b[i - 1], mode=0, epi=F_.EPI_RELU_MASK, aux=xin, status=st)
                self._count()
        self._stamp("bot_bwd_done")
        # ---- dense gradients (complete once `side` has drained): all-reduce + SGD, beside the sparse optimizer
        solo = self.world == 1
        side.wait_stream(self.s_col)                               # bias gradients are part of the flat buffer
        side.wait_stream(self.s_wgrad2)
        with torch.cuda.stream(side):
            if not solo:
                self.ctx.sync(CH_GRADS)                            # every rank's gradients are complete
                if early_bucket:                                   # what is left: bottom-MLP weights, then biases + head
                    F_.allreduce_push(self.Gflat.table, self.Rflat.table, self.world, self.rank, self.top_w_off)
                    F_.allreduce_push(self.Gflat.table, self.Rflat.table, self.world, self.rank, self.tail_n, offset=self.n_w)
                    self._count()
                else:
                    F_.allreduce_push(self.Gflat.table, self.Rflat.table, self.world, self.rank, self.n_params)
                self.ctx.sync(CH_REDUCED)                          # every rank's slices have landed here
                self._count(3)
            # SGD on the reduced gradients; it also clears this rank's own accumulation buffer (same layout,
            # `delta` elements away), so no memset launch follows
            delta = 0 if solo else (self.grads.data_ptr() - self.reduced.data_ptr()) // 4
            call("rs_dense_sgd_multi", self._sgd_desc.data_ptr(), self._sgd_prefix.data_ptr(), len(self.layers), self._sgd_tiles,
                 self.master[self.tail_off:].data_ptr(), self.reduced[self.tail_off:].data_ptr(), self.tail_n, c.mlp_lr,
                 1 if solo else 0, delta, 0 if solo else 1, stream_ptr())
            self._count()
        main.wait_stream(self.s_comm)
        self._stamp("emb_bwd_done")
        main.wait_stream(side)
        self._stamp("sgd_done")

    # ------------------------------------------------------------------ public API
    def _copy_in(self, batch: PinnedBatch, slot: int):
        cs = self.copy_stream
        with torch.cuda.stream(cs):
            cs.wait_event(self._consumed[slot])       # previous user of this slot has finished
            self.in_dense[slot].copy_(batch.dense, non_blocking=True)
            self.in_ids[slot].copy_(batch.ids, non_blocking=True)
            if self.K:
                self.in_ids_rw[slot].copy_(batch.ids_rw, non_blocking=True)
            self.in_labels[slot].copy_(batch.labels, non_blocking=True)
            self._copied[slot].record(cs)

    def _launch(self, slot: int, mode: str):
        """Step graph (or eager launch sequence) of input slot ``slot`` on the compute stream, then the result copies."""
        ms = self.compute_stream
        with torch.cuda.stream(ms):
            if self.cfg.use_cuda_graph:
                g = self._graphs.get((slot, mode))
                if g is None:
                    g = self._capture(slot, mode)
                g.replay()
            else:
                self._run_step(slot, mode)
            self._consumed[slot].record(ms)
            self._loss_host[slot].copy_(self._loss_dev[slot], non_blocking=True)
            self._status_host[slot].copy_(self.ctx.status, non_blocking=True)
            self._done[slot].record(ms)
        self._launched += 1

    def _launch_lookup(self, slot: int):
        ms = self.compute_stream
        with torch.cuda.stream(ms):
            if self.cfg.use_cuda_graph:
                g = self._graphs.get((slot, "lookup"))
                if g is None:
                    g = self._capture(slot, "lookup")
                g.replay()
            else:
                self._run_lookup(slot)

    def _run_lookup(self, slot: int):
        main = torch.cuda.current_stream(self.dev)
        self.s_comm.wait_stream(main)
        with torch.cuda.stream(self.s_comm):
            self._lookup(slot)
        main.wait_stream(self.s_comm)

    def flush(self) -> None:
        """Pipelined mode: launches the step that is still waiting for its successor (without a look-ahead)."""
        if self._pending is not None:
            slot, self._pending = self._pending, None
            self._launch(slot, "none")

    def submit(self, batch: PinnedBatch) -> StepHandle:
        """Enqueues H2D copies of ``batch`` and one training step; returns immediately.  With ``pipeline_lookup`` the
        step itself is launched when the NEXT batch is submitted (its graph ends with that batch's lookup) or when its
        result is asked for; the lookup of this batch is launched now."""
        if self.heartbeat is not None:       # a peer that is gone must be noticed here, on the host, not inside a peer wait
            self.heartbeat.check(self.heartbeat_timeout_s)
        slot = self._step_no & 1
        step = self._step_no
        self._step_no += 1
        self._copy_in(batch, slot)
        ms = self.compute_stream
        with torch.cuda.stream(ms):
            ms.wait_event(self._copied[slot])
        if not self._pipe:
            self._launch(slot, "self")
        elif self._pending is None:
            self._launch_lookup(slot)                  # nothing to hide it behind: the pipeline starts here
            self._pending = slot
        else:
            self._launch(self._pending, "next")        # the previous step, ending with this batch's lookup
            self._pending = slot
        return StepHandle(self, slot, self._done[slot], step)

    def train_step(self, batch: PinnedBatch) -> float:
        return self.submit(batch).result()

    def time_steps_on_device(self, steps: int) -> float:
        """Runs ``steps`` training steps on the batches already resident in the two input slots and
        returns the elapsed milliseconds measured with CUDA events on the compute stream.  Pipelined mode: the lookup of
        the first batch precedes the timed region, every timed step ends with the lookup of the following batch (so the
        region holds ``steps`` lookups and ``steps`` dense passes, like the unpipelined one)."""
        self.flush()
        ms = self.compute_stream
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(self.dev)
        mode = "next" if self._pipe else "self"
        with torch.cuda.stream(ms):
            if self.cfg.use_cuda_graph:
                for slot in (0, 1):
                    if (slot, mode) not in self._graphs:
                        self._capture(slot, mode)
            if self._pipe:
                self._launch_lookup(0)
            e0.record(ms)
            for i in range(steps):
                slot = i & 1
                if self.cfg.use_cuda_graph:
                    self._graphs[(slot, mode)].replay()
                else:
                    self._run_step(slot, mode)
            e1.record(ms)
        e1.synchronize()
        return e0.elapsed_time(e1)

    def _capture(self, slot: int, mode: str = "self") -> torch.cuda.CUDAGraph:
        torch.cuda.current_stream().synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=torch.cuda.current_stream(), capture_error_mode="relaxed"):
            if mode == "lookup":
                self._run_lookup(slot)
            else:
                self._run_step(slot, mode)
        self._graphs[(slot, mode)] = g
        return g

    @torch.no_grad()
    def predict(self, batch: PinnedBatch) -> torch.Tensor:
        """Click probabilities of this rank's samples (inference, no parameter update)."""
        self.flush()
        with torch.cuda.stream(self.compute_stream):
            self.in_dense[0].copy_(batch.dense, non_blocking=True)
            self.in_ids[0].copy_(batch.ids, non_blocking=True)
            if self.K:
                self.in_ids_rw[0].copy_(batch.ids_rw, non_blocking=True)
            self._no_stamp = True          # the phase stamps describe the last training step, not an inference pass
            try:
                x = self._forward(0)
            finally:
                self._no_stamp = False
            F_.head_bce(x, self.head_w, self.head_b, None, 1.0 / self.B, prob=self.prob)
            if self.world > 1:
                self.ctx.barrier(CH_MISC)  # nobody may overwrite the interaction buffer before all have read it
            out = self.prob.clone()
        self.compute_stream.synchronize()
        return out

    def check(self):
        self.flush()
        self.ctx.check_status()

    # ------------------------------------------------------------------ state access (tests, checkpoints)
    def _named_layers(self):
        """Parameter-name prefixes shared with the PyTorch implementation (``baseline/dlrm_torch.py``)."""
        return (("bot", self.bot), ("top", self.top), ("crossV", self.crossV), ("crossW", self.crossW),
                ("proj1", self.projB[0]), ("proj2", self.projB[1]))

    def dense_state(self) -> Dict[str, torch.Tensor]:
        self.flush()
        torch.cuda.synchronize(self.dev)
        out = {}
        for name, Ls in self._named_layers():
            for i, L in enumerate(Ls):
                out[f"{name}.{i}.weight"] = L.w[:, :L.K].clone()
                out[f"{name}.{i}.bias"] = L.b.clone()
        out["head.weight"] = self.head_w.clone()
        out["head.bias"] = self.head_b.clone()
        return out

    def load_dense_state(self, sd: Dict[str, torch.Tensor]) -> None:
        for name, Ls in self._named_layers():
            for i, L in enumerate(Ls):
                L.w.zero_()
                L.w[:, :L.K].copy_(sd[f"{name}.{i}.weight"])
                L.b.copy_(sd[f"{name}.{i}.bias"])
        self.head_w.copy_(sd["head.weight"].reshape(-1))
        self.head_b.copy_(sd["head.bias"].reshape(-1))
        self._refresh_bf16()

    def describe(self) -> dict:
        """Shape of the model, as stored beside a checkpoint."""
        c = self.cfg
        return {"table_rows": list(c.table_rows), "emb_dim": c.emb_dim, "hotness": list(c.hotness), "num_dense": c.num_dense,
                "bottom_mlp": list(c.bottom_mlp), "top_mlp": list(c.top_mlp), "interaction": c.interaction,
                "dcn_layers": c.dcn_layers, "dcn_rank": c.dcn_rank, "projection_sizes": list(c.projection_sizes),
                "projection_hidden": [list(h) for h in c.projection_hidden]}

    def save_checkpoint(self, path: str, step: int = 0) -> None:
        from .checkpoint import save_checkpoint
        self.flush()
        torch.cuda.synchronize(self.dev)
        save_checkpoint(self, path, step)

    def load_checkpoint(self, path: str) -> dict:
        from .checkpoint import load_checkpoint
        meta = load_checkpoint(self, path)
        torch.cuda.synchronize(self.dev)
        return meta

    def gather_table(self, t: int, what: str = "weight") -> Optional[torch.Tensor]:
        """Collective: the whole table ``t`` (``what`` = "weight" or "state") on rank 0, wherever its rows live (``None``
        on the other ranks).  Tests and checkpoint tools use it; rows of a row-sharded table are re-interleaved."""
        import torch.distributed as dist
        self.flush()
        torch.cuda.synchronize(self.dev)
        mine = (self.table_weight if what == "weight" else self.table_state)
        n = self.cfg.table_rows[t]
        shape = (n, self.D) if what == "weight" else (n,)
        if self.world == 1:
            return mine(t).clone()
        if self.owner[t] >= 0:
            if self.owner[t] == 0:
                return mine(t).clone() if self.rank == 0 else None
            if self.rank == self.owner[t]:
                dist.send(mine(t).contiguous(), dst=0, group=self.ctx.group)
                return None
            if self.rank == 0:
                out = torch.empty(*shape, device=self.dev)
                dist.recv(out, src=self.owner[t], group=self.ctx.group)
                return out
            return None
        out = torch.empty(*shape, device=self.dev) if self.rank == 0 else None
        for r in range(self.world):
            if r == 0:
                if self.rank == 0:
                    out[0::self.world] = mine(t)
            elif self.rank == r:
                dist.send(mine(t).contiguous(), dst=0, group=self.ctx.group)
            elif self.rank == 0:
                part = torch.empty_like(out[r::self.world]).contiguous()
                dist.recv(part, src=r, group=self.ctx.group)
                out[r::self.world] = part
        return out

    def table_weight(self, t: int) -> torch.Tensor:
        """View of table ``t`` if this rank owns it (of this rank's rows, ids = rank, rank + world, ..., if the table is
        row-sharded)."""
        j = self.local_tables.index(t)
        b0 = int(self.table_base[j].item())
        return self.weight[b0:b0 + int(self.table_rows[j].item())]

    def table_state(self, t: int) -> torch.Tensor:
        j = self.local_tables.index(t)
        b0 = int(self.table_base[j].item())
        return self.state[b0:b0 + int(self.table_rows[j].item())]
