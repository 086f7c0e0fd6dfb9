"""DLRM training driver with the flag names of the reference's ``dlrm_model.py``.

    python -m recstore_b200.cli.dlrm_main --arch-sparse-feature-size 64 --arch-embedding-size 1000-2000-500 \
        --arch-mlp-bot 13-128-64 --arch-mlp-top 128-64-1 --mini-batch-size 2048 --num-batches 100 --use-gpu

Recognised flags (src/executable/dlrm/dlrm_model.py:618-760): ``--arch-sparse-feature-size --arch-embedding-size
--arch-mlp-bot --arch-mlp-top --arch-interaction-op dot|dcn|projection --mini-batch-size --nepochs --num-batches
--learning-rate --num-indices-per-lookup --num-indices-per-lookup-fixed --data-generation random|synthetic
--numpy-rand-seed --print-freq --test-freq --test-mini-batch-size --save-model --load-model --use-gpu``, plus
``--emb-learning-rate --emb-optimizer --zipf-alpha --dcn-layers --dcn-rank``; further ``--inference-only --data-size
--max-ind-range --rand-data-dist/-min/-max/-mu/-sigma --round-targets --loss-function bce|mse|wbce --loss-weights
--loss-threshold --lr-num-warmup-steps --lr-decay-start-step --lr-num-decay-steps --mlperf-acc-threshold
--enable-profiling --print-time``.  Flags of features this engine does not have (QR / mixed-dimension embeddings,
quantisation, ONNX export, ``--arch-interaction-itself``, ``--weighted-pooling``) are recognised and refused with a
message; ``--data-generation dataset`` trains on Criteo-format files (``--raw-data-file`` text or a ``--processed-data-file``
.npz; table sizes from the category counts, ``--data-sub-sample-rate``, ``--data-randomize``, ``--max-ind-range``); the
remaining loader / logging flags of the Criteo pipeline are accepted and have no effect.  The first number of
``--arch-mlp-bot`` is the count of dense features, its last must equal the sparse feature size; the first number of
``--arch-mlp-top`` is the interaction width and is checked, as the reference does (:914-951).

With ``--use-gpu`` the native engine runs (one process per GPU under ``torch.distributed.run``); without it the
PyTorch restatement runs on the CPU, same data, same checkpoints.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np
import torch


def dash_ints(s: str):
    return [int(x) for x in s.split("-") if x != ""]


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--arch-sparse-feature-size", type=int, default=16)
    p.add_argument("--arch-embedding-size", type=dash_ints, default=[4, 3, 2])
    p.add_argument("--arch-mlp-bot", type=dash_ints, default=[4, 16])
    p.add_argument("--arch-mlp-top", type=dash_ints, default=None, help="default: <interaction width>-64-1")
    p.add_argument("--arch-interaction-op", choices=["dot", "dcn", "projection"], default="dot",
                   help="dot: DLRM; dcn: low-rank DCNv2 cross network; projection: DLRM_Projection")
    p.add_argument("--interaction-branch-sizes", type=dash_ints, default=[4, 4], help="I1-I2 of the projection interaction")
    p.add_argument("--interaction-branch1-hidden", type=dash_ints, default=[], help="hidden widths of branch 1's MLP, e.g. 512-256")
    p.add_argument("--interaction-branch2-hidden", type=dash_ints, default=[], help="hidden widths of branch 2's MLP")
    p.add_argument("--dcn-layers", type=int, default=3)
    p.add_argument("--dcn-rank", type=int, default=64)
    p.add_argument("--mini-batch-size", type=int, default=128)
    p.add_argument("--nepochs", type=int, default=1)
    p.add_argument("--num-batches", type=int, default=50)
    p.add_argument("--learning-rate", type=float, default=0.01)
    p.add_argument("--emb-learning-rate", type=float, default=None)
    p.add_argument("--emb-optimizer", choices=["rowwise_adagrad", "sgd"], default="rowwise_adagrad")
    p.add_argument("--num-indices-per-lookup", type=int, default=1)
    p.add_argument("--num-indices-per-lookup-fixed", action="store_true", default=True)
    p.add_argument("--data-generation", choices=["random", "synthetic", "dataset"], default="random",
                   help="random: uniform ids; synthetic: Zipf ids (--zipf-alpha) or a trace profile (--data-trace-file); "
                        "dataset: Criteo-format files (--raw-data-file / --processed-data-file)")
    p.add_argument("--zipf-alpha", type=float, default=1.2)
    p.add_argument("--numpy-rand-seed", type=int, default=123)
    p.add_argument("--print-freq", type=int, default=10)
    p.add_argument("--test-freq", type=int, default=0)
    p.add_argument("--test-mini-batch-size", type=int, default=0)
    p.add_argument("--save-model", default="")
    p.add_argument("--load-model", default="")
    p.add_argument("--use-gpu", action="store_true")
    p.add_argument("--optimizer", default="sgd", choices=["sgd"], help="dense optimizer (the embeddings use --emb-optimizer)")
    p.add_argument("--dist-backend", default="nccl", choices=["nccl"], help="bootstrap backend; the data plane is NVLink peer memory")
    # ---- more of the reference's surface (dlrm_model.py:618-760)
    p.add_argument("--activation-function", default="relu", choices=["relu"], help="MLP activation (the fused epilogues implement ReLU)")
    p.add_argument("--arch-interaction-itself", action="store_true", help="not offered: the interaction kernels take the strict lower triangle")
    p.add_argument("--loss-function", default="bce", choices=["bce", "mse", "wbce"], help="mse / wbce run on the PyTorch path")
    p.add_argument("--loss-weights", type=lambda v: [float(x) for x in v.split("-")], default=[1.0, 1.0], help="wbce: weight of label 0 - label 1")
    p.add_argument("--loss-threshold", type=float, default=0.0, help="clamp predictions to [t, 1 - t] when reporting")
    p.add_argument("--round-targets", action="store_true", help="round the labels to 0 / 1")
    p.add_argument("--data-size", type=int, default=0, help="samples per epoch when --num-batches is 0")
    p.add_argument("--rand-data-dist", default="uniform", choices=["uniform", "gaussian"], help="random ids: uniform or clipped gaussian")
    p.add_argument("--rand-data-min", type=float, default=0.0)
    p.add_argument("--rand-data-max", type=float, default=1.0)
    p.add_argument("--rand-data-mu", type=float, default=-1.0)
    p.add_argument("--rand-data-sigma", type=float, default=1.0)
    p.add_argument("--max-ind-range", type=int, default=-1, help="cap every table at this many rows")
    p.add_argument("--inference-only", action="store_true")
    p.add_argument("--lr-num-warmup-steps", type=int, default=0)
    p.add_argument("--lr-decay-start-step", type=int, default=0)
    p.add_argument("--lr-num-decay-steps", type=int, default=0)
    p.add_argument("--print-time", action="store_true")
    p.add_argument("--print-wall-time", action="store_true")
    p.add_argument("--print-precision", type=int, default=5)
    p.add_argument("--debug-mode", action="store_true")
    p.add_argument("--local_rank", type=int, default=-1, help="set by launchers; LOCAL_RANK of the environment wins")
    p.add_argument("--num-workers", type=int, default=0, help="accepted: batches are generated in-process")
    p.add_argument("--test-num-workers", type=int, default=-1)
    p.add_argument("--sync-dense-params", type=lambda v: str(v).lower() in ("1", "true", "yes"), default=True,
                   help="accepted: the dense replicas are always kept identical by the all-reduce")
    p.add_argument("--weighted-pooling", default=None, choices=[None, "fixed", "learned"], help="not offered: bags are summed")
    p.add_argument("--enable-profiling", action="store_true", help="stamp the GPU timer at the phase boundaries and print the timeline")
    p.add_argument("--heartbeat-timeout", type=float, default=0.0,
                   help="multi-GPU: seconds without a sign of life after which a rank counts as lost (0: off); the others then "
                        "raise before their next step instead of waiting for it inside a kernel")
    p.add_argument("--tensor-board-filename", default="", help="directory that receives scalars.jsonl (step, loss, lr, test metrics)")
    p.add_argument("--data-set", default="kaggle", help="accepted; data here is generated (--data-generation)")
    for name in ("--raw-data-file", "--processed-data-file", "--data-trace-file"):
        p.add_argument(name, default="")
    for name in ("--data-randomize",):
        p.add_argument(name, default="total")
    p.add_argument("--data-sub-sample-rate", type=float, default=0.0)
    for name in ("--memory-map", "--data-trace-enable-padding", "--dataset-multiprocessing", "--mlperf-logging", "--mlperf-bin-loader",
                 "--mlperf-bin-shuffle", "--plot-compute-graph", "--save-onnx", "--qr-flag", "--md-flag", "--md-round-dims"):
        p.add_argument(name, action="store_true")
    p.add_argument("--mlperf-acc-threshold", type=float, default=0.0, help="stop once the test accuracy reaches this")
    p.add_argument("--mlperf-auc-threshold", type=float, default=0.0)
    p.add_argument("--mlperf-grad-accum-iter", type=int, default=1)
    p.add_argument("--qr-threshold", type=int, default=200)
    p.add_argument("--qr-operation", default="mult")
    p.add_argument("--qr-collisions", type=int, default=4)
    p.add_argument("--md-threshold", type=int, default=200)
    p.add_argument("--md-temperature", type=float, default=0.3)
    p.add_argument("--quantize-mlp-with-bit", type=int, default=32)
    p.add_argument("--quantize-emb-with-bit", type=int, default=32)
    a = p.parse_args(argv)
    closed = [n for n, on in (("--arch-interaction-itself", a.arch_interaction_itself), ("--weighted-pooling", a.weighted_pooling),
                              ("--qr-flag", a.qr_flag), ("--md-flag", a.md_flag), ("--save-onnx", a.save_onnx),
                              ("--plot-compute-graph", a.plot_compute_graph), ("--mlperf-bin-loader", a.mlperf_bin_loader),
                              ("--quantize-mlp-with-bit", a.quantize_mlp_with_bit != 32),
                              ("--quantize-emb-with-bit", a.quantize_emb_with_bit != 32),
                              ("--mlperf-grad-accum-iter", a.mlperf_grad_accum_iter != 1)) if on]
    if closed:
        p.error("not offered by this engine: " + ", ".join(closed))
    if a.max_ind_range > 0:
        a.arch_embedding_size = [min(n, a.max_ind_range) for n in a.arch_embedding_size]
    if a.num_batches <= 0 and a.data_size > 0:
        a.num_batches = -(-a.data_size // a.mini_batch_size)
    return a


def _trace_id_fn(args):
    """Ids with the stack-distance profile of a recorded access trace (``--data-generation synthetic --data-trace-file F``,
    the trace-driven generator of the reference's dlrm_data_pytorch.py:774-1286): the file holds integers separated by
    commas or white space; every table replays a synthetic trace of that profile, folded into its row count."""
    import re
    from recstore_b200.utils.dlrm_data import trace_generate, trace_profile
    with open(args.data_trace_file) as f:
        trace = [int(x) for x in re.split(r"[,\s]+", f.read().strip()) if x]
    if not trace:
        sys.exit(f"ERROR: {args.data_trace_file} holds no ids")
    uniq, dist, prob = trace_profile(trace)
    calls = [0]

    def fn(n_ids, n_rows, table):
        calls[0] += 1
        return trace_generate(uniq, dist, prob, n_ids, seed=args.numpy_rand_seed * 7919 + calls[0]) % n_rows
    return fn


def roc_auc(scores: torch.Tensor, labels: torch.Tensor) -> float:
    """Area under the ROC curve from ranks (ties get their average rank); NaN if only one class is present."""
    s, y = scores.double().reshape(-1), labels.double().reshape(-1)
    n_pos, n_neg = float(y.sum()), float((1 - y).sum())
    if n_pos == 0 or n_neg == 0:
        return float("nan")
    order = torch.argsort(s)
    ss = s[order]
    ranks = torch.empty_like(ss)
    ranks[:] = torch.arange(1, ss.numel() + 1, dtype=torch.double)
    uniq, inv, cnt = torch.unique_consecutive(ss, return_inverse=True, return_counts=True)      # average rank inside ties
    ends = torch.cumsum(cnt, 0).double()
    ranks = (ends - (cnt.double() - 1) / 2)[inv]
    r_pos = ranks[y[order] > 0.5].sum()
    return float((r_pos - n_pos * (n_pos + 1) / 2) / (n_pos * n_neg))


def lr_at(step: int, base: float, warmup: int, decay_start: int, decay_steps: int) -> float:
    """Learning-rate policy of the reference's driver (dlrm_model.py LRPolicyScheduler): linear warm-up over ``warmup``
    steps, constant, then a quadratic decay from ``decay_start`` over ``decay_steps`` steps down to a floor of 1e-7."""
    step += 1
    if step < warmup:
        return base * step / warmup
    end = decay_start + decay_steps
    if decay_steps > 0 and step >= decay_start:
        if step >= end:
            return 1e-7
        return max(1e-7, base * ((end - step) / decay_steps) ** 2)
    return base


def interaction_width(args) -> int:
    T, D = len(args.arch_embedding_size), args.arch_sparse_feature_size
    if args.arch_interaction_op == "projection":
        return D + args.interaction_branch_sizes[0] * args.interaction_branch_sizes[1]
    return (T + 1) * D if args.arch_interaction_op == "dcn" else D + (T + 1) * T // 2


def validate(args):
    D = args.arch_sparse_feature_size
    if args.arch_mlp_bot[-1] != D:
        sys.exit(f"ERROR: arch-sparse-feature-size {D} does not match last dim of bottom mlp {args.arch_mlp_bot[-1]}")
    w = interaction_width(args)
    if args.arch_mlp_top is None:
        args.arch_mlp_top = [w, 64, 1]
    if args.arch_mlp_top[0] != w:
        sys.exit(f"ERROR: # of feature interactions {w} does not match first dimension of top mlp {args.arch_mlp_top[0]}")
    if args.arch_mlp_top[-1] != 1:
        sys.exit("ERROR: the top mlp must end in one output")


class _CpuModel:
    """Adapter giving the PyTorch restatement the engine's train_step / predict signature."""

    def __init__(self, m):
        self.m = m
        self.rank, self.world = m.rank, m.world

    def train_step(self, b):
        return float(self.m.train_step(b.dense, b.ids, b.labels))

    def predict(self, b):
        return self.m.predict(b.dense, b.ids)

    def set_lr(self, lr):
        self.m.mlp_lr = lr

    def save(self, path, step):
        from recstore_b200.models.checkpoint import save_checkpoint
        save_checkpoint(self.m, path, step)

    def load(self, path):
        from recstore_b200.models.checkpoint import load_checkpoint
        return load_checkpoint(self.m, path)


class _GpuModel:
    def __init__(self, eng):
        self.e = eng
        self.rank, self.world = eng.rank, eng.world

    def _pin(self, b):
        return self.e.make_pinned_batch(b.dense, b.ids, b.labels)

    def train_step(self, b):
        return self.e.train_step(self._pin(b))

    def predict(self, b):
        return self.e.predict(self._pin(b)).float().cpu()

    def set_lr(self, lr):
        self.e.cfg.mlp_lr = lr                    # read at every launch of the (eager) step

    def save(self, path, step):
        self.e.save_checkpoint(path, step)

    def load(self, path):
        return self.e.load_checkpoint(path)


class _DatasetSource:
    """``next()`` over a ``CriteoDataset`` that starts over (reshuffled when asked) at the end of an epoch."""

    def __init__(self, make):
        self.make, self.it = make, None

    def next(self):
        if self.it is None:
            self.it = iter(self.make())
        try:
            return next(self.it)
        except StopIteration:
            self.it = iter(self.make())
            return next(self.it)


def _open_dataset(args):
    """Criteo-format data (``--data-generation dataset``): a preprocessed ``.npz`` (``--processed-data-file``) or the raw
    tab-separated text (``--raw-data-file``: label, 13 integer and 26 hexadecimal categorical columns), preprocessed on the
    fly and cached in the processed file if one is named (dlrm_data_pytorch.py:50-323 and data_utils.py of the
    reference).  Returns the arrays; the table sizes of the model come from the category counts, as the reference does."""
    from recstore_b200.utils import dlrm_data as Dd
    if args.processed_data_file and os.path.exists(args.processed_data_file):
        d = dict(np.load(args.processed_data_file))
    elif args.raw_data_file:
        with open(args.raw_data_file) as f:
            d = Dd.criteo_preprocess(f, args.processed_data_file or None, args.max_ind_range)
    else:
        sys.exit("ERROR: --data-generation dataset needs --raw-data-file or an existing --processed-data-file")
    if args.data_sub_sample_rate > 0.0:                 # drop that share of the negatives (the reference's sub-sampling)
        rng = np.random.default_rng(args.numpy_rand_seed)
        keep = (d["y"] > 0.5) | (rng.random(d["y"].shape[0]) >= args.data_sub_sample_rate)
        d = {"y": d["y"][keep], "X_int": d["X_int"][keep], "X_cat": d["X_cat"][keep], "counts": d["counts"]}
    if d["y"].shape[0] < 2 * args.mini_batch_size:
        sys.exit(f"ERROR: {d['y'].shape[0]} samples are fewer than two mini-batches of {args.mini_batch_size}")
    return d


def run(args) -> dict:
    data = None
    if args.data_generation == "dataset":
        from recstore_b200.utils import dlrm_data as Dd
        data = _open_dataset(args)
        args.arch_embedding_size = [max(1, int(c)) for c in data["counts"]]
        if args.arch_mlp_bot[0] != Dd.NUM_INT:
            sys.exit(f"ERROR: the data has {Dd.NUM_INT} dense features; --arch-mlp-bot must start with {Dd.NUM_INT}")
        args.num_indices_per_lookup = 1
        args.arch_mlp_top = None if args.arch_mlp_top is None else args.arch_mlp_top
    validate(args)
    from recstore_b200.utils.data import DLRMBatchSource
    rows, D = args.arch_embedding_size, args.arch_sparse_feature_size
    hot = [args.num_indices_per_lookup] * len(rows)
    nd = args.arch_mlp_bot[0]
    kw = dict(emb_dim=D, hotness=hot, num_dense=nd, bottom_mlp=tuple(args.arch_mlp_bot[1:]), top_mlp=tuple(args.arch_mlp_top[1:]),
              emb_lr=args.emb_learning_rate if args.emb_learning_rate is not None else args.learning_rate,
              emb_optimizer=args.emb_optimizer, mlp_lr=args.learning_rate, seed=args.numpy_rand_seed,
              interaction=args.arch_interaction_op, dcn_layers=args.dcn_layers, dcn_rank=args.dcn_rank)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    scheduled = args.lr_num_warmup_steps > 0 or args.lr_num_decay_steps > 0
    if args.use_gpu and args.loss_function != "bce":
        sys.exit(f"ERROR: --loss-function {args.loss_function} runs on the PyTorch path only (drop --use-gpu)")
    if args.use_gpu:
        if scheduled:
            kw["use_cuda_graph"] = False          # the learning rate is a launch argument: a replayed graph would freeze it
        if args.enable_profiling:
            kw["trace_phases"] = True
        from recstore_b200.models.dlrm import DLRM, DLRMConfig
        from recstore_b200.parallel.peer import PeerContext
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{local}"))
        model = _GpuModel(DLRM(DLRMConfig(table_rows=rows, batch=args.mini_batch_size,
                                          projection_sizes=tuple(args.interaction_branch_sizes),
                                          projection_hidden=(tuple(args.interaction_branch1_hidden),
                                                             tuple(args.interaction_branch2_hidden)), **kw), ctx))
        if world > 1 and args.heartbeat_timeout > 0:      # liveness word per rank, checked on the host before every launch
            from recstore_b200.utils.liveness import Heartbeat
            hb = Heartbeat(rank, world, name=f"dlrm_heartbeat_{os.environ.get('MASTER_PORT', '0')}",
                           period_s=min(0.2, args.heartbeat_timeout / 5)).start()
            hb.wait_all_alive(max(60.0, args.heartbeat_timeout))
            model.e.heartbeat, model.e.heartbeat_timeout_s = hb, args.heartbeat_timeout
    else:
        from recstore_b200.baseline.dlrm_torch import TorchDLRM
        model = _CpuModel(TorchDLRM(rows, args.mini_batch_size, device="cpu", rank=0, world=1,
                                    projection_sizes=tuple(args.interaction_branch_sizes),
                                    projection_hidden=(tuple(args.interaction_branch1_hidden),
                                                       tuple(args.interaction_branch2_hidden)), **kw))
        model.m.loss_function, model.m.loss_weights = args.loss_function, tuple(args.loss_weights)
    alpha = args.zipf_alpha if args.data_generation == "synthetic" else 0.0
    gauss = ((args.rand_data_mu, args.rand_data_sigma, args.rand_data_min, args.rand_data_max)
             if args.data_generation == "random" and args.rand_data_dist == "gaussian" else None)
    id_fn = _trace_id_fn(args) if (args.data_generation == "synthetic" and args.data_trace_file) else None
    if data is not None:
        from recstore_b200.utils.dlrm_data import CriteoDataset
        shuffle = args.data_randomize in ("total", "day")
        src = _DatasetSource(lambda: CriteoDataset(data, args.mini_batch_size, shuffle=shuffle, seed=args.numpy_rand_seed + 1, split="train"))
        test_src = _DatasetSource(lambda: CriteoDataset(data, args.mini_batch_size, seed=args.numpy_rand_seed + 2, split="test"))
        n_train = len(CriteoDataset(data, args.mini_batch_size, split="train"))
        if args.num_batches <= 0 or args.num_batches > n_train:
            args.num_batches = n_train                    # one epoch = one pass over the training split
        if len(CriteoDataset(data, args.mini_batch_size, split="test")) == 0:
            test_src = _DatasetSource(lambda: CriteoDataset(data, args.mini_batch_size, seed=args.numpy_rand_seed + 2, split="train"))
    else:
        src = DLRMBatchSource(rows, hot, args.mini_batch_size, num_dense=nd, alpha=alpha, seed=args.numpy_rand_seed + 1, gaussian=gauss,
                              id_fn=id_fn)
        test_src = DLRMBatchSource(rows, hot, args.mini_batch_size, num_dense=nd, alpha=alpha, seed=args.numpy_rand_seed + 2,
                                   gaussian=gauss, id_fn=id_fn)
    step0 = 0
    if args.load_model:
        step0 = int(model.load(args.load_model).get("step", 0))
        if rank == 0:
            print(f"Loaded checkpoint {args.load_model} (step {step0})", flush=True)
    losses, t0, done = [], time.time(), 0
    test_acc = None

    last_auc = [float("nan")]

    def test_once():
        tb = test_src.next()
        lo, hi = (model.rank * (args.mini_batch_size // model.world), (model.rank + 1) * (args.mini_batch_size // model.world))
        p = model.predict(tb).reshape(-1)
        if args.loss_threshold > 0:
            p = p.clamp(args.loss_threshold, 1.0 - args.loss_threshold)
        last_auc[0] = roc_auc(p, tb.labels[lo:hi])
        return float(((p > 0.5).float() == tb.labels[lo:hi]).float().mean())

    if args.inference_only:
        accs = [test_once() for _ in range(max(1, args.num_batches))]
        out = {"steps": 0, "inference_batches": len(accs), "test_accuracy": float(np.mean(accs)),
               "ms_per_batch": (time.time() - t0) / len(accs) * 1e3}
        if rank == 0:
            print(json.dumps(out), flush=True)
        _teardown(args, world, model)
        return out
    stop = False
    scalars = None
    if args.tensor_board_filename and rank == 0:          # one JSON object per line: a plain-text stand-in for the event file
        os.makedirs(args.tensor_board_filename, exist_ok=True)
        scalars = open(os.path.join(args.tensor_board_filename, "scalars.jsonl"), "a")
    for ep in range(args.nepochs):
        if stop:
            break
        for j in range(args.num_batches):
            b = src.next()
            if args.round_targets:
                b.labels.round_()
            if scheduled:
                model.set_lr(lr_at(step0 + done, args.learning_rate, args.lr_num_warmup_steps, args.lr_decay_start_step,
                                   args.lr_num_decay_steps))
            loss = model.train_step(b)
            losses.append(loss)
            done += 1
            if scalars is not None:
                scalars.write(json.dumps({"step": step0 + done, "epoch": ep, "train_loss": float(loss)}) + "\n")
            if rank == 0 and args.print_freq and done % args.print_freq == 0:
                el = (time.time() - t0) / done * 1e3
                print(f"Finished training it {j + 1}/{args.num_batches} of epoch {ep}, {el:.2f} ms/it, "
                      f"loss {np.mean(losses[-args.print_freq:]):.6f}", flush=True)
            if args.test_freq and done % args.test_freq == 0:
                test_acc = test_once()
                if rank == 0:
                    print(f"Testing at - {done}: accuracy {test_acc * 100:.3f} % (rank 0 share)", flush=True)
                if scalars is not None:
                    scalars.write(json.dumps({"step": step0 + done, "test_accuracy": test_acc, "test_auc": last_auc[0]}) + "\n")
                reached_auc = args.mlperf_auc_threshold > 0 and last_auc[0] >= args.mlperf_auc_threshold
                if (reached_auc or (args.mlperf_acc_threshold > 0 and test_acc >= args.mlperf_acc_threshold)) and world == 1:
                    stop = True                   # the reference's early exit once the accuracy target is met
                    break
    if scalars is not None:
        scalars.close()
    if args.save_model:
        model.save(args.save_model, step0 + done)
        if rank == 0:
            print(f"Saved checkpoint {args.save_model}", flush=True)
    out = {"steps": done, "first_loss": losses[0] if losses else None, "last_loss": losses[-1] if losses else None,
           "mean_last_10": float(np.mean(losses[-10:])) if losses else None, "test_accuracy": test_acc,
           "test_auc": None if last_auc[0] != last_auc[0] else last_auc[0]}
    if args.print_time or args.print_wall_time:
        out["ms_per_iteration"] = (time.time() - t0) / max(1, done) * 1e3
    if args.enable_profiling and args.use_gpu:
        out["phases_us"] = {k: round(v, 1) for k, v in model.e.phase_times().items()}
    if rank == 0:
        print(json.dumps(out), flush=True)
    _teardown(args, world, model)
    return out


def _teardown(args, world, model=None):
    if args.use_gpu and world > 1:
        import torch.distributed as dist
        dist.barrier()
        hb = getattr(getattr(model, "e", None), "heartbeat", None)
        if hb is not None:                   # after the barrier: a rank that finishes early keeps beating until all are done
            hb.stop(leaving=True)
        dist.destroy_process_group()


def main(argv=None):
    return run(parse_args(argv))


if __name__ == "__main__":
    main()
