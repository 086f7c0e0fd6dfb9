"""``bench.py --impl reference``: the UNMODIFIED reference DLRM on the same config.

What is run: ``DLRM_Net`` of the reference's DLRM fork (src/executable/dlrm/dlrm_model.py:71-423),
through its own constructor, ``forward`` (``sequential_forward`` on one GPU,
``distributed_forward`` with ``extend_distributed.alltoall`` + DDP MLPs on several), its own
``loss_fn`` and the optimizer its ``run()`` builds for GPUs (``torch.optim.SGD`` over the sparse
``nn.EmbeddingBag`` gradients and the MLPs, dlrm_model.py:1039-1068; the reference exits on
"GPU version of Adagrad is not supported", :1040-1041, so SGD is its only stock GPU optimizer; it
computes in fp32).  None of this package's models, kernels or engine is on that path; this module
only generates the synthetic batch, calls the reference and times it.

Where the files come from: the reference tree is not pip-installable (no setup.py /
pyproject.toml) and its native parts do not build offline, so the four pure-Python files of the
DLRM fork are copied verbatim into ``baseline/_ref/dlrm``.  ``torch.utils.tensorboard`` (imported at
module level by dlrm_model.py for logging, never used here) needs the ``tensorboard`` package,
which is absent: a stand-in module with an inert ``SummaryWriter`` is registered before the import.
If the files are missing, the arm reports itself unavailable and exits 0.
"""
from __future__ import annotations

import contextlib
import io
import json
import os
import sys
import time
import types

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline", "_ref", "dlrm")
NEEDED = ("dlrm_model.py", "extend_distributed.py", "dlrm_data_pytorch.py", "data_utils.py")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _import_reference():
    if "torch.utils.tensorboard" not in sys.modules:
        try:
            import torch.utils.tensorboard  # noqa: F401
        except Exception:
            stub = types.ModuleType("torch.utils.tensorboard")

            class SummaryWriter:  # inert stand-in for the absent tensorboard package
                def __init__(self, *a, **k): pass
                def add_scalar(self, *a, **k): pass
                def close(self): pass

            stub.SummaryWriter = SummaryWriter
            sys.modules["torch.utils.tensorboard"] = stub
    sys.path.insert(0, REF_DIR)
    import extend_distributed as ext_dist
    import dlrm_model
    return ext_dist, dlrm_model


def main(args) -> None:
    if not all(os.path.exists(os.path.join(REF_DIR, f)) for f in NEEDED):
        _unavailable("reference is not installable with pip (no setup.py/pyproject.toml) and its DLRM sources are "
                     "not present under baseline/_ref/dlrm")
        return
    import numpy as np
    import torch
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    import bench as B
    from recstore_b200.utils.data import DLRMBatchSource

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    quiet = io.StringIO()
    try:
        with contextlib.redirect_stdout(quiet):
            ext_dist, dm = _import_reference()
            torch.cuda.set_device(local)
            ext_dist.init_distributed(rank=rank if world > 1 else -1, local_rank=local, size=world if world > 1 else -1,
                                      use_gpu=True, backend="nccl" if world > 1 else "")
    except Exception as e:
        _unavailable(f"reference import/initialisation failed: {type(e).__name__}: {e}")
        return
    device = torch.device("cuda", local)
    rows = B.table_rows(args.seed)
    ln_emb = np.array(rows)
    ln_bot = np.array([13, 512, 256, 128])
    ln_top = np.array([479, 1024, 1024, 512, 256, 1])
    np.random.seed(args.seed)
    torch.manual_seed(args.seed)
    with contextlib.redirect_stdout(quiet):
        dlrm = dm.DLRM_Net(128, ln_emb, ln_bot, ln_top, arch_interaction_op="dot", arch_interaction_itself=False,
                           sigmoid_bot=-1, sigmoid_top=ln_top.size - 2, sync_dense_params=True, loss_threshold=0.0,
                           ndevices=1, loss_function="bce")
        dlrm = dlrm.to(device)
        if world > 1:
            dlrm.bot_l = ext_dist.DDP(dlrm.bot_l, device_ids=[local])
            dlrm.top_l = ext_dist.DDP(dlrm.top_l, device_ids=[local])
    lr = 0.01
    if world == 1:
        params = dlrm.parameters()
    else:
        params = [{"params": [p for emb in dlrm.emb_l for p in emb.parameters()], "lr": lr},
                  {"params": dlrm.bot_l.parameters(), "lr": lr}, {"params": dlrm.top_l.parameters(), "lr": lr}]
    optimizer = torch.optim.SGD(params, lr=lr)

    BATCH, T = B.BATCH, B.TABLES
    Bl = BATCH // world
    src = DLRMBatchSource(rows, [1] * T, BATCH, alpha=B.ALPHA, seed=args.seed + 1)
    nb = 4
    host = []
    offsets = torch.arange(BATCH, dtype=torch.int64)
    for _ in range(nb):
        b = src.next()
        host.append((b.dense.pin_memory(), [i.pin_memory() for i in b.ids],
                     b.labels[rank * Bl:(rank + 1) * Bl].reshape(-1, 1).contiguous().pin_memory()))
    off_dev = offsets.unsqueeze(0).repeat(T, 1).to(device)   # stacked [T, B]: the reference prints lS_o.shape

    def to_dev(hb):
        X, ids, y = hb
        return X.to(device, non_blocking=True), [i.to(device, non_blocking=True) for i in ids], y.to(device, non_blocking=True)

    def step(X, ids, y):
        optimizer.zero_grad()
        with contextlib.redirect_stdout(quiet):       # sequential_forward prints tensor shapes every call
            Z = dlrm(X, off_dev, ids)
        E = dlrm.loss_fn(Z, y)
        E.backward()
        optimizer.step()
        quiet.seek(0); quiet.truncate(0)
        return E

    devb = [to_dev(h) for h in host]
    W = max(args.warmup, 3)
    try:
        for i in range(W):
            step(*devb[i % nb])
    except Exception as e:
        _unavailable(f"reference step failed: {type(e).__name__}: {str(e)[:200]}")
        return
    sampler = B.ClockSampler(local)
    B.barrier(world)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(*devb[i % nb])
    e1.record()
    B.barrier(world)
    clocks = sampler.stop() if rank == 0 else None
    ms_dev = B.max_over_ranks(e0.elapsed_time(e1), world)
    B.barrier(world)
    t0 = time.perf_counter()
    last = None
    for i in range(args.steps):
        E = step(*to_dev(host[i % nb]))
        last = float(E.item())
    torch.cuda.synchronize()
    ms_e2e = B.max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    h2d = host[0][0].numel() * 4 + sum(i.numel() * 8 for i in host[0][1]) + host[0][2].numel() * 4
    if rank == 0:
        print(json.dumps({
            "metric": B.METRIC, "value": BATCH * args.steps / (ms_dev * 1e-3), "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": W, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (the reference's own precision)",
            "data": "synthetic (Zipf 1.2 ids, random-init weights)", "impl": "reference",
            "config": {"model": "reference DLRM_Net, dot interaction, 26 tables x dim 128, ~34M rows, bot 13-512-256-128, "
                                "top 479-1024-1024-512-256-1", "global_batch": BATCH,
                       "parallelism": f"table-wise MP embeddings x{world} (all_to_all) + DDP MLP x{world}",
                       "optimizer": "torch.optim.SGD on sparse EmbeddingBag grads and MLPs (the reference refuses Adagrad on GPUs)"},
            "clocks": clocks,
            "e2e": {"value": BATCH * args.steps / (ms_e2e * 1e-3), "unit": "samples/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "last_loss": last}), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
