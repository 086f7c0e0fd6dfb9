"""Checkpoints of a DLRM trainer: one directory, dense weights from rank 0, every table from its owner.

    <dir>/meta.json          table rows, embedding width, MLP shapes, interaction, step counter, world size at save time
    <dir>/dense.pt           {"bot.0.weight": ..., "head.bias": ...}  (fp32, torch.save)
    <dir>/table_<t>.pt       {"weight": [rows, D] fp32, "state": [rows] fp32 row-wise Adagrad accumulator}

Tables are keyed by table index, not by rank, so a checkpoint written by N ranks loads on M ranks (each rank reads
the tables it owns under the new placement) and moves between the GPU engine and the PyTorch restatement: both
expose ``dense_state / load_dense_state / local_tables / table_weight / table_state``.  The reference DLRM saves a
single ``torch.save`` dict of the whole model from rank 0 (src/executable/dlrm/dlrm_model.py:1252-1291); per-table
files are what makes the save scale with the tables and reshard on load.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch


def save_checkpoint(model, path: str, step: int = 0, extra: Optional[dict] = None) -> None:
    os.makedirs(path, exist_ok=True)
    rank = getattr(model, "rank", 0)
    for t in model.local_tables:
        tmp = os.path.join(path, f".table_{t}.pt.tmp")
        torch.save({"weight": model.table_weight(t).detach().cpu(), "state": model.table_state(t).detach().cpu()}, tmp)
        os.replace(tmp, os.path.join(path, f"table_{t}.pt"))
    if rank == 0:
        tmp = os.path.join(path, ".dense.pt.tmp")
        torch.save({k: v.detach().cpu() for k, v in model.dense_state().items()}, tmp)
        os.replace(tmp, os.path.join(path, "dense.pt"))
        meta = {"format": 1, "step": int(step), "world_at_save": getattr(model, "world", 1)}
        meta.update(model.describe())
        meta.update(extra or {})
        with open(os.path.join(path, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)


def load_checkpoint(model, path: str) -> dict:
    with open(os.path.join(path, "meta.json")) as f:
        meta = json.load(f)
    mine = model.describe()
    for k in ("table_rows", "emb_dim", "bottom_mlp", "top_mlp", "interaction"):
        if k in meta and list(meta[k]) != list(mine[k]) if isinstance(mine[k], (list, tuple)) else meta.get(k, mine[k]) != mine[k]:
            raise ValueError(f"checkpoint {path} was written for {k}={meta[k]}, this model has {mine[k]}")
    model.load_dense_state(torch.load(os.path.join(path, "dense.pt"), map_location="cpu"))
    for t in model.local_tables:
        d = torch.load(os.path.join(path, f"table_{t}.pt"), map_location="cpu")
        model.table_weight(t).copy_(d["weight"])
        model.table_state(t).copy_(d["state"])
    return meta
