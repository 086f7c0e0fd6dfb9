"""Checkpoints of a DLRM trainer: one directory, dense weights from rank 0, every table from its owner.

    <dir>/meta.json          table rows, embedding width, MLP shapes, interaction, step counter, world size at save time
    <dir>/dense.pt           {"bot.0.weight": ..., "head.bias": ...}  (fp32, torch.save)
    <dir>/table_<t>.pt       {"weight": [rows, D] fp32, "state": [rows] fp32 row-wise Adagrad accumulator}
    <dir>/table_<t>.shard<r>of<w>.pt   the same for a table that is spread row-wise over w ranks: rank r's rows
                                        (ids r, r + w, r + 2w, ...), one file per rank

Every file carries the step of the save it belongs to, and ``meta.json`` is replaced last (atomically): a save that was
interrupted leaves the old ``meta.json`` beside some newer files, and ``load_checkpoint`` refuses that mix ("torn
checkpoint") instead of restoring tables and dense weights of different steps.  Files are read with
``weights_only=True`` (tensors only, no pickled code) and checked for shape before anything is copied into the model.

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
    split = set(getattr(model, "split_tables", []))
    world = getattr(model, "world", 1)
    for t in model.local_tables:
        name = f"table_{t}.shard{rank}of{world}.pt" if t in split else f"table_{t}.pt"
        tmp = os.path.join(path, "." + name + ".tmp")
        torch.save({"weight": model.table_weight(t).detach().cpu(), "state": model.table_state(t).detach().cpu(),
                    "save_step": torch.tensor(int(step))}, tmp)
        os.replace(tmp, os.path.join(path, name))
    if rank == 0:
        tmp = os.path.join(path, ".dense.pt.tmp")
        dense = {k: v.detach().cpu() for k, v in model.dense_state().items()}
        dense["__save_step__"] = torch.tensor(int(step))
        torch.save(dense, tmp)
        os.replace(tmp, os.path.join(path, "dense.pt"))
        meta = {"format": 2, "step": int(step), "world_at_save": getattr(model, "world", 1)}
        meta.update(model.describe())
        meta.update(extra or {})
        tmp = os.path.join(path, ".meta.json.tmp")
        with open(tmp, "w") as f:
            json.dump(meta, f, indent=1)
        os.replace(tmp, os.path.join(path, "meta.json"))      # last: the files above are complete when this appears


def load_checkpoint(model, path: str) -> dict:
    with open(os.path.join(path, "meta.json")) as f:
        meta = json.load(f)
    mine = model.describe()
    for k in ("table_rows", "emb_dim", "bottom_mlp", "top_mlp", "interaction"):
        if k in meta and list(meta[k]) != list(mine[k]) if isinstance(mine[k], (list, tuple)) else meta.get(k, mine[k]) != mine[k]:
            raise ValueError(f"checkpoint {path} was written for {k}={meta[k]}, this model has {mine[k]}")
    step = meta.get("step") if meta.get("format", 1) >= 2 else None
    dense = _read(os.path.join(path, "dense.pt"), "dense.pt")
    _same_save(dense.pop("__save_step__", None), step, path, "dense.pt")
    want = {k: v.numel() for k, v in model.dense_state().items()}     # sizes, not shapes: the engine and the PyTorch
    have = {k: v.numel() for k, v in dense.items()}                   # restatement lay some vectors out differently
    if want != have:
        bad = sorted(k for k in set(want) | set(have) if want.get(k) != have.get(k))
        raise ValueError(f"checkpoint {path}: dense.pt does not fit this model (first differences: {bad[:4]})")
    split = set(getattr(model, "split_tables", []))
    rank, world = getattr(model, "rank", 0), getattr(model, "world", 1)
    loaded = {}
    for t in model.local_tables:             # read and check everything first: a bad file must not leave the model half restored
        d = _load_table(path, t, int(mine["table_rows"][t]), int(mine["emb_dim"]), step)
        if t in split:       # this rank keeps ids rank, rank + world, ...
            d = {"weight": d["weight"][rank::world], "state": d["state"][rank::world]}
        if tuple(d["weight"].shape) != tuple(model.table_weight(t).shape) or tuple(d["state"].shape) != tuple(model.table_state(t).shape):
            raise ValueError(f"checkpoint {path}: table {t} holds {tuple(d['weight'].shape)}, this model expects "
                             f"{tuple(model.table_weight(t).shape)}")
        loaded[t] = d
    model.load_dense_state(dense)
    for t, d in loaded.items():
        model.table_weight(t).copy_(d["weight"])
        model.table_state(t).copy_(d["state"])
    return meta


def _read(file: str, what: str) -> dict:
    try:
        d = torch.load(file, map_location="cpu", weights_only=True)
    except FileNotFoundError:
        raise
    except Exception as e:                       # truncated, bit-flipped or not a tensor file at all
        raise ValueError(f"checkpoint file {file} is damaged or not a tensor file: {type(e).__name__}: {e}") from e
    if not isinstance(d, dict):
        raise ValueError(f"checkpoint file {file}: expected a dict of tensors ({what})")
    return d


def _same_save(got, step, path: str, what: str) -> None:
    if step is not None and got is not None and int(got) != int(step):
        raise ValueError(f"torn checkpoint {path}: meta.json is of step {step}, {what} of step {int(got)} "
                         "(a save was interrupted; use an older complete checkpoint)")


def _load_table(path: str, t: int, rows: int, dim: int, step=None) -> dict:
    """The whole table ``t`` from its file, or re-interleaved from the shard files of a row-wise spread save."""
    whole = os.path.join(path, f"table_{t}.pt")
    if os.path.exists(whole):
        d = _read(whole, f"table {t}")
        _same_save(d.pop("save_step", None), step, path, f"table_{t}.pt")
        if "weight" not in d or "state" not in d:
            raise ValueError(f"checkpoint file {whole} has no weight / state")
        return d
    import glob
    import re
    shards = {}
    for f in glob.glob(os.path.join(path, f"table_{t}.shard*of*.pt")):
        m = re.search(r"shard(\d+)of(\d+)\.pt$", f)
        shards[int(m.group(1))] = (int(m.group(2)), f)
    if not shards:
        raise FileNotFoundError(f"checkpoint {path} has no file for table {t}")
    w = next(iter(shards.values()))[0]
    if sorted(shards) != list(range(w)):
        raise ValueError(f"checkpoint {path}: table {t} needs shards 0..{w - 1}, found {sorted(shards)}")
    weight, state = torch.empty(rows, dim), torch.empty(rows)
    for r, (_, f) in shards.items():
        d = _read(f, f"table {t}, shard {r}")
        _same_save(d.pop("save_step", None), step, path, os.path.basename(f))
        if tuple(d["weight"].shape) != tuple(weight[r::w].shape):
            raise ValueError(f"checkpoint file {f} holds {tuple(d['weight'].shape)}, expected {tuple(weight[r::w].shape)}")
        weight[r::w] = d["weight"]
        state[r::w] = d["state"]
    return {"weight": weight, "state": state}
