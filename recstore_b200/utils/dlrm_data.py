"""DLRM input data: Criteo click logs, random batches, and trace-driven synthetic ids.

* ``criteo_preprocess`` / ``CriteoDataset``: the Criteo Kaggle / Terabyte text format (label, 13 integer features,
  26 hexadecimal categorical features, tab separated, missing values allowed) -> ``log(1 + x)`` dense features and
  per-feature dictionary ids, stored as one ``.npz`` (``X_int, X_cat, y, counts``) as the reference's preprocessing does
  (src/executable/dlrm/data_utils.py, dlrm_data_pytorch.py:50-323).  No dataset ships with an air-gapped box; the
  parser is exercised on generated lines.
* ``RandomDataset``: uniform or Zipf ids with fixed or variable bag lengths (dlrm_data_pytorch.py:572-772).
* ``trace_profile`` / ``trace_generate``: stack-distance profile of an id trace and a synthetic trace with the same
  reuse behaviour (dlrm_data_pytorch.py:1041-1286): the generator draws a stack distance from the measured
  distribution and emits the id found at that depth of an LRU stack (or a new id for a cold miss).
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .data import DLRMBatch, zipf_ids

NUM_INT, NUM_CAT = 13, 26


def criteo_preprocess(lines: Iterable[str], out_path: Optional[str] = None, max_ind_range: int = -1) -> Dict[str, np.ndarray]:
    """Parses Criteo text lines; categorical values are renumbered densely per feature in order of first appearance
    (optionally folded modulo ``max_ind_range`` first, as ``--max-ind-range`` of the reference does)."""
    ys, xi, xc = [], [], []
    dicts: List[Dict[int, int]] = [dict() for _ in range(NUM_CAT)]
    for line in lines:
        f = line.rstrip("\n").split("\t")
        if len(f) != 1 + NUM_INT + NUM_CAT:
            continue
        ys.append(int(f[0] or 0))
        xi.append([max(int(v), 0) if v not in ("", None) else 0 for v in f[1:1 + NUM_INT]])
        row = []
        for j, v in enumerate(f[1 + NUM_INT:]):
            h = int(v, 16) if v else 0
            if max_ind_range > 0:
                h %= max_ind_range
            row.append(dicts[j].setdefault(h, len(dicts[j])))
        xc.append(row)
    out = {"y": np.array(ys, dtype=np.float32), "X_int": np.array(xi, dtype=np.float32).reshape(-1, NUM_INT),
           "X_cat": np.array(xc, dtype=np.int64).reshape(-1, NUM_CAT), "counts": np.array([len(d) for d in dicts], dtype=np.int64)}
    if out_path:
        np.savez_compressed(out_path, **out)
    return out


def create_mini_dataset(src_npz: str, dst_npz: str, n_samples: int = 100_000) -> int:
    """Truncates a preprocessed ``.npz`` to its first ``n_samples`` samples and re-counts the categories that remain
    (the role of the reference's create_mini_dataset.py, which cuts its id / offset / label arrays to 100 k samples)."""
    d = np.load(src_npz)
    n = min(int(n_samples), int(d["y"].shape[0]))
    xc = d["X_cat"][:n]
    counts = np.array([int(xc[:, j].max()) + 1 if n else 0 for j in range(xc.shape[1])], dtype=np.int64)
    np.savez_compressed(dst_npz, y=d["y"][:n], X_int=d["X_int"][:n], X_cat=xc, counts=counts)
    return n


class CriteoDataset:
    """Batches of a preprocessed ``.npz`` in the engine's input form (global batch, ids per table)."""

    def __init__(self, npz_path_or_dict, batch: int, shuffle: bool = False, seed: int = 0, split: str = "train", test_frac: float = 0.1):
        d = np.load(npz_path_or_dict) if isinstance(npz_path_or_dict, (str, os.PathLike)) else npz_path_or_dict
        n = d["y"].shape[0]
        cut = int(n * (1 - test_frac))
        sl = slice(0, cut) if split == "train" else slice(cut, n)
        self.y, self.xi, self.xc = d["y"][sl], np.log1p(d["X_int"][sl]), d["X_cat"][sl]
        self.counts = [int(c) for c in d["counts"]]
        self.batch, self.rng, self.shuffle = batch, np.random.default_rng(seed), shuffle

    @property
    def table_rows(self) -> List[int]:
        return [max(1, c) for c in self.counts]

    def __len__(self) -> int:
        return self.y.shape[0] // self.batch

    def __iter__(self) -> Iterator[DLRMBatch]:
        order = self.rng.permutation(self.y.shape[0]) if self.shuffle else np.arange(self.y.shape[0])
        for b in range(len(self)):
            i = order[b * self.batch:(b + 1) * self.batch]
            yield DLRMBatch(torch.from_numpy(self.xi[i].astype(np.float32)), [torch.from_numpy(self.xc[i, t].copy()) for t in range(NUM_CAT)],
                            torch.from_numpy(self.y[i]))


class RandomDataset:
    """``num_batches`` random global batches; bag lengths fixed (``num_indices_per_lookup_fixed``) or uniform in
    ``[1, num_indices_per_lookup]`` with offsets, ids uniform or Zipf."""

    def __init__(self, table_rows: Sequence[int], num_dense: int, batch: int, num_batches: int, num_indices_per_lookup: int = 1,
                 fixed: bool = True, alpha: float = 0.0, seed: int = 0):
        self.rows, self.nd, self.batch, self.nb = list(table_rows), num_dense, batch, num_batches
        self.L, self.fixed, self.alpha = num_indices_per_lookup, fixed, alpha
        self.rng = np.random.default_rng(seed)

    def __len__(self):
        return self.nb

    def __iter__(self):
        for _ in range(self.nb):
            dense = torch.from_numpy(np.log1p(self.rng.exponential(1.0, (self.batch, self.nd))).astype(np.float32))
            labels = torch.from_numpy((self.rng.random(self.batch) < 0.5).astype(np.float32))
            ids, offsets = [], []
            for n in self.rows:
                lens = np.full(self.batch, self.L) if self.fixed else self.rng.integers(1, self.L + 1, self.batch)
                ids.append(torch.from_numpy(zipf_ids(int(lens.sum()), n, self.alpha, self.rng)))
                offsets.append(torch.from_numpy(np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int64)))
            b = DLRMBatch(dense, ids, labels)
            b.offsets = offsets
            yield b


def trace_profile(trace: Sequence[int]) -> Tuple[List[int], np.ndarray, np.ndarray]:
    """-> (ids in order of first appearance, distinct stack distances, their probabilities).  Distance 0 = cold miss
    (first reference); distance d >= 1 = the id was the d-th most recently used distinct id."""
    stack: List[int] = []
    uniq: List[int] = []
    dist: Dict[int, int] = {}
    for x in trace:
        x = int(x)
        if x in stack:
            d = len(stack) - stack.index(x)
            stack.remove(x)
        else:
            d = 0
            uniq.append(x)
        stack.append(x)
        dist[d] = dist.get(d, 0) + 1
    ds = np.array(sorted(dist), dtype=np.int64)
    p = np.array([dist[int(d)] for d in ds], dtype=np.float64)
    return uniq, ds, p / p.sum()


def trace_generate(uniq: Sequence[int], distances: np.ndarray, probs: np.ndarray, n: int, seed: int = 0) -> np.ndarray:
    """Synthetic trace of length ``n`` with the stack-distance distribution of the profiled one."""
    rng = np.random.default_rng(seed)
    stack: List[int] = []
    fresh = list(uniq)
    nxt = 0
    out = np.empty(n, dtype=np.int64)
    for i in range(n):
        d = int(rng.choice(distances, p=probs))
        if d == 0 or d > len(stack):
            if nxt < len(fresh):
                x = fresh[nxt]; nxt += 1
            elif stack:                      # every known id has been introduced: fall back to the coldest one
                x = stack.pop(0)
            else:
                x = 0
        else:
            x = stack.pop(len(stack) - d)
        stack.append(x)
        out[i] = x
    return out
