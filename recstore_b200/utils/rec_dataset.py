"""Click-log datasets as flat id streams: Criteo Kaggle (26 categorical features), Avazu (21), Criteo Terabyte (26).

On-disk form (what the reference's loader reads, src/executable/dlrm/rec_dataloader.py:20-47): ``<root>/<name>.npy``, an
int64 array ``[num_samples, num_features]`` of per-feature ids, and ``<root>/<name>_offsets.npy``, the first global id
of every feature (``num_features + 1`` entries, the last one is the total number of embeddings).  When the files are
absent (no datasets on an air-gapped box) the loader synthesises a stream of the same shape: per-feature
cardinalities spread log-uniformly, Zipf-distributed ids.
"""
from __future__ import annotations

import os
from typing import Iterator, Optional

import numpy as np
import torch

from .data import loguniform_table_rows, zipf_ids

NUM_FEATURES = {"criteo": 26, "avazu": 21, "criteoTB": 26}
DEFAULT_TOTAL = {"criteo": 33_762_577, "avazu": 9_449_445, "criteoTB": 882_774_592}


class RecDatasetLoader:
    def __init__(self, dataset: str, batch_size: int, root: Optional[str] = None, rank: int = 0, world: int = 1,
                 synthetic_total: Optional[int] = None, alpha: float = 1.05, seed: int = 0):
        assert dataset in NUM_FEATURES, f"unknown dataset {dataset}"
        self.dataset, self.batch_size, self.rank, self.world = dataset, batch_size, rank, world
        self.F = NUM_FEATURES[dataset]
        self.ids = None
        path = os.path.join(root, f"{dataset}.npy") if root else None
        if path and os.path.exists(path):
            self.ids = np.load(path, mmap_mode="r")
            assert self.ids.ndim == 2 and self.ids.shape[1] == self.F, self.ids.shape
            self.offsets = np.load(os.path.join(root, f"{dataset}_offsets.npy")).astype(np.int64)
            assert self.offsets.size == self.F + 1
            self.synthetic = False
        else:
            total = synthetic_total or min(DEFAULT_TOTAL[dataset], 10_000_000)
            rows = loguniform_table_rows(self.F, 4, max(8, total // 3), total, seed)
            self.offsets = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
            self.synthetic = True
        self.rows = np.diff(self.offsets)
        self.alpha = alpha
        self.rng = np.random.default_rng(seed * 1000 + rank + 1)
        self.cursor = rank * batch_size

    @property
    def num_embeddings(self) -> int:
        return int(self.offsets[-1])

    def next_batch(self) -> torch.Tensor:
        """-> int64 ``[batch_size, num_features]`` of GLOBAL ids (feature offset added)."""
        B = self.batch_size
        if self.ids is not None:
            n = self.ids.shape[0]
            idx = (self.cursor + np.arange(B)) % n
            self.cursor = (self.cursor + B * self.world) % n
            local = np.asarray(self.ids[np.sort(idx)], dtype=np.int64)
        else:
            local = np.stack([zipf_ids(B, int(r), self.alpha, self.rng) for r in self.rows], 1)
        return torch.from_numpy(local + self.offsets[:-1][None, :])

    def __iter__(self) -> Iterator[torch.Tensor]:
        while True:
            yield self.next_batch()
