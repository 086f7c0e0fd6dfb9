"""Synthetic data generators shared by tests, baselines and benchmarks.

* ``zipf_ids``: bounded Zipf-like ids for ANY exponent (the reference's generator,
  ``mehcached_zipf`` in src/base/zipf.h:78-175, only supports theta < 1; the benchmark configs
  need alpha up to 1.3).  Inverse-CDF of the continuous density x^-alpha on [1, N+1), floored,
  so the same closed form runs in numpy, in torch on the CPU and in torch on the GPU and gives
  identical ids for identical uniforms.
* ``loguniform_table_rows``: per-table row counts log-uniform in [lo, hi], rescaled to a target
  total, reproducible from a seed.
* ``powerlaw_triples``: KG triples whose head/tail entity degrees follow a power law.
* ``DLRMBatchSource``: endless stream of (dense, sparse ids, labels) batches of the DLRM
  benchmark shapes (dense = log(1 + Exp(1)), labels ~ Bernoulli(0.25)), mirroring
  make_random_data_and_loader of the reference (src/executable/dlrm/dlrm_data_pytorch.py:572-772).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


def zipf_from_uniform(u, n_rows: int, alpha: float):
    """Maps uniforms in [0,1) to ids in [0, n_rows) with P(id = k) ~ (k+1)^-alpha (continuous approx.)."""
    is_torch = isinstance(u, torch.Tensor)
    n1 = float(n_rows) + 1.0
    if abs(alpha - 1.0) < 1e-9:
        x = (torch.exp(u * math.log(n1)) if is_torch else np.exp(u * math.log(n1)))
    else:
        e = 1.0 - alpha
        c = n1 ** e - 1.0
        x = (u * c + 1.0) ** (1.0 / e)
    if is_torch:
        k = torch.clamp(torch.floor(x).to(torch.int64) - 1, 0, n_rows - 1)
    else:
        k = np.clip(np.floor(x).astype(np.int64) - 1, 0, n_rows - 1)
    return k


def zipf_ids(n: int, n_rows: int, alpha: float, rng: np.random.Generator) -> np.ndarray:
    return zipf_from_uniform(rng.random(n), n_rows, alpha)


def zipf_ids_torch(n: int, n_rows: int, alpha: float, generator: Optional[torch.Generator] = None,
                   device="cpu") -> torch.Tensor:
    u = torch.rand(n, generator=generator, device=device, dtype=torch.float64)
    return zipf_from_uniform(u, n_rows, alpha)


def device_uniform_ids(n: int, n_rows: int, seed: int, counter: int, out: Optional[torch.Tensor] = None, device="cuda") -> torch.Tensor:
    """``n`` uniform ids in ``[0, n_rows)`` drawn on the device: element i comes from ``hash(seed, counter + i)``."""
    from .. import _lib
    _register_gen()
    if out is None:
        out = torch.empty(n, dtype=torch.int64, device=device)
    _lib.call("rs_gen_uniform_ids", out.data_ptr(), n, n_rows, seed & 0xFFFFFFFFFFFFFFFF, counter, _lib.stream_ptr())
    return out


def device_zipf_ids(n: int, n_rows: int, alpha: float, seed: int, counter: int, out: Optional[torch.Tensor] = None, device="cuda",
                    spread: bool = False) -> torch.Tensor:
    """``n`` bounded Zipf-like ids drawn on the device with the closed form of :func:`zipf_from_uniform`.  ``spread``
    applies the affine permutation of :func:`powerlaw_triples` so that the popular ids do not all sit on one shard."""
    from .. import _lib
    _register_gen()
    if out is None:
        out = torch.empty(n, dtype=torch.int64, device=device)
    a, b = (spread_permutation(n_rows) if spread else (0, 0))
    _lib.call("rs_gen_zipf_ids", out.data_ptr(), n, n_rows, float(alpha), seed & 0xFFFFFFFFFFFFFFFF, counter, a, b, _lib.stream_ptr())
    return out


def spread_permutation(n_rows: int) -> Tuple[int, int]:
    """Multiplier (coprime to ``n_rows``) and offset of the popularity-rank -> id permutation."""
    a = 0x9E3779B97F4A7C15 % n_rows | 1
    while math.gcd(a, n_rows) != 1:
        a += 2
    return a, 12345


_gen_registered = False


def _register_gen():
    global _gen_registered
    if not _gen_registered:
        import ctypes as C
        from .. import _lib
        _lib.register_signatures({
            "rs_gen_uniform_ids": (C.c_int, [C.c_void_p, C.c_longlong, C.c_longlong, C.c_ulonglong, C.c_ulonglong, C.c_void_p]),
            "rs_gen_zipf_ids": (C.c_int, [C.c_void_p, C.c_longlong, C.c_longlong, C.c_double, C.c_ulonglong, C.c_ulonglong,
                                          C.c_ulonglong, C.c_ulonglong, C.c_void_p]),
            "rs_gen_draw": (C.c_ulonglong, [C.c_ulonglong, C.c_ulonglong]),
        })
        _gen_registered = True


def loguniform_table_rows(num_tables: int, lo: int, hi: int, total: Optional[int], seed: int,
                          pin_largest: Optional[int] = None) -> List[int]:
    """Row counts drawn log-uniform in [lo, hi] from ``seed``; rescaled (and clamped) so the sum is ~``total``."""
    rng = np.random.default_rng(seed)
    rows = np.exp(rng.uniform(math.log(lo), math.log(hi), size=num_tables))
    if pin_largest is not None:
        rows[np.argmax(rows)] = pin_largest
    if total is not None:
        for _ in range(50):
            free = rows < hi if pin_largest is None else (rows < hi) & (rows != pin_largest)
            s = rows.sum()
            if abs(s - total) / total < 1e-3 or not free.any():
                break
            scale = (total - rows[~free].sum()) / max(rows[free].sum(), 1.0)
            rows[free] = np.clip(rows[free] * scale, lo, hi)
    return [int(max(lo, min(hi, round(r)))) for r in rows]


def powerlaw_triples(n_triples: int, n_entities: int, n_relations: int, alpha: float, seed: int):
    """(head, rel, tail) int64 arrays; entity popularity ~ rank^-alpha, relations uniform."""
    rng = np.random.default_rng(seed)
    h = zipf_ids(n_triples, n_entities, alpha, rng)
    t = zipf_ids(n_triples, n_entities, alpha, rng)
    # decorrelate popularity rank from id so that hot entities are spread over all shards
    a, b = spread_permutation(n_entities)
    h = (h * a + b) % n_entities
    t = (t * a + b) % n_entities
    r = rng.integers(0, n_relations, size=n_triples, dtype=np.int64)
    return h, r, t


@dataclass
class DLRMBatch:
    dense: torch.Tensor            # [B, num_dense] fp32
    ids: List[torch.Tensor]        # per table: [B * hotness_t] int64 (sample-major)
    labels: torch.Tensor           # [B] fp32


class DLRMBatchSource:
    """Generates global batches on the CPU; every rank constructs the same stream from the seed.  Ids are Zipf
    (``alpha``; 0 = uniform) or, with ``gaussian=(mu, sigma, lo, hi)``, a normal draw clipped to ``[lo, hi]`` and scaled
    to the table (the ``--rand-data-dist gaussian`` generator of the reference's driver, dlrm_data_pytorch.py)."""

    def __init__(self, table_rows: Sequence[int], hotness: Sequence[int], batch: int, num_dense: int = 13,
                 alpha: float = 1.2, seed: int = 0, gaussian: Optional[Tuple[float, float, float, float]] = None,
                 id_fn=None):
        self.gaussian = gaussian
        self.id_fn = id_fn                   # optional ``id_fn(n_ids, n_rows, table_index) -> int64 array``: overrides the generators
        self.table_rows = list(table_rows)
        self.hotness = list(hotness)
        self.batch = batch
        self.num_dense = num_dense
        self.alpha = alpha
        self.rng = np.random.default_rng(seed)

    def next(self) -> DLRMBatch:
        B = self.batch
        dense = np.log1p(self.rng.exponential(1.0, size=(B, self.num_dense))).astype(np.float32)
        labels = (self.rng.random(B) < 0.25).astype(np.float32)
        if self.id_fn is not None:
            ids = [torch.from_numpy(np.ascontiguousarray(self.id_fn(B * h, n, t), dtype=np.int64))
                   for t, (n, h) in enumerate(zip(self.table_rows, self.hotness))]
        elif self.gaussian is not None:
            mu, sigma, lo, hi = self.gaussian
            mu = (lo + hi) / 2.0 if mu == -1 else mu
            ids = []
            for n, h in zip(self.table_rows, self.hotness):
                r = np.clip(self.rng.normal(mu, sigma, size=B * h), lo, hi)
                ids.append(torch.from_numpy(np.minimum((n * (r - lo) / (hi - lo)).astype(np.int64), n - 1)))
        else:
            ids = [torch.from_numpy(zipf_ids(B * h, n, self.alpha, self.rng)) for n, h in zip(self.table_rows, self.hotness)]
        return DLRMBatch(torch.from_numpy(dense), ids, torch.from_numpy(labels))
