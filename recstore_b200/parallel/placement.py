"""Table-wise placement of embedding tables on ranks.

``round_robin`` (table ``t`` on rank ``t % world``) is what the reference's model-parallel DLRM does
(src/executable/dlrm/dlrm_model.py: tables are dealt out by index).  ``balanced`` is a longest-processing-time greedy:
tables in decreasing order of their per-sample lookup count (ties: more rows first, then lower index) go to the rank
with the smallest load so far (ties: fewer tables, then lower rank), which evens out multi-hot configurations where a
few tables carry most of the ids.  With equal costs it reproduces the round-robin assignment exactly.
"""
from __future__ import annotations

from typing import List, Sequence


def place_tables(hotness: Sequence[int], rows: Sequence[int], world: int, policy: str = "round_robin") -> List[int]:
    """Owner rank of every table."""
    T = len(hotness)
    assert len(rows) == T and world >= 1
    if policy == "round_robin":
        return [t % world for t in range(T)]
    if policy != "balanced":
        raise ValueError(f"unknown placement policy {policy!r}; one of 'round_robin', 'balanced'")
    order = sorted(range(T), key=lambda t: (-int(hotness[t]), -int(rows[t]) if len(set(hotness)) > 1 else 0, t))
    load = [0] * world
    count = [0] * world
    owner = [0] * T
    for t in order:
        r = min(range(world), key=lambda k: (load[k], count[k], k))
        owner[t] = r
        load[r] += int(hotness[t])
        count[r] += 1
    return owner


def placement_stats(owner: Sequence[int], hotness: Sequence[int], world: int) -> dict:
    """Lookups per sample on every rank and the imbalance (max / mean)."""
    load = [0] * world
    for o, h in zip(owner, hotness):
        load[o] += int(h)
    mean = sum(load) / world if world else 0.0
    return {"lookups_per_rank": load, "imbalance": (max(load) / mean) if mean > 0 else 1.0}
