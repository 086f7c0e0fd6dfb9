"""Variable-size collectives used by the cached-embedding front ends.

Same helper surface as the reference (src/python/pytorch/recstore/utils.py:227-453):
``all2all_data_transfer`` (per-peer tensors of different lengths), ``gather_variable_shape_tensor``,
``reduce_sparse_kv_tensor``, ``all2all_sparse_tensor`` and ``sum_sparse_tensor``.  The reference
stages every message through pinned CPU buffers and gloo point-to-point calls; here the payload
stays on its device and moves with one ``all_to_all_single`` (NCCL) or, where the backend has no
all-to-all (gloo), with ``all_gather`` of padded buffers.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def _world(group=None) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def all2all_data_transfer(send: Sequence[torch.Tensor], group=None) -> List[torch.Tensor]:
    """``send[j]`` goes to rank j; returns ``recv`` with ``recv[i]`` = what rank i sent to this rank.
    All tensors share dtype, device and trailing dimensions; first dimensions are free."""
    rank, world = _world(group)
    if world == 1:
        return [send[0]]
    dev, dtype, tail = send[0].device, send[0].dtype, tuple(send[0].shape[1:])
    counts = torch.tensor([t.shape[0] for t in send], dtype=torch.int64, device=dev)
    all_counts = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts, group=group)
    recv_counts = [int(c[rank].item()) for c in all_counts]
    row = 1
    for s in tail:
        row *= s
    backend = dist.get_backend(group)
    if backend == "nccl":
        sbuf = torch.cat([t.reshape(-1) for t in send])
        rbuf = torch.empty(sum(recv_counts) * row, dtype=dtype, device=dev)
        dist.all_to_all_single(rbuf, sbuf, output_split_sizes=[c * row for c in recv_counts],
                               input_split_sizes=[t.shape[0] * row for t in send], group=group)
        return [p.view(c, *tail) for p, c in zip(torch.split(rbuf, [c * row for c in recv_counts]), recv_counts)]
    # gloo: all_gather of one padded [world, max_rows, ...] block per rank
    m = max(int(c.max().item()) for c in all_counts)
    block = torch.zeros(world, max(m, 1), *tail, dtype=dtype, device=dev)
    for j, t in enumerate(send):
        block[j, : t.shape[0]] = t
    blocks = [torch.empty_like(block) for _ in range(world)]
    dist.all_gather(blocks, block, group=group)
    return [blocks[i][rank, : recv_counts[i]].clone() for i in range(world)]


def gather_variable_shape_tensor(t: torch.Tensor, dst: int = 0, group=None) -> Optional[List[torch.Tensor]]:
    """Gathers tensors whose first dimension differs per rank; returns the list on ``dst``, ``None`` elsewhere."""
    rank, world = _world(group)
    if world == 1:
        return [t]
    n = torch.tensor([t.shape[0]], dtype=torch.int64, device=t.device)
    ns = [torch.empty_like(n) for _ in range(world)]
    dist.all_gather(ns, n, group=group)
    m = max(int(x.item()) for x in ns)
    pad = torch.zeros(max(m, 1), *t.shape[1:], dtype=t.dtype, device=t.device)
    pad[: t.shape[0]] = t
    outs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(outs, pad, group=group)
    if rank != dst:
        return None
    return [o[: int(k.item())] for o, k in zip(outs, ns)]


def sum_sparse_tensor(keys_list: Sequence[torch.Tensor], values_list: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Coalesces (keys, rows) pairs: unique keys and the SUM of the rows of equal keys."""
    keys = torch.cat(list(keys_list))
    vals = torch.cat(list(values_list))
    if keys.numel() == 0:
        return keys, vals
    uniq, inv = torch.unique(keys, return_inverse=True)
    out = torch.zeros(uniq.shape[0], *vals.shape[1:], dtype=vals.dtype, device=vals.device)
    out.index_add_(0, inv, vals)
    return uniq, out


def reduce_sparse_kv_tensor(keys: torch.Tensor, values: torch.Tensor, dst: int = 0, group=None):
    """Sums the (keys, rows) of every rank on ``dst`` (coalesced); ``(None, None)`` elsewhere."""
    rank, _ = _world(group)
    ks = gather_variable_shape_tensor(keys, dst, group)
    vs = gather_variable_shape_tensor(values, dst, group)
    if rank != dst:
        return None, None
    return sum_sparse_tensor(ks, vs)


def all2all_sparse_tensor(keys_per_dst: Sequence[torch.Tensor], values_per_dst: Sequence[torch.Tensor], group=None):
    """Sends (keys, rows) buckets to their destination ranks and coalesces what arrives here."""
    ks = all2all_data_transfer(keys_per_dst, group)
    vs = all2all_data_transfer(values_per_dst, group)
    return sum_sparse_tensor(ks, vs)


@torch.no_grad()
def kv_to_sparse_tensor(keys: torch.Tensor, values: torch.Tensor, shape) -> torch.Tensor:
    """(row ids ``[n]``, rows ``[n, D]``) as a sparse COO matrix of ``shape`` (duplicates stay uncoalesced)."""
    idx = keys if keys.dim() == 2 else keys.unsqueeze(0)
    return torch.sparse_coo_tensor(idx, values, size=tuple(shape), check_invariants=True)


def reduce_sparse_tensor(sparse_tensor: torch.Tensor, dst: int = 0, group=None) -> Optional[torch.Tensor]:
    """Sum of every rank's sparse COO matrix (row-sparse: one index row, values ``[nnz, D]``) on ``dst`` as one
    coalesced sparse matrix; ``None`` elsewhere (src/python/pytorch/recstore/utils.py:352-380)."""
    rank, _ = _world(group)
    st = sparse_tensor if sparse_tensor.is_coalesced() else sparse_tensor.coalesce()
    keys, values = st.indices(), st.values()
    assert keys.shape[0] == 1 and values.dim() == 2, "row-sparse matrices only: indices [1, nnz], values [nnz, D]"
    uniq, rows = reduce_sparse_kv_tensor(keys[0].contiguous(), values.contiguous(), dst, group)
    if rank != dst:
        return None
    return torch.sparse_coo_tensor(uniq.unsqueeze(0), rows, size=tuple(st.shape), check_invariants=True).coalesce()
