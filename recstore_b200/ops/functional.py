"""Functional wrappers of the native sm_100a kernels (thin: shape checks + pointer passing).

Each function launches on the current CUDA stream and allocates nothing unless it says so, so
all of them can be captured in a CUDA graph.  ``status`` is a 1-element int64 device tensor
that receives device-side error bits (see ``_lib.decode_status``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib
from .._lib import call, ptr, stream_ptr

EPI_NONE, EPI_RELU, EPI_RELU_MASK, EPI_ATOMIC_F32, EPI_F32, EPI_CROSS, EPI_ADD = range(7)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.RecStoreError(_lib.ERR_INVALID, "native GPU op called with a CPU tensor")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, mode: int = 0, epi: int = EPI_NONE,
              bias: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None,
              x0: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None, bn: int = 0,
              splits: int = 0, n: Optional[int] = None, k: Optional[int] = None) -> torch.Tensor:
    """tcgen05 GEMM.

    mode 0: ``out[M,N] = epi(a[M,K] @ b[N,K].T)``; mode 1: ``out[M,N] (+)= a[K,M].T @ b[K,N]``
    (``out`` fp32, epi ``EPI_ATOMIC_F32``).  Operands are 2-D bf16 with unit inner stride; the
    leading dimensions are taken from ``stride(0)`` so column slices of wider buffers work.
    """
    _need_cuda(a, b, out)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    if mode == 0:
        M, K = a.shape
        N = b.shape[0]
        assert b.shape[1] == K, (a.shape, b.shape)
    else:
        K, M = a.shape
        N = b.shape[1]
        assert b.shape[0] == K, (a.shape, b.shape)
    if n is not None:
        N = n
    if k is not None:
        K = k
    assert out.shape[0] >= M and out.shape[1] >= N
    call("rs_gemm_bf16", ptr(a), ptr(b), ptr(out), ptr(bias), ptr(aux), ptr(x0), M, N, K, a.stride(0), b.stride(0),
         out.stride(0), aux.stride(0) if aux is not None else 0, x0.stride(0) if x0 is not None else 0, mode, epi,
         bn, splits, ptr(status), stream_ptr())
    return out


def emb_forward(weight, table_base, table_rows, indices, *, offsets=None, hotness=None, hot_base=None,
                per_sample_weights=None, T: int, B: int, D: int, B_local: int, dst_table, dst_row_stride: int,
                dst_col, out_bf16: bool = True, row_idx=None, occ2bag=None, ht=None, status=None) -> None:
    """Pooled gather of every (table, sample) bag, stored through ``dst_table[sample // B_local]``."""
    _need_cuda(weight, indices)
    import ctypes as C
    call("rs_emb_forward", ptr(weight), ptr(table_base), ptr(table_rows), ptr(indices), ptr(offsets), ptr(hotness),
         ptr(hot_base), ptr(per_sample_weights), T, B, D, B_local, ptr(dst_table), dst_row_stride, ptr(dst_col),
         1 if out_bf16 else 0, ptr(row_idx), ptr(occ2bag), C.byref(ht) if ht is not None else None, ptr(status),
         stream_ptr())


def emb_backward(weight, state, row_idx, occ2bag, nnz: int, grad, *, grad_col=None, grad_row_stride: int, B: int,
                 D: int, grad_bf16: bool = True, per_sample_weights=None, lr: float, eps: float = 1e-10,
                 optimizer: str = "rowwise_adagrad", status=None, gnorm=None, gnorm_stride: int = 0) -> None:
    """Segment-reduces duplicate rows and applies SGD / row-wise Adagrad in place.

    ``gnorm`` (optional, fp32 ``[B, gnorm_stride]``): sum of squares of every bag gradient, indexed
    ``[sample, local table]``, as produced by :func:`interaction_backward`."""
    _need_cuda(weight, row_idx, grad)
    opt = {"sgd": 0, "rowwise_adagrad": 1}[optimizer]
    call("rs_emb_backward", ptr(weight), ptr(state), weight.shape[0], ptr(row_idx), ptr(occ2bag), nnz, ptr(grad),
         ptr(grad_col), grad_row_stride, ptr(gnorm), gnorm_stride, B, D, 1 if grad_bf16 else 0,
         ptr(per_sample_weights), lr, eps, opt,
         ptr(status), stream_ptr())


def emb_forward_ex(weight, table_base, table_rows, indices, hotness, hot_base, *, T: int, B: int, D: int, B_local: int,
                   dst_table, dst_row_stride: int, dst_col, row_idx=None, occ2bag=None, status=None, counts=None,
                   id_div: int = 1, id_rem: int = 0, occ_cursor=None, ctx=None, wait_channel: int = -1,
                   sig_channel: int = -1, sig_done=None) -> None:
    """:func:`emb_forward` (bf16 output, fixed-capacity bags) with the multi-GPU extras: bags shortened by ``counts`` and
    ids mapped to the rows of a cyclic shard (``id_div``, ``id_rem``), a compacted occurrence list (``occ_cursor``), a
    bounded in-kernel wait on ``wait_channel`` for the rank each bag comes from, and the flag of ``sig_channel``
    published by the kernel itself when its grid is done.  ``indices`` / ``counts`` may be raw device addresses."""
    _need_cuda(weight)
    wait = ctx is not None and wait_channel >= 0
    sig = ctx is not None and sig_channel >= 0
    iptr = indices if isinstance(indices, int) else ptr(indices)
    cptr = counts if isinstance(counts, int) or counts is None else ptr(counts)
    call("rs_emb_forward_ex", ptr(weight), ptr(table_base), ptr(table_rows), iptr, ptr(hotness), ptr(hot_base), T, B, D,
         B_local, ptr(dst_table), dst_row_stride, ptr(dst_col), 1, ptr(row_idx), ptr(occ2bag), ptr(status), cptr, id_div,
         id_rem, ptr(occ_cursor), ctx.my_flags_ptr if wait else None, ctx.counters_ptr if (wait or sig) else None,
         ctx.wait_timeout_ns if ctx is not None else 0, max(wait_channel, 0), ctx.flags_table_ptr if sig else None,
         ptr(sig_done) if sig else None, max(sig_channel, 0), ctx.world if ctx is not None else 1,
         ctx.rank if ctx is not None else 0, stream_ptr())


def emb_backward_ex(weight, state, row_idx, occ2bag, nnz: int, grad, *, grad_col=None, grad_row_stride: int, B: int, D: int,
                    lr: float, eps: float = 1e-10, optimizer: str = "rowwise_adagrad", status=None, gnorm=None,
                    gnorm_stride: int = 0, nnz_dev=None, ctx=None, wait_channel: int = -1, grad_bf16: bool = True) -> None:
    """:func:`emb_backward` with a device-side occurrence count (``nnz_dev``; ``nnz`` is then the capacity
    of the lists) and a bounded in-kernel wait on ``wait_channel`` for the peers' gradient pushes."""
    _need_cuda(weight, row_idx, grad)
    opt = {"sgd": 0, "rowwise_adagrad": 1}[optimizer]
    wait = ctx is not None and wait_channel >= 0
    call("rs_emb_backward_ex", ptr(weight), ptr(state), weight.shape[0], ptr(row_idx), ptr(occ2bag), nnz, ptr(grad),
         ptr(grad_col), grad_row_stride, gnorm if isinstance(gnorm, int) else ptr(gnorm), gnorm_stride, B, D,
         1 if grad_bf16 else 0, lr, eps, opt,
         ptr(status), ptr(nnz_dev), ctx.my_flags_ptr if wait else None, ctx.counters_ptr if wait else None,
         ctx.wait_timeout_ns if ctx is not None else 0, max(wait_channel, 0), ctx.world if ctx is not None else 1, stream_ptr())


def push_rows(src, B: int, T: int, D: int, gdst_table, owner, gcol, grow_stride: int, sample_base: int, *, ndst_table=None,
              nstride: int = 0, ctx=None, sig_channel: int = -1, sig_done=None) -> None:
    """Thin all-to-all push: row (b, f) of ``src`` (bf16 ``[B, >= T*D]``) goes to ``gdst_table[owner[f]]`` at
    ``(sample_base + b) * grow_stride + gcol[f]`` (to every rank when ``owner[f] < 0``), its sum of squares to
    ``ndst_table``; optionally publishes ``sig_channel`` when done."""
    _need_cuda(src)
    sig = ctx is not None and sig_channel >= 0
    call("rs_push_rows", ptr(src), src.stride(0), B, T, D, ctx.world if ctx is not None else 1, ptr(gdst_table), ptr(owner),
         ptr(gcol), grow_stride, sample_base, ptr(ndst_table), nstride, ctx.flags_table_ptr if sig else None,
         ctx.counters_ptr if sig else None, ptr(sig_done) if sig else None, max(sig_channel, 0),
         ctx.rank if ctx is not None else 0, stream_ptr())


def rw_push_keys(ids, id_base, hot, key_base, K: int, B_local: int, B: int, key_win_table, cnt_win_table, occ_cursor, *,
                 ctx, sig_channel: int, sig_done, status=None) -> None:
    """Row-sharded tables, forward step 1: the ids of this rank's bags go to their owners' key windows (owner = id %
    world) with per-(bag, owner) counts; publishes ``sig_channel``."""
    call("rs_rw_push_keys", ptr(ids), ptr(id_base), ptr(hot), ptr(key_base), K, B_local, B, ctx.world, ctx.rank,
         ptr(key_win_table), ptr(cnt_win_table), ptr(occ_cursor), ptr(status), ctx.flags_table_ptr, ctx.counters_ptr,
         ptr(sig_done), sig_channel, stream_ptr())


def rw_reduce_partials(part_ptr: int, out, dst_col, B_local: int, K: int, D: int, *, ctx, wait_channel: int, status=None) -> None:
    """Row-sharded tables, forward step 3: sums the ``world`` partial pooled rows of every (sample, table) into its slot
    of the feature buffer, after a bounded in-kernel wait on ``wait_channel``."""
    call("rs_rw_reduce_partials", part_ptr, ptr(out), ptr(dst_col), out.stride(0), B_local, K, ctx.world, D, ctx.my_flags_ptr,
         ctx.counters_ptr, ctx.wait_timeout_ns, wait_channel, ptr(status), stream_ptr())


def interaction_forward_ex(T, B: int, F: int, D: int, out, *, ctx, wait_channel: int, status=None) -> torch.Tensor:
    """:func:`interaction_forward` whose CTAs first wait (bounded) for ``wait_channel``: the forward all-to-all."""
    _need_cuda(T, out)
    call("rs_interaction_forward_ex", ptr(T), B, F, D, ptr(out), out.stride(0), ctx.my_flags_ptr, ctx.counters_ptr,
         ctx.wait_timeout_ns, wait_channel, ctx.world, ptr(status), stream_ptr())
    return out


def rows_gather(weight, rows, out) -> torch.Tensor:
    call("rs_rows_gather", ptr(weight), ptr(rows), rows.numel(), weight.shape[1], ptr(out), stream_ptr())
    return out


def rows_scatter(weight, rows, values) -> None:
    call("rs_rows_scatter", ptr(weight), ptr(rows), rows.numel(), weight.shape[1], ptr(values), stream_ptr())


def interaction_forward(T, B: int, F: int, D: int, out) -> torch.Tensor:
    """``out[b] = [T[b,0,:], lower_triangle(T[b] @ T[b].T)]`` zero padded to ``out.stride(0)``."""
    _need_cuda(T, out)
    call("rs_interaction_forward", ptr(T), B, F, D, ptr(out), out.stride(0), stream_ptr())
    return out


def interaction_backward(T, dout, B: int, F: int, D: int, dx, gdst_table, owner, gcol, grow_stride: int,
                         sample_base: int, relu_mask_dx: bool = True, ndst_table=None, nstride: int = 0,
                         rows: int = 0) -> None:
    """Backward of :func:`interaction_forward`.  ``rows``: 0 = everything, 1 = only ``dx`` (so that the bottom MLP can
    start its backward early), 2 = only the embedding rows.  Row 0 of dT goes to ``dx``; row f>=1 of sample b is stored
    at ``gdst_table[owner[f-1]] + (sample_base + b) * grow_stride + gcol[f-1]`` (bf16).  With
    ``ndst_table`` the sum of squares of each stored row also goes to
    ``ndst_table[owner[f-1]][(sample_base + b) * nstride + gcol[f-1] // D]`` (fp32)."""
    _need_cuda(T, dout, dx)
    call("rs_interaction_backward", ptr(T), ptr(dout), B, F, D, dout.stride(0), ptr(dx), dx.stride(0),
         ptr(gdst_table), ptr(owner), ptr(gcol), grow_stride, sample_base, 1 if relu_mask_dx else 0,
         ptr(ndst_table), nstride, rows, stream_ptr())


def interaction_dx(T, dout, B: int, F: int, D: int, dx, relu_mask_dx: bool = True) -> None:
    """Only the gradient of feature 0 of :func:`interaction_forward` (a matrix-vector product per sample); the rest of
    the backward can then run beside whatever consumes ``dx``."""
    _need_cuda(T, dout, dx)
    call("rs_interaction_dx", ptr(T), ptr(dout), B, F, D, dout.stride(0), ptr(dx), dx.stride(0), 1 if relu_mask_dx else 0,
         stream_ptr())


def head_bce(x, w, bias, labels, inv_batch: float, *, prob=None, loss_sum=None, dx=None, dw=None, db=None) -> None:
    """Final 1-output linear layer + sigmoid + BCE and all its gradients in one kernel."""
    _need_cuda(x, w)
    M, K = x.shape
    call("rs_head_bce", ptr(x), x.stride(0), M, K, ptr(w), ptr(bias), ptr(labels), inv_batch, ptr(prob),
         ptr(loss_sum), ptr(dx), dx.stride(0) if dx is not None else 0, ptr(dw), ptr(db), stream_ptr())


def colsum_bf16(dy, db) -> None:
    M, N = dy.shape
    call("rs_colsum_bf16", ptr(dy), dy.stride(0), M, N, ptr(db), stream_ptr())


def dense_sgd(w, g, lr: float, wb=None, wt=None, zero_grad: bool = True) -> None:
    N, K = w.shape
    call("rs_dense_sgd", ptr(w), ptr(g), N, K, lr, ptr(wb), wb.stride(0) if wb is not None else 0, ptr(wt),
         wt.stride(0) if wt is not None else 0, 1 if zero_grad else 0, stream_ptr())


def vec_sgd(w, g, lr: float, zero_grad: bool = True) -> None:
    call("rs_vec_sgd", ptr(w), ptr(g), w.numel(), lr, 1 if zero_grad else 0, stream_ptr())


def pad_cast_bf16(x, out) -> torch.Tensor:
    M, K = x.shape
    call("rs_pad_cast_bf16", ptr(x), M, K, x.stride(0), ptr(out), out.stride(0), stream_ptr())
    return out


def mse_fwd_bwd(pred, target, loss_sum, dpred=None) -> None:
    n = pred.numel()
    call("rs_mse_fwd_bwd", ptr(pred), ptr(target), n, 1.0 / n, ptr(loss_sum), ptr(dpred), stream_ptr())


def allreduce_push(grads_table, reduced_table, world: int, rank: int, n: int, scale: float = 1.0, offset: int = 0) -> None:
    """Two-shot all-reduce over peer memory of elements ``[offset, offset + n)`` of the flat buffers (multiples of 4)."""
    call("rs_allreduce_push", ptr(grads_table), ptr(reduced_table), world, rank, offset, n, scale, stream_ptr())


def cross_fwd(x0, u, xl, out) -> None:
    """DCNv2 cross update ``out = x0 * u + xl`` (bf16, element-wise)."""
    call("rs_cross_fwd", ptr(x0), ptr(u), ptr(xl), ptr(out), out.numel(), stream_ptr())


def cross_bwd(dx, x0, u, du, dx0_acc, accumulate: bool) -> None:
    """``du = dx * x0`` (bf16) and ``dx0_acc (+)= dx * u`` (fp32)."""
    call("rs_cross_bwd", ptr(dx), ptr(x0), ptr(u), ptr(du), ptr(dx0_acc), dx.numel(), 1 if accumulate else 0, stream_ptr())


def push_feature_grads(acc, dxb, T, B: int, F: int, D: int, dx, gdst_table, owner, gcol, grow_stride: int, sample_base: int,
                       relu_mask_dx: bool = True, ndst_table=None, nstride: int = 0, dense_extra=None, world: int = 1) -> None:
    """Splits the gradient of the feature matrix ``[B, F, D]`` (``acc`` fp32, optional, plus ``dxb`` bf16): feature 0 to
    ``dx``, features 1.. through the owners' peer pointers, with squared norms (see :func:`interaction_backward`).
    ``dense_extra`` (bf16 ``[B, >= D]``, optional) is added to feature 0: the gradient of a direct path of the dense
    feature into the over-arch.  A feature whose ``owner`` entry is negative (a row-sharded table) goes to ranks
    ``0..world-1``."""
    call("rs_push_feature_grads", ptr(acc), ptr(dxb), ptr(T), B, F, D, ptr(dx), dx.stride(0), ptr(gdst_table), ptr(owner),
         ptr(gcol), grow_stride, sample_base, 1 if relu_mask_dx else 0, ptr(ndst_table), nstride, ptr(dense_extra),
         dense_extra.stride(0) if dense_extra is not None else 0, world, stream_ptr())


def proj_inter_forward(T, b1, b2, I1: int, I2: int, D: int, z) -> None:
    """``z[b] = [T[b, :D] | b1[b].view(I1, D) @ b2[b].view(I2, D).T | 0]`` (bf16; DLRM_Projection, model_zoo/dlrm.py:289-404)."""
    call("rs_proj_inter_fwd", ptr(T), T.stride(0), ptr(b1), ptr(b2), T.shape[0], I1, I2, D, ptr(z), z.stride(0), z.shape[1],
         stream_ptr())


def proj_inter_backward(dz, b1, b2, I1: int, I2: int, D: int, db1, db2) -> None:
    """Gradients of the two (post-ReLU) branches from ``dz[:, D:D + I1 * I2]``, ReLU masks applied."""
    call("rs_proj_inter_bwd", ptr(dz), dz.stride(0), dz.shape[1], ptr(b1), ptr(b2), dz.shape[0], I1, I2, D, ptr(db1), ptr(db2),
         stream_ptr())
