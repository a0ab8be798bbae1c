"""Arbitrary ``(query, document)`` pair lists on packed batches: ``score_pairs_packed``
(reference: score_pairs.py:281-511).

The forward runs on the tensor-core kernel (one pair per work unit; consecutive pairs of the same query share the
resident query tile).  The backward groups the pairs by query and by document with two stable device sorts and then
uses the same destination-owned kernels as the other layouts, so the gradients are bitwise reproducible (the
reference scatters both with fp32 atomics, score_pairs.py:148-273)."""

from __future__ import annotations

import torch

from . import _lib, _ops
from ._utils import common_dtype, max_seqlen_from_cu


def _scatter_forward(Q, D, cu_q, cu_d, pair_q, pair_d, max_q, max_d, save_argmax):
    # the longest query sizes the query tiles of the tensor-core path (and the saved winners); like the reference it
    # costs one device->host sync when the caller does not pass it.  The longest document is only needed by the backward.
    max_q = max_seqlen_from_cu(cu_q) if max_q is None else int(max_q)
    if save_argmax:
        max_d = max_seqlen_from_cu(cu_d) if max_d is None else int(max_d)
    else:
        max_d = 0 if max_d is None else int(max_d)
    dt = common_dtype(Q, D)
    q = _ops.packed_spec(Q.to(dt), cu_q, max_q)
    d = _ops.packed_spec(D.to(dt), cu_d, max_d)
    out, argmax = _ops.forward(q, d, pairing=_lib.PAIR_LIST, pair_q=pair_q, pair_d=pair_d, save_argmax=save_argmax,
                               argmax_stride=max_q)
    return out, argmax, max_q, max_d


class _MaxSimScorePairsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, D, cu_q, cu_d, pair_q, pair_d, max_q, max_d):
        out, argmax, max_q, max_d = _scatter_forward(Q, D, cu_q, cu_d, pair_q, pair_d, max_q, max_d, True)
        ctx.save_for_backward(Q, D, cu_q, cu_d, pair_q, pair_d, argmax)
        ctx.max_q, ctx.max_d = max_q, max_d
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, D, cu_q, cu_d, pair_q, pair_d, argmax = ctx.saved_tensors
        dt = common_dtype(Q, D)
        q = _ops.packed_spec(Q.to(dt), cu_q, ctx.max_q)
        d = _ops.packed_spec(D.to(dt), cu_d, ctx.max_d)
        gq, gd = _ops.backward(
            q, d, grad_out, argmax, pairing=_lib.PAIR_LIST, pair_q=pair_q, pair_d=pair_d, deterministic=True,
            grad_dtype=dt, need_q=ctx.needs_input_grad[0], need_d=ctx.needs_input_grad[1],
        )
        gq = None if gq is None else gq.to(Q.dtype)
        gd = None if gd is None else gd.to(D.dtype)
        return gq, gd, None, None, None, None, None, None


def score_pairs_packed(Q_packed, D_packed, cu_seqlens_q, cu_seqlens_d, pair_q_idx, pair_d_idx, *,
                       max_seqlen_q=None, max_seqlen_d=None):
    """``scores[k] = MaxSim(query pair_q_idx[k], document pair_d_idx[k])`` on packed batches -> fp32
    ``[num_pairs]``; autograd-aware (score_pairs.py:423-508).  A pair index outside the batch scores 0
    and sets the device status word instead of faulting."""
    if Q_packed.dim() != 2 or D_packed.dim() != 2:
        raise ValueError(
            f"Q_packed / D_packed must be 2-D [sum(L), d]; got Q={tuple(Q_packed.shape)}, D={tuple(D_packed.shape)}."
        )
    if D_packed.shape[1] != Q_packed.shape[1]:
        raise ValueError(f"Q / D embedding dims mismatch: {Q_packed.shape[1]} vs {D_packed.shape[1]}.")
    if pair_q_idx.shape != pair_d_idx.shape or pair_q_idx.dim() != 1:
        raise ValueError(
            f"pair_q_idx / pair_d_idx must be matching 1-D tensors; got {tuple(pair_q_idx.shape)} vs {tuple(pair_d_idx.shape)}."
        )
    _lib.require_cuda(Q_packed, D_packed, cu_seqlens_q, cu_seqlens_d, pair_q_idx, pair_d_idx, op="score_pairs_packed")
    cu_q = cu_seqlens_q.to(torch.int32).contiguous()
    cu_d = cu_seqlens_d.to(torch.int32).contiguous()
    pq = pair_q_idx.to(torch.int32).contiguous()
    pd = pair_d_idx.to(torch.int32).contiguous()
    Q_packed, D_packed = Q_packed.contiguous(), D_packed.contiguous()
    if torch.is_grad_enabled() and (Q_packed.requires_grad or D_packed.requires_grad):
        return _MaxSimScorePairsFn.apply(Q_packed, D_packed, cu_q, cu_d, pq, pd, max_seqlen_q, max_seqlen_d)
    if pq.numel() == 0:
        return torch.empty(0, device=Q_packed.device, dtype=torch.float32)
    out, _, _, _ = _scatter_forward(Q_packed, D_packed, cu_q, cu_d, pq, pd, max_seqlen_q, max_seqlen_d, False)
    return out


__all__ = ["score_pairs_packed"]
