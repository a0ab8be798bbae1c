"""MaxSim on packed (padding-free) inputs: ``maxsim_varlen`` (reference: varlen.py:271-493).

``Q_packed`` / ``D_packed`` are ``[sum L, d]`` token matrices with int32 cumulative offsets.
The kernels take their loop bounds from ``cu_seqlens`` themselves, so ``max_seqlen_*`` only
sizes per-query buffers: a value that is too small for the queries is reported through the
device status word (``check_device_status()``) instead of a device-side assert, and a too-small
``max_seqlen_d`` cannot truncate documents.
"""

from __future__ import annotations

import torch

from . import _lib, _ops
from ._utils import common_dtype, max_seqlen_from_cu


def _check_packed(Q_packed, D_packed):
    if Q_packed.dim() != 2:
        raise ValueError(
            f"Q_packed must be 2-D [sum(Lq_i), d]; got shape {tuple(Q_packed.shape)} (ndim={Q_packed.dim()}). "
            "For padded inputs use `maxsim(Q, D, ...)` instead."
        )
    if D_packed.dim() != 2:
        raise ValueError(
            f"D_packed must be 2-D [sum(Ld_j), d]; got shape {tuple(D_packed.shape)} (ndim={D_packed.dim()}). "
            "For padded inputs use `maxsim(Q, D, ...)` instead."
        )
    if D_packed.shape[1] != Q_packed.shape[1]:
        raise ValueError(
            "Q_packed and D_packed must share the embedding dim; got "
            f"Q_packed.shape[1]={Q_packed.shape[1]} vs D_packed.shape[1]={D_packed.shape[1]}."
        )


def _varlen_forward(Q_packed, D_packed, cu_seqlens_q, cu_seqlens_d, max_seqlen_q, max_seqlen_d, save_argmax):
    """Returns ``(scores [Nq, Nd], argmax [Nq, Nd, max_q] | None, max_q, max_d)`` (varlen.py:271-364)."""
    _check_packed(Q_packed, D_packed)
    _lib.require_cuda(Q_packed, D_packed, cu_seqlens_q, cu_seqlens_d, op="maxsim_varlen")
    cu_q = cu_seqlens_q.to(torch.int32).contiguous()
    cu_d = cu_seqlens_d.to(torch.int32).contiguous()
    Nq, Nd = cu_q.numel() - 1, cu_d.numel() - 1
    # the longest query sizes the query tiles (and the saved argmax); like the reference it costs one
    # device->host sync when the caller does not pass it.  The longest document is only needed by the backward.
    max_q = max_seqlen_from_cu(cu_q) if max_seqlen_q is None else int(max_seqlen_q)
    if save_argmax:
        max_d = max_seqlen_from_cu(cu_d) if max_seqlen_d is None else int(max_seqlen_d)
    else:
        max_d = 0 if max_seqlen_d is None else int(max_seqlen_d)
    dt = common_dtype(Q_packed, D_packed)
    q = _ops.packed_spec(Q_packed.to(dt), cu_q, max_q)
    d = _ops.packed_spec(D_packed.to(dt), cu_d, max_d)
    scores, argmax = _ops.forward(q, d, pairing=_lib.PAIR_CROSS, save_argmax=save_argmax, argmax_stride=max_q)
    if argmax is not None:
        argmax = argmax.view(Nq, Nd, max_q)
    return scores.view(Nq, Nd), argmax, max_q, max_d


class _MaxSimVarlenFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, D, cu_q, cu_d, max_q, max_d):
        scores, argmax, max_q, max_d = _varlen_forward(Q, D, cu_q, cu_d, max_q, max_d, save_argmax=True)
        ctx.save_for_backward(Q, D, cu_q, cu_d, argmax)
        ctx.max_q, ctx.max_d = max_q, max_d
        return scores

    @staticmethod
    def backward(ctx, grad_scores):
        Q, D, cu_q, cu_d, argmax = ctx.saved_tensors
        dt = common_dtype(Q, D)
        q = _ops.packed_spec(Q.to(dt), cu_q, ctx.max_q)
        d = _ops.packed_spec(D.to(dt), cu_d, ctx.max_d)
        gq, gd = _ops.backward(
            q, d, grad_scores, argmax.view(-1, argmax.shape[-1]), pairing=_lib.PAIR_CROSS, deterministic=True,
            grad_dtype=dt, need_q=ctx.needs_input_grad[0], need_d=ctx.needs_input_grad[1],
        )
        gq = None if gq is None else gq.to(Q.dtype)
        gd = None if gd is None else gd.to(D.dtype)
        return gq, gd, None, None, None, None


def maxsim_varlen(Q_packed, D_packed, cu_seqlens_q, cu_seqlens_d, max_seqlen_q=None, max_seqlen_d=None):
    """MaxSim on packed inputs -> fp32 ``[Nq, Nd]``; autograd-aware (varlen.py:452-493).

    Empty sequences score 0.  ``max_seqlen_q`` sizes the query tiles and the saved argmax, ``max_seqlen_d``
    the backward grid; when omitted they are read from ``cu_seqlens`` with one device->host sync (pass them
    to stay sync-free, e.g. under CUDA-graph capture)."""
    if torch.is_grad_enabled() and (Q_packed.requires_grad or D_packed.requires_grad):
        _check_packed(Q_packed, D_packed)
        return _MaxSimVarlenFn.apply(
            Q_packed.contiguous(), D_packed.contiguous(), cu_seqlens_q.to(torch.int32).contiguous(),
            cu_seqlens_d.to(torch.int32).contiguous(), max_seqlen_q, max_seqlen_d,
        )
    scores, _, _, _ = _varlen_forward(Q_packed, D_packed, cu_seqlens_q, cu_seqlens_d, max_seqlen_q, max_seqlen_d, False)
    return scores
