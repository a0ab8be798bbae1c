"""Positive and explicit-negative MaxSim scores of a training batch in one scoring launch.

The explicit-negative heads of colpali-engine score ``B`` positive pairs and ``B x K`` hard negatives; the reference
does it with two operators (``maxsim_pairs`` for the positives, the candidate-list ``maxsim`` for the negatives,
colpali_compat.py:205-282), i.e. two forward launches and two backward passes, the first of which has only ``B`` work
units for the whole GPU.  Here the positive document of a query becomes candidate 0 of its list and the negatives
candidates ``1 .. K``: one ``[B, 1 + K, L, d]`` candidate tensor (a differentiable ``cat``: one copy of the documents),
one launch of the candidate-list kernel forward and one deterministic backward, whose gradient autograd splits back
onto the two inputs.  Rows that the common length adds to the shorter side are masked out, so the scores are exactly
those of the two separate calls.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .autograd import maxsim


def _pad_tokens(x: torch.Tensor, mask: torch.Tensor | None, length: int):
    """Pad the token axis (second to last) of ``x`` to ``length`` with zero rows; returns (x, mask or None)."""
    cur = x.shape[-2]
    if cur == length:
        return x, mask
    x = F.pad(x, (0, 0, 0, length - cur))
    if mask is None:
        mask = torch.ones(x.shape[:-1], dtype=torch.bool, device=x.device)
        mask[..., cur:] = False
    else:
        mask = F.pad(mask, (0, length - cur), value=False)
    return x, mask


def maxsim_pos_neg(Q, pos_D, neg_D, q_mask=None, pos_mask=None, neg_mask=None, *, normalize: bool = False, backward=None):
    """``(pos [B], neg [B, K])`` fp32: MaxSim of query ``b`` with its positive ``pos_D[b]`` and with its ``K``
    negatives ``neg_D[b]``, autograd-aware in all three tensors.

    ``Q [B, Lq, d]``, ``pos_D [B, Lp, d]``, ``neg_D [B, K, Ln, d]``; boolean masks ``[B, Lq]``, ``[B, Lp]``,
    ``[B, K, Ln]``.  Identical to ``maxsim_pairs(Q, pos_D)`` and ``maxsim(Q, neg_D)``.
    """
    if Q.dim() != 3 or pos_D.dim() != 3 or neg_D.dim() != 4:
        raise ValueError(f"expected Q [B, Lq, d], pos_D [B, Lp, d], neg_D [B, K, Ln, d]; got {tuple(Q.shape)}, {tuple(pos_D.shape)}, {tuple(neg_D.shape)}")
    B = Q.shape[0]
    if pos_D.shape[0] != B or neg_D.shape[0] != B:
        raise ValueError(f"batch sizes differ: Q {B}, pos_D {pos_D.shape[0]}, neg_D {neg_D.shape[0]}")
    if pos_D.shape[-1] != Q.shape[-1] or neg_D.shape[-1] != Q.shape[-1]:
        raise ValueError("Q, pos_D and neg_D must share the embedding width")
    if pos_D.device != Q.device or neg_D.device != Q.device:
        raise ValueError("Q, pos_D and neg_D must be on the same device.")
    L = max(pos_D.shape[1], neg_D.shape[2])
    dt = torch.promote_types(pos_D.dtype, neg_D.dtype)
    p, pm = _pad_tokens(pos_D.to(dt).unsqueeze(1), None if pos_mask is None else pos_mask.unsqueeze(1), L)
    n, nm = _pad_tokens(neg_D.to(dt), neg_mask, L)
    cand = torch.cat([p, n], dim=1)  # [B, 1 + K, L, d]
    mask = None
    if pm is not None or nm is not None:
        if pm is None:
            pm = torch.ones(p.shape[:-1], dtype=torch.bool, device=Q.device)
        if nm is None:
            nm = torch.ones(n.shape[:-1], dtype=torch.bool, device=Q.device)
        mask = torch.cat([pm, nm], dim=1)
    scores = maxsim(Q, cand, q_mask=q_mask, d_mask=mask, normalize=normalize, backward=backward)  # [B, 1 + K]
    return scores[:, 0], scores[:, 1:]


__all__ = ["maxsim_pos_neg"]
