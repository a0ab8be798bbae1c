"""Loss-head helpers: several MaxSim calls of a training step folded into one scoring launch.

``maxsim_pos_neg``: positive and explicit-negative scores of a batch.  ``maxsim_tiles``: the whole tile grid of a
cached-contrastive loss (see its docstring).

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


def maxsim_tiles(q_chunks, d_chunks, q_masks=None, d_masks=None, *, normalize: bool = False, backward=None):
    """All-pairs scores of mini-batched embeddings in one launch -> fp32 ``[sum Bq, sum Bd]``.

    A cached-contrastive loss (PyLate's ``CachedContrastive``, docs/benchmarks.md:396-426 of the reference) embeds a
    large batch in mini-batches and scores every (query mini-batch, document mini-batch) tile with its own
    ``colbert_scores`` call: ``(bs / mini) ** 2`` forward launches and as many backward passes, each re-reading its
    documents.  This takes the lists of mini-batch embeddings - ``q_chunks[i] [Bq_i, Lq_i, d]``, ``d_chunks[j]
    [Bd_j, Ld_j, d]``, optional boolean masks per chunk - pads the token axes to the longest chunk (added rows are
    masked out), concatenates (a differentiable ``cat``) and scores the whole grid at once; block ``(i, j)`` of the
    result is the tile the loss would have computed, and autograd splits the gradients back onto the chunks.
    """
    if not q_chunks or not d_chunks:
        raise ValueError("maxsim_tiles needs at least one query chunk and one document chunk")
    for name, chunks in (("q_chunks", q_chunks), ("d_chunks", d_chunks)):
        for c in chunks:
            if c.dim() != 3 or c.shape[-1] != q_chunks[0].shape[-1] or c.device != q_chunks[0].device:
                raise ValueError(f"{name}: every chunk must be [B, L, d] with the same d, on one device")

    def gather(chunks, masks):
        if masks is not None and len(masks) != len(chunks):
            raise ValueError("one mask (or None) per chunk")
        L = max(c.shape[1] for c in chunks)
        dt = chunks[0].dtype
        for c in chunks[1:]:
            dt = torch.promote_types(dt, c.dtype)
        xs, ms = [], []
        for k, c in enumerate(chunks):
            x, m = _pad_tokens(c.to(dt), None if masks is None else masks[k], L)
            xs.append(x)
            ms.append(m)
        if all(m is None for m in ms):
            return torch.cat(xs, 0), None
        ms = [torch.ones(x.shape[:-1], dtype=torch.bool, device=x.device) if m is None else m.to(torch.bool) for x, m in zip(xs, ms)]
        return torch.cat(xs, 0), torch.cat(ms, 0)

    Q, qm = gather(list(q_chunks), q_masks)
    D, dm = gather(list(d_chunks), d_masks)
    return maxsim(Q, D, q_mask=qm, d_mask=dm, normalize=normalize, backward=backward)


__all__ = ["maxsim_pos_neg", "maxsim_tiles"]
