"""Document-sharded top-k retrieval across the GPUs of one node.

The reference has no distributed code; this is the multi-GPU face of ``retrieve`` / PLAID scoring
that shards naturally: documents are independent, so every rank scores its own contiguous slice of
the corpus, keeps a local top-k, and one collective exchanges the ``[Nq, k]`` candidates.

    rank r owns documents [r * ceil(Nd / W), min((r + 1) * ceil(Nd / W), Nd))
    local:   fused score + top-k over the shard          -> (scores fp32 [Nq, k], global index int64 [Nq, k])
    gather:  one all_gather of both arrays over NCCL      -> [W, Nq, k]
    merge:   lik_topk_merge (score desc, index asc)       -> [Nq, min(k, Nd)]

Shards with fewer than ``k`` documents pad their list with ``(-inf, -1)``; padding never wins the
merge.  No peer memory is read: each GPU touches its own shard and the gathered buffer only.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist


def shard_bounds(n_docs: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous document range ``[lo, hi)`` owned by ``rank``."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    per = math.ceil(n_docs / world_size) if n_docs > 0 else 0
    lo = min(rank * per, n_docs)
    return lo, min(lo + per, n_docs)


def pad_candidates(scores: torch.Tensor, index: torch.Tensor, k: int, *, largest: bool = True):
    """Pad ``[Nq, k_loc]`` candidate lists to width ``k`` with ``(-inf | +inf, -1)``."""
    nq, k_loc = scores.shape
    if k_loc == k:
        return scores.contiguous(), index.contiguous()
    if k_loc > k:
        raise ValueError(f"local list wider than k: {k_loc} > {k}")
    fill = float("-inf") if largest else float("inf")
    s = torch.full((nq, k), fill, dtype=torch.float32, device=scores.device)
    i = torch.full((nq, k), -1, dtype=torch.int64, device=scores.device)
    s[:, :k_loc] = scores
    i[:, :k_loc] = index
    return s, i


def gather_candidates(scores: torch.Tensor, index: torch.Tensor, group=None):
    """All-gather ``[Nq, k]`` candidate lists from every rank -> ``([W, Nq, k], [W, Nq, k])``.
    Works on any backend (NCCL on GPUs, gloo on CPU tensors)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return scores.unsqueeze(0), index.unsqueeze(0)
    gs = torch.empty((world,) + tuple(scores.shape), dtype=scores.dtype, device=scores.device)
    gi = torch.empty((world,) + tuple(index.shape), dtype=index.dtype, device=index.device)
    if scores.is_cuda:
        dist.all_gather_into_tensor(gs, scores.contiguous(), group=group)
        dist.all_gather_into_tensor(gi, index.contiguous(), group=group)
    else:  # gloo has no all_gather_into_tensor for every build: use the list form
        dist.all_gather(list(gs.unbind(0)), scores.contiguous(), group=group)
        dist.all_gather(list(gi.unbind(0)), index.contiguous(), group=group)
    return gs, gi


def merge_candidates(gs: torch.Tensor, gi: torch.Tensor, k: int, *, largest: bool = True):
    """Top-k of the union of ``W`` candidate lists per query (CUDA kernel ``lik_topk_merge``)."""
    from . import _ops

    return _ops.topk_merge(gs, gi, k, largest=largest)


def retrieve_sharded(Q, D_local, top_k, q_mask=None, d_mask=None, *, doc_offset: int, n_docs_total: int | None = None,
                     normalize: bool = True, chunk: int | None = None, largest: bool = True, group=None):
    """Top-``top_k`` retrieval over a corpus sharded by document.

    Every rank passes the same ``Q`` and its own slice ``D_local`` (``[Nd_r, Ld, d]``, with the matching
    ``d_mask`` slice) plus ``doc_offset``, the global index of its first document.  Returns, on every
    rank, ``(scores fp32 [Nq, k], indices int64 [Nq, k])`` with global document indices and
    ``k = min(top_k, n_docs_total)``; identical to ``retrieve`` on the concatenated corpus.
    """
    from .retrieve import retrieve

    if top_k <= 0:
        raise ValueError(f"top_k must be positive, got {top_k}")
    q2 = Q.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    nd_local = D_local.shape[0]
    if n_docs_total is None:
        t = torch.tensor([nd_local], dtype=torch.int64, device=Q.device)
        if world > 1:
            dist.all_reduce(t, group=group)
        n_docs_total = int(t.item())
    k = min(top_k, n_docs_total)
    if nd_local > 0:
        s, i = retrieve(Q, D_local, min(k, nd_local), q_mask=q_mask, d_mask=d_mask, normalize=normalize, chunk=chunk,
                        largest=largest)
        i = i + doc_offset
    else:
        s = torch.empty((Q.shape[0], 0), dtype=torch.float32, device=Q.device)
        i = torch.empty((Q.shape[0], 0), dtype=torch.int64, device=Q.device)
    s, i = pad_candidates(s, i, k, largest=largest)
    if world > 1:
        gs, gi = gather_candidates(s, i, group)
        s, i = merge_candidates(gs, gi, k, largest=largest)
    if q2:
        s, i = s.squeeze(0), i.squeeze(0)
    return s, i


def retrieve_plaid_sharded(Q, codes_local, residuals_local, cu_local, centroids, bucket_weights, nbits, top_k, *,
                           doc_offset: int, n_docs_total: int, normalize: bool = True, chunk: int = 4096,
                           largest: bool = True, group=None, doc_lengths_host=None):
    """Sharded top-k over a PLAID index: every rank holds the codes / residuals / offsets of its own
    contiguous document range (``cu_local`` re-based to start at 0) and the replicated centroids and bucket
    weights; local fused decompress + score + top-k, one all-gather, one merge.  ``doc_lengths_host`` (CPU int64
    lengths of the local documents) saves the device->host copy of the offsets when the corpus is scored in pieces."""
    from .plaid import retrieve_residual_varlen

    q2 = Q.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    k = min(top_k, n_docs_total)
    nd_local = cu_local.numel() - 1
    if nd_local > 0:
        s, i = retrieve_residual_varlen(Q, codes_local, residuals_local, cu_local, centroids, bucket_weights, nbits,
                                        min(k, nd_local), normalize=normalize, chunk=chunk, largest=largest,
                                        doc_lengths_host=doc_lengths_host)
        i = i + doc_offset
    else:
        s = torch.empty((Q.shape[0], 0), dtype=torch.float32, device=Q.device)
        i = torch.empty((Q.shape[0], 0), dtype=torch.int64, device=Q.device)
    s, i = pad_candidates(s, i, k, largest=largest)
    if world > 1:
        gs, gi = gather_candidates(s, i, group)
        s, i = merge_candidates(gs, gi, k, largest=largest)
    if q2:
        s, i = s.squeeze(0), i.squeeze(0)
    return s, i


__all__ = ["retrieve_plaid_sharded", "shard_bounds", "pad_candidates", "gather_candidates", "merge_candidates", "retrieve_sharded"]
