"""Padded reranking batches: ``pack_padded`` and ``maxsim_padded`` (reference: padded.py:25-268).

``maxsim_padded`` does not pack: the kernels read the padded ``[B, Lq, d]`` / ``[B, C, Ld, d]``
tensors with their length vectors directly (grouped pairing), which removes the two boolean-mask
gathers and the host sync of the reference path.  ``pack_padded`` is kept for callers that want
the packed form for :func:`score_pairs_packed` / :func:`maxsim_varlen`.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib, _ops
from ._utils import common_dtype


@dataclass(frozen=True)
class PackedBatch:
    """Result of :func:`pack_padded`; iterating yields the fields in order (8-tuple unpacking)."""

    Q_packed: torch.Tensor  # [sum(Lq_b), d]
    cu_seqlens_q: torch.Tensor  # [B + 1] int32
    D_packed: torch.Tensor  # [sum(Ld_bc), d]
    cu_seqlens_d: torch.Tensor  # [B*C + 1] int32, row-major over (b, c)
    pair_q_idx: torch.Tensor  # [B*C] int32, pair_q_idx[b*C + c] = b
    pair_d_idx: torch.Tensor  # [B*C] int32, pair_d_idx[b*C + c] = b*C + c
    max_seqlen_q: int
    max_seqlen_d: int

    def __iter__(self):
        yield from (self.Q_packed, self.cu_seqlens_q, self.D_packed, self.cu_seqlens_d, self.pair_q_idx,
                    self.pair_d_idx, self.max_seqlen_q, self.max_seqlen_d)


def _check_padded(queries, documents, query_lengths, doc_lengths):
    if queries.dim() != 3:
        raise ValueError(f"queries must be [B, Lq, d]; got shape {tuple(queries.shape)}")
    if documents.dim() != 4:
        raise ValueError(f"documents must be [B, C, Ld, d]; got shape {tuple(documents.shape)}")
    B, _, d = queries.shape
    Bd, C, _, Dd = documents.shape
    if B != Bd:
        raise ValueError(f"batch size mismatch: queries B={B}, documents B={Bd}")
    if d != Dd:
        raise ValueError(f"embedding dim mismatch: queries d={d}, documents d={Dd}")
    if query_lengths.shape != (B,):
        raise ValueError(f"query_lengths must be [B={B}]; got {tuple(query_lengths.shape)}")
    if doc_lengths.shape != (B, C):
        raise ValueError(f"doc_lengths must be [B={B}, C={C}]; got {tuple(doc_lengths.shape)}")


def _validate_lengths(qlen, dlen, Lq, Ld):
    if (qlen <= 0).any().item():
        raise ValueError("query_lengths must all be > 0")
    if (dlen <= 0).any().item():
        raise ValueError("doc_lengths must all be > 0")
    if (qlen > Lq).any().item() or (dlen > Ld).any().item():
        raise ValueError("a length exceeds the padded extent")


def pack_padded(queries, documents, query_lengths, doc_lengths, *, validate=False) -> PackedBatch:
    """Padded ``[B, Lq, d]`` / ``[B, C, Ld, d]`` + lengths -> packed layout (padded.py:77-208).
    Lengths above the padded extent are clamped to it (``validate=True`` raises instead).  One
    device->host sync fetches both maxima."""
    _check_padded(queries, documents, query_lengths, doc_lengths)
    B, Lq, d = queries.shape
    _, C, Ld, _ = documents.shape
    dev = queries.device
    if B == 0:
        z1 = torch.zeros(1, dtype=torch.int32, device=dev)
        z0 = torch.zeros(0, dtype=torch.int32, device=dev)
        return PackedBatch(queries.reshape(0, d), z1, documents.reshape(0, d), z1.clone(), z0, z0.clone(), 0, 0)
    qlen = query_lengths.to(device=dev, dtype=torch.int32)
    dlen = doc_lengths.to(device=dev, dtype=torch.int32)
    if validate:
        _validate_lengths(qlen, dlen, Lq, Ld)
    qlen = qlen.clamp(0, Lq)
    dlen = dlen.clamp(0, Ld)
    q_keep = torch.arange(Lq, device=dev, dtype=torch.int32)[None, :] < qlen[:, None]
    Q_packed = queries.reshape(B * Lq, d)[q_keep.reshape(-1)]
    cu_q = torch.zeros(B + 1, dtype=torch.int32, device=dev)
    cu_q[1:] = qlen.cumsum(0)
    d_keep = torch.arange(Ld, device=dev, dtype=torch.int32)[None, None, :] < dlen[:, :, None]
    D_packed = documents.reshape(B * C * Ld, d)[d_keep.reshape(-1)]
    cu_d = torch.zeros(B * C + 1, dtype=torch.int32, device=dev)
    cu_d[1:] = dlen.reshape(-1).cumsum(0)
    flat = torch.arange(B * C, dtype=torch.int32, device=dev)
    pair_q = torch.div(flat, max(C, 1), rounding_mode="floor").to(torch.int32)
    if C > 0:
        max_q, max_d = torch.stack([qlen.max(), dlen.max()]).tolist()
    else:
        max_q, max_d = int(qlen.max().item()), 0
    return PackedBatch(Q_packed, cu_q, D_packed, cu_d, pair_q.contiguous(), flat.contiguous(), int(max_q), int(max_d))


class _MaxSimPaddedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, queries, documents, qlen, dlen):
        B, Lq, d = queries.shape
        _, C, Ld, _ = documents.shape
        dt = common_dtype(queries, documents)
        q = _ops.padded_spec(queries.to(dt), lens=qlen)
        dd = _ops.padded_spec(documents.to(dt).view(B * C, Ld, d), lens=dlen)
        scores, argmax = _ops.forward(q, dd, pairing=_lib.PAIR_GROUPED, group=C, save_argmax=True, argmax_stride=Lq)
        ctx.save_for_backward(queries, documents, qlen, dlen, argmax)
        return scores.view(B, C)

    @staticmethod
    def backward(ctx, grad):
        queries, documents, qlen, dlen, argmax = ctx.saved_tensors
        B, Lq, d = queries.shape
        _, C, Ld, _ = documents.shape
        dt = common_dtype(queries, documents)
        q = _ops.padded_spec(queries.to(dt), lens=qlen)
        dd = _ops.padded_spec(documents.to(dt).view(B * C, Ld, d), lens=dlen)
        gq, gd = _ops.backward(q, dd, grad, argmax, pairing=_lib.PAIR_GROUPED, group=C, deterministic=True, grad_dtype=dt,
                               need_q=ctx.needs_input_grad[0], need_d=ctx.needs_input_grad[1])
        gq = None if gq is None else gq.view(B, Lq, d).to(queries.dtype)
        gd = None if gd is None else gd.view(B, C, Ld, d).to(documents.dtype)
        return gq, gd, None, None


def maxsim_padded(queries, documents, query_lengths, doc_lengths, *, validate=False):
    """Score ``C`` candidates per query from padded inputs -> fp32 ``[B, C]``; autograd-aware
    (padded.py:216-268).  Only the first ``query_lengths[b]`` / ``doc_lengths[b, c]`` tokens count;
    an empty query or document scores 0.  ``validate=True`` checks the lengths on the host (three
    syncs) and raises ``ValueError`` on zero or out-of-range values."""
    _check_padded(queries, documents, query_lengths, doc_lengths)
    _lib.require_cuda(queries, documents, op="maxsim_padded")
    B, Lq, d = queries.shape
    _, C, Ld, _ = documents.shape
    dev = queries.device
    if B == 0 or C == 0:
        return torch.empty((B, C), dtype=torch.float32, device=dev)
    qlen = query_lengths.to(device=dev, dtype=torch.int32).contiguous()
    dlen = doc_lengths.to(device=dev, dtype=torch.int32).contiguous().reshape(-1)
    if validate:
        _validate_lengths(qlen, dlen, Lq, Ld)
    queries, documents = queries.contiguous(), documents.contiguous()
    if torch.is_grad_enabled() and (queries.requires_grad or documents.requires_grad):
        return _MaxSimPaddedFn.apply(queries, documents, qlen, dlen)
    dt = common_dtype(queries, documents)
    q = _ops.padded_spec(queries.to(dt), lens=qlen)
    dd = _ops.padded_spec(documents.to(dt).view(B * C, Ld, d), lens=dlen)
    scores, _ = _ops.forward(q, dd, pairing=_lib.PAIR_GROUPED, group=C)
    return scores.view(B, C)


__all__ = ["PackedBatch", "pack_padded", "maxsim_padded"]
