"""PLAID / ColBERTv2 scoring entry points (reference: plaid.py:82-963).

``plaid_approx_score`` is the IVF-prune step.  ``maxsim_residual`` / ``maxsim_residual_varlen``
score queries against a compressed index (centroid codes + bit-packed residuals).  The reference
decompresses every document token once per (query, document) program; here every token is
decompressed once per call (``lik_plaid_decompress``) into the operand dtype and then scored by the
regular MaxSim forward, in document chunks so the decompressed rows stay small.
"""

from __future__ import annotations

import torch

from . import _lib, _ops

# decompressed tokens held at once (rows of `dim` operand-dtype values)
_DECOMPRESS_TOKENS = 1 << 22
# The index can also be decoded INSIDE the scoring kernel (``lik_plaid_fwd``: the kernel's producer warps gather,
# unpack, normalise and write the operand tiles, so no operand row ever exists in memory).  Every query-tile group
# (256 query-token rows = eight 32-token queries) then decodes the tokens it scores, with three decoder warps per SM.
# Measured on B200 that is slower than decoding once per call with the whole machine (``lik_plaid_decompress``, about
# half the HBM copy rate) and scoring the rows, even for a single query (4.0 ms against 0.64 ms for 25 000 documents),
# so by default no problem takes it: this is the largest number of tile groups for which it is used.  Both ways
# produce the same bits.
_FUSED_DECODE_MAX_GROUPS = 0


def _tile_groups(Nq: int, Lq: int) -> int:
    tiles = -(-Nq // (128 // Lq)) if Lq <= 128 else Nq * -(-Lq // 128)
    return -(-tiles // 2)


@_ops._no_trace
def plaid_approx_score(query_centroid_scores, codes, doc_lengths):
    """``out[b] = sum_s max_{t < doc_lengths[b]} qcs[codes[b, t], s]`` -> fp32 ``[B]`` (plaid.py:82-136).
    Empty documents score 0; out-of-range codes read centroid 0."""
    import ctypes as C

    if query_centroid_scores.dim() != 2:
        raise ValueError("query_centroid_scores must be [n_centroids, Lq]")
    if codes.dim() != 2:
        raise ValueError("codes must be [B, max_Ld]")
    if doc_lengths.dim() != 1 or doc_lengths.shape[0] != codes.shape[0]:
        raise ValueError("doc_lengths must be [B] with B matching codes")
    _lib.require_cuda(query_centroid_scores, codes, doc_lengths, op="plaid_approx_score")
    lib = _lib.load()
    qcs = query_centroid_scores.contiguous().to(torch.float32)
    codes = codes.contiguous().to(torch.int32)
    lens = doc_lengths.contiguous().to(torch.int64)
    B, max_ld = codes.shape
    out = torch.empty(B, device=codes.device, dtype=torch.float32)
    if B:
        with torch.cuda.device(codes.device):
            _lib.check(
                lib.lik_plaid_approx(qcs.data_ptr(), qcs.shape[0], qcs.shape[1], codes.data_ptr() if codes.numel() else None,
                                     B, max_ld, lens.data_ptr(), out.data_ptr(), _lib.stream_ptr(codes.device)),
                "lik_plaid_approx",
            )
    return out


def _prepare_index(Q, codes, residuals, centroids, bucket_weights, nbits):
    if nbits not in (2, 4, 8):
        raise ValueError(f"nbits must be 2, 4, or 8; got {nbits}")
    d = Q.shape[-1]
    codes = codes.contiguous().to(torch.int32)
    residuals = residuals.contiguous().to(torch.uint8)
    if centroids.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        centroids = centroids.to(torch.float32)
    centroids = centroids.contiguous()
    bucket_weights = bucket_weights.contiguous().to(torch.float32)
    expected = (d * nbits + 7) // 8
    return codes, residuals, centroids, bucket_weights, expected


def _operand_dtype(Q):
    # fp16 queries keep fp16 operands, everything else scores in bf16 (plaid.py:466)
    return torch.float16 if Q.dtype == torch.float16 else torch.bfloat16


def _residual_scores(Q, ix, cu_or_lens, max_ld, padded, normalize, save_argmax):
    """Score Q [Nq, Lq, d] against the index in document chunks."""
    dev = Q.device
    Nq, Lq, d = Q.shape
    odt = _operand_dtype(Q)
    Qo = Q.to(odt)
    q = _ops.padded_spec(Qo)
    norm = _lib.NORM_Q if normalize else _lib.NORM_NONE
    if Nq > 0 and _tile_groups(Nq, Lq) <= _FUSED_DECODE_MAX_GROUPS and ix.n_tokens > 0:
        if padded:
            nd = cu_or_lens.numel()
            lay = _ops.layout_spec(nd * max_ld, nd, max_ld, lens=cu_or_lens, seq_stride=max_ld)
        else:
            nd = cu_or_lens.numel() - 1
            lay = _ops.layout_spec(ix.n_tokens, nd, max(int(max_ld), 0), cu=cu_or_lens)
        fused = _ops.forward_fused(q, lay, normalize=(_lib.NORM_BOTH if normalize else _lib.NORM_NONE), plaid=ix,
                                   save_argmax=save_argmax, argmax_stride=Lq)
        if fused is not None:
            s, am = fused
            return s.view(Nq, nd), (am.view(Nq, nd, Lq) if am is not None else None)
    if padded:
        lens = cu_or_lens
        Nd = lens.numel()
        out = torch.empty((Nq, Nd), dtype=torch.float32, device=dev)
        argmax = torch.empty((Nq, Nd, Lq), dtype=torch.int32, device=dev) if save_argmax else None
        docs_per = max(1, _DECOMPRESS_TOKENS // max(max_ld, 1))
        for j0 in range(0, Nd, docs_per):
            j1 = min(Nd, j0 + docs_per)
            emb = _ops.plaid_decompress(ix, j0 * max_ld, (j1 - j0) * max_ld, normalize, odt, dev)
            dd = _ops.padded_spec(emb.view(j1 - j0, max_ld, d), lens=lens[j0:j1])
            s, am = _ops.forward(q, dd, normalize=norm, save_argmax=save_argmax, argmax_stride=Lq)
            out[:, j0:j1] = s.view(Nq, j1 - j0)
            if save_argmax:
                argmax[:, j0:j1] = am.view(Nq, j1 - j0, Lq)
        return out, argmax
    cu = cu_or_lens
    Nd = cu.numel() - 1
    total = ix.n_tokens
    if total <= _DECOMPRESS_TOKENS:
        emb = _ops.plaid_decompress(ix, 0, total, normalize, odt, dev)
        dd = _ops.packed_spec(emb, cu, max_ld)
        s, _ = _ops.forward(q, dd, normalize=norm)
        return s.view(Nq, Nd), None
    # large ragged index: split at document boundaries (one host read of the offsets)
    cu_host = cu.cpu()
    out = torch.empty((Nq, Nd), dtype=torch.float32, device=dev)
    j0 = 0
    while j0 < Nd:
        j1 = int(torch.searchsorted(cu_host, cu_host[j0] + _DECOMPRESS_TOKENS, right=True).item()) - 1
        j1 = min(Nd, max(j1, j0 + 1))
        t0, t1 = int(cu_host[j0]), int(cu_host[j1])
        emb = _ops.plaid_decompress(ix, t0, t1 - t0, normalize, odt, dev)
        dd = _ops.packed_spec(emb, (cu[j0 : j1 + 1] - t0), max_ld)
        s, _ = _ops.forward(q, dd, normalize=norm)
        out[:, j0:j1] = s.view(Nq, j1 - j0)
        j0 = j1
    return out, None


def _maxsim_residual_forward(Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, normalize, save_argmax):
    if nbits not in (2, 4, 8):
        raise ValueError(f"nbits must be 2, 4, or 8; got {nbits}")
    if codes.dim() != 2:
        raise ValueError("codes must be [Nd, max_Ld]")
    if residuals.dim() != 3:
        raise ValueError("residuals must be [Nd, max_Ld, packed_dim]")
    _lib.require_cuda(Q, codes, residuals, centroids, op="maxsim_residual")
    Q = Q.contiguous()
    codes, residuals, centroids, bucket_weights, expected = _prepare_index(Q, codes, residuals, centroids, bucket_weights, nbits)
    doc_lengths = doc_lengths.contiguous().to(device=Q.device, dtype=torch.int64)
    if save_argmax and bool((doc_lengths < 1).any()):
        raise ValueError(
            "maxsim_residual backward does not support zero-length documents; every doc must have >= 1 token. "
            "Filter empty docs out before training, or score them with the inference path (no requires_grad), "
            "which returns 0 for an empty doc."
        )
    if residuals.shape[-1] != expected:
        raise ValueError(f"residuals last dim {residuals.shape[-1]} != expected {expected} for d={Q.shape[-1]}, nbits={nbits}")
    Nd, max_ld = codes.shape
    ix, keep = _ops.plaid_index(codes.view(-1), residuals.view(Nd * max_ld, -1), centroids, bucket_weights, nbits, Q.shape[-1])
    lens32 = doc_lengths.to(torch.int32)
    out, argmax = _residual_scores(Q, ix, lens32, max_ld, True, normalize, save_argmax)
    return out, argmax, (Q, codes, residuals, centroids, bucket_weights)


class _MaxSimResidualFn(torch.autograd.Function):
    """Only ``Q`` is differentiable; the index tensors are frozen quantisation artefacts."""

    @staticmethod
    def forward(ctx, Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, normalize):
        scores, argmax, packed = _maxsim_residual_forward(
            Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, normalize, True
        )
        ctx.save_for_backward(*packed, argmax)
        ctx.nbits, ctx.normalize = nbits, normalize
        return scores

    @staticmethod
    def backward(ctx, grad_scores):
        import ctypes as C

        Q, codes, residuals, centroids, bucket_weights, argmax = ctx.saved_tensors
        lib = _lib.load()
        Nq, Lq, d = Q.shape
        Nd, max_ld = codes.shape
        ix, keep = _ops.plaid_index(codes.view(-1), residuals.view(Nd * max_ld, -1), centroids, bucket_weights, ctx.nbits, d)
        g = grad_scores.contiguous().to(torch.float32)
        gq = torch.empty((Nq, Lq, d), dtype=torch.float32, device=Q.device)
        with torch.cuda.device(Q.device):
            _lib.check(
                lib.lik_plaid_bwd_dq(C.byref(ix), max_ld, Nd, Q.data_ptr(), _lib.lik_dtype(Q.dtype), Nq, Lq, g.data_ptr(),
                                     argmax.data_ptr(), int(ctx.normalize), gq.data_ptr(), _lib.stream_ptr(Q.device)),
                "lik_plaid_bwd_dq",
            )
        return gq.to(Q.dtype), None, None, None, None, None, None, None


def maxsim_residual(Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, *, normalize=True):
    """Fused PLAID residual decompression + L2-normalise + MaxSim -> fp32 ``[Nq, Nd]`` (plaid.py:619-672).

    ``codes [Nd, max_Ld]`` centroid indices, ``residuals [Nd, max_Ld, ceil(d*nbits/8)]`` uint8 with
    ``8/nbits`` bucket codes per byte (little-endian inside the byte), ``doc_lengths [Nd]``,
    ``centroids [n_centroids, d]`` fp16/bf16/fp32, ``bucket_weights [2**nbits]``.  Autograd flows into
    ``Q`` only."""
    q2 = Q.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    if torch.is_grad_enabled() and Q.requires_grad:
        scores = _MaxSimResidualFn.apply(Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, normalize)
    else:
        scores, _, _ = _maxsim_residual_forward(Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, normalize, False)
    return scores.squeeze(0) if q2 else scores


def maxsim_residual_varlen(Q, codes_flat, residuals_flat, cu_seqlens_d, centroids, bucket_weights, nbits, *,
                           max_seqlen_d=None, normalize=True):
    """Ragged PLAID decompress + MaxSim on the on-disk layout (``codes_flat [T]``, ``residuals_flat
    [T, packed_dim]``, ``cu_seqlens_d [Nd+1]``) -> fp32 ``[Nq, Nd]``; inference only (plaid.py:832-963).
    ``max_seqlen_d`` is accepted for compatibility; document bounds always come from ``cu_seqlens_d``."""
    if nbits not in (2, 4, 8):
        raise ValueError(f"nbits must be 2, 4, or 8; got {nbits}")
    q2 = Q.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    if codes_flat.dim() != 1:
        raise ValueError("codes_flat must be 1-D [total_d_tokens]")
    if residuals_flat.dim() != 2:
        raise ValueError("residuals_flat must be 2-D [total_d_tokens, packed_dim]")
    if cu_seqlens_d.dim() != 1:
        raise ValueError("cu_seqlens_d must be 1-D [Nd + 1]")
    _lib.require_cuda(Q, codes_flat, residuals_flat, cu_seqlens_d, centroids, op="maxsim_residual_varlen")
    Q = Q.contiguous()
    codes_flat, residuals_flat, centroids, bucket_weights, expected = _prepare_index(
        Q, codes_flat, residuals_flat, centroids, bucket_weights, nbits
    )
    cu = cu_seqlens_d.contiguous().to(torch.int32)
    if residuals_flat.shape[-1] != expected:
        raise ValueError(
            f"residuals_flat last dim {residuals_flat.shape[-1]} != expected {expected} for d={Q.shape[-1]}, nbits={nbits}"
        )
    Nq = Q.shape[0]
    Nd = cu.numel() - 1
    if Nd <= 0:
        out = torch.empty((Nq, 0), device=Q.device, dtype=torch.float32)
        return out.squeeze(0) if q2 else out
    ix, keep = _ops.plaid_index(codes_flat, residuals_flat, centroids, bucket_weights, nbits, Q.shape[-1])
    with torch.no_grad():
        out, _ = _residual_scores(Q, ix, cu, 0 if max_seqlen_d is None else int(max_seqlen_d), False, normalize, False)
    return out.squeeze(0) if q2 else out


def retrieve_residual_varlen(Q, codes_flat, residuals_flat, cu_seqlens_d, centroids, bucket_weights, nbits, top_k, *,
                             normalize=True, chunk=4096, largest=True, doc_lengths_host=None):
    """Top-``top_k`` documents per query straight from a ragged PLAID index, never materialising
    ``[Nq, Nd]``: documents are decompressed ``chunk`` at a time into operand rows, scored, and merged
    into a running ``[Nq, k]`` list (score desc, index asc).  This is the fused form of "call
    ``maxsim_residual_varlen`` then ``torch.topk``" (docs/benchmarks.md:191-206 of the reference).

    ``cu_seqlens_d`` is read on the host once to place chunk boundaries (pass ``doc_lengths_host``, a CPU
    int64 tensor of per-document lengths, to skip that device->host copy).  Returns
    ``(scores fp32 [Nq, k], indices int64 [Nq, k])`` with ``k = min(top_k, Nd)``; 2-D ``Q`` squeezes."""
    if nbits not in (2, 4, 8):
        raise ValueError(f"nbits must be 2, 4, or 8; got {nbits}")
    if top_k <= 0:
        raise ValueError(f"top_k must be positive, got {top_k}")
    q2 = Q.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    _lib.require_cuda(Q, codes_flat, residuals_flat, cu_seqlens_d, centroids, op="retrieve_residual_varlen")
    Q = Q.contiguous()
    codes_flat, residuals_flat, centroids, bucket_weights, expected = _prepare_index(
        Q, codes_flat, residuals_flat, centroids, bucket_weights, nbits
    )
    if residuals_flat.shape[-1] != expected:
        raise ValueError(
            f"residuals_flat last dim {residuals_flat.shape[-1]} != expected {expected} for d={Q.shape[-1]}, nbits={nbits}"
        )
    cu = cu_seqlens_d.contiguous().to(torch.int32)
    Nd = cu.numel() - 1
    k = min(top_k, max(Nd, 0))
    if k > _lib.TOPK_MAX:
        raise ValueError(f"k={k} exceeds the supported maximum {_lib.TOPK_MAX}")
    Nq, Lq, d = Q.shape
    dev = Q.device
    if Nd <= 0:
        out = (torch.empty((Nq, 0), dtype=torch.float32, device=dev), torch.empty((Nq, 0), dtype=torch.int64, device=dev))
        return (out[0].squeeze(0), out[1].squeeze(0)) if q2 else out
    ix, keep = _ops.plaid_index(codes_flat, residuals_flat, centroids, bucket_weights, nbits, d)
    odt = _operand_dtype(Q)
    q = _ops.padded_spec(Q.to(odt))
    norm = _lib.NORM_Q if normalize else _lib.NORM_NONE
    out = None
    with torch.no_grad():
        if k <= _lib.TOPK_FUSED_MAX and _tile_groups(Nq, Lq) <= _FUSED_DECODE_MAX_GROUPS:
            # few queries: one kernel decodes, scores and keeps the candidates; nothing is read on the host
            lay = _ops.layout_spec(ix.n_tokens, Nd, 0, cu=cu)
            out = _ops.forward_fused(q, lay, normalize=(_lib.NORM_BOTH if normalize else _lib.NORM_NONE), plaid=ix, topk=k,
                                     largest=largest)
            if out is not None:
                return (out[0].squeeze(0), out[1].squeeze(0)) if q2 else out
        if doc_lengths_host is not None:
            cu_host = torch.zeros(Nd + 1, dtype=torch.int64)
            cu_host[1:] = doc_lengths_host.to(torch.int64).cumsum(0)
        else:
            cu_host = cu.cpu().to(torch.int64)
        # many queries: every token is decoded once (in pieces of `chunk` documents, sized so that a piece's operand
        # rows stay small) and the scoring kernel carries its candidate lists from piece to piece
        state = _ops.TopkState() if k <= _lib.TOPK_FUSED_MAX else None
        # a piece holds at least `chunk` documents and as many more as keep its operand rows within the budget
        per_piece = max(int(chunk), int(_DECOMPRESS_TOKENS * Nd // max(int(cu_host[Nd]), 1)), 1)
        pieces = [(j0, min(Nd, j0 + per_piece)) for j0 in range(0, Nd, per_piece)]
        for n, (j0, j1) in enumerate(pieces):
            t0, t1 = int(cu_host[j0]), int(cu_host[j1])
            emb = _ops.plaid_decompress(ix, t0, t1 - t0, normalize, odt, dev)
            max_ld = int((cu_host[j0 + 1 : j1 + 1] - cu_host[j0:j1]).max())
            dd = _ops.packed_spec(emb, cu[j0 : j1 + 1] - t0, max_ld)
            if state is not None:
                r = _ops.forward_fused(q, dd, normalize=norm, topk=k, largest=largest, doc_base=j0, state=state,
                                       last=n == len(pieces) - 1)
                if r is None:
                    if state.started:
                        raise RuntimeError("the fused top-k refused a later piece of a corpus it had started on")
                    state = None
                elif n == len(pieces) - 1:
                    out = r
            if state is None:
                s, _ = _ops.forward(q, dd, normalize=norm)
                out = _ops.topk_rows(s.view(Nq, j1 - j0), k, largest=largest, index_offset=j0, out=out)
    ts, ti = out
    return (ts.squeeze(0), ti.squeeze(0)) if q2 else (ts, ti)


__all__ = ["plaid_approx_score", "maxsim_residual", "maxsim_residual_varlen", "retrieve_residual_varlen"]
