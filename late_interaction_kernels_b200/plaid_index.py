"""The PLAID stages in front of the residual scorer: a reader for the fast-plaid on-disk index, the inverted
file, and the three-stage search that feeds ``plaid_approx_score`` and the decode + MaxSim rerank.

The reference ships only the two scoring kernels and, in its benchmark, a reader for the files fast-plaid
writes (benchmarks/plaid/bench_fastplaid_e2e.py:76-140: ``metadata.json``, ``centroids.npy``,
``bucket_weights.npy``, ``merged_codes.npy`` / ``codes.*.npy``, ``merged_residuals.npy`` / ``residuals.*.npy``,
``doclens.*.json``); candidate generation is left to fast-plaid itself, which is not part of the reference.  This
module restates the published PLAID search (Santhanam et al. 2022) on top of this library's kernels:

    1. centroid scores  qcs = centroids @ Q^T                       (a plain GEMM: cuBLAS through torch.matmul)
    2. probe            the ``nprobe`` best centroids per query token (``lik_topk_rows``), their inverted lists
    3. approximate      ``plaid_approx_score`` on the candidates' codes, keep the ``ndocs`` best (``lik_topk_rows``)
    4. exact            decode + MaxSim + top-k on the survivors       (``retrieve_residual_varlen``)

Steps 2-4 move ragged, data-dependent id lists between kernels with torch indexing ops; every score is computed by
this library's kernels.
"""

from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib, _ops
from .plaid import plaid_approx_score, retrieve_residual_varlen


@dataclass
class PlaidIndexData:
    """A compressed index resident on one device (the tensors ``maxsim_residual_varlen`` takes, plus the inverted file)."""

    nbits: int
    centroids: torch.Tensor        # [n_centroids, d] fp16 / bf16 / fp32
    bucket_weights: torch.Tensor   # [2 ** nbits] fp32
    codes_flat: torch.Tensor       # [T] int32
    residuals_flat: torch.Tensor   # [T, ceil(d * nbits / 8)] uint8
    doc_lengths: torch.Tensor      # [Nd] int64
    cu_seqlens_d: torch.Tensor     # [Nd + 1] int32
    ivf_docs: torch.Tensor | None = None     # [sum of list lengths] int32: documents that use each centroid, by centroid
    ivf_offsets: torch.Tensor | None = None  # [n_centroids + 1] int64

    @property
    def n_docs(self) -> int:
        return int(self.doc_lengths.numel())

    @property
    def dim(self) -> int:
        return int(self.centroids.shape[1])


def read_fastplaid_index(index_path: str, device="cuda", *, dim: int | None = None) -> PlaidIndexData:
    """Load the files fast-plaid serialises (layout as read by the reference's benchmark,
    benchmarks/plaid/bench_fastplaid_e2e.py:76-140).  Trailing padding rows of the merged arrays are clipped to
    ``sum(doclens)``; without merged arrays the per-chunk ``codes.*.npy`` / ``residuals.*.npy`` are concatenated in
    chunk order.  ``dim`` is only needed when the residual array is stored flat."""
    with open(os.path.join(index_path, "metadata.json")) as f:
        meta = json.load(f)
    nbits = int(meta["nbits"])
    if nbits not in (2, 4, 8):
        raise ValueError(f"nbits must be 2, 4, or 8; got {nbits}")
    num_chunks = int(meta["num_chunks"])
    centroids = torch.from_numpy(np.load(os.path.join(index_path, "centroids.npy")))
    if centroids.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        centroids = centroids.to(torch.float32)
    d = int(centroids.shape[1]) if dim is None else int(dim)
    packed = (d * nbits + 7) // 8
    bucket_weights = torch.from_numpy(np.load(os.path.join(index_path, "bucket_weights.npy"))).to(torch.float32)
    if bucket_weights.numel() != 2**nbits:
        raise ValueError(f"bucket_weights holds {bucket_weights.numel()} values, expected {2 ** nbits} for nbits={nbits}")
    lens = []
    for i in range(num_chunks):
        with open(os.path.join(index_path, f"doclens.{i}.json")) as f:
            lens.extend(json.load(f))
    doc_lengths = torch.tensor(lens, dtype=torch.int64)
    total = int(doc_lengths.sum())

    def chunk_files(stem):
        files = glob.glob(os.path.join(index_path, f"{stem}.*.npy"))
        return sorted(files, key=lambda p: int(os.path.basename(p).split(".")[1]))

    merged_codes = os.path.join(index_path, "merged_codes.npy")
    if os.path.exists(merged_codes):
        codes = torch.from_numpy(np.load(merged_codes)).reshape(-1)
        residuals = torch.from_numpy(np.load(os.path.join(index_path, "merged_residuals.npy")))
    else:
        codes = torch.cat([torch.from_numpy(np.load(p)).reshape(-1) for p in chunk_files("codes")])
        residuals = torch.cat([torch.from_numpy(np.load(p)).reshape(-1, packed) for p in chunk_files("residuals")])
    residuals = residuals.to(torch.uint8).reshape(-1, packed)
    if codes.numel() < total or residuals.shape[0] < total:
        raise ValueError(f"the index holds {codes.numel()} codes / {residuals.shape[0]} residual rows for {total} tokens")
    cu = torch.zeros(doc_lengths.numel() + 1, dtype=torch.int32)
    cu[1:] = doc_lengths.cumsum(0).to(torch.int32)
    dev = torch.device(device)
    return PlaidIndexData(
        nbits=nbits, centroids=centroids.to(dev).contiguous(), bucket_weights=bucket_weights.to(dev),
        codes_flat=codes[:total].to(torch.int32).to(dev).contiguous(), residuals_flat=residuals[:total].to(dev).contiguous(),
        doc_lengths=doc_lengths.to(dev), cu_seqlens_d=cu.to(dev),
    )


def build_ivf(index: PlaidIndexData) -> PlaidIndexData:
    """Inverted file: for every centroid the ascending list of documents with at least one token on it."""
    dev = index.codes_flat.device
    n_c = index.centroids.shape[0]
    nd = index.n_docs
    tok_doc = torch.repeat_interleave(torch.arange(nd, device=dev), index.doc_lengths)
    key = index.codes_flat.to(torch.int64).clamp(0, n_c - 1) * max(nd, 1) + tok_doc  # (centroid, document), unique-sorted below
    key = torch.unique(key)
    cent = torch.div(key, max(nd, 1), rounding_mode="floor")
    index.ivf_docs = (key - cent * max(nd, 1)).to(torch.int32)
    counts = torch.bincount(cent, minlength=n_c)
    index.ivf_offsets = torch.zeros(n_c + 1, dtype=torch.int64, device=dev)
    index.ivf_offsets[1:] = counts.cumsum(0)
    return index


def _ragged_gather_positions(starts: torch.Tensor, lens: torch.Tensor):
    """Positions ``starts[i] + [0, lens[i])`` of every row i, concatenated, and the row of every position."""
    total = int(lens.sum())
    row = torch.repeat_interleave(torch.arange(lens.numel(), device=lens.device), lens)
    first = torch.zeros(lens.numel() + 1, dtype=torch.int64, device=lens.device)
    first[1:] = lens.cumsum(0)
    pos = starts[row] + (torch.arange(total, device=lens.device) - first[row])
    return pos, row, first


@torch.no_grad()
def plaid_candidates(index: PlaidIndexData, qcs: torch.Tensor, nprobe: int) -> torch.Tensor:
    """Documents on the inverted lists of the ``nprobe`` best centroids of every query token -> ascending int64 ids.
    ``qcs`` is ``[n_centroids, Lq]`` fp32."""
    if index.ivf_docs is None:
        build_ivf(index)
    n_c = qcs.shape[0]
    probe = min(int(nprobe), n_c, _lib.TOPK_MAX)
    _, cid = _ops.topk_rows(qcs.t().contiguous(), probe)
    cid = torch.unique(cid.reshape(-1))
    starts = index.ivf_offsets[cid]
    lens = index.ivf_offsets[cid + 1] - starts
    pos, _, _ = _ragged_gather_positions(starts, lens)
    return torch.unique(index.ivf_docs[pos].to(torch.int64))


@torch.no_grad()
def plaid_search(index: PlaidIndexData, Q: torch.Tensor, top_k: int, *, nprobe: int = 4, ndocs: int = 1024,
                 normalize: bool = True):
    """PLAID search of one query ``[Lq, d]`` (or ``[Nq, Lq, d]``: one search per query, their candidate sets differ).
    Returns ``(scores fp32 [k], document ids int64 [k])`` (``[Nq, k]`` for a batch, padded with ``-inf`` / ``-1``
    when a query has fewer than ``k`` candidates), best first."""
    if top_k <= 0:
        raise ValueError(f"top_k must be positive, got {top_k}")
    if not 0 < ndocs <= _lib.TOPK_MAX:
        raise ValueError(f"ndocs must be in [1, {_lib.TOPK_MAX}] (the widest list the top-k kernels keep); got {ndocs}")
    _lib.require_cuda(Q, index.codes_flat, op="plaid_search")
    if Q.dim() == 3:
        outs = [plaid_search(index, q, top_k, nprobe=nprobe, ndocs=ndocs, normalize=normalize) for q in Q]
        s = torch.full((len(outs), top_k), float("-inf"), dtype=torch.float32, device=Q.device)
        i = torch.full((len(outs), top_k), -1, dtype=torch.int64, device=Q.device)
        for n, (a, b) in enumerate(outs):
            s[n, : a.numel()], i[n, : b.numel()] = a, b
        return s, i
    if Q.dim() != 2 or Q.shape[1] != index.dim:
        raise ValueError(f"Q must be [Lq, {index.dim}] or [Nq, Lq, {index.dim}]; got {tuple(Q.shape)}")
    Qn = torch.nn.functional.normalize(Q.float(), dim=-1) if normalize else Q.float()
    qcs = (index.centroids.float() @ Qn.t()).contiguous()  # [n_centroids, Lq]
    cand = plaid_candidates(index, qcs, nprobe)
    if cand.numel() == 0:
        return (torch.empty(0, dtype=torch.float32, device=Q.device), torch.empty(0, dtype=torch.int64, device=Q.device))
    # stage 3: approximate scores from the codes alone
    lens = index.doc_lengths[cand]
    if cand.numel() > ndocs:
        max_ld = int(lens.max())
        starts = index.cu_seqlens_d[cand].to(torch.int64)
        t = torch.arange(max_ld, device=Q.device)
        pos = (starts[:, None] + t[None, :]).clamp_(max=index.codes_flat.numel() - 1)
        approx = plaid_approx_score(qcs, index.codes_flat[pos], lens)
        _, keep = _ops.topk_rows(approx[None, :], int(ndocs))
        cand = cand[torch.sort(keep[0]).values]
        lens = index.doc_lengths[cand]
    # stage 4: exact decode + MaxSim on the survivors
    pos, _, first = _ragged_gather_positions(index.cu_seqlens_d[cand].to(torch.int64), lens)
    s, i = retrieve_residual_varlen(Q, index.codes_flat[pos], index.residuals_flat[pos], first.to(torch.int32), index.centroids,
                                    index.bucket_weights, index.nbits, min(top_k, cand.numel()), normalize=normalize)
    return s, cand[i]


__all__ = ["PlaidIndexData", "read_fastplaid_index", "build_ivf", "plaid_candidates", "plaid_search"]
