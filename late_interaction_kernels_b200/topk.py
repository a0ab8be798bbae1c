"""Top-k MaxSim (reference: topk.py:12-91).

The reference scores a chunk, calls ``torch.topk``, concatenates with the running list and calls
``torch.topk`` again.  Here the scoring kernel itself keeps the candidates (``lik_maxsim_fwd_topk``): one
launch walks all documents, no ``[Nq, chunk]`` score matrix is written, and a merge kernel returns the
``k`` best per query.  Problems that path does not take (fp32 inputs, packed or very long queries,
``k > 128``) score chunks with ``lik_maxsim_fwd`` and merge them with ``lik_topk_rows`` (``k`` up to 8192; beyond
that the chunks' scores are merged with library sorts).  Either way ties go to the lower document index, so chunked
and unchunked calls return identical indices.
"""

from __future__ import annotations

import torch

from . import _lib, _ops
from ._utils import common_dtype, ensure_contiguous_last
from .forward import maxsim_forward


def maxsim_topk(Q, D, k, q_mask=None, d_mask=None, *, normalize=False, chunk_size=None, largest=True, sorted=True):
    """Top-``k`` documents per query -> ``(fp32 [Nq, k], int64 [Nq, k])`` (2-D Q squeezes);
    ``k`` is clamped to ``Nd``.  Results are always sorted best first."""
    if k <= 0:
        raise ValueError(f"k must be positive, got {k}")
    q2 = Q.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    if D.dim() == 2:
        D = D.unsqueeze(0)
    if q_mask is not None and q_mask.dim() == 1:
        q_mask = q_mask.unsqueeze(0)
    if d_mask is not None and d_mask.dim() == 1:
        d_mask = d_mask.unsqueeze(0)
    _lib.require_cuda(Q, D, op="maxsim_topk")
    Nd = D.shape[0]
    k = min(k, Nd)
    step = Nd if (chunk_size is None or chunk_size >= Nd) else int(chunk_size)
    out = None
    with torch.no_grad():
        if Nd > 0 and Q.shape[0] > 0 and k <= _lib.TOPK_FUSED_MAX and Q.shape[-1] == D.shape[-1]:
            dt = common_dtype(Q, D)
            q = _ops.padded_spec(ensure_contiguous_last(Q).to(dt), q_mask)
            dd = _ops.padded_spec(ensure_contiguous_last(D).to(dt), d_mask)
            out = _ops.forward_fused(q, dd, normalize=_lib.NORM_BOTH if normalize else _lib.NORM_NONE, topk=k, largest=largest)
        for start in range(0, Nd if out is None else 0, max(step, 1)):
            end = min(start + step, Nd)
            dm = d_mask[start:end] if d_mask is not None else None
            s, _ = maxsim_forward(Q, D[start:end], q_mask=q_mask, d_mask=dm, save_argmax=False, normalize=normalize)
            out = _ops.topk_rows(s, k, largest=largest, index_offset=start, out=out)
        if out is None:  # Nd == 0
            out = (torch.empty((Q.shape[0], 0), dtype=torch.float32, device=Q.device),
                   torch.empty((Q.shape[0], 0), dtype=torch.int64, device=Q.device))
    ts, ti = out
    if q2:
        ts, ti = ts.squeeze(0), ti.squeeze(0)
    return ts, ti


__all__ = ["maxsim_topk"]
