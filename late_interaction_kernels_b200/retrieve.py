"""High-level entry points: :class:`MaxSimScorer` and :func:`retrieve` (reference: retrieve.py:31-310).

Both default to ``normalize=True``.  Everything runs on the CUDA kernels; tensors on any other
device raise ``RuntimeError`` (this build has no CPU path).
"""

from __future__ import annotations

import contextlib
from typing import Literal

import torch

from . import _lib

BackwardMethod = Literal["auto", "unified", "lowmem"]
_VALID_METHODS: tuple[str, ...] = ("auto", "unified", "lowmem")


def _score(Q, D, q_mask, d_mask, *, normalize, backward, inference):
    if Q.device != D.device:
        raise ValueError(f"Q and D must be on the same device; got Q.device={Q.device} vs D.device={D.device}.")
    _lib.require_cuda(Q, D, op="MaxSimScorer")
    from .autograd import maxsim

    # score() must stay out of autograd even for requires_grad inputs; forward() leaves the caller's
    # grad mode untouched.
    with torch.no_grad() if inference else contextlib.nullcontext():
        return maxsim(Q, D, q_mask=q_mask, d_mask=d_mask, normalize=normalize, backward=backward)


class MaxSimScorer(torch.nn.Module):
    """Stateless ``nn.Module`` for late-interaction scoring (no parameters).

    Args:
        normalize: L2-normalise Q and D per token inside the kernel (default ``True``).
        backward: gradient strategy, ``"auto" | "unified" | "lowmem"``.
        mask_pad_token: pad-token id used by :meth:`forward_with_ids` to derive masks.
    """

    def __init__(self, *, normalize: bool = True, backward: BackwardMethod = "auto", mask_pad_token: int | None = None):
        super().__init__()
        if backward not in _VALID_METHODS:
            raise ValueError(f"backward= must be one of {_VALID_METHODS}, got {backward!r}")
        self.normalize = normalize
        self.backward = backward
        self.mask_pad_token = mask_pad_token

    def extra_repr(self) -> str:
        return f"normalize={self.normalize}, backward={self.backward!r}, mask_pad_token={self.mask_pad_token!r}"

    def forward(self, Q, D, q_mask=None, d_mask=None):
        """MaxSim scores ``[Nq, Nd]``; autograd-aware; identical to ``maxsim(...)``."""
        return _score(Q, D, q_mask, d_mask, normalize=self.normalize, backward=self.backward, inference=False)

    def score(self, Q, D, q_mask=None, d_mask=None):
        """Inference-only MaxSim (never records autograd state, never saves an argmax)."""
        return _score(Q, D, q_mask, d_mask, normalize=self.normalize, backward=self.backward, inference=True)

    def retrieve(self, Q, D, top_k, q_mask=None, d_mask=None, *, chunk=None):
        """``(top_k_scores, top_k_indices)`` per query; see :func:`retrieve`."""
        return retrieve(Q, D, top_k=top_k, q_mask=q_mask, d_mask=d_mask, normalize=self.normalize, chunk=chunk)

    def forward_with_ids(self, Q, D, q_ids, d_ids):
        """Like :meth:`forward` with masks derived from ``ids != mask_pad_token``."""
        if self.mask_pad_token is None:
            raise ValueError("`forward_with_ids` requires `mask_pad_token` set on the scorer.")
        return self.forward(Q, D, q_mask=q_ids != self.mask_pad_token, d_mask=d_ids != self.mask_pad_token)


def retrieve(Q, D, top_k, q_mask=None, d_mask=None, *, normalize=True, chunk=None, largest=True, sorted=True):
    """Top-``top_k`` late-interaction retrieval: equivalent to ``maxsim(Q, D).topk(top_k)`` with an
    optional ``chunk=`` that bounds peak memory to ``Nq * (chunk + top_k)`` scores.

    Returns ``(scores fp32 [Nq, k], indices int64 [Nq, k])`` with ``k = min(top_k, Nd)`` (``[k]`` for a
    2-D Q), sorted best first.  Inference only."""
    if top_k <= 0:
        raise ValueError(f"top_k must be positive, got {top_k}")
    if Q.device != D.device:
        raise ValueError(f"Q and D must be on the same device; got Q.device={Q.device} vs D.device={D.device}.")
    _lib.require_cuda(Q, D, op="retrieve")
    from .topk import maxsim_topk

    return maxsim_topk(Q, D, k=top_k, q_mask=q_mask, d_mask=d_mask, normalize=normalize, chunk_size=chunk,
                       largest=largest, sorted=sorted)


__all__ = ["MaxSimScorer", "retrieve"]
