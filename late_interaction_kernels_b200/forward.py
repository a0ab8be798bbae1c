"""Fused MaxSim forward on padded ``[N, L, d]`` inputs.

Host-side twin of the reference's ``forward.py``: same two entry points
(``_run_forward`` for the autograd layer, ``maxsim_forward`` for callers that
want scores and the optional argmax), same shapes and return conventions
(forward.py:228-398).  The work is done by ``lik_maxsim_fwd``.
"""

from __future__ import annotations

import torch

from . import _lib, _ops
from ._utils import common_dtype, ensure_contiguous_last


def _run_forward(Q, D, q_mask, d_mask, save_argmax, normalize=False, *, kd_layout=False, engine=0, rounded_norm=False):
    """Q ``[Nq, Lq, d]``; D ``[Nd, Ld, d]`` (cross product) or the flat ``[Nq*K, Ld, d]`` view of
    per-query candidate lists (``kd_layout=True``).  Masks are ``[Nq, Lq]`` / ``[D.shape[0], Ld]``
    (bool or int8, nonzero = valid).  Returns ``(scores fp32 [Nq, Nd_eff], argmax int32
    [Nq*Nd_eff, Lq] | None)`` with ``-1`` marking "no valid document token"
    (forward.py:228-346)."""
    _lib.require_cuda(Q, D, q_mask, d_mask, op="maxsim forward")
    Nq, Lq, d = Q.shape
    if kd_layout:
        if Nq == 0 or D.shape[0] % Nq != 0:
            raise ValueError(f"kd_layout=True requires D.shape[0] (={D.shape[0]}) to be a multiple of Nq (={Nq}).")
        nd_eff = D.shape[0] // Nq
    else:
        nd_eff = D.shape[0]
    dt = common_dtype(Q, D)
    q = _ops.padded_spec(Q.to(dt), q_mask)
    dd = _ops.padded_spec(D.to(dt), d_mask)
    scores, argmax = _ops.forward(
        q, dd,
        pairing=_lib.PAIR_GROUPED if kd_layout else _lib.PAIR_CROSS,
        group=nd_eff if kd_layout else 0,
        normalize=(_lib.NORM_BOTH | (_lib.NORM_ROUNDED if rounded_norm else 0)) if normalize else _lib.NORM_NONE,
        save_argmax=save_argmax, argmax_stride=Lq, engine=engine,
    )
    return scores.view(Nq, nd_eff), argmax


def maxsim_forward(Q, D, q_mask=None, d_mask=None, *, save_argmax=False, normalize=False, _rounded_norm=False):
    """Fused MaxSim forward without autograd (forward.py:349-398).

    Q ``[Nq, Lq, d]`` or ``[Lq, d]``; D ``[Nd, Ld, d]`` or ``[Ld, d]``; optional bool masks.
    Returns ``(scores, argmax | None)``; scores are fp32 ``[Nq, Nd]`` (squeezed for 2-D inputs),
    argmax is int32 ``[Nq*Nd, Lq]``.

    ``_rounded_norm=True`` (not part of the reference signature) selects, for 16-bit inputs with
    ``normalize=True``, normalised operand copies rounded to the input dtype instead of fp32 inverse
    norms applied to the raw scores: about a third faster, scores move by ~1e-3 relative and near-ties
    may resolve differently, so nothing in this package turns it on by itself."""
    q2, d2 = Q.dim() == 2, D.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    if d2:
        D = D.unsqueeze(0)
    if q_mask is not None and q_mask.dim() == 1:
        q_mask = q_mask.unsqueeze(0)
    if d_mask is not None and d_mask.dim() == 1:
        d_mask = d_mask.unsqueeze(0)
    if Q.shape[-1] != D.shape[-1]:
        raise ValueError(f"Q and D must share the embedding dim; got {Q.shape[-1]} vs {D.shape[-1]}.")
    scores, argmax = _run_forward(ensure_contiguous_last(Q), ensure_contiguous_last(D), q_mask, d_mask, save_argmax, normalize,
                                  rounded_norm=_rounded_norm)
    if q2 and d2:
        return scores.reshape(()), argmax
    if q2:
        return scores.squeeze(0), argmax
    if d2:
        return scores.squeeze(-1), argmax
    return scores, argmax
