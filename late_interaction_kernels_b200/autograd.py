"""User-facing differentiable MaxSim: ``maxsim`` and ``maxsim_pairs``.

Same signatures, shape dispatch, error messages and warn-once behaviour as the
reference's ``autograd.py`` (autograd.py:356-501).  What is gone is everything
that only served the Triton autotuner: no power-of-two padding of ``Lq``
(autograd.py:49-98) and no 128-token chunking of long queries
(autograd.py:322-353) — the kernels take any ``Lq`` directly.
"""

from __future__ import annotations

import os
import warnings

import torch

from . import _lib
from .backward._launch import run_backward
from .forward import _run_forward

_VALID_METHODS = ("auto", "unified", "lowmem")

# The un-normalised-input heuristic needs a device->host sync, so it runs on the first call only
# (same policy as autograd.py:129-166).
_NORM_CHECKED = False


def _validate_devices(Q, D, q_mask, d_mask) -> None:
    if Q.device != D.device:
        raise ValueError(f"Q and D must be on the same device; got Q.device={Q.device} vs D.device={D.device}.")
    if q_mask is not None and q_mask.device != Q.device:
        raise ValueError(f"q_mask must be on the same device as Q; got {q_mask.device} vs {Q.device}.")
    if d_mask is not None and d_mask.device != D.device:
        raise ValueError(f"d_mask must be on the same device as D; got {d_mask.device} vs {D.device}.")


def _maybe_warn_unnormalized(Q: torch.Tensor) -> None:
    """Warn once when ``normalize=False`` meets queries whose median token norm is far from 1.
    Silence with ``LIK_SUPPRESS_NORM_WARN=1``."""
    global _NORM_CHECKED
    if _NORM_CHECKED or os.environ.get("LIK_SUPPRESS_NORM_WARN", "0") == "1":
        return
    _NORM_CHECKED = True
    if torch.cuda.is_current_stream_capturing():
        return
    with torch.no_grad():
        sample = Q.detach().reshape(-1, Q.shape[-1])[:64]
        if sample.numel() == 0:
            return
        med = sample.float().norm(dim=-1).median().item()
    if not (0.9 <= med <= 1.1):
        warnings.warn(
            f"late-interaction-kernels: `maxsim(..., normalize=False)` but Q's median L2 norm is {med:.3f} "
            "(ColBERT-style models expect ≈1.0). Pass `normalize=True` to fuse the L2-norm into the kernel, "
            "or pre-normalize with `F.normalize(Q, dim=-1)`. Silence with `LIK_SUPPRESS_NORM_WARN=1`.",
            UserWarning,
            stacklevel=3,
        )


def _as_mask(m):
    if m is None:
        return None
    m = m.contiguous()
    return m if m.dtype in (torch.bool, torch.uint8, torch.int8) else (m != 0)


class _MaxSimFn(torch.autograd.Function):
    """Fused MaxSim with saved argmax on 3-D inputs; ``kd_layout`` marks ``D`` as the flat
    ``[Nq*K, Ld, d]`` view of per-query candidate lists."""

    @staticmethod
    def forward(ctx, Q, D, q_mask, d_mask, normalize, backward_method, kd_layout):
        scores, argmax = _run_forward(Q, D, q_mask, d_mask, save_argmax=True, normalize=normalize, kd_layout=kd_layout)
        ctx.save_for_backward(Q, D, argmax, q_mask, d_mask)
        ctx.backward_method = backward_method
        ctx.normalize = normalize
        ctx.kd_layout = kd_layout
        return scores

    @staticmethod
    def backward(ctx, grad_scores):
        Q, D, argmax, q_mask, d_mask = ctx.saved_tensors
        # "unified" keeps the fp32-atomic scatter; "lowmem" and "auto" use the destination-owned
        # reduction, which on this hardware is both the deterministic and the faster one.
        deterministic = ctx.backward_method != "unified"
        gq, gd = run_backward(
            "maxsim backward", grad_scores, Q, D, argmax, q_mask, kd_layout=ctx.kd_layout, deterministic=deterministic,
            d_mask=d_mask, normalize=ctx.normalize, need_q=ctx.needs_input_grad[0], need_d=ctx.needs_input_grad[1],
        )
        return gq, gd, None, None, None, None, None


def _maxsim_3d(Q, D, q_mask, d_mask, normalize, method, kd_layout):
    Q = Q.contiguous()
    D = D.contiguous()
    q_mask, d_mask = _as_mask(q_mask), _as_mask(d_mask)
    if torch.is_grad_enabled() and (Q.requires_grad or D.requires_grad):
        return _MaxSimFn.apply(Q, D, q_mask, d_mask, normalize, method, kd_layout)
    scores, _ = _run_forward(Q, D, q_mask, d_mask, save_argmax=False, normalize=normalize, kd_layout=kd_layout)
    return scores


def _maxsim_kd(Q, D, q_mask, d_mask, *, normalize, backward_method):
    """``[Nq, Lq, d] x [Nq, K, Ld, d] -> [Nq, K]`` (autograd.py:232-287)."""
    if Q.dim() != 3:
        raise ValueError(f"KD layout (D.dim()==4) needs Q to be [Nq, Lq, d]; got Q.shape={tuple(Q.shape)}")
    Nq, Lq, d_q = Q.shape
    Nq_d, K, Ld, d_d = D.shape
    if Nq != Nq_d:
        raise ValueError(f"KD layout needs D.shape[0] == Q.shape[0]; got Q.shape[0]={Nq} vs D.shape[0]={Nq_d}.")
    if d_q != d_d:
        raise ValueError(f"Q and D must share the embedding dim; got {d_q} vs {d_d}.")
    if q_mask is not None and q_mask.shape != (Nq, Lq):
        raise ValueError(f"q_mask must be [Nq={Nq}, Lq={Lq}] for KD layout; got {tuple(q_mask.shape)}.")
    if d_mask is not None and d_mask.shape != (Nq, K, Ld):
        raise ValueError(f"d_mask must be [Nq={Nq}, K={K}, Ld={Ld}] for KD layout; got {tuple(d_mask.shape)}.")
    _validate_devices(Q, D, q_mask, d_mask)
    if Nq == 0 or K == 0:
        return torch.zeros((Nq, K), dtype=torch.float32, device=Q.device)
    D_flat = D.contiguous().view(Nq * K, Ld, d_d)
    dm_flat = d_mask.contiguous().view(Nq * K, Ld) if d_mask is not None else None
    return _maxsim_3d(Q, D_flat, q_mask, dm_flat, normalize, backward_method, True)


def maxsim(Q, D, q_mask=None, d_mask=None, *, normalize=False, backward=None):
    """Differentiable fused MaxSim; drop-in for PyLate's ``colbert_scores`` (autograd.py:356-459).

    Args:
        Q: ``[Nq, Lq, d]`` or ``[Lq, d]``.
        D: ``[Ld, d]`` (one document), ``[Nd, Ld, d]`` (cross product -> ``[Nq, Nd]``) or
            ``[Nq, K, Ld, d]`` (per-query candidate lists -> ``[Nq, K]``).
        q_mask, d_mask: bool tensors shaped like the token axes (``True`` = valid token); any pattern.
        normalize: L2-normalise every token inside the kernel.
        backward: ``None``/"auto", "unified" (fp32 atomics) or "lowmem" (deterministic, dtype-direct).

    Returns fp32 scores; 2-D inputs squeeze the matching axis.  Inputs may be fp16 / bf16 / fp32;
    gradients flow into Q and D in their own dtypes.
    """
    if backward is None:
        method = "auto"
    elif backward not in _VALID_METHODS:
        raise ValueError(f"backward= must be one of {_VALID_METHODS} or None, got {backward!r}")
    else:
        method = backward

    if D.dim() == 4:
        return _maxsim_kd(Q, D, q_mask, d_mask, normalize=normalize, backward_method=method)

    q2, d2 = Q.dim() == 2, D.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    if d2:
        D = D.unsqueeze(0)
    if q_mask is not None and q_mask.dim() == 1:
        q_mask = q_mask.unsqueeze(0)
    if d_mask is not None and d_mask.dim() == 1:
        d_mask = d_mask.unsqueeze(0)
    if Q.dim() != 3 or D.dim() != 3:
        raise ValueError(f"maxsim needs Q [Nq, Lq, d] and D [Nd, Ld, d]; got {tuple(Q.shape)} and {tuple(D.shape)}.")
    if Q.shape[-1] != D.shape[-1]:
        raise ValueError(
            f"Q and D must share the embedding dim; got Q.shape[-1]={Q.shape[-1]} vs D.shape[-1]={D.shape[-1]}."
        )
    _validate_devices(Q, D, q_mask, d_mask)
    _lib.require_cuda(Q, D, op="maxsim")
    if not normalize:
        _maybe_warn_unnormalized(Q)

    scores = _maxsim_3d(Q, D, q_mask, d_mask, normalize, method, False)

    if q2 and d2:
        return scores.reshape(())
    if q2:
        return scores.squeeze(0)
    if d2:
        return scores.squeeze(-1)
    return scores


def maxsim_pairs(Q, D, q_mask=None, d_mask=None, *, normalize=False, backward=None):
    """Same-index pairs ``(Q[i], D[i]) -> [B]``; drop-in for PyLate's ``colbert_scores_pairwise``
    (autograd.py:462-501).  This is the K = 1 case of the candidate-list layout."""
    if Q.dim() != 3 or D.dim() != 3:
        raise ValueError(
            f"maxsim_pairs needs both Q and D to be [B, L, d]; got Q.shape={tuple(Q.shape)}, D.shape={tuple(D.shape)}."
        )
    if Q.shape[0] != D.shape[0]:
        raise ValueError(f"maxsim_pairs needs Q.shape[0] == D.shape[0]; got {Q.shape[0]} vs {D.shape[0]}.")
    dm = d_mask.unsqueeze(1) if d_mask is not None else None
    return maxsim(Q, D.unsqueeze(1), q_mask=q_mask, d_mask=dm, normalize=normalize, backward=backward).squeeze(-1)
