"""Document head in front of MaxSim: ``maxsim_from_hidden`` (reference: fused_head.py:262-456).

``scores = maxsim(Q, normalize(H_d @ W.T + b), d_mask)`` for corpora stored as hidden states ``[Nd, Ld, d_model]``
with a small projection to ``d_out``.  The reference folds the projection into its Triton scoring kernel so that
the projected documents never exist in memory.  Here the projection is a plain GEMM (cuBLAS through
``torch.nn.functional.linear``) run over *pieces* of the corpus into a bounded scratch buffer, and everything after
it is this library's kernels: the L2 normalisation is fused into the tensor-core scoring kernel (fp32 inverse norms
applied in the epilogue), the backward is the deterministic argmax-driven pair of kernels with the normalise
Jacobian of the document side, followed by the three GEMMs of the linear layer.  Peak extra memory is one piece of
projected tokens (``_PIECE_TOKENS`` rows of ``d_out``), whatever the corpus size.

A single kernel that chains the projection MMA into the scoring MMA through tensor memory is not built.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib, _ops
from ._utils import common_dtype

# projected document tokens held at once
_PIECE_TOKENS = 1 << 21


def _pieces(Nd: int, Ld: int):
    per = max(1, _PIECE_TOKENS // max(Ld, 1))
    return [(j0, min(Nd, j0 + per)) for j0 in range(0, Nd, per)]


def _project(H, W, b, dt):
    return F.linear(H.to(dt), W.to(dt), None if b is None else b.to(dt))


def _forward(Q, H_d, W, b, d_mask, normalize, save_argmax):
    Nq, Lq, d_out = Q.shape
    Nd, Ld, _ = H_d.shape
    dt = common_dtype(Q, H_d)
    q = _ops.padded_spec(Q.to(dt))
    scores = torch.empty((Nq, Nd), dtype=torch.float32, device=Q.device)
    argmax = torch.empty((Nq, Nd, Lq), dtype=torch.int32, device=Q.device) if save_argmax else None
    norm = _lib.NORM_D if normalize else _lib.NORM_NONE
    for j0, j1 in _pieces(Nd, Ld):
        D = _project(H_d[j0:j1], W, b, dt)
        dd = _ops.padded_spec(D, None if d_mask is None else d_mask[j0:j1])
        s, am = _ops.forward(q, dd, normalize=norm, save_argmax=save_argmax, argmax_stride=Lq)
        scores[:, j0:j1] = s.view(Nq, j1 - j0)
        if save_argmax:
            argmax[:, j0:j1] = am.view(Nq, j1 - j0, Lq)
    return scores, argmax


class _MaxSimFromHiddenFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, H_d, W, b, d_mask, normalize):
        scores, argmax = _forward(Q, H_d, W, b, d_mask, normalize, True)
        ctx.save_for_backward(Q, H_d, W, b, d_mask, argmax)
        ctx.normalize = normalize
        return scores

    @staticmethod
    def backward(ctx, grad_scores):
        Q, H_d, W, b, d_mask, argmax = ctx.saved_tensors
        Nq, Lq, d_out = Q.shape
        Nd, Ld, d_model = H_d.shape
        dt = common_dtype(Q, H_d)
        q = _ops.padded_spec(Q.to(dt))
        g = grad_scores.contiguous().to(torch.float32)
        need_q, need_h, need_w, need_b = ctx.needs_input_grad[:4]
        need_d = need_h or need_w or (b is not None and need_b)
        gQ = torch.zeros((Nq * Lq, d_out), dtype=torch.float32, device=Q.device) if need_q else None
        gH = torch.empty_like(H_d) if need_h else None
        gW = torch.zeros((d_out, d_model), dtype=torch.float32, device=Q.device) if need_w else None
        gb = torch.zeros(d_out, dtype=torch.float32, device=Q.device) if (b is not None and need_b) else None
        norm = _lib.NORM_D if ctx.normalize else _lib.NORM_NONE
        for j0, j1 in _pieces(Nd, Ld):
            D = _project(H_d[j0:j1], W, b, dt)  # recomputed: the projected tokens are never kept
            dd = _ops.padded_spec(D, None if d_mask is None else d_mask[j0:j1])
            am = argmax[:, j0:j1].reshape(Nq * (j1 - j0), Lq)
            gq, gd = _ops.backward(q, dd, g[:, j0:j1].contiguous(), am, normalize=norm, deterministic=True, grad_dtype=torch.float32,
                                   need_q=need_q, need_d=need_d)
            if need_q:
                gQ += gq
            if need_d:
                gp = gd.view(j1 - j0, Ld, d_out)  # gradient w.r.t. the projected tokens before normalisation
                if need_h:
                    gH[j0:j1] = (gp @ W.float()).to(H_d.dtype)
                if need_w:
                    gW += torch.einsum("jto,jtm->om", gp, H_d[j0:j1].float())
                if gb is not None:
                    gb += gp.sum((0, 1))
        return (None if gQ is None else gQ.view(Nq, Lq, d_out).to(Q.dtype), gH, None if gW is None else gW.to(W.dtype),
                None if gb is None else gb.to(b.dtype), None, None)


def maxsim_from_hidden(Q, H_d, W, b=None, d_mask=None, normalize=True):
    """MaxSim against documents projected on the fly -> fp32 ``[Nq, Nd]`` (``[Nd]`` for a 2-D Q); autograd-aware
    in ``Q``, ``H_d``, ``W`` and ``b`` (fused_head.py:262-330).

    ``Q [Lq, d_out]`` or ``[Nq, Lq, d_out]`` (already projected, and normalised by the caller when ``normalize``),
    ``H_d [Nd, Ld, d_model]`` raw hidden states, ``W [d_out, d_model]``, ``b [d_out]`` or None, ``d_mask [Nd, Ld]``
    bool, ``normalize``: L2-normalise every projected document token."""
    q2 = Q.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
    if d_mask is not None and d_mask.dim() == 1:
        d_mask = d_mask.unsqueeze(0)
    if Q.dim() != 3:
        raise ValueError(f"Q must be [Lq, d_out] or [Nq, Lq, d_out]; got {Q.shape}")
    if H_d.dim() != 3:
        raise ValueError(f"H_d must be [Nd, Ld, d_model]; got {H_d.shape}")
    if W.dim() != 2 or W.shape != (Q.shape[-1], H_d.shape[-1]):
        raise ValueError(f"W must be [d_out={Q.shape[-1]}, d_model={H_d.shape[-1]}]; got {W.shape}")
    if Q.device != H_d.device or W.device != Q.device:
        raise ValueError("Q, H_d, W must be on the same device.")
    if b is not None and (b.dim() != 1 or b.shape[0] != Q.shape[-1]):
        raise ValueError(f"b must be [d_out={Q.shape[-1]}]; got {tuple(b.shape)}")
    _lib.require_cuda(Q, H_d, W, op="maxsim_from_hidden")
    Qc, Hc, Wc = Q.contiguous(), H_d.contiguous(), W.contiguous()
    bc = None if b is None else b.contiguous()
    mc = None if d_mask is None else d_mask.contiguous()
    needs_grad = torch.is_grad_enabled() and (Qc.requires_grad or Hc.requires_grad or Wc.requires_grad or (bc is not None and bc.requires_grad))
    if needs_grad:
        scores = _MaxSimFromHiddenFn.apply(Qc, Hc, Wc, bc, mc, normalize)
    else:
        with torch.no_grad():
            scores, _ = _forward(Qc, Hc, Wc, bc, mc, normalize, False)
    return scores.squeeze(0) if q2 else scores


__all__ = ["maxsim_from_hidden"]
