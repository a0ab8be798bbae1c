"""Document head in front of MaxSim: ``maxsim_from_hidden`` (reference: fused_head.py:262-456).

``scores = maxsim(Q, normalize(H_d @ W.T + b), d_mask)`` for corpora stored as hidden states ``[Nd, Ld, d_model]``
with a small projection to ``d_out``.  The reference folds the projection into its Triton scoring kernel so that
the projected documents never exist in memory; so does this forward, on the tensor cores: ``lik_maxsim_hidden_fwd``
chains the projection MMA into the scoring MMA through tensor memory and shared memory (16-bit inputs, at most 256
query tokens in all, ``d_out`` a multiple of 32 up to 128).  Anything else projects pieces of the corpus with a plain
GEMM (cuBLAS through ``torch.nn.functional.linear``) into a bounded buffer of ``_PIECE_TOKENS`` rows and scores each
piece with the fused-normalisation kernel.  Both ways round the projected tokens to the input type and apply fp32
inverse norms to the raw dot products, so they agree far inside the 16-bit tolerance.

The backward works on the winning tokens alone: ``lik_hidden_winners`` turns the distinct winners of every document
into a short "compact" document, those rows of ``H_d`` are gathered and projected again, the deterministic
argmax-driven kernels (with the normalise Jacobian of the document side) produce the gradient of the projected rows,
the three GEMMs of the linear layer run on those rows, and ``lik_hidden_scatter_rows`` writes ``grad_H`` in one pass
(a winner's row or zeros).
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


# set to False to force the GEMM-in-pieces forward (tests compare the two)
_CHAINED = True


def _forward(Q, H_d, W, b, d_mask, normalize, save_argmax):
    Nq, Lq, d_out = Q.shape
    Nd, Ld, _ = H_d.shape
    dt = common_dtype(Q, H_d)
    q = _ops.padded_spec(Q.to(dt))
    if _CHAINED and dt in (torch.bfloat16, torch.float16):
        # one kernel: projection MMA -> tensor memory -> rounded operand tile in shared memory -> scoring MMA
        h = _ops.padded_spec(H_d.to(dt), d_mask)
        got = _ops.hidden_forward(q, h, W.to(dt).contiguous(), None if b is None else b.to(dt).contiguous(), normalize=normalize,
                                  save_argmax=save_argmax)
        if got is not None:
            s, am = got
            return s.view(Nq, Nd), (am.view(Nq, Nd, Lq) if save_argmax else None)
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
        # Only winning tokens carry gradient (fused_head.py:332-456 gathers H_d at the winners too): the distinct winners
        # of every document, in token order, form a short "compact" document of at most Nq * Lq tokens
        # (lik_hidden_winners).  Those rows of H_d are gathered and projected again, the deterministic backward kernels
        # run on the compact documents (with the document-side normalise Jacobian), the three GEMMs of the linear layer
        # see the winner rows alone, and one pass writes grad_H: a winner's row or zeros (lik_hidden_scatter_rows).
        # No host synchronisation; cost follows the winners, apart from that one pass over grad_H.
        Q, H_d, W, b, d_mask, argmax = ctx.saved_tensors
        Nq, Lq, d_out = Q.shape
        Nd, Ld, d_model = H_d.shape
        dev = Q.device
        dt = common_dtype(Q, H_d)
        need_q, need_h, need_w, need_b = ctx.needs_input_grad[:4]
        need_b = need_b and b is not None
        need_d = need_h or need_w or need_b
        g = grad_scores.contiguous().to(torch.float32)
        S = max(1, min(Nq * Lq, Ld))  # slots of a compact document
        am_c, rows, counts, bitmap, prefix = _ops.hidden_winners(argmax, Nq, Nd, Lq, Ld, S)
        H_rows = H_d.reshape(Nd * Ld, d_model).index_select(0, rows)  # [Nd * S, d_model]
        P_rows = _project(H_rows, W, b, dt)
        q = _ops.padded_spec(Q.to(dt))
        dd = _ops.padded_spec(P_rows.view(Nd, S, d_out), lens=counts)
        norm = _lib.NORM_D if ctx.normalize else _lib.NORM_NONE
        gq, gp = _ops.backward(q, dd, g, am_c.view(Nq * Nd, Lq), normalize=norm, deterministic=True, grad_dtype=torch.float32,
                               need_q=need_q, need_d=need_d)  # gp: gradient w.r.t. the projected winner rows before normalisation
        gQ = gq.view(Nq, Lq, d_out).to(Q.dtype) if need_q else None
        gH = gW = gb = None
        if need_d:
            # 16-bit models: the linear layer's gradient GEMMs take 16-bit operands with fp32 accumulation, as its forward does
            low = dt in (torch.bfloat16, torch.float16)
            gpl = gp.to(dt) if low else gp
            if need_h:
                g_rows = (gpl @ (W.to(dt) if low else W.float())).to(H_d.dtype)
                gH = torch.empty_like(H_d)
                if (d_model * gH.element_size()) % 16 == 0:
                    _ops.hidden_scatter_rows(g_rows, bitmap, prefix, gH.view(Nd * Ld, d_model), Nd, Ld, S)  # one pass, every row written once
                else:
                    gH.zero_()
                    live = (torch.arange(S, device=dev).unsqueeze(0) < counts.unsqueeze(1)).reshape(-1)
                    gH.view(Nd * Ld, d_model).index_copy_(0, rows[live], g_rows[live])
            if need_w:
                gW = (gpl.t() @ (H_rows.to(dt) if low else H_rows.float())).to(W.dtype)
            if need_b:
                gb = gp.sum(0).to(b.dtype)
        return gQ, gH, gW, gb, None, None


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
