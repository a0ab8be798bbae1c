"""FP8 (e4m3) MaxSim inference and the quantisation helpers (reference: fp8.py:33-431).

``maxsim_inference_fp8`` scores e4m3 inputs directly (no dequantised copy): per-tensor scales fold
into one multiplier, per-token scales are applied to the score tile inside the kernel.  Beyond the
reference it also accepts the 4-D candidate-list layout ``D [Nq, K, Ld, d]`` with ``scale_D``
``[Nq, K, Ld]``.
"""

from __future__ import annotations

import torch

from . import _lib, _ops

_FP8_E4M3_MAX = 448.0


def quantize_fp8_per_tensor(X: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn):
    """One fp32 scale for the whole tensor: ``scale = max(amax|X|, 1e-6) / 448``; read back as
    ``X_fp8.float() * scale`` (fp8.py:35-49)."""
    if X.numel() == 0:
        return X.to(dtype), torch.ones((), device=X.device, dtype=torch.float32)
    scale = X.abs().amax().clamp_min(1e-6).to(torch.float32) / _FP8_E4M3_MAX
    Xq = (X.to(torch.float32) / scale).clamp(-_FP8_E4M3_MAX, _FP8_E4M3_MAX).to(dtype)
    return Xq.contiguous(), scale


def quantize_fp8_per_token(X: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn):
    """One fp32 scale per row of the last axis; ``scale.shape == X.shape[:-1]`` (fp8.py:52-61)."""
    scale = X.abs().amax(dim=-1).clamp_min(1e-6).to(torch.float32) / _FP8_E4M3_MAX
    Xq = (X.to(torch.float32) / scale.unsqueeze(-1)).clamp(-_FP8_E4M3_MAX, _FP8_E4M3_MAX).to(dtype)
    return Xq.contiguous(), scale


def dequantize_fp8_per_tensor(X_fp8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return X_fp8.to(torch.float32) * scale


def dequantize_fp8_per_token(X_fp8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return X_fp8.to(torch.float32) * scale.unsqueeze(-1)


def _scale_args(scale, token_shape, name):
    """-> (per-token fp32 tensor | None, scalar multiplier tensor | None)."""
    if scale.dim() == 0:
        return None, scale.to(torch.float32)
    if tuple(scale.shape) != tuple(token_shape):
        raise ValueError(f"{name} must be a scalar or have shape {tuple(token_shape)}; got {tuple(scale.shape)}.")
    return scale.to(torch.float32).contiguous(), None


def maxsim_inference_fp8(Q, D, *, scale_Q, scale_D, q_mask=None, d_mask=None):
    """Inference MaxSim on e4m3 inputs -> fp32 scores (fp8.py:234-422).

    Q ``[Nq, Lq, d]`` / ``[Lq, d]``; D ``[Nd, Ld, d]`` / ``[Ld, d]`` / ``[Nq, K, Ld, d]``; scales are
    0-d (per tensor) or shaped like the token axes (per token).  Masks as in :func:`maxsim`."""
    if Q.dtype != torch.float8_e4m3fn or D.dtype != torch.float8_e4m3fn:
        raise ValueError(f"maxsim_inference_fp8 expects float8_e4m3fn inputs; got {Q.dtype} and {D.dtype}.")
    _lib.require_cuda(Q, D, op="maxsim_inference_fp8")
    kd = D.dim() == 4
    q2, d2 = Q.dim() == 2, D.dim() == 2
    if q2:
        Q = Q.unsqueeze(0)
        if scale_Q.dim() > 0:
            scale_Q = scale_Q.unsqueeze(0)
        if q_mask is not None and q_mask.dim() == 1:
            q_mask = q_mask.unsqueeze(0)
    if d2:
        D = D.unsqueeze(0)
        if scale_D.dim() > 0:
            scale_D = scale_D.unsqueeze(0)
        if d_mask is not None and d_mask.dim() == 1:
            d_mask = d_mask.unsqueeze(0)
    if Q.shape[-1] != D.shape[-1]:
        raise ValueError(f"Q and D must share the embedding dim; got {Q.shape[-1]} vs {D.shape[-1]}.")
    Nq, Lq, d = Q.shape
    if kd:
        if D.shape[0] != Nq:
            raise ValueError(f"KD layout needs D.shape[0] == Q.shape[0]; got Q.shape[0]={Nq} vs D.shape[0]={D.shape[0]}.")
        K, Ld = D.shape[1], D.shape[2]
        D3 = D.contiguous().view(Nq * K, Ld, d)
        dm = d_mask.contiguous().view(Nq * K, Ld) if d_mask is not None else None
        sd_tok, sd_sc = _scale_args(scale_D, (Nq, K, Ld), "scale_D")
        nd_eff = K
    else:
        D3, dm = D.contiguous(), d_mask
        sd_tok, sd_sc = _scale_args(scale_D, D3.shape[:2], "scale_D")
        nd_eff = D3.shape[0]
    sq_tok, sq_sc = _scale_args(scale_Q, (Nq, Lq), "scale_Q")
    # per-tensor multipliers stay on the device: fold them into a per-token vector of the other
    # side when there is one, otherwise into a one-element-per-token expansion of the query side.
    mult = None
    for s in (sq_sc, sd_sc):
        if s is not None:
            mult = s if mult is None else mult * s
    if mult is not None:
        if sq_tok is not None:
            sq_tok = sq_tok * mult
        elif sd_tok is not None:
            sd_tok = sd_tok * mult
        else:
            sq_tok = mult.expand(Nq, Lq).contiguous()
    q = _ops.padded_spec(Q, q_mask, scale=sq_tok)
    dd = _ops.padded_spec(D3, dm, scale=sd_tok)
    scores, _ = _ops.forward(q, dd, pairing=_lib.PAIR_GROUPED if kd else _lib.PAIR_CROSS, group=nd_eff if kd else 0)
    scores = scores.view(Nq, nd_eff)
    if kd:
        return scores
    if q2 and d2:
        return scores.reshape(())
    if q2:
        return scores.squeeze(0)
    if d2:
        return scores.squeeze(-1)
    return scores


__all__ = [
    "maxsim_inference_fp8", "quantize_fp8_per_tensor", "quantize_fp8_per_token",
    "dequantize_fp8_per_tensor", "dequantize_fp8_per_token",
]
