"""Shared launcher of the two padded-layout backward entry points."""

from __future__ import annotations

import torch

from .. import _lib, _ops
from .._utils import common_dtype


def run_backward(name, grad_scores, Q, D, argmax, q_mask, *, kd_layout, deterministic, d_mask=None, normalize=False,
                 need_q=True, need_d=True):
    if not (Q.is_cuda and D.is_cuda):
        raise RuntimeError(f"{name} requires CUDA tensors.")
    Nq, Lq, d = Q.shape
    nd_total, Ld, _ = D.shape
    dt = common_dtype(Q, D)
    q = _ops.padded_spec(Q.to(dt), q_mask)
    dd = _ops.padded_spec(D.to(dt), d_mask)
    group = nd_total // Nq if kd_layout else 0
    gq, gd = _ops.backward(
        q, dd, grad_scores, argmax,
        pairing=_lib.PAIR_GROUPED if kd_layout else _lib.PAIR_CROSS, group=group,
        normalize=_lib.NORM_BOTH if normalize else _lib.NORM_NONE, deterministic=deterministic,
        grad_dtype=dt, need_q=need_q, need_d=need_d,
    )
    if gq is not None:
        gq = gq.view(Nq, Lq, d).to(Q.dtype)
    if gd is not None:
        gd = gd.view(nd_total, Ld, d).to(D.dtype)
    return gq, gd
