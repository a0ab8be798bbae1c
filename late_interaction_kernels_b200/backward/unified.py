"""``grad_Q`` gather + fp32 atomic ``grad_D`` scatter (reference: backward/unified.py:205-289)."""

from ._launch import run_backward


def maxsim_backward_unified(grad_scores, Q, D, argmax, q_mask=None, *, kd_layout=False):
    """``grad_scores`` fp32 ``[Nq, Nd_eff]``; Q ``[Nq, Lq, d]``; D ``[Nd, Ld, d]`` or the flat
    ``[Nq*K, Ld, d]`` view (``kd_layout=True``); ``argmax`` int32 ``[Nq*Nd_eff, Lq]`` from the forward
    (``-1`` entries contribute nothing); optional ``q_mask`` ``[Nq, Lq]``.  Returns
    ``(grad_Q, grad_D)`` in the dtypes of Q and D.  ``grad_D`` accumulates in fp32 with atomics, so
    it can differ in the last bits between runs; use :func:`maxsim_backward_lowmem` for
    reproducible results."""
    return run_backward("maxsim_backward_unified", grad_scores, Q, D, argmax, q_mask, kd_layout=kd_layout, deterministic=False)
