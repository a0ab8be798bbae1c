"""Destination-owned backward: no fp32 buffers, no atomics (reference: backward/lowmem.py:205-322)."""

from ._launch import run_backward


def maxsim_backward_lowmem(grad_scores, Q, D, argmax, q_mask=None, *, kd_layout=False):
    """Same arguments and return value as :func:`maxsim_backward_unified`.  Each output row is
    reduced in fp32 registers in a fixed order and stored once in the input dtype, so results are
    bitwise reproducible and no full-size fp32 gradient buffer exists."""
    return run_backward("maxsim_backward_lowmem", grad_scores, Q, D, argmax, q_mask, kd_layout=kd_layout, deterministic=True)
