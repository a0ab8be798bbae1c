"""Dispatch rule shared by the PyLate and colpali-engine hooks."""

from __future__ import annotations

import os

import torch


def kernel_path_ok(q: torch.Tensor, d: torch.Tensor) -> bool:
    """True when a hooked call should run on the B200 kernels; False hands the call back to the
    third-party library's own implementation (``LIK_DISABLE=1``, tensors on different devices,
    embedding width below 8, not a CUDA device, or a GPU that is not sm_100)."""
    if os.environ.get("LIK_DISABLE", "0") == "1":
        return False
    if q.device != d.device or q.shape[-1] < 8:
        return False
    if not (q.is_cuda and d.is_cuda):
        return False
    try:
        major, _ = torch.cuda.get_device_capability(q.device)
    except Exception:
        return False
    return major == 10
