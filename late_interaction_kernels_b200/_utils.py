"""Small host-side helpers shared by the API modules."""

from __future__ import annotations

import torch


def package_at_least(name: str, minimum: str) -> bool:
    """True when the installed distribution ``name`` is at least ``minimum``; absent -> False.
    Only the leading numeric release parts are compared, so dev/rc/post suffixes do not matter
    (same contract as the reference's ``_utils.package_at_least``, _utils.py:53-79)."""
    from importlib.metadata import PackageNotFoundError, version

    def release(v: str) -> tuple[int, ...]:
        out = []
        for chunk in v.split("."):
            digits = ""
            for ch in chunk:
                if not ch.isdigit():
                    break
                digits += ch
            if not digits:
                break
            out.append(int(digits))
        return tuple(out)

    try:
        return release(version(name)) >= release(minimum)
    except PackageNotFoundError:
        return False


def ensure_contiguous_last(x: torch.Tensor) -> torch.Tensor:
    """Return ``x`` with a unit stride on the last dimension (copying only when needed)."""
    return x if x.stride(-1) == 1 else x.contiguous()


def common_dtype(Q: torch.Tensor, D: torch.Tensor) -> torch.dtype:
    """Element type both operands are brought to before the kernel runs.

    Same dtype -> kept (fp32 stays fp32 and is scored by the exact fp32 kernel).  Mixed
    inputs follow the reference's rule (_utils.py:137-148): bf16 if either side is bf16,
    otherwise fp16."""
    if Q.dtype == D.dtype:
        return Q.dtype
    if torch.bfloat16 in (Q.dtype, D.dtype):
        return torch.bfloat16
    return torch.float16


def max_seqlen_from_cu(cu: torch.Tensor) -> int:
    """Longest sequence in a cumulative-offset vector (one device->host sync)."""
    if cu.numel() <= 1:
        return 0
    return int((cu[1:] - cu[:-1]).max().item())
