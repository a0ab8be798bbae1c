"""PyLate drop-in: ``patch_pylate()`` swaps ``pylate.scores.colbert_*`` for the B200 kernels
(reference: pylate_compat.py:120-342).

PyLate releases from 1.5.1 on select a late-interaction-kernels backend by themselves; there
``patch_pylate()`` only emits a ``DeprecationWarning`` and changes nothing.  A hooked call goes
back to PyLate's own function when the tensors are not on a B200 (see ``_hooks.kernel_path_ok``).
PyLate does not normalise inside ``colbert_scores``, so the hooks call ``maxsim(normalize=False)``.
"""

from __future__ import annotations

import importlib
import warnings

import torch

from ._hooks import kernel_path_ok
from ._utils import package_at_least

_ORIGINAL: dict = {}  # stashed PyLate callables; non-empty == patched
_PYLATE_NATIVE_MIN = "1.5.1"
_NATIVE_NOTICE_SHOWN = False

_HOOKED = ("colbert_scores", "colbert_kd_scores", "colbert_scores_pairwise")


def _bool_mask(m):
    """PyLate masks arrive as float 0/1, bool, or None."""
    if m is None or m.dtype == torch.bool:
        return m
    return m != 0


def _resolve_masks(queries_mask, documents_mask, legacy_mask):
    """PyLate < 1.1 passed a single ``mask=`` (document mask).  Returns the two masks as bool plus the
    raw document mask for handing back to PyLate's own function."""
    if documents_mask is None and legacy_mask is not None:
        documents_mask = legacy_mask
    return _bool_mask(queries_mask), _bool_mask(documents_mask), documents_mask


def _tensors(queries_embeddings, documents_embeddings):
    from pylate.utils.tensor import convert_to_tensor  # type: ignore

    return convert_to_tensor(queries_embeddings), convert_to_tensor(documents_embeddings)


def patched_colbert_scores(queries_embeddings, documents_embeddings, queries_mask=None, documents_mask=None, *, mask=None):
    """Replacement for ``pylate.scores.colbert_scores``: ``[Nq, Lq, d] x [Nd, Ld, d] -> [Nq, Nd]``."""
    Q, D = _tensors(queries_embeddings, documents_embeddings)
    qm, dm, raw_dm = _resolve_masks(queries_mask, documents_mask, mask)
    if not kernel_path_ok(Q, D):
        return _ORIGINAL["colbert_scores"](Q, D, queries_mask=queries_mask, documents_mask=raw_dm)
    from .autograd import maxsim

    return maxsim(Q, D, q_mask=qm, d_mask=dm)


def patched_colbert_kd_scores(queries_embeddings, documents_embeddings, queries_mask=None, documents_mask=None, *, mask=None):
    """Replacement for ``pylate.scores.colbert_kd_scores``: ``[Nq, Lq, d] x [Nq, K, Ld, d] -> [Nq, K]``."""
    Q, D = _tensors(queries_embeddings, documents_embeddings)
    qm, dm, raw_dm = _resolve_masks(queries_mask, documents_mask, mask)
    if not kernel_path_ok(Q, D):
        return _ORIGINAL["colbert_kd_scores"](Q, D, queries_mask=queries_mask, documents_mask=raw_dm)
    if D.dim() != 4:
        raise ValueError(f"colbert_kd_scores expects D.dim()==4, got {D.dim()}")
    from .autograd import maxsim

    return maxsim(Q, D, q_mask=qm, d_mask=dm)


def patched_colbert_scores_pairwise(queries_embeddings, documents_embeddings, queries_mask=None, documents_mask=None, *, mask=None):
    """Replacement for ``pylate.scores.colbert_scores_pairwise``: ``[B, Lq, d] x [B, Ld, d] -> [B]``."""
    Q, D = _tensors(queries_embeddings, documents_embeddings)
    qm, dm, raw_dm = _resolve_masks(queries_mask, documents_mask, mask)
    if not kernel_path_ok(Q, D):
        return _ORIGINAL["colbert_scores_pairwise"](Q, D, queries_mask=queries_mask, documents_mask=raw_dm)
    from .autograd import maxsim_pairs

    return maxsim_pairs(Q, D, q_mask=qm, d_mask=dm)


_PATCHED = {
    "colbert_scores": patched_colbert_scores,
    "colbert_kd_scores": patched_colbert_kd_scores,
    "colbert_scores_pairwise": patched_colbert_scores_pairwise,
}


def _defining_module():
    """PyLate <= 1.4 defines the scorers in ``pylate.scores.scores``, PyLate 1.5 in ``pylate.scores.colbert``."""
    try:
        return importlib.import_module("pylate.scores.scores"), False
    except ImportError:
        return importlib.import_module("pylate.scores.colbert"), True


def _loss_capture_targets(new_layout: bool):
    """Loss modules that bound a scorer at import time and need their own reference swapped."""
    if new_layout:
        return (("pylate.losses.distillation", "colbert_kd_scores"),)
    return (
        ("pylate.losses.contrastive", "colbert_scores"),
        ("pylate.losses.cached_contrastive", "colbert_scores"),
        ("pylate.losses.distillation", "colbert_kd_scores"),
    )


def patch_pylate():
    """Install the kernels as PyLate's MaxSim (idempotent).  No-op with a ``DeprecationWarning`` on
    PyLate >= 1.5.1, which selects the backend itself."""
    global _NATIVE_NOTICE_SHOWN
    if package_at_least("pylate", _PYLATE_NATIVE_MIN):
        if not _NATIVE_NOTICE_SHOWN:
            _NATIVE_NOTICE_SHOWN = True
            warnings.warn(
                f"late-interaction-kernels: PyLate >= {_PYLATE_NATIVE_MIN} ships native LIK support, so "
                "`patch_pylate()` is now a no-op. LIK is used automatically when installed; force it with "
                '`PYLATE_SCORES_BACKEND=lik` (or `backend="lik"`).',
                DeprecationWarning,
                stacklevel=2,
            )
        return
    if _ORIGINAL:
        return
    api = importlib.import_module("pylate.scores")
    defining, new_layout = _defining_module()
    for name in _HOOKED:
        if not hasattr(defining, name):  # colbert_scores_pairwise only exists in recent PyLate
            continue
        _ORIGINAL[name] = getattr(defining, name)
        setattr(defining, name, _PATCHED[name])
        setattr(api, name, _PATCHED[name])
    missed = []
    for mod_name, attr in _loss_capture_targets(new_layout):
        try:
            mod = importlib.import_module(mod_name)
        except ImportError:
            continue  # that loss module does not exist in this PyLate version
        except Exception as exc:  # noqa: BLE001
            missed.append(f"{mod_name}.{attr} ({type(exc).__name__}: {exc})")
            continue
        if hasattr(mod, attr):
            setattr(mod, attr, _PATCHED[attr])
        else:
            missed.append(f"{mod_name}.{attr}")
    if missed:
        warnings.warn(
            "late-interaction-kernels: `patch_pylate()` could not reach " + ", ".join(missed) + ". "
            "`pylate.scores.colbert_scores` is hooked, but any loss module that captured the un-patched symbol at "
            "import time will keep using vanilla PyLate. This usually means PyLate was refactored — check you're "
            "on a supported version (`pylate>=1.3.3`).",
            RuntimeWarning,
            stacklevel=2,
        )


def unpatch_pylate():
    """Restore PyLate's own scorers (no-op when not patched)."""
    if not _ORIGINAL:
        return
    api = importlib.import_module("pylate.scores")
    defining, new_layout = _defining_module()
    for name, fn in _ORIGINAL.items():
        setattr(defining, name, fn)
        setattr(api, name, fn)
    for mod_name, attr in _loss_capture_targets(new_layout):
        try:
            setattr(importlib.import_module(mod_name), attr, _ORIGINAL[attr])
        except Exception:  # noqa: BLE001
            pass
    _ORIGINAL.clear()
