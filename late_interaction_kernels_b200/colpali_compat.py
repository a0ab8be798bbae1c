"""colpali-engine drop-in: ``patch_colpali_engine()`` routes its MaxSim call sites through the B200
kernels (reference: colpali_compat.py:97-407).

Hooked: ``BaseVisualRetrieverProcessor.score_multi_vector`` (evaluation scoring) and the ``forward``
of the five ColBERT loss heads in ``colpali_engine.loss.late_interaction_losses``.  In-batch scores
use :func:`maxsim`; explicit negatives score the positive and the negatives of a query as one candidate list
(:func:`late_interaction_kernels_b200.loss_heads.maxsim_pos_neg`: one launch where the reference uses
:func:`maxsim_pairs` plus the 4-D :func:`maxsim`).  colpali-engine >= 0.3.17 selects the backend
itself; there the call only emits a ``DeprecationWarning``.  Anything the kernels do not take
(``use_smooth_max``, ``LIK_DISABLE=1``, tensors not on a B200) goes back to the original code.
"""

from __future__ import annotations

import importlib
import warnings

import torch

from ._hooks import kernel_path_ok
from ._utils import package_at_least

_COLPALI_NATIVE_MIN = "0.3.17"
_NATIVE_NOTICE_SHOWN = False
_ORIGINAL: dict = {}

_LOSSES_MODULE = "colpali_engine.loss.late_interaction_losses"
_SCORE_KEY = "BaseVisualRetrieverProcessor.score_multi_vector"


def patched_score_multi_vector(qs, ps, batch_size: int = 128, device=None):
    """Replacement for ``score_multi_vector``: pad each (query batch, passage batch) tile and score it
    with one kernel call; returns fp32 ``[len(qs), len(ps)]`` on the CPU like the original."""
    from colpali_engine.utils.torch_utils import get_torch_device  # type: ignore

    device = device or get_torch_device("auto")
    if len(qs) == 0:
        raise ValueError("No queries provided")
    if len(ps) == 0:
        raise ValueError("No passages provided")
    pad = torch.nn.utils.rnn.pad_sequence
    rows = []
    for i in range(0, len(qs), batch_size):
        q = pad(qs[i : i + batch_size], batch_first=True, padding_value=0).to(device)
        tiles = []
        for j in range(0, len(ps), batch_size):
            p = pad(ps[j : j + batch_size], batch_first=True, padding_value=0).to(device)
            if kernel_path_ok(q, p):
                from .autograd import maxsim

                tiles.append(maxsim(q, p))
            else:
                tiles.append(torch.einsum("bnd,csd->bcns", q, p).max(dim=3)[0].sum(dim=2))
        rows.append(torch.cat(tiles, dim=1).cpu())
    scores = torch.cat(rows, dim=0).to(torch.float32)
    assert scores.shape[0] == len(qs), f"Expected {len(qs)} scores, got {scores.shape[0]}"
    return scores


def _inbatch_scores(self, Q, D):
    """In-batch ``[B, B]`` scores for a loss head, or ``None`` to fall through to the original."""
    if self.use_smooth_max or not kernel_path_ok(Q, D):
        return None
    from .autograd import maxsim

    lengths = (Q[:, :, 0] != 0).sum(dim=1)
    scores = maxsim(Q, D)
    if self.normalize_scores:
        scores = self._apply_normalization(scores, lengths)
    return scores


def _prepared_scores(self, Q, D, offset, key):
    scores = _inbatch_scores(self, Q, D)
    if scores is None:
        return None, None
    _, pos_idx = self._get_idx(scores.size(0), offset, scores.device)
    if self.pos_aware_negative_filtering:
        self._filter_high_negatives(scores, pos_idx)
    return scores, pos_idx


def patched_colbert_loss_forward(self, query_embeddings, doc_embeddings, offset: int = 0):
    """Replacement for ``ColbertLoss.forward`` (softmax cross-entropy over in-batch scores)."""
    scores, pos_idx = _prepared_scores(self, query_embeddings, doc_embeddings, offset, "ColbertLoss.forward")
    if scores is None:
        return _ORIGINAL["ColbertLoss.forward"](self, query_embeddings, doc_embeddings, offset)
    return self.ce_loss(scores / self.temperature, pos_idx)


def patched_colbert_pairwise_ce_forward(self, query_embeddings, doc_embeddings, offset: int = 0):
    """Replacement for ``ColbertPairwiseCELoss.forward`` (softplus of hardest negative minus positive)."""
    scores, _ = _prepared_scores(self, query_embeddings, doc_embeddings, offset, "ColbertPairwiseCELoss.forward")
    if scores is None:
        return _ORIGINAL["ColbertPairwiseCELoss.forward"](self, query_embeddings, doc_embeddings, offset)
    pos = scores.diagonal(offset=offset)
    top2 = scores.topk(2, dim=1).values
    neg = torch.where(top2[:, 0] == pos, top2[:, 1], top2[:, 0])
    return torch.nn.functional.softplus((neg - pos) / self.temperature).mean()


def patched_colbert_sigmoid_forward(self, query_embeddings, doc_embeddings, offset: int = 0):
    """Replacement for ``ColbertSigmoidLoss.forward`` (pairwise sigmoid over all in-batch pairs)."""
    scores, pos_idx = _prepared_scores(self, query_embeddings, doc_embeddings, offset, "ColbertSigmoidLoss.forward")
    if scores is None:
        return _ORIGINAL["ColbertSigmoidLoss.forward"](self, query_embeddings, doc_embeddings, offset)
    B = scores.size(0)
    sign = -torch.ones(B * B, device=scores.device)
    sign[pos_idx * (B + 1)] = 1.0
    return torch.nn.functional.softplus(-(scores.view(-1) / self.temperature) * sign).mean()


def _negative_scores(self, Q, pos_D, neg_D, offset):
    """``(pos [B], neg [B, n_neg])`` for the explicit-negative heads, or ``None`` to fall through."""
    if self.use_smooth_max or not kernel_path_ok(Q, pos_D):
        return None
    if neg_D.device != Q.device or neg_D.shape[-1] < 8:
        return None
    from .loss_heads import maxsim_pos_neg

    lengths = (Q[:, :, 0] != 0).sum(dim=1)
    # positives and negatives in one candidate list per query: one scoring launch, one backward
    pos, neg = maxsim_pos_neg(Q, pos_D[offset : offset + Q.size(0)], neg_D)
    if self.normalize_scores:
        pos = self._apply_normalization(pos, lengths)
        neg = self._apply_normalization(neg, lengths)
    return pos, neg


def _negative_loss(self, Q, pos_D, neg_D, offset, key, inner_attr):
    scored = _negative_scores(self, Q, pos_D, neg_D, offset)
    if scored is None:
        return _ORIGINAL[key](self, Q, pos_D, neg_D, offset)
    pos, neg = scored
    loss = torch.nn.functional.softplus((neg - pos.unsqueeze(1)) / self.temperature).mean()
    w = self.in_batch_term_weight
    if w > 0:
        # the inner head's forward is hooked at class level, so this term is fused too
        loss = loss * (1 - w) + getattr(self, inner_attr)(Q, pos_D, offset) * w
    return loss


def patched_colbert_negative_ce_forward(self, query_embeddings, doc_embeddings, neg_doc_embeddings, offset: int = 0):
    """Replacement for ``ColbertNegativeCELoss.forward``."""
    return _negative_loss(self, query_embeddings, doc_embeddings, neg_doc_embeddings, offset,
                          "ColbertNegativeCELoss.forward", "inner_loss")


def patched_colbert_pairwise_negative_ce_forward(self, query_embeddings, doc_embeddings, neg_doc_embeddings, offset: int = 0):
    """Replacement for ``ColbertPairwiseNegativeCELoss.forward``."""
    return _negative_loss(self, query_embeddings, doc_embeddings, neg_doc_embeddings, offset,
                          "ColbertPairwiseNegativeCELoss.forward", "inner_pairwise")


_LOSS_HOOKS = (
    ("ColbertLoss", patched_colbert_loss_forward),
    ("ColbertPairwiseCELoss", patched_colbert_pairwise_ce_forward),
    ("ColbertSigmoidLoss", patched_colbert_sigmoid_forward),
    ("ColbertNegativeCELoss", patched_colbert_negative_ce_forward),
    ("ColbertPairwiseNegativeCELoss", patched_colbert_pairwise_negative_ce_forward),
)


def patch_colpali_engine():
    """Install the kernels across colpali-engine's MaxSim call sites (idempotent)."""
    global _NATIVE_NOTICE_SHOWN
    if package_at_least("colpali-engine", _COLPALI_NATIVE_MIN):
        if not _NATIVE_NOTICE_SHOWN:
            _NATIVE_NOTICE_SHOWN = True
            warnings.warn(
                f"late-interaction-kernels: colpali-engine >= {_COLPALI_NATIVE_MIN} ships native LIK support, so "
                "`patch_colpali_engine()` is now a no-op. LIK is used automatically when installed; force it over "
                "torch with `COLPALI_SCORES_BACKEND=lik`.",
                DeprecationWarning,
                stacklevel=2,
            )
        return
    if _ORIGINAL:
        return
    missed = []
    try:
        proc = importlib.import_module("colpali_engine.utils.processing_utils").BaseVisualRetrieverProcessor
        _ORIGINAL[_SCORE_KEY] = proc.score_multi_vector
        proc.score_multi_vector = staticmethod(patched_score_multi_vector)
    except ImportError:
        missed.append("colpali_engine.utils.processing_utils")
    try:
        losses = importlib.import_module(_LOSSES_MODULE)
    except ImportError:
        losses = None
        missed.append(_LOSSES_MODULE)
    if losses is not None:
        for cls_name, fn in _LOSS_HOOKS:
            cls = getattr(losses, cls_name, None)
            if cls is None:
                missed.append(f"{_LOSSES_MODULE}.{cls_name}")
                continue
            _ORIGINAL[f"{cls_name}.forward"] = cls.forward
            cls.forward = fn
    if not _ORIGINAL:
        raise ImportError(
            "late-interaction-kernels: `patch_colpali_engine()` couldn't reach any expected colpali_engine entry "
            "point. Install with `pip install colpali-engine` and check the version is >=0.3.10."
        )
    if missed:
        warnings.warn(
            "late-interaction-kernels: `patch_colpali_engine()` could not reach " + ", ".join(missed) + ". The "
            "reachable entry points are still hooked; any unreachable one keeps using vanilla colpali_engine. This "
            "usually means colpali_engine was refactored — check the installed version.",
            RuntimeWarning,
            stacklevel=2,
        )


def unpatch_colpali_engine():
    """Restore colpali-engine's own implementations (no-op when not patched)."""
    if not _ORIGINAL:
        return
    if _SCORE_KEY in _ORIGINAL:
        proc = importlib.import_module("colpali_engine.utils.processing_utils").BaseVisualRetrieverProcessor
        # class attribute access unwrapped the staticmethod when it was stashed: wrap it again
        proc.score_multi_vector = staticmethod(_ORIGINAL[_SCORE_KEY])
    losses = None
    for cls_name, _ in _LOSS_HOOKS:
        key = f"{cls_name}.forward"
        if key in _ORIGINAL:
            losses = losses or importlib.import_module(_LOSSES_MODULE)
            getattr(losses, cls_name).forward = _ORIGINAL[key]
    _ORIGINAL.clear()
