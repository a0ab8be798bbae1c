"""patch_pylate / patch_colpali_engine against fake module trees injected into sys.modules: patching,
idempotence, restore, legacy ``mask=``, fall-through to the library's own function when the tensors are
not on a B200, and the no-op + DeprecationWarning on library versions that ship their own backend."""

import sys
import types
import warnings

import pytest
import torch

from late_interaction_kernels_b200 import colpali_compat, pylate_compat


def _fake_pylate(new_layout=False):
    calls = []

    def colbert_scores(q, d, queries_mask=None, documents_mask=None):
        calls.append(("scores", queries_mask, documents_mask))
        return torch.einsum("ash,bth->abst", q, d).amax(3).sum(2)

    def colbert_kd_scores(q, d, queries_mask=None, documents_mask=None):
        calls.append(("kd", queries_mask, documents_mask))
        return torch.einsum("ash,abth->abst", q, d).amax(3).sum(2)

    def colbert_scores_pairwise(q, d, queries_mask=None, documents_mask=None):
        calls.append(("pair", queries_mask, documents_mask))
        return torch.einsum("ash,ath->ast", q, d).amax(2).sum(1)

    mods = {}
    def mod(name):
        m = types.ModuleType(name)
        mods[name] = m
        return m

    pylate = mod("pylate")
    scores = mod("pylate.scores")
    defining = mod("pylate.scores.colbert" if new_layout else "pylate.scores.scores")
    utils = mod("pylate.utils")
    tensor = mod("pylate.utils.tensor")
    losses = mod("pylate.losses")
    contrastive = mod("pylate.losses.contrastive")
    cached = mod("pylate.losses.cached_contrastive")
    distillation = mod("pylate.losses.distillation")
    tensor.convert_to_tensor = lambda x: x if isinstance(x, torch.Tensor) else torch.stack(list(x))
    for m in (scores, defining):
        m.colbert_scores, m.colbert_kd_scores, m.colbert_scores_pairwise = colbert_scores, colbert_kd_scores, colbert_scores_pairwise
    contrastive.colbert_scores = colbert_scores
    cached.colbert_scores = colbert_scores
    distillation.colbert_kd_scores = colbert_kd_scores
    pylate.scores, pylate.utils, pylate.losses = scores, utils, losses
    utils.tensor = tensor
    return mods, calls, (colbert_scores, colbert_kd_scores, colbert_scores_pairwise)


@pytest.fixture
def fake_pylate(monkeypatch):
    mods, calls, originals = _fake_pylate()
    for k, v in mods.items():
        monkeypatch.setitem(sys.modules, k, v)
    monkeypatch.setattr(pylate_compat, "package_at_least", lambda name, minimum: False)
    pylate_compat._ORIGINAL.clear()
    yield mods, calls, originals
    pylate_compat._ORIGINAL.clear()


def test_patch_unpatch_pylate_and_cpu_fallthrough(fake_pylate):
    mods, calls, (orig_s, orig_kd, orig_p) = fake_pylate
    pylate_compat.patch_pylate()
    pylate_compat.patch_pylate()  # idempotent
    s = mods["pylate.scores"]
    assert s.colbert_scores is pylate_compat.patched_colbert_scores
    assert mods["pylate.scores.scores"].colbert_kd_scores is pylate_compat.patched_colbert_kd_scores
    assert mods["pylate.losses.contrastive"].colbert_scores is pylate_compat.patched_colbert_scores
    assert mods["pylate.losses.distillation"].colbert_kd_scores is pylate_compat.patched_colbert_kd_scores
    # CPU tensors are handed back to PyLate's own function, with the legacy mask= forwarded
    Q, D = torch.randn(2, 3, 8), torch.randn(4, 5, 8)
    m = torch.ones(4, 5)
    out = s.colbert_scores(Q, D, mask=m)
    assert out.shape == (2, 4) and calls[-1][0] == "scores" and calls[-1][2] is m
    out = s.colbert_kd_scores(Q, torch.randn(2, 3, 5, 8))
    assert out.shape == (2, 3) and calls[-1][0] == "kd"
    out = s.colbert_scores_pairwise(Q, torch.randn(2, 5, 8))
    assert out.shape == (2,) and calls[-1][0] == "pair"
    pylate_compat.unpatch_pylate()
    assert s.colbert_scores is orig_s and mods["pylate.losses.distillation"].colbert_kd_scores is orig_kd
    assert not pylate_compat._ORIGINAL
    pylate_compat.unpatch_pylate()  # no-op


def test_lik_disable_env_falls_through(fake_pylate, monkeypatch):
    from late_interaction_kernels_b200._hooks import kernel_path_ok

    Q, D = torch.randn(2, 3, 8), torch.randn(4, 5, 8)
    assert kernel_path_ok(Q, D) is False  # CPU
    monkeypatch.setenv("LIK_DISABLE", "1")
    assert kernel_path_ok(Q, D) is False
    assert kernel_path_ok(torch.randn(2, 3, 4), torch.randn(2, 3, 4)) is False  # d < 8


def test_native_pylate_is_a_noop_with_deprecation_warning(fake_pylate, monkeypatch):
    mods, _, (orig_s, _, _) = fake_pylate
    monkeypatch.setattr(pylate_compat, "package_at_least", lambda name, minimum: True)
    monkeypatch.setattr(pylate_compat, "_NATIVE_NOTICE_SHOWN", False)
    with pytest.warns(DeprecationWarning, match="no-op"):
        pylate_compat.patch_pylate()
    assert mods["pylate.scores"].colbert_scores is orig_s and not pylate_compat._ORIGINAL
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        pylate_compat.patch_pylate()  # the notice is shown once


def test_missing_loss_capture_warns(fake_pylate):
    mods, _, _ = fake_pylate
    del mods["pylate.losses.contrastive"].colbert_scores
    with pytest.warns(RuntimeWarning, match="could not reach"):
        pylate_compat.patch_pylate()
    pylate_compat.unpatch_pylate()


def _fake_colpali(monkeypatch):
    def mod(name):
        m = types.ModuleType(name)
        monkeypatch.setitem(sys.modules, name, m)
        return m

    root = mod("colpali_engine")
    utils = mod("colpali_engine.utils")
    proc = mod("colpali_engine.utils.processing_utils")
    tu = mod("colpali_engine.utils.torch_utils")
    loss = mod("colpali_engine.loss")
    lil = mod("colpali_engine.loss.late_interaction_losses")
    tu.get_torch_device = lambda _: "cpu"

    class BaseVisualRetrieverProcessor:
        @staticmethod
        def score_multi_vector(qs, ps, batch_size=128, device=None):
            return "original"

    proc.BaseVisualRetrieverProcessor = BaseVisualRetrieverProcessor

    class _Head(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.use_smooth_max = False
            self.normalize_scores = False
            self.temperature = 0.5
            self.pos_aware_negative_filtering = False
            self.in_batch_term_weight = 0.0
            self.ce_loss = torch.nn.CrossEntropyLoss()

        def _get_idx(self, b, offset, device):
            idx = torch.arange(b, device=device)
            return idx, idx + offset

        def forward(self, *a, **k):
            return "original-forward"

    for name in ("ColbertLoss", "ColbertPairwiseCELoss", "ColbertSigmoidLoss", "ColbertNegativeCELoss", "ColbertPairwiseNegativeCELoss"):
        setattr(lil, name, type(name, (_Head,), {}))
    root.utils, root.loss = utils, loss
    return proc, lil


def test_patch_unpatch_colpali(monkeypatch):
    proc, lil = _fake_colpali(monkeypatch)
    monkeypatch.setattr(colpali_compat, "package_at_least", lambda name, minimum: False)
    colpali_compat._ORIGINAL.clear()
    colpali_compat.patch_colpali_engine()
    colpali_compat.patch_colpali_engine()
    assert lil.ColbertLoss.forward is colpali_compat.patched_colbert_loss_forward
    P = proc.BaseVisualRetrieverProcessor
    # CPU inputs: the patched scorer still returns the right numbers through the einsum tile
    qs = [torch.randn(3, 8), torch.randn(5, 8)]
    ps = [torch.randn(4, 8), torch.randn(6, 8), torch.randn(2, 8)]
    out = P.score_multi_vector(qs, ps, batch_size=2, device="cpu")
    want = torch.stack([torch.stack([(q @ p.T).amax(1).sum() for p in ps]) for q in qs])
    assert out.shape == (2, 3) and torch.allclose(out, want, atol=1e-5)
    with pytest.raises(ValueError, match="No queries"):
        P.score_multi_vector([], ps)
    # loss heads fall through to the original forward on CPU tensors
    assert lil.ColbertLoss()(torch.randn(2, 3, 8), torch.randn(2, 4, 8)) == "original-forward"
    assert lil.ColbertNegativeCELoss()(torch.randn(2, 3, 8), torch.randn(2, 4, 8), torch.randn(2, 2, 4, 8)) == "original-forward"
    colpali_compat.unpatch_colpali_engine()
    assert P.score_multi_vector(qs, ps) == "original" and not colpali_compat._ORIGINAL
    assert lil.ColbertLoss()(None, None) == "original-forward"
    monkeypatch.setattr(colpali_compat, "package_at_least", lambda name, minimum: True)
    monkeypatch.setattr(colpali_compat, "_NATIVE_NOTICE_SHOWN", False)
    with pytest.warns(DeprecationWarning, match="no-op"):
        colpali_compat.patch_colpali_engine()
    assert not colpali_compat._ORIGINAL


def test_public_api_keywords_are_frozen():
    import inspect

    import late_interaction_kernels_b200 as lik

    for fn in (lik.maxsim, lik.maxsim_pairs):
        assert {"Q", "D", "q_mask", "d_mask", "normalize"} <= set(inspect.signature(fn).parameters)
    assert {"Q", "D", "top_k", "q_mask", "d_mask", "normalize", "chunk", "largest", "sorted"} <= set(inspect.signature(lik.retrieve).parameters)
