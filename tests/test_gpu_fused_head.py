"""GPU tests of ``maxsim_from_hidden`` (documents projected on the fly), following the reference's
tests/test_fused_head.py and tests/test_fused_head_train.py: fp32 inputs against the committed golden file
(scores 1e-5, gradients 1e-4: the winners are unambiguous in fp32), bf16 inputs against the CPU oracle at the
bf16 tolerance of the reference's own test (2e-2), gradient buffers only for what asked for them, the piece loop
against one piece, and the error messages."""

import numpy as np
import pytest
import torch

import cases
from conftest import load_golden
from oracle import maxsim_oracle as O

pytestmark = pytest.mark.gpu


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def f32(t):
    return t.detach().float().cpu().numpy()


def test_fp32_scores_and_gradients_match_the_golden_file():
    from late_interaction_kernels_b200.fused_head import maxsim_from_hidden

    g = load_golden("from_hidden")
    Q, H, W, b, dm = cases.from_hidden_case(13)
    tQ, tH, tW, tb, tm = dev(Q), dev(H), dev(W), dev(b), dev(dm)
    assert O.rel_err(f32(maxsim_from_hidden(tQ, tH, tW, tb, tm)), g["scores_norm1"]) < 1e-5
    assert O.rel_err(f32(maxsim_from_hidden(tQ, tH, tW, tb, tm, normalize=False)), g["scores_norm0"]) < 1e-5
    assert O.rel_err(f32(maxsim_from_hidden(tQ, tH, tW, None, tm)), g["scores_nobias"]) < 1e-5
    # 2-D query -> [Nd]
    s1 = maxsim_from_hidden(tQ[0], tH, tW, tb, tm)
    assert s1.shape == (H.shape[0],) and O.rel_err(f32(s1), g["scores_norm1"][0]) < 1e-5
    for t in (tQ, tH, tW, tb):
        t.requires_grad_(True)
    out = maxsim_from_hidden(tQ, tH, tW, tb, tm)
    assert O.rel_err(f32(out), g["scores_norm1"]) < 1e-5
    (out * dev(g["g"])).sum().backward()
    for got, want in ((tQ.grad, g["gQ"]), (tH.grad, g["gH"]), (tW.grad, g["gW"]), (tb.grad, g["gb"])):
        assert O.rel_err(f32(got), want) < 1e-4


@pytest.mark.parametrize("need", [["Q"], ["H"], ["W"], ["Q", "H", "W", "b"]])
def test_only_requested_gradients_exist(need):
    from late_interaction_kernels_b200.fused_head import maxsim_from_hidden

    Q, H, W, b, dm = cases.from_hidden_case(5, Nq=1, Nd=4, Lq=16, Ld=64, d_model=256, d_out=64)
    t = {"Q": dev(Q), "H": dev(H), "W": dev(W), "b": dev(b)}
    for n in need:
        t[n].requires_grad_(True)
    maxsim_from_hidden(t["Q"], t["H"], t["W"], t["b"], dev(dm)).sum().backward()
    gQ, gH, gW, gb = O.from_hidden_grads(np.ones((1, 4), np.float32), Q, H, W, b, dm)
    want = {"Q": gQ, "H": gH, "W": gW, "b": gb}
    for n in ("Q", "H", "W", "b"):
        if n in need:
            assert O.rel_err(f32(t[n].grad), want[n]) < 1e-4, n
        else:
            assert t[n].grad is None


def test_bf16_documents_at_retrieval_shape_and_in_pieces(monkeypatch):
    from late_interaction_kernels_b200 import fused_head

    Q, H, W, b, dm = cases.from_hidden_case(21, Nq=4, Nd=300, Lq=32, Ld=96, d_model=256, d_out=128)
    tQ, tH, tW, tb, tm = dev(Q, torch.bfloat16), dev(H, torch.bfloat16), dev(W, torch.bfloat16), dev(b, torch.bfloat16), dev(dm)
    whole = fused_head.maxsim_from_hidden(tQ, tH, tW, tb, tm)
    want = O.maxsim_from_hidden(f32(tQ), f32(tH), f32(tW), f32(tb), dm)
    assert O.rel_err(f32(whole), want) < 2e-2
    monkeypatch.setattr(fused_head, "_PIECE_TOKENS", 96 * 37)  # 9 pieces, the last one short
    pieces = fused_head.maxsim_from_hidden(tQ, tH, tW, tb, tm)
    assert torch.equal(whole, pieces)
    # training through the pieces: same winners, so the same gradients as one piece up to fp32 summation order
    grads = []
    for ptok in (1 << 21, 96 * 37):
        monkeypatch.setattr(fused_head, "_PIECE_TOKENS", ptok)
        leaves = [x.clone().requires_grad_(True) for x in (tQ, tH, tW, tb)]
        fused_head.maxsim_from_hidden(*leaves, tm).sum().backward()
        grads.append([f32(x.grad) for x in leaves])
    for a, c in zip(*grads):
        assert O.rel_err(a, c) < 1e-2


def test_error_messages():
    from late_interaction_kernels_b200.fused_head import maxsim_from_hidden

    Q, H, W, b, dm = cases.from_hidden_case(3)
    tQ, tH, tW, tb = dev(Q), dev(H), dev(W), dev(b)
    with pytest.raises(ValueError, match="W must be"):
        maxsim_from_hidden(tQ, tH, tW[:, :-1].contiguous())
    with pytest.raises(ValueError, match="H_d must be"):
        maxsim_from_hidden(tQ, tH[0], tW)
    with pytest.raises(ValueError, match="b must be"):
        maxsim_from_hidden(tQ, tH, tW, tb[:-1])
    with pytest.raises(ValueError, match="same device"):
        maxsim_from_hidden(tQ, tH.cpu(), tW)


# ----------------------------------------------------------------------------- positives + explicit negatives in one launch
@pytest.mark.parametrize("lp,ln,masks", [(40, 40, False), (33, 50, False), (48, 20, True)])
def test_pos_neg_head_equals_the_two_separate_calls(lp, ln, masks):
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import _lib
    from late_interaction_kernels_b200.loss_heads import maxsim_pos_neg

    rng = np.random.default_rng(lp * 100 + ln)
    B, K, Lq, d = 6, 3, 16, 128
    Q = dev(cases.unit(rng.standard_normal((B, Lq, d))).astype(np.float32), torch.bfloat16)
    P = dev(cases.unit(rng.standard_normal((B, lp, d))).astype(np.float32), torch.bfloat16)
    N = dev(cases.unit(rng.standard_normal((B, K, ln, d))).astype(np.float32), torch.bfloat16)
    pm = nm = None
    if masks:
        pm = dev(cases.prefix_mask(rng.integers(1, lp + 1, size=B), lp))
        nm = dev(cases.prefix_mask(rng.integers(1, ln + 1, size=B * K), ln).reshape(B, K, ln))
    leaves = [x.clone().requires_grad_(True) for x in (Q, P, N)]
    n0 = _lib.load().lik_launch_count()
    pos, neg = maxsim_pos_neg(*leaves, pos_mask=pm, neg_mask=nm)
    fwd_launches = _lib.load().lik_launch_count() - n0
    ref = [x.clone().requires_grad_(True) for x in (Q, P, N)]
    pos_r = lik.maxsim_pairs(ref[0], ref[1], d_mask=pm)
    neg_r = lik.maxsim(ref[0], ref[2], d_mask=nm)
    assert torch.equal(pos, pos_r) and torch.equal(neg, neg_r)  # same kernel arithmetic on the same tokens
    assert fwd_launches <= 2, "mask lengths + one scoring launch"
    gp, gn = torch.randn_like(pos), torch.randn_like(neg)
    ((pos * gp).sum() + (neg * gn).sum()).backward()
    ((pos_r * gp).sum() + (neg_r * gn).sum()).backward()
    for a, b in zip(leaves, ref):
        assert O.rel_err(f32(a.grad), f32(b.grad)) < 2e-2  # grad_Q sums the two calls' bf16 results in another order
    # and against the oracle on the positives
    want = O.maxsim_pairs(f32(Q), f32(P), d_mask=None if pm is None else pm.cpu().numpy()) if hasattr(O, "maxsim_pairs") else None
    if want is not None:
        assert O.rel_err(f32(pos), want) < 2e-2
