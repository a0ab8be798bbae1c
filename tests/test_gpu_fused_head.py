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

    monkeypatch.setattr(fused_head, "_CHAINED", False)  # the GEMM-in-pieces forward
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


# ----------------------------------------------------------------------------- projection chained into the scoring MMA
def _chained_case(seed, Nq, Nd, Lq, Ld, d_model, d_out, dtype, mask):
    Q, H, W, b, dm = cases.from_hidden_case(seed, Nq=Nq, Nd=Nd, Lq=Lq, Ld=Ld, d_model=d_model, d_out=d_out)
    rng = np.random.default_rng(seed + 1)
    if mask == "none":
        dm = None
    elif mask == "holes":
        dm = rng.random((Nd, Ld)) < 0.7
        dm[0] = False  # a document without a valid token
        dm[1] = True
    t = [dev(x, dtype) for x in (Q, H, W, b)]
    return t, dm


@pytest.mark.parametrize("Nq,Nd,Lq,Ld,d_model,d_out,dtype,mask,bias,normalize", [
    (4, 40, 32, 300, 768, 128, torch.bfloat16, "prefix", True, True),    # one query tile, ragged lengths
    (8, 33, 32, 130, 384, 96, torch.bfloat16, "holes", True, True),      # two query tiles, d_out 96, masks with holes
    (1, 200, 32, 257, 200, 64, torch.float16, "none", False, True),      # K slab with a zero-filled tail, more documents than SMs
    (3, 17, 40, 128, 256, 128, torch.bfloat16, "prefix", True, False),   # queries that do not fill the tile, no normalisation
    (2, 9, 128, 1024, 768, 128, torch.bfloat16, "none", True, True),     # one query per tile, long documents
    (2, 50, 16, 70, 64, 32, torch.bfloat16, "prefix", True, True),       # one K slab on either side (d_model 64, d_out 32)
    (5, 3, 8, 4100, 1024, 128, torch.float16, "holes", False, True),     # few long documents, 16 K slabs, 40 query rows
])
def test_chained_kernel_against_the_oracle_and_the_gemm_path(monkeypatch, Nq, Nd, Lq, Ld, d_model, d_out, dtype, mask, bias, normalize):
    from late_interaction_kernels_b200 import _lib, fused_head

    (tQ, tH, tW, tb), dm = _chained_case(Nq * 7 + Nd, Nq, Nd, Lq, Ld, d_model, d_out, dtype, mask)
    tm = None if dm is None else dev(dm)
    if not bias:
        tb = None
    n0 = _lib.load().lik_launch_count()
    got = fused_head.maxsim_from_hidden(tQ, tH, tW, tb, tm, normalize=normalize)
    launches = _lib.load().lik_launch_count() - n0
    assert launches == (1 if dm is None else 2), "one kernel (plus the mask lengths)"
    torch.cuda.synchronize()
    from late_interaction_kernels_b200 import _ops
    _ops.check_device_status()
    want = O.maxsim_from_hidden(f32(tQ), f32(tH), f32(tW), None if tb is None else f32(tb), dm, normalize=normalize)
    assert got.shape == (Nq, Nd)
    assert O.rel_err(f32(got), want) < 2e-2
    # the GEMM-in-pieces forward rounds the same projected values: the two agree far inside the bf16 tolerance
    monkeypatch.setattr(fused_head, "_CHAINED", False)
    ref = fused_head.maxsim_from_hidden(tQ, tH, tW, tb, tm, normalize=normalize)
    assert O.rel_err(f32(got), f32(ref)) < 3e-3
    # a second run gives the same bits
    monkeypatch.setattr(fused_head, "_CHAINED", True)
    assert torch.equal(got, fused_head.maxsim_from_hidden(tQ, tH, tW, tb, tm, normalize=normalize))


def test_chained_kernel_winners_and_training_step(monkeypatch):
    from late_interaction_kernels_b200 import fused_head

    (tQ, tH, tW, tb), dm = _chained_case(5, 4, 24, 32, 200, 256, 128, torch.bfloat16, "holes")
    tm = dev(dm)
    s, am = fused_head._forward(tQ, tH, tW, tb, tm, True, True)
    monkeypatch.setattr(fused_head, "_CHAINED", False)
    s_ref, am_ref = fused_head._forward(tQ, tH, tW, tb, tm, True, True)
    monkeypatch.setattr(fused_head, "_CHAINED", True)
    assert (am == am_ref).float().mean().item() > 0.97  # near-ties may fall the other way between two GEMM orders
    assert (am[:, 0] == -1).all() and (am[:, 1] >= 0).all()
    # every winner is a valid token and reproduces its score from the projected, normalised tokens
    P = torch.nn.functional.normalize(torch.nn.functional.linear(tH, tW, tb).float(), dim=-1)
    idx = am.clamp(min=0).long()
    picked = torch.gather(P.unsqueeze(0).expand(4, -1, -1, -1), 2, idx.unsqueeze(-1).expand(-1, -1, -1, P.shape[-1]))
    sims = (picked * tQ.float().unsqueeze(1)).sum(-1) * (am >= 0)
    assert O.rel_err(f32(sims.sum(-1)), f32(s)) < 1e-2
    assert torch.gather(tm.unsqueeze(0).expand(4, -1, -1), 2, idx)[am >= 0].all()
    # gradients through the chained forward: against torch autograd (fp32) on the same winners - an fp64 oracle picks
    # other winners in near-ties, which swaps whole rows of the gradients
    leaves = [x.clone().requires_grad_(True) for x in (tQ, tH, tW, tb)]
    g = torch.randn(4, 24, device="cuda")
    (fused_head.maxsim_from_hidden(*leaves, tm) * g).sum().backward()
    rQ, rH, rW, rb = [x.detach().float().requires_grad_(True) for x in (tQ, tH, tW, tb)]
    P = torch.nn.functional.normalize(torch.nn.functional.linear(rH, rW, rb), dim=-1)
    picked = torch.gather(P.unsqueeze(0).expand(4, -1, -1, -1), 2, idx.unsqueeze(-1).expand(-1, -1, -1, P.shape[-1]))
    (((picked * rQ.unsqueeze(1)).sum(-1) * (am >= 0)).sum(-1) * g).sum().backward()
    for got, want in zip(leaves, (rQ, rH, rW, rb)):
        assert O.rel_err(f32(got.grad), f32(want.grad)) < 2e-2


def test_chained_kernel_declines_what_it_cannot_hold():
    from late_interaction_kernels_b200 import _ops

    Q, H, W, b, dm = cases.from_hidden_case(2, Nq=9, Nd=6, Lq=32, Ld=64, d_model=128, d_out=128)  # three query tiles
    q = _ops.padded_spec(dev(Q, torch.bfloat16))
    h = _ops.padded_spec(dev(H, torch.bfloat16))
    assert _ops.hidden_forward(q, h, dev(W, torch.bfloat16), None, normalize=True) is None
    W48 = dev(W[:48], torch.bfloat16)  # d_out not a multiple of 32
    q48 = _ops.padded_spec(dev(Q[:2, :, :48], torch.bfloat16))
    assert _ops.hidden_forward(q48, h, W48, None, normalize=True) is None


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


def test_tile_grid_in_one_launch_equals_the_per_tile_calls():
    """The (query mini-batch, document mini-batch) grid of a cached-contrastive loss: one call gives the blocks the
    per-tile calls give, and the same gradients on every chunk."""
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200.loss_heads import maxsim_tiles

    rng = np.random.default_rng(77)
    d = 128
    qs = [dev(cases.unit(rng.standard_normal((b, l, d))).astype(np.float32), torch.bfloat16) for b, l in ((3, 40), (2, 33), (4, 40))]
    ds = [dev(cases.unit(rng.standard_normal((b, l, d))).astype(np.float32), torch.bfloat16) for b, l in ((5, 120), (3, 257))]
    dms = [dev(cases.prefix_mask(rng.integers(1, 121, size=5), 120)), None]
    a = [x.clone().requires_grad_(True) for x in qs + ds]
    b = [x.clone().requires_grad_(True) for x in qs + ds]
    grid = maxsim_tiles(a[:3], a[3:], d_masks=dms)
    assert grid.shape == (9, 8)
    g = torch.randn_like(grid)
    (grid * g).sum().backward()
    r0 = 0
    total = 0.0
    for i, q in enumerate(b[:3]):
        c0 = 0
        for j, dd in enumerate(b[3:]):
            tile = lik.maxsim(q, dd, d_mask=dms[j])
            blk = grid[r0:r0 + q.shape[0], c0:c0 + dd.shape[0]]
            assert torch.equal(tile, blk), (i, j)  # same kernel arithmetic on the same tokens
            total = total + (tile * g[r0:r0 + q.shape[0], c0:c0 + dd.shape[0]]).sum()
            c0 += dd.shape[0]
        r0 += q.shape[0]
    total.backward()
    for x, y in zip(a, b):
        assert O.rel_err(f32(x.grad), f32(y.grad)) < 2e-2  # the per-tile path sums bf16 partial gradients


def test_hidden_winners_and_scatter_rows_against_numpy():
    from late_interaction_kernels_b200 import _ops

    rng = np.random.default_rng(3)
    Nq, Nd, Lq, Ld, width = 3, 7, 10, 77, 24
    am = rng.integers(-1, Ld, size=(Nq, Nd, Lq)).astype(np.int32)
    am[:, 2] = -1  # a document nobody picked
    am[:, 3] = 5   # one token picked by everybody
    S = min(Nq * Lq, Ld)
    am_c, rows, counts, bitmap, prefix = _ops.hidden_winners(dev(am), Nq, Nd, Lq, Ld, S)
    am_c, rows, counts = am_c.cpu().numpy(), rows.cpu().numpy().reshape(Nd, S), counts.cpu().numpy()
    for j in range(Nd):
        uniq = np.unique(am[:, j][am[:, j] >= 0])
        assert counts[j] == len(uniq)
        assert (rows[j, :len(uniq)] == j * Ld + uniq).all()
        assert (rows[j, len(uniq):] == j * Ld).all()
        want = np.where(am[:, j] >= 0, np.searchsorted(uniq, np.maximum(am[:, j], 0)), -1)
        assert (am_c[:, j] == want).all()
    compact = torch.randn(Nd * S, width, device="cuda")
    out = torch.full((Nd * Ld, width), 7.0, device="cuda")
    _ops.hidden_scatter_rows(compact, bitmap, prefix, out, Nd, Ld, S)
    want = torch.zeros_like(out)
    for j in range(Nd):
        want[torch.from_numpy(rows[j, :counts[j]]).cuda()] = compact[j * S:j * S + counts[j]]
    assert torch.equal(out, want)
