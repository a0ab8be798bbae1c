"""GPU parity: the CUDA path (through the public API and the C ABI) against the CPU oracle and the
golden vectors written by the reference.  Tolerances: fp32 1e-5, bf16/fp16 2e-2, FP8 6e-2 relative
(``rel_err`` = max|a-b| / max|b|), gradients the same; integer outputs exact.
"""

import numpy as np
import pytest
import torch
from conftest import load_golden

import cases
from oracle import maxsim_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def L():
    import late_interaction_kernels_b200 as lik

    return lik


def dev(x, dtype=None):
    if x is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def f32(t):
    return t.detach().float().cpu().numpy()


def rounded(x, dtype):
    """numpy fp32 view of x after rounding to the torch dtype (what the kernel actually sees)."""
    return torch.from_numpy(np.ascontiguousarray(x)).to(dtype).float().numpy()


# ----------------------------------------------------------------------------- dense forward
def test_config1_fp32_matches_reference_golden():
    g = load_golden("config1")
    Q, D, qm, dm = cases.config1()
    s = L().maxsim(dev(Q), dev(D), dev(qm), dev(dm), normalize=True)
    assert s.dtype == torch.float32 and s.shape == (32, 32)
    assert O.rel_err(f32(s), g["scores"]) < 1e-5
    s2 = L().maxsim(dev(Q), dev(D), dev(qm), dev(dm), normalize=False)
    assert O.rel_err(f32(s2), g["scores_nonorm"]) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 16), (3, 5, 7, 19, 16), (4, 6, 32, 300, 128), (2, 3, 33, 65, 96),
                                   (8, 8, 32, 64, 128), (2, 2, 130, 257, 64), (3, 4, 5, 9, 37), (1, 9, 128, 40, 128)])
@pytest.mark.parametrize("normalize", [False, True])
def test_dense_forward_shapes(dtype, shape, normalize):
    Nq, Nd, Lq, Ld, d = shape
    Q, D, qm, dm = cases.dense_case(sum(shape), Nq, Nd, Lq, Ld, d, q_len=(1, Lq), d_len=(1, Ld), normalized=not normalize)
    Qr, Dr = rounded(Q, dtype), rounded(D, dtype)
    want, want_am = O.maxsim(Qr, Dr, qm, dm, normalize=normalize, return_argmax=True)
    from late_interaction_kernels_b200.forward import maxsim_forward

    s, am = maxsim_forward(dev(Q, dtype), dev(D, dtype), dev(qm), dev(dm), save_argmax=True, normalize=normalize)
    s_noarg, none = maxsim_forward(dev(Q, dtype), dev(D, dtype), dev(qm), dev(dm), save_argmax=False, normalize=normalize)
    assert none is None
    assert torch.equal(s, s_noarg), "argmax and no-argmax paths must give bit-identical scores"
    assert O.rel_err(f32(s), want) < TOL[dtype]
    assert am.shape == (Nq * Nd, Lq) and am.dtype == torch.int32
    if dtype == torch.float32:
        got = am.cpu().numpy().reshape(Nq, Nd, Lq)
        valid_q = qm  # only rows the score uses are compared
        assert (got[np.broadcast_to(valid_q[:, None, :], got.shape)] ==
                want_am[np.broadcast_to(valid_q[:, None, :], got.shape)]).mean() > 0.999


def test_random_masks_and_fully_masked_rows():
    g = load_golden("random_mask")
    Q, D, qm, dm = cases.random_mask_case(1)
    s = L().maxsim(dev(Q), dev(D), dev(qm), dev(dm))
    assert O.rel_err(f32(s), g["scores"]) < 1e-5
    assert (s[:, 1] == 0).all() and (s[2] == 0).all()
    sn = L().maxsim(dev(Q), dev(D), dev(qm), dev(dm), normalize=True)
    assert O.rel_err(f32(sn), g["scores_norm"]) < 1e-5
    assert O.rel_err(f32(L().maxsim(dev(Q), dev(D))), g["scores_nomask"]) < 1e-5
    s2 = L().maxsim(dev(Q[0]), dev(D[0]), dev(qm[0]), dev(dm[0]))
    assert s2.shape == () and abs(float(s2) - float(g["scores_2d"])) < 1e-4
    assert O.rel_err(f32(L().maxsim(dev(Q[0]), dev(D))), g["scores_q2d"]) < 1e-5
    from late_interaction_kernels_b200.forward import maxsim_forward

    _, am = maxsim_forward(dev(Q), dev(D), dev(qm), dev(dm), save_argmax=True)
    assert (am.view(3, 5, 7)[:, 1] == -1).all(), "a fully masked document has no winner"


def test_forward_is_bitwise_deterministic_and_strided_inputs():
    Q, D, qm, dm = cases.dense_case(5, 6, 40, 32, 77, 128, d_len=(1, 77), normalized=True)
    a = L().maxsim(dev(Q, torch.bfloat16), dev(D, torch.bfloat16), None, dev(dm))
    b = L().maxsim(dev(Q, torch.bfloat16), dev(D, torch.bfloat16), None, dev(dm))
    assert torch.equal(a, b)
    Qs = dev(np.concatenate([Q, Q], -1), torch.bfloat16)[..., :128]  # non-contiguous view
    assert torch.equal(L().maxsim(Qs, dev(D, torch.bfloat16), None, dev(dm)), a)


def test_errors():
    lik = L()
    Q, D = torch.randn(2, 3, 16, device="cuda"), torch.randn(2, 4, 16, device="cuda")
    with pytest.raises(ValueError, match="backward= must be one of"):
        lik.maxsim(Q, D, backward="fast")
    with pytest.raises(ValueError, match="share the embedding dim"):
        lik.maxsim(Q, torch.randn(2, 4, 8, device="cuda"))
    with pytest.raises(ValueError, match="same device"):
        lik.maxsim(Q, D.cpu())
    with pytest.raises(RuntimeError, match="CUDA"):
        lik.maxsim(Q.cpu(), D.cpu())
    with pytest.raises(ValueError, match="needs Q to be"):
        lik.maxsim(Q[0], torch.randn(2, 2, 4, 16, device="cuda"))
    with pytest.raises(ValueError, match=r"D.shape\[0\] == Q.shape\[0\]"):
        lik.maxsim(Q, torch.randn(3, 2, 4, 16, device="cuda"))
    with pytest.raises(ValueError, match="q_mask must be"):
        lik.maxsim(Q, torch.randn(2, 2, 4, 16, device="cuda"), q_mask=torch.ones(2, 5, dtype=torch.bool, device="cuda"))
    with pytest.raises(ValueError, match=r"\[B, L, d\]"):
        lik.maxsim_pairs(Q[0], D)
    with pytest.raises(ValueError, match="top_k must be positive"):
        lik.retrieve(Q, D, 0)


# ----------------------------------------------------------------------------- KD / pairs
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kd_and_pairs(dtype):
    g = load_golden("kd")
    Q, D, qm, dm = cases.kd_case(5)
    if dtype == torch.float32:
        s = L().maxsim(dev(Q), dev(D), dev(qm), dev(dm))
        assert s.shape == (4, 3) and O.rel_err(f32(s), g["scores"]) < 1e-5
    Q, D, qm, dm = cases.kd_case(6, Nq=8, K=5, Lq=32, Ld=70, d=128)
    want = O.maxsim_kd(rounded(Q, dtype), rounded(D, dtype), qm, dm, normalize=True)
    s = L().maxsim(dev(Q, dtype), dev(D, dtype), dev(qm), dev(dm), normalize=True)
    assert O.rel_err(f32(s), want) < TOL[dtype]
    p = L().maxsim_pairs(dev(Q, dtype), dev(D[:, 0], dtype), dev(qm), dev(dm[:, 0]), normalize=True)
    assert p.shape == (8,) and O.rel_err(f32(p), want[:, 0]) < TOL[dtype]


# ----------------------------------------------------------------------------- packed layouts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_varlen_pair_list_padded(dtype):
    from late_interaction_kernels_b200.padded import pack_padded
    from late_interaction_kernels_b200.score_pairs import score_pairs_packed

    if dtype == torch.float32:
        g = load_golden("varlen")
        Q, D, cu_q, cu_d = cases.varlen_case(6)
        s = L().maxsim_varlen(dev(Q), dev(D), dev(cu_q), dev(cu_d))
        assert O.rel_err(f32(s), g["scores"]) < 1e-5 and (s[:, 3] == 0).all()
        g = load_golden("pair_list")
        Q, D, cu_q, cu_d, pq, pd = cases.pair_list_case(7)
        s = score_pairs_packed(dev(Q), dev(D), dev(cu_q), dev(cu_d), dev(pq), dev(pd))
        assert O.rel_err(f32(s), g["scores"]) < 1e-5
        g = load_golden("padded")
        q, docs, ql, dl = cases.padded_case(8)
        s = L().maxsim_padded(dev(q), dev(docs), dev(ql), dev(dl))
        assert s.shape == (3, 4) and O.rel_err(f32(s), g["scores"]) < 1e-5
        pk = pack_padded(dev(q), dev(docs), dev(ql), dev(dl))
        Qp, cq, Dp, cd, pq_, pd_, mq, md = pk
        for a, k in ((Qp, "Q_packed"), (cq, "cu_q"), (Dp, "D_packed"), (cd, "cu_d"), (pq_, "pair_q"), (pd_, "pair_d")):
            assert np.array_equal(a.cpu().numpy(), g[k]), k
        assert (mq, md) == (int(g["max_q"]), int(g["max_d"]))
        s2 = score_pairs_packed(Qp, Dp, cq, cd, pq_, pd_, max_seqlen_q=mq, max_seqlen_d=md)
        assert O.rel_err(f32(s2).reshape(3, 4), g["scores"]) < 1e-5
    # ColPali-like ragged shapes
    Q, D, cu_q, cu_d = cases.varlen_case(16, Nq=9, Nd=7, lq=(16, 32), ld=(100, 330), d=128, normalized=True)
    want = O.maxsim_varlen(rounded(Q, dtype), rounded(D, dtype), cu_q, cu_d)
    s = L().maxsim_varlen(dev(Q, dtype), dev(D, dtype), dev(cu_q.astype(np.int64)), dev(cu_d.astype(np.int64)))
    assert O.rel_err(f32(s), want) < TOL[dtype]


def test_pair_index_out_of_range_is_reported_not_fatal():
    from late_interaction_kernels_b200.score_pairs import score_pairs_packed

    Q, D, cu_q, cu_d, pq, pd = cases.pair_list_case(7)
    pq = pq.copy()
    pq[0] = 99
    s = score_pairs_packed(dev(Q), dev(D), dev(cu_q), dev(cu_d), dev(pq), dev(pd))
    assert float(s[0]) == 0.0
    with pytest.raises(RuntimeError, match="pair index"):
        L().check_device_status()
    L().check_device_status()  # cleared


# ----------------------------------------------------------------------------- backward
def _grad_check(gq, gd, wq, wd, tol):
    assert O.rel_err(f32(gq), wq) < tol, f"grad_Q {O.rel_err(f32(gq), wq)}"
    assert O.rel_err(f32(gd), wd) < tol, f"grad_D {O.rel_err(f32(gd), wd)}"


@pytest.mark.parametrize("method", ["auto", "unified", "lowmem"])
@pytest.mark.parametrize("normalize", [False, True])
def test_backward_golden_fp32(method, normalize):
    g = load_golden("grads_norm" if normalize else "grads")
    Q, D, qm, dm = cases.random_mask_case(3, Nq=4, Nd=5, Lq=6, Ld=13, d=16)
    go = np.random.default_rng(33).standard_normal((4, 5))
    Qt, Dt = dev(Q).requires_grad_(), dev(D).requires_grad_()
    s = L().maxsim(Qt, Dt, dev(qm), dev(dm), normalize=normalize, backward=method)
    (s * dev(go, torch.float32)).sum().backward()
    _grad_check(Qt.grad, Dt.grad, g["gQ"], g["gD"], 1e-5)
    assert (Qt.grad[~dev(qm)] == 0).all() and (Dt.grad[~dev(dm)] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("method", ["unified", "lowmem"])
@pytest.mark.parametrize("shape", [(6, 7, 32, 50, 128), (3, 4, 9, 31, 48), (5, 3, 40, 20, 200)])
def test_backward_shapes(dtype, method, shape):
    Nq, Nd, Lq, Ld, d = shape
    Q, D, qm, dm = cases.dense_case(7 + sum(shape), Nq, Nd, Lq, Ld, d, q_len=(1, Lq), d_len=(1, Ld), normalized=True)
    go = np.random.default_rng(1).standard_normal((Nq, Nd)).astype(np.float32)
    wq, wd = O.maxsim_grads(go, rounded(Q, dtype), rounded(D, dtype), qm, dm)
    Qt, Dt = dev(Q, dtype).requires_grad_(), dev(D, dtype).requires_grad_()
    s = L().maxsim(Qt, Dt, dev(qm), dev(dm), backward=method)
    (s * dev(go)).sum().backward()
    assert Qt.grad.dtype == dtype and Dt.grad.dtype == dtype
    # bf16 winners can differ from the fp64 oracle on near-ties; gradients are compared at operand tolerance
    _grad_check(Qt.grad, Dt.grad, wq, wd, max(TOL[dtype], 1e-5) if dtype != torch.float32 else 1e-5)


def test_backward_given_argmax_and_determinism():
    from late_interaction_kernels_b200.backward import maxsim_backward_lowmem, maxsim_backward_unified

    g = load_golden("bwd_argmax")
    Q, D, qm, _ = cases.random_mask_case(4, Nq=3, Nd=4, Lq=5, Ld=8, d=8)
    rng = np.random.default_rng(44)
    am = rng.integers(0, 8, size=(12, 5)).astype(np.int32)
    go = rng.standard_normal((3, 4)).astype(np.float32)
    for fn in (maxsim_backward_unified, maxsim_backward_lowmem):
        gq, gd = fn(dev(go), dev(Q), dev(D), dev(am), dev(qm))
        _grad_check(gq, gd, g["gQ"], g["gD"], 1e-5)
    with pytest.raises(RuntimeError, match="CUDA"):
        maxsim_backward_lowmem(torch.tensor(go), torch.tensor(Q), torch.tensor(D), torch.tensor(am))
    # hot bucket: every winner on one token; -1 sentinel keeps a document's grad exactly zero
    Nq, Nd, Lq, Ld, d = 64, 3, 32, 40, 128
    rng = np.random.default_rng(2)
    Q = rng.standard_normal((Nq, Lq, d)).astype(np.float32)
    D = rng.standard_normal((Nd, Ld, d)).astype(np.float32)
    am = np.full((Nq, Nd, Lq), 7, np.int32)
    am[:, 1] = -1
    go = rng.standard_normal((Nq, Nd)).astype(np.float32)
    wq, wd = O.backward_from_argmax(go, rounded(Q, torch.bfloat16), rounded(D, torch.bfloat16), am)
    outs = [maxsim_backward_lowmem(dev(go), dev(Q, torch.bfloat16), dev(D, torch.bfloat16), dev(am.reshape(-1, Lq))) for _ in range(3)]
    _grad_check(outs[0][0], outs[0][1], wq, wd, 2e-2)
    assert (outs[0][1][1] == 0).all()
    for o in outs[1:]:
        assert torch.equal(o[0], outs[0][0]) and torch.equal(o[1], outs[0][1]), "lowmem must be bitwise deterministic"
    u = maxsim_backward_unified(dev(go), dev(Q, torch.bfloat16), dev(D, torch.bfloat16), dev(am.reshape(-1, Lq)))
    _grad_check(u[0], u[1], wq, wd, 2e-2)
    assert torch.equal(u[0], outs[0][0]), "grad_Q is row-owned in both methods"


@pytest.mark.parametrize("dtype,normalize", [(torch.bfloat16, False), (torch.bfloat16, True), (torch.float32, True)])
def test_backward_few_queries_many_documents(dtype, normalize):
    """grad_Q of a couple of queries against hundreds of documents: the documents of a query are split over several
    CTAs whose partial rows are summed in a fixed order (same result as the oracle, same bits every run)."""
    from late_interaction_kernels_b200 import _lib, _ops

    Nq, Nd, Lq, Ld, d = 2, 333, 20, 24, 64
    rng = np.random.default_rng(9)
    Q = rng.standard_normal((Nq, Lq, d)).astype(np.float32)
    D = rng.standard_normal((Nd, Ld, d)).astype(np.float32)
    am = rng.integers(-1, Ld, size=(Nq, Nd, Lq)).astype(np.int32)
    go = rng.standard_normal((Nq, Nd)).astype(np.float32)
    Qr, Dr = rounded(Q, dtype), rounded(D, dtype)
    if normalize:
        wq, wd = O.backward_from_argmax(go, O.l2_normalize(Qr), O.l2_normalize(Dr), am)
        wq, wd = O.normalize_jacobian(wq, Qr, eps=1e-12), O.normalize_jacobian(wd, Dr, eps=1e-12)
    else:
        wq, wd = O.backward_from_argmax(go, Qr, Dr, am)
    q, dd = _ops.padded_spec(dev(Q, dtype)), _ops.padded_spec(dev(D, dtype))
    outs = [_ops.backward(q, dd, dev(go), dev(am.reshape(-1, Lq)), normalize=_lib.NORM_BOTH if normalize else _lib.NORM_NONE,
                          grad_dtype=torch.float32) for _ in range(2)]
    _grad_check(outs[0][0].view(Nq, Lq, d), outs[0][1].view(Nd, Ld, d), wq, wd, 1e-4 if dtype == torch.float32 else 2e-2)
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_backward_kd_varlen_pairs_padded():
    from late_interaction_kernels_b200.score_pairs import score_pairs_packed

    g = load_golden("kd")
    Q, D, qm, dm = cases.kd_case(5)
    Qt, Dt = dev(Q).requires_grad_(), dev(D).requires_grad_()
    s = L().maxsim(Qt, Dt, dev(qm), dev(dm), normalize=True)
    (s * dev(g["g"], torch.float32)).sum().backward()
    _grad_check(Qt.grad, Dt.grad, g["gQ_norm"], g["gD_norm"], 1e-5)

    g = load_golden("varlen")
    Q, D, cu_q, cu_d = cases.varlen_case(6)
    Qt, Dt = dev(Q).requires_grad_(), dev(D).requires_grad_()
    s = L().maxsim_varlen(Qt, Dt, dev(cu_q), dev(cu_d))
    (s * dev(g["g"])).sum().backward()
    _grad_check(Qt.grad, Dt.grad, g["gQ"], g["gD"], 1e-5)

    g = load_golden("pair_list")
    Q, D, cu_q, cu_d, pq, pd = cases.pair_list_case(7)
    Qt, Dt = dev(Q).requires_grad_(), dev(D).requires_grad_()
    s = score_pairs_packed(Qt, Dt, dev(cu_q), dev(cu_d), dev(pq), dev(pd))
    (s * dev(g["g"])).sum().backward()
    _grad_check(Qt.grad, Dt.grad, g["gQ"], g["gD"], 1e-5)

    q, docs, ql, dl = cases.padded_case(8)
    Qp, cu_q, Dp, cu_d, pq, pd, _, _ = O.pack_padded(q, docs, ql, dl)
    go = np.random.default_rng(3).standard_normal((3, 4)).astype(np.float32)
    wq, wd = O.pair_list_grads(go.reshape(-1), Qp, Dp, cu_q, cu_d, pq, pd)
    qt, dt = dev(q).requires_grad_(), dev(docs).requires_grad_()
    s = L().maxsim_padded(qt, dt, dev(ql), dev(dl))
    (s * dev(go)).sum().backward()
    gq = np.concatenate([f32(qt.grad)[b, : ql[b]] for b in range(3)])
    gd = np.concatenate([f32(dt.grad).reshape(12, 13, 16)[k, : dl.reshape(-1)[k]] for k in range(12)])
    assert O.rel_err(gq, wq) < 1e-5 and O.rel_err(gd, wd) < 1e-5
    assert all((qt.grad[b, ql[b]:] == 0).all() for b in range(3)), "padding rows get exactly zero gradient"


# ----------------------------------------------------------------------------- FP8
@pytest.mark.parametrize("q_tok,d_tok", [(True, True), (False, False), (True, False), (False, True)])
def test_fp8_forward(q_tok, d_tok):
    from late_interaction_kernels_b200 import fp8

    g = load_golden("fp8")
    rng = np.random.default_rng(9)
    X = (rng.standard_normal((5, 7, 32)) * np.array([1e-3, 0.1, 1, 10, 300]).reshape(5, 1, 1)).astype(np.float32)
    X[0, 0] = 0.0
    xq, sc = fp8.quantize_fp8_per_token(dev(X))
    # the helpers are torch ops; CUDA and CPU division can differ in the last ulp of the scale
    np.testing.assert_allclose(f32(sc), g["s_tok"], rtol=3e-7)
    assert (f32(xq) != g["q_tok"]).mean() < 1e-3
    xq2, sc2 = fp8.quantize_fp8_per_tensor(dev(X))
    np.testing.assert_allclose(f32(sc2), g["s_ten"], rtol=3e-7)
    assert (f32(xq2) != g["q_ten"]).mean() < 1e-3

    Q, D, qm, dm = cases.dense_case(21, 5, 9, 32, 70, 128, q_len=(4, 32), d_len=(5, 70), normalized=True)
    qf = (fp8.quantize_fp8_per_token if q_tok else fp8.quantize_fp8_per_tensor)(dev(Q))
    df = (fp8.quantize_fp8_per_token if d_tok else fp8.quantize_fp8_per_tensor)(dev(D))
    s = fp8.maxsim_inference_fp8(qf[0], df[0], scale_Q=qf[1], scale_D=df[1], q_mask=dev(qm), d_mask=dev(dm))
    exact = O.maxsim(Q, D, qm, dm)
    assert O.rel_err(f32(s), exact) < 6e-2
    # against the oracle on the dequantised values the kernel is exact to fp32 rounding
    deq = O.maxsim_fp8(f32(qf[0]), f32(df[0]), f32(qf[1]), f32(df[1]), qm, dm)
    assert O.rel_err(f32(s), deq) < 1e-4


def test_fp8_kd_layout():
    from late_interaction_kernels_b200 import fp8

    Q, D, qm, dm = cases.kd_case(31, Nq=6, K=4, Lq=32, Ld=90, d=128)
    Q, D = cases.unit(Q), cases.unit(D)
    qf = fp8.quantize_fp8_per_token(dev(Q))
    df = fp8.quantize_fp8_per_token(dev(D))
    s = fp8.maxsim_inference_fp8(qf[0], df[0], scale_Q=qf[1], scale_D=df[1], q_mask=dev(qm), d_mask=dev(dm))
    assert s.shape == (6, 4)
    assert O.rel_err(f32(s), O.maxsim_kd(Q, D, qm, dm)) < 6e-2


# ----------------------------------------------------------------------------- retrieve / top-k
def test_retrieve_matches_reference_and_chunking_is_exact():
    g = load_golden("retrieve")
    Q, D, dm = cases.retrieve_case(10)
    lik = L()
    cfg = {"full": dict(top_k=5), "chunk4": dict(top_k=10, chunk=4), "chunk8_k50": dict(top_k=50, chunk=8),
           "nonorm": dict(top_k=7, chunk=16, normalize=False), "smallest": dict(top_k=6, chunk=5, largest=False)}
    for tag, kw in cfg.items():
        s, i = lik.retrieve(dev(Q), dev(D), d_mask=dev(dm), **kw)
        assert i.dtype == torch.int64 and s.dtype == torch.float32
        assert np.array_equal(i.cpu().numpy(), g[f"{tag}_i"]), tag
        assert O.rel_err(f32(s), g[f"{tag}_s"]) < 1e-5
    s1, i1 = lik.retrieve(dev(Q[0]), dev(D), 3, d_mask=dev(dm))
    assert s1.shape == (3,) and i1.shape == (3,)
    # bigger: chunked == unchunked exactly, == maxsim + torch.topk
    Q, D, _, dm = cases.dense_case(3, 16, 700, 32, 48, 128, d_len=(1, 48), normalized=True)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    full = lik.maxsim(Qb, Db, None, dev(dm), normalize=True)
    ts, ti = torch.topk(full, 100, dim=-1)
    for chunk in (None, 64, 333):
        s, i = lik.retrieve(Qb, Db, 100, d_mask=dev(dm), chunk=chunk)
        assert torch.equal(i, ti) and torch.equal(s, ts), chunk
    sc = lik.MaxSimScorer()
    assert torch.equal(sc(Qb, Db, d_mask=dev(dm)), full) and torch.equal(sc.score(Qb, Db, d_mask=dev(dm)), full)
    assert "normalize=True" in repr(sc)


def test_topk_merge_c_abi():
    from late_interaction_kernels_b200 import _ops

    rng = np.random.default_rng(0)
    s = rng.standard_normal((3, 5, 16)).astype(np.float32)  # [lists, rows, k]
    idx = rng.permutation(3 * 5 * 16).reshape(3, 5, 16).astype(np.int64)
    idx[2, :, 10:] = -1
    s[2, :, 10:] = -np.inf
    ws, wi = O.merge_topk(np.moveaxis(s, 0, 1).reshape(5, -1), np.moveaxis(idx, 0, 1).reshape(5, -1), 16)
    gs, gi = _ops.topk_merge(dev(s), dev(idx), 16)
    assert np.array_equal(gi.cpu().numpy(), wi) and np.array_equal(f32(gs), ws)


# ----------------------------------------------------------------------------- PLAID
@pytest.mark.parametrize("nbits", [2, 4, 8])
def test_plaid(nbits):
    from late_interaction_kernels_b200 import plaid

    g = load_golden(f"plaid_nbits{nbits}")
    Q, codes, res, lens, cent, bw, _ = cases.plaid_case(11 + nbits, nbits=nbits)
    args = (dev(codes), dev(res), dev(lens), dev(cent), dev(bw), nbits)
    for norm in (True, False):
        s = plaid.maxsim_residual(dev(Q), *args, normalize=norm)
        assert O.rel_err(f32(s), g[f"scores_norm{int(norm)}"]) < (3e-2 if norm else 2e-2)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cf = np.concatenate([codes[j, : lens[j]] for j in range(len(lens))])
    rf = np.concatenate([res[j, : lens[j]] for j in range(len(lens))])
    sv = plaid.maxsim_residual_varlen(dev(Q), dev(cf), dev(rf), dev(cu), dev(cent), dev(bw), nbits)
    assert O.rel_err(f32(sv), f32(plaid.maxsim_residual(dev(Q), *args))) < 1e-4
    assert plaid.maxsim_residual(dev(Q[0]), *args).shape == (5,)
    Qt = dev(Q).requires_grad_()
    s = plaid.maxsim_residual(Qt, *args)
    (s * dev(g["g"], torch.float32)).sum().backward()
    assert O.rel_err(f32(Qt.grad), g["gQ"]) < 3e-2
    with pytest.raises(ValueError, match="zero-length document"):
        plaid.maxsim_residual(dev(Q).requires_grad_(), dev(codes), dev(res), dev(lens * 0), dev(cent), dev(bw), nbits)
    assert (plaid.maxsim_residual(dev(Q), dev(codes), dev(res), dev(lens * 0), dev(cent), dev(bw), nbits) == 0).all()
    assert plaid.maxsim_residual_varlen(dev(Q), dev(cf[:0]), dev(rf[:0]), dev(cu[:1]), dev(cent), dev(bw), nbits).shape == (3, 0)


def test_plaid_approx():
    from late_interaction_kernels_b200 import plaid

    g = load_golden("plaid_approx")
    rng = np.random.default_rng(12)
    qcs = rng.standard_normal((40, 6)).astype(np.float32)
    codes = rng.integers(-2, 44, size=(7, 11)).astype(np.int32)
    lens = np.array([0, 1, 11, 5, 7, 3, 11], dtype=np.int64)
    s = plaid.plaid_approx_score(dev(qcs), dev(codes), dev(lens))
    assert O.rel_err(f32(s), g["scores"]) < 1e-6 and float(s[0]) == 0.0


# ----------------------------------------------------------------------------- robustness
def test_cuda_graph_capture_and_inference_mode():
    Q, D, _, dm = cases.dense_case(9, 8, 24, 32, 60, 128, d_len=(1, 60), normalized=True)
    Qb, Db, dmb = dev(Q, torch.bfloat16), dev(D, torch.bfloat16), dev(dm)
    lik = L()
    eager = lik.maxsim(Qb, Db, None, dmb)
    with torch.inference_mode():
        assert torch.equal(lik.maxsim(Qb, Db, None, dmb), eager)
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        lik.maxsim(Qb, Db, None, dmb)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(graph):
        out = lik.maxsim(Qb, Db, None, dmb)
    Qb.copy_(dev(Q[::-1].copy(), torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, lik.maxsim(Qb, Db, None, dmb))
