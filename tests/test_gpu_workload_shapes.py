"""GPU parity at the full benchmark workload shapes.

The oracle cannot score these shapes whole in test time, so every test runs the CUDA path on the FULL
shape and compares a sampled block with the oracle: scores of sampled (query, document) blocks, winners
on integer-valued data (exact arithmetic, compared with ``==``), and gradients through an upstream
gradient that is zero outside the sampled block — then the full-size kernels still process every entry,
the sampled rows must match the oracle on the sub-batch and every other row must be exactly zero.
Tolerances: bf16 2e-2, e4m3 6e-2 relative (max|a-b| / max|b|), integers exact.
"""

import numpy as np
import pytest
import torch

import cases
from oracle import maxsim_oracle as O

pytestmark = pytest.mark.gpu


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def f32(t):
    return t.detach().float().cpu().numpy()


# ----------------------------------------------------------------------------- packed ColPali shape
def _colpali_packed(seed, integer=False):
    """128 queries of U[16,32] tokens, 128 documents of U[900,1030] tokens, d = 128, packed."""
    rng = np.random.default_rng(seed)
    ql = rng.integers(16, 33, size=128)
    dl = rng.integers(900, 1031, size=128)
    if integer:
        Q = rng.integers(-2, 3, size=(int(ql.sum()), 128)).astype(np.float32)
        D = rng.integers(-2, 3, size=(int(dl.sum()), 128)).astype(np.float32)
    else:
        Q = cases.unit(rng.standard_normal((int(ql.sum()), 128))).astype(np.float32)
        D = cases.unit(rng.standard_normal((int(dl.sum()), 128))).astype(np.float32)
    cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    cu_d = np.concatenate([[0], np.cumsum(dl)]).astype(np.int32)
    return Q, D, cu_q, cu_d


def _sub_packed(X, cu, idx):
    """Rows of the sequences `idx` of a packed matrix, re-packed, with their offsets."""
    parts = [X[cu[i]:cu[i + 1]] for i in idx]
    lens = [p.shape[0] for p in parts]
    return np.concatenate(parts), np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)


def test_colpali_packed_forward_and_winners():
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200.varlen import _varlen_forward

    Q, D, cu_q, cu_d = _colpali_packed(41)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    s = lik.maxsim_varlen(Qb, Db, dev(cu_q), dev(cu_d), 32, 1030)
    assert s.shape == (128, 128)
    qi, dj = [0, 1, 17, 63, 64, 100, 126, 127], [0, 5, 31, 32, 77, 90, 126, 127]
    Qs, cqs = _sub_packed(f32(Qb), cu_q, qi)
    Ds, cds = _sub_packed(f32(Db), cu_d, dj)
    want = O.maxsim_varlen(Qs, Ds, cqs, cds)
    assert O.rel_err(f32(s)[np.ix_(qi, dj)], want) < 2e-2
    # the call that derives the maxima itself gives the same bits
    assert torch.equal(lik.maxsim_varlen(Qb, Db, dev(cu_q), dev(cu_d)), s)

    # integer-valued data: scores and winners are exact, so they are compared with ==
    Q, D, cu_q, cu_d = _colpali_packed(42, integer=True)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    s, am, _, _ = _varlen_forward(Qb, Db, dev(cu_q), dev(cu_d), 32, 1030, True)
    Qs, cqs = _sub_packed(Q, cu_q, qi)
    Ds, cds = _sub_packed(D, cu_d, dj)
    want, want_am = O.maxsim_varlen(Qs, Ds, cqs, cds, return_argmax=True)
    assert np.array_equal(f32(s)[np.ix_(qi, dj)], want)
    got_am = am.cpu().numpy()[np.ix_(qi, dj)]
    assert got_am.shape[-1] == 32
    assert np.array_equal(got_am[..., :want_am.shape[-1]], want_am)
    assert (got_am[..., want_am.shape[-1]:] == -1).all()


def test_colpali_packed_backward_sampled_block():
    """bf16 packed backward (query-tile packing -> forward with argmax -> sorted grad_D / gathered grad_Q on
    packed rows) against the oracle's packed gradients."""
    import late_interaction_kernels_b200 as lik

    Q, D, cu_q, cu_d = _colpali_packed(43)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    qi, dj = [3, 4, 40, 41, 64, 99, 120, 127], [0, 9, 10, 50, 64, 65, 101, 127]
    rng = np.random.default_rng(5)
    g_blk = rng.standard_normal((8, 8)).astype(np.float32)
    g = np.zeros((128, 128), np.float32)
    g[np.ix_(qi, dj)] = g_blk
    Qt, Dt = Qb.clone().requires_grad_(), Db.clone().requires_grad_()
    out = lik.maxsim_varlen(Qt, Dt, dev(cu_q), dev(cu_d), 32, 1030)
    out.backward(dev(g))
    lik.check_device_status()
    Qs, cqs = _sub_packed(f32(Qb), cu_q, qi)
    Ds, cds = _sub_packed(f32(Db), cu_d, dj)
    wq, wd = O.varlen_grads(g_blk, Qs, Ds, cqs, cds)
    gq, gd = f32(Qt.grad), f32(Dt.grad)
    got_q, _ = _sub_packed(gq, cu_q, qi)
    got_d, _ = _sub_packed(gd, cu_d, dj)
    assert O.rel_err(got_q, wq) < 2e-2
    assert O.rel_err(got_d, wd) < 2e-2
    # every row outside the sampled block has a zero upstream gradient: exactly zero
    mq = np.ones(gq.shape[0], bool)
    for i in qi:
        mq[cu_q[i]:cu_q[i + 1]] = False
    md = np.ones(gd.shape[0], bool)
    for j in dj:
        md[cu_d[j]:cu_d[j + 1]] = False
    assert (gq[mq] == 0).all() and (gd[md] == 0).all()
    # bitwise reproducible
    Qt2, Dt2 = Qb.clone().requires_grad_(), Db.clone().requires_grad_()
    lik.maxsim_varlen(Qt2, Dt2, dev(cu_q), dev(cu_d), 32, 1030).backward(dev(g))
    assert torch.equal(Qt2.grad, Qt.grad) and torch.equal(Dt2.grad, Dt.grad)


# ----------------------------------------------------------------------------- KD shape
def _kd_full(seed):
    rng = np.random.default_rng(seed)
    Q = cases.unit(rng.standard_normal((64, 32, 128))).astype(np.float32)
    D = cases.unit(rng.standard_normal((64, 32, 300, 128))).astype(np.float32)
    lens = rng.integers(64, 301, size=(64, 32))
    dm = cases.prefix_mask(lens, 300)
    return Q, D, dm


def test_kd_full_shape_bf16_scores_and_gradients():
    import late_interaction_kernels_b200 as lik

    Q, D, dm = _kd_full(51)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    Qt, Dt = Qb.clone().requires_grad_(), Db.clone().requires_grad_()
    s = lik.maxsim(Qt, Dt, d_mask=dev(dm))
    assert s.shape == (64, 32)
    want = O.maxsim_kd(f32(Qb), f32(Db), None, dm)
    assert O.rel_err(f32(s), want) < 2e-2
    g = np.random.default_rng(6).standard_normal((64, 32)).astype(np.float32)
    s.backward(dev(g))
    wq, wd = O.maxsim_grads(g, f32(Qb), f32(Db), None, dm, kd_layout=True)
    assert O.rel_err(f32(Qt.grad), wq) < 2e-2
    assert O.rel_err(f32(Dt.grad), np.asarray(wd).reshape(64, 32, 300, 128)) < 2e-2
    assert (Dt.grad[~dev(dm)] == 0).all()


def test_kd_full_shape_e4m3_scores():
    from late_interaction_kernels_b200 import fp8

    Q, D, dm = _kd_full(52)
    qf = fp8.quantize_fp8_per_token(dev(Q))
    df = fp8.quantize_fp8_per_token(dev(D))
    s = fp8.maxsim_inference_fp8(qf[0], df[0], scale_Q=qf[1], scale_D=df[1], d_mask=dev(dm))
    assert s.shape == (64, 32)
    assert O.rel_err(f32(s), O.maxsim_kd(Q, D, None, dm)) < 6e-2
    # on the dequantised values the kernel is exact up to fp32 summation order
    deq_q = O.dequantize_fp8(f32(qf[0]), f32(qf[1]))
    deq_d = O.dequantize_fp8(f32(df[0]), f32(df[1]))
    assert O.rel_err(f32(s), O.maxsim_kd(deq_q, deq_d, None, dm)) < 1e-4


# ----------------------------------------------------------------------------- in-batch training shape
def test_inbatch_full_shape_grad_d_against_oracle():
    """Q[512,32,128] x D[512,300,128] bf16: grad_D of every document from an upstream gradient that is non-zero on
    eight queries only, against the oracle on those eight queries; grad_Q of the other 504 queries exactly zero."""
    import late_interaction_kernels_b200 as lik

    rng = np.random.default_rng(61)
    Q = cases.unit(rng.standard_normal((512, 32, 128))).astype(np.float32)
    D = cases.unit(rng.standard_normal((512, 300, 128))).astype(np.float32)
    dm = cases.prefix_mask(rng.integers(64, 301, size=512), 300)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    qi = [0, 1, 130, 131, 255, 256, 400, 511]
    g = np.zeros((512, 512), np.float32)
    g[qi] = rng.standard_normal((8, 512)).astype(np.float32)
    for method in ("lowmem", "unified"):
        Qt, Dt = Qb.clone().requires_grad_(), Db.clone().requires_grad_()
        lik.maxsim(Qt, Dt, d_mask=dev(dm), backward=method).backward(dev(g))
        wq, wd = O.maxsim_grads(g[qi], f32(Qb)[qi], f32(Db), None, dm)
        assert O.rel_err(f32(Dt.grad), wd) < 2e-2, method
        assert O.rel_err(f32(Qt.grad)[qi], wq) < 2e-2, method
        rest = np.setdiff1d(np.arange(512), qi)
        assert (Qt.grad[dev(rest)] == 0).all(), method
        assert (Dt.grad[~dev(dm)] == 0).all(), method


# ----------------------------------------------------------------------------- exact winners in 16-bit types
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(3, 5, 7, 19, 16), (4, 6, 32, 300, 128), (2, 3, 33, 65, 96), (8, 8, 32, 64, 128),
                                   (2, 2, 130, 257, 64), (1, 9, 128, 40, 128),
                                   (3, 6, 32, 5000, 128), (2, 5, 128, 2300, 64)])  # long documents: the lazy winner scan
def test_dense_winners_exact_on_integer_data(dtype, shape):
    from late_interaction_kernels_b200.forward import maxsim_forward

    Nq, Nd, Lq, Ld, d = shape
    rng = np.random.default_rng(sum(shape))
    Q = rng.integers(-2, 3, size=(Nq, Lq, d)).astype(np.float32)
    D = rng.integers(-2, 3, size=(Nd, Ld, d)).astype(np.float32)
    qm = cases.prefix_mask(rng.integers(1, Lq + 1, size=Nq), Lq)
    dm = cases.prefix_mask(rng.integers(1, Ld + 1, size=Nd), Ld)
    want, want_am = O.maxsim(Q, D, qm, dm, return_argmax=True)
    s, am = maxsim_forward(dev(Q, dtype), dev(D, dtype), dev(qm), dev(dm), save_argmax=True)
    assert np.array_equal(f32(s), want)
    got = am.cpu().numpy().reshape(Nq, Nd, Lq)
    sel = np.broadcast_to(qm[:, None, :], got.shape)
    assert np.array_equal(got[sel], want_am[sel])


# ----------------------------------------------------------------------------- empty queries, stale winners
def test_empty_queries_score_zero_on_the_tensor_core_path():
    import late_interaction_kernels_b200 as lik

    rng = np.random.default_rng(71)
    q = cases.unit(rng.standard_normal((3, 32, 128))).astype(np.float32)
    docs = cases.unit(rng.standard_normal((3, 4, 50, 128))).astype(np.float32)
    ql = np.array([32, 0, 7], np.int64)
    dl = rng.integers(1, 51, size=(3, 4)).astype(np.int64)
    for dtype in (torch.bfloat16, torch.float16):
        s = lik.maxsim_padded(dev(q, dtype), dev(docs, dtype), dev(ql), dev(dl))
        want = O.maxsim_padded(f32(dev(q, dtype)), f32(dev(docs, dtype)), ql, dl)
        assert (s[1] == 0).all(), "a zero-length query scores exactly 0 against every candidate"
        assert O.rel_err(f32(s), want) < 2e-2
    # packed: an empty query between 32-token queries (every tile stays warp-aligned)
    cu_q = np.array([0, 32, 32, 64, 96], np.int32)
    Q = cases.unit(rng.standard_normal((96, 128))).astype(np.float32)
    dlen = rng.integers(1, 80, size=5)
    cu_d = np.concatenate([[0], np.cumsum(dlen)]).astype(np.int32)
    Dp = cases.unit(rng.standard_normal((int(dlen.sum()), 128))).astype(np.float32)
    Qb, Db = dev(Q, torch.bfloat16), dev(Dp, torch.bfloat16)
    s = lik.maxsim_varlen(Qb, Db, dev(cu_q), dev(cu_d))
    assert (s[1] == 0).all()
    assert O.rel_err(f32(s), O.maxsim_varlen(f32(Qb), f32(Db), cu_q, cu_d)) < 2e-2
    Qt = Qb.clone().requires_grad_()
    lik.maxsim_varlen(Qt, Db, dev(cu_q), dev(cu_d)).sum().backward()
    assert torch.isfinite(Qt.grad).all()


def test_out_of_range_saved_winner_contributes_nothing():
    """The backward takes the winner table from the caller: an entry beyond its document must be skipped by
    every kernel (no fault, no contribution)."""
    from late_interaction_kernels_b200 import _ops
    from late_interaction_kernels_b200.backward import maxsim_backward_lowmem, maxsim_backward_unified

    rng = np.random.default_rng(81)
    Q = dev(cases.unit(rng.standard_normal((6, 32, 128))).astype(np.float32), torch.bfloat16)
    D = dev(cases.unit(rng.standard_normal((9, 40, 128))).astype(np.float32), torch.bfloat16)
    dm = dev(cases.prefix_mask(rng.integers(5, 41, size=9), 40))
    g = dev(rng.standard_normal((6, 9)).astype(np.float32))
    _, am = _ops.forward(_ops.padded_spec(Q), _ops.padded_spec(D, dm), save_argmax=True)
    for fn in (maxsim_backward_lowmem, maxsim_backward_unified):
        gq0, gd0 = fn(g, Q, D, am)
        bad = am.clone()
        bad[5, 3] = 1 << 20       # far outside every document
        bad[17, 0] = 40           # one past the padded length
        gq1, gd1 = fn(g, Q, D, bad)
        good = am.clone()
        good[5, 3] = -1           # what "contributes nothing" means: the same as no winner
        good[17, 0] = -1
        gq2, gd2 = fn(g, Q, D, good)
        assert torch.isfinite(gq1.float()).all() and torch.isfinite(gd1.float()).all()
        if fn is maxsim_backward_lowmem:
            assert torch.equal(gq1, gq2) and torch.equal(gd1, gd2)
        else:
            assert torch.allclose(gq1.float(), gq2.float(), atol=1e-3) and torch.allclose(gd1.float(), gd2.float(), atol=1e-3)
