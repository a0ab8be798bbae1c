"""Pins the CPU oracle to outputs of the reference implementation itself.

``tests/golden/*.npz`` were written by ``tests/golden/make_golden.py`` running the
reference's own CPU code on the seeded inputs of ``tests/golden/cases.py``.
"""

import numpy as np
import pytest
from conftest import load_golden

import cases
from oracle import maxsim_oracle as O


def _chk(g, *arrays):
    assert float(g["chk"]) == pytest.approx(cases.checksum(*arrays), rel=1e-12), "input generator drifted"


def test_config1_matches_reference():
    g = load_golden("config1")
    Q, D, qm, dm = cases.config1()
    _chk(g, Q, D, qm, dm)
    np.testing.assert_allclose(O.maxsim(Q, D, qm, dm, normalize=True), g["scores"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.maxsim(Q, D, qm, dm), g["scores_nonorm"], rtol=1e-5, atol=1e-4)


def test_random_masks_and_squeeze():
    g = load_golden("random_mask")
    Q, D, qm, dm = cases.random_mask_case(1)
    _chk(g, Q, D, qm, dm)
    np.testing.assert_allclose(O.maxsim(Q, D, qm, dm), g["scores"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.maxsim(Q, D, qm, dm, normalize=True), g["scores_norm"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.maxsim(Q, D), g["scores_nomask"], rtol=1e-5, atol=1e-5)
    s2 = O.maxsim(Q[0], D[0], qm[0], dm[0])
    assert s2.shape == () and g["scores_2d"].shape == ()
    np.testing.assert_allclose(s2, g["scores_2d"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.maxsim(Q[0], D), g["scores_q2d"], rtol=1e-5, atol=1e-5)
    # fully masked doc / query contribute exactly zero
    s = O.maxsim(Q, D, qm, dm)
    assert (s[:, 1] == 0).all() and (s[2] == 0).all()


def test_fp64_preserved():
    g = load_golden("dense_fp64")
    Q, D, _, dm = cases.dense_case(2, 6, 7, 9, 21, 24, d_len=(3, 21))
    _chk(g, Q, D, dm)
    s = O.maxsim(Q.astype(np.float64), D.astype(np.float64), None, dm)
    assert s.dtype == np.float64
    np.testing.assert_allclose(s, g["scores"], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("name,norm", [("grads", False), ("grads_norm", True)])
def test_grads_match_autograd(name, norm):
    g = load_golden(name)
    Q, D, qm, dm = cases.random_mask_case(3, Nq=4, Nd=5, Lq=6, Ld=13, d=16)
    go = np.random.default_rng(33).standard_normal((4, 5))
    _chk(g, Q, D, qm, dm, go)
    gQ, gD = O.maxsim_grads(go, Q, D, qm, dm, normalize=norm)
    np.testing.assert_allclose(gQ, g["gQ"], rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(gD, g["gD"], rtol=1e-9, atol=1e-9)
    # masked query tokens / masked doc tokens get exactly zero gradient
    assert (gQ[~qm] == 0).all() and (gD[~dm] == 0).all()


def test_backward_from_argmax():
    g = load_golden("bwd_argmax")
    Q, D, qm, _ = cases.random_mask_case(4, Nq=3, Nd=4, Lq=5, Ld=8, d=8)
    rng = np.random.default_rng(44)
    am = rng.integers(0, 8, size=(12, 5)).astype(np.int32)
    go = rng.standard_normal((3, 4)).astype(np.float32)
    _chk(g, Q, D, qm, am, go)
    gQ, gD = O.backward_from_argmax(go, Q, D, am, qm)
    np.testing.assert_allclose(gQ, g["gQ"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(gD, g["gD"], rtol=1e-5, atol=1e-5)


def test_kd_layout():
    g = load_golden("kd")
    Q, D, qm, dm = cases.kd_case(5)
    _chk(g, Q, D, qm, dm)
    np.testing.assert_allclose(O.maxsim_kd(Q, D, qm, dm), g["scores"], rtol=1e-5, atol=1e-5)
    gQ, gD = O.maxsim_grads(g["g"], Q, D, qm, dm, normalize=True, kd_layout=True)
    np.testing.assert_allclose(gQ, g["gQ_norm"], rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(gD, g["gD_norm"], rtol=1e-9, atol=1e-9)
    # maxsim_pairs is the K=1 case
    np.testing.assert_allclose(O.maxsim_pairs(Q, D[:, 0], qm, dm[:, 0]), g["scores"][:, 0], rtol=1e-5, atol=1e-5)


def test_varlen_and_pair_list():
    g = load_golden("varlen")
    Q, D, cu_q, cu_d = cases.varlen_case(6)
    _chk(g, Q, D, cu_q, cu_d)
    s, am = O.maxsim_varlen(Q, D, cu_q, cu_d, return_argmax=True)
    np.testing.assert_allclose(s, g["scores"], rtol=1e-5, atol=1e-5)
    assert (s[:, (len(cu_d) - 1) // 2] == 0).all(), "empty doc scores 0"
    assert (am[:, (len(cu_d) - 1) // 2] == -1).all()
    gQ, gD = O.varlen_grads(g["g"], Q, D, cu_q, cu_d)
    np.testing.assert_allclose(gQ, g["gQ"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(gD, g["gD"], rtol=1e-5, atol=1e-5)

    g = load_golden("pair_list")
    Q, D, cu_q, cu_d, pq, pd = cases.pair_list_case(7)
    _chk(g, Q, D, cu_q, cu_d, pq, pd)
    np.testing.assert_allclose(O.maxsim_pair_list(Q, D, cu_q, cu_d, pq, pd), g["scores"], rtol=1e-5, atol=1e-5)
    gQ, gD = O.pair_list_grads(g["g"], Q, D, cu_q, cu_d, pq, pd)
    np.testing.assert_allclose(gQ, g["gQ"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(gD, g["gD"], rtol=1e-5, atol=1e-5)


def test_padded_and_pack():
    g = load_golden("padded")
    q, docs, ql, dl = cases.padded_case(8)
    _chk(g, q, docs, ql, dl)
    np.testing.assert_allclose(O.maxsim_padded(q, docs, ql, dl), g["scores"], rtol=1e-5, atol=1e-5)
    Qp, cu_q, Dp, cu_d, pq, pd, mq, md = O.pack_padded(q, docs, ql, dl)
    for a, k in ((Qp, "Q_packed"), (cu_q, "cu_q"), (Dp, "D_packed"), (cu_d, "cu_d"), (pq, "pair_q"), (pd, "pair_d")):
        assert np.array_equal(a, g[k]), k
    assert mq == int(g["max_q"]) and md == int(g["max_d"])
    # padded == pair list on the packed form
    np.testing.assert_allclose(
        O.maxsim_pair_list(Qp, Dp, cu_q, cu_d, pq, pd).reshape(g["scores"].shape), g["scores"], rtol=1e-6, atol=1e-6
    )


def test_fp8_quantisers_bit_exact():
    g = load_golden("fp8")
    rng = np.random.default_rng(9)
    X = (rng.standard_normal((5, 7, 32)) * np.array([1e-3, 0.1, 1, 10, 300]).reshape(5, 1, 1)).astype(np.float32)
    X[0, 0] = 0.0
    _chk(g, X)
    grid = np.linspace(-460, 460, 20001).astype(np.float32)
    assert np.array_equal(O.round_to_e4m3(np.clip(grid, -448, 448)), g["grid_q"])
    q, s = O.quantize_fp8_per_token(X)
    assert np.array_equal(s, g["s_tok"]) and np.array_equal(q, g["q_tok"])
    q2, s2 = O.quantize_fp8_per_tensor(X)
    assert np.array_equal(s2, g["s_ten"]) and np.array_equal(q2, g["q_ten"])
    assert np.array_equal(O.dequantize_fp8(q, s), g["deq_tok"])


def test_retrieve_matches_reference_cpu_loop():
    g = load_golden("retrieve")
    Q, D, dm = cases.retrieve_case(10)
    _chk(g, Q, D, dm)
    cfg = {
        "full": dict(top_k=5), "chunk4": dict(top_k=10, chunk=4), "chunk8_k50": dict(top_k=50, chunk=8),
        "nonorm": dict(top_k=7, chunk=16, normalize=False), "smallest": dict(top_k=6, chunk=5, largest=False),
    }
    for tag, kw in cfg.items():
        s, i = O.retrieve(Q, D, d_mask=dm, **kw)
        assert np.array_equal(i, g[f"{tag}_i"]), tag
        np.testing.assert_allclose(s, g[f"{tag}_s"], rtol=1e-5, atol=1e-5)
    assert O.retrieve(Q, D, 50, d_mask=dm)[1].shape == (4, 37), "k clamps to Nd"
    with pytest.raises(ValueError):
        O.retrieve(Q, D, 0)


@pytest.mark.parametrize("nbits", [2, 4, 8])
def test_plaid(nbits):
    g = load_golden(f"plaid_nbits{nbits}")
    Q, codes, res, lens, cent, bw, _ = cases.plaid_case(11 + nbits, nbits=nbits)
    _chk(g, Q, codes, res, lens, cent, bw)
    d = Q.shape[-1]
    assert np.array_equal(O.unpack_residuals(res, nbits, d), g["unpacked"])
    assert np.array_equal(O.pack_residuals(g["unpacked"], nbits), res)
    for norm in (True, False):
        s = O.maxsim_residual(Q, codes, res, lens, cent, bw, nbits, normalize=norm)
        np.testing.assert_allclose(s, g[f"scores_norm{int(norm)}"], rtol=1e-5, atol=1e-5)
    # ragged form on the concatenated valid tokens gives the same scores
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cf = np.concatenate([codes[j, : lens[j]] for j in range(len(lens))])
    rf = np.concatenate([res[j, : lens[j]] for j in range(len(lens))])
    np.testing.assert_allclose(
        O.maxsim_residual_varlen(Q, cf, rf, cu, cent, bw, nbits), g["scores_norm1"], rtol=1e-5, atol=1e-5
    )
    gQ = O.residual_grad_q(g["g"], Q, codes, res, lens, cent, bw, nbits)
    np.testing.assert_allclose(gQ, g["gQ"], rtol=1e-5, atol=1e-6)


def test_plaid_approx():
    g = load_golden("plaid_approx")
    rng = np.random.default_rng(12)
    qcs = rng.standard_normal((40, 6)).astype(np.float32)
    codes = rng.integers(-2, 44, size=(7, 11)).astype(np.int32)
    lens = np.array([0, 1, 11, 5, 7, 3, 11], dtype=np.int64)
    _chk(g, qcs, codes, lens)
    s = O.plaid_approx_score(qcs, codes, lens)
    np.testing.assert_allclose(s, g["scores"], rtol=1e-6, atol=1e-6)
    assert s[0] == 0


def test_merge_topk_orders_by_score_then_index():
    s = np.array([[1.0, 3.0, 3.0, -np.inf, 2.0, 9.0]], np.float32)
    i = np.array([[7, 5, 2, -1, 9, -1]], np.int64)
    ms, mi = O.merge_topk(s, i, 3)
    assert mi.tolist() == [[2, 5, 9]] and ms.tolist() == [[3.0, 3.0, 2.0]]


def test_document_head_matches_reference():
    g = load_golden("from_hidden")
    Q, H, W, b, dm = cases.from_hidden_case(13)
    _chk(g, Q, H, W, b, dm)
    assert O.rel_err(O.maxsim_from_hidden(Q, H, W, b, dm), g["scores_norm1"]) < 1e-5
    assert O.rel_err(O.maxsim_from_hidden(Q, H, W, b, dm, normalize=False), g["scores_norm0"]) < 1e-5
    assert O.rel_err(O.maxsim_from_hidden(Q, H, W, None, dm), g["scores_nobias"]) < 1e-5
    gQ, gH, gW, gb = O.from_hidden_grads(g["g"], Q, H, W, b, dm)
    for got, want in ((gQ, g["gQ"]), (gH, g["gH"]), (gW, g["gW"]), (gb, g["gb"])):
        assert O.rel_err(got, want) < 1e-4
