"""Seeded random shapes through the public API against the CPU oracle: widths, lengths and masks that the hand-picked
cases do not line up (documents whose stride is or is not a multiple of four, one-token queries, queries longer than a
tile, masks with holes, fused normalisation), forward with winners and backward.

Integer-valued inputs make the arithmetic exact, so scores and winners are compared with ``==``; real-valued inputs use
the tolerances of the other parity tests (fp32 1e-5, 16-bit 2e-2 relative) and the kernel's own winners for the
gradients (an oracle working in fp64 may pick the other side of a near-tie)."""

import numpy as np
import pytest
import torch

import cases
from oracle import maxsim_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def dev(x, dtype=None):
    if x is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def f32(t):
    return t.detach().float().cpu().numpy()


def _mask(rng, n, length, kind):
    if kind == "none":
        return None
    if kind == "prefix":
        return cases.prefix_mask(rng.integers(1, length + 1, size=n), length)
    m = rng.random((n, length)) < 0.75
    m[rng.integers(0, n)] = False  # one sequence without a valid token
    m[:, 0] |= rng.random(n) < 0.5
    return m


def _shape(rng):
    return dict(
        Nq=int(rng.integers(1, 10)), Nd=int(rng.integers(1, 41)),
        Lq=int(rng.choice([1, 2, 7, 16, 31, 32, 33, 64, 100, 128, 140])),
        Ld=int(rng.choice([1, 3, 17, 64, 127, 128, 130, 255, 256, 257, 300, 513, 700])),
        d=int(rng.choice([16, 32, 64, 96, 128])),
        dtype=[torch.bfloat16, torch.float16, torch.float32][int(rng.integers(0, 3))],
        qk=str(rng.choice(["none", "prefix", "holes"])), dk=str(rng.choice(["none", "prefix", "holes"])),
    )


@pytest.mark.parametrize("seed", range(40))
def test_integer_data_scores_and_winners_exact(seed):
    from late_interaction_kernels_b200.forward import maxsim_forward

    rng = np.random.default_rng(1000 + seed)
    c = _shape(rng)
    Q = rng.integers(-2, 3, size=(c["Nq"], c["Lq"], c["d"])).astype(np.float32)
    D = rng.integers(-2, 3, size=(c["Nd"], c["Ld"], c["d"])).astype(np.float32)
    qm, dm = _mask(rng, c["Nq"], c["Lq"], c["qk"]), _mask(rng, c["Nd"], c["Ld"], c["dk"])
    want, want_am = O.maxsim(Q, D, qm, dm, return_argmax=True)
    s, am = maxsim_forward(dev(Q, c["dtype"]), dev(D, c["dtype"]), dev(qm), dev(dm), save_argmax=True)
    assert np.array_equal(f32(s), want), c
    got = am.cpu().numpy().reshape(c["Nq"], c["Nd"], c["Lq"])
    sel = np.ones(got.shape, bool) if qm is None else np.broadcast_to(qm[:, None, :], got.shape)
    assert np.array_equal(got[sel], want_am[sel]), c
    # without winners: the same scores, bit for bit
    s2, _ = maxsim_forward(dev(Q, c["dtype"]), dev(D, c["dtype"]), dev(qm), dev(dm), save_argmax=False)
    assert torch.equal(s, s2), c


@pytest.mark.parametrize("seed", range(30))
def test_real_data_forward_and_backward(seed):
    import late_interaction_kernels_b200 as lik

    rng = np.random.default_rng(2000 + seed)
    c = _shape(rng)
    normalize = bool(rng.integers(0, 2))
    dt = c["dtype"]
    Q = rng.standard_normal((c["Nq"], c["Lq"], c["d"])).astype(np.float32)
    D = rng.standard_normal((c["Nd"], c["Ld"], c["d"])).astype(np.float32)
    if not normalize:
        Q, D = cases.unit(Q).astype(np.float32), cases.unit(D).astype(np.float32)
    qm, dm = _mask(rng, c["Nq"], c["Lq"], c["qk"]), _mask(rng, c["Nd"], c["Ld"], c["dk"])
    tQ, tD = dev(Q, dt).requires_grad_(True), dev(D, dt).requires_grad_(True)
    Qr, Dr = f32(tQ), f32(tD)  # what the kernels see
    s = lik.maxsim(tQ, tD, dev(qm), dev(dm), normalize=normalize)
    want = O.maxsim(Qr, Dr, qm, dm, normalize=normalize)
    assert O.rel_err(f32(s), want) < TOL[dt], c
    g = rng.standard_normal(want.shape).astype(np.float32)
    (s * dev(g)).sum().backward()
    # gradients for the kernel's own winners
    from late_interaction_kernels_b200.forward import maxsim_forward
    _, am = maxsim_forward(tQ.detach(), tD.detach(), dev(qm), dev(dm), save_argmax=True, normalize=normalize)
    am = am.cpu().numpy().reshape(c["Nq"], c["Nd"], c["Lq"])
    Qh, Dh = (O.l2_normalize(Qr, 1e-12), O.l2_normalize(Dr, 1e-12)) if normalize else (Qr, Dr)
    wq, wd = O.backward_from_argmax(g, Qh, Dh, am, qm)
    if normalize:
        wq, wd = O.normalize_jacobian(wq, Qr, eps=1e-12), O.normalize_jacobian(wd, Dr, eps=1e-12)
    tol = 1e-4 if dt == torch.float32 else 2e-2
    assert O.rel_err(f32(tQ.grad), wq) < tol, c
    assert O.rel_err(f32(tD.grad), wd) < tol, c


@pytest.mark.parametrize("seed", range(16))
def test_candidate_lists_packed_and_retrieve_on_integer_data(seed):
    """The other layouts on exact arithmetic: per-query candidate lists (4-D documents), packed sequences with a pair
    list, and retrieve (indices exact, ties to the lower document)."""
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200.score_pairs import score_pairs_packed

    rng = np.random.default_rng(3000 + seed)
    dt = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    d = int(rng.choice([32, 64, 128]))
    # candidate lists
    Nq, K, Lq, Ld = int(rng.integers(1, 7)), int(rng.integers(1, 9)), int(rng.choice([1, 8, 32, 40])), int(rng.choice([5, 64, 257, 300]))
    Q = rng.integers(-2, 3, size=(Nq, Lq, d)).astype(np.float32)
    D = rng.integers(-2, 3, size=(Nq, K, Ld, d)).astype(np.float32)
    dm = cases.prefix_mask(rng.integers(1, Ld + 1, size=Nq * K), Ld).reshape(Nq, K, Ld)
    s = lik.maxsim(dev(Q, dt), dev(D, dt), d_mask=dev(dm))
    assert np.array_equal(f32(s), O.maxsim_kd(Q, D, None, dm))
    # packed sequences + pair list
    ql, dl = rng.integers(1, 34, size=5), rng.integers(1, 300, size=7)
    cu_q, cu_d = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32), np.concatenate([[0], np.cumsum(dl)]).astype(np.int32)
    Qp = rng.integers(-2, 3, size=(int(ql.sum()), d)).astype(np.float32)
    Dp = rng.integers(-2, 3, size=(int(dl.sum()), d)).astype(np.float32)
    sv = lik.maxsim_varlen(dev(Qp, dt), dev(Dp, dt), dev(cu_q), dev(cu_d), int(ql.max()), int(dl.max()))
    assert np.array_equal(f32(sv), O.maxsim_varlen(Qp, Dp, cu_q, cu_d))
    pq, pd = rng.integers(0, 5, size=11).astype(np.int32), rng.integers(0, 7, size=11).astype(np.int32)
    sp = score_pairs_packed(dev(Qp, dt), dev(Dp, dt), dev(cu_q), dev(cu_d), dev(pq), dev(pd), max_seqlen_q=int(ql.max()),
                            max_seqlen_d=int(dl.max()))
    assert np.array_equal(f32(sp), O.maxsim_pair_list(Qp, Dp, cu_q, cu_d, pq, pd))
    # retrieve: integer scores tie often, so the index order is a real check
    Nd = int(rng.integers(3, 400))
    Dr = rng.integers(-1, 2, size=(Nd, 24, d)).astype(np.float32)
    Qr = rng.integers(-1, 2, size=(3, 8, d)).astype(np.float32)
    k = min(int(rng.integers(1, 60)), Nd)
    ts, ti = lik.retrieve(dev(Qr, dt), dev(Dr, dt), k, normalize=False)
    ws, wi = O.retrieve(Qr, Dr, k, normalize=False)
    assert np.array_equal(f32(ts), ws) and np.array_equal(ti.cpu().numpy(), wi)


@pytest.mark.parametrize("seed", range(12))
def test_fp8_and_plaid_random_shapes(seed):
    """e4m3 inputs with per-token scales (document strides that are and are not multiples of four: the multipliers
    travel with the tiles or are staged per tile), and PLAID indexes of every bit width, padded and ragged."""
    from late_interaction_kernels_b200 import fp8, plaid

    rng = np.random.default_rng(4000 + seed)
    # ---- e4m3
    Nq, Nd, Lq = int(rng.integers(1, 6)), int(rng.integers(1, 30)), int(rng.choice([4, 32, 50]))
    Ld = int(rng.choice([7, 64, 130, 256, 300, 301]))
    d = int(rng.choice([64, 128, 256]))
    Q = cases.unit(rng.standard_normal((Nq, Lq, d))).astype(np.float32)
    D = (cases.unit(rng.standard_normal((Nd, Ld, d))) * rng.uniform(0.2, 3.0, size=(Nd, Ld, 1))).astype(np.float32)
    dm = _mask(rng, Nd, Ld, str(rng.choice(["none", "prefix", "holes"])))
    q8, sq = fp8.quantize_fp8_per_token(dev(Q))
    d8, sd = fp8.quantize_fp8_per_token(dev(D))
    s = fp8.maxsim_inference_fp8(q8, d8, scale_Q=sq, scale_D=sd, d_mask=dev(dm))
    want = O.maxsim(f32(q8) * f32(sq)[..., None], f32(d8) * f32(sd)[..., None], None, dm)
    assert O.rel_err(f32(s), want) < 1e-3, (Nq, Nd, Lq, Ld, d)  # bf16 output of the reference kernel is coarser; this one is fp32
    # ---- PLAID
    nbits = int(rng.choice([2, 4, 8]))
    dp = int(rng.choice([32, 64, 96, 128]))
    Qp, codes, res, lens, cent, bw, _ = cases.plaid_case(seed, Nq=int(rng.integers(1, 5)), Nd=int(rng.integers(1, 40)), Lq=int(rng.choice([3, 32])),
                                                        Ld=int(rng.choice([9, 70, 300])), d=dp, nbits=nbits, n_centroids=int(rng.choice([16, 300])))
    for norm in (True, False):
        sp = plaid.maxsim_residual(dev(Qp), dev(codes), dev(res), dev(lens), dev(cent), dev(bw), nbits, normalize=norm)
        wp = O.maxsim_residual(Qp, codes, res, lens, cent, bw, nbits, normalize=norm)
        assert O.rel_err(f32(sp), wp) < 3e-2, (nbits, dp, norm)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cf = np.concatenate([codes[j, : lens[j]] for j in range(len(lens))])
    rf = np.concatenate([res[j, : lens[j]] for j in range(len(lens))])
    sv = plaid.maxsim_residual_varlen(dev(Qp), dev(cf), dev(rf), dev(cu), dev(cent), dev(bw), nbits)
    assert O.rel_err(f32(sv), O.maxsim_residual_varlen(Qp, cf, rf, cu, cent, bw, nbits)) < 3e-2
    k = min(5, len(lens))
    ts, ti = plaid.retrieve_residual_varlen(dev(Qp), dev(cf), dev(rf), dev(cu), dev(cent), dev(bw), nbits, k)
    full = f32(sv)
    # the returned documents are the k best of the dense scores (scores compared: near-ties may swap neighbours)
    assert O.rel_err(f32(ts), -np.sort(-full, axis=-1)[:, :k]) < 1e-3
