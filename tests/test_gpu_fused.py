"""GPU tests of the fused paths of the tensor-core kernel: scoring fused with the per-query top-k, PLAID tokens
decoded inside the kernel's producer warps, and pair lists.  Each is compared with the unfused path of this
library bit for bit (same kernel arithmetic, so equality is exact) and with the CPU oracle within the
bf16 tolerance (2e-2; 3e-2 for the 2-bit PLAID index, as in the reference's own tests)."""

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


def _stable_topk(scores, k, largest=True):
    """Top-k of every row with ties to the lower index (what the kernels promise)."""
    order = torch.sort(scores, dim=-1, descending=largest, stable=True).indices[:, :k]
    return torch.gather(scores, 1, order), order


# ----------------------------------------------------------------------------- fused top-k
@pytest.mark.parametrize("nq,lq,nd,ld,d,k", [(1, 32, 37, 9, 64, 5), (3, 32, 700, 40, 128, 100), (8, 32, 5000, 30, 128, 128),
                                             (40, 32, 3000, 50, 128, 10), (5, 20, 900, 33, 64, 17), (9, 7, 400, 12, 32, 1),
                                             (2, 128, 300, 70, 128, 50), (70, 16, 2000, 20, 64, 64)])
def test_fused_topk_equals_score_then_sort(nq, lq, nd, ld, d, k):
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import _lib

    rng = np.random.default_rng(nq * 1000 + nd)
    Q = dev(cases.unit(rng.standard_normal((nq, lq, d))).astype(np.float32), torch.bfloat16)
    D = dev(cases.unit(rng.standard_normal((nd, ld, d))).astype(np.float32), torch.bfloat16)
    dm = dev(cases.prefix_mask(rng.integers(1, ld + 1, size=nd), ld))
    launches = _lib.load().lik_launch_count()
    s, i = lik.retrieve(Q, D, k, d_mask=dm, normalize=False)
    used = _lib.load().lik_launch_count() - launches
    assert used <= 4, f"one pass over the documents, not one launch per chunk (saw {used} launches)"
    full = lik.maxsim(Q, D, d_mask=dm)
    ws, wi = _stable_topk(full, k)
    assert torch.equal(i, wi) and torch.equal(s, ws)
    # chunk= bounds memory in the reference; here it changes nothing
    s2, i2 = lik.retrieve(Q, D, k, d_mask=dm, normalize=False, chunk=64)
    assert torch.equal(i2, i) and torch.equal(s2, s)
    # smallest-k and the default fused normalisation
    from late_interaction_kernels_b200.topk import maxsim_topk

    s3, i3 = maxsim_topk(Q, D, k, d_mask=dm, largest=False)
    ws3, wi3 = _stable_topk(full, k, largest=False)
    assert torch.equal(i3, wi3) and torch.equal(s3, ws3)
    s4, i4 = lik.retrieve(Q, D, k, d_mask=dm)
    ws4, wi4 = _stable_topk(lik.maxsim(Q, D, d_mask=dm, normalize=True), k)
    assert torch.equal(i4, wi4) and torch.equal(s4, ws4)
    lik.check_device_status()


def test_fused_topk_ties_superblocks_and_oracle():
    import late_interaction_kernels_b200 as lik

    rng = np.random.default_rng(7)
    # (a) every document empty: all scores are exactly 0, the k lowest indices win, and every candidate list
    #     overflows with ties many times
    Q = dev(cases.unit(rng.standard_normal((5, 32, 64))).astype(np.float32), torch.bfloat16)
    D = dev(cases.unit(rng.standard_normal((4000, 8, 64))).astype(np.float32), torch.bfloat16)
    none = torch.zeros((4000, 8), dtype=torch.bool, device="cuda")
    s, i = lik.retrieve(Q, D, 100, d_mask=none, normalize=False)
    assert (s == 0).all() and torch.equal(i, torch.arange(100, device="cuda").expand(5, 100))
    # (b) integer-valued data: plenty of exact ties between different documents
    Qi = dev(rng.integers(-1, 2, size=(6, 32, 32)).astype(np.float32), torch.bfloat16)
    Di = dev(rng.integers(-1, 2, size=(3000, 6, 32)).astype(np.float32), torch.bfloat16)
    s, i = lik.retrieve(Qi, Di, 128, normalize=False)
    ws, wi = _stable_topk(lik.maxsim(Qi, Di), 128)
    assert torch.equal(i, wi) and torch.equal(s, ws)
    # (c) a document matrix above the super-block threshold with several query-tile groups
    Q = dev(cases.unit(rng.standard_normal((24, 32, 128))).astype(np.float32), torch.bfloat16)
    D = dev(cases.unit(rng.standard_normal((7000, 64, 128))).astype(np.float32), torch.bfloat16)
    dm = dev(cases.prefix_mask(rng.integers(8, 65, size=7000), 64))
    s, i = lik.retrieve(Q, D, 100, d_mask=dm, normalize=False)
    full = lik.maxsim(Q, D, d_mask=dm)
    ws, wi = _stable_topk(full, 100)
    assert torch.equal(i, wi) and torch.equal(s, ws)
    # ... and against the oracle for two of the queries
    want = O.maxsim(f32(Q[:2]), f32(D), None, dm.cpu().numpy())
    assert O.rel_err(f32(full[:2]), want) < 2e-2
    wsi = O.topk_rows(want, 100)[1]
    got = i[:2].cpu().numpy()
    for r in range(2):
        diff = got[r] != wsi[r]
        # where the order differs the oracle's own scores are within fp32 summation noise of each other
        assert np.all(np.abs(want[r, got[r][diff]] - want[r, wsi[r][diff]]) < 1e-4)


# ----------------------------------------------------------------------------- PLAID decoded inside the kernel
def _plaid_ragged(seed, nd, d, nbits, ncent, max_len, cdtype=np.float16):
    rng = np.random.default_rng(seed)
    lens = rng.integers(0, max_len + 1, size=nd)
    lens[nd // 3] = 0
    T = int(lens.sum())
    codes = rng.integers(0, ncent, size=T).astype(np.int32)
    res = rng.integers(0, 256, size=(T, d * nbits // 8)).astype(np.uint8)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cent = cases.unit(rng.standard_normal((ncent, d))).astype(cdtype)
    bw = np.linspace(-0.1, 0.1, 2**nbits).astype(np.float32)
    return codes, res, cu, cent, bw


@pytest.mark.parametrize("nbits", [2, 4, 8])
@pytest.mark.parametrize("d,cdtype", [(128, torch.float16), (64, torch.float32), (96, torch.bfloat16)])
def test_plaid_decoded_in_kernel_equals_decode_then_score(nbits, d, cdtype, monkeypatch):
    from late_interaction_kernels_b200 import plaid

    codes, res, cu, cent, bw = _plaid_ragged(nbits * 100 + d, 500, d, nbits, 256, 70, np.float32)
    rng = np.random.default_rng(3)
    for nq, lq, qdtype in ((1, 32, torch.bfloat16), (7, 9, torch.float16), (12, 32, torch.bfloat16)):
        Q = dev(rng.standard_normal((nq, lq, d)).astype(np.float32), qdtype)
        args = (Q, dev(codes), dev(res), dev(cu), dev(cent).to(cdtype), dev(bw), nbits)
        for normalize in (True, False):
            monkeypatch.setattr(plaid, "_FUSED_DECODE_MAX_GROUPS", 1 << 30)
            fused = plaid.maxsim_residual_varlen(*args, normalize=normalize)
            monkeypatch.setattr(plaid, "_FUSED_DECODE_MAX_GROUPS", 0)
            split = plaid.maxsim_residual_varlen(*args, normalize=normalize)
            assert torch.equal(fused, split), (nq, lq, normalize)
            want = O.maxsim_residual_varlen(f32(Q), codes, res, cu, f32(args[4]), bw, nbits, normalize=normalize)
            assert O.rel_err(f32(fused), want) < 3e-2
            assert (fused[:, 500 // 3] == 0).all(), "an empty document scores 0"


def test_plaid_padded_training_path_in_kernel(monkeypatch):
    from late_interaction_kernels_b200 import plaid

    Q, codes, res, lens, cent, bw, nbits = cases.plaid_case(5, Nq=6, Nd=40, Lq=32, Ld=50, d=128, nbits=4, n_centroids=512)
    args = (dev(codes), dev(res), dev(lens), dev(cent), dev(bw), nbits)
    outs = []
    for groups in (1 << 30, 0):
        monkeypatch.setattr(plaid, "_FUSED_DECODE_MAX_GROUPS", groups)
        Qt = dev(Q, torch.bfloat16).requires_grad_()
        s = plaid.maxsim_residual(Qt, *args)
        g = torch.arange(s.numel(), device="cuda", dtype=torch.float32).view_as(s) / s.numel() - 0.3
        s.backward(g)
        outs.append((s.detach(), Qt.grad.detach()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    want = O.maxsim_residual(f32(dev(Q, torch.bfloat16)), codes, res, lens, cent, bw, nbits)
    assert O.rel_err(f32(outs[0][0]), want) < 3e-2
    # The gradient of a max jumps when a near-tie flips, and the operands here are rounded to bf16 while the oracle
    # decodes in fp32: so the winners are taken from the kernel (the scores above pin them within tolerance) and the
    # oracle supplies the gradient arithmetic for those winners, including the query-side normalise Jacobian.
    Qb = dev(Q, torch.bfloat16)
    _, am, _ = plaid._maxsim_residual_forward(Qb, *args, True, True)
    emb = O.plaid_decompress(codes, res, cent, bw, nbits, normalize=True)
    g_hat, _ = O.backward_from_argmax(f32(g), O.l2_normalize(f32(Qb)), emb, am.cpu().numpy())
    wq = O.normalize_jacobian(g_hat, f32(Qb))
    assert O.rel_err(f32(outs[0][1]), wq) < 3e-2


def test_plaid_retrieve_in_one_kernel_and_in_pieces(monkeypatch):
    from late_interaction_kernels_b200 import _lib, plaid

    codes, res, cu, cent, bw = _plaid_ragged(11, 3000, 128, 2, 1024, 60)
    rng = np.random.default_rng(4)
    # (queries, decode inside the scoring kernel?, token budget of a piece of decoded rows)
    for nq, in_kernel, budget in ((2, True, 1 << 22), (2, False, 1 << 22), (40, False, 20_000), (40, False, 1 << 22)):
        monkeypatch.setattr(plaid, "_FUSED_DECODE_MAX_GROUPS", (1 << 30) if in_kernel else 0)
        monkeypatch.setattr(plaid, "_DECOMPRESS_TOKENS", budget)
        Q = dev(rng.standard_normal((nq, 32, 128)).astype(np.float32), torch.bfloat16)
        args = (Q, dev(codes), dev(res), dev(cu), dev(cent), dev(bw), 2)
        full = plaid.maxsim_residual_varlen(*args)
        ws, wi = _stable_topk(full, 100)
        n0 = _lib.load().lik_launch_count()
        s, i = plaid.retrieve_residual_varlen(*args, 100, chunk=700)
        used = _lib.load().lik_launch_count() - n0
        assert torch.equal(i, wi) and torch.equal(s, ws), (nq, in_kernel, budget)
        if in_kernel:
            assert used <= 4, f"query norms, decode + score + top-k in one kernel, merge in parts + of the parts (saw {used} launches)"
        elif budget == 20_000:
            assert used >= 4 * 3, "several pieces, each decoded and scored into the same candidate lists"
        s, i = plaid.retrieve_residual_varlen(*args, 100, chunk=700, largest=False)
        ws2, wi2 = _stable_topk(full, 100, largest=False)
        assert torch.equal(i, wi2) and torch.equal(s, ws2), (nq, in_kernel, budget)


# ----------------------------------------------------------------------------- pair lists on the tensor cores
def test_pair_list_on_tensor_cores():
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import _lib, _ops
    from late_interaction_kernels_b200.score_pairs import score_pairs_packed

    Q, D, cu_q, cu_d, pq, pd = cases.pair_list_case(7, n_pairs=300, Nq=20, Nd=30, lq=(1, 32), ld=(0, 300), d=128, normalized=True)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    s = score_pairs_packed(Qb, Db, dev(cu_q), dev(cu_d), dev(pq), dev(pd))
    want = O.maxsim_pair_list(f32(Qb), f32(Db), cu_q, cu_d, pq, pd)
    assert O.rel_err(f32(s), want) < 2e-2
    # the tensor-core kernel took it, and agrees with the portable kernel
    q = _ops.packed_spec(Qb, dev(cu_q), 32)
    d = _ops.packed_spec(Db, dev(cu_d), 300)
    s2, a2 = _ops.forward(q, d, pairing=_lib.PAIR_LIST, pair_q=dev(pq), pair_d=dev(pd), save_argmax=True, argmax_stride=32, engine=2)
    s1, a1 = _ops.forward(q, d, pairing=_lib.PAIR_LIST, pair_q=dev(pq), pair_d=dev(pd), save_argmax=True, argmax_stride=32, engine=1)
    assert torch.equal(s2, s)
    assert torch.allclose(s1, s2, rtol=2e-5, atol=2e-5)
    assert (a1 == a2).float().mean() > 0.999
    # integer data: winners exact
    rng = np.random.default_rng(2)
    Qi = dev(rng.integers(-2, 3, size=Q.shape).astype(np.float32), torch.bfloat16)
    Di = dev(rng.integers(-2, 3, size=D.shape).astype(np.float32), torch.bfloat16)
    qi, di = _ops.packed_spec(Qi, dev(cu_q), 32), _ops.packed_spec(Di, dev(cu_d), 300)
    si, ai = _ops.forward(qi, di, pairing=_lib.PAIR_LIST, pair_q=dev(pq), pair_d=dev(pd), save_argmax=True, argmax_stride=32, engine=2)
    wsi, wai = O.maxsim_pair_list(f32(Qi), f32(Di), cu_q, cu_d, pq, pd, return_argmax=True)
    assert np.array_equal(f32(si), wsi)
    assert np.array_equal(ai.cpu().numpy()[:, :wai.shape[1]], wai)
    # gradients through the tensor-core forward
    Qt, Dt = Qb.clone().requires_grad_(), Db.clone().requires_grad_()
    g = rng.standard_normal(300).astype(np.float32)
    (score_pairs_packed(Qt, Dt, dev(cu_q), dev(cu_d), dev(pq), dev(pd)) * dev(g)).sum().backward()
    wq, wd = O.pair_list_grads(g, f32(Qb), f32(Db), cu_q, cu_d, pq, pd)
    assert O.rel_err(f32(Qt.grad), wq) < 2e-2 and O.rel_err(f32(Dt.grad), wd) < 2e-2
    # the backward is destination-owned for pair lists too: the same bits every time, and nothing from atomics
    from late_interaction_kernels_b200 import _lib as L_

    n0 = L_.load().lik_launch_count()
    for _ in range(3):
        Q2, D2 = Qb.clone().requires_grad_(), Db.clone().requires_grad_()
        (score_pairs_packed(Q2, D2, dev(cu_q), dev(cu_d), dev(pq), dev(pd)) * dev(g)).sum().backward()
        assert torch.equal(Q2.grad, Qt.grad) and torch.equal(D2.grad, Dt.grad)
    assert L_.load().lik_launch_count() > n0
    # fp32 inputs (the exact FMA forward) go through the same grouped backward
    Qf, Df = dev(Q).requires_grad_(), dev(D).requires_grad_()
    (score_pairs_packed(Qf, Df, dev(cu_q), dev(cu_d), dev(pq), dev(pd)) * dev(g)).sum().backward()
    wq32, wd32 = O.pair_list_grads(g, Q, D, cu_q, cu_d, pq, pd)
    assert O.rel_err(f32(Qf.grad), wq32) < 1e-5 and O.rel_err(f32(Df.grad), wd32) < 1e-5
    # an index outside the batch scores 0 and is reported
    bad = pq.copy()
    bad[5] = 99
    sb = score_pairs_packed(Qb, Db, dev(cu_q), dev(cu_d), dev(bad), dev(pd))
    assert float(sb[5]) == 0.0
    with pytest.raises(RuntimeError, match="pair index"):
        lik.check_device_status()
    keep = np.arange(300) != 5
    assert torch.equal(sb[dev(keep)], s[dev(keep)])


# ----------------------------------------------------------------------------- PLAID stages in front of the scorer
def test_plaid_search_pipeline(tmp_path):
    """Reader -> inverted file -> probe -> approximate score -> exact rerank, against the oracle's restatement of the
    same stages (fed the same centroid scores, so that both probe the same lists) and, with nothing pruned, against
    the exhaustive rerank of this library."""
    from test_plaid_index_cpu import write_fastplaid_files

    from late_interaction_kernels_b200 import plaid
    from late_interaction_kernels_b200.plaid_index import build_ivf, plaid_candidates, plaid_search, read_fastplaid_index

    rng = np.random.default_rng(21)
    nd, d, nbits, ncent = 600, 128, 2, 256
    lens = rng.integers(1, 40, size=nd)
    T = int(lens.sum())
    cent = cases.unit(rng.standard_normal((ncent, d))).astype(np.float16)
    # tokens near their centroid, as in a trained index: code = nearest centroid of a random direction
    tok = cases.unit(rng.standard_normal((T, d))).astype(np.float32)
    codes = (tok @ cent.astype(np.float32).T).argmax(-1).astype(np.int32)
    res = rng.integers(0, 256, size=(T, d * nbits // 8)).astype(np.uint8)
    bw = np.linspace(-0.05, 0.05, 4).astype(np.float32)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    path = str(tmp_path / "index")
    write_fastplaid_files(path, codes, res, lens, cent, bw, nbits, merged=True, pad_rows=7)
    ix = build_ivf(read_fastplaid_index(path, device="cuda"))
    Q = dev(rng.standard_normal((32, d)).astype(np.float32), torch.bfloat16)
    # nothing pruned: identical to scoring the whole index
    s_all, i_all = plaid_search(ix, Q, 10, nprobe=ncent, ndocs=nd)
    ws, wi = plaid.retrieve_residual_varlen(Q, ix.codes_flat, ix.residuals_flat, ix.cu_seqlens_d, ix.centroids, ix.bucket_weights, nbits, 10)
    assert torch.equal(i_all, wi) and torch.equal(s_all, ws)
    # pruned: same candidates, survivors and ranking as the oracle's pipeline on the same centroid scores
    Qn = torch.nn.functional.normalize(Q.float(), dim=-1)
    qcs = (ix.centroids.float() @ Qn.t()).contiguous()
    cand = plaid_candidates(ix, qcs, 3)
    s, i = plaid_search(ix, Q, 10, nprobe=3, ndocs=50)
    os_, oi = O.plaid_search(f32(Q), codes, res, cu, cent, bw, nbits, 10, nprobe=3, ndocs=50, qcs=f32(qcs))
    assert 50 < cand.numel() < nd, "the probe prunes, and leaves more than ndocs for the approximate stage to cut"
    assert set(i.tolist()) <= set(cand.tolist())
    assert O.rel_err(f32(s), os_) < 3e-2
    same = i.cpu().numpy() == oi
    assert same.mean() >= 0.8 and np.all(np.abs(f32(s)[~same] - os_[~same]) < 3e-2 * np.abs(os_).max())
    # a batch is one search per query
    sb, ib = plaid_search(ix, torch.stack([Q, Q.flip(0)]), 10, nprobe=3, ndocs=50)
    assert torch.equal(sb[0], s) and torch.equal(ib[0], i) and sb.shape == (2, 10)
