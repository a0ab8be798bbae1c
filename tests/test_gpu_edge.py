"""GPU edge cases and size-independent properties (the reference's test_edge_cases / test_robustness,
plus checks at the headline workload sizes where the CPU oracle is too slow to be the checker)."""

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


@pytest.mark.parametrize("d", [8, 16, 33, 37, 63, 96, 111, 250, 513])
def test_embedding_widths(d):
    import late_interaction_kernels_b200 as lik

    Q, D, _, dm = cases.dense_case(d, 3, 5, 7, 21, d, d_len=(1, 21), normalized=True)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        want = O.maxsim(f32(dev(Q, dtype)), f32(dev(D, dtype)), None, dm)
        got = lik.maxsim(dev(Q, dtype), dev(D, dtype), None, dev(dm))
        assert O.rel_err(f32(got), want) < tol, (d, dtype)


def test_degenerate_lengths_and_many_docs():
    import late_interaction_kernels_b200 as lik

    rng = np.random.default_rng(0)
    for Lq, Ld in ((1, 1), (1, 40), (33, 1), (200, 3)):
        Q = cases.unit(rng.standard_normal((2, Lq, 64))).astype(np.float32)
        D = cases.unit(rng.standard_normal((3, Ld, 64))).astype(np.float32)
        got = lik.maxsim(dev(Q, torch.bfloat16), dev(D, torch.bfloat16))
        assert O.rel_err(f32(got), O.maxsim(f32(dev(Q, torch.bfloat16)), f32(dev(D, torch.bfloat16)))) < 2e-2
    Q = cases.unit(rng.standard_normal((1, 32, 128))).astype(np.float32)
    D = cases.unit(rng.standard_normal((1000, 60, 128))).astype(np.float32)
    got = lik.maxsim(dev(Q, torch.float16), dev(D, torch.float16))
    assert got.shape == (1, 1000)
    assert O.rel_err(f32(got), O.maxsim(f32(dev(Q, torch.float16)), f32(dev(D, torch.float16)))) < 5e-3
    # empty batches
    assert lik.maxsim(dev(Q), dev(D[:0])).shape == (1, 0)
    assert lik.maxsim(dev(Q[:0]), dev(D[:4])).shape == (0, 4)


def test_long_queries_are_chunked_exactly():
    import late_interaction_kernels_b200 as lik

    Q, D, qm, dm = cases.dense_case(77, 3, 4, 300, 140, 128, q_len=(130, 300), d_len=(1, 140), normalized=True)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    want = O.maxsim(f32(Qb), f32(Db), qm, dm)
    got = lik.maxsim(Qb, Db, dev(qm), dev(dm))
    assert O.rel_err(f32(got), want) < 2e-2
    # summing per-128-token pieces of the query reproduces the full score (MaxSim is additive over query tokens)
    parts = sum(lik.maxsim(Qb[:, a:a + 128], Db, dev(qm[:, a:a + 128]), dev(dm)) for a in range(0, 300, 128))
    assert torch.allclose(parts, got, rtol=1e-5, atol=1e-4)
    Qt, Dt = Qb.clone().requires_grad_(), Db.clone().requires_grad_()
    go = np.random.default_rng(1).standard_normal((3, 4)).astype(np.float32)
    (lik.maxsim(Qt, Dt, dev(qm), dev(dm)) * dev(go)).sum().backward()
    wq, wd = O.maxsim_grads(go, f32(Qb), f32(Db), qm, dm)
    assert O.rel_err(f32(Qt.grad), wq) < 2e-2 and O.rel_err(f32(Dt.grad), wd) < 2e-2


def test_tensor_core_engine_agrees_with_portable_engine():
    from late_interaction_kernels_b200 import _lib, _ops

    rng = np.random.default_rng(5)
    for (nq, nd, lq, ld, d, dtype) in ((9, 31, 32, 300, 128, torch.bfloat16), (5, 12, 17, 77, 64, torch.float16),
                                      (3, 6, 128, 513, 96, torch.bfloat16), (2, 8, 150, 64, 128, torch.bfloat16)):
        Q = dev(cases.unit(rng.standard_normal((nq, lq, d))).astype(np.float32), dtype)
        D = dev(cases.unit(rng.standard_normal((nd, ld, d))).astype(np.float32), dtype)
        holes = dev(rng.random((nd, ld)) > 0.3)
        holes[:, 0] = True
        holes[1] = False
        q, dd = _ops.padded_spec(Q), _ops.padded_spec(D, holes)
        for norm in (_lib.NORM_NONE, _lib.NORM_BOTH):
            s1, a1 = _ops.forward(q, dd, normalize=norm, save_argmax=True, engine=1)
            s2, a2 = _ops.forward(q, dd, normalize=norm, save_argmax=True, engine=2)
            assert torch.allclose(s1, s2, rtol=2e-5, atol=2e-5), (nq, nd, lq, ld, d, norm)
            assert (a1 == a2).float().mean() > 0.999
            assert (a2.view(nq, nd, lq)[:, 1] == -1).all()


def test_int64_offsets_explicit_maxima_and_status_word():
    import late_interaction_kernels_b200 as lik

    Q, D, cu_q, cu_d = cases.varlen_case(16, Nq=6, Nd=5, lq=(3, 20), ld=(10, 90), d=64, normalized=True)
    Qb, Db = dev(Q, torch.bfloat16), dev(D, torch.bfloat16)
    base = lik.maxsim_varlen(Qb, Db, dev(cu_q.astype(np.int64)), dev(cu_d.astype(np.int64)))
    assert torch.equal(lik.maxsim_varlen(Qb, Db, dev(cu_q), dev(cu_d), 20, 90), base)
    assert torch.equal(lik.maxsim_varlen(Qb, Db, dev(cu_q), dev(cu_d), 64, 1000), base), "generous maxima change nothing"
    lik.check_device_status()
    # a max_seqlen_q below the longest query cannot store every winner: reported through the status word
    Qt = Qb.clone().requires_grad_()
    lik.maxsim_varlen(Qt, Db, dev(cu_q), dev(cu_d), 2, 90)
    with pytest.raises(RuntimeError, match="max_seqlen_q|padded extent"):
        lik.check_device_status()


def test_full_size_inbatch_properties():
    """The headline in-batch shape: checked through properties instead of the (too slow) oracle."""
    import late_interaction_kernels_b200 as lik

    g = torch.Generator(device="cuda").manual_seed(0)
    Q = torch.nn.functional.normalize(torch.randn(512, 32, 128, generator=g, device="cuda"), dim=-1).bfloat16()
    D = torch.nn.functional.normalize(torch.randn(512, 300, 128, generator=g, device="cuda"), dim=-1).bfloat16()
    lens = torch.randint(64, 301, (512,), generator=g, device="cuda")
    dm = torch.arange(300, device="cuda")[None] < lens[:, None]
    s = lik.maxsim(Q, D, d_mask=dm)
    # 1. a block of the score matrix equals scoring that block alone (tiling independence), bit for bit
    assert torch.equal(lik.maxsim(Q[100:228], D[37:300], d_mask=dm[37:300]), s[100:228, 37:300])
    # 2. permuting documents permutes columns
    perm = torch.randperm(512, generator=g, device="cuda")
    assert torch.equal(lik.maxsim(Q, D[perm], d_mask=dm[perm]), s[:, perm])
    # 3. a sampled corner against the oracle
    want = O.maxsim(f32(Q[:8]), f32(D[:16]), None, dm[:16].cpu().numpy())
    assert O.rel_err(f32(s[:8, :16]), want) < 2e-2
    # 4. backward is linear in the upstream gradient and deterministic
    Qt, Dt = Q.clone().requires_grad_(), D.clone().requires_grad_()
    g1 = torch.randn(512, 512, generator=g, device="cuda")
    out = lik.maxsim(Qt, Dt, d_mask=dm)
    gq1, gd1 = torch.autograd.grad(out, (Qt, Dt), g1, retain_graph=True)
    gq1b, gd1b = torch.autograd.grad(out, (Qt, Dt), g1, retain_graph=True)
    assert torch.equal(gq1, gq1b) and torch.equal(gd1, gd1b)
    gq2, gd2 = torch.autograd.grad(out, (Qt, Dt), 2 * g1)
    assert torch.allclose(gq2.float(), 2 * gq1.float(), rtol=2e-2, atol=1e-3)
    assert torch.allclose(gd2.float(), 2 * gd1.float(), rtol=2e-2, atol=1e-3)
    assert (gd1[~dm] == 0).all(), "masked document tokens get exactly zero gradient"
    # 5. sampled gradient rows against the oracle (first 4 queries see every document)
    wq, _ = O.maxsim_grads(f32(g1[:4]), f32(Q[:4]), f32(D), None, dm.cpu().numpy())
    assert O.rel_err(f32(gq1[:4]), wq) < 2e-2


def test_torch_compile_and_module_in_a_model():
    import late_interaction_kernels_b200 as lik

    scorer = lik.MaxSimScorer(normalize=True)
    Q = torch.randn(4, 16, 64, device="cuda", dtype=torch.bfloat16)
    D = torch.randn(6, 40, 64, device="cuda", dtype=torch.bfloat16)
    eager = scorer(Q, D)

    @torch.compile(fullgraph=False)
    def f(q, d):
        return scorer(q, d) * 2

    assert torch.allclose(f(Q, D), eager * 2)
    ids_q = torch.randint(1, 5, (4, 16), device="cuda")
    ids_d = torch.randint(0, 5, (6, 40), device="cuda")
    s = lik.MaxSimScorer(mask_pad_token=0).forward_with_ids(Q, D, ids_q, ids_d)
    assert torch.equal(s, lik.maxsim(Q, D, q_mask=ids_q != 0, d_mask=ids_d != 0, normalize=True))


def test_plaid_retrieve_matches_score_then_topk():
    from late_interaction_kernels_b200 import plaid, sharded

    rng = np.random.default_rng(3)
    Nd, d, nbits, ncent = 300, 64, 2, 128
    lens = rng.integers(0, 40, size=Nd)
    lens[5] = 0
    T = int(lens.sum())
    codes = rng.integers(0, ncent, size=T).astype(np.int32)
    res = rng.integers(0, 256, size=(T, d * nbits // 8)).astype(np.uint8)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cent = cases.unit(rng.standard_normal((ncent, d))).astype(np.float16)
    bw = np.linspace(-0.1, 0.1, 4).astype(np.float32)
    Q = rng.standard_normal((7, 9, d)).astype(np.float32)
    args = (dev(Q, torch.bfloat16), dev(codes), dev(res), dev(cu), dev(cent), dev(bw), nbits)
    full = plaid.maxsim_residual_varlen(*args)
    ws, wi = torch.topk(full, 25, dim=-1)
    for chunk in (16, 64, 1000):
        s, i = plaid.retrieve_residual_varlen(*args, 25, chunk=chunk)
        assert torch.equal(s, ws), chunk
        assert torch.equal(torch.gather(full, 1, i), ws), "indices point at the top scores"
    want = O.maxsim_residual_varlen(f32(args[0]), codes, res, cu, cent, bw, nbits)
    assert O.rel_err(f32(full), want) < 3e-2
    # single-process "sharded" call degenerates to the local top-k
    s, i = sharded.retrieve_plaid_sharded(*args, 25, doc_offset=0, n_docs_total=Nd, chunk=64)
    assert torch.equal(s, ws)
    s1, i1 = sharded.retrieve_sharded(dev(Q, torch.bfloat16), dev(rng.standard_normal((40, 12, d)).astype(np.float32), torch.bfloat16),
                                      10, doc_offset=1000, n_docs_total=40)
    assert s1.shape == (7, 10) and int(i1.min()) >= 1000


def test_exact_ties_pick_the_lowest_column_everywhere():
    """Integer-valued embeddings make the scores exact, so duplicated document tokens tie exactly: the saved
    winner must be the lowest column wherever the copies sit — inside one 32-column chunk, in chunks read by
    different warps, in the partial last chunk, and in the second tile of a document longer than 256 tokens
    (reference contract: lowest index wins, forward.py:168-169)."""
    from late_interaction_kernels_b200 import _ops

    rng = np.random.default_rng(17)
    nq, lq, d, ld = 5, 32, 64, 300
    lens = np.array([300, 257, 256, 255, 97, 33, 31, 1])
    nd = len(lens)
    Q = rng.integers(-2, 3, size=(nq, lq, d)).astype(np.float32)
    D = rng.integers(-2, 3, size=(nd, ld, d)).astype(np.float32)
    # copies of one row at columns chosen to straddle chunk, warp-half and tile boundaries
    for j, cols in enumerate(([3, 35, 64, 131, 255, 256, 299], [40, 8, 256], [255, 0, 31, 32], [254, 224, 200], [96, 64, 65],
                              [32, 1], [30, 29, 2], [0])):
        for c in cols[1:]:
            D[j, c] = D[j, cols[0]]
    D[2, :256] = D[2, 17]  # a document whose tokens are all the same: every winner is column 0
    D[2, 0] = D[2, 17]
    dm = np.arange(ld)[None, :] < lens[:, None]
    S = np.einsum("isk,jtk->ijst", Q, D)
    S = np.where(dm[None, :, None, :], S, -np.inf)
    want_arg = S.argmax(-1).astype(np.int32)  # first occurrence of the maximum
    want = S.max(-1).sum(-1)
    for dtype in (torch.bfloat16, torch.float16):
        q, dd = _ops.padded_spec(dev(Q, dtype)), _ops.padded_spec(dev(D, dtype), dev(dm))
        for engine in (1, 2):
            s, a = _ops.forward(q, dd, save_argmax=True, engine=engine)
            assert np.array_equal(f32(s).reshape(nq, nd), want), (dtype, engine)
            assert np.array_equal(a.cpu().numpy().reshape(nq, nd, lq), want_arg), (dtype, engine)
        s0, _ = _ops.forward(q, dd, engine=2)  # the path without argmax gives the same bits
        assert torch.equal(s0, s)


def test_opt_in_rounded_normalisation_stays_within_tolerance():
    """LIK_NORM_ROUNDED (normalised 16-bit operand copies, the reference GPU kernel's arithmetic) is opt-in: it
    must stay within the bf16 tolerance of the oracle and of the default fp32-inverse-norm path."""
    from late_interaction_kernels_b200.forward import maxsim_forward

    Q, D, _, dm = cases.dense_case(21, 9, 40, 32, 77, 128, d_len=(1, 77), normalized=False)
    for dtype in (torch.bfloat16, torch.float16):
        Qt, Dt = dev(Q * 3.0, dtype), dev(D * 0.25, dtype)
        want = O.maxsim(f32(Qt), f32(Dt), None, dm, normalize=True)
        base, _ = maxsim_forward(Qt, Dt, d_mask=dev(dm), normalize=True)
        fast, _ = maxsim_forward(Qt, Dt, d_mask=dev(dm), normalize=True, _rounded_norm=True)
        assert O.rel_err(f32(base), want) < 1e-3
        assert O.rel_err(f32(fast), want) < 2e-2
        assert not torch.equal(fast, base), "the two forms are different arithmetic"


def test_backward_with_forked_stream_is_graph_capturable():
    """Both gradients on a large enough problem: the grad_Q kernel runs on the library's second stream
    between an event fork and join.  That pattern must survive CUDA-graph capture and replay, and give the
    same bits as the eager call."""
    from late_interaction_kernels_b200 import _ops

    g = torch.Generator().manual_seed(3)
    Q = torch.nn.functional.normalize(torch.randn(192, 32, 64, generator=g), dim=-1).cuda().bfloat16()
    D = torch.nn.functional.normalize(torch.randn(192, 200, 64, generator=g), dim=-1).cuda().bfloat16()
    go = torch.randn(192, 192, generator=g).cuda()
    q, d = _ops.padded_spec(Q), _ops.padded_spec(D)
    _, am = _ops.forward(q, d, save_argmax=True)
    assert am.numel() >= 1 << 20  # large enough for the fork
    eq, ed = _ops.backward(q, d, go, am)
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            gq, gd = _ops.backward(q, d, go, am)
    gq.zero_()
    gd.zero_()
    gr.replay()
    torch.cuda.synchronize()
    assert torch.equal(gq, eq) and torch.equal(gd, ed)


def test_a_bounded_wait_that_runs_out_reports_and_returns():
    """Failure detection without a fault: the wait the tensor-core kernel's roles use, on a barrier nothing arrives
    at, must give up after its cycle limit, raise the time-out bit in the status word and let the kernel return."""
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import _lib, _ops

    lib = _lib.load()
    status = _ops.status_word("cuda")
    lik.check_device_status()
    res = torch.full((3,), -1, dtype=torch.int32, device="cuda")
    limit = 2_000_000  # about a millisecond
    _lib.check(lib.lik_selftest_wait_timeout(limit, status.data_ptr(), res.data_ptr(), _lib.stream_ptr(res.device)), "selftest")
    torch.cuda.synchronize()
    got, aborted, cycles = res.tolist()
    assert got == 0 and aborted == 1
    assert limit <= cycles < 50 * limit
    with pytest.raises(RuntimeError, match="bounded wait expired"):
        lik.check_device_status()
    lik.check_device_status()  # the word was reset; the context is healthy
    assert float(lik.maxsim(torch.ones(1, 2, 16, device="cuda").bfloat16(), torch.ones(1, 3, 16, device="cuda").bfloat16())) == 32.0
    assert lib.lik_selftest_wait_timeout(10**10, None, res.data_ptr(), None) == -1
