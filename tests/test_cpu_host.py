"""CPU-side checks: the C-ABI library loads and exports everything ``include/lik_b200.h`` declares,
host-side validation raises the documented errors, and nothing falls back to the CPU."""

import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from late_interaction_kernels_b200 import _build, _lib

    _build.build()
    return _lib.load()


def test_header_symbols_are_exported(lib):
    from late_interaction_kernels_b200 import _lib

    text = open(os.path.join(ROOT, "include", "lik_b200.h")).read()
    declared = set(re.findall(r"\b(lik_[a-z0-9_]+)\s*\(", text))
    assert declared, "no declarations found"
    for sym in declared:
        assert hasattr(lib, sym), f"{sym} declared in the header but not exported"
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    assert lib.lik_version() >= 200


def test_struct_sizes_match_the_header_layout():
    import ctypes as C

    from late_interaction_kernels_b200 import _lib

    assert C.sizeof(_lib.Seqs) == 80
    assert C.sizeof(_lib.FwdArgs) == 2 * 80 + 96
    assert C.sizeof(_lib.PlaidIndex) == 56
    assert C.sizeof(_lib.TopkSpec) == 40
    assert C.sizeof(_lib.HiddenFwdArgs) == 2 * 80 + 88


def test_argument_validation_without_a_gpu(lib):
    import ctypes as C

    from late_interaction_kernels_b200 import _lib

    a = _lib.FwdArgs()
    a.dim = 0
    assert lib.lik_maxsim_fwd(C.byref(a), None) == -1
    assert b"dim" in lib.lik_last_error()
    assert lib.lik_maxsim_fwd(None, None) == -1
    assert lib.lik_topk_rows(None, 1, 1, 1, 0, 1, 0, 0, None, None, None) == -1
    ix = _lib.PlaidIndex()
    ix.nbits = 3
    assert lib.lik_plaid_decompress(C.byref(ix), 0, 0, 1, None, 2, None, None) == -1
    assert b"nbits must be 2, 4, or 8" in lib.lik_last_error()
    # document head: NULL arguments and bad sizes are refused before any CUDA call; without a GPU nothing is supported
    assert lib.lik_maxsim_hidden_fwd(None, None) == -1
    h = _lib.HiddenFwdArgs()
    assert lib.lik_maxsim_hidden_fwd(C.byref(h), None) == -1
    assert b"must not be NULL" in lib.lik_last_error()
    assert lib.lik_maxsim_hidden_fwd_supported(C.byref(h)) == 0
    assert lib.lik_maxsim_hidden_fwd_workspace(C.byref(h)) == 0
    assert lib.lik_hidden_winners(None, 1, 1, 0, 1, 1, None, None, None, None, None, None, None) == -1
    assert lib.lik_hidden_winners(None, 1, 0, 4, 8, 4, None, None, None, None, None, None, None) == 0  # no documents: nothing to do
    assert lib.lik_hidden_scatter_rows(None, 24, 1, 8, 4, None, None, None, None) == -1


def test_no_cpu_fallback_anywhere():
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import fp8, plaid
    from late_interaction_kernels_b200.backward import maxsim_backward_lowmem, maxsim_backward_unified
    from late_interaction_kernels_b200.score_pairs import score_pairs_packed

    Q, D = torch.randn(2, 3, 16), torch.randn(2, 4, 16)
    cu = torch.tensor([0, 3, 6], dtype=torch.int32)
    for fn in (
        lambda: lik.maxsim(Q, D),
        lambda: lik.maxsim_pairs(Q, D),
        lambda: lik.maxsim_varlen(Q.view(-1, 16), D.view(-1, 16), cu, torch.tensor([0, 4, 8], dtype=torch.int32)),
        lambda: lik.maxsim_padded(Q, D[:, None], torch.tensor([3, 3]), torch.tensor([[4], [4]])),
        lambda: lik.retrieve(Q, D, 1),
        lambda: lik.MaxSimScorer()(Q, D),
        lambda: score_pairs_packed(Q.view(-1, 16), D.view(-1, 16), cu, cu, torch.tensor([0]), torch.tensor([1])),
        lambda: maxsim_backward_unified(torch.zeros(2, 2), Q, D, torch.zeros(4, 3, dtype=torch.int32)),
        lambda: maxsim_backward_lowmem(torch.zeros(2, 2), Q, D, torch.zeros(4, 3, dtype=torch.int32)),
        lambda: plaid.plaid_approx_score(torch.randn(4, 3), torch.zeros(2, 5, dtype=torch.int32), torch.tensor([1, 2])),
    ):
        with pytest.raises(RuntimeError, match="CUDA"):
            fn()
    with pytest.raises(ValueError, match="float8_e4m3fn"):
        fp8.maxsim_inference_fp8(Q, D, scale_Q=torch.ones(()), scale_D=torch.ones(()))


def test_host_validation_messages():
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import plaid
    from late_interaction_kernels_b200.padded import pack_padded

    Q, D = torch.randn(2, 3, 16), torch.randn(2, 4, 16)
    with pytest.raises(ValueError, match="backward= must be one of"):
        lik.maxsim(Q, D, backward="nope")
    with pytest.raises(ValueError, match="backward= must be one of"):
        lik.MaxSimScorer(backward="nope")
    with pytest.raises(ValueError, match="top_k must be positive"):
        lik.retrieve(Q, D, 0)
    with pytest.raises(ValueError, match="mask_pad_token"):
        lik.MaxSimScorer().forward_with_ids(Q, D, None, None)
    with pytest.raises(ValueError, match="2-D"):
        lik.maxsim_varlen(Q, D, None, None)
    with pytest.raises(ValueError, match="nbits must be 2, 4, or 8"):
        plaid.maxsim_residual_varlen(Q, None, None, None, None, None, 3)
    with pytest.raises(ValueError, match=r"queries must be \[B, Lq, d\]"):
        pack_padded(Q[0], D[:, None], torch.tensor([3]), torch.tensor([[4]]))
    with pytest.raises(ValueError, match="doc_lengths must be"):
        pack_padded(Q, D[:, None], torch.tensor([3, 3]), torch.tensor([4, 4]))


def test_loss_head_helpers_validate_on_the_host():
    from late_interaction_kernels_b200.loss_heads import maxsim_pos_neg, maxsim_tiles

    q, d = torch.randn(2, 3, 16), torch.randn(2, 4, 16)
    with pytest.raises(ValueError, match="at least one"):
        maxsim_tiles([], [d])
    with pytest.raises(ValueError, match="same d"):
        maxsim_tiles([q], [torch.randn(2, 4, 8)])
    with pytest.raises(ValueError, match="one mask"):
        maxsim_tiles([q, q], [d], q_masks=[None])
    with pytest.raises(RuntimeError, match="CUDA"):
        maxsim_tiles([q], [d])  # host tensors: no CPU path
    with pytest.raises(ValueError, match="expected Q"):
        maxsim_pos_neg(q, d, d)


def test_pack_padded_on_cpu_matches_reference_golden():
    """pack_padded is pure host/torch logic, so it also runs on CPU tensors."""
    import numpy as np
    from conftest import load_golden

    import cases
    from late_interaction_kernels_b200.padded import pack_padded

    g = load_golden("padded")
    q, docs, ql, dl = cases.padded_case(8)
    pk = pack_padded(torch.tensor(q), torch.tensor(docs), torch.tensor(ql), torch.tensor(dl))
    Qp, cq, Dp, cd, pq, pd, mq, md = pk
    for a, k in ((Qp, "Q_packed"), (cq, "cu_q"), (Dp, "D_packed"), (cd, "cu_d"), (pq, "pair_q"), (pd, "pair_d")):
        assert np.array_equal(a.numpy(), g[k]), k
    assert (mq, md) == (int(g["max_q"]), int(g["max_d"]))
    with pytest.raises(ValueError, match="> 0"):
        pack_padded(torch.tensor(q), torch.tensor(docs), torch.tensor(ql * 0), torch.tensor(dl), validate=True)
    with pytest.raises(ValueError, match="exceeds the padded extent"):
        pack_padded(torch.tensor(q), torch.tensor(docs), torch.tensor(ql + 100), torch.tensor(dl), validate=True)
    e = pack_padded(torch.zeros(0, 8, 16), torch.zeros(0, 4, 13, 16), torch.zeros(0, dtype=torch.long), torch.zeros(0, 4, dtype=torch.long))
    assert e.Q_packed.shape == (0, 16) and e.max_seqlen_q == 0 and e.cu_seqlens_d.tolist() == [0]


def test_fp8_quantisers_on_cpu_match_reference_golden():
    import numpy as np
    from conftest import load_golden

    from late_interaction_kernels_b200 import fp8

    g = load_golden("fp8")
    rng = np.random.default_rng(9)
    X = (rng.standard_normal((5, 7, 32)) * np.array([1e-3, 0.1, 1, 10, 300]).reshape(5, 1, 1)).astype(np.float32)
    X[0, 0] = 0.0
    xq, sc = fp8.quantize_fp8_per_token(torch.tensor(X))
    assert np.array_equal(xq.float().numpy(), g["q_tok"]) and np.array_equal(sc.numpy(), g["s_tok"])
    assert np.array_equal(fp8.dequantize_fp8_per_token(xq, sc).numpy(), g["deq_tok"])
    xq2, sc2 = fp8.quantize_fp8_per_tensor(torch.tensor(X))
    assert np.array_equal(xq2.float().numpy(), g["q_ten"]) and np.array_equal(sc2.numpy(), g["s_ten"])


def test_reference_package_name_resolves_to_this_build():
    import importlib

    import late_interaction_kernels as alias
    import late_interaction_kernels_b200 as impl

    assert alias.maxsim is impl.maxsim and alias.MaxSimScorer is impl.MaxSimScorer and callable(alias.retrieve)
    assert importlib.import_module("late_interaction_kernels.plaid").maxsim_residual is impl.plaid.maxsim_residual
    assert importlib.import_module("late_interaction_kernels.retrieve").retrieve is impl.retrieve
    from late_interaction_kernels.backward.lowmem import maxsim_backward_lowmem  # noqa: F401
