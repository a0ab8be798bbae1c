"""Regenerate ``tests/golden/*.npz`` from the reference implementation itself.

Run once, in a container that has the reference checkout (read-only is fine):

    python tests/golden/make_golden.py --reference /path/to/late-interaction-kernels

It imports the reference's CPU-runnable code (``reference.py``, the pure-torch
backward reference, the FP8 quantisers, ``pack_padded``, CPU ``retrieve``) and
stores their outputs on the seeded inputs of ``cases.py``.  The tests never
need the reference checkout: they read the ``.npz`` files.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of hcompai/late-interaction-kernels to import")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    import torch
    import torch.nn.functional as F
    from late_interaction_kernels import fp8 as rfp8
    from late_interaction_kernels import padded as rpad
    from late_interaction_kernels import reference as ref
    import importlib

    rret = importlib.import_module("late_interaction_kernels.retrieve")
    from late_interaction_kernels.backward.unified import maxsim_backward_unified_reference

    T = torch.from_numpy
    tb = lambda m: None if m is None else T(np.ascontiguousarray(m))  # noqa: E731
    out = {}

    # ---- dense forward (reference.py:26-98) ---------------------------------
    Q, D, qm, dm = cases.config1()
    out["config1"] = dict(
        chk=cases.checksum(Q, D, qm, dm),
        scores=ref.maxsim_reference(T(Q), T(D), tb(qm), tb(dm), normalize=True).numpy(),
        scores_nonorm=ref.maxsim_reference(T(Q), T(D), tb(qm), tb(dm)).numpy(),
    )
    Q, D, qm, dm = cases.random_mask_case(1)
    out["random_mask"] = dict(
        chk=cases.checksum(Q, D, qm, dm),
        scores=ref.maxsim_reference(T(Q), T(D), tb(qm), tb(dm)).numpy(),
        scores_norm=ref.maxsim_reference(T(Q), T(D), tb(qm), tb(dm), normalize=True).numpy(),
        scores_nomask=ref.maxsim_reference(T(Q), T(D)).numpy(),
        scores_2d=ref.maxsim_reference(T(Q[0]), T(D[0]), tb(qm[0]), tb(dm[0])).numpy(),
        scores_q2d=ref.maxsim_reference(T(Q[0]), T(D)).numpy(),
    )
    Q, D, qm, dm = cases.dense_case(2, 6, 7, 9, 21, 24, d_len=(3, 21))
    Q64, D64 = Q.astype(np.float64), D.astype(np.float64)
    out["dense_fp64"] = dict(
        chk=cases.checksum(Q, D, dm), scores=ref.maxsim_reference(T(Q64), T(D64), None, tb(dm)).numpy()
    )

    # ---- gradients through the reference (autograd) --------------------------
    for name, norm in (("grads", False), ("grads_norm", True)):
        Q, D, qm, dm = cases.random_mask_case(3, Nq=4, Nd=5, Lq=6, Ld=13, d=16)
        g = np.random.default_rng(33).standard_normal((4, 5))
        Qt = T(Q.astype(np.float64)).requires_grad_()
        Dt = T(D.astype(np.float64)).requires_grad_()
        s = ref.maxsim_reference(Qt, Dt, tb(qm), tb(dm), normalize=norm)
        (s * T(g)).sum().backward()
        out[name] = dict(chk=cases.checksum(Q, D, qm, dm, g), gQ=Qt.grad.numpy(), gD=Dt.grad.numpy())

    # ---- backward from a given argmax (backward/unified.py:27-85) ------------
    Q, D, qm, _ = cases.random_mask_case(4, Nq=3, Nd=4, Lq=5, Ld=8, d=8)
    rng = np.random.default_rng(44)
    am = rng.integers(0, 8, size=(3 * 4, 5)).astype(np.int32)
    g = rng.standard_normal((3, 4)).astype(np.float32)
    gQ, gD = maxsim_backward_unified_reference(T(g), T(Q), T(D), T(am), tb(qm))
    out["bwd_argmax"] = dict(chk=cases.checksum(Q, D, qm, am, g), gQ=gQ.numpy(), gD=gD.numpy())

    # ---- KD layout: per-query loops of the dense reference -------------------
    Q, D, qm, dm = cases.kd_case(5)
    sc = np.stack(
        [ref.maxsim_reference(T(Q[i : i + 1]), T(D[i]), tb(qm[i : i + 1]), tb(dm[i])).numpy()[0] for i in range(Q.shape[0])]
    )
    Qt = T(Q.astype(np.float64)).requires_grad_()
    Dt = T(D.astype(np.float64)).requires_grad_()
    g = np.random.default_rng(55).standard_normal(sc.shape)
    tot = 0
    for i in range(Q.shape[0]):
        tot = tot + (ref.maxsim_reference(Qt[i : i + 1], Dt[i], tb(qm[i : i + 1]), tb(dm[i]), normalize=True)[0] * T(g[i])).sum()
    tot.backward()
    out["kd"] = dict(chk=cases.checksum(Q, D, qm, dm), scores=sc, g=g, gQ_norm=Qt.grad.numpy(), gD_norm=Dt.grad.numpy())

    # ---- packed layouts (reference.py:213-306) -------------------------------
    Q, D, cu_q, cu_d = cases.varlen_case(6)
    Qt, Dt = T(Q.astype(np.float64)).requires_grad_(), T(D.astype(np.float64)).requires_grad_()
    s = ref.maxsim_reference_varlen(Qt, Dt, T(cu_q), T(cu_d))
    g = np.random.default_rng(66).standard_normal(tuple(s.shape)).astype(np.float32)
    (s * T(g)).sum().backward()
    out["varlen"] = dict(chk=cases.checksum(Q, D, cu_q, cu_d), scores=s.detach().numpy(), g=g, gQ=Qt.grad.numpy(), gD=Dt.grad.numpy())

    Q, D, cu_q, cu_d, pq, pd = cases.pair_list_case(7)
    Qt, Dt = T(Q.astype(np.float64)).requires_grad_(), T(D.astype(np.float64)).requires_grad_()
    s = ref.maxsim_reference_scatter(Qt, Dt, T(cu_q), T(cu_d), T(pq), T(pd))
    g = np.random.default_rng(77).standard_normal(tuple(s.shape)).astype(np.float32)
    (s * T(g)).sum().backward()
    out["pair_list"] = dict(chk=cases.checksum(Q, D, cu_q, cu_d, pq, pd), scores=s.detach().numpy(), g=g, gQ=Qt.grad.numpy(), gD=Dt.grad.numpy())

    q, docs, ql, dl = cases.padded_case(8)
    pk = rpad.pack_padded(T(q), T(docs), T(ql), T(dl))
    out["padded"] = dict(
        chk=cases.checksum(q, docs, ql, dl),
        scores=ref.maxsim_padded_reference(T(q), T(docs), T(ql), T(dl)).numpy(),
        Q_packed=pk.Q_packed.numpy(), cu_q=pk.cu_seqlens_q.numpy(), D_packed=pk.D_packed.numpy(),
        cu_d=pk.cu_seqlens_d.numpy(), pair_q=pk.pair_q_idx.numpy(), pair_d=pk.pair_d_idx.numpy(),
        max_q=np.int64(pk.max_seqlen_q), max_d=np.int64(pk.max_seqlen_d),
    )

    # ---- FP8 quantisers (fp8.py:35-67) ---------------------------------------
    rng = np.random.default_rng(9)
    X = (rng.standard_normal((5, 7, 32)) * np.array([1e-3, 0.1, 1, 10, 300]).reshape(5, 1, 1)).astype(np.float32)
    X[0, 0] = 0.0
    xq, sc = rfp8.quantize_fp8_per_token(T(X))
    xq2, sc2 = rfp8.quantize_fp8_per_tensor(T(X))
    grid = np.linspace(-460, 460, 20001).astype(np.float32)
    out["fp8"] = dict(
        chk=cases.checksum(X), q_tok=xq.float().numpy(), s_tok=sc.numpy(), q_ten=xq2.float().numpy(), s_ten=sc2.numpy(),
        grid_q=T(grid).clamp(-448, 448).to(torch.float8_e4m3fn).float().numpy(),
        deq_tok=rfp8.dequantize_fp8_per_token(xq, sc).numpy(),
    )

    # ---- CPU retrieve (retrieve.py:254-310) ----------------------------------
    Q, D, dm = cases.retrieve_case(10)
    r = {"chk": cases.checksum(Q, D, dm)}
    for tag, kw in {
        "full": dict(top_k=5), "chunk4": dict(top_k=10, chunk=4), "chunk8_k50": dict(top_k=50, chunk=8),
        "nonorm": dict(top_k=7, chunk=16, normalize=False), "smallest": dict(top_k=6, chunk=5, largest=False),
    }.items():
        s, i = rret.retrieve(T(Q), T(D), d_mask=tb(dm), **kw)
        r[f"{tag}_s"], r[f"{tag}_i"] = s.numpy(), i.numpy()
    out["retrieve"] = r

    # ---- PLAID (reference.py:101-179) ----------------------------------------
    for nbits in (2, 4, 8):
        Q, codes, res, lens, cent, bw, _ = cases.plaid_case(11 + nbits, nbits=nbits)
        e = dict(chk=cases.checksum(Q, codes, res, lens, cent, bw))
        e["unpacked"] = ref.unpack_residuals_reference(T(res), nbits, Q.shape[-1]).numpy()
        for norm in (True, False):
            e[f"scores_norm{int(norm)}"] = ref.maxsim_residual_reference(
                T(Q), T(codes), T(res), T(lens), T(cent), T(bw), nbits, normalize=norm
            ).numpy()
        # grad_Q: autograd through dense unpack + maxsim (tests/test_plaid.py's ground truth)
        Qt = T(Q.astype(np.float64)).requires_grad_()
        emb = T(cent.astype(np.float64))[T(codes).long()] + T(bw.astype(np.float64))[T(e["unpacked"]).long()]
        emb = F.normalize(emb, dim=-1, eps=1e-12)
        dmask = torch.arange(codes.shape[1])[None] < T(lens)[:, None]
        s = ref.maxsim_reference(F.normalize(Qt, dim=-1, eps=1e-12), emb, None, dmask)
        g = np.random.default_rng(200 + nbits).standard_normal(tuple(s.shape))
        (s * T(g)).sum().backward()
        e["g"], e["gQ"] = g, Qt.grad.numpy()
        out[f"plaid_nbits{nbits}"] = e
    rng = np.random.default_rng(12)
    qcs = rng.standard_normal((40, 6)).astype(np.float32)
    codes = rng.integers(-2, 44, size=(7, 11)).astype(np.int32)  # some out of range -> centroid 0 in the kernel
    lens = np.array([0, 1, 11, 5, 7, 3, 11], dtype=np.int64)
    codes_ok = np.where((codes >= 0) & (codes < 40), codes, 0)
    out["plaid_approx"] = dict(
        chk=cases.checksum(qcs, codes, lens), scores=ref.plaid_approx_score_reference(T(qcs), T(codes_ok), T(lens)).numpy()
    )

    # ---- document head: projection + normalise + MaxSim (reference.py:182-210) and its autograd gradients ----
    Q, H, W, b, dm = cases.from_hidden_case(13)
    e = dict(chk=cases.checksum(Q, H, W, b, dm))
    for norm in (True, False):
        e[f"scores_norm{int(norm)}"] = ref.maxsim_from_hidden_reference(T(Q), T(H), T(W), T(b), tb(dm), normalize=norm).numpy()
    e["scores_nobias"] = ref.maxsim_from_hidden_reference(T(Q), T(H), T(W), None, tb(dm)).numpy()
    ts = [T(x.astype(np.float32)).requires_grad_() for x in (Q, H, W, b)]
    s = ref.maxsim_from_hidden_reference(ts[0], ts[1], ts[2], ts[3], tb(dm))
    # the reference promotes to fp32 inside; gradients are taken through that graph
    g = np.random.default_rng(213).standard_normal(tuple(s.shape)).astype(np.float32)
    (s * T(g)).sum().backward()
    e["g"] = g
    e["gQ"], e["gH"], e["gW"], e["gb"] = (t.grad.numpy() for t in ts)
    out["from_hidden"] = e

    for name, d in out.items():
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **{k: np.asarray(v) for k, v in d.items()})
        print(f"{name}: {sorted(d)}")


if __name__ == "__main__":
    main()
