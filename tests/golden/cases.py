"""Seeded input generators shared by ``make_golden.py`` (which feeds them to the
reference) and by the tests (which feed them to the oracle and the CUDA path).

Inputs come from ``numpy.random.default_rng(seed)`` so they can be rebuilt
anywhere; every golden file also stores a checksum of its inputs so a drift in
the generator is detected instead of silently comparing different data.
"""

from __future__ import annotations

import numpy as np


def checksum(*arrays) -> float:
    """Order-sensitive fp64 checksum of a list of arrays."""
    tot = 0.0
    for k, a in enumerate(arrays):
        a = np.asarray(a, dtype=np.float64).reshape(-1)
        tot += float((a * (1.0 + (np.arange(a.size) % 7))).sum()) * (k + 1)
    return tot


def prefix_mask(lengths, L):
    return np.arange(L)[None, :] < np.asarray(lengths)[..., None]


def unit(x):
    return x / np.maximum(np.linalg.norm(x, axis=-1, keepdims=True), 1e-12)


def dense_case(seed, Nq, Nd, Lq, Ld, d, *, q_len=None, d_len=None, normalized=False, dtype=np.float32):
    """Q[Nq,Lq,d], D[Nd,Ld,d] ~ N(0,1); optional prefix masks with lengths U[lo,hi]."""
    rng = np.random.default_rng(seed)
    Q = rng.standard_normal((Nq, Lq, d)).astype(dtype)
    D = rng.standard_normal((Nd, Ld, d)).astype(dtype)
    if normalized:
        Q, D = unit(Q).astype(dtype), unit(D).astype(dtype)
    qm = dm = None
    if q_len is not None:
        qm = prefix_mask(rng.integers(q_len[0], q_len[1] + 1, size=Nq), Lq)
    if d_len is not None:
        dm = prefix_mask(rng.integers(d_len[0], d_len[1] + 1, size=Nd), Ld)
    return Q, D, qm, dm


def config1():
    """The small fp32 configuration: fp32 Q[32,32,128], D[32,180,128], normalize=True,
    q lengths U[8,32], d lengths U[32,180]."""
    return dense_case(0, 32, 32, 32, 180, 128, q_len=(8, 32), d_len=(32, 180))


def random_mask_case(seed, Nq=3, Nd=5, Lq=7, Ld=19, d=16):
    """Arbitrary (non-prefix) boolean masks, one fully masked doc and one fully masked query."""
    rng = np.random.default_rng(seed)
    Q = rng.standard_normal((Nq, Lq, d)).astype(np.float32)
    D = rng.standard_normal((Nd, Ld, d)).astype(np.float32)
    qm = rng.random((Nq, Lq)) > 0.3
    dm = rng.random((Nd, Ld)) > 0.4
    dm[1] = False
    qm[2] = False
    qm[0, 0] = True
    dm[0, 0] = True
    return Q, D, qm, dm


def kd_case(seed, Nq=4, K=3, Lq=6, Ld=11, d=16, masks=True):
    rng = np.random.default_rng(seed)
    Q = rng.standard_normal((Nq, Lq, d)).astype(np.float32)
    D = rng.standard_normal((Nq, K, Ld, d)).astype(np.float32)
    qm = dm = None
    if masks:
        qm = prefix_mask(rng.integers(1, Lq + 1, size=Nq), Lq)
        dm = prefix_mask(rng.integers(1, Ld + 1, size=(Nq, K)), Ld)
    return Q, D, qm, dm


def varlen_case(seed, Nq=5, Nd=6, lq=(1, 9), ld=(0, 17), d=16, dtype=np.float32, normalized=False):
    """Packed layout with an empty document (and lengths from U[lo,hi])."""
    rng = np.random.default_rng(seed)
    ql = rng.integers(lq[0], lq[1] + 1, size=Nq)
    dl = rng.integers(ld[0], ld[1] + 1, size=Nd)
    if ld[0] == 0:
        dl[Nd // 2] = 0
    Q = rng.standard_normal((int(ql.sum()), d)).astype(dtype)
    D = rng.standard_normal((int(dl.sum()), d)).astype(dtype)
    if normalized:
        Q, D = unit(Q).astype(dtype), unit(D).astype(dtype)
    cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    cu_d = np.concatenate([[0], np.cumsum(dl)]).astype(np.int32)
    return Q, D, cu_q, cu_d


def pair_list_case(seed, n_pairs=9, **kw):
    Q, D, cu_q, cu_d = varlen_case(seed, **kw)
    rng = np.random.default_rng(seed + 1000)
    pq = rng.integers(0, len(cu_q) - 1, size=n_pairs).astype(np.int32)
    pd = rng.integers(0, len(cu_d) - 1, size=n_pairs).astype(np.int32)
    return Q, D, cu_q, cu_d, pq, pd


def padded_case(seed, B=3, C=4, Lq=8, Ld=13, d=16):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, Lq, d)).astype(np.float32)
    docs = rng.standard_normal((B, C, Ld, d)).astype(np.float32)
    ql = rng.integers(1, Lq + 1, size=B).astype(np.int64)
    dl = rng.integers(1, Ld + 1, size=(B, C)).astype(np.int64)
    return q, docs, ql, dl


def plaid_case(seed, Nq=3, Nd=5, Lq=6, Ld=14, d=32, nbits=2, n_centroids=64):
    """PLAID index: codes, packed residual bytes, fp16 centroids, linspace buckets
    (the reference's own test setup, tests/test_plaid.py:23)."""
    rng = np.random.default_rng(seed)
    Q = rng.standard_normal((Nq, Lq, d)).astype(np.float32)
    codes = rng.integers(0, n_centroids, size=(Nd, Ld)).astype(np.int32)
    pd = (d * nbits + 7) // 8
    residuals = rng.integers(0, 256, size=(Nd, Ld, pd)).astype(np.uint8)
    lens = rng.integers(1, Ld + 1, size=Nd).astype(np.int64)
    centroids = unit(rng.standard_normal((n_centroids, d))).astype(np.float16)
    buckets = np.linspace(-0.1, 0.1, 2**nbits).astype(np.float32)
    return Q, codes, residuals, lens, centroids, buckets, nbits


def retrieve_case(seed, Nq=4, Nd=37, Lq=5, Ld=9, d=16):
    rng = np.random.default_rng(seed)
    Q = rng.standard_normal((Nq, Lq, d)).astype(np.float32)
    D = rng.standard_normal((Nd, Ld, d)).astype(np.float32)
    dm = prefix_mask(rng.integers(1, Ld + 1, size=Nd), Ld)
    return Q, D, dm


def from_hidden_case(seed, Nq=3, Nd=5, Lq=6, Ld=11, d_model=24, d_out=16):
    """Document hidden states with a projection head: Q[Nq,Lq,d_out], H[Nd,Ld,d_model], W[d_out,d_model], b[d_out]."""
    rng = np.random.default_rng(seed)
    Q = unit(rng.standard_normal((Nq, Lq, d_out))).astype(np.float32)
    H = rng.standard_normal((Nd, Ld, d_model)).astype(np.float32)
    W = (rng.standard_normal((d_out, d_model)) / np.sqrt(d_model)).astype(np.float32)
    b = (0.1 * rng.standard_normal(d_out)).astype(np.float32)
    dm = prefix_mask(rng.integers(1, Ld + 1, size=Nd), Ld)
    return Q, H, W, b, dm
