"""CPU oracle for the MaxSim hot path (TEST INFRASTRUCTURE, not product code).

A numpy restatement of the reference project's pure-PyTorch ground truth
(``late_interaction_kernels/reference.py``) plus the parts of its GPU launchers
whose behaviour is part of the contract (argmax convention, backward math,
FP8 quantisation, top-k merge, PLAID bit layout).  Every function cites the
reference file:line it follows.

Only the test-suite, ``__graft_entry__.smoke()`` and the CPU-baseline leg of
``bench.py`` may import this module.  The shipped package never does: its
operators fail loudly when the CUDA library is missing.

Parity is pinned: ``tests/test_oracle_golden.py`` checks every function here
against vectors produced by the reference itself (``tests/golden/make_golden.py``
imports the reference and writes ``tests/golden/*.npz``).
"""

from __future__ import annotations

import numpy as np

NEG_INF = -np.inf


# --------------------------------------------------------------------------- #
# helpers                                                                     #
# --------------------------------------------------------------------------- #
def _f(x, dtype=None):
    """Promote to a float type: fp64 stays fp64, everything else becomes fp32
    (reference.py:62-71 promotes fp16/bf16 to fp32 and preserves fp64)."""
    x = np.asarray(x)
    if dtype is not None:
        return x.astype(dtype, copy=False)
    if x.dtype == np.float64:
        return x
    return x.astype(np.float32, copy=False)


def l2_normalize(x, eps=1e-12):
    """``F.normalize(x, p=2, dim=-1, eps)``: x / max(||x||, eps) (reference.py:72-74)."""
    x = _f(x)
    n = np.sqrt((x * x).sum(-1, keepdims=True))
    return x / np.maximum(n, x.dtype.type(eps))


def rel_err(actual, expected) -> float:
    """max|a-b| / max(1e-6, max|b|) — the reference's tolerance metric (tests/conftest.py:30-33)."""
    a = np.asarray(actual, dtype=np.float64)
    b = np.asarray(expected, dtype=np.float64)
    if a.size == 0:
        return 0.0
    return float(np.abs(a - b).max() / max(1e-6, np.abs(b).max()))


# --------------------------------------------------------------------------- #
# dense MaxSim (reference.py:26-98) with the argmax convention of the forward  #
# launcher (forward.py:128-183: -1 sentinel, lowest index wins ties)          #
# --------------------------------------------------------------------------- #
def maxsim(Q, D, q_mask=None, d_mask=None, *, normalize=False, return_argmax=False, q_chunk=16):
    """score[i,j] = sum_{s in q_mask[i]} max_{t in d_mask[j]} <Q[i,s], D[j,t]>.

    Follows reference.py:26-98: masked doc tokens get -inf before the max, a row
    whose max stays -inf contributes 0, masked query tokens contribute 0.
    ``return_argmax`` adds the int32 ``[Nq, Nd, Lq]`` winner table of
    forward.py:128-183 (-1 where no doc token is active).  Queries are
    processed ``q_chunk`` at a time so the [Nq,Nd,Lq,Ld] tensor never exists.
    """
    Q = _f(Q)
    D = _f(D)
    q2, d2 = Q.ndim == 2, D.ndim == 2
    if q2:
        Q = Q[None]
    if d2:
        D = D[None]
    if Q.shape[-1] != D.shape[-1]:
        raise ValueError(f"embedding dims don't match: Q has d={Q.shape[-1]}, D has d={D.shape[-1]}")
    if q_mask is not None:
        q_mask = np.asarray(q_mask).astype(bool)
        if q_mask.ndim == 1:
            q_mask = q_mask[None]
    if d_mask is not None:
        d_mask = np.asarray(d_mask).astype(bool)
        if d_mask.ndim == 1:
            d_mask = d_mask[None]
    if normalize:
        Q = l2_normalize(Q)
        D = l2_normalize(D)
    Nq, Lq, d = Q.shape
    Nd, Ld, _ = D.shape
    out_dt = np.result_type(Q.dtype, D.dtype)
    scores = np.zeros((Nq, Nd), dtype=out_dt)
    argmax = np.full((Nq, Nd, Lq), -1, dtype=np.int32) if return_argmax else None
    Dt = D.reshape(Nd * Ld, d).T
    for i0 in range(0, Nq, q_chunk):
        i1 = min(Nq, i0 + q_chunk)
        S = (Q[i0:i1].reshape(-1, d) @ Dt).reshape(i1 - i0, Lq, Nd, Ld)
        if d_mask is not None:
            S = np.where(d_mask[None, None, :, :], S, NEG_INF)
        m = S.max(-1) if Ld > 0 else np.full(S.shape[:-1], NEG_INF, dtype=S.dtype)
        finite = np.isfinite(m)
        if return_argmax and Ld > 0:
            am = S.argmax(-1).astype(np.int32)  # numpy argmax = first (lowest) index
            argmax[i0:i1] = np.where(finite, am, -1).transpose(0, 2, 1)
        m = np.where(finite, m, 0)
        if q_mask is not None:
            m = m * q_mask[i0:i1, :, None].astype(m.dtype)
        scores[i0:i1] = m.sum(1)
    if q2 and d2:
        scores = scores.reshape(())
    elif q2:
        scores = scores[0]
    elif d2:
        scores = scores[:, 0]
    if return_argmax:
        return scores, argmax
    return scores


def maxsim_kd(Q, D, q_mask=None, d_mask=None, *, normalize=False, return_argmax=False):
    """Per-query candidate lists: Q[Nq,Lq,d] x D[Nq,K,Ld,d] -> [Nq,K]
    (autograd.py:232-287 reshapes D to [Nq*K,Ld,d] and lets query i read slab i)."""
    Q = _f(Q)
    D = _f(D)
    Nq, K = D.shape[0], D.shape[1]
    scores = np.zeros((Nq, K), dtype=np.result_type(Q.dtype, D.dtype))
    argmax = np.full((Nq, K, Q.shape[1]), -1, dtype=np.int32)
    for i in range(Nq):
        r = maxsim(
            Q[i : i + 1],
            D[i],
            None if q_mask is None else np.asarray(q_mask)[i : i + 1],
            None if d_mask is None else np.asarray(d_mask)[i],
            normalize=normalize,
            return_argmax=True,
        )
        scores[i], argmax[i] = r[0][0], r[1][0]
    return (scores, argmax) if return_argmax else scores


def maxsim_pairs(Q, D, q_mask=None, d_mask=None, *, normalize=False):
    """Diagonal scoring: the K=1 case of the KD layout (autograd.py:462-501)."""
    D = np.asarray(D)
    dm = None if d_mask is None else np.asarray(d_mask)[:, None]
    return maxsim_kd(Q, D[:, None], q_mask, dm, normalize=normalize)[:, 0]


# --------------------------------------------------------------------------- #
# packed layouts (reference.py:213-306)                                       #
# --------------------------------------------------------------------------- #
def _pair_score(qi, dj, want_argmax=False):
    """One (query, doc) pair on already-sliced token matrices; empty side -> 0."""
    if qi.shape[0] == 0 or dj.shape[0] == 0:
        return (0.0, np.full(qi.shape[0], -1, np.int32)) if want_argmax else 0.0
    S = _f(qi) @ _f(dj).T
    if want_argmax:
        return S.max(-1).sum(), S.argmax(-1).astype(np.int32)
    return S.max(-1).sum()


def maxsim_varlen(Q, D, cu_q, cu_d, *, return_argmax=False):
    """Packed inputs: Q [sum Lq, d], D [sum Ld, d], cumulative offsets (reference.py:213-245).
    Argmax follows varlen.py:327-331: int32 [Nq, Nd, max_lq] filled with -1."""
    cu_q = np.asarray(cu_q).astype(np.int64)
    cu_d = np.asarray(cu_d).astype(np.int64)
    Nq, Nd = len(cu_q) - 1, len(cu_d) - 1
    out = np.zeros((Nq, Nd), dtype=np.float32)
    max_lq = int((cu_q[1:] - cu_q[:-1]).max()) if Nq else 0
    am = np.full((Nq, Nd, max_lq), -1, dtype=np.int32)
    for i in range(Nq):
        qi = Q[cu_q[i] : cu_q[i + 1]]
        for j in range(Nd):
            s, a = _pair_score(qi, D[cu_d[j] : cu_d[j + 1]], True)
            out[i, j] = s
            am[i, j, : len(a)] = a
    return (out, am) if return_argmax else out


def maxsim_pair_list(Q, D, cu_q, cu_d, pair_q, pair_d, *, return_argmax=False):
    """Arbitrary (query, doc) pair list on packed inputs (reference.py:248-270)."""
    cu_q = np.asarray(cu_q).astype(np.int64)
    cu_d = np.asarray(cu_d).astype(np.int64)
    P = len(pair_q)
    out = np.zeros(P, dtype=np.float32)
    max_lq = int((cu_q[1:] - cu_q[:-1]).max()) if len(cu_q) > 1 else 0
    am = np.full((P, max_lq), -1, dtype=np.int32)
    for k in range(P):
        i, j = int(pair_q[k]), int(pair_d[k])
        s, a = _pair_score(Q[cu_q[i] : cu_q[i + 1]], D[cu_d[j] : cu_d[j + 1]], True)
        out[k] = s
        am[k, : len(a)] = a
    return (out, am) if return_argmax else out


def maxsim_padded(queries, documents, query_lengths, doc_lengths):
    """Padded reranking batch [B,Lq,d] x [B,C,Ld,d] with lengths -> [B,C] fp32 (reference.py:273-306)."""
    B, C = documents.shape[0], documents.shape[1]
    out = np.zeros((B, C), dtype=np.float32)
    for b in range(B):
        q = queries[b, : int(query_lengths[b])]
        for c in range(C):
            out[b, c] = _pair_score(q, documents[b, c, : int(doc_lengths[b][c])])
    return out


def pack_padded(queries, documents, query_lengths, doc_lengths):
    """Padded -> packed conversion (padded.py:77-208): row-major (b,c) doc order,
    pair_q_idx[b*C+c] = b, pair_d_idx[b*C+c] = b*C+c, int32 offsets."""
    B, Lq, d = queries.shape
    _, C, Ld, _ = documents.shape
    ql = np.asarray(query_lengths).astype(np.int64)
    dl = np.asarray(doc_lengths).astype(np.int64).reshape(-1)
    Qp = np.concatenate([queries[b, : ql[b]] for b in range(B)] or [queries.reshape(0, d)])
    docs = documents.reshape(B * C, Ld, d)
    Dp = np.concatenate([docs[k, : dl[k]] for k in range(B * C)] or [documents.reshape(0, d)])
    cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    cu_d = np.concatenate([[0], np.cumsum(dl)]).astype(np.int32)
    flat = np.arange(B * C, dtype=np.int32)
    return Qp, cu_q, Dp, cu_d, (flat // max(C, 1)).astype(np.int32), flat, int(ql.max(initial=0)), int(dl.max(initial=0))


# --------------------------------------------------------------------------- #
# backward (backward/unified.py:27-85; Jacobian autograd.py:213-225)           #
# --------------------------------------------------------------------------- #
def backward_from_argmax(grad_scores, Q, D, argmax, q_mask=None, *, kd_layout=False):
    """grad_Q[i,s] = sum_j g[i,j] D[j, t*];  grad_D[j,t*] += g[i,j] Q[i,s], t* = argmax[i,j,s].

    Winners < 0 (fully masked doc) and masked query tokens contribute nothing
    (backward/unified.py:149-157, 170-196).  ``kd_layout``: D is [Nq*K, Ld, d]
    and pair (i,k) reads doc i*K+k.  Returns fp64 grads.
    """
    Q = np.asarray(Q, dtype=np.float64)
    D = np.asarray(D, dtype=np.float64)
    g = np.asarray(grad_scores, dtype=np.float64)
    Nq, Lq, d = Q.shape
    K = g.shape[1]
    am = np.asarray(argmax).reshape(Nq, K, Lq)
    gQ = np.zeros_like(Q)
    gD = np.zeros_like(D)
    qm = np.ones((Nq, Lq), bool) if q_mask is None else np.asarray(q_mask).astype(bool)
    for i in range(Nq):
        for k in range(K):
            j = i * K + k if kd_layout else k
            t = am[i, k]
            act = (t >= 0) & qm[i]
            if not act.any():
                continue
            s_idx = np.nonzero(act)[0]
            gQ[i, s_idx] += g[i, k] * D[j, t[s_idx]]
            np.add.at(gD[j], t[s_idx], g[i, k] * Q[i, s_idx])
    return gQ, gD


def normalize_jacobian(grad_hat, X, eps=1e-6):
    """Pull a gradient w.r.t. x/||x|| back to x: (g - <g,xh> xh)/||x|| with
    ||x|| clamped at 1e-6 (autograd.py:218-225)."""
    X = np.asarray(X, dtype=np.float64)
    n = np.maximum(np.sqrt((X * X).sum(-1, keepdims=True)), eps)
    xh = X / n
    return (grad_hat - (grad_hat * xh).sum(-1, keepdims=True) * xh) / n


def maxsim_grads(grad_scores, Q, D, q_mask=None, d_mask=None, *, normalize=False, kd_layout=False):
    """Gradients of ``sum(grad_scores * maxsim(...))`` w.r.t. Q and D in fp64 —
    what autograd through reference.py:26-98 gives when winners are unique."""
    Q64 = np.asarray(Q, dtype=np.float64)
    D64 = np.asarray(D, dtype=np.float64)
    Dflat = D64.reshape(-1, D64.shape[-2], D64.shape[-1]) if kd_layout else D64
    if normalize:
        Qh, Dh = l2_normalize(Q64, 1e-12), l2_normalize(Dflat, 1e-12)
    else:
        Qh, Dh = Q64, Dflat
    if kd_layout:
        K = D64.shape[1]
        dm = None if d_mask is None else np.asarray(d_mask).reshape(Q64.shape[0], K, -1)
        _, am = maxsim_kd(Qh, Dh.reshape(Q64.shape[0], K, *Dh.shape[1:]), q_mask, dm, return_argmax=True)
    else:
        _, am = maxsim(Qh, Dh, q_mask, d_mask, return_argmax=True)
    gQ, gD = backward_from_argmax(grad_scores, Qh, Dh, am, q_mask, kd_layout=kd_layout)
    if normalize:
        gQ = normalize_jacobian(gQ, Q64)
        gD = normalize_jacobian(gD, Dflat)
    return gQ, gD.reshape(D64.shape)


def varlen_grads(grad_scores, Q, D, cu_q, cu_d):
    """Packed-layout gradients (varlen.py:141-263): same gather/scatter on packed rows."""
    Q64 = np.asarray(Q, dtype=np.float64)
    D64 = np.asarray(D, dtype=np.float64)
    g = np.asarray(grad_scores, dtype=np.float64)
    gQ, gD = np.zeros_like(Q64), np.zeros_like(D64)
    cu_q = np.asarray(cu_q).astype(np.int64)
    cu_d = np.asarray(cu_d).astype(np.int64)
    for i in range(len(cu_q) - 1):
        qi = Q64[cu_q[i] : cu_q[i + 1]]
        for j in range(len(cu_d) - 1):
            dj = D64[cu_d[j] : cu_d[j + 1]]
            if qi.shape[0] == 0 or dj.shape[0] == 0:
                continue
            t = (qi @ dj.T).argmax(-1)
            gQ[cu_q[i] : cu_q[i + 1]] += g[i, j] * dj[t]
            np.add.at(gD[cu_d[j] : cu_d[j + 1]], t, g[i, j] * qi)
    return gQ, gD


def pair_list_grads(grad_out, Q, D, cu_q, cu_d, pair_q, pair_d):
    """Pair-list gradients (score_pairs.py:148-273)."""
    Q64 = np.asarray(Q, dtype=np.float64)
    D64 = np.asarray(D, dtype=np.float64)
    g = np.asarray(grad_out, dtype=np.float64)
    gQ, gD = np.zeros_like(Q64), np.zeros_like(D64)
    cu_q = np.asarray(cu_q).astype(np.int64)
    cu_d = np.asarray(cu_d).astype(np.int64)
    for k in range(len(pair_q)):
        i, j = int(pair_q[k]), int(pair_d[k])
        qi = Q64[cu_q[i] : cu_q[i + 1]]
        dj = D64[cu_d[j] : cu_d[j + 1]]
        if qi.shape[0] == 0 or dj.shape[0] == 0:
            continue
        t = (qi @ dj.T).argmax(-1)
        gQ[cu_q[i] : cu_q[i + 1]] += g[k] * dj[t]
        np.add.at(gD[cu_d[j] : cu_d[j + 1]], t, g[k] * qi)
    return gQ, gD


# --------------------------------------------------------------------------- #
# FP8 e4m3 (fp8.py:33-67)                                                      #
# --------------------------------------------------------------------------- #
E4M3_MAX = 448.0


def round_to_e4m3(x):
    """Round fp32 values to the nearest float8_e4m3fn value (ties to even),
    returned as fp32.  Inputs are expected inside [-448, 448] as after the
    clamp of fp8.py:47, 60."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    e = np.floor(np.log2(np.maximum(a, 1e-300)))
    e = np.clip(e, -6, 8)  # normal exponents -6..8; below 2^-6 the step stays 2^-9
    step = np.exp2(e - 3)
    q = np.round(a / step) * step  # np.round = half-to-even
    q = np.minimum(q, E4M3_MAX)
    return (np.sign(x) * q).astype(np.float32)


def quantize_fp8_per_token(X):
    """scale = max(amax|x|, 1e-6)/448 per row; q = e4m3(clamp(x/scale)) (fp8.py:52-61).
    Returns (q as fp32 holding exact e4m3 values, scale fp32 [..])."""
    X = np.asarray(X, dtype=np.float32)
    amax = np.maximum(np.abs(X).max(-1), np.float32(1e-6)).astype(np.float32)
    scale = (amax / np.float32(E4M3_MAX)).astype(np.float32)
    q = np.clip(X / scale[..., None], -E4M3_MAX, E4M3_MAX)
    return round_to_e4m3(q), scale


def quantize_fp8_per_tensor(X):
    """One scale for the whole tensor (fp8.py:35-49)."""
    X = np.asarray(X, dtype=np.float32)
    if X.size == 0:
        return X.copy(), np.float32(1.0)
    amax = np.maximum(np.abs(X).max(), np.float32(1e-6)).astype(np.float32)
    scale = np.float32(amax / np.float32(E4M3_MAX))
    return round_to_e4m3(np.clip(X / scale, -E4M3_MAX, E4M3_MAX)), scale


def dequantize_fp8(Xq, scale):
    """x = q * scale, per-tensor (0-d scale) or per-token (fp8.py:64-67)."""
    scale = np.asarray(scale, dtype=np.float32)
    Xq = np.asarray(Xq, dtype=np.float32)
    return Xq * (scale[..., None] if scale.ndim else scale)


def maxsim_fp8(Qq, Dq, scale_Q, scale_D, q_mask=None, d_mask=None):
    """FP8 scoring = dequantise then dense MaxSim in fp32 (fp8.py:186-204 applies
    the same scales to the score tile)."""
    return maxsim(dequantize_fp8(Qq, scale_Q), dequantize_fp8(Dq, scale_D), q_mask, d_mask)


# --------------------------------------------------------------------------- #
# top-k retrieval (retrieve.py:254-310, topk.py:41-86)                         #
# --------------------------------------------------------------------------- #
def topk_rows(scores, k, largest=True):
    """Row-wise top-k, sorted, ties broken by lower index (a stable refinement of
    ``torch.topk`` which leaves tie order unspecified)."""
    s = np.asarray(scores)
    key = -s if largest else s
    idx = np.argsort(key, axis=-1, kind="stable")[..., :k]
    return np.take_along_axis(s, idx, -1), idx.astype(np.int64)


def retrieve(Q, D, top_k, q_mask=None, d_mask=None, *, normalize=True, chunk=None, largest=True):
    """Chunked score + running top-k merge (retrieve.py:254-310).  Returns
    (fp32 [Nq,k], int64 [Nq,k]); k = min(top_k, Nd)."""
    if top_k <= 0:
        raise ValueError(f"top_k must be positive, got {top_k}")
    Q = np.asarray(Q)
    D = np.asarray(D)
    q2 = Q.ndim == 2
    if q2:
        Q = Q[None]
    if D.ndim == 2:
        D = D[None]
    Nd = D.shape[0]
    k = min(top_k, Nd)
    if chunk is None or chunk >= Nd:
        s = maxsim(Q, D, q_mask, d_mask, normalize=normalize)
        ts, ti = topk_rows(s, k, largest)
    else:
        ts = ti = None
        for st in range(0, Nd, chunk):
            en = min(st + chunk, Nd)
            dm = None if d_mask is None else np.asarray(d_mask)[st:en]
            s = maxsim(Q, D[st:en], q_mask, dm, normalize=normalize)
            cs, ci = topk_rows(s, min(k, en - st), largest)
            ci = ci + st
            if ts is None:
                ts, ti = cs, ci
            else:
                ms, mi = np.concatenate([ts, cs], -1), np.concatenate([ti, ci], -1)
                ts, sel = topk_rows(ms, min(k, ms.shape[-1]), largest)
                ti = np.take_along_axis(mi, sel, -1)
    ts = ts.astype(np.float32)
    return (ts[0], ti[0]) if q2 else (ts, ti)


# --------------------------------------------------------------------------- #
# PLAID (reference.py:101-179)                                                 #
# --------------------------------------------------------------------------- #
def unpack_residuals(residuals, nbits, d):
    """Feature f sits in byte f // (8/nbits) at bit offset (f % (8/nbits))*nbits,
    little-endian inside the byte (reference.py:124-139).  int32 [..., d]."""
    cpb = 8 // nbits
    r = np.asarray(residuals).astype(np.int32)
    f = np.arange(d)
    return (r[..., f // cpb] >> ((f % cpb) * nbits)) & ((1 << nbits) - 1)


def pack_residuals(bucket_codes, nbits):
    """Inverse of :func:`unpack_residuals` (tests/test_reference_cpu.py round trip)."""
    cpb = 8 // nbits
    b = np.asarray(bucket_codes).astype(np.int64)
    d = b.shape[-1]
    pd = (d * nbits + 7) // 8
    out = np.zeros(b.shape[:-1] + (pd,), dtype=np.int64)
    for f in range(d):
        out[..., f // cpb] |= b[..., f] << ((f % cpb) * nbits)
    return out.astype(np.uint8)


def plaid_decompress(codes, residuals, centroids, bucket_weights, nbits, *, normalize=True):
    """emb = centroids[code] + bucket_weights[bucket]; optional L2 norm (reference.py:164-171)."""
    cent = _f(centroids, np.float32)
    bw = _f(bucket_weights, np.float32)
    d = cent.shape[-1]
    bc = np.clip(unpack_residuals(residuals, nbits, d), 0, bw.size - 1)
    emb = cent[np.asarray(codes).astype(np.int64)] + bw[bc]
    return l2_normalize(emb) if normalize else emb


def maxsim_residual(Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, *, normalize=True, return_argmax=False):
    """Padded PLAID decompress + MaxSim -> [Nq, Nd] (reference.py:142-179)."""
    Q = _f(Q, np.float32)
    q2 = Q.ndim == 2
    if q2:
        Q = Q[None]
    emb = plaid_decompress(codes, residuals, centroids, bucket_weights, nbits, normalize=normalize)
    Qn = l2_normalize(Q) if normalize else Q
    Ld = np.asarray(codes).shape[1]
    d_mask = np.arange(Ld)[None, :] < np.asarray(doc_lengths).astype(np.int64)[:, None]
    r = maxsim(Qn, emb, None, d_mask, return_argmax=return_argmax)
    if return_argmax:
        return (r[0][0], r[1][0]) if q2 else r
    return r[0] if q2 else r


def maxsim_residual_varlen(Q, codes_flat, residuals_flat, cu_d, centroids, bucket_weights, nbits, *, normalize=True):
    """Ragged PLAID scoring (plaid.py:832-963): same math on concatenated docs; empty doc -> 0."""
    Q = _f(Q, np.float32)
    q2 = Q.ndim == 2
    if q2:
        Q = Q[None]
    emb = plaid_decompress(codes_flat, residuals_flat, centroids, bucket_weights, nbits, normalize=normalize)
    Qn = l2_normalize(Q) if normalize else Q
    cu_d = np.asarray(cu_d).astype(np.int64)
    Nq, Nd = Q.shape[0], len(cu_d) - 1
    out = np.zeros((Nq, Nd), dtype=np.float32)
    for j in range(Nd):
        dj = emb[cu_d[j] : cu_d[j + 1]]
        if dj.shape[0]:
            out[:, j] = np.einsum("isd,td->ist", Qn, dj).max(-1).sum(-1)
    return out[0] if q2 else out


def plaid_approx_score(qcs, codes, doc_lengths):
    """sum_s max_{t < len} qcs[codes[b,t], s]; empty doc -> 0 (reference.py:101-121).
    Out-of-range codes read centroid 0 (plaid.py:64-66)."""
    qcs = _f(qcs, np.float32)
    codes = np.asarray(codes).astype(np.int64)
    codes = np.where((codes >= 0) & (codes < qcs.shape[0]), codes, 0)
    B, Ld = codes.shape
    g = qcs[codes.reshape(-1)].reshape(B, Ld, -1)
    mask = np.arange(Ld)[None, :] < np.asarray(doc_lengths).astype(np.int64)[:, None]
    g = np.where(mask[..., None], g, NEG_INF)
    m = g.max(1) if Ld else np.full((B, qcs.shape[1]), NEG_INF, np.float32)
    return np.where(np.isfinite(m), m, 0).sum(-1).astype(np.float32)


def residual_grad_q(grad_scores, Q, codes, residuals, doc_lengths, centroids, bucket_weights, nbits, *, normalize=True):
    """grad wrt Q of maxsim_residual (plaid.py:310-401, 596-605): gather the winning
    reconstructed token, then the Q-side normalise Jacobian."""
    Q64 = np.asarray(Q, dtype=np.float64)
    emb = plaid_decompress(codes, residuals, centroids, bucket_weights, nbits, normalize=normalize).astype(np.float64)
    Qn = l2_normalize(Q64, 1e-12) if normalize else Q64
    Ld = np.asarray(codes).shape[1]
    d_mask = np.arange(Ld)[None, :] < np.asarray(doc_lengths).astype(np.int64)[:, None]
    _, am = maxsim(Qn, emb, None, d_mask, return_argmax=True)
    gQ, _ = backward_from_argmax(grad_scores, Qn, emb, am)
    return normalize_jacobian(gQ, Q64) if normalize else gQ


# --------------------------------------------------------------------------- #
# document head (reference.py:182-210)                                        #
# --------------------------------------------------------------------------- #
def maxsim_from_hidden(Q, H_d, W, b=None, d_mask=None, *, normalize=True):
    """D = H_d W^T (+ b) in fp32, optional L2 norm (eps 1e-12), then MaxSim against Q (reference.py:182-210)."""
    H = _f(H_d, np.float32)
    D = H @ _f(W, np.float32).T
    if b is not None:
        D = D + _f(b, np.float32)
    if normalize:
        D = l2_normalize(D)
    return maxsim(Q, D, None, d_mask)


def from_hidden_grads(grad_scores, Q, H_d, W, b=None, d_mask=None, *, normalize=True):
    """Gradients of maxsim_from_hidden w.r.t. (Q, H_d, W, b) in fp64: MaxSim backward onto the projected tokens,
    the normalise Jacobian (norm clamped at 1e-12, as F.normalize differentiates), then the linear layer."""
    Q64, H64, W64 = (np.asarray(x, dtype=np.float64) for x in (Q, H_d, W))
    P = H64 @ W64.T + (0 if b is None else np.asarray(b, dtype=np.float64))
    D = l2_normalize(P, 1e-12) if normalize else P
    _, am = maxsim(Q64, D, None, d_mask, return_argmax=True)
    gQ, gD = backward_from_argmax(grad_scores, Q64, D, am)
    gP = normalize_jacobian(gD, P, eps=1e-12) if normalize else gD
    gH = gP @ W64
    gW = np.einsum("jto,jtm->om", gP, H64)
    gb = gP.sum((0, 1))
    return gQ, gH, gW, gb


# --------------------------------------------------------------------------- #
# PLAID candidate generation (PARITY UNPINNED: the reference ships the scoring #
# kernels only; these stages live in fast-plaid, which is not in the reference #
# tree.  Restated from the published algorithm, Santhanam et al. 2022, and     #
# anchored on the reference's own reader of the index files,                   #
# benchmarks/plaid/bench_fastplaid_e2e.py:76-140.)                             #
# --------------------------------------------------------------------------- #
def plaid_ivf(codes_flat, cu_d, n_centroids):
    """Inverted file: for every centroid the ascending documents with a token on it -> (docs, offsets)."""
    cu_d = np.asarray(cu_d).astype(np.int64)
    nd = len(cu_d) - 1
    tok_doc = np.repeat(np.arange(nd), cu_d[1:] - cu_d[:-1])
    codes = np.clip(np.asarray(codes_flat).astype(np.int64), 0, n_centroids - 1)
    key = np.unique(codes * max(nd, 1) + tok_doc)
    cent = key // max(nd, 1)
    offsets = np.zeros(n_centroids + 1, np.int64)
    offsets[1:] = np.cumsum(np.bincount(cent, minlength=n_centroids))
    return (key - cent * max(nd, 1)).astype(np.int32), offsets


def plaid_search(Q, codes_flat, residuals_flat, cu_d, centroids, bucket_weights, nbits, top_k, *, nprobe=4, ndocs=4096,
                 normalize=True, qcs=None):
    """Three-stage PLAID search of one query [Lq, d]: probe the nprobe best centroids per query token, score the
    candidates approximately from their codes, rerank the ndocs best exactly.  Ties go to the lower index at every
    selection.  ``qcs`` ([n_centroids, Lq]) may be passed in so that a test feeds both sides the same centroid scores.
    Returns (scores [k], document ids [k])."""
    Q = _f(Q, np.float32)
    cent = _f(centroids, np.float32)
    cu_d = np.asarray(cu_d).astype(np.int64)
    lens = cu_d[1:] - cu_d[:-1]
    Qn = l2_normalize(Q) if normalize else Q
    if qcs is None:
        qcs = cent @ Qn.T
    ivf_docs, ivf_off = plaid_ivf(codes_flat, cu_d, cent.shape[0])
    probe = min(nprobe, cent.shape[0])
    cid = np.unique(topk_rows(np.asarray(qcs).T, probe)[1])
    cand = np.unique(np.concatenate([ivf_docs[ivf_off[c]:ivf_off[c + 1]] for c in cid]).astype(np.int64)) if len(cid) else np.zeros(0, np.int64)
    if cand.size == 0:
        return np.zeros(0, np.float32), np.zeros(0, np.int64)
    if cand.size > ndocs:
        max_ld = int(lens[cand].max())
        pad = np.zeros((cand.size, max_ld), np.int64)
        for n, j in enumerate(cand):
            pad[n, : lens[j]] = np.asarray(codes_flat)[cu_d[j]:cu_d[j + 1]]
        approx = plaid_approx_score(qcs, pad, lens[cand])
        keep = np.sort(topk_rows(approx[None], ndocs)[1][0])
        cand = cand[keep]
    sub_c = np.concatenate([np.asarray(codes_flat)[cu_d[j]:cu_d[j + 1]] for j in cand])
    sub_r = np.concatenate([np.asarray(residuals_flat)[cu_d[j]:cu_d[j + 1]] for j in cand])
    sub_cu = np.concatenate([[0], np.cumsum(lens[cand])])
    full = maxsim_residual_varlen(Q, sub_c, sub_r, sub_cu, centroids, bucket_weights, nbits, normalize=normalize)
    ts, ti = topk_rows(full[None], min(top_k, cand.size))
    return ts[0].astype(np.float32), cand[ti[0]]


# --------------------------------------------------------------------------- #
# sharded retrieval merge (the build's own multi-GPU step; no reference twin) #
# --------------------------------------------------------------------------- #
def merge_topk(cand_scores, cand_idx, k, largest=True):
    """Merge candidate lists [..., n] -> top-k by (score desc, index asc); entries
    with index < 0 are padding and never win."""
    s = np.asarray(cand_scores, dtype=np.float32)
    i = np.asarray(cand_idx, dtype=np.int64)
    bad = i < 0
    key = np.where(bad, np.inf, -s if largest else s)
    order = np.lexsort((np.where(bad, np.iinfo(np.int64).max, i), key), axis=-1)[..., :k]
    return np.take_along_axis(s, order, -1), np.take_along_axis(i, order, -1)
