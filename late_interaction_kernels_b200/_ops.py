"""Thin launch layer between the public API modules and the C ABI.

Everything here takes torch CUDA tensors, allocates outputs / workspaces with
torch (so the caching allocator and CUDA-graph capture keep working), fills the
argument structs of ``include/lik_b200.h`` and calls the library on the current
stream.  No arithmetic happens in Python.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import BwdArgs, FwdArgs, HiddenFwdArgs, PlaidIndex, Seqs, TopkSpec

# The launchers hand raw pointers to a C library: keep torch.compile from tracing into them (it
# breaks the graph around the call instead).
_no_trace = getattr(getattr(torch, "compiler", None), "disable", None) or (lambda f: f)


@dataclass
class SeqSpec:
    """One side of a MaxSim problem (mirrors ``lik_seqs``)."""

    data: torch.Tensor  # [n_rows, dim], last dim contiguous
    n_seq: int
    max_len: int
    seq_stride: int = 0
    cu: torch.Tensor | None = None  # int32 [n_seq + 1]
    lens: torch.Tensor | None = None  # int32 [n_seq]
    mask: torch.Tensor | None = None  # uint8 [n_rows]
    scale: torch.Tensor | None = None  # fp32 [n_rows]
    scale_scalar: float = 1.0

    def c_struct(self) -> Seqs:
        d = self.data
        return Seqs(
            data=d.data_ptr() if d.numel() else None,
            row_stride=d.stride(0) if d.shape[0] > 0 else d.shape[1],
            n_rows=d.shape[0],
            n_seq=self.n_seq,
            max_len=self.max_len,
            seq_stride=self.seq_stride,
            cu=_lib.ptr(self.cu),
            lens=_lib.ptr(self.lens),
            mask=_lib.ptr(self.mask),
            scale=_lib.ptr(self.scale),
            scale_scalar=float(self.scale_scalar),
            reserved=0,
        )


def _as_u8_mask(mask: torch.Tensor | None) -> torch.Tensor | None:
    if mask is None:
        return None
    m = mask.contiguous()
    if m.dtype == torch.bool:
        return m.view(torch.uint8)
    if m.dtype in (torch.uint8, torch.int8):
        return m.view(torch.uint8)
    return (m != 0).view(torch.uint8)


def padded_spec(x: torch.Tensor, mask=None, lens=None, scale=None, scale_scalar=1.0) -> SeqSpec:
    """[N, L, d] tensor -> padded SeqSpec (copies only if not contiguous)."""
    x = x.contiguous()
    N, L, d = x.shape
    m = _as_u8_mask(mask)
    if m is not None:
        m = m.reshape(-1)
    if lens is not None:
        lens = lens.to(device=x.device, dtype=torch.int32).contiguous()
    if scale is not None:
        scale = scale.to(device=x.device, dtype=torch.float32).contiguous().reshape(-1)
    return SeqSpec(x.view(N * L, d), N, L, L, None, lens, m, scale, scale_scalar)


def packed_spec(x: torch.Tensor, cu: torch.Tensor, max_len: int, scale=None) -> SeqSpec:
    """[sum L, d] tensor + int32 cumulative offsets -> packed SeqSpec."""
    x = x.contiguous()
    cu = cu.to(device=x.device, dtype=torch.int32).contiguous()
    return SeqSpec(x, cu.numel() - 1, int(max_len), 0, cu, None, None, scale, 1.0)


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word the kernels OR their LIK_DEV_* bits into."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


def check_device_status(device=None, *, reset=True):
    """Synchronise and raise ``RuntimeError`` if a kernel reported a data error
    (the replacement for the reference's device-side asserts, which would kill
    the CUDA context)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = status_word(dev)
    v = int(t.item())
    if v:
        if reset:
            t.zero_()
        reasons = [txt for bit, txt in _lib.DEV_STATUS_TEXT.items() if v & bit]
        raise RuntimeError("late-interaction kernels reported: " + "; ".join(reasons))


def n_scores(pairing, q: SeqSpec, d: SeqSpec, n_pairs) -> int:
    if pairing == _lib.PAIR_CROSS:
        return q.n_seq * d.n_seq
    if pairing == _lib.PAIR_GROUPED:
        return d.n_seq
    return n_pairs


@_no_trace
def forward(q: SeqSpec, d: SeqSpec, *, pairing=_lib.PAIR_CROSS, group=0, pair_q=None, pair_d=None,
            normalize=0, save_argmax=False, argmax_stride=None, engine=0):
    """Launch ``lik_maxsim_fwd``.  Returns (scores fp32 [n_scores], argmax int32 [n_scores, stride] | None)."""
    lib = _lib.load()
    dev = q.data.device
    _lib.require_cuda(q.data, d.data, op="maxsim forward")
    if q.data.dtype != d.data.dtype:
        raise ValueError(f"Q and D must share a dtype on the kernel path; got {q.data.dtype} vs {d.data.dtype}")
    dim = q.data.shape[1]
    n_pairs = 0 if pair_q is None else pair_q.numel()
    ns = n_scores(pairing, q, d, n_pairs)
    scores = torch.empty(ns, dtype=torch.float32, device=dev)
    stride = q.max_len if argmax_stride is None else int(argmax_stride)
    argmax = torch.empty((ns, stride), dtype=torch.int32, device=dev) if save_argmax else None
    if ns == 0:
        return scores, argmax
    a = FwdArgs(
        q=q.c_struct(), d=d.c_struct(), dtype=_lib.lik_dtype(q.data.dtype), dim=dim, pairing=pairing, group=group,
        pair_q=_lib.ptr(pair_q), pair_d=_lib.ptr(pair_d), n_pairs=n_pairs, normalize=int(normalize), engine=engine,
        scores=scores.data_ptr(), argmax=_lib.ptr(argmax) if (argmax is not None and argmax.numel()) else None,
        argmax_stride=stride, reserved=0, workspace=None, workspace_bytes=0, status=status_word(dev).data_ptr(),
    )
    nbytes = lib.lik_maxsim_fwd_workspace(C.byref(a))
    ws = None
    if nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    with torch.cuda.device(dev):
        _lib.check(lib.lik_maxsim_fwd(C.byref(a), _lib.stream_ptr(dev)), "lik_maxsim_fwd")
    return scores, argmax


@_no_trace
def hidden_forward(q: SeqSpec, h: SeqSpec, w: torch.Tensor, bias, *, normalize: bool, save_argmax=False):
    """Launch ``lik_maxsim_hidden_fwd`` (projection chained into the scoring MMA).  Returns
    (scores fp32 [n_q * n_d], argmax int32 [n_q * n_d, Lq] | None), or None when the kernel does not take the problem."""
    lib = _lib.load()
    dev = q.data.device
    _lib.require_cuda(q.data, h.data, w, op="maxsim_from_hidden")
    if not (q.data.dtype == h.data.dtype == w.dtype) or (bias is not None and bias.dtype != w.dtype):
        return None
    if q.data.dtype not in (torch.bfloat16, torch.float16) or w.stride(1) != 1:
        return None
    ns = q.n_seq * h.n_seq
    a = HiddenFwdArgs(
        q=q.c_struct(), h=h.c_struct(), w=w.data_ptr(), w_stride=w.stride(0), bias=_lib.ptr(bias),
        dtype=_lib.lik_dtype(w.dtype), d_model=w.shape[1], d_out=w.shape[0],
        normalize=_lib.NORM_D if normalize else _lib.NORM_NONE, scores=None, argmax=None, argmax_stride=q.max_len, reserved=0,
        workspace=None, workspace_bytes=0, status=status_word(dev).data_ptr(),
    )
    if ns == 0 or not lib.lik_maxsim_hidden_fwd_supported(C.byref(a)):
        return None
    scores = torch.empty(ns, dtype=torch.float32, device=dev)
    argmax = torch.empty((ns, q.max_len), dtype=torch.int32, device=dev) if save_argmax else None
    a.scores = scores.data_ptr()
    a.argmax = _lib.ptr(argmax)
    nbytes = lib.lik_maxsim_hidden_fwd_workspace(C.byref(a))
    ws = None
    if nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    with torch.cuda.device(dev):
        _lib.check(lib.lik_maxsim_hidden_fwd(C.byref(a), _lib.stream_ptr(dev)), "lik_maxsim_hidden_fwd")
    return scores, argmax


@_no_trace
def hidden_winners(argmax: torch.Tensor, n_q: int, n_d: int, lq: int, ld: int, slots: int):
    """Launch ``lik_hidden_winners``: the distinct winners of every document as a compact document.  Returns
    (compact_argmax int32 like argmax, rows int64 [n_d * slots], counts int32 [n_d], bitmap, prefix)."""
    lib = _lib.load()
    dev = argmax.device
    _lib.require_cuda(argmax, op="maxsim_from_hidden backward")
    words = (ld + 31) // 32
    am_c = torch.empty_like(argmax)
    rows = torch.empty(n_d * slots, dtype=torch.int64, device=dev)
    counts = torch.empty(n_d, dtype=torch.int32, device=dev)
    bitmap = torch.empty((n_d, words), dtype=torch.int32, device=dev)
    prefix = torch.empty((n_d, words), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.lik_hidden_winners(argmax.data_ptr(), n_q, n_d, lq, ld, slots, am_c.data_ptr(), rows.data_ptr(), counts.data_ptr(),
                                          bitmap.data_ptr(), prefix.data_ptr(), status_word(dev).data_ptr(), _lib.stream_ptr(dev)),
                   "lik_hidden_winners")
    return am_c, rows, counts, bitmap, prefix


@_no_trace
def hidden_scatter_rows(compact_rows: torch.Tensor, bitmap: torch.Tensor, prefix: torch.Tensor, out: torch.Tensor, n_d: int, ld: int, slots: int):
    """Launch ``lik_hidden_scatter_rows``: ``out`` [n_d * ld, width] = compact rows of the winners, zeros elsewhere."""
    lib = _lib.load()
    dev = out.device
    _lib.require_cuda(compact_rows, out, op="maxsim_from_hidden backward")
    row_bytes = out.shape[-1] * out.element_size()
    with torch.cuda.device(dev):
        _lib.check(lib.lik_hidden_scatter_rows(compact_rows.data_ptr(), row_bytes, n_d, ld, slots, bitmap.data_ptr(), prefix.data_ptr(),
                                               out.data_ptr(), _lib.stream_ptr(dev)), "lik_hidden_scatter_rows")
    return out


def layout_spec(n_tokens: int, n_seq: int, max_len: int, *, cu=None, lens=None, seq_stride=0) -> Seqs:
    """Document layout without a token matrix (the documents are a compressed index): rows = tokens."""
    return Seqs(data=None, row_stride=0, n_rows=n_tokens, n_seq=n_seq, max_len=max_len, seq_stride=seq_stride,
                cu=_lib.ptr(cu), lens=_lib.ptr(lens), mask=None, scale=None, scale_scalar=1.0, reserved=0)


class TopkState:
    """Workspace of a fused top-k that runs over several pieces of a corpus (same queries, same k)."""

    def __init__(self):
        self.ws = None
        self.started = False


@_no_trace
def forward_fused(q: SeqSpec, d, *, normalize=0, plaid: PlaidIndex | None = None, topk=None, largest=True, index_offset=0,
                  doc_base=0, state: TopkState | None = None, last=True, save_argmax=False, argmax_stride=None):
    """The fused forms of the forward: scores fused with the per-query top-k (``topk=k``), and / or documents
    decoded from a PLAID index inside the scoring kernel (``plaid=``; ``d`` is then a ``layout_spec``).

    Returns ``None`` when the library does not take the problem on this path (the caller then scores chunks
    with :func:`forward`).  Otherwise ``(scores, argmax)`` or, with ``topk``, ``(scores [n_q, k], index
    [n_q, k])`` -- ``None`` for every piece but the last when ``state`` carries a corpus scored in pieces."""
    lib = _lib.load()
    dev = q.data.device
    _lib.require_cuda(q.data, op="maxsim fused forward")
    d_struct = d if isinstance(d, Seqs) else d.c_struct()
    n_d = d_struct.n_seq
    dim = q.data.shape[1]
    ns = q.n_seq * n_d
    tk = None
    out_s = out_i = scores = argmax = None
    stride = q.max_len if argmax_stride is None else int(argmax_stride)
    if topk is not None:
        flags = (_lib.TOPK_CONTINUE if (state is not None and state.started) else 0) | (0 if last else _lib.TOPK_PARTIAL)
        if last:
            out_s = torch.empty((q.n_seq, topk), dtype=torch.float32, device=dev)
            out_i = torch.empty((q.n_seq, topk), dtype=torch.int64, device=dev)
        tk = TopkSpec(k=topk, largest=int(bool(largest)), index_offset=index_offset, out_scores=_lib.ptr(out_s),
                      out_index=_lib.ptr(out_i), flags=flags, doc_base=doc_base)
    else:
        scores = torch.empty(ns, dtype=torch.float32, device=dev)
        argmax = torch.empty((ns, stride), dtype=torch.int32, device=dev) if save_argmax else None
    a = FwdArgs(
        q=q.c_struct(), d=d_struct, dtype=_lib.lik_dtype(q.data.dtype), dim=dim, pairing=_lib.PAIR_CROSS, group=0,
        pair_q=None, pair_d=None, n_pairs=0, normalize=int(normalize), engine=0, scores=_lib.ptr(scores),
        argmax=_lib.ptr(argmax) if (argmax is not None and argmax.numel()) else None, argmax_stride=stride, reserved=0,
        workspace=None, workspace_bytes=0, status=status_word(dev).data_ptr(),
    )
    tkp = C.byref(tk) if tk is not None else None
    with torch.cuda.device(dev):
        if plaid is not None:
            if not lib.lik_plaid_fwd_supported(C.byref(a), C.byref(plaid), tkp):
                return None
            nbytes = lib.lik_plaid_fwd_workspace(C.byref(a), C.byref(plaid), tkp)
        else:
            if not lib.lik_maxsim_fwd_topk_supported(C.byref(a), tkp):
                return None
            nbytes = lib.lik_maxsim_fwd_topk_workspace(C.byref(a), tkp)
        if state is not None and state.ws is not None and state.ws.numel() >= nbytes:
            ws = state.ws  # the candidate lists of the earlier pieces live here
        else:
            if state is not None and state.started:
                raise RuntimeError("the workspace of a top-k in pieces must not grow: score the largest piece first")
            ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        if plaid is not None:
            _lib.check(lib.lik_plaid_fwd(C.byref(a), C.byref(plaid), tkp, _lib.stream_ptr(dev)), "lik_plaid_fwd")
        else:
            _lib.check(lib.lik_maxsim_fwd_topk(C.byref(a), tkp, _lib.stream_ptr(dev)), "lik_maxsim_fwd_topk")
    if state is not None:
        state.ws, state.started = ws, True
    if topk is not None:
        return (out_s, out_i) if last else (None, None)
    return scores, argmax


@_no_trace
def backward(q: SeqSpec, d: SeqSpec, grad_scores: torch.Tensor, argmax: torch.Tensor, *, pairing=_lib.PAIR_CROSS,
             group=0, pair_q=None, pair_d=None, normalize=0, deterministic=True, grad_dtype=None,
             need_q=True, need_d=True):
    """Launch ``lik_maxsim_bwd``.  Returns (grad_q [n_rows_q, dim] | None, grad_d [n_rows_d, dim] | None)."""
    lib = _lib.load()
    dev = q.data.device
    _lib.require_cuda(q.data, d.data, grad_scores, argmax, op="maxsim backward")
    dim = q.data.shape[1]
    gdt = q.data.dtype if grad_dtype is None else grad_dtype
    gq = torch.empty((q.data.shape[0], dim), dtype=gdt, device=dev) if need_q else None
    gd = torch.empty((d.data.shape[0], dim), dtype=gdt, device=dev) if need_d else None
    n_pairs = 0 if pair_q is None else pair_q.numel()
    ns = n_scores(pairing, q, d, n_pairs)
    if ns == 0 or argmax.numel() == 0:
        if gq is not None:
            gq.zero_()
        if gd is not None:
            gd.zero_()
        return gq, gd
    g = grad_scores.contiguous().to(torch.float32).reshape(-1)
    a = BwdArgs(
        q=q.c_struct(), d=d.c_struct(), dtype=_lib.lik_dtype(q.data.dtype), dim=dim, pairing=pairing, group=group,
        pair_q=_lib.ptr(pair_q), pair_d=_lib.ptr(pair_d), n_pairs=n_pairs, normalize=int(normalize),
        deterministic=int(bool(deterministic)), grad_scores=g.data_ptr(), argmax=argmax.data_ptr(),
        argmax_stride=argmax.shape[-1], grad_dtype=_lib.lik_dtype(gdt),
        grad_q=_lib.ptr(gq) if (gq is not None and gq.numel()) else None,
        grad_d=_lib.ptr(gd) if (gd is not None and gd.numel()) else None,
        workspace=None, workspace_bytes=0, status=status_word(dev).data_ptr(),
    )
    nbytes = lib.lik_maxsim_bwd_workspace(C.byref(a))
    ws = None
    if nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    with torch.cuda.device(dev):
        _lib.check(lib.lik_maxsim_bwd(C.byref(a), _lib.stream_ptr(dev)), "lik_maxsim_bwd")
    return gq, gd


def _topk_rows_sorted(scores, k, largest, index_offset, out):
    """``k`` beyond the selection kernels' list (``LIK_TOPK_MAX``): library sorts.  The candidates (the running list and
    the new columns) are ordered by index, then stably by score, so ties go to the lower index as in the kernels."""
    n_rows, n_cols = scores.shape
    dev = scores.device
    key = scores.to(torch.float32) if largest else -scores.to(torch.float32)
    idx = (torch.arange(n_cols, device=dev, dtype=torch.int64) + index_offset).expand(n_rows, n_cols)
    if out is not None:
        live = out[1] >= 0
        old_key = torch.where(live, out[0] if largest else -out[0], -torch.inf)
        key = torch.cat([old_key, key], 1)
        idx = torch.cat([torch.where(live, out[1], torch.iinfo(torch.int64).max), idx], 1)
    idx, order = torch.sort(idx, dim=1, stable=True)
    key = torch.gather(key, 1, order)
    key, order = torch.sort(key, dim=1, descending=True, stable=True)
    idx = torch.gather(idx, 1, order)
    n = key.shape[1]
    top_s = torch.full((n_rows, k), -torch.inf if largest else torch.inf, dtype=torch.float32, device=dev)
    top_i = torch.full((n_rows, k), -1, dtype=torch.int64, device=dev)
    m = min(k, n)
    top_s[:, :m] = key[:, :m] if largest else -key[:, :m]
    top_i[:, :m] = torch.where(idx[:, :m] == torch.iinfo(torch.int64).max, -1, idx[:, :m])
    if out is not None:
        out[0].copy_(top_s)
        out[1].copy_(top_i)
        return out
    return top_s, top_i


@_no_trace
def topk_rows(scores: torch.Tensor, k: int, *, largest=True, index_offset=0, out=None):
    """Per-row top-k of a [n_rows, n_cols] fp32 matrix; ``out=(scores, idx)`` merges into a running list."""
    lib = _lib.load()
    _lib.require_cuda(scores, op="top-k")
    n_rows, n_cols = scores.shape
    if k > _lib.TOPK_MAX:
        return _topk_rows_sorted(scores, k, largest, index_offset, out)
    if scores.stride(1) != 1:
        scores = scores.contiguous()
    merge = out is not None
    if merge:
        out_s, out_i = out
    else:
        out_s = torch.empty((n_rows, k), dtype=torch.float32, device=scores.device)
        out_i = torch.empty((n_rows, k), dtype=torch.int64, device=scores.device)
    with torch.cuda.device(scores.device):
        _lib.check(
            lib.lik_topk_rows(scores.data_ptr() if scores.numel() else None, n_rows, n_cols, scores.stride(0) if n_rows else n_cols,
                              k, int(largest), index_offset, int(merge), out_s.data_ptr(), out_i.data_ptr(),
                              _lib.stream_ptr(scores.device)),
            "lik_topk_rows",
        )
    return out_s, out_i


@_no_trace
def topk_merge(cand_scores: torch.Tensor, cand_index: torch.Tensor, k: int, *, largest=True):
    """Merge candidate lists [n_lists, n_rows, k] into the per-row top k."""
    lib = _lib.load()
    _lib.require_cuda(cand_scores, cand_index, op="top-k merge")
    n_lists, n_rows, kk = cand_scores.shape
    assert kk == k and cand_index.shape == cand_scores.shape
    cs = cand_scores.contiguous().to(torch.float32)
    ci = cand_index.contiguous().to(torch.int64)
    out_s = torch.empty((n_rows, k), dtype=torch.float32, device=cs.device)
    out_i = torch.empty((n_rows, k), dtype=torch.int64, device=cs.device)
    with torch.cuda.device(cs.device):
        _lib.check(
            lib.lik_topk_merge(cs.data_ptr(), ci.data_ptr(), n_lists, n_rows, k, int(largest), out_s.data_ptr(),
                               out_i.data_ptr(), _lib.stream_ptr(cs.device)),
            "lik_topk_merge",
        )
    return out_s, out_i


def plaid_index(codes, residuals, centroids, bucket_weights, nbits, dim) -> tuple[PlaidIndex, tuple]:
    """Build the ``lik_plaid_index`` struct (tensors must already be contiguous int32 / uint8 / float)."""
    ix = PlaidIndex(
        codes=codes.data_ptr() if codes.numel() else None,
        residuals=residuals.data_ptr() if residuals.numel() else None,
        n_tokens=codes.numel(), centroids=centroids.data_ptr(), centroid_dtype=_lib.lik_dtype(centroids.dtype),
        n_centroids=centroids.shape[0], bucket_weights=bucket_weights.data_ptr(), nbits=nbits, dim=dim,
    )
    return ix, (codes, residuals, centroids, bucket_weights)


@_no_trace
def plaid_decompress(ix: PlaidIndex, token_begin: int, token_count: int, normalize: bool, out_dtype, device):
    lib = _lib.load()
    out = torch.empty((token_count, ix.dim), dtype=out_dtype, device=device)
    if token_count:
        with torch.cuda.device(device):
            _lib.check(
                lib.lik_plaid_decompress(C.byref(ix), token_begin, token_count, int(normalize), out.data_ptr(),
                                         _lib.lik_dtype(out_dtype), status_word(device).data_ptr(), _lib.stream_ptr(device)),
                "lik_plaid_decompress",
            )
    return out
