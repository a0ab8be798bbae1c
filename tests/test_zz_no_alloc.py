"""lik_maxsim_fwd_static: the forward for embedders that cannot allocate device memory.

Hosts that own every byte of device memory (a serving runtime with a fixed memory plan, a sandboxed
plugin) can hand this library inputs and outputs but no workspace.  The static entry point keeps its
scratch inside the library image.  It must give the same scores as lik_maxsim_fwd, call after call,
and refuse problems that do not fit its buffer.  Collected last on purpose.
"""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(Q, D, dm, scores, argmax=None):
    from late_interaction_kernels_b200 import _lib, _ops

    q, d = _ops.padded_spec(Q), _ops.padded_spec(D, dm)
    a = _lib.FwdArgs(
        q=q.c_struct(), d=d.c_struct(), dtype=_lib.lik_dtype(Q.dtype), dim=Q.shape[-1], pairing=_lib.PAIR_CROSS, group=0,
        pair_q=None, pair_d=None, n_pairs=0, normalize=_lib.NORM_BOTH, engine=0, scores=scores.data_ptr(),
        argmax=None if argmax is None else argmax.data_ptr(), argmax_stride=Q.shape[1], reserved=0, workspace=None,
        workspace_bytes=0, status=_ops.status_word(Q.device).data_ptr(),
    )
    return a, (q, d)


def _run_both(seed, dtype, shape):
    from late_interaction_kernels_b200 import _lib

    lib = _lib.load()
    Nq, Nd, Lq, Ld, d = shape
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(Nq, Lq, d, generator=g).cuda().to(dtype)
    D = torch.randn(Nd, Ld, d, generator=g).cuda().to(dtype)
    dm = (torch.arange(Ld)[None] < torch.randint(1, Ld + 1, (Nd,), generator=g)[:, None]).cuda()
    stream = torch.cuda.current_stream().cuda_stream

    ref = torch.empty(Nq * Nd, dtype=torch.float32, device="cuda")
    ref_am = torch.empty((Nq * Nd, Lq), dtype=torch.int32, device="cuda")
    a, keep = _args(Q, D, dm, ref, ref_am)
    n = lib.lik_maxsim_fwd_workspace(C.byref(a))
    assert 0 < n <= _lib.STATIC_SCRATCH_BYTES
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = ws.data_ptr(), n
    _lib.check(lib.lik_maxsim_fwd(C.byref(a), stream), "lik_maxsim_fwd")

    got = torch.full((Nq * Nd,), float("nan"), dtype=torch.float32, device="cuda")
    got_am = torch.full((Nq * Nd, Lq), -7, dtype=torch.int32, device="cuda")
    b, keep2 = _args(Q, D, dm, got, got_am)  # no workspace at all
    _lib.check(lib.lik_maxsim_fwd_static(C.byref(b), stream), "lik_maxsim_fwd_static")
    torch.cuda.synchronize()
    assert torch.equal(got, ref), "static-scratch forward must reproduce the caller-workspace forward bit for bit"
    assert torch.equal(got_am, ref_am)
    return got


def test_static_forward_matches_on_two_calls_in_a_row():
    # two different problems back to back: the second must not see anything of the first in the scratch
    a = _run_both(1, torch.bfloat16, (8, 24, 32, 90, 128))
    b = _run_both(2, torch.bfloat16, (5, 40, 32, 150, 128))
    c = _run_both(3, torch.float32, (3, 7, 9, 33, 48))  # portable fp32 kernel uses the same scratch for the norms
    assert a.shape != b.shape and torch.isfinite(a).all() and torch.isfinite(b).all() and torch.isfinite(c).all()


def test_static_forward_refuses_what_does_not_fit():
    from late_interaction_kernels_b200 import _lib

    lib = _lib.load()
    rows = _lib.STATIC_SCRATCH_BYTES // 4 + 1024  # inverse norms alone exceed the buffer
    D = torch.zeros((rows // 64, 64, 16), dtype=torch.bfloat16, device="cuda")
    Q = torch.zeros((1, 4, 16), dtype=torch.bfloat16, device="cuda")
    out = torch.empty(D.shape[0], dtype=torch.float32, device="cuda")
    a, keep = _args(Q, D, None, out)
    rc = lib.lik_maxsim_fwd_static(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == -4 and b"built-in buffer" in lib.lik_last_error()
