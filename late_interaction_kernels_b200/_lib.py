"""ctypes binding of ``liblik_b200.so`` (the C ABI declared in ``include/lik_b200.h``).

The library is loaded lazily on first use.  There is no CPU or eager fallback:
if the shared library is missing or a call fails, a ``RuntimeError`` is raised.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "liblik_b200.so")

LIK_F32, LIK_F16, LIK_BF16, LIK_E4M3 = 0, 1, 2, 3
PAIR_CROSS, PAIR_GROUPED, PAIR_LIST = 0, 1, 2
NORM_NONE, NORM_Q, NORM_D, NORM_BOTH = 0, 1, 2, 3
NORM_ROUNDED = 4  # search paths: normalised operands rounded to the input dtype (workspace copies), see lik_b200.h
TOPK_MAX = 8192
TOPK_CONTINUE, TOPK_PARTIAL = 1, 2
TOPK_FUSED_MAX = 128  # largest k of the fused scoring + top-k kernel
STATIC_SCRATCH_BYTES = 16 << 20

DEV_STATUS_TEXT = {
    1: "a pair index is outside [0, n_seq)",
    2: "a query has more tokens than max_seqlen_q (argmax stride)",
    4: "a bounded wait expired inside the tensor-core kernel",
    8: "a PLAID centroid code is outside [0, n_centroids)",
    16: "a sequence length exceeds the padded extent",
    32: "an internal consistency check of a kernel failed",
}

_DTYPES = {torch.float32: LIK_F32, torch.float16: LIK_F16, torch.bfloat16: LIK_BF16}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = LIK_E4M3


def lik_dtype(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"dtype {dt} is not supported (float32, float16, bfloat16, float8_e4m3fn)") from None


class Seqs(C.Structure):
    _fields_ = [
        ("data", C.c_void_p), ("row_stride", C.c_int64), ("n_rows", C.c_int64), ("n_seq", C.c_int32),
        ("max_len", C.c_int32), ("seq_stride", C.c_int64), ("cu", C.c_void_p), ("lens", C.c_void_p),
        ("mask", C.c_void_p), ("scale", C.c_void_p), ("scale_scalar", C.c_float), ("reserved", C.c_int32),
    ]


class FwdArgs(C.Structure):
    _fields_ = [
        ("q", Seqs), ("d", Seqs), ("dtype", C.c_int32), ("dim", C.c_int32), ("pairing", C.c_int32),
        ("group", C.c_int32), ("pair_q", C.c_void_p), ("pair_d", C.c_void_p), ("n_pairs", C.c_int64),
        ("normalize", C.c_int32), ("engine", C.c_int32), ("scores", C.c_void_p), ("argmax", C.c_void_p),
        ("argmax_stride", C.c_int32), ("reserved", C.c_int32), ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("q", Seqs), ("d", Seqs), ("dtype", C.c_int32), ("dim", C.c_int32), ("pairing", C.c_int32),
        ("group", C.c_int32), ("pair_q", C.c_void_p), ("pair_d", C.c_void_p), ("n_pairs", C.c_int64),
        ("normalize", C.c_int32), ("deterministic", C.c_int32), ("grad_scores", C.c_void_p),
        ("argmax", C.c_void_p), ("argmax_stride", C.c_int32), ("grad_dtype", C.c_int32),
        ("grad_q", C.c_void_p), ("grad_d", C.c_void_p), ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
    ]


class HiddenFwdArgs(C.Structure):
    _fields_ = [
        ("q", Seqs), ("h", Seqs), ("w", C.c_void_p), ("w_stride", C.c_int64), ("bias", C.c_void_p),
        ("dtype", C.c_int32), ("d_model", C.c_int32), ("d_out", C.c_int32), ("normalize", C.c_int32),
        ("scores", C.c_void_p), ("argmax", C.c_void_p), ("argmax_stride", C.c_int32), ("reserved", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
    ]


class TopkSpec(C.Structure):
    _fields_ = [
        ("k", C.c_int32), ("largest", C.c_int32), ("index_offset", C.c_int64), ("out_scores", C.c_void_p),
        ("out_index", C.c_void_p), ("flags", C.c_int32), ("doc_base", C.c_int32),
    ]


class PlaidIndex(C.Structure):
    _fields_ = [
        ("codes", C.c_void_p), ("residuals", C.c_void_p), ("n_tokens", C.c_int64), ("centroids", C.c_void_p),
        ("centroid_dtype", C.c_int32), ("n_centroids", C.c_int32), ("bucket_weights", C.c_void_p),
        ("nbits", C.c_int32), ("dim", C.c_int32),
    ]


_lib = None
_lock = threading.Lock()


def _declare(lib):
    vp, i32, i64, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
    lib.lik_maxsim_fwd_workspace.argtypes = [C.POINTER(FwdArgs)]
    lib.lik_maxsim_fwd_workspace.restype = sz
    lib.lik_maxsim_fwd.argtypes = [C.POINTER(FwdArgs), vp]
    lib.lik_maxsim_fwd.restype = i32
    lib.lik_maxsim_fwd_static.argtypes = [C.POINTER(FwdArgs), vp]
    lib.lik_maxsim_fwd_static.restype = i32
    lib.lik_maxsim_bwd_workspace.argtypes = [C.POINTER(BwdArgs)]
    lib.lik_maxsim_bwd_workspace.restype = sz
    lib.lik_maxsim_bwd.argtypes = [C.POINTER(BwdArgs), vp]
    lib.lik_maxsim_bwd.restype = i32
    lib.lik_maxsim_fwd_topk_supported.argtypes = [C.POINTER(FwdArgs), C.POINTER(TopkSpec)]
    lib.lik_maxsim_fwd_topk_supported.restype = i32
    lib.lik_maxsim_fwd_topk_workspace.argtypes = [C.POINTER(FwdArgs), C.POINTER(TopkSpec)]
    lib.lik_maxsim_fwd_topk_workspace.restype = sz
    lib.lik_maxsim_fwd_topk.argtypes = [C.POINTER(FwdArgs), C.POINTER(TopkSpec), vp]
    lib.lik_maxsim_fwd_topk.restype = i32
    lib.lik_plaid_fwd_supported.argtypes = [C.POINTER(FwdArgs), C.POINTER(PlaidIndex), C.POINTER(TopkSpec)]
    lib.lik_plaid_fwd_supported.restype = i32
    lib.lik_plaid_fwd_workspace.argtypes = [C.POINTER(FwdArgs), C.POINTER(PlaidIndex), C.POINTER(TopkSpec)]
    lib.lik_plaid_fwd_workspace.restype = sz
    lib.lik_plaid_fwd.argtypes = [C.POINTER(FwdArgs), C.POINTER(PlaidIndex), C.POINTER(TopkSpec), vp]
    lib.lik_plaid_fwd.restype = i32
    lib.lik_maxsim_hidden_fwd_supported.argtypes = [C.POINTER(HiddenFwdArgs)]
    lib.lik_maxsim_hidden_fwd_supported.restype = i32
    lib.lik_maxsim_hidden_fwd_workspace.argtypes = [C.POINTER(HiddenFwdArgs)]
    lib.lik_maxsim_hidden_fwd_workspace.restype = sz
    lib.lik_maxsim_hidden_fwd.argtypes = [C.POINTER(HiddenFwdArgs), vp]
    lib.lik_maxsim_hidden_fwd.restype = i32
    lib.lik_hidden_winners.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp]
    lib.lik_hidden_winners.restype = i32
    lib.lik_hidden_scatter_rows.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp, vp]
    lib.lik_hidden_scatter_rows.restype = i32
    lib.lik_selftest_wait_timeout.argtypes = [i64, vp, vp, vp]
    lib.lik_selftest_wait_timeout.restype = i32
    lib.lik_launch_count.argtypes = []
    lib.lik_launch_count.restype = C.c_uint64
    lib.lik_topk_rows.argtypes = [vp, i64, i64, i64, i32, i32, i64, i32, vp, vp, vp]
    lib.lik_topk_rows.restype = i32
    lib.lik_topk_merge.argtypes = [vp, vp, i32, i64, i32, i32, vp, vp, vp]
    lib.lik_topk_merge.restype = i32
    lib.lik_plaid_decompress.argtypes = [C.POINTER(PlaidIndex), i64, i64, i32, vp, i32, vp, vp]
    lib.lik_plaid_decompress.restype = i32
    lib.lik_plaid_approx.argtypes = [vp, i32, i32, vp, i64, i32, vp, vp, vp]
    lib.lik_plaid_approx.restype = i32
    lib.lik_plaid_bwd_dq.argtypes = [C.POINTER(PlaidIndex), i32, i64, vp, i32, i32, i32, vp, vp, i32, vp, vp]
    lib.lik_plaid_bwd_dq.restype = i32
    lib.lik_row_inv_norm.argtypes = [vp, i32, i64, i32, i64, f32, vp, vp]
    lib.lik_row_inv_norm.restype = i32
    lib.lik_last_error.argtypes = []
    lib.lik_last_error.restype = C.c_char_p
    lib.lik_version.restype = i32
    lib.lik_device_supported.restype = i32


EXPORTED_SYMBOLS = (
    "lik_maxsim_fwd_workspace", "lik_maxsim_fwd", "lik_maxsim_fwd_static", "lik_maxsim_bwd_workspace", "lik_maxsim_bwd", "lik_topk_rows",
    "lik_maxsim_fwd_topk_supported", "lik_maxsim_fwd_topk_workspace", "lik_maxsim_fwd_topk",
    "lik_maxsim_hidden_fwd_supported", "lik_maxsim_hidden_fwd_workspace", "lik_maxsim_hidden_fwd",
    "lik_hidden_winners", "lik_hidden_scatter_rows",
    "lik_plaid_fwd_supported", "lik_plaid_fwd_workspace", "lik_plaid_fwd", "lik_launch_count", "lik_selftest_wait_timeout",
    "lik_topk_merge", "lik_plaid_decompress", "lik_plaid_approx", "lik_plaid_bwd_dq", "lik_row_inv_norm",
    "lik_last_error", "lik_version", "lik_device_supported",
)


def load():
    """Return the loaded library; raise if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: the CUDA extension has not been built "
                        "(run `python -m late_interaction_kernels_b200._build`). There is no CPU fallback."
                    )
                lib = C.CDLL(LIB_PATH)
                _declare(lib)
                _lib = lib
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().lik_last_error().decode(errors="replace")
        raise RuntimeError(f"{what} failed (status {rc}): {msg}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors, op: str):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(f"{op} requires CUDA tensors; got a tensor on {t.device}. There is no CPU fallback.")


def raise_on_status(status: torch.Tensor, what: str):
    """Read the device status word (one D2H sync) and raise if any bit is set."""
    v = int(status.item())
    if v:
        reasons = [txt for bit, txt in DEV_STATUS_TEXT.items() if v & bit]
        raise RuntimeError(f"{what}: " + "; ".join(reasons))
