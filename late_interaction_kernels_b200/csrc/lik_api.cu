// C-ABI entry points of the forward path and the small utilities.
#include <mutex>

#include "lik_common.cuh"
#include "lik_tc.cuh"

namespace lik {
int launch_row_inv_norm(const void* data, int dtype, long long n_rows, int dim, long long stride, float eps, float* out,
                        cudaStream_t st);
int launch_row_normalize(const void* data, int dtype, long long n_rows, int dim, long long stride, float eps, void* out,
                         cudaStream_t st);
int launch_fwd_generic(const lik_fwd_args& a, const float* qn, const float* dn, cudaStream_t st);

namespace {
constexpr float kFwdNormEps = 1e-12f;

struct FwdPlan {
  size_t qn_off, dn_off, qcopy_off, dcopy_off, tc_off, total;
  bool use_tc;
  bool copies;  // fused normalisation through normalised operand copies instead of per-row multipliers
};

int validate_seqs(const lik_seqs& s, const char* name, bool compressed = false) {
  LIK_REQUIRE(s.n_seq >= 0 && s.max_len >= 0 && s.n_rows >= 0, "%s: negative size", name);
  if (!compressed) {
    LIK_REQUIRE(s.data != nullptr || s.n_rows == 0, "%s.data is NULL", name);
    LIK_REQUIRE(s.row_stride > 0 || s.n_rows == 0, "%s.row_stride must be positive", name);
  }
  if (!s.cu) {
    LIK_REQUIRE(s.seq_stride >= s.max_len, "%s.seq_stride < max_len", name);
    LIK_REQUIRE(s.n_seq == 0 || (int64_t)(s.n_seq - 1) * s.seq_stride + s.max_len <= s.n_rows,
                "%s: padded sequences exceed n_rows", name);
  }
  return LIK_OK;
}

int validate_fwd(const lik_fwd_args& a, bool compressed_docs = false, bool topk = false) {
  int rc = validate_seqs(a.q, "q");
  if (rc) return rc;
  rc = validate_seqs(a.d, "d", compressed_docs);
  if (rc) return rc;
  LIK_REQUIRE(a.dim > 0, "dim must be positive");
  LIK_REQUIRE(a.dtype >= LIK_F32 && a.dtype <= LIK_E4M3, "unknown dtype %d", a.dtype);
  LIK_REQUIRE(a.pairing >= LIK_PAIR_CROSS && a.pairing <= LIK_PAIR_LIST, "unknown pairing %d", a.pairing);
  if (a.pairing == LIK_PAIR_GROUPED)
    LIK_REQUIRE(a.group > 0 && (int64_t)a.q.n_seq * a.group == a.d.n_seq, "grouped pairing needs d.n_seq == q.n_seq * group");
  if (a.pairing == LIK_PAIR_LIST)
    LIK_REQUIRE(a.n_pairs >= 0 && (a.n_pairs == 0 || (a.pair_q && a.pair_d)), "pair list missing");
  LIK_REQUIRE(topk || a.scores != nullptr || n_scores_of(a.pairing, a.q.n_seq, a.d.n_seq, a.n_pairs) == 0, "scores is NULL");
  LIK_REQUIRE(!a.argmax || a.argmax_stride >= 0, "argmax_stride negative");
  return LIK_OK;
}

// Fused L2 normalisation.  Default: fp32 inverse norms per row, applied to the raw dot products inside the scoring
// kernel (the fp32 oracle's arithmetic).  With LIK_NORM_ROUNDED and 16-bit inputs: the way the reference kernel does
// it (forward.py:120-126) — operands normalised in fp32 and rounded back to their dtype, here once per call into
// workspace copies, then scored like pre-normalised inputs on the kernel's multiplier-free path.  Every entry point
// plans the same way, so the same call gives the same bits whichever one runs it.
FwdPlan plan_fwd(const lik_fwd_args& a, const TcExtra& x = TcExtra()) {
  FwdPlan pl{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  pl.qn_off = pl.dn_off = pl.qcopy_off = pl.dcopy_off = pl.tc_off = (size_t)-1;
  pl.copies = (a.normalize & LIK_NORM_ROUNDED) && (a.normalize & LIK_NORM_BOTH) && (a.dtype == LIK_BF16 || a.dtype == LIK_F16) &&
              !x.plaid;
  const size_t eb = dtype_size(a.dtype);
  const bool norm_d = (a.normalize & LIK_NORM_D) && !x.plaid;  // a compressed index is normalised while it is decoded
  lik_fwd_args b = a;
  if (pl.copies) {  // what the scoring kernel will see: dense rows, nothing left to normalise
    if (a.normalize & LIK_NORM_Q) b.q.row_stride = a.dim;
    if (norm_d) b.d.row_stride = a.dim;
    b.normalize = 0;
  } else {
    b.normalize = a.normalize & LIK_NORM_BOTH;
  }
  if (x.plaid)
    pl.use_tc = fwd_tc_plaid_supported(b, x) && (x.topk_k == 0 || fwd_tc_topk_supported(b, x));
  else if (x.topk_k > 0)
    pl.use_tc = fwd_tc_topk_supported(b, x);
  else
    pl.use_tc = a.engine != 1 && fwd_tc_supported(b);
  // the kernel's own workspace comes first: its leading part (the candidate lists of a fused top-k) then sits at
  // the same place for every piece of a corpus that is scored piece by piece into one workspace
  if (pl.use_tc) pl.tc_off = take(fwd_tc_workspace(b, x));
  if (a.normalize & LIK_NORM_Q) {
    if (pl.copies) pl.qcopy_off = take((size_t)a.q.n_rows * a.dim * eb);
    else pl.qn_off = take((size_t)a.q.n_rows * 4);
  }
  if (norm_d) {
    if (pl.copies) pl.dcopy_off = take((size_t)a.d.n_rows * a.dim * eb);
    else pl.dn_off = take((size_t)a.d.n_rows * 4);
  }
  pl.total = off;
  return pl;
}

int run_fwd(const lik_fwd_args& a, const FwdPlan& pl, cudaStream_t st, const TcExtra& x = TcExtra()) {
  char* ws = (char*)a.workspace;
  int rc;
  lik_fwd_args b = a;
  const float *qn = nullptr, *dn = nullptr;
  if (a.normalize & LIK_NORM_Q) {
    if (pl.copies) {
      rc = launch_row_normalize(a.q.data, a.dtype, a.q.n_rows, a.dim, a.q.row_stride, kFwdNormEps, ws + pl.qcopy_off, st);
      if (rc) return rc;
      b.q.data = ws + pl.qcopy_off;
      b.q.row_stride = a.dim;
    } else {
      float* w = (float*)(ws + pl.qn_off);
      rc = launch_row_inv_norm(a.q.data, a.dtype, a.q.n_rows, a.dim, a.q.row_stride, kFwdNormEps, w, st);
      if (rc) return rc;
      qn = w;
    }
  }
  if ((a.normalize & LIK_NORM_D) && !x.plaid) {
    if (pl.copies) {
      rc = launch_row_normalize(a.d.data, a.dtype, a.d.n_rows, a.dim, a.d.row_stride, kFwdNormEps, ws + pl.dcopy_off, st);
      if (rc) return rc;
      b.d.data = ws + pl.dcopy_off;
      b.d.row_stride = a.dim;
    } else {
      float* w = (float*)(ws + pl.dn_off);
      rc = launch_row_inv_norm(a.d.data, a.dtype, a.d.n_rows, a.dim, a.d.row_stride, kFwdNormEps, w, st);
      if (rc) return rc;
      dn = w;
    }
  }
  b.normalize = pl.copies ? 0 : (a.normalize & LIK_NORM_BOTH);
  if (pl.use_tc) return launch_fwd_tc(b, qn, dn, ws + pl.tc_off, fwd_tc_workspace(b, x), st, x);
  if (x.plaid || x.topk_k > 0) {
    set_error("this problem is outside what the fused tensor-core path takes");
    return LIK_ERR_UNSUPPORTED;
  }
  return launch_fwd_generic(b, qn, dn, st);
}
}  // namespace
}  // namespace lik

extern "C" size_t lik_maxsim_fwd_workspace(const lik_fwd_args* a) {
  if (!a) return 0;
  return lik::plan_fwd(*a).total;
}

namespace lik {
namespace {
int fwd_entry(const lik_fwd_args* a, lik_stream_t stream) {
  LIK_REQUIRE(a != nullptr, "args is NULL");
  int rc = validate_fwd(*a);
  if (rc) return rc;
  FwdPlan pl = plan_fwd(*a);
  if (a->engine == 2 && !pl.use_tc) {
    set_error("tcgen05 engine requested but this problem is outside what it takes");
    return LIK_ERR_UNSUPPORTED;
  }
  if (pl.total > a->workspace_bytes || (pl.total && !a->workspace)) {
    set_error("workspace too small: need %zu bytes, got %zu", pl.total, a->workspace_bytes);
    return LIK_ERR_WORKSPACE;
  }
  return run_fwd(*a, pl, (cudaStream_t)stream);
}
}  // namespace
}  // namespace lik

extern "C" int lik_maxsim_fwd(const lik_fwd_args* a, lik_stream_t stream) { return lik::fwd_entry(a, stream); }

// ---------------------------------------------------------------------------------------------
// Fused scoring + top-k, and scoring straight from a compressed (PLAID) index
// ---------------------------------------------------------------------------------------------
namespace lik {
namespace {
int fill_extra(const lik_fwd_args& a, const lik_plaid_index* ix, const lik_topk_spec* tk, TcExtra& x, PlaidSrc& src) {
  if (tk) {
    LIK_REQUIRE(tk->k > 0, "k must be positive");
    LIK_REQUIRE((tk->flags & LIK_TOPK_PARTIAL) || (tk->out_scores && tk->out_index), "top-k outputs are NULL");
    LIK_REQUIRE(tk->doc_base >= 0, "doc_base must not be negative");
    x.topk_flags = tk->flags;
    x.topk_doc_base = tk->doc_base;
    x.topk_k = tk->k;
    x.topk_largest = tk->largest != 0;
    x.topk_index_offset = tk->index_offset;
    x.topk_scores = tk->out_scores;
    x.topk_index = tk->out_index;
  }
  if (ix) {
    LIK_REQUIRE(ix->nbits == 2 || ix->nbits == 4 || ix->nbits == 8, "nbits must be 2, 4, or 8; got %d", ix->nbits);
    LIK_REQUIRE(ix->codes && ix->residuals && ix->centroids && ix->bucket_weights, "NULL index pointer");
    LIK_REQUIRE(ix->n_centroids > 0 && ix->dim == a.dim, "index width %d does not match the query width %d", ix->dim, a.dim);
    LIK_REQUIRE(ix->n_tokens >= a.d.n_rows, "the document layout addresses more tokens than the index holds");
    src.codes = ix->codes;
    src.residuals = ix->residuals;
    src.centroids = ix->centroids;
    src.bucket_weights = ix->bucket_weights;
    src.centroid_dtype = ix->centroid_dtype;
    src.n_centroids = ix->n_centroids;
    src.nbits = ix->nbits;
    src.packed_dim = (ix->dim * ix->nbits + 7) / 8;
    src.dim = ix->dim;
    src.normalize = (a.normalize & LIK_NORM_D) ? 1 : 0;
    x.plaid = &src;
  }
  return LIK_OK;
}

int fused_entry(const lik_fwd_args* a, const lik_plaid_index* ix, const lik_topk_spec* tk, lik_stream_t stream, int mode) {
  // mode 0: supported?  1: workspace size (through *out)  2: run
  (void)mode;
  LIK_REQUIRE(a != nullptr, "args is NULL");
  int rc = validate_fwd(*a, ix != nullptr, tk != nullptr);
  if (rc) return rc;
  TcExtra x;
  PlaidSrc src{};
  rc = fill_extra(*a, ix, tk, x, src);
  if (rc) return rc;
  FwdPlan pl = plan_fwd(*a, x);
  if (!pl.use_tc) {
    set_error("this problem is outside what the fused tensor-core path takes");
    return LIK_ERR_UNSUPPORTED;
  }
  if (pl.total > a->workspace_bytes || (pl.total && !a->workspace)) {
    set_error("workspace too small: need %zu bytes, got %zu", pl.total, a->workspace_bytes);
    return LIK_ERR_WORKSPACE;
  }
  return run_fwd(*a, pl, (cudaStream_t)stream, x);
}

size_t fused_workspace(const lik_fwd_args* a, const lik_plaid_index* ix, const lik_topk_spec* tk, int* supported) {
  if (supported) *supported = 0;
  if (!a || validate_fwd(*a, ix != nullptr, tk != nullptr)) return 0;
  TcExtra x;
  PlaidSrc src{};
  if (fill_extra(*a, ix, tk, x, src)) return 0;
  FwdPlan pl = plan_fwd(*a, x);
  if (supported) *supported = pl.use_tc ? 1 : 0;
  return pl.total;
}
}  // namespace
}  // namespace lik

extern "C" int lik_maxsim_fwd_topk_supported(const lik_fwd_args* a, const lik_topk_spec* tk) {
  int ok = 0;
  if (tk) lik::fused_workspace(a, nullptr, tk, &ok);
  return ok;
}
extern "C" size_t lik_maxsim_fwd_topk_workspace(const lik_fwd_args* a, const lik_topk_spec* tk) {
  return tk ? lik::fused_workspace(a, nullptr, tk, nullptr) : 0;
}
extern "C" int lik_maxsim_fwd_topk(const lik_fwd_args* a, const lik_topk_spec* tk, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(tk != nullptr, "top-k spec is NULL");
  return fused_entry(a, nullptr, tk, stream, 2);
}
extern "C" int lik_plaid_fwd_supported(const lik_fwd_args* a, const lik_plaid_index* ix, const lik_topk_spec* tk) {
  int ok = 0;
  if (ix) lik::fused_workspace(a, ix, tk, &ok);
  return ok;
}
extern "C" size_t lik_plaid_fwd_workspace(const lik_fwd_args* a, const lik_plaid_index* ix, const lik_topk_spec* tk) {
  return ix ? lik::fused_workspace(a, ix, tk, nullptr) : 0;
}
extern "C" int lik_plaid_fwd(const lik_fwd_args* a, const lik_plaid_index* ix, const lik_topk_spec* tk, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(ix != nullptr, "index is NULL");
  return fused_entry(a, ix, tk, stream, 2);
}

// ---------------------------------------------------------------------------------------------
// Forward without a caller workspace: the scratch lives in this library's device image.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[LIK_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of g_static_scratch on the current device.  In host code the array's name is only
// a handle; the address a kernel can use comes from cudaGetSymbolAddress, once per device.
int static_scratch(void** out) {
  int dev = 0;
  LIK_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    lik::set_error("device ordinal %d not supported by lik_maxsim_fwd_static", dev);
    return LIK_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    LIK_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return LIK_OK;
}
}  // namespace

extern "C" int lik_maxsim_fwd_static(const lik_fwd_args* a, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(a != nullptr, "args is NULL");
  int rc = validate_fwd(*a);
  if (rc) return rc;
  const size_t need = plan_fwd(*a).total;
  if (need > (size_t)LIK_STATIC_SCRATCH_BYTES) {
    set_error("lik_maxsim_fwd_static: this problem needs %zu bytes of scratch, the built-in buffer holds %zu; "
              "use lik_maxsim_fwd with a caller workspace", need, (size_t)LIK_STATIC_SCRATCH_BYTES);
    return LIK_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  rc = static_scratch(&scratch);
  if (rc) return rc;
  lik_fwd_args b = *a;
  b.workspace = scratch;
  b.workspace_bytes = LIK_STATIC_SCRATCH_BYTES;
  return fwd_entry(&b, stream);
}

extern "C" int lik_row_inv_norm(const void* data, int32_t dtype, int64_t n_rows, int32_t dim, int64_t row_stride, float eps,
                                float* out, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(n_rows >= 0 && dim > 0 && row_stride >= dim, "bad shape");
  LIK_REQUIRE((data && out) || n_rows == 0, "NULL pointer");
  return launch_row_inv_norm(data, dtype, n_rows, dim, row_stride, eps, out, (cudaStream_t)stream);
}

extern "C" const char* lik_last_error(void) { return lik::get_error(); }
extern "C" uint64_t lik_launch_count(void) { return lik::launch_count(); }
extern "C" int lik_version(void) { return 200; }
extern "C" int lik_device_supported(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
  return major == 10;
}
