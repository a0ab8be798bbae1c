// Argmax-driven MaxSim backward.
//
//   grad_q[row(i,s)] = sum_p g[p] * d_hat[row(j_p, t*)]          (row-owned gather)
//   grad_d[row(j,t)] = sum_{(p,s): t*(p,s) = t} g[p] * q_hat[row(i_p, s)]
//
// grad_d comes in two flavours: a destination-owned reduction (every CTA owns 32
// document tokens, compacts the winners that point at them in a fixed order and
// reduces them in registers: no atomics, one store per output row, bitwise
// reproducible) and an fp32-atomic scatter followed by a finalise pass.  The
// L2-normalise Jacobian is applied in the same kernels.
#include "lik_common.cuh"

namespace lik {

constexpr float kBwdNormEps = 1e-6f;  // the backward clamps ||x|| at 1e-6

struct BwdParams {
  SeqView q, d;  // inv_norm members hold 1/max(||x||,1e-6) when normalize
  PairMap pm;
  int dim;
  int normalize;
  const float* g;
  const int* argmax;
  int argmax_stride;
  void* grad_q;
  void* grad_d;
  float* gq32;  // atomic path accumulators
  float* gd32;
  int* status;
};

// slots of query i are contiguous for CROSS and GROUPED pairing
__device__ __forceinline__ void query_slots(const PairMap& pm, int i, long long& p0, int& count, int& j0) {
  if (pm.pairing == LIK_PAIR_CROSS) {
    p0 = (long long)i * pm.n_d;
    count = pm.n_d;
    j0 = 0;
  } else {
    p0 = (long long)i * pm.group;
    count = pm.group;
    j0 = i * pm.group;
  }
}

template <typename G>
__device__ __forceinline__ void store_row(G* out, long long row, int dim, int lane, const float* acc, int cmax) {
  for (int c = 0; c < cmax; ++c) {
    int k = c * 32 + lane;
    if (k < dim) out[row * dim + k] = from_f32<G>(acc[c]);
  }
}

// ---------------------------------------------------------------------------------
// grad_q, row-owned.  grid = (n_q, ceil(max_lq / 8)), 8 warps, warp = query token.
// ---------------------------------------------------------------------------------
template <typename T, typename G, int CMAX>
__global__ void __launch_bounds__(256) bwd_dq_kernel(BwdParams P) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = blockIdx.x;
  const int s = blockIdx.y * 8 + warp;
  long long qrow0;
  int qlen;
  seq_bounds(P.q, i, qrow0, qlen, nullptr);
  const int q_rows = P.q.cu ? qlen : P.q.max_len;  // rows this query owns in grad_q
  if (s >= q_rows) return;
  const long long qrow = qrow0 + s;
  float acc[CMAX];
#pragma unroll
  for (int c = 0; c < CMAX; ++c) acc[c] = 0.f;
  const bool active = s < qlen && s < P.argmax_stride && row_valid(P.q, qrow);
  if (active) {
    long long p0;
    int count, j0;
    query_slots(P.pm, i, p0, count, j0);
    const T* __restrict__ Dg = (const T*)P.d.data;
    for (int jj = 0; jj < count; ++jj) {
      const int t = P.argmax[(p0 + jj) * P.argmax_stride + s];
      if (t < 0) continue;
      long long drow0;
      int dlen;
      seq_bounds(P.d, j0 + jj, drow0, dlen, nullptr);
      if (t >= dlen) continue;
      const long long drow = drow0 + t;
      float f = P.g[p0 + jj] * row_factor(P.d, drow);
      const T* src = Dg + drow * P.d.row_stride;
#pragma unroll
      for (int c = 0; c < CMAX; ++c) {
        int k = c * 32 + lane;
        if (k < P.dim) acc[c] = fmaf(f, to_f32(src[k]), acc[c]);
      }
    }
    const float qf = P.q.scale_scalar * (P.q.scale ? P.q.scale[qrow] : 1.f);
    if (P.normalize) {
      // acc is the gradient w.r.t. q_hat = q * inv; pull it back through the normalisation
      const float inv = P.q.inv_norm[qrow];
      const T* qsrc = (const T*)P.q.data + qrow * P.q.row_stride;
      float qh[CMAX];
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < CMAX; ++c) {
        int k = c * 32 + lane;
        qh[c] = k < P.dim ? to_f32(qsrc[k]) * inv : 0.f;
        dot = fmaf(acc[c], qh[c], dot);
      }
      dot = warp_sum(dot);
#pragma unroll
      for (int c = 0; c < CMAX; ++c) acc[c] = (acc[c] - dot * qh[c]) * inv;
    } else if (qf != 1.f) {
#pragma unroll
      for (int c = 0; c < CMAX; ++c) acc[c] *= qf;
    }
  }
  store_row((G*)P.grad_q, qrow, P.dim, lane, acc, CMAX);
}

// ---------------------------------------------------------------------------------
// grad_d, destination-owned.  grid = (n_d, ceil(max_ld / 32)); 8 warps; warp w owns
// tokens t0 + w*4 .. +3 of the tile.  Winners are streamed in (query, token) order,
// compacted into shared memory in that order, and reduced in that order.
// ---------------------------------------------------------------------------------
constexpr int DD_TOK = 32;     // document tokens per CTA
constexpr int DD_CHUNK = 2048; // winner entries scanned per pass

template <typename T, typename G, int CMAX>
__global__ void __launch_bounds__(256) bwd_dd_owned_kernel(BwdParams P) {
  __shared__ int list_row[DD_CHUNK];   // query row of a matching winner (relative to q.data)
  __shared__ float list_g[DD_CHUNK];   // its weight g[p] * q-row factor
  __shared__ unsigned char list_t[DD_CHUNK];
  __shared__ int warp_cnt[8];
  __shared__ int list_n;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = blockIdx.x;
  const int t0 = blockIdx.y * DD_TOK;
  long long drow0;
  int dlen;
  seq_bounds(P.d, j, drow0, dlen, nullptr);
  const int d_rows = P.d.cu ? dlen : P.d.max_len;
  if (t0 >= d_rows) return;

  float acc[4][CMAX];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < CMAX; ++c) acc[r][c] = 0.f;

  // queries that score this document
  int i_begin, i_end;
  if (P.pm.pairing == LIK_PAIR_CROSS) {
    i_begin = 0;
    i_end = P.pm.n_q;
  } else {
    i_begin = j / P.pm.group;
    i_end = i_begin + 1;
  }
  const int lq = P.argmax_stride;
  const long long total = (long long)(i_end - i_begin) * lq;
  const T* __restrict__ Qg = (const T*)P.q.data;

  for (long long e0 = 0; e0 < total; e0 += DD_CHUNK) {
    // ---- ordered compaction of the entries whose winner lies in this tile ----
    int my_cnt = 0;
    int my_row[DD_CHUNK / 256];
    float my_g[DD_CHUNK / 256];
    int my_t[DD_CHUNK / 256];
    // thread tid takes entries e0 + tid*8 .. +7 so that order == thread order
#pragma unroll
    for (int u = 0; u < DD_CHUNK / 256; ++u) {
      long long e = e0 + (long long)tid * (DD_CHUNK / 256) + u;
      my_t[u] = -1;
      if (e < total) {
        int i = i_begin + (int)(e / lq);
        int s = (int)(e - (long long)(i - i_begin) * lq);
        long long p = P.pm.pairing == LIK_PAIR_CROSS ? (long long)i * P.pm.n_d + j : (long long)j;
        int t = P.argmax[p * lq + s];
        if (t >= t0 && t < t0 + DD_TOK && t < dlen) {
          long long qrow0;
          int qlen;
          seq_bounds(P.q, i, qrow0, qlen, nullptr);
          long long qrow = qrow0 + s;
          if (s < qlen && row_valid(P.q, qrow)) {
            my_t[u] = t - t0;
            my_row[u] = (int)qrow;
            my_g[u] = P.g[p] * row_factor(P.q, qrow);
            ++my_cnt;
          }
        }
      }
    }
    // block-wide exclusive scan of my_cnt (thread order)
    int incl = my_cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_cnt[warp] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += warp_cnt[w];
    if (tid == 255) list_n = base + incl;
    int pos = base + incl - my_cnt;
#pragma unroll
    for (int u = 0; u < DD_CHUNK / 256; ++u) {
      if (my_t[u] >= 0) {
        list_row[pos] = my_row[u];
        list_g[pos] = my_g[u];
        list_t[pos] = (unsigned char)my_t[u];
        ++pos;
      }
    }
    __syncthreads();
    const int n = list_n;
    // ---- ordered reduction: warp w handles tokens w*4 .. w*4+3 ----
    for (int e = 0; e < n; ++e) {
      const int tt = list_t[e];
      if ((tt >> 2) != warp) continue;
      const int r = tt & 3;
      const float f = list_g[e];
      const T* src = Qg + (long long)list_row[e] * P.q.row_stride;
      float v[CMAX];
#pragma unroll
      for (int c = 0; c < CMAX; ++c) {
        int k = c * 32 + lane;
        v[c] = k < P.dim ? to_f32(src[k]) : 0.f;
      }
#pragma unroll
      for (int rr = 0; rr < 4; ++rr)
        if (rr == r) {
#pragma unroll
          for (int c = 0; c < CMAX; ++c) acc[rr][c] = fmaf(f, v[c], acc[rr][c]);
        }
    }
    __syncthreads();
  }

  // ---- Jacobian + store ----
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = t0 + warp * 4 + r;
    if (t >= d_rows) continue;
    const long long drow = drow0 + t;
    const float df = P.d.scale_scalar * (P.d.scale ? P.d.scale[drow] : 1.f);
    if (P.normalize) {
      const float inv = P.d.inv_norm[drow];
      const T* dsrc = (const T*)P.d.data + drow * P.d.row_stride;
      float dh[CMAX];
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < CMAX; ++c) {
        int k = c * 32 + lane;
        dh[c] = k < P.dim ? to_f32(dsrc[k]) * inv : 0.f;
        dot = fmaf(acc[r][c], dh[c], dot);
      }
      dot = warp_sum(dot);
#pragma unroll
      for (int c = 0; c < CMAX; ++c) acc[r][c] = (acc[r][c] - dot * dh[c]) * inv;
    } else if (df != 1.f) {
#pragma unroll
      for (int c = 0; c < CMAX; ++c) acc[r][c] *= df;
    }
    store_row((G*)P.grad_d, drow, P.dim, lane, acc[r], CMAX);
  }
}

// ---------------------------------------------------------------------------------
// Atomic scatter: one warp per (score slot, query token).  Adds into fp32 buffers.
// WITH_DQ also scatters grad_q (pair lists, where a query's slots are not contiguous).
// ---------------------------------------------------------------------------------
template <typename T, bool WITH_DQ>
__global__ void __launch_bounds__(256) bwd_scatter_kernel(BwdParams P) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lq = P.argmax_stride;
  if (w >= P.pm.n_scores * lq) return;
  const long long p = w / lq;
  const int s = (int)(w - p * lq);
  int i, j;
  if (!decode_pair(P.pm, p, i, j, nullptr)) return;
  long long qrow0, drow0;
  int qlen, dlen;
  seq_bounds(P.q, i, qrow0, qlen, nullptr);
  if (s >= qlen) return;
  const long long qrow = qrow0 + s;
  if (!row_valid(P.q, qrow)) return;
  const int t = P.argmax[p * lq + s];
  if (t < 0) return;
  seq_bounds(P.d, j, drow0, dlen, nullptr);
  if (t >= dlen) return;
  const long long drow = drow0 + t;
  const float g = P.g[p];
  const T* qsrc = (const T*)P.q.data + qrow * P.q.row_stride;
  const T* dsrc = (const T*)P.d.data + drow * P.d.row_stride;
  const float fq = g * row_factor(P.q, qrow);
  const float fd = g * row_factor(P.d, drow);
  for (int k = lane; k < P.dim; k += 32) {
    if (P.gd32) atomicAdd(P.gd32 + drow * P.dim + k, fq * to_f32(qsrc[k]));
    if (WITH_DQ && P.gq32) atomicAdd(P.gq32 + qrow * P.dim + k, fd * to_f32(dsrc[k]));
  }
}

// Finalise an fp32 accumulator: optional Jacobian, optional scale, cast.  Warp per row.
template <typename T, typename G>
__global__ void __launch_bounds__(256) bwd_finalize_kernel(const float* __restrict__ acc32, SeqView v, int dim, int normalize,
                                                         G* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= v.n_rows) return;
  const float* a = acc32 + row * dim;
  if (normalize) {
    const float inv = v.inv_norm[row];
    const T* src = (const T*)v.data + row * v.row_stride;
    float dot = 0.f;
    for (int k = lane; k < dim; k += 32) dot = fmaf(a[k], to_f32(src[k]) * inv, dot);
    dot = warp_sum(dot);
    for (int k = lane; k < dim; k += 32) out[row * dim + k] = from_f32<G>((a[k] - dot * to_f32(src[k]) * inv) * inv);
  } else {
    const float f = v.scale_scalar * (v.scale ? v.scale[row] : 1.f);
    for (int k = lane; k < dim; k += 32) out[row * dim + k] = from_f32<G>(a[k] * f);
  }
}

int launch_row_inv_norm(const void* data, int dtype, long long n_rows, int dim, long long stride, float eps, float* out,
                        cudaStream_t st);

namespace {

struct BwdPlan {
  size_t qn_off, dn_off, gq32_off, gd32_off, total;
};

BwdPlan plan_bwd(const lik_bwd_args& a) {
  BwdPlan pl{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  pl.qn_off = pl.dn_off = pl.gq32_off = pl.gd32_off = (size_t)-1;
  if (a.normalize) {
    pl.qn_off = take((size_t)a.q.n_rows * 4);
    pl.dn_off = take((size_t)a.d.n_rows * 4);
  }
  const bool list = a.pairing == LIK_PAIR_LIST;
  if (a.grad_q && list) pl.gq32_off = take((size_t)a.q.n_rows * a.dim * 4);
  if (a.grad_d && (list || !a.deterministic)) pl.gd32_off = take((size_t)a.d.n_rows * a.dim * 4);
  pl.total = off;
  return pl;
}

template <typename T, typename G>
int run_bwd(const lik_bwd_args& a, BwdParams& P, const BwdPlan& pl, cudaStream_t st) {
  const bool list = a.pairing == LIK_PAIR_LIST;
  const int cmax = (a.dim + 31) / 32;
  char* ws = (char*)a.workspace;
#define LIK_BY_CMAX(KERNEL, GRID, ...)                                          \
  do {                                                                          \
    if (cmax <= 4)                                                              \
      KERNEL<T, G, 4><<<GRID, 256, 0, st>>>(__VA_ARGS__);                        \
    else if (cmax <= 8)                                                         \
      KERNEL<T, G, 8><<<GRID, 256, 0, st>>>(__VA_ARGS__);                        \
    else if (cmax <= 16)                                                        \
      KERNEL<T, G, 16><<<GRID, 256, 0, st>>>(__VA_ARGS__);                       \
    else                                                                        \
      KERNEL<T, G, 32><<<GRID, 256, 0, st>>>(__VA_ARGS__);                       \
  } while (0)

  if (a.grad_q && !list && a.q.n_seq > 0 && a.q.max_len > 0) {
    dim3 grid((unsigned)a.q.n_seq, (unsigned)ceil_div(a.q.max_len, 8));
    LIK_BY_CMAX(bwd_dq_kernel, grid, P);
    LIK_CUDA_OK(cudaGetLastError());
  }
  if (a.grad_d && !list && a.deterministic && a.d.n_seq > 0 && a.d.max_len > 0) {
    dim3 grid((unsigned)a.d.n_seq, (unsigned)ceil_div(a.d.max_len, DD_TOK));
    LIK_BY_CMAX(bwd_dd_owned_kernel, grid, P);
    LIK_CUDA_OK(cudaGetLastError());
  }
#undef LIK_BY_CMAX
  const bool scatter_q = a.grad_q && list;
  const bool scatter_d = a.grad_d && (list || !a.deterministic);
  if (scatter_q || scatter_d) {
    P.gq32 = scatter_q ? (float*)(ws + pl.gq32_off) : nullptr;
    P.gd32 = scatter_d ? (float*)(ws + pl.gd32_off) : nullptr;
    if (P.gq32) LIK_CUDA_OK(cudaMemsetAsync(P.gq32, 0, (size_t)a.q.n_rows * a.dim * 4, st));
    if (P.gd32) LIK_CUDA_OK(cudaMemsetAsync(P.gd32, 0, (size_t)a.d.n_rows * a.dim * 4, st));
    long long warps = P.pm.n_scores * (long long)a.argmax_stride;
    if (warps > 0) {
      unsigned grid = (unsigned)ceil_div(warps, 8);
      if (scatter_q)
        bwd_scatter_kernel<T, true><<<grid, 256, 0, st>>>(P);
      else
        bwd_scatter_kernel<T, false><<<grid, 256, 0, st>>>(P);
      LIK_CUDA_OK(cudaGetLastError());
    }
    if (P.gq32 && a.q.n_rows > 0) {
      bwd_finalize_kernel<T, G><<<(unsigned)ceil_div(a.q.n_rows, 8), 256, 0, st>>>(P.gq32, P.q, a.dim, a.normalize, (G*)a.grad_q);
      LIK_CUDA_OK(cudaGetLastError());
    }
    if (P.gd32 && a.d.n_rows > 0) {
      bwd_finalize_kernel<T, G><<<(unsigned)ceil_div(a.d.n_rows, 8), 256, 0, st>>>(P.gd32, P.d, a.dim, a.normalize, (G*)a.grad_d);
      LIK_CUDA_OK(cudaGetLastError());
    }
  }
  return LIK_OK;
}

template <typename T>
int run_bwd_g(const lik_bwd_args& a, BwdParams& P, const BwdPlan& pl, cudaStream_t st) {
  switch (a.grad_dtype) {
    case LIK_F32:
      return run_bwd<T, float>(a, P, pl, st);
    case LIK_F16:
      return run_bwd<T, __half>(a, P, pl, st);
    case LIK_BF16:
      return run_bwd<T, __nv_bfloat16>(a, P, pl, st);
  }
  set_error("grad_dtype %d not supported", a.grad_dtype);
  return LIK_ERR_INVALID;
}

}  // namespace
}  // namespace lik

extern "C" size_t lik_maxsim_bwd_workspace(const lik_bwd_args* a) {
  if (!a) return 0;
  return lik::plan_bwd(*a).total;
}

extern "C" int lik_maxsim_bwd(const lik_bwd_args* a, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(a != nullptr, "args is NULL");
  LIK_REQUIRE(a->dim > 0 && a->dim <= 1024, "dim %d outside (0, 1024]", a->dim);
  LIK_REQUIRE(a->pairing >= 0 && a->pairing <= 2, "unknown pairing %d", a->pairing);
  LIK_REQUIRE(a->pairing != LIK_PAIR_GROUPED || a->group > 0, "group must be positive");
  LIK_REQUIRE(a->grad_scores && a->argmax, "grad_scores and argmax are required");
  LIK_REQUIRE(a->argmax_stride > 0 || a->q.max_len == 0, "argmax_stride must be positive");
  cudaStream_t st = (cudaStream_t)stream;
  BwdPlan pl = plan_bwd(*a);
  if (pl.total > a->workspace_bytes || (pl.total && !a->workspace)) {
    set_error("workspace too small: need %zu bytes, got %zu", pl.total, a->workspace_bytes);
    return LIK_ERR_WORKSPACE;
  }
  const float *qn = nullptr, *dn = nullptr;
  if (a->normalize) {
    char* ws = (char*)a->workspace;
    float* qnw = (float*)(ws + pl.qn_off);
    float* dnw = (float*)(ws + pl.dn_off);
    int rc = launch_row_inv_norm(a->q.data, a->dtype, a->q.n_rows, a->dim, a->q.row_stride, kBwdNormEps, qnw, st);
    if (rc) return rc;
    rc = launch_row_inv_norm(a->d.data, a->dtype, a->d.n_rows, a->dim, a->d.row_stride, kBwdNormEps, dnw, st);
    if (rc) return rc;
    qn = qnw;
    dn = dnw;
  }
  BwdParams P;
  P.q = make_view(a->q, qn);
  P.d = make_view(a->d, dn);
  P.pm = PairMap{a->pairing, a->group, a->q.n_seq, a->d.n_seq, a->pair_q, a->pair_d,
                 n_scores_of(a->pairing, a->q.n_seq, a->d.n_seq, a->n_pairs)};
  P.dim = a->dim;
  P.normalize = a->normalize;
  P.g = a->grad_scores;
  P.argmax = a->argmax;
  P.argmax_stride = a->argmax_stride;
  P.grad_q = a->grad_q;
  P.grad_d = a->grad_d;
  P.gq32 = P.gd32 = nullptr;
  P.status = a->status;
  switch (a->dtype) {
    case LIK_F32:
      return run_bwd_g<float>(*a, P, pl, st);
    case LIK_F16:
      return run_bwd_g<__half>(*a, P, pl, st);
    case LIK_BF16:
      return run_bwd_g<__nv_bfloat16>(*a, P, pl, st);
  }
  set_error("dtype %d not supported by the backward", a->dtype);
  return LIK_ERR_UNSUPPORTED;
}
