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
#include <mutex>

#include "lik_common.cuh"
#include "lik_sort.cuh"

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
  // pair lists, deterministic path: the pairs grouped by query and by document (stable sorts of the pair index)
  const int* perm_q;   // [n_pairs] pair indices ordered by query, ties in list order
  const int* start_q;  // [n_q + 1] run of query i in perm_q
  const int* perm_d;   // [n_pairs] pair indices ordered by document
  const int* start_d;  // [n_d + 1]
  // grad_q with few query tokens and many documents: the documents of a query are cut into dq_split ranges, one
  // CTA each, whose fp32 partial rows [dq_split][q rows][dim] are summed in range order by a second kernel
  int dq_split;
  float* dq_partial;
};

// The scores of query i: `count` of them, numbered p0 .. p0 + count - 1 (CROSS, GROUPED: score slots; LIST:
// positions in perm_q).
__device__ __forceinline__ void query_slots(const BwdParams& P, int i, long long& p0, int& count, int& j0) {
  const PairMap& pm = P.pm;
  if (pm.pairing == LIK_PAIR_CROSS) {
    p0 = (long long)i * pm.n_d;
    count = pm.n_d;
    j0 = 0;
  } else if (pm.pairing == LIK_PAIR_GROUPED) {
    p0 = (long long)i * pm.group;
    count = pm.group;
    j0 = i * pm.group;
  } else {
    p0 = P.start_q[i];
    count = P.start_q[i + 1] - (int)p0;
    j0 = 0;
  }
}
// score slot and document of the jj-th score of a query
__device__ __forceinline__ void nth_score(const BwdParams& P, long long p0, int j0, int jj, long long& slot, int& j) {
  if (P.pm.pairing == LIK_PAIR_LIST) {
    slot = P.perm_q[p0 + jj];
    j = P.pm.pair_d[slot];
  } else {
    slot = p0 + jj;
    j = j0 + jj;
  }
}
// The scores of document j: n_qr of them; the ii-th one is score slot doc_slot(ii) of query doc_query(ii, slot).
struct DocScores {
  int n_qr, i_begin;
  long long first;  // LIST: run of the document in perm_d
};
__device__ __forceinline__ DocScores doc_scores(const BwdParams& P, int j) {
  DocScores d{0, 0, 0};
  if (P.pm.pairing == LIK_PAIR_CROSS) {
    d.n_qr = P.pm.n_q;
  } else if (P.pm.pairing == LIK_PAIR_GROUPED) {
    d.n_qr = 1;
    d.i_begin = j / P.pm.group;
  } else {
    d.first = P.start_d[j];
    d.n_qr = P.start_d[j + 1] - (int)d.first;
  }
  return d;
}
__device__ __forceinline__ long long doc_slot(const BwdParams& P, const DocScores& d, int j, int ii) {
  if (P.pm.pairing == LIK_PAIR_CROSS) return (long long)(d.i_begin + ii) * P.pm.n_d + j;
  if (P.pm.pairing == LIK_PAIR_GROUPED) return j;
  return __ldg(P.perm_d + d.first + ii);
}
__device__ __forceinline__ int doc_query(const BwdParams& P, const DocScores& d, int ii, long long slot) {
  return P.pm.pairing == LIK_PAIR_LIST ? __ldg(P.pm.pair_q + slot) : d.i_begin + ii;
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
    query_slots(P, i, p0, count, j0);
    const T* __restrict__ Dg = (const T*)P.d.data;
    for (int jj = 0; jj < count; ++jj) {
      long long slot;
      int j;
      nth_score(P, p0, j0, jj, slot, j);
      const int t = P.argmax[slot * P.argmax_stride + s];
      if (t < 0) continue;
      long long drow0;
      int dlen;
      seq_bounds(P.d, j, drow0, dlen, nullptr);
      if (t >= dlen) continue;
      const long long drow = drow0 + t;
      float f = P.g[slot] * row_factor(P.d, drow);
      const T* src = Dg + drow * P.d.row_stride;
#pragma unroll
      for (int c = 0; c < CMAX; ++c) {
        int k = c * 32 + lane;
        if (k < P.dim) acc[c] = fmaf(f, to_f32(src[k]), acc[c]);
      }
    }
    const float qf = P.q.scale_scalar * (P.q.scale ? P.q.scale[qrow] : 1.f);
    if (P.normalize & LIK_NORM_Q) {
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
    if (P.normalize & LIK_NORM_D) {
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


// =================================================================================
// Fast paths (embedding width a multiple of 4, at most 256): every lane moves 4
// consecutive elements per 128-column chunk with one vector load.
// =================================================================================
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  float4 x = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
  uint2 x = __ldg(reinterpret_cast<const uint2*>(p));
  float2 a = __half22float2(*reinterpret_cast<__half2*>(&x.x)), b = __half22float2(*reinterpret_cast<__half2*>(&x.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 x = __ldg(reinterpret_cast<const uint2*>(p));
  v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
  v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
}
// Four elements as they sit in memory (two 32-bit words for 16-bit types): gather loops keep several
// of these in flight and unpack only when they multiply, which halves the registers a load in flight costs.
template <typename T>
struct Raw4 {
  uint2 x;
};
template <>
struct Raw4<float> {
  float4 x;
};
template <typename T>
__device__ __forceinline__ Raw4<T> load4_raw(const T* p) {
  Raw4<T> r;
  r.x = __ldg(reinterpret_cast<const decltype(r.x)*>(p));
  return r;
}
template <typename T>
__device__ __forceinline__ Raw4<T> zero4_raw() {
  Raw4<T> r;
  r.x = decltype(r.x){};
  return r;
}
__device__ __forceinline__ void unpack4(const Raw4<float>& r, float (&v)[4]) {
  v[0] = r.x.x; v[1] = r.x.y; v[2] = r.x.z; v[3] = r.x.w;
}
__device__ __forceinline__ void unpack4(const Raw4<__half>& r, float (&v)[4]) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&r.x.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void unpack4(const Raw4<__nv_bfloat16>& r, float (&v)[4]) {
  v[0] = __uint_as_float(r.x.x << 16); v[1] = __uint_as_float(r.x.x & 0xffff0000u);
  v[2] = __uint_as_float(r.x.y << 16); v[3] = __uint_as_float(r.x.y & 0xffff0000u);
}
template <typename T>
__device__ __forceinline__ void fma4_raw(float (&acc)[4], float w, const Raw4<T>& r) {
  float v[4];
  unpack4(r, v);
#pragma unroll
  for (int x = 0; x < 4; ++x) acc[x] = fmaf(w, v[x], acc[x]);
}

template <typename G>
__device__ __forceinline__ void store4(G* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, const float (&v)[4]) {
  __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  uint2 x;
  x.x = *reinterpret_cast<unsigned*>(&a);
  x.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = x;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 x;
  x.x = *reinterpret_cast<unsigned*>(&a);
  x.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = x;
}

// Pull a gradient w.r.t. x_hat = x * inv back to x:  (g - <g, x_hat> x_hat) * inv.   acc is [CH][4] per lane.
template <typename T, int CH>
__device__ __forceinline__ void normalize_jacobian_row(float (&acc)[CH][4], const T* src, float inv, int dim, int lane) {
  float xh[CH][4];
  float dot = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int k = c * 128 + lane * 4;
    if (k < dim) {
      load4<T>(src + k, xh[c]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        xh[c][e] *= inv;
        dot = fmaf(acc[c][e], xh[c][e], dot);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) xh[c][e] = 0.f;
    }
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[c][e] = (acc[c][e] - dot * xh[c][e]) * inv;
}

// ---------------------------------------------------------------------------------
// grad_q fast: grid = (n_q, ceil(rows / 8)); warp = query token.  The winners and
// upstream gradients of 32 documents at a time are staged through shared memory
// (coalesced), then every warp gathers its 32 winning rows with independent loads.
// ---------------------------------------------------------------------------------
constexpr int DQ_JC = 32;
#ifndef LIK_DQ_UNROLL
#define LIK_DQ_UNROLL 8
#endif
constexpr int DQ_UNROLL = LIK_DQ_UNROLL;  // row loads in flight per warp of the grad_Q gather
static_assert(DQ_JC % DQ_UNROLL == 0, "the chunk is walked in whole groups");

template <typename T, typename G, int CH>
__global__ void __launch_bounds__(256) bwd_dq_fast_kernel(BwdParams P) {
  // per (document of the chunk, query token of the CTA): winning document row (-1: none) and the weight
  // g * row factor, prepared once by the whole CTA so that the gather loop is load + fma only
  __shared__ int2 s_e[DQ_JC][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int i = blockIdx.x;
  const int s0 = blockIdx.y * 8;
  const int s = s0 + warp;
  long long qrow0;
  int qlen;
  seq_bounds(P.q, i, qrow0, qlen, nullptr);
  const int q_rows = P.q.cu ? qlen : P.q.max_len;
  if (s0 >= q_rows) return;  // whole CTA out of range
  const long long qrow = qrow0 + s;
  const bool owns = s < q_rows;
  const bool active = owns && s < qlen && s < P.argmax_stride && row_valid(P.q, qrow);
  float acc[CH][4];
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;
  long long p0;
  int count, j0;
  query_slots(P, i, p0, count, j0);
  const int lq = P.argmax_stride;
  const long long pitch = P.d.row_stride;
  const T* __restrict__ Dlane = (const T*)P.d.data + lane * 4;
  bool lane_on[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) lane_on[c] = c * 128 + lane * 4 < P.dim;
  const bool d_factor = P.d.inv_norm || P.d.scale || P.d.scale_scalar != 1.f;
  for (int jb = 0; jb < count; jb += DQ_JC) {
    __syncthreads();
    {
      // thread (jj, r): winner of document jb + jj for query token s0 + r
      const int jj = tid >> 3, r = tid & 7;
      int2 e = make_int2(-1, 0);
      if (jb + jj < count && s0 + r < lq) {
        long long slot;
        int j;
        nth_score(P, p0, j0, jb + jj, slot, j);
        const int t = P.argmax[slot * lq + s0 + r];
        if (t >= 0) {
          long long r0;
          int dl;
          seq_bounds(P.d, j, r0, dl, nullptr);
          const long long drow = r0 + t;
          if (t < dl && drow < P.d.n_rows) {  // a saved winner outside its document contributes nothing
            float f = P.g[slot];
            if (d_factor) f *= row_factor(P.d, drow);
            e = make_int2((int)drow, __float_as_int(f));
          }
        }
      }
      s_e[jj][r] = e;
    }
    __syncthreads();
    if (active) {
      // DQ_UNROLL winners at a time: all their row loads are issued before the first one is used (an
      // entry without a winner loads nothing and multiplies zeros)
#pragma unroll 1
      for (int j0g = 0; j0g < DQ_JC; j0g += DQ_UNROLL) {
        int2 e[DQ_UNROLL];
#pragma unroll
        for (int u = 0; u < DQ_UNROLL; ++u) e[u] = s_e[j0g + u][warp];
        Raw4<T> v[DQ_UNROLL][CH];
#pragma unroll
        for (int u = 0; u < DQ_UNROLL; ++u) {
          const bool on = e[u].x >= 0;
          const T* src = Dlane + (on ? e[u].x : 0) * pitch;
#pragma unroll
          for (int c = 0; c < CH; ++c) v[u][c] = (on && lane_on[c]) ? load4_raw<T>(src + c * 128) : zero4_raw<T>();
        }
#pragma unroll
        for (int u = 0; u < DQ_UNROLL; ++u) {
          const float f = e[u].x >= 0 ? __int_as_float(e[u].y) : 0.f;
#pragma unroll
          for (int c = 0; c < CH; ++c) fma4_raw<T>(acc[c], f, v[u][c]);
        }
      }
    }
  }
  if (!owns) return;
  if (active) {
    if (P.normalize & LIK_NORM_Q) {
      normalize_jacobian_row<T, CH>(acc, (const T*)P.q.data + qrow * P.q.row_stride, P.q.inv_norm[qrow], P.dim, lane);
    } else {
      const float qf = P.q.scale_scalar * (P.q.scale ? P.q.scale[qrow] : 1.f);
      if (qf != 1.f) {
#pragma unroll
        for (int c = 0; c < CH; ++c)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[c][e] *= qf;
      }
    }
  }
  G* out = (G*)P.grad_q + qrow * P.dim;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int k = c * 128 + lane * 4;
    if (k < P.dim) store4<G>(out + k, acc[c]);
  }
}


// =================================================================================
// 16-byte gathers.  A row of the operand matrix is covered by 16 lanes that each move 16 bytes per
// 256-byte chunk, so one warp-wide load instruction fetches two different rows (one per half-warp):
// half the load instructions per gathered byte of the 8-byte version above, and twice the bytes in
// flight per instruction slot.  Every half-warp owns one output row from start to finish, so nothing
// is combined across lanes except the normalisation dot product.
// Needs 16-byte-aligned rows and a width that is a multiple of 16 bytes.
// =================================================================================
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / (int)sizeof(T);  // elements per 16-byte load
};

// volatile: the loads of a round keep their program order, i.e. all of them are issued before the
// first multiply-add that consumes one (the compiler otherwise interleaves them to save registers,
// which serialises the round trips to L2)
template <typename T>
__device__ __forceinline__ uint4 load16_raw(const T* p) {
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void unpack16(const uint4& r, float (&v)[4], const float*) {
  v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
}
__device__ __forceinline__ void unpack16(const uint4& r, float (&v)[8], const __nv_bfloat16*) {
  v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
  v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
  v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
  v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
}
__device__ __forceinline__ void unpack16(const uint4& r, float (&v)[8], const __half*) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
  const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&r.z)), d = __half22float2(*reinterpret_cast<const __half2*>(&r.w));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <typename T>
__device__ __forceinline__ void fma16_raw(float (&acc)[Vec16<T>::N], float w, const uint4& r) {
  float v[Vec16<T>::N];
  unpack16(r, v, (const T*)nullptr);
#pragma unroll
  for (int x = 0; x < Vec16<T>::N; ++x) acc[x] = fmaf(w, v[x], acc[x]);
}
// bf16 rows: two features per 32-bit word, folded in with one two-wide FMA per word (fma.rn.f32x2: the same IEEE
// operation per element as fmaf, half the FMA instructions)
template <>
__device__ __forceinline__ void fma16_raw<__nv_bfloat16>(float (&acc)[8], float w, const uint4& r) {
  unsigned long long ww;
  asm("mov.b64 %0, {%1, %1};" : "=l"(ww) : "f"(w));
  const unsigned x[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    unsigned long long v, a;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(x[i] << 16), "r"(x[i] & 0xffff0000u));
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(acc[2 * i]), "f"(acc[2 * i + 1]));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a) : "l"(ww), "l"(v));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[2 * i]), "=f"(acc[2 * i + 1]) : "l"(a));
  }
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// element offset of chunk c for lane hl of the half-warp
template <typename T>
__device__ __forceinline__ int elt16(int c, int hl) {
  return (c * 16 + hl) * Vec16<T>::N;
}

// (g - <g, x_hat> x_hat) * inv for a row held by one half-warp
template <typename T, int CH>
__device__ __forceinline__ void normalize_jacobian_row16(float (&acc)[CH][Vec16<T>::N], const T* src, float inv, int dim, int hl) {
  constexpr int N = Vec16<T>::N;
  float xh[CH][N];
  float dot = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int k = elt16<T>(c, hl);
    if (k < dim) {
      unpack16(load16_raw<T>(src + k), xh[c], (const T*)nullptr);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        xh[c][e] *= inv;
        dot = fmaf(acc[c][e], xh[c][e], dot);
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) xh[c][e] = 0.f;
    }
  }
  dot = half_warp_sum(dot);
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < N; ++e) acc[c][e] = (acc[c][e] - dot * xh[c][e]) * inv;
}

template <typename T, typename G, int CH>
__device__ __forceinline__ void store_row16(G* out, const float (&acc)[CH][Vec16<T>::N], int dim, int hl) {
  constexpr int N = Vec16<T>::N;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int k = elt16<T>(c, hl);
    if (k < dim) {
#pragma unroll
      for (int q = 0; q < N; q += 4) {
        const float v[4] = {acc[c][q], acc[c][q + 1], acc[c][q + 2], acc[c][q + 3]};
        store4<G>(out + k + q, v);
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// grad_q, 16-byte gathers: grid = (n_q, ceil(rows / 16)); half-warp = query token.  The winners and
// weights of 32 documents at a time are staged through shared memory by the whole CTA.
// ---------------------------------------------------------------------------------
constexpr int DQ16_TOK = 16;  // query tokens per CTA (one per half-warp)

// What a grad_q row still needs once its sum over the documents is complete: the normalise Jacobian or the query's
// dequantisation factor, then the store.
template <typename T, typename G, int CH>
__device__ __forceinline__ void dq16_finish_row(const BwdParams& P, float (&acc)[CH][Vec16<T>::N], long long qrow, bool active, int hl) {
  constexpr int N = Vec16<T>::N;
  if (active) {
    if (P.normalize & LIK_NORM_Q) {
      normalize_jacobian_row16<T, CH>(acc, (const T*)P.q.data + qrow * P.q.row_stride, P.q.inv_norm[qrow], P.dim, hl);
    } else {
      const float qf = P.q.scale_scalar * (P.q.scale ? P.q.scale[qrow] : 1.f);
      if (qf != 1.f) {
#pragma unroll
        for (int c = 0; c < CH; ++c)
#pragma unroll
          for (int e = 0; e < N; ++e) acc[c][e] *= qf;
      }
    }
  }
  store_row16<T, G, CH>((G*)P.grad_q + qrow * P.dim, acc, P.dim, hl);
}

template <typename T, typename G, int CH>
__global__ void __launch_bounds__(256) bwd_dq16_kernel(BwdParams P) {
  constexpr int N = Vec16<T>::N;
  constexpr int U = 8 / CH;  // rows in flight per half-warp
  __shared__ int2 s_e[DQ_JC][DQ16_TOK];
  const int tid = threadIdx.x, hl = tid & 15, hw = tid >> 4;
  const int i = blockIdx.x;
  const int s0 = blockIdx.y * DQ16_TOK;
  const int s = s0 + hw;
  long long qrow0;
  int qlen;
  seq_bounds(P.q, i, qrow0, qlen, nullptr);
  const int q_rows = P.q.cu ? qlen : P.q.max_len;
  if (s0 >= q_rows) return;  // whole CTA out of range
  const long long qrow = qrow0 + s;
  const bool owns = s < q_rows;
  const bool active = owns && s < qlen && s < P.argmax_stride && row_valid(P.q, qrow);
  float acc[CH][N];
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < N; ++e) acc[c][e] = 0.f;
  long long p0;
  int count, j0;
  query_slots(P, i, p0, count, j0);
  const int lq = P.argmax_stride;
  const long long pitch = P.d.row_stride;
  const T* __restrict__ Dlane = (const T*)P.d.data + hl * N;
  bool lane_on[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) lane_on[c] = elt16<T>(c, hl) < P.dim;
  const bool d_factor = P.d.inv_norm || P.d.scale || P.d.scale_scalar != 1.f;
  // this CTA's range of the query's documents (all of them unless the documents are split over blockIdx.z)
  int jb_lo = 0, jb_hi = count;
  if (P.dq_split > 1) {
    const int chunk = ((count + DQ_JC - 1) / DQ_JC + P.dq_split - 1) / P.dq_split * DQ_JC;
    jb_lo = min(count, (int)blockIdx.z * chunk);
    jb_hi = min(count, jb_lo + chunk);
  }
  for (int jb = jb_lo; jb < jb_hi; jb += DQ_JC) {
    __syncthreads();
#pragma unroll
    for (int x = tid; x < DQ_JC * DQ16_TOK; x += 256) {
      // entry (jj, r): winner of document jb + jj for query token s0 + r
      const int jj = x >> 4, r = x & 15;
      int2 e = make_int2(-1, 0);
      if (jb + jj < jb_hi && s0 + r < lq) {
        long long slot;
        int j;
        nth_score(P, p0, j0, jb + jj, slot, j);
        const int t = P.argmax[slot * lq + s0 + r];
        if (t >= 0) {
          long long r0;
          int dl;
          seq_bounds(P.d, j, r0, dl, nullptr);
          const long long drow = r0 + t;
          if (t < dl && drow < P.d.n_rows) {  // a saved winner outside its document contributes nothing
            float f = P.g[slot];
            if (d_factor) f *= row_factor(P.d, drow);
            e = make_int2((int)drow, __float_as_int(f));
          }
        }
      }
      s_e[jj][r] = e;
    }
    __syncthreads();
    if (active) {
#pragma unroll 1
      for (int j0g = 0; j0g < DQ_JC; j0g += U) {
        int2 e[U];
#pragma unroll
        for (int u = 0; u < U; ++u) e[u] = s_e[j0g + u][hw];
        uint4 v[U][CH];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const bool on = e[u].x >= 0;
          const T* src = Dlane + (on ? e[u].x : 0) * pitch;
#pragma unroll
          for (int c = 0; c < CH; ++c) v[u][c] = (on && lane_on[c]) ? load16_raw<T>(src + c * 16 * N) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float f = e[u].x >= 0 ? __int_as_float(e[u].y) : 0.f;
#pragma unroll
          for (int c = 0; c < CH; ++c) fma16_raw<T>(acc[c], f, v[u][c]);
        }
      }
    }
  }
  if (!owns) return;
  if (P.dq_split > 1) {  // the partial sum of this range; bwd_dq16_sum_kernel finishes the row
    store_row16<T, float, CH>(P.dq_partial + ((long long)blockIdx.z * P.q.n_rows + qrow) * P.dim, acc, P.dim, hl);
    return;
  }
  dq16_finish_row<T, G, CH>(P, acc, qrow, active, hl);
}

// Second half of the split grad_q: the partial rows of the document ranges, summed in range order.
template <typename T, typename G, int CH>
__global__ void __launch_bounds__(256) bwd_dq16_sum_kernel(BwdParams P) {
  constexpr int N = Vec16<T>::N;
  const int tid = threadIdx.x, hl = tid & 15, hw = tid >> 4;
  const int i = blockIdx.x;
  const int s = blockIdx.y * DQ16_TOK + hw;
  long long qrow0;
  int qlen;
  seq_bounds(P.q, i, qrow0, qlen, nullptr);
  const int q_rows = P.q.cu ? qlen : P.q.max_len;
  if (s >= q_rows) return;
  const long long qrow = qrow0 + s;
  const bool active = s < qlen && s < P.argmax_stride && row_valid(P.q, qrow);
  float acc[CH][N];
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < N; ++e) acc[c][e] = 0.f;
  for (int z = 0; z < P.dq_split; ++z) {
    const float* src = P.dq_partial + ((long long)z * P.q.n_rows + qrow) * P.dim;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int k = elt16<T>(c, hl);
      if (k < P.dim) {
#pragma unroll
        for (int q4 = 0; q4 < N; q4 += 4) {
          const float4 v = *reinterpret_cast<const float4*>(src + k + q4);
          acc[c][q4] += v.x;
          acc[c][q4 + 1] += v.y;
          acc[c][q4 + 2] += v.z;
          acc[c][q4 + 3] += v.w;
        }
      }
    }
  }
  dq16_finish_row<T, G, CH>(P, acc, qrow, active, hl);
}

// ---------------------------------------------------------------------------------
// grad_d fast, destination-owned, in two kernels.
//
// bwd_dd_sort_kernel, one CTA (16 warps) per document: a stable counting sort of the document's
// winners by token.
//   1. every warp histograms the winners of its contiguous slice of (query, token) entries;
//   2. a scan turns the histograms into write offsets (token-major, then warp, so the order inside
//      a token's list is the entry order);
//   3. the entries are placed into the document's slice of a global list as (query row, weight).
// bwd_dd_reduce_kernel, one warp per document token: reads its list (coalesced), gathers the query
// rows with independent vector loads, accumulates in list order and stores the row once.
// ---------------------------------------------------------------------------------
constexpr int DDS_WARPS = 16;  // most warps a sort CTA uses
#ifndef LIK_DD_UNROLL
#define LIK_DD_UNROLL 8
#endif
constexpr int DD_UNROLL = LIK_DD_UNROLL;  // independent list entries in flight per warp of the reduce kernel

struct DdSortOut {
  int2* pairs;            // [n_scores * lq] (query row, weight bits), grouped by document then token
  long long* tok_begin;   // [d.n_rows] first list entry of every document row
  int* tok_cnt;           // [d.n_rows] list length (zero-initialised by the launcher)
};

// Offsets of the winner sort.  In: hist[w][t] = winners of token t counted by warp w (n_hist of the CTA's n_warps warps
// count).  Out: the token's first list entry and count (global), and hist[w][t] = first write position of warp w for token
// t.  All warps work: each takes whole blocks of 32 tokens (totals, prefix inside the block), warp 0 scans the block
// totals, then every warp finishes its blocks.  tok_off [ld_pad] and blk [ceil(ld_pad / 32) + 1] are scratch in shared memory.
__device__ __forceinline__ void dds_offsets(int* hist, int* tok_off, int* blk, int n_warps, int n_hist, int ld_pad, int dlen,
                                            long long base, long long drow0, const DdSortOut& O, int warp, int lane) {
  const int n_blk = (dlen + 31) >> 5;
  for (int b = warp; b < n_blk; b += n_warps) {
    const int t = b * 32 + lane;
    int tot = 0;
    if (t < dlen)
      for (int w = 0; w < n_hist; ++w) tot += hist[w * ld_pad + t];
    int incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (t < dlen) tok_off[t] = incl - tot;
    if (lane == 31) blk[b] = incl;
  }
  __syncthreads();
  if (warp == 0) {
    int running = 0;
    for (int b0 = 0; b0 < n_blk; b0 += 32) {
      const int b = b0 + lane;
      const int tot = b < n_blk ? blk[b] : 0;
      int incl = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (b < n_blk) blk[b] = running + incl - tot;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  for (int b = warp; b < n_blk; b += n_warps) {
    const int t = b * 32 + lane;
    if (t < dlen) {
      const int excl = blk[b] + tok_off[t];
      int pos = excl;
      for (int w = 0; w < n_hist; ++w) {
        const int c = hist[w * ld_pad + t];
        hist[w * ld_pad + t] = pos;
        pos += c;
      }
      O.tok_begin[drow0 + t] = base + excl;
      O.tok_cnt[drow0 + t] = pos - excl;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(DDS_WARPS * 32) bwd_dd_sort_kernel(BwdParams P, DdSortOut O, int ld_pad, int n_hist) {
  // n_hist warps take the entries, one histogram each (the launcher sizes that to the entries per document); the CTA may
  // have more warps than that for the work that goes with the document's length (clearing, offsets)
  const int n_warps = blockDim.x >> 5;
  extern __shared__ int dds_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = blockIdx.x;
  long long drow0;
  int dlen;
  seq_bounds(P.d, j, drow0, dlen, nullptr);
  if (dlen <= 0) return;
  if (dlen >= ld_pad) {  // max_len understated the longest document: report instead of overrunning shared memory
    if (tid == 0 && P.status) atomicOr(P.status, LIK_DEV_LEN_RANGE);
    return;
  }
  const DocScores ds = doc_scores(P, j);
  const bool list = P.pm.pairing == LIK_PAIR_LIST;
  const int t_bits = 32 - __clz(ld_pad);  // winners are below ld_pad
  const int lq = P.argmax_stride;
  const int n_ent = ds.n_qr * lq;
  const long long base = list ? ds.first * lq : (long long)j * n_ent;  // first entry of the document's slice of the list
  int* hist = dds_raw;                          // [n_hist][ld_pad]
  int* tok_off = hist + n_hist * ld_pad;      // [ld_pad + 1]
  int* blk = tok_off + ld_pad + 1;            // [ceil(ld_pad / 32) + 1]
  float* gcol = reinterpret_cast<float*>(blk + (ld_pad + 31) / 32 + 1);  // [n_qr] (not for pair lists)

  for (int x = tid; x < n_hist * ld_pad; x += blockDim.x) hist[x] = 0;
  if (!list)
    for (int x = tid; x < ds.n_qr; x += blockDim.x) gcol[x] = P.g[doc_slot(P, ds, j, x)];
  __syncthreads();

  // entry e = ii * lq + s ; slice of this warp (multiple of 32 so rounds stay aligned)
  const int per_warp = ((n_ent + n_hist - 1) / n_hist + 31) & ~31;  // (warps beyond n_hist get an empty slice)
  const int e_lo = warp * per_warp, e_hi = min(n_ent, e_lo + per_warp);

  // raw saved winner of entry e (no validation): a plain load that can be issued ahead of its use
  auto raw_winner = [&](int e) -> int {
    if (e >= e_hi) return -1;
    const int ii = e / lq, s = e - ii * lq;
    return __ldg(P.argmax + doc_slot(P, ds, j, ii) * lq + s);
  };
  // validate a raw winner: -1 when the entry contributes nothing
  auto checked = [&](int e, int t, int& qrow_out, float& g_out) -> int {
    if (t < 0 || t >= dlen) return -1;
    const int ii = e / lq, s = e - ii * lq;
    const long long slot = doc_slot(P, ds, j, ii);
    long long qrow0;
    int qlen;
    seq_bounds(P.q, doc_query(P, ds, ii, slot), qrow0, qlen, nullptr);
    if (s >= qlen || !row_valid(P.q, qrow0 + s)) return -1;
    qrow_out = (int)(qrow0 + s);
    g_out = list ? P.g[slot] : gcol[ii];
    return t;
  };

  for (int e = e_lo + lane; e < e_hi; e += 128) {
    int t4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) t4[u] = raw_winner(e + 32 * u);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int qr;
      float gg;
      const int t = checked(e + 32 * u, t4[u], qr, gg);
      if (t >= 0) atomicAdd(&hist[warp * ld_pad + t], 1);
    }
  }
  __syncthreads();
  // offsets: warp 0 scans the tokens; hist[w][t] becomes the first write position of warp w for token t
  dds_offsets(hist, tok_off, blk, n_warps, n_hist, ld_pad, dlen, base, drow0, O, warp, lane);
  // stable placement
  int t_next = raw_winner(e_lo + lane);
  for (int eb = e_lo; eb < e_hi; eb += 32) {
    const int e = eb + lane;
    int qrow = 0;
    float gg = 0.f;
    const int t_raw = t_next;
    t_next = raw_winner(e + 32);  // in flight while this round is placed
    const int t = e < e_hi ? checked(e, t_raw, qrow, gg) : -1;
    const unsigned peers = warp_peers(t, t_bits);
    if (t >= 0) {
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int pos = hist[warp * ld_pad + t] + rank;
      O.pairs[base + pos] = make_int2(qrow, __float_as_int(gg * row_factor(P.q, qrow)));
    }
    __syncwarp();
    if (t >= 0 && (peers & ((1u << lane) - 1u)) == 0) hist[warp * ld_pad + t] += __popc(peers);
    __syncwarp();
  }
}

template <typename T, typename G, int CH>
__global__ void __launch_bounds__(256) bwd_dd_reduce_kernel(BwdParams P, DdSortOut O) {
  const int lane = threadIdx.x & 31;
  const long long drow = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (drow >= P.d.n_rows) return;
  float acc[CH][4];
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;
  // both loads are issued together; tok_begin is only meaningful when the count is non-zero
  const int cnt = __ldg(O.tok_cnt + drow);
  const long long begin = __ldg(O.tok_begin + drow);
  const T* __restrict__ Qg = (const T*)P.q.data;
  if (cnt > 0) {
    // every lane reads the same list entry (one broadcast transaction), then its own slice of the query row:
    // DD_UNROLL independent entries per round, accumulated in list order
    const int2* __restrict__ list = O.pairs + begin;
    const long long pitch = P.q.row_stride;
    const T* __restrict__ Qlane = Qg + lane * 4;
    bool lane_on[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) lane_on[c] = c * 128 + lane * 4 < P.dim;
    int k = 0;
    for (; k + DD_UNROLL <= cnt; k += DD_UNROLL) {
      int2 e[DD_UNROLL];
#pragma unroll
      for (int u = 0; u < DD_UNROLL; ++u) e[u] = __ldg(list + k + u);
      Raw4<T> v[DD_UNROLL][CH];
#pragma unroll
      for (int u = 0; u < DD_UNROLL; ++u) {
        const T* src = Qlane + e[u].x * pitch;
#pragma unroll
        for (int c = 0; c < CH; ++c) v[u][c] = lane_on[c] ? load4_raw<T>(src + c * 128) : zero4_raw<T>();
      }
#pragma unroll
      for (int u = 0; u < DD_UNROLL; ++u) {
        const float w = __int_as_float(e[u].y);
#pragma unroll
        for (int c = 0; c < CH; ++c) fma4_raw<T>(acc[c], w, v[u][c]);
      }
    }
    for (; k < cnt; ++k) {
      const int2 e = __ldg(list + k);
      const float w = __int_as_float(e.y);
      const T* src = Qlane + e.x * pitch;
#pragma unroll
      for (int c = 0; c < CH; ++c)
        if (lane_on[c]) {
          float v[4];
          load4<T>(src + c * 128, v);
#pragma unroll
          for (int x = 0; x < 4; ++x) acc[c][x] = fmaf(w, v[x], acc[c][x]);
        }
    }
  }
  if (P.normalize & LIK_NORM_D) {
    normalize_jacobian_row<T, CH>(acc, (const T*)P.d.data + drow * P.d.row_stride, P.d.inv_norm[drow], P.dim, lane);
  } else {
    const float df = P.d.scale_scalar * (P.d.scale ? P.d.scale[drow] : 1.f);
    if (df != 1.f) {
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[c][x] *= df;
    }
  }
  G* out = (G*)P.grad_d + drow * P.dim;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int kk = c * 128 + lane * 4;
    if (kk < P.dim) store4<G>(out + kk, acc[c]);
  }
}


// The same sort for argmax strides that are a multiple of four: a lane reads four consecutive winners with
// one 16-byte load and a warp keeps four such loads in flight (eight made the straight-line code twice as long for no gain), so a pass over the document's winners is a
// few round trips to L2 instead of one per 32 entries.  The order inside a token's list is (warp, round,
// load, word, lane): fixed by the data alone, hence reproducible.
constexpr int DDS_LOADS = 4;  // 16-byte loads in flight per lane

__global__ void __launch_bounds__(DDS_WARPS * 32) bwd_dd_sort4_kernel(BwdParams P, DdSortOut O, int ld_pad, int n_hist) {
  // n_hist warps take the entries, one histogram each (the launcher sizes that to the entries per document); the CTA may
  // have more warps than that for the work that goes with the document's length (clearing, offsets)
  const int n_warps = blockDim.x >> 5;
  extern __shared__ int dds_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = blockIdx.x;
  long long drow0;
  int dlen;
  seq_bounds(P.d, j, drow0, dlen, nullptr);
  if (dlen <= 0) return;
  if (dlen >= ld_pad) {  // max_len understated the longest document: report instead of overrunning shared memory
    if (tid == 0 && P.status) atomicOr(P.status, LIK_DEV_LEN_RANGE);
    return;
  }
  const DocScores ds = doc_scores(P, j);
  const bool list = P.pm.pairing == LIK_PAIR_LIST;
  const int t_bits = 32 - __clz(ld_pad);  // winners are below ld_pad
  const int lq = P.argmax_stride;          // multiple of 4
  const int qpr = lq >> 2;                 // 16-byte groups per score slot
  const int n_quad = ds.n_qr * qpr;
  const int n_ent = n_quad * 4;
  const long long base = list ? ds.first * lq : (long long)j * n_ent;
  int* hist = dds_raw;                          // [n_hist][ld_pad]
  int* tok_off = hist + n_hist * ld_pad;      // [ld_pad + 1]
  int* blk = tok_off + ld_pad + 1;            // [ceil(ld_pad / 32) + 1]
  float* gcol = reinterpret_cast<float*>(blk + (ld_pad + 31) / 32 + 1);  // [n_qr] (not for pair lists)
  int* q_first = reinterpret_cast<int*>(gcol + ds.n_qr);  // [n_qr] first row and length of every score's query (not for pair lists)
  int* q_len = q_first + ds.n_qr;

  for (int x = tid; x < n_hist * ld_pad; x += blockDim.x) hist[x] = 0;
  if (!list)
    for (int x = tid; x < ds.n_qr; x += blockDim.x) {
      const long long slot = doc_slot(P, ds, j, x);
      gcol[x] = P.g[slot];
      long long r0;
      int len;
      seq_bounds(P.q, doc_query(P, ds, x, slot), r0, len, nullptr);
      q_first[x] = (int)r0;
      q_len[x] = len;
    }
  __syncthreads();

  // slice of this warp in 16-byte groups (whole warp loads); a round is DDS_LOADS loads per lane
  const int round_quads = 32 * DDS_LOADS;
  const int per_warp = ((n_quad + n_hist - 1) / n_hist + 31) & ~31;  // (warps beyond n_hist get an empty slice)
  const int m_lo = warp * per_warp, m_hi = min(n_quad, m_lo + per_warp);
  const int4 none = make_int4(-1, -1, -1, -1);

  auto load_quad = [&](int m) -> int4 {
    if (m >= m_hi) return none;
    const int ii = m / qpr, sq = m - ii * qpr;
    return __ldg(reinterpret_cast<const int4*>(P.argmax + doc_slot(P, ds, j, ii) * lq) + sq);
  };
  // first query row and length of the query of score ii (and its upstream gradient)
  auto query_of = [&](int ii, long long& qrow0, int& qlen, float& gg) {
    if (list) {
      const long long slot = doc_slot(P, ds, j, ii);
      seq_bounds(P.q, doc_query(P, ds, ii, slot), qrow0, qlen, nullptr);
      gg = P.g[slot];
    } else {
      qrow0 = q_first[ii];
      qlen = q_len[ii];
      gg = gcol[ii];
    }
  };

  // ---- pass 1: per-warp histogram of the winners per token ----
  for (int mb = m_lo; mb < m_hi; mb += round_quads) {
    int4 w[DDS_LOADS];
#pragma unroll
    for (int u = 0; u < DDS_LOADS; ++u) w[u] = load_quad(mb + u * 32 + lane);
#pragma unroll
    for (int u = 0; u < DDS_LOADS; ++u) {
      const int m = mb + u * 32 + lane;
      if (m >= m_hi) continue;
      const int ii = m / qpr, s4 = (m - ii * qpr) * 4;
      long long qrow0;
      int qlen;
      float gg;
      query_of(ii, qrow0, qlen, gg);
      // (the four winners of a load go through one copy of the code: the kernel runs once per CTA, straight through,
      // and its time is instruction fetch as much as anything)
#pragma unroll 1
      for (int k = 0; k < 4; ++k) {
        const int t = k == 0 ? w[u].x : (k == 1 ? w[u].y : (k == 2 ? w[u].z : w[u].w));
        if (t >= 0 && t < dlen && s4 + k < qlen && row_valid(P.q, qrow0 + s4 + k)) atomicAdd(&hist[warp * ld_pad + t], 1);
      }
    }
  }
  __syncthreads();
  // ---- offsets: warp 0 scans the per-token totals ----
  dds_offsets(hist, tok_off, blk, n_warps, n_hist, ld_pad, dlen, base, drow0, O, warp, lane);
  // ---- pass 2: placement (the winners come from L2 this time) ----
  for (int mb = m_lo; mb < m_hi; mb += round_quads) {
    int4 w[DDS_LOADS];
#pragma unroll
    for (int u = 0; u < DDS_LOADS; ++u) w[u] = load_quad(mb + u * 32 + lane);
#pragma unroll
    for (int u = 0; u < DDS_LOADS; ++u) {
      const int m = mb + u * 32 + lane;
      const bool in = m < m_hi;
      const int ii = in ? m / qpr : 0, s4 = in ? (m - ii * qpr) * 4 : 0;
      long long qrow0 = 0;
      int qlen = 0;
      float gi = 0.f;
      if (in) query_of(ii, qrow0, qlen, gi);
#pragma unroll 1
      for (int k = 0; k < 4; ++k) {
        int t = k == 0 ? w[u].x : (k == 1 ? w[u].y : (k == 2 ? w[u].z : w[u].w));
        const int qrow = (int)(qrow0 + s4 + k);
        if (!(in && t >= 0 && t < dlen && s4 + k < qlen && row_valid(P.q, qrow))) t = -1;
        const unsigned peers = warp_peers(t, t_bits);
        if (t >= 0) {
          const int rank = __popc(peers & ((1u << lane) - 1u));
          const int pos = hist[warp * ld_pad + t] + rank;
          O.pairs[base + pos] = make_int2(qrow, __float_as_int(gi * row_factor(P.q, qrow)));
        }
        __syncwarp();
        if (t >= 0 && (peers & ((1u << lane) - 1u)) == 0) hist[warp * ld_pad + t] += __popc(peers);
        __syncwarp();
      }
    }
  }
}

// grad_d reduce with 16-byte gathers: one half-warp per document token, 16 tokens per CTA.
template <typename T, typename G, int CH>
__device__ __forceinline__ void dd_reduce16_row(const BwdParams& P, const DdSortOut& O, long long drow, int hl) {
  constexpr int N = Vec16<T>::N;
  constexpr int U = 8 / CH;
  float acc[CH][N];
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < N; ++e) acc[c][e] = 0.f;
  const int cnt = __ldg(O.tok_cnt + drow);
  const long long begin = __ldg(O.tok_begin + drow);
  if (cnt > 0) {
    const int2* __restrict__ list = O.pairs + begin;
    const long long pitch = P.q.row_stride;
    const T* __restrict__ Qlane = (const T*)P.q.data + hl * N;
    bool lane_on[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) lane_on[c] = elt16<T>(c, hl) < P.dim;
    int k = 0;
    for (; k + U <= cnt; k += U) {
      int2 e[U];
#pragma unroll
      for (int u = 0; u < U; ++u) e[u] = __ldg(list + k + u);
      uint4 v[U][CH];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const T* src = Qlane + e[u].x * pitch;
#pragma unroll
        for (int c = 0; c < CH; ++c) v[u][c] = lane_on[c] ? load16_raw<T>(src + c * 16 * N) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float w = __int_as_float(e[u].y);
#pragma unroll
        for (int c = 0; c < CH; ++c) fma16_raw<T>(acc[c], w, v[u][c]);
      }
    }
    for (; k < cnt; ++k) {
      const int2 e = __ldg(list + k);
      const float w = __int_as_float(e.y);
      const T* src = Qlane + e.x * pitch;
#pragma unroll
      for (int c = 0; c < CH; ++c)
        if (lane_on[c]) fma16_raw<T>(acc[c], w, load16_raw<T>(src + c * 16 * N));
    }
  }
  if (P.normalize & LIK_NORM_D) {
    normalize_jacobian_row16<T, CH>(acc, (const T*)P.d.data + drow * P.d.row_stride, P.d.inv_norm[drow], P.dim, hl);
  } else {
    const float df = P.d.scale_scalar * (P.d.scale ? P.d.scale[drow] : 1.f);
    if (df != 1.f) {
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int x = 0; x < N; ++x) acc[c][x] *= df;
    }
  }
  store_row16<T, G, CH>((G*)P.grad_d + drow * P.dim, acc, P.dim, hl);
}

template <typename T, typename G, int CH>
__global__ void __launch_bounds__(256) bwd_dd_reduce16_kernel(BwdParams P, DdSortOut O) {
  const int hl = threadIdx.x & 15;
  const long long drow = (long long)blockIdx.x * 16 + (threadIdx.x >> 4);
  if (drow >= P.d.n_rows) return;
  dd_reduce16_row<T, G, CH>(P, O, drow, hl);
}

// The same for very many document tokens (long documents), nearly all of them without a winner: a stream of zero rows.
// One CTA per 16 tokens costs more to schedule than to run there, so a capped grid walks the tokens, and a token without
// a winner stores its zero row without looking at anything else.
template <typename T, typename G, int CH>
__global__ void __launch_bounds__(256) bwd_dd_reduce16_walk_kernel(BwdParams P, DdSortOut O) {
  const int hl = threadIdx.x & 15;
  for (long long drow = (long long)blockIdx.x * 16 + (threadIdx.x >> 4); drow < P.d.n_rows; drow += (long long)gridDim.x * 16) {
    if (__ldg(O.tok_cnt + drow) == 0) {
      float zero[CH][Vec16<T>::N];
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < Vec16<T>::N; ++e) zero[c][e] = 0.f;
      store_row16<T, G, CH>((G*)P.grad_d + drow * P.dim, zero, P.dim, hl);
    } else {
      dd_reduce16_row<T, G, CH>(P, O, drow, hl);
    }
  }
}

// ---------------------------------------------------------------------------------
// Atomic scatter: one warp per (score slot, query token).  Adds into fp32 buffers.
// WITH_DQ also scatters grad_q (pair lists, where a query's slots are not contiguous).
// ---------------------------------------------------------------------------------
template <typename T, bool WITH_DQ, bool VEC>
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
  if (VEC) {
    // four consecutive elements per lane and one 16-byte reduction per lane (rows and width are multiples of 4)
    for (int k = lane * 4; k < P.dim; k += 128) {
      float v[4];
      if (P.gd32) {
        load4<T>(qsrc + k, v);
        atomicAdd(reinterpret_cast<float4*>(P.gd32 + drow * P.dim + k), make_float4(fq * v[0], fq * v[1], fq * v[2], fq * v[3]));
      }
      if (WITH_DQ && P.gq32) {
        load4<T>(dsrc + k, v);
        atomicAdd(reinterpret_cast<float4*>(P.gq32 + qrow * P.dim + k), make_float4(fd * v[0], fd * v[1], fd * v[2], fd * v[3]));
      }
    }
  } else {
    for (int k = lane; k < P.dim; k += 32) {
      if (P.gd32) atomicAdd(P.gd32 + drow * P.dim + k, fq * to_f32(qsrc[k]));
      if (WITH_DQ && P.gq32) atomicAdd(P.gq32 + qrow * P.dim + k, fd * to_f32(dsrc[k]));
    }
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

// Sort keys of a pair list: the query and the document of every pair (a pair with an index out of range gets the key
// one past the last sequence on both sides, so it sorts behind every run and no gradient kernel visits it), and the
// pair index as the value that travels with them.
__global__ void pair_keys_kernel(const int* __restrict__ pair_q, const int* __restrict__ pair_d, long long n, int n_q, int n_d,
                                 unsigned* __restrict__ kq, unsigned* __restrict__ kd, unsigned* __restrict__ vq,
                                 unsigned* __restrict__ vd, int* status) {
  const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  const int i = pair_q[p], j = pair_d[p];
  const bool ok = i >= 0 && i < n_q && j >= 0 && j < n_d;
  if (!ok && status) atomicOr(status, LIK_DEV_PAIR_RANGE);
  kq[p] = ok ? (unsigned)i : (unsigned)n_q;
  kd[p] = ok ? (unsigned)j : (unsigned)n_d;
  vq[p] = (unsigned)p;
  vd[p] = (unsigned)p;
}

namespace {

struct BwdPlan {
  size_t qn_off, dn_off, gq32_off, gd32_off, pairs_off, begin_off, cnt_off, total;
  size_t kq_off, kd_off, pq_off, pd_off, sq_off, sd_off, sort_off;  // pair lists grouped by query / by document
  bool fast, sorted;
  bool list_sorted;  // pair list on the deterministic kernels
  int sort_warps;    // warps of the winner sort that take entries (a histogram each): at least 256 entries of a document per warp
  int sort_threads;  // threads of its CTAs: more warps than that when the documents are long (clearing and offsets go with the length)
  bool row16;  // 16-byte gathers: rows 16-byte aligned, width a multiple of 16 bytes, at most 1024 bytes
  int dq_split;    // grad_q: document ranges per query (1: one CTA walks all the documents of its query tokens)
  size_t dqp_off;  // their partial rows
  int ld_pad;
  size_t sort_smem;
};

bool bwd_fast_ok(const lik_bwd_args& a) {
  // vector fast paths: rows 8/16-byte aligned, width a multiple of 4 and at most 256
  const size_t eb = dtype_size(a.dtype);
  return a.dim % 4 == 0 && a.dim <= 256 && (a.q.row_stride * eb) % (4 * eb) == 0 && (a.d.row_stride * eb) % (4 * eb) == 0 &&
         ((uintptr_t)a.q.data % (4 * eb)) == 0 && ((uintptr_t)a.d.data % (4 * eb)) == 0 && ((uintptr_t)a.grad_q % 16) == 0 &&
         ((uintptr_t)a.grad_d % 16) == 0 && a.q.n_rows < (1ll << 31) && a.d.n_rows < (1ll << 31);  // row indices travel as int
}

bool bwd_row16_ok(const lik_bwd_args& a) {
  const size_t eb = dtype_size(a.dtype);
  return bwd_fast_ok(a) && (a.dim * eb) % 16 == 0 && a.dim * eb <= 1024 && (a.q.row_stride * eb) % 16 == 0 &&
         (a.d.row_stride * eb) % 16 == 0 && ((uintptr_t)a.q.data % 16) == 0 && ((uintptr_t)a.d.data % 16) == 0;
}

BwdPlan plan_bwd(const lik_bwd_args& a) {
  BwdPlan pl{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  pl.qn_off = pl.dn_off = pl.gq32_off = pl.gd32_off = pl.pairs_off = pl.begin_off = pl.cnt_off = (size_t)-1;
  pl.fast = bwd_fast_ok(a);
  pl.row16 = bwd_row16_ok(a);
  pl.sorted = false;
  if (a.normalize & LIK_NORM_Q) pl.qn_off = take((size_t)a.q.n_rows * 4);
  if (a.normalize & LIK_NORM_D) pl.dn_off = take((size_t)a.d.n_rows * 4);
  const bool list = a.pairing == LIK_PAIR_LIST;
  pl.kq_off = pl.kd_off = pl.pq_off = pl.pd_off = pl.sq_off = pl.sd_off = pl.sort_off = (size_t)-1;
  // a pair list goes through the same deterministic kernels once its pairs are grouped by query and by document
  pl.list_sorted = list && a.deterministic && pl.fast && a.n_pairs > 0 && a.n_pairs < (1ll << 31) && a.d.max_len > 0 &&
                   a.q.max_len > 0 && a.q.n_seq > 0 && a.d.n_seq > 0;
  if (pl.list_sorted) {
    const size_t ws_sort = ((size_t)(a.d.max_len + 1) + a.d.max_len + 2) * 4;  // with one warp per CTA
    if (ws_sort > 200 * 1024) pl.list_sorted = false;
  }
  if (pl.list_sorted) {
    pl.kq_off = take((size_t)a.n_pairs * 4);
    pl.kd_off = take((size_t)a.n_pairs * 4);
    pl.pq_off = take((size_t)a.n_pairs * 4);
    pl.pd_off = take((size_t)a.n_pairs * 4);
    pl.sq_off = take((size_t)(a.q.n_seq + 1) * 4);
    pl.sd_off = take((size_t)(a.d.n_seq + 1) * 4);
    pl.sort_off = take(sort_pairs_scratch(a.n_pairs));
  }
  // few query tokens against many documents: one CTA per 16 query tokens would leave most of the GPU idle
  pl.dq_split = 1;
  pl.dqp_off = (size_t)-1;
  if (a.grad_q && pl.row16 && a.pairing == LIK_PAIR_CROSS && a.q.n_seq > 0 && a.q.max_len > 0 && a.dim % 4 == 0) {
    const long long base = (long long)a.q.n_seq * ceil_div(a.q.max_len, DQ16_TOK);
    const long long chunks = ceil_div(a.d.n_seq, DQ_JC);
    long long z = (2ll * sm_count()) / base;
    if (z > chunks / 2) z = chunks / 2;  // at least two rounds of documents per range
    if (z > 64) z = 64;
    if (z >= 2) {
      pl.dq_split = (int)z;
      pl.dqp_off = take((size_t)z * a.q.n_rows * a.dim * 4);
    }
  }
  const bool scatter = list && !pl.list_sorted;
  if (a.grad_q && scatter) pl.gq32_off = take((size_t)a.q.n_rows * a.dim * 4);
  if (a.grad_d && (scatter || !a.deterministic)) pl.gd32_off = take((size_t)a.d.n_rows * a.dim * 4);
  if (a.grad_d && !scatter && a.deterministic && pl.fast && a.d.n_seq > 0 && a.d.max_len > 0 && a.d.n_rows < (1ll << 31) &&
      a.q.n_rows < (1ll << 31)) {
    const long long n_qrange = a.pairing == LIK_PAIR_CROSS ? a.q.n_seq : (list ? 0 : 1);
    pl.ld_pad = a.d.max_len + 1;
    // entries (query token, winner) per document: every document has the same number, except in a pair list (average)
    const long long ent = a.pairing == LIK_PAIR_CROSS ? (long long)a.q.n_seq * a.argmax_stride
                          : a.pairing == LIK_PAIR_GROUPED ? (long long)a.argmax_stride
                                                          : ceil_div(a.n_pairs, a.d.n_seq) * a.argmax_stride;
    long long nw = ceil_div(ent, 256);  // a warp per 256 entries: few, long documents still fill their CTAs
    pl.sort_warps = (int)(nw < 1 ? 1 : (nw > DDS_WARPS ? DDS_WARPS : nw));
    auto smem_for = [&](int w) {
      return ((size_t)w * pl.ld_pad + pl.ld_pad + 1 + (size_t)(pl.ld_pad + 31) / 32 + 1 + 3 * (size_t)n_qrange) * 4;
    };
    while (pl.sort_warps > 1 && smem_for(pl.sort_warps) > 200 * 1024) pl.sort_warps >>= 1;  // long documents: fewer histograms
    pl.sort_smem = smem_for(pl.sort_warps);
    {
      long long by_len = ceil_div(pl.ld_pad, 512);
      if (by_len > DDS_WARPS) by_len = DDS_WARPS;
      pl.sort_threads = 32 * (int)(by_len > pl.sort_warps ? by_len : pl.sort_warps);
    }
    if (pl.sort_smem <= 200 * 1024) {
      pl.sorted = true;
      const long long n_ent = n_scores_of(a.pairing, a.q.n_seq, a.d.n_seq, a.n_pairs) * (long long)a.argmax_stride;
      pl.pairs_off = take((size_t)n_ent * sizeof(int2));
      pl.begin_off = take((size_t)a.d.n_rows * sizeof(long long));
      pl.cnt_off = take((size_t)a.d.n_rows * sizeof(int));
    }
  }
  pl.total = off;
  return pl;
}

// grad_Q and grad_D are independent, and both are bound by gather latency rather than by any
// throughput limit, so when both are wanted the grad_Q kernel runs on a second stream beside the
// grad_D kernels: fork after everything already enqueued on the caller's stream, join before returning
// to it.  One auxiliary stream and two events per device, created on first use; the enqueue sequence
// holds a lock because the events are shared by every caller on that device.
struct ForkJoin {
  cudaStream_t aux = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool ok = false;
};
std::mutex g_fork_mutex;
ForkJoin g_fork[64];

ForkJoin* fork_join_locked() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  ForkJoin& f = g_fork[dev];
  if (!f.aux) {
    f.ok = cudaStreamCreateWithFlags(&f.aux, cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&f.fork, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&f.join, cudaEventDisableTiming) == cudaSuccess;
    if (!f.ok) (void)cudaGetLastError();
  }
  return f.ok ? &f : nullptr;
}

template <typename T, typename G>
int run_bwd(const lik_bwd_args& a, BwdParams& P, const BwdPlan& pl, cudaStream_t st_main) {
  const bool list = a.pairing == LIK_PAIR_LIST && !pl.list_sorted;  // pair list on the atomic path
  if (pl.list_sorted) {
    // group the pairs by query and by document: two stable sorts of the pair index
    char* w = (char*)a.workspace;
    unsigned *kq = (unsigned*)(w + pl.kq_off), *kd = (unsigned*)(w + pl.kd_off);
    unsigned *pq = (unsigned*)(w + pl.pq_off), *pd = (unsigned*)(w + pl.pd_off);
    pair_keys_kernel<<<(unsigned)ceil_div(a.n_pairs, 256), 256, 0, st_main>>>(a.pair_q, a.pair_d, a.n_pairs, a.q.n_seq, a.d.n_seq, kq, kd,
                                                                            pq, pd, a.status), ::lik::count_launch();
    LIK_CUDA_OK(cudaGetLastError());
    auto bits = [](int n) { int b = 1; while ((1ll << b) <= n) ++b; return b; };
    int rc = stable_sort_pairs(kq, pq, a.n_pairs, bits(a.q.n_seq), w + pl.sort_off, st_main);
    if (rc) return rc;
    rc = stable_sort_pairs(kd, pd, a.n_pairs, bits(a.d.n_seq), w + pl.sort_off, st_main);
    if (rc) return rc;
    rc = run_starts(kq, a.n_pairs, a.q.n_seq, (int*)(w + pl.sq_off), st_main);
    if (rc) return rc;
    rc = run_starts(kd, a.n_pairs, a.d.n_seq, (int*)(w + pl.sd_off), st_main);
    if (rc) return rc;
    P.perm_q = (const int*)pq;
    P.perm_d = (const int*)pd;
    P.start_q = (const int*)(w + pl.sq_off);
    P.start_d = (const int*)(w + pl.sd_off);
  }
  // fork only when both gradients run the gather kernels and the problem is large enough to matter
  const bool want_fork = a.grad_q && a.grad_d && !list && a.deterministic && pl.fast && pl.sorted &&
                         P.pm.n_scores * (long long)a.argmax_stride >= (1ll << 20);
  std::unique_lock<std::mutex> fork_lock(g_fork_mutex, std::defer_lock);
  ForkJoin* fj = nullptr;
  if (want_fork) {
    fork_lock.lock();
    fj = fork_join_locked();
    if (fj) {
      LIK_CUDA_OK(cudaEventRecord(fj->fork, st_main));
      LIK_CUDA_OK(cudaStreamWaitEvent(fj->aux, fj->fork, 0));
    } else {
      fork_lock.unlock();
    }
  }
  cudaStream_t st = fj ? fj->aux : st_main;  // stream of the grad_Q kernel; grad_D switches back below
  const int cmax = (a.dim + 31) / 32;
  char* ws = (char*)a.workspace;
#define LIK_BY_CMAX(KERNEL, GRID, ...)                                          \
  do {                                                                          \
    if (cmax <= 4)                                                              \
      KERNEL<T, G, 4><<<GRID, 256, 0, st>>>(__VA_ARGS__), ::lik::count_launch();                        \
    else if (cmax <= 8)                                                         \
      KERNEL<T, G, 8><<<GRID, 256, 0, st>>>(__VA_ARGS__), ::lik::count_launch();                        \
    else if (cmax <= 16)                                                        \
      KERNEL<T, G, 16><<<GRID, 256, 0, st>>>(__VA_ARGS__), ::lik::count_launch();                       \
    else                                                                        \
      KERNEL<T, G, 32><<<GRID, 256, 0, st>>>(__VA_ARGS__), ::lik::count_launch();                       \
  } while (0)

  const bool fast = pl.fast;
  if (a.grad_q && !list && a.q.n_seq > 0 && a.q.max_len > 0) {
    dim3 grid((unsigned)a.q.n_seq, (unsigned)ceil_div(a.q.max_len, 8));
    if (pl.row16) {
      const dim3 grid16((unsigned)a.q.n_seq, (unsigned)ceil_div(a.q.max_len, DQ16_TOK), (unsigned)pl.dq_split);
      const dim3 grid_sum((unsigned)a.q.n_seq, (unsigned)ceil_div(a.q.max_len, DQ16_TOK));
      const size_t row_bytes = (size_t)a.dim * sizeof(T);
#define LIK_DQ16(CH_)                                                                              \
  do {                                                                                             \
    bwd_dq16_kernel<T, G, CH_><<<grid16, 256, 0, st>>>(P), ::lik::count_launch();                  \
    if (pl.dq_split > 1) bwd_dq16_sum_kernel<T, G, CH_><<<grid_sum, 256, 0, st>>>(P), ::lik::count_launch(); \
  } while (0)
      if (row_bytes <= 256) LIK_DQ16(1);
      else if (row_bytes <= 512) LIK_DQ16(2);
      else LIK_DQ16(4);
#undef LIK_DQ16
    } else if (fast) {
      if (a.dim <= 128)
        bwd_dq_fast_kernel<T, G, 1><<<grid, 256, 0, st>>>(P), ::lik::count_launch();
      else
        bwd_dq_fast_kernel<T, G, 2><<<grid, 256, 0, st>>>(P), ::lik::count_launch();
    } else {
      LIK_BY_CMAX(bwd_dq_kernel, grid, P);
    }
    LIK_CUDA_OK(cudaGetLastError());
  }
  if (fj) {
    LIK_CUDA_OK(cudaEventRecord(fj->join, fj->aux));
    st = st_main;
  }
  if (a.grad_d && !list && a.deterministic && a.d.n_seq > 0 && a.d.max_len > 0) {
    if (pl.sorted) {
      DdSortOut O;
      O.pairs = (int2*)(ws + pl.pairs_off);
      O.tok_begin = (long long*)(ws + pl.begin_off);
      O.tok_cnt = (int*)(ws + pl.cnt_off);
      LIK_CUDA_OK(cudaMemsetAsync(O.tok_cnt, 0, (size_t)a.d.n_rows * sizeof(int), st));
      const bool quads = a.argmax_stride % 4 == 0 && ((uintptr_t)a.argmax % 16) == 0;
      if (quads) {
        LIK_CUDA_OK(cudaFuncSetAttribute(bwd_dd_sort4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.sort_smem));
        bwd_dd_sort4_kernel<<<(unsigned)a.d.n_seq, pl.sort_threads, pl.sort_smem, st>>>(P, O, pl.ld_pad, pl.sort_warps), ::lik::count_launch();
      } else {
        LIK_CUDA_OK(cudaFuncSetAttribute(bwd_dd_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.sort_smem));
        bwd_dd_sort_kernel<<<(unsigned)a.d.n_seq, pl.sort_threads, pl.sort_smem, st>>>(P, O, pl.ld_pad, pl.sort_warps), ::lik::count_launch();
      }
      LIK_CUDA_OK(cudaGetLastError());
      if (pl.row16) {
        // one CTA per 16 tokens, except for very many tokens (long documents): there a capped grid walks them
        const long long rg = ceil_div(a.d.n_rows, 16);
        const bool walk = rg > 65536;
        const unsigned rgrid = (unsigned)(walk ? (long long)sm_count() * 32 : rg);
        const size_t row_bytes = (size_t)a.dim * sizeof(T);
#define LIK_REDUCE16(CH_)                                                                                     \
  do {                                                                                                        \
    if (walk) bwd_dd_reduce16_walk_kernel<T, G, CH_><<<rgrid, 256, 0, st>>>(P, O), ::lik::count_launch();     \
    else bwd_dd_reduce16_kernel<T, G, CH_><<<rgrid, 256, 0, st>>>(P, O), ::lik::count_launch();               \
  } while (0)
        if (row_bytes <= 256) LIK_REDUCE16(1);
        else if (row_bytes <= 512) LIK_REDUCE16(2);
        else LIK_REDUCE16(4);
#undef LIK_REDUCE16
      } else {
        const unsigned rgrid = (unsigned)ceil_div(a.d.n_rows, 8);
        if (a.dim <= 128)
          bwd_dd_reduce_kernel<T, G, 1><<<rgrid, 256, 0, st>>>(P, O), ::lik::count_launch();
        else
          bwd_dd_reduce_kernel<T, G, 2><<<rgrid, 256, 0, st>>>(P, O), ::lik::count_launch();
      }
    } else {
      dim3 grid((unsigned)a.d.n_seq, (unsigned)ceil_div(a.d.max_len, DD_TOK));
      LIK_BY_CMAX(bwd_dd_owned_kernel, grid, P);
    }
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
      if (scatter_q && fast)
        bwd_scatter_kernel<T, true, true><<<grid, 256, 0, st>>>(P), ::lik::count_launch();
      else if (scatter_q)
        bwd_scatter_kernel<T, true, false><<<grid, 256, 0, st>>>(P), ::lik::count_launch();
      else if (fast)
        bwd_scatter_kernel<T, false, true><<<grid, 256, 0, st>>>(P), ::lik::count_launch();
      else
        bwd_scatter_kernel<T, false, false><<<grid, 256, 0, st>>>(P), ::lik::count_launch();
      LIK_CUDA_OK(cudaGetLastError());
    }
    if (P.gq32 && a.q.n_rows > 0) {
      bwd_finalize_kernel<T, G><<<(unsigned)ceil_div(a.q.n_rows, 8), 256, 0, st>>>(P.gq32, P.q, a.dim, a.normalize & LIK_NORM_Q, (G*)a.grad_q), ::lik::count_launch();
      LIK_CUDA_OK(cudaGetLastError());
    }
    if (P.gd32 && a.d.n_rows > 0) {
      bwd_finalize_kernel<T, G><<<(unsigned)ceil_div(a.d.n_rows, 8), 256, 0, st>>>(P.gd32, P.d, a.dim, a.normalize & LIK_NORM_D, (G*)a.grad_d), ::lik::count_launch();
      LIK_CUDA_OK(cudaGetLastError());
    }
  }
  if (fj) LIK_CUDA_OK(cudaStreamWaitEvent(st_main, fj->join, 0));
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
  if (a->normalize & LIK_NORM_Q) {
    float* w = (float*)((char*)a->workspace + pl.qn_off);
    int rc = launch_row_inv_norm(a->q.data, a->dtype, a->q.n_rows, a->dim, a->q.row_stride, kBwdNormEps, w, st);
    if (rc) return rc;
    qn = w;
  }
  if (a->normalize & LIK_NORM_D) {
    float* w = (float*)((char*)a->workspace + pl.dn_off);
    int rc = launch_row_inv_norm(a->d.data, a->dtype, a->d.n_rows, a->dim, a->d.row_stride, kBwdNormEps, w, st);
    if (rc) return rc;
    dn = w;
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
  P.perm_q = P.start_q = P.perm_d = P.start_d = nullptr;
  P.dq_split = pl.dq_split;
  P.dq_partial = pl.dq_split > 1 ? (float*)((char*)a->workspace + pl.dqp_off) : nullptr;
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
