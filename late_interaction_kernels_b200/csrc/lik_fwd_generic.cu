// Portable fp32-accumulate MaxSim forward: any element type, any embedding
// width, every layout and pairing.  It is the exact path (fp32 FMA in a fixed
// order, so fp32 inputs keep fp32 accuracy) and the home of shapes the tcgen05
// kernel does not take (odd widths, pair lists).
#include <atomic>

#include "lik_common.cuh"

namespace lik {

namespace {
thread_local char g_err[512] = "";
std::atomic<unsigned long long> g_launches{0};
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* get_error() { return g_err; }

int sm_count() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n > 0 ? n : 148;
}

// ---------------------------------------------------------------------------------
// Row inverse norms: out[r] = 1 / max(||x_r||, eps).  One warp per row.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void row_inv_norm_kernel(const T* __restrict__ x, long long n_rows, int dim, long long stride, float eps,
                                    float* __restrict__ out) {
  long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  int lane = threadIdx.x & 31;
  const T* p = x + row * stride;
  float ss = 0.f;
  for (int k = lane; k < dim; k += 32) {
    float v = to_f32(p[k]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) out[row] = 1.0f / fmaxf(sqrtf(ss), eps);
}

int launch_row_inv_norm(const void* data, int dtype, long long n_rows, int dim, long long stride, float eps, float* out,
                        cudaStream_t st) {
  if (n_rows <= 0) return LIK_OK;
  const int warps = 8;
  dim3 grid((unsigned)ceil_div(n_rows, warps)), block(warps * 32);
  switch (dtype) {
    case LIK_F32:
      row_inv_norm_kernel<<<grid, block, 0, st>>>((const float*)data, n_rows, dim, stride, eps, out), ::lik::count_launch();
      break;
    case LIK_F16:
      row_inv_norm_kernel<<<grid, block, 0, st>>>((const __half*)data, n_rows, dim, stride, eps, out), ::lik::count_launch();
      break;
    case LIK_BF16:
      row_inv_norm_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)data, n_rows, dim, stride, eps, out), ::lik::count_launch();
      break;
    case LIK_E4M3:
      row_inv_norm_kernel<<<grid, block, 0, st>>>((const e4m3_t*)data, n_rows, dim, stride, eps, out), ::lik::count_launch();
      break;
    default:
      set_error("unknown dtype %d", dtype);
      return LIK_ERR_INVALID;
  }
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

// y[row] = round_to_T(x[row] / max(||x[row]||, eps)), dense rows of `dim` elements.  One warp per row; the row is
// read once (it stays in registers between the norm and the scaling for widths up to 256).
template <typename T>
__global__ void row_normalize_kernel(const T* __restrict__ x, long long n_rows, int dim, long long stride, float eps,
                                     T* __restrict__ y) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const T* p = x + row * stride;
  T* o = y + row * dim;
  float v[8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int k = c * 32 + lane;
    v[c] = k < dim ? to_f32(p[k]) : 0.f;
    ss = fmaf(v[c], v[c], ss);
  }
  for (int k = 256 + lane; k < dim; k += 32) {
    const float w = to_f32(p[k]);
    ss = fmaf(w, w, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / fmaxf(sqrtf(ss), eps);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int k = c * 32 + lane;
    if (k < dim) o[k] = from_f32<T>(v[c] * inv);
  }
  for (int k = 256 + lane; k < dim; k += 32) o[k] = from_f32<T>(to_f32(p[k]) * inv);
}

// Normalised copy of a 16-bit matrix (dense output rows).
int launch_row_normalize(const void* data, int dtype, long long n_rows, int dim, long long stride, float eps, void* out,
                         cudaStream_t st) {
  if (n_rows <= 0) return LIK_OK;
  const int warps = 8;
  dim3 grid((unsigned)ceil_div(n_rows, warps)), block(warps * 32);
  switch (dtype) {
    case LIK_F16:
      row_normalize_kernel<<<grid, block, 0, st>>>((const __half*)data, n_rows, dim, stride, eps, (__half*)out), ::lik::count_launch();
      break;
    case LIK_BF16:
      row_normalize_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)data, n_rows, dim, stride, eps, (__nv_bfloat16*)out), ::lik::count_launch();
      break;
    default:
      set_error("normalised copies exist for 16-bit inputs only (dtype %d)", dtype);
      return LIK_ERR_INVALID;
  }
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

// ---------------------------------------------------------------------------------
// Generic forward.  One CTA (4 warps) per score slot.  Tiles: 32 query tokens
// (lane = token) x 64 document tokens (16 per warp) x 32 embedding columns.
// ---------------------------------------------------------------------------------
constexpr int G_QC = 32;  // query tokens per tile
constexpr int G_DC = 64;  // document tokens per tile
constexpr int G_KC = 32;  // embedding columns per staging step
constexpr int G_TPW = G_DC / 4;
constexpr int G_QS = G_QC + 1;  // padded row of the transposed query tile (bank-conflict-free)

struct GenericFwdParams {
  SeqView q, d;
  PairMap pm;
  int dim;
  int dim_pad;  // dim rounded up to G_KC
  float* scores;
  int* argmax;
  int argmax_stride;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(128) fwd_generic_kernel(GenericFwdParams P) {
  extern __shared__ float smem[];
  float* Qs = smem;                          // [dim_pad][G_QS]  (column-major: lane = query token)
  float* Ds = smem + (size_t)P.dim_pad * G_QS;  // [G_DC][G_KC]
  __shared__ float red_m[4][G_QC];
  __shared__ int red_i[4][G_QC];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* __restrict__ Qg = (const T*)P.q.data;
  const T* __restrict__ Dg = (const T*)P.d.data;

  for (long long p = blockIdx.x; p < P.pm.n_scores; p += gridDim.x) {
    int qi, dj;
    bool ok = decode_pair(P.pm, p, qi, dj, P.status);
    long long qrow0 = 0, drow0 = 0;
    int qlen = 0, dlen = 0;
    if (ok) {
      seq_bounds(P.q, qi, qrow0, qlen, P.status);
      seq_bounds(P.d, dj, drow0, dlen, P.status);
    }
    if (P.argmax && qlen > P.argmax_stride) {
      if (tid == 0 && P.status) atomicOr(P.status, LIK_DEV_ARGMAX_STRIDE);
      qlen = P.argmax_stride;
    }
    float score = 0.f;  // meaningful in warp 0
    for (int qc = 0; qc < qlen; qc += G_QC) {
      __syncthreads();
      // stage the query tile, transposed, as fp32
      for (int idx = tid; idx < P.dim_pad * G_QC; idx += 128) {
        int s = idx / P.dim_pad, k = idx - s * P.dim_pad;
        float v = 0.f;
        if (qc + s < qlen && k < P.dim) v = to_f32(Qg[(qrow0 + qc + s) * P.q.row_stride + k]);
        Qs[k * G_QS + s] = v;
      }
      float m = -INFINITY;
      int mi = -1;
      for (int dc = 0; dc < dlen; dc += G_DC) {
        float acc[G_TPW];
#pragma unroll
        for (int t = 0; t < G_TPW; ++t) acc[t] = 0.f;
        for (int kc = 0; kc < P.dim_pad; kc += G_KC) {
          __syncthreads();
          for (int idx = tid; idx < G_DC * G_KC; idx += 128) {
            int t = idx / G_KC, k = idx - t * G_KC;
            float v = 0.f;
            if (dc + t < dlen && kc + k < P.dim) v = to_f32(Dg[(drow0 + dc + t) * P.d.row_stride + kc + k]);
            Ds[t * G_KC + k] = v;
          }
          __syncthreads();
#pragma unroll
          for (int k4 = 0; k4 < G_KC; k4 += 4) {
            float q0 = Qs[(kc + k4 + 0) * G_QS + lane];
            float q1 = Qs[(kc + k4 + 1) * G_QS + lane];
            float q2 = Qs[(kc + k4 + 2) * G_QS + lane];
            float q3 = Qs[(kc + k4 + 3) * G_QS + lane];
#pragma unroll
            for (int t = 0; t < G_TPW; ++t) {
              float4 dv = *reinterpret_cast<const float4*>(&Ds[(warp * G_TPW + t) * G_KC + k4]);
              acc[t] = fmaf(q0, dv.x, acc[t]);
              acc[t] = fmaf(q1, dv.y, acc[t]);
              acc[t] = fmaf(q2, dv.z, acc[t]);
              acc[t] = fmaf(q3, dv.w, acc[t]);
            }
          }
        }
#pragma unroll
        for (int t = 0; t < G_TPW; ++t) {
          int tok = dc + warp * G_TPW + t;
          if (tok < dlen) {
            long long row = drow0 + tok;
            if (row_valid(P.d, row)) {
              float v = acc[t] * row_factor(P.d, row);
              if (v > m) {
                m = v;
                mi = tok;
              }
            }
          }
        }
      }
      // combine the four warps (each saw a different quarter of every tile)
      red_m[warp][lane] = m;
      red_i[warp][lane] = mi;
      __syncthreads();
      if (warp == 0) {
        float bm = red_m[0][lane];
        int bi = red_i[0][lane];
#pragma unroll
        for (int w = 1; w < 4; ++w) {
          float wm = red_m[w][lane];
          int wi = red_i[w][lane];
          if (wi >= 0 && (bi < 0 || wm > bm || (wm == bm && wi < bi))) {
            bm = wm;
            bi = wi;
          }
        }
        int s = qc + lane;
        float val = 0.f;
        if (s < qlen) {
          long long qrow = qrow0 + s;
          if (bi >= 0 && row_valid(P.q, qrow)) val = bm * row_factor(P.q, qrow);
          if (P.argmax) P.argmax[p * P.argmax_stride + s] = bi;
        }
        score += warp_sum(val);
      }
    }
    if (warp == 0) {
      if (lane == 0) P.scores[p] = score;
      if (P.argmax) {
        int from = qlen < 0 ? 0 : qlen;
        for (int s = from + lane; s < P.argmax_stride; s += 32) P.argmax[p * P.argmax_stride + s] = -1;
      }
    }
  }
}

int launch_fwd_generic(const lik_fwd_args& a, const float* qn, const float* dn, cudaStream_t st) {
  GenericFwdParams P;
  P.q = make_view(a.q, qn);
  P.d = make_view(a.d, dn);
  P.pm = PairMap{a.pairing, a.group, a.q.n_seq, a.d.n_seq, a.pair_q, a.pair_d,
                 n_scores_of(a.pairing, a.q.n_seq, a.d.n_seq, a.n_pairs)};
  P.dim = a.dim;
  P.dim_pad = (int)align_up((size_t)a.dim, G_KC);
  P.scores = a.scores;
  P.argmax = a.argmax;
  P.argmax_stride = a.argmax_stride;
  P.status = a.status;
  if (P.pm.n_scores <= 0) return LIK_OK;
  size_t smem = ((size_t)P.dim_pad * G_QS + (size_t)G_DC * G_KC) * sizeof(float);
  if (smem > 200 * 1024) {
    set_error("embedding dim %d too large for the portable kernel", a.dim);
    return LIK_ERR_UNSUPPORTED;
  }
  unsigned grid = (unsigned)(P.pm.n_scores < (1ll << 30) ? P.pm.n_scores : (1ll << 30));
#define LIK_LAUNCH_GENERIC(T)                                                                                    \
  do {                                                                                                           \
    LIK_CUDA_OK(cudaFuncSetAttribute(fwd_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    fwd_generic_kernel<T><<<grid, 128, smem, st>>>(P), ::lik::count_launch();                                                           \
  } while (0)
  switch (a.dtype) {
    case LIK_F32:
      LIK_LAUNCH_GENERIC(float);
      break;
    case LIK_F16:
      LIK_LAUNCH_GENERIC(__half);
      break;
    case LIK_BF16:
      LIK_LAUNCH_GENERIC(__nv_bfloat16);
      break;
    case LIK_E4M3:
      LIK_LAUNCH_GENERIC(e4m3_t);
      break;
    default:
      set_error("unknown dtype %d", a.dtype);
      return LIK_ERR_INVALID;
  }
#undef LIK_LAUNCH_GENERIC
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

}  // namespace lik
