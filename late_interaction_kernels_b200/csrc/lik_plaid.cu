// PLAID / ColBERTv2 compressed-index kernels: decompress (centroid gather +
// residual bit-unpack + bucket lookup + optional L2 norm), the IVF-prune
// approximate score, and the grad_Q backward of the residual scorer.
#include "lik_common.cuh"
#include "lik_plaid_row.cuh"

namespace lik {

struct PlaidView {
  const int* codes;
  const unsigned char* residuals;
  long long n_tokens;
  const void* centroids;
  int centroid_dtype;
  int n_centroids;
  const float* bucket_weights;
  int nbits, dim, packed_dim;
};

static PlaidView make_plaid_view(const lik_plaid_index& ix) {
  PlaidView v;
  v.codes = ix.codes;
  v.residuals = ix.residuals;
  v.n_tokens = ix.n_tokens;
  v.centroids = ix.centroids;
  v.centroid_dtype = ix.centroid_dtype;
  v.n_centroids = ix.n_centroids;
  v.bucket_weights = ix.bucket_weights;
  v.nbits = ix.nbits;
  v.dim = ix.dim;
  v.packed_dim = (ix.dim * ix.nbits + 7) / 8;
  return v;
}

__device__ __forceinline__ float centroid_at(const PlaidView& v, long long off) {
  if (v.centroid_dtype == LIK_F16) return __half2float(((const __half*)v.centroids)[off]);
  if (v.centroid_dtype == LIK_BF16) return __bfloat162float(((const __nv_bfloat16*)v.centroids)[off]);
  return ((const float*)v.centroids)[off];
}

// Reconstruct feature f of token tok: centroid + bucket weight.
// Feature f lives in byte f / cpb at bit offset (f % cpb) * nbits.
__device__ __forceinline__ float plaid_feature(const PlaidView& v, long long tok, int code, int f, const float* bw) {
  const int cpb = 8 / v.nbits;
  const unsigned byte = v.residuals[tok * v.packed_dim + f / cpb];
  const unsigned bucket = (byte >> ((f % cpb) * v.nbits)) & ((1u << v.nbits) - 1u);
  return centroid_at(v, (long long)code * v.dim + f) + bw[bucket];
}

__device__ __forceinline__ int checked_code(const PlaidView& v, long long tok, int* status) {
  int c = v.codes[tok];
  if (c < 0 || c >= v.n_centroids) {
    if (status) atomicOr(status, LIK_DEV_CODE_RANGE);
    c = 0;
  }
  return c;
}

// One warp per token.  FMAX = ceil(dim / 32) register slots per lane.
template <typename O, int FMAX>
__global__ void __launch_bounds__(256) plaid_decompress_kernel(PlaidView v, long long tok0, long long count, int normalize,
                                                             O* __restrict__ out, int* status) {
  __shared__ float bw[256];
  for (int b = threadIdx.x; b < (1 << v.nbits); b += blockDim.x) bw[b] = v.bucket_weights[b];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= count) return;
  const long long tok = tok0 + w;
  const int code = checked_code(v, tok, status);
  float e[FMAX];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < FMAX; ++c) {
    int f = c * 32 + lane;
    e[c] = f < v.dim ? plaid_feature(v, tok, code, f, bw) : 0.f;
    ss = fmaf(e[c], e[c], ss);
  }
  float inv = 1.f;
  if (normalize) inv = 1.f / fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
#pragma unroll
  for (int c = 0; c < FMAX; ++c) {
    int f = c * 32 + lane;
    if (f < v.dim) out[w * v.dim + f] = from_f32<O>(e[c] * inv);
  }
}

// Half-warp per run of tokens, the arithmetic of lik_plaid_row.cuh (the scoring kernel's producer warps decode
// tokens with the same functions, so rows written here and tiles decoded there hold the same bits):
// 16-byte centroid loads, one load for a lane's eight bucket codes, 16-byte stores.
constexpr int PD_RUN = 64;  // consecutive tokens per half-warp

template <typename O, bool CF32>
__global__ void __launch_bounds__(256) plaid_decompress16_kernel(PlaidSrc S, long long tok0, long long count, O* __restrict__ out,
                                                               int* status) {
  __shared__ float bw[256];
  for (int b = threadIdx.x; b < (1 << S.nbits); b += blockDim.x) bw[b] = S.bucket_weights[b];
  __syncthreads();
  const int lane = threadIdx.x & 31, hl = lane & 15;
  const long long first = ((long long)blockIdx.x * 16 + (threadIdx.x >> 4)) * PD_RUN;  // first token of this half-warp's run
  long long left = count - first;
  const int n = left <= 0 ? 0 : (left < PD_RUN ? (int)left : PD_RUN);
  O* dst = out + first * S.dim + hl * 8;
  const int dim = S.dim;
  auto sink = [&](int t, const float (&e)[8]) {
    O* p = dst + (long long)t * dim;
    if (sizeof(O) == 4) {
      reinterpret_cast<float4*>(p)[0] = make_float4(e[0], e[1], e[2], e[3]);
      reinterpret_cast<float4*>(p)[1] = make_float4(e[4], e[5], e[6], e[7]);
    } else {
      *reinterpret_cast<uint4*>(p) = plaid_pack16(e, dtype_of<O>::value == LIK_F16);
    }
  };
  plaid_decode_range<CF32, CF32 ? 4 : 8>(S, bw, tok0 + first, n, PD_RUN, lane, hl * 8 < dim, status, sink);
}

// Approximate score: one warp per document, lane = query token (chunks of 32).  The document's codes are read 32
// at a time (one per lane, coalesced) and handed round with shuffles; the score-table rows of eight tokens are in
// flight at once (the table, n_centroids x lq floats, is an L2 resident gather target).
__global__ void __launch_bounds__(256) plaid_approx_kernel(const float* __restrict__ qcs, int n_centroids, int lq,
                                                         const int* __restrict__ codes, long long n_docs, int max_ld,
                                                         const long long* __restrict__ lens, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long b = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (b >= n_docs) return;
  long long len = lens[b];
  if (len > max_ld) len = max_ld;
  const int* __restrict__ doc = codes + b * max_ld;
  float total = 0.f;
  for (int s0 = 0; s0 < lq; s0 += 32) {
    const int s = s0 + lane;
    const float* __restrict__ col = qcs + (s < lq ? s : 0);
    float m = -INFINITY;
    for (int t0 = 0; t0 < len; t0 += 32) {
      int c = t0 + lane < len ? __ldg(doc + t0 + lane) : 0;
      if (c < 0 || c >= n_centroids) c = 0;  // out-of-range codes read centroid 0
      const int n = (int)min((long long)32, len - t0);
#pragma unroll 1
      for (int u0 = 0; u0 < n; u0 += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int cu = __shfl_sync(0xffffffffu, c, (u0 + u) & 31);
          v[u] = u0 + u < n ? __ldg(col + (long long)cu * lq) : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) m = fmaxf(m, v[u]);
      }
    }
    total += warp_sum((s < lq && m != -INFINITY) ? m : 0.f);
  }
  if (lane == 0) out[b] = total;
}

// grad_Q of the residual scorer: one warp per (query, token).
template <typename T, int FMAX>
__global__ void __launch_bounds__(256) plaid_bwd_dq_kernel(PlaidView v, int max_ld, long long n_docs, const T* __restrict__ q,
                                                         int n_q, int lq, const float* __restrict__ g,
                                                         const int* __restrict__ argmax, int normalize,
                                                         float* __restrict__ grad_q) {
  __shared__ float bw[256];
  for (int b = threadIdx.x; b < (1 << v.nbits); b += blockDim.x) bw[b] = v.bucket_weights[b];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= (long long)n_q * lq) return;
  const int i = (int)(w / lq), s = (int)(w - (long long)i * lq);
  float acc[FMAX];
#pragma unroll
  for (int c = 0; c < FMAX; ++c) acc[c] = 0.f;
  for (long long j = 0; j < n_docs; ++j) {
    const int t = argmax[((long long)i * n_docs + j) * lq + s];
    if (t < 0 || t >= max_ld) continue;
    const long long tok = j * max_ld + t;
    const int code = checked_code(v, tok, nullptr);
    float e[FMAX];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < FMAX; ++c) {
      int f = c * 32 + lane;
      e[c] = f < v.dim ? plaid_feature(v, tok, code, f, bw) : 0.f;
      ss = fmaf(e[c], e[c], ss);
    }
    float f = g[(long long)i * n_docs + j];
    if (normalize) f *= 1.f / fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
#pragma unroll
    for (int c = 0; c < FMAX; ++c) acc[c] = fmaf(f, e[c], acc[c]);
  }
  const T* qrow = q + w * v.dim;
  if (normalize) {
    float qv[FMAX];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < FMAX; ++c) {
      int f = c * 32 + lane;
      qv[c] = f < v.dim ? to_f32(qrow[f]) : 0.f;
      ss = fmaf(qv[c], qv[c], ss);
    }
    const float inv = 1.f / fmaxf(sqrtf(warp_sum(ss)), 1e-6f);
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < FMAX; ++c) {
      qv[c] *= inv;
      dot = fmaf(acc[c], qv[c], dot);
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int c = 0; c < FMAX; ++c) acc[c] = (acc[c] - dot * qv[c]) * inv;
  }
#pragma unroll
  for (int c = 0; c < FMAX; ++c) {
    int f = c * 32 + lane;
    if (f < v.dim) grad_q[w * v.dim + f] = acc[c];
  }
}

static int check_index(const lik_plaid_index* ix) {
  LIK_REQUIRE(ix != nullptr, "index is NULL");
  LIK_REQUIRE(ix->nbits == 2 || ix->nbits == 4 || ix->nbits == 8, "nbits must be 2, 4, or 8; got %d", ix->nbits);
  LIK_REQUIRE(ix->dim > 0 && ix->dim <= 1024, "dim %d outside (0, 1024]", ix->dim);
  LIK_REQUIRE(ix->n_centroids > 0, "n_centroids must be positive");
  LIK_REQUIRE(ix->centroid_dtype == LIK_F32 || ix->centroid_dtype == LIK_F16 || ix->centroid_dtype == LIK_BF16,
              "centroid dtype %d not supported", ix->centroid_dtype);
  LIK_REQUIRE(ix->codes && ix->residuals && ix->centroids && ix->bucket_weights, "NULL index pointer");
  return LIK_OK;
}

}  // namespace lik

#define LIK_BY_FMAX(fm, CALL4, CALL8, CALL16, CALL32) \
  do {                                                \
    if ((fm) <= 4) {                                  \
      CALL4;                                          \
    } else if ((fm) <= 8) {                           \
      CALL8;                                          \
    } else if ((fm) <= 16) {                          \
      CALL16;                                         \
    } else {                                          \
      CALL32;                                         \
    }                                                 \
  } while (0)

extern "C" int lik_plaid_decompress(const lik_plaid_index* index, int64_t token_begin, int64_t token_count,
                                    int32_t normalize, void* out, int32_t out_dtype, int32_t* status,
                                    lik_stream_t stream) {
  using namespace lik;
  int rc = check_index(index);
  if (rc) return rc;
  LIK_REQUIRE(token_begin >= 0 && token_count >= 0 && token_begin + token_count <= index->n_tokens,
              "token range [%lld, +%lld) outside the index", (long long)token_begin, (long long)token_count);
  LIK_REQUIRE(out != nullptr || token_count == 0, "out is NULL");
  if (token_count == 0) return LIK_OK;
  PlaidView v = make_plaid_view(*index);
  cudaStream_t st = (cudaStream_t)stream;
  {
    PlaidSrc S{index->codes, index->residuals, index->centroids, index->bucket_weights, index->centroid_dtype, index->n_centroids,
               index->nbits, v.packed_dim, index->dim, normalize ? 1 : 0};
    if (plaid_row16_ok(S) && ((uintptr_t)out % 16) == 0 && (out_dtype == LIK_F32 || out_dtype == LIK_F16 || out_dtype == LIK_BF16)) {
      const unsigned blocks = (unsigned)ceil_div(token_count, 16 * PD_RUN);
      const bool cf32 = index->centroid_dtype == LIK_F32;
#define LIK_DEC16(O)                                                                                                  \
  do {                                                                                                                \
    if (cf32)                                                                                                         \
      plaid_decompress16_kernel<O, true><<<blocks, 256, 0, st>>>(S, token_begin, token_count, (O*)out, status), ::lik::count_launch(); \
    else                                                                                                              \
      plaid_decompress16_kernel<O, false><<<blocks, 256, 0, st>>>(S, token_begin, token_count, (O*)out, status), ::lik::count_launch(); \
  } while (0)
      if (out_dtype == LIK_F32)
        LIK_DEC16(float);
      else if (out_dtype == LIK_F16)
        LIK_DEC16(__half);
      else
        LIK_DEC16(__nv_bfloat16);
#undef LIK_DEC16
      LIK_CUDA_OK(cudaGetLastError());
      return LIK_OK;
    }
  }
  unsigned grid = (unsigned)ceil_div(token_count, 8);
  const int fm = (v.dim + 31) / 32;
#define LIK_DEC(O, F) plaid_decompress_kernel<O, F><<<grid, 256, 0, st>>>(v, token_begin, token_count, normalize, (O*)out, status), ::lik::count_launch()
  switch (out_dtype) {
    case LIK_F32:
      LIK_BY_FMAX(fm, LIK_DEC(float, 4), LIK_DEC(float, 8), LIK_DEC(float, 16), LIK_DEC(float, 32));
      break;
    case LIK_F16:
      LIK_BY_FMAX(fm, LIK_DEC(__half, 4), LIK_DEC(__half, 8), LIK_DEC(__half, 16), LIK_DEC(__half, 32));
      break;
    case LIK_BF16:
      LIK_BY_FMAX(fm, LIK_DEC(__nv_bfloat16, 4), LIK_DEC(__nv_bfloat16, 8), LIK_DEC(__nv_bfloat16, 16),
                  LIK_DEC(__nv_bfloat16, 32));
      break;
    default:
      set_error("out_dtype %d not supported", out_dtype);
      return LIK_ERR_INVALID;
  }
#undef LIK_DEC
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

extern "C" int lik_plaid_approx(const float* qcs, int32_t n_centroids, int32_t lq, const int32_t* codes, int64_t n_docs,
                                int32_t max_ld, const int64_t* doc_lengths, float* out, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(n_centroids > 0 && lq >= 0 && n_docs >= 0 && max_ld >= 0, "bad sizes");
  if (n_docs == 0) return LIK_OK;
  LIK_REQUIRE(qcs && codes && doc_lengths && out, "NULL pointer");
  plaid_approx_kernel<<<(unsigned)ceil_div(n_docs, 8), 256, 0, (cudaStream_t)stream>>>(
      qcs, n_centroids, lq, codes, n_docs, max_ld, (const long long*)doc_lengths, out), ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

extern "C" int lik_plaid_bwd_dq(const lik_plaid_index* index, int32_t max_ld, int64_t n_docs, const void* q,
                                int32_t q_dtype, int32_t n_q, int32_t lq, const float* grad_scores,
                                const int32_t* argmax, int32_t normalize, float* grad_q, lik_stream_t stream) {
  using namespace lik;
  int rc = check_index(index);
  if (rc) return rc;
  LIK_REQUIRE(n_docs >= 0 && max_ld >= 0 && n_docs * (int64_t)max_ld <= index->n_tokens, "padded index smaller than n_docs*max_ld");
  if ((int64_t)n_q * lq == 0) return LIK_OK;
  LIK_REQUIRE(q && grad_scores && argmax && grad_q, "NULL pointer");
  PlaidView v = make_plaid_view(*index);
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = (unsigned)ceil_div((int64_t)n_q * lq, 8);
  const int fm = (v.dim + 31) / 32;
#define LIK_PB(T, F) \
  plaid_bwd_dq_kernel<T, F><<<grid, 256, 0, st>>>(v, max_ld, n_docs, (const T*)q, n_q, lq, grad_scores, argmax, normalize, grad_q), ::lik::count_launch()
  switch (q_dtype) {
    case LIK_F32:
      LIK_BY_FMAX(fm, LIK_PB(float, 4), LIK_PB(float, 8), LIK_PB(float, 16), LIK_PB(float, 32));
      break;
    case LIK_F16:
      LIK_BY_FMAX(fm, LIK_PB(__half, 4), LIK_PB(__half, 8), LIK_PB(__half, 16), LIK_PB(__half, 32));
      break;
    case LIK_BF16:
      LIK_BY_FMAX(fm, LIK_PB(__nv_bfloat16, 4), LIK_PB(__nv_bfloat16, 8), LIK_PB(__nv_bfloat16, 16),
                  LIK_PB(__nv_bfloat16, 32));
      break;
    default:
      set_error("q_dtype %d not supported", q_dtype);
      return LIK_ERR_INVALID;
  }
#undef LIK_PB
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}
