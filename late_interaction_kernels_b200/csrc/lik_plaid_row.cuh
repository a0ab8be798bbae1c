// Reconstruction of one PLAID / ColBERTv2 token by a half-warp (16 lanes), shared by the stand-alone
// decompress kernel and by the producer warps of the tensor-core scorer so that both give the same
// bits.  Lane hl of the half-warp owns the eight consecutive features [8 hl, 8 hl + 8):
//   - one 16-byte load of the centroid row slice (fp16 / bf16; two for fp32 centroids),
//   - one load of the nbits bytes that hold the eight bucket codes (feature f sits in byte
//     f / (8/nbits) at bit (f % (8/nbits)) * nbits, little-endian inside the byte, so the eight codes
//     of a lane are eight consecutive nbits-wide fields of one little-endian word),
//   - bucket weights from a table in shared memory, fp32 add, and for the L2 norm a half-warp
//     shuffle reduction in a fixed order.
// Needs: embedding width a multiple of 8, centroid rows 16-byte aligned, residual rows nbits-byte aligned.
#pragma once

#include "lik_common.cuh"

namespace lik {

struct PlaidSrc {
  const int* codes;                // [n_tokens]
  const unsigned char* residuals;  // [n_tokens, packed_dim]
  const void* centroids;           // [n_centroids, dim]
  const float* bucket_weights;     // [1 << nbits]
  int centroid_dtype;              // LIK_F32 / LIK_F16 / LIK_BF16
  int n_centroids;
  int nbits;                       // 2, 4 or 8
  int packed_dim;                  // ceil(dim * nbits / 8)
  int dim;
  int normalize;                   // divide the reconstructed token by max(||x||, 1e-12)
};

// raw loads of one token slice: issued for several tokens before any of them is used
template <bool CF32>
struct PlaidRaw {
  uint4 c0;                 // centroid slice: eight 16-bit values, or the first four fp32 values
  unsigned long long w;     // the lane's eight bucket codes
};
template <>
struct PlaidRaw<true> {
  uint4 c0, c1;             // eight fp32 centroid values
  unsigned long long w;
};

__device__ __forceinline__ int plaid_code(const PlaidSrc& S, long long tok, int* status) {
  int c = __ldg(S.codes + tok);
  if (c < 0 || c >= S.n_centroids) {
    if (status) atomicOr(status, LIK_DEV_CODE_RANGE);
    c = 0;
  }
  return c;
}

template <bool CF32>
__device__ __forceinline__ PlaidRaw<CF32> plaid_load(const PlaidSrc& S, long long tok, int code, int hl, bool on) {
  PlaidRaw<CF32> r;
  r.c0 = make_uint4(0, 0, 0, 0);
  r.w = 0ull;
  if constexpr (CF32) r.c1 = make_uint4(0, 0, 0, 0);
  if (!on) return r;
  const long long off = (long long)code * S.dim + hl * 8;
  if constexpr (CF32) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const float*>(S.centroids) + off);
    r.c0 = __ldg(p);
    r.c1 = __ldg(p + 1);
  } else {
    r.c0 = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(S.centroids) + off));
  }
  const unsigned char* rp = S.residuals + tok * S.packed_dim + hl * S.nbits;
  if (S.nbits == 2)
    r.w = __ldg(reinterpret_cast<const unsigned short*>(rp));
  else if (S.nbits == 4)
    r.w = __ldg(reinterpret_cast<const unsigned int*>(rp));
  else
    r.w = __ldg(reinterpret_cast<const unsigned long long*>(rp));
  return r;
}

// e[i] = centroid + bucket weight for the lane's eight features; bw points at the table in shared memory
template <bool CF32>
__device__ __forceinline__ void plaid_features(const PlaidSrc& S, const PlaidRaw<CF32>& r, const float* bw, float (&e)[8]) {
  float c[8];
  if constexpr (CF32) {
    c[0] = __uint_as_float(r.c0.x); c[1] = __uint_as_float(r.c0.y); c[2] = __uint_as_float(r.c0.z); c[3] = __uint_as_float(r.c0.w);
    c[4] = __uint_as_float(r.c1.x); c[5] = __uint_as_float(r.c1.y); c[6] = __uint_as_float(r.c1.z); c[7] = __uint_as_float(r.c1.w);
  } else if (S.centroid_dtype == LIK_BF16) {
    c[0] = __uint_as_float(r.c0.x << 16); c[1] = __uint_as_float(r.c0.x & 0xffff0000u);
    c[2] = __uint_as_float(r.c0.y << 16); c[3] = __uint_as_float(r.c0.y & 0xffff0000u);
    c[4] = __uint_as_float(r.c0.z << 16); c[5] = __uint_as_float(r.c0.z & 0xffff0000u);
    c[6] = __uint_as_float(r.c0.w << 16); c[7] = __uint_as_float(r.c0.w & 0xffff0000u);
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.c0.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&r.c0.y));
    const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&r.c0.z)), f = __half22float2(*reinterpret_cast<const __half2*>(&r.c0.w));
    c[0] = a.x; c[1] = a.y; c[2] = b.x; c[3] = b.y; c[4] = d.x; c[5] = d.y; c[6] = f.x; c[7] = f.y;
  }
  const unsigned mask = (1u << S.nbits) - 1u;
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = c[i] + bw[(unsigned)(r.w >> (i * S.nbits)) & mask];
}

// Multiplier that normalises the token: 1 / max(||x||, 1e-12), the same on all 16 lanes of the half-warp
// (lanes whose features lie beyond the width pass zeros).  1.0f when the index is scored un-normalised.
__device__ __forceinline__ float plaid_inv_norm(const PlaidSrc& S, const float (&e)[8]) {
  if (!S.normalize) return 1.f;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(e[i], e[i], ss);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  return 1.f / fmaxf(sqrtf(ss), 1e-12f);
}

// A half-warp decodes the `n` consecutive tokens [tok0, tok0 + n) and hands the lane's eight finished values of
// token t (0-based) to sink(t, values).  The centroid codes are read 16 at a time (one per lane, a chunk ahead of
// their use) and passed around with shuffles; U row loads are in flight per half-warp.  Both half-warps of a warp
// must call this with the same n_uniform >= n (the shuffles are warp-wide): tokens past n are computed on zeros and
// dropped.  `lane` is the lane in the warp, `lane_on` whether the lane's features exist (8 * (lane & 15) < dim).
template <bool CF32, int U, typename Sink>
__device__ __forceinline__ void plaid_decode_range(const PlaidSrc& S, const float* bw, long long tok0, int n, int n_uniform, int lane,
                                                   bool lane_on, int* status, Sink sink) {
  const int hl = lane & 15;
  int code_next = hl < n ? plaid_code(S, tok0 + hl, status) : 0;
  for (int c0 = 0; c0 < n_uniform; c0 += 16) {
    const int code_cur = code_next;
    code_next = c0 + 16 + hl < n ? plaid_code(S, tok0 + c0 + 16 + hl, status) : 0;
#pragma unroll 1
    for (int b = 0; b < 16; b += U) {
      PlaidRaw<CF32> r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int t = c0 + b + u;
        const int code = __shfl_sync(0xffffffffu, code_cur, (lane & 16) | (b + u));
        r[u] = plaid_load<CF32>(S, tok0 + t, code, hl, t < n && lane_on);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int t = c0 + b + u;
        float e[8];
        plaid_features<CF32>(S, r[u], bw, e);
        if (!lane_on) {
#pragma unroll
          for (int i = 0; i < 8; ++i) e[i] = 0.f;
        }
        const float inv = plaid_inv_norm(S, e);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] *= inv;
        if (t < n && lane_on) sink(t, e);
      }
    }
  }
}

// eight fp32 values -> eight 16-bit operand values (bf16 or fp16), round to nearest even
__device__ __forceinline__ uint4 plaid_pack16(const float (&v)[8], bool f16) {
  uint4 o;
  if (f16) {
    __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
    o.x = *reinterpret_cast<unsigned*>(&a); o.y = *reinterpret_cast<unsigned*>(&b);
    o.z = *reinterpret_cast<unsigned*>(&c); o.w = *reinterpret_cast<unsigned*>(&d);
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    o.x = *reinterpret_cast<unsigned*>(&a); o.y = *reinterpret_cast<unsigned*>(&b);
    o.z = *reinterpret_cast<unsigned*>(&c); o.w = *reinterpret_cast<unsigned*>(&d);
  }
  return o;
}

// the index can go through the half-warp path
inline bool plaid_row16_ok(const PlaidSrc& S) {
  const size_t ceb = S.centroid_dtype == LIK_F32 ? 4 : 2;
  return S.dim % 8 == 0 && S.dim <= 128 && ((uintptr_t)S.centroids % 16) == 0 && ((size_t)S.dim * ceb) % 16 == 0 &&
         ((uintptr_t)S.residuals % 8) == 0 && S.packed_dim == S.dim * S.nbits / 8 && (S.packed_dim % S.nbits) == 0;
}

}  // namespace lik
