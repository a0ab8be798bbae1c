// Shared device/host helpers for the MaxSim kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "lik_b200.h"

namespace lik {

// ---- host side error reporting ------------------------------------------------
void set_error(const char* fmt, ...);
const char* get_error();

#define LIK_CUDA_OK(expr)                                                                      \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      ::lik::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return LIK_ERR_CUDA;                                                                     \
    }                                                                                          \
  } while (0)

#define LIK_REQUIRE(cond, ...)        \
  do {                                \
    if (!(cond)) {                    \
      ::lik::set_error(__VA_ARGS__);  \
      return LIK_ERR_INVALID;         \
    }                                 \
  } while (0)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
int sm_count();
// every kernel launch of the library is followed by this (read back through lik_launch_count)
void count_launch();
unsigned long long launch_count();

// ---- element types -------------------------------------------------------------
struct e4m3_t {
  uint8_t bits;
};

template <typename T>
struct dtype_of;
template <>
struct dtype_of<float> {
  static constexpr int value = LIK_F32;
};
template <>
struct dtype_of<__half> {
  static constexpr int value = LIK_F16;
};
template <>
struct dtype_of<__nv_bfloat16> {
  static constexpr int value = LIK_BF16;
};
template <>
struct dtype_of<e4m3_t> {
  static constexpr int value = LIK_E4M3;
};

inline size_t dtype_size(int dt) { return dt == LIK_F32 ? 4 : (dt == LIK_E4M3 ? 1 : 2); }

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(e4m3_t x) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(x.bits, __NV_E4M3);
  return __half2float(__half(h));
}

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) {
  return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// ---- sequence views --------------------------------------------------------------
// Device copy of lik_seqs plus the optional per-row inverse norms computed for
// fused L2 normalisation.
struct SeqView {
  const void* data;
  long long row_stride;
  long long n_rows;
  int n_seq;
  int max_len;
  long long seq_stride;
  const int* cu;
  const int* lens;
  const unsigned char* mask;
  const float* scale;
  float scale_scalar;
  const float* inv_norm;  // [n_rows] or nullptr
};

inline SeqView make_view(const lik_seqs& s, const float* inv_norm) {
  SeqView v;
  v.data = s.data;
  v.row_stride = s.row_stride;
  v.n_rows = s.n_rows;
  v.n_seq = s.n_seq;
  v.max_len = s.max_len;
  v.seq_stride = s.seq_stride;
  v.cu = s.cu;
  v.lens = s.lens;
  v.mask = s.mask;
  v.scale = s.scale;
  v.scale_scalar = s.scale_scalar;
  v.inv_norm = inv_norm;
  return v;
}

// First row and token count of sequence i.  Padded lengths are clamped to
// [0, max_len]; a violation is reported through *status.
__device__ __forceinline__ void seq_bounds(const SeqView& v, int i, long long& row0, int& len, int* status) {
  if (v.cu) {
    int a = v.cu[i], b = v.cu[i + 1];
    row0 = a;
    len = b > a ? b - a : 0;
    if ((long long)a + len > v.n_rows) {
      len = v.n_rows > a ? (int)(v.n_rows - a) : 0;
      if (status) atomicOr(status, LIK_DEV_LEN_RANGE);
    }
  } else {
    row0 = (long long)i * v.seq_stride;
    len = v.max_len;
    if (v.lens) {
      int l = v.lens[i];
      if (l > v.max_len || l < 0) {
        if (status) atomicOr(status, LIK_DEV_LEN_RANGE);
        l = l < 0 ? 0 : v.max_len;
      }
      len = l;
    }
  }
}

// Multiplier applied to every dot product involving this row: dequantisation
// scale times the fused-normalisation factor.
__device__ __forceinline__ float row_factor(const SeqView& v, long long row) {
  float f = v.scale_scalar;
  if (v.scale) f *= v.scale[row];
  if (v.inv_norm) f *= v.inv_norm[row];
  return f;
}

__device__ __forceinline__ bool row_valid(const SeqView& v, long long row) { return v.mask ? v.mask[row] != 0 : true; }

// Decode score slot p into (query, document).  Returns false (and flags status)
// when a pair-list entry is out of range.
struct PairMap {
  int pairing;
  int group;
  int n_q, n_d;
  const int* pair_q;
  const int* pair_d;
  long long n_scores;
};

__device__ __forceinline__ bool decode_pair(const PairMap& m, long long p, int& i, int& j, int* status) {
  if (m.pairing == LIK_PAIR_CROSS) {
    i = (int)(p / m.n_d);
    j = (int)(p - (long long)i * m.n_d);
    return true;
  }
  if (m.pairing == LIK_PAIR_GROUPED) {
    j = (int)p;
    i = (int)(p / m.group);
    return true;
  }
  i = m.pair_q[p];
  j = m.pair_d[p];
  if (i < 0 || i >= m.n_q || j < 0 || j >= m.n_d) {
    if (status) atomicOr(status, LIK_DEV_PAIR_RANGE);
    return false;
  }
  return true;
}

inline long long n_scores_of(int pairing, int n_q, int n_d, long long n_pairs) {
  if (pairing == LIK_PAIR_CROSS) return (long long)n_q * n_d;
  if (pairing == LIK_PAIR_GROUPED) return n_d;
  return n_pairs;
}

// Lanes of the warp whose value equals this lane's, for values in [0, 2^nbits); lanes with a negative value are in
// nobody's set (their own result is meaningless).  One ballot per bit: the cost does not depend on how many
// different values the warp holds, unlike match.any, which on this GPU slows down with every distinct value.
__device__ __forceinline__ unsigned warp_peers(int v, int nbits) {
  unsigned peers = __ballot_sync(0xffffffffu, v >= 0);
  for (int b = 0; b < nbits; ++b) {
    const bool bit = (v >> b) & 1;
    const unsigned m = __ballot_sync(0xffffffffu, bit);
    peers &= bit ? m : ~m;
  }
  return peers;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace lik
