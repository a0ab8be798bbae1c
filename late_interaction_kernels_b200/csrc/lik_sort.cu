// Stable LSD radix sort of 32-bit (key, value) pairs, 8 bits per pass.
//
// A pass is three kernels over blocks of RS_BLOCK consecutive elements: (1) per-block histogram of the digit,
// (2) exclusive scan of the histograms in (digit, block) order, which gives every block the first output
// position of each digit, (3) scatter: inside a block every warp owns a contiguous slice, counts its digits,
// the block turns the counts into per-(warp, digit) start positions (digit-major, then warp), and the warp
// places its elements in slice order, ranking equal digits of one 32-element round with eight ballots.  Every step
// keeps the input order of equal keys, so the sort is stable and its result does not depend on timing.
#include "lik_sort.cuh"

namespace lik {

namespace {
constexpr int RS_WARPS = 8;
constexpr int RS_PER_WARP = 512;                  // elements per warp slice (16 rounds of 32)
constexpr int RS_BLOCK = RS_WARPS * RS_PER_WARP;  // 4096 elements per block

__global__ void __launch_bounds__(RS_WARPS * 32) rs_hist_kernel(const unsigned* __restrict__ keys, long long n, int shift,
                                                              unsigned* __restrict__ hist, int n_blocks) {
  __shared__ unsigned h[256];
  h[threadIdx.x] = 0;
  __syncthreads();
  const long long b0 = (long long)blockIdx.x * RS_BLOCK;
  for (int i = threadIdx.x; i < RS_BLOCK; i += RS_WARPS * 32) {
    const long long e = b0 + i;
    if (e < n) atomicAdd(&h[(keys[e] >> shift) & 255u], 1u);
  }
  __syncthreads();
  hist[(long long)threadIdx.x * n_blocks + blockIdx.x] = h[threadIdx.x];
}

// exclusive scan of `total` words in place; one CTA of 1024 threads walks the array with a running carry
__global__ void __launch_bounds__(1024) rs_scan_kernel(unsigned* __restrict__ a, long long total) {
  __shared__ unsigned warp_sum_s[32];
  __shared__ unsigned carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (long long base = 0; base < total; base += 1024) {
    const long long i = base + tid;
    const unsigned v = i < total ? a[i] : 0u;
    unsigned incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned x = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += x;
    }
    if (lane == 31) warp_sum_s[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      unsigned w = warp_sum_s[lane], wi = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned x = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += x;
      }
      warp_sum_s[lane] = wi - w;  // exclusive prefix of the warp totals
    }
    __syncthreads();
    const unsigned carry = carry_s;
    if (i < total) a[i] = carry + warp_sum_s[warp] + incl - v;
    __syncthreads();
    if (tid == 1023) carry_s = carry + warp_sum_s[31] + incl;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(RS_WARPS * 32) rs_scatter_kernel(const unsigned* __restrict__ keys_in, const unsigned* __restrict__ vals_in,
                                                                 unsigned* __restrict__ keys_out, unsigned* __restrict__ vals_out,
                                                                 long long n, int shift, const unsigned* __restrict__ offs, int n_blocks) {
  __shared__ unsigned cnt[RS_WARPS][256];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < RS_WARPS * 256; i += RS_WARPS * 32) (&cnt[0][0])[i] = 0;
  __syncthreads();
  const long long s0 = (long long)blockIdx.x * RS_BLOCK + (long long)warp * RS_PER_WARP;
  for (int r = 0; r < RS_PER_WARP; r += 32) {
    const long long e = s0 + r + lane;
    if (e < n) atomicAdd(&cnt[warp][(keys_in[e] >> shift) & 255u], 1u);
  }
  __syncthreads();
  {  // thread d: first output position of digit d for every warp of this block
    unsigned base = offs[(long long)tid * n_blocks + blockIdx.x];
    for (int w = 0; w < RS_WARPS; ++w) {
      const unsigned c = cnt[w][tid];
      cnt[w][tid] = base;
      base += c;
    }
  }
  __syncthreads();
  for (int r = 0; r < RS_PER_WARP; r += 32) {
    const long long e = s0 + r + lane;
    const bool in = e < n;
    const unsigned k = in ? keys_in[e] : 0u;
    const unsigned v = in ? vals_in[e] : 0u;
    const int d = in ? (int)((k >> shift) & 255u) : -1;  // lanes past the end match nobody
    const unsigned peers = warp_peers(d, 8);
    if (in) {
      const unsigned pos = cnt[warp][d] + (unsigned)__popc(peers & ((1u << lane) - 1u));
      keys_out[pos] = k;
      vals_out[pos] = v;
    }
    __syncwarp();
    if (in && (peers & ((1u << lane) - 1u)) == 0) cnt[warp][d] += (unsigned)__popc(peers);
    __syncwarp();
  }
}

__global__ void run_starts_kernel(const unsigned* __restrict__ keys, long long n, int n_seg, int* __restrict__ start) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n_seg) return;
  long long lo = 0, hi = n;  // first position whose key is >= i
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (keys[mid] < (unsigned)i) lo = mid + 1;
    else hi = mid;
  }
  start[i] = (int)lo;
}
}  // namespace

size_t sort_pairs_scratch(long long n) {
  const long long n_blocks = ceil_div(n > 0 ? n : 1, RS_BLOCK);
  return align_up((size_t)(n > 0 ? n : 1) * 4, 256) * 2 + align_up((size_t)n_blocks * 256 * 4, 256);
}

int stable_sort_pairs(unsigned* keys, unsigned* vals, long long n, int key_bits, void* scratch, cudaStream_t st) {
  if (n <= 0) return LIK_OK;
  const int n_blocks = (int)ceil_div(n, RS_BLOCK);
  char* sc = (char*)scratch;
  unsigned* alt_k = (unsigned*)sc;
  unsigned* alt_v = (unsigned*)(sc + align_up((size_t)n * 4, 256));
  unsigned* hist = (unsigned*)(sc + 2 * align_up((size_t)n * 4, 256));
  int passes = (key_bits + 7) / 8;
  if (passes < 1) passes = 1;
  if (passes & 1) ++passes;  // an even number of passes leaves the result in the caller's arrays
  unsigned *ki = keys, *vi = vals, *ko = alt_k, *vo = alt_v;
  for (int p = 0; p < passes; ++p) {
    const int shift = p * 8;
    rs_hist_kernel<<<n_blocks, RS_WARPS * 32, 0, st>>>(ki, n, shift, hist, n_blocks), ::lik::count_launch();
    rs_scan_kernel<<<1, 1024, 0, st>>>(hist, (long long)n_blocks * 256), ::lik::count_launch();
    rs_scatter_kernel<<<n_blocks, RS_WARPS * 32, 0, st>>>(ki, vi, ko, vo, n, shift, hist, n_blocks), ::lik::count_launch();
    LIK_CUDA_OK(cudaGetLastError());
    unsigned* t = ki; ki = ko; ko = t;
    t = vi; vi = vo; vo = t;
  }
  return LIK_OK;
}

int run_starts(const unsigned* sorted_keys, long long n, int n_seg, int* start, cudaStream_t st) {
  run_starts_kernel<<<(unsigned)ceil_div(n_seg + 1, 256), 256, 0, st>>>(sorted_keys, n, n_seg, start), ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

}  // namespace lik
