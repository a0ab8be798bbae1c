// Per-query top-k selection and merge.
//
// One CTA per query row keeps the current best KP = pow2(k) candidates sorted in
// shared memory.  New candidates arrive KP at a time (a slice of a score row, or
// one of several already-selected lists), are bitonic-sorted, combined with the
// kept list by the "best of top[i] and block[KP-1-i]" step (which leaves the KP
// best of the union as a bitonic sequence) and re-sorted by a bitonic merge.  Blocks
// of a score row in which nothing beats the current k-th best are skipped after one
// read of their values.
// Order: better score first, ties to the lower document index; padding
// (index < 0) last.
#include <climits>

#include "lik_common.cuh"

namespace lik {

struct Cand {
  float key;  // score for largest=true, -score otherwise
  long long idx;
};

__device__ __forceinline__ bool before(const Cand& a, const Cand& b) {
  return a.key > b.key || (a.key == b.key && a.idx < b.idx);
}

constexpr long long kPadIdx = LLONG_MAX;

// sort KP entries in shared memory, best first
__device__ void bitonic_sort(float* key, long long* idx, int KP, int tid, int nthreads) {
  for (int size = 2; size <= KP; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int t = tid; t < (KP >> 1); t += nthreads) {
        int i = 2 * t - (t & (stride - 1));
        int j = i + stride;
        bool up = (i & size) == 0;  // this sub-sequence is ordered best first
        Cand a{key[i], idx[i]}, b{key[j], idx[j]};
        bool swap = up ? before(b, a) : before(a, b);
        if (swap) {
          key[i] = b.key;
          idx[i] = b.idx;
          key[j] = a.key;
          idx[j] = a.idx;
        }
      }
    }
  }
  __syncthreads();
}

// merge a bitonic sequence of KP entries into best-first order
__device__ void bitonic_merge(float* key, long long* idx, int KP, int tid, int nthreads) {
  for (int stride = KP >> 1; stride > 0; stride >>= 1) {
    __syncthreads();
    for (int t = tid; t < (KP >> 1); t += nthreads) {
      int i = 2 * t - (t & (stride - 1));
      int j = i + stride;
      Cand a{key[i], idx[i]}, b{key[j], idx[j]};
      if (before(b, a)) {
        key[i] = b.key;
        idx[i] = b.idx;
        key[j] = a.key;
        idx[j] = a.idx;
      }
    }
  }
  __syncthreads();
}

struct TopkParams {
  // mode 0: slices of a score row; mode 1: lists [n_lists, n_rows, k]
  int mode;
  const float* scores;
  long long n_cols, ld, index_offset;
  const float* cand_scores;
  const long long* cand_index;
  int n_lists;
  long long n_rows;
  int k, KP, largest, merge;
  float* out_scores;
  long long* out_index;
};

template <int NT, int MIN_CTAS>
__global__ void __launch_bounds__(NT, MIN_CTAS) topk_kernel(TopkParams P) {
  extern __shared__ unsigned char raw[];
  long long* top_i = reinterpret_cast<long long*>(raw);
  long long* blk_i = top_i + P.KP;
  float* top_k = reinterpret_cast<float*>(blk_i + P.KP);
  float* blk_k = top_k + P.KP;
  const int tid = threadIdx.x, nt = blockDim.x;
  const long long row = blockIdx.x;
  const float sgn = P.largest ? 1.f : -1.f;

  for (int t = tid; t < P.KP; t += nt) {
    float key = -INFINITY;
    long long id = kPadIdx;
    if (P.merge && t < P.k) {
      long long o = P.out_index[row * P.k + t];
      if (o >= 0) {
        id = o;
        key = sgn * P.out_scores[row * P.k + t];
      }
    }
    top_k[t] = key;
    top_i[t] = id;
  }
  __syncthreads();
  if (P.merge) bitonic_sort(top_k, top_i, P.KP, tid, nt);

  const long long n_blocks = P.mode == 0 ? (P.n_cols + P.KP - 1) / P.KP : P.n_lists;
  for (long long b = 0; b < n_blocks; ++b) {
    // A block of new candidates matters only if one of them beats the current k-th best: the kept list
    // never gets worse, so anything behind that entry can never reach the output.  Once the list is warm
    // almost every block is dismissed by this one pass over its values.
    if (P.mode == 0) {
      const Cand kth{top_k[P.k - 1], top_i[P.k - 1]};
      int hit = 0;
      for (int t = tid; t < P.KP; t += nt) {
        const long long c = b * P.KP + t;
        if (c < P.n_cols && before(Cand{sgn * P.scores[row * P.ld + c], c + P.index_offset}, kth)) hit = 1;
      }
      if (!__syncthreads_or(hit)) continue;
    }
    for (int t = tid; t < P.KP; t += nt) {
      float key = -INFINITY;
      long long id = kPadIdx;
      if (P.mode == 0) {
        long long c = b * P.KP + t;
        if (c < P.n_cols) {
          key = sgn * P.scores[row * P.ld + c];
          id = c + P.index_offset;
        }
      } else if (t < P.k) {
        long long o = (b * P.n_rows + row) * P.k + t;
        long long ci = P.cand_index[o];
        if (ci >= 0) {
          id = ci;
          key = sgn * P.cand_scores[o];
        }
      }
      blk_k[t] = key;
      blk_i[t] = id;
    }
    bitonic_sort(blk_k, blk_i, P.KP, tid, nt);
    for (int t = tid; t < P.KP; t += nt) {
      Cand a{top_k[t], top_i[t]}, c{blk_k[P.KP - 1 - t], blk_i[P.KP - 1 - t]};
      if (before(c, a)) {
        top_k[t] = c.key;
        top_i[t] = c.idx;
      }
    }
    bitonic_merge(top_k, top_i, P.KP, tid, nt);
  }
  for (int t = tid; t < P.k; t += nt) {
    bool pad = top_i[t] == kPadIdx;
    P.out_scores[row * P.k + t] = pad ? -sgn * INFINITY : sgn * top_k[t];
    P.out_index[row * P.k + t] = pad ? -1 : top_i[t];
  }
}

// Merge of the candidate lists the fused scoring kernel leaves (lik_fwd_tc.cu): list slot of (CTA c, tile
// group g) is c + g, each slot holds 2 * qpt lists of up to `cap` entries (unsorted), and CTA c of n_ctas can
// only have worked on the groups [n_groups * c / n_ctas, n_groups * (c + 1) / n_ctas] (a superset of the ones
// it really met; lists it never touched are empty).  A group is `mt` query tiles of `qpt` queries; with two
// tiles a query has one list per slot (tile * qpt + position), with one tile it has two (the kernel's two
// epilogue groups take alternate documents).  One CTA per (query, part): with few tile groups a query has lists
// from many CTAs, which would make one CTA walk hundreds of lists one after the other, so the CTAs' range is cut
// in `parts` parts merged side by side into [parts, n_q, k] lists, and the plain list merge (topk_kernel) makes
// the answer from those.
struct SlotParams {
  const float* keys;
  const int* idx;
  const int2* hdr;
  int cap, n_ctas, n_groups, mt, qpt;
  long long n_q, index_offset, n_lists;
  int k, KP, largest;
  float* out_scores;
  long long* out_index;
  int parts;  // > 1: blockIdx.y is the part, the outputs are [parts, n_q, k] and carry keys' signs undone
};

constexpr int SLOT_W = 256;  // merge width: the capacity of a candidate list, and the block size

// The kept list (SLOT_W entries, best first; the first k are the answer so far) absorbs the pending block.
__device__ void slots_flush(float* top_k, long long* top_i, float* blk_k, long long* blk_i, int n_pend, int tid) {
  if (tid >= n_pend) {
    blk_k[tid] = -INFINITY;
    blk_i[tid] = kPadIdx;
  }
  bitonic_sort(blk_k, blk_i, SLOT_W, tid, SLOT_W);
  {
    Cand a{top_k[tid], top_i[tid]}, c{blk_k[SLOT_W - 1 - tid], blk_i[SLOT_W - 1 - tid]};
    if (before(c, a)) {
      top_k[tid] = c.key;
      top_i[tid] = c.idx;
    }
  }
  bitonic_merge(top_k, top_i, SLOT_W, tid, SLOT_W);
}

// One CTA of SLOT_W threads per query.  Every list of the query is read once (one entry per thread); only
// entries that beat the current k-th best are collected, and the collected block is sorted and merged when it
// would overflow.  After the first list few entries survive the filter, so the sorts are rare.
__global__ void __launch_bounds__(SLOT_W) topk_slots_kernel(SlotParams P) {
  __shared__ long long top_i[SLOT_W], blk_i[SLOT_W];
  __shared__ float top_k[SLOT_W], blk_k[SLOT_W];
  __shared__ int n_pend_s;
  const int tid = threadIdx.x, lane = tid & 31;
  const long long q = blockIdx.x;
  const int tile = (int)(q / P.qpt), et = (int)(q - (long long)tile * P.qpt);
  const int g = tile / P.mt, m = tile - g * P.mt;
  const int n_sub = P.mt == 2 ? 1 : 2;
  top_k[tid] = -INFINITY;
  top_i[tid] = kPadIdx;
  if (tid == 0) n_pend_s = 0;
  __syncthreads();
  const int c_lo = (int)((long long)P.n_ctas * blockIdx.y / P.parts), c_hi = (int)((long long)P.n_ctas * (blockIdx.y + 1) / P.parts);
  for (int c = c_lo; c < c_hi; ++c) {
    const long long g_lo = (long long)P.n_groups * c / P.n_ctas, g_hi = (long long)P.n_groups * (c + 1) / P.n_ctas;
    if (g < g_lo || g > g_hi) continue;
    for (int sub = 0; sub < n_sub; ++sub) {
      const long long list = (long long)(c + g) * (2 * P.qpt) + (P.mt == 2 ? m : sub) * P.qpt + et;
      if (list >= P.n_lists) continue;
      int cnt = P.hdr[list].x;
      if (cnt > P.cap) cnt = P.cap;
      if (cnt <= 0) continue;
      int n_pend = n_pend_s;
      __syncthreads();  // every thread has read the count before this list's survivors are added to it
      if (n_pend + cnt > SLOT_W) {  // the pending block could overflow: absorb it first
        slots_flush(top_k, top_i, blk_k, blk_i, n_pend, tid);
        if (tid == 0) n_pend_s = 0;
        __syncthreads();
        n_pend = 0;
      }
      Cand mine{-INFINITY, kPadIdx};
      if (tid < cnt) mine = Cand{P.keys[list * P.cap + tid], (long long)P.idx[list * P.cap + tid]};
      const Cand kth{top_k[P.k - 1], top_i[P.k - 1]};
      const bool pass = tid < cnt && before(mine, kth);
      const unsigned mask = __ballot_sync(0xffffffffu, pass);
      int base = 0;
      if (lane == 0 && mask) base = atomicAdd(&n_pend_s, __popc(mask));
      base = __shfl_sync(0xffffffffu, base, 0);
      if (pass) {
        const int pos = base + __popc(mask & ((1u << lane) - 1u));
        blk_k[pos] = mine.key;
        blk_i[pos] = mine.idx;
      }
      __syncthreads();
    }
  }
  {
    const int n_pend = n_pend_s;
    __syncthreads();
    if (n_pend > 0) slots_flush(top_k, top_i, blk_k, blk_i, n_pend, tid);
  }
  const float sgn = P.largest ? 1.f : -1.f;
  if (tid < P.k) {
    const bool pad = top_i[tid] == kPadIdx;
    const long long o = ((long long)blockIdx.y * P.n_q + q) * P.k + tid;
    P.out_scores[o] = pad ? -sgn * INFINITY : sgn * top_k[tid];
    P.out_index[o] = pad ? -1 : top_i[tid] + P.index_offset;
  }
}

static int launch_topk(TopkParams& P, cudaStream_t st);

// In how many parts the lists of a query are merged first: a part should not walk more than about 24 CTAs' lists.
int topk_merge_parts(int n_ctas, int n_groups) {
  if (n_ctas <= 0 || n_groups <= 0) return 1;
  const int ctas_per_group = n_ctas / n_groups + 2;  // CTAs whose share of the units can touch one tile group
  if (ctas_per_group <= 32) return 1;
  const int parts = (ctas_per_group + 15) / 16;
  return parts > 16 ? 16 : parts;
}

int launch_topk_slots(const float* keys, const int* idx, const int2* hdr, long long n_lists, int cap, int n_ctas, int n_groups,
                      int mt, int qpt, long long n_q, int k, int largest, long long index_offset, float* out_scores,
                      long long* out_index, int parts, void* part_buf, cudaStream_t st) {
  if (n_q <= 0 || k <= 0) return LIK_OK;
  if (cap > SLOT_W || k > SLOT_W) {
    set_error("candidate lists of %d entries / k = %d exceed the merge width %d", cap, k, SLOT_W);
    return LIK_ERR_UNSUPPORTED;
  }
  if (parts <= 1 || !part_buf) {
    SlotParams P{keys, idx, hdr, cap, n_ctas, n_groups, mt, qpt, n_q, index_offset, n_lists, k, 2, largest, out_scores, out_index, 1};
    topk_slots_kernel<<<(unsigned)n_q, SLOT_W, 0, st>>>(P), ::lik::count_launch();
    LIK_CUDA_OK(cudaGetLastError());
    return LIK_OK;
  }
  float* part_scores = (float*)part_buf;
  long long* part_index = (long long*)((char*)part_buf + align_up((size_t)parts * n_q * k * sizeof(float), 8));
  SlotParams P{keys, idx, hdr, cap, n_ctas, n_groups, mt, qpt, n_q, index_offset, n_lists, k, 2, largest, part_scores, part_index, parts};
  topk_slots_kernel<<<dim3((unsigned)n_q, (unsigned)parts), SLOT_W, 0, st>>>(P), ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  TopkParams M{};
  M.mode = 1;
  M.cand_scores = part_scores;
  M.cand_index = part_index;
  M.n_lists = parts;
  M.n_rows = n_q;
  M.k = k;
  M.largest = largest;
  M.merge = 0;
  M.out_scores = out_scores;
  M.out_index = out_index;
  return launch_topk(M, st);
}


// ---------------------------------------------------------------------------------------------
// Top-k of score rows by selection instead of sorting (mode 0 of TopkParams).
//
// One CTA per row.  The row is taken in slabs of SEL_SLAB columns that live in registers (SEL_PER per thread,
// column = slab + j * threads + thread); the k entries kept so far (the running list, or the list the caller
// merges into) are SEL_OLD more elements per thread.  The k-th best key of all of them is
// found by a radix select on the order-preserving 32-bit image of the float (four passes of 256 shared-memory
// counters); entries above it are kept, and of the entries equal to it the ones with the lowest document
// index (a second select, on the index, only when the equal entries do not all fit).  The kept k are sorted
// once per slab that changed anything (best first, ties to the lower index) - a slab with nothing above the
// current k-th best is dismissed after one pass over its values.
// ---------------------------------------------------------------------------------------------
// Two shapes of the CTA, both with slabs of 4096 columns: 256 threads x (16 slab + 4 kept) elements for k <= 1024
// (three CTAs per SM), 1024 threads x (4 slab + 8 kept) elements for k <= LIK_TOPK_MAX = 8192.
constexpr int SEL_SLAB = 4096;
constexpr int SEL_K_SMALL = 1024;

// Monotone map float -> unsigned (larger float, larger key); 0 is below every float.
__device__ __forceinline__ unsigned sel_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct SelShared {
  int hist[256];
  int digit, want, n_eq, count;
};

// Radix select over the elements every thread holds: key[e] (larger is better) of the elements with on[e], `nbits`
// wide.  Returns the key of rank `want` (1 = the best) to every thread; *need_eq = how many of the elements equal to
// it belong to the best `want`, *n_eq = how many elements equal it.  All threads of the block call it.
template <typename K, int NE>
__device__ K block_select(const K (&key)[NE], const bool (&on)[NE], int nbits, int want, SelShared* sh, int* need_eq, int* n_eq) {
  const int tid = threadIdx.x, lane = tid & 31;
  K prefix = 0;
  for (int shift = nbits - 8; shift >= 0; shift -= 8) {
    if (tid < 256) sh->hist[tid] = 0;
    __syncthreads();
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      // bits above this digit must match what is fixed already (nothing in the first pass)
      const bool same = shift + 8 >= nbits || (key[e] >> (shift + 8)) == (prefix >> (shift + 8));
      if (on[e] && same) atomicAdd(&sh->hist[(int)((key[e] >> shift) & 255)], 1);
    }
    __syncthreads();
    if (tid < 32) {
      // lane l owns the bins 255 - 8 l ... 248 - 8 l (best first); find the bin in which the running count reaches `want`
      int c[8], s = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        c[i] = sh->hist[255 - 8 * lane - i];
        s += c[i];
      }
      int incl = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int above = incl - s;
      if (above < want && want <= incl) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (above < want && want <= above + c[i]) {
            sh->digit = 255 - 8 * lane - i;
            sh->want = want - above;
            sh->n_eq = c[i];
          }
          above += c[i];
        }
      }
    }
    __syncthreads();
    prefix |= (K)sh->digit << shift;
    want = sh->want;
  }
  *need_eq = want;
  *n_eq = sh->n_eq;
  __syncthreads();  // the shared words may be rewritten by the next call
  return prefix;
}

template <int SEL_T, int SEL_PER, int SEL_OLD, int MIN_CTAS>
__global__ void __launch_bounds__(SEL_T, MIN_CTAS) topk_select_kernel(TopkParams P) {
  static_assert(SEL_T * SEL_PER == SEL_SLAB, "a slab is 4096 columns");
  constexpr int SEL_NE = SEL_PER + SEL_OLD;
  extern __shared__ unsigned char raw[];
  long long* top_i = reinterpret_cast<long long*>(raw);
  float* top_k = reinterpret_cast<float*>(top_i + P.KP);
  __shared__ SelShared sh;
  const int tid = threadIdx.x;
  const long long row = blockIdx.x;
  const float sgn = P.largest ? 1.f : -1.f;

  // the kept list: what the caller merges into, or empty
  for (int t = tid; t < P.KP; t += SEL_T) {
    float key = -INFINITY;
    long long id = kPadIdx;
    if (P.merge && t < P.k) {
      const long long o = P.out_index[row * P.k + t];
      if (o >= 0) {
        id = o;
        key = sgn * P.out_scores[row * P.k + t] + 0.f;
      }
    }
    top_k[t] = key;
    top_i[t] = id;
  }
  if (tid == 0) sh.count = 0;
  __syncthreads();
  bool sorted = !P.merge;  // an empty list is in order; a caller's list is taken as it comes
  // k-th best of the kept list as a key (0: the list is not full) - a slab must beat it to matter
  unsigned kth_key = 0;

  const long long n_slabs = (P.n_cols + SEL_SLAB - 1) / SEL_SLAB;
  for (long long sl = 0; sl < (n_slabs > 0 ? n_slabs : 1); ++sl) {
    float f[SEL_NE];
    unsigned u[SEL_NE];
    bool on[SEL_NE];
    int hit = 0;
#pragma unroll
    for (int j = 0; j < SEL_PER; ++j) {
      const long long c = sl * SEL_SLAB + (long long)j * SEL_T + tid;
      on[j] = c < P.n_cols;
      f[j] = on[j] ? sgn * P.scores[row * P.ld + c] + 0.f : -INFINITY;
      u[j] = on[j] ? sel_key(f[j]) : 0u;
      if (on[j] && u[j] >= kth_key) hit = 1;  // (an equal key only matters against a higher kept index; rare, so let it through)
    }
    const bool last = sl + 1 >= n_slabs;
    if (!__syncthreads_or(hit) && !(last && !sorted)) continue;
#pragma unroll
    for (int m = 0; m < SEL_OLD; ++m) {
      const int t = m * SEL_T + tid;
      on[SEL_PER + m] = t < P.k && top_i[t] != kPadIdx;
      f[SEL_PER + m] = on[SEL_PER + m] ? top_k[t] : -INFINITY;
      u[SEL_PER + m] = on[SEL_PER + m] ? sel_key(f[SEL_PER + m]) : 0u;
    }
    // kept entries carry their document index; a slab element's is its column
    long long my_idx[SEL_OLD];
#pragma unroll
    for (int m = 0; m < SEL_OLD; ++m) my_idx[m] = on[SEL_PER + m] ? top_i[m * SEL_T + tid] : kPadIdx;
    // how many real elements there are: with fewer than k, all of them are kept
    int mine = 0;
#pragma unroll
    for (int e = 0; e < SEL_NE; ++e) mine += on[e] ? 1 : 0;
    // block-wide count of the elements
    {
      int w = mine;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
      if ((tid & 31) == 0 && w) atomicAdd(&sh.count, w);
    }
    __syncthreads();
    const int n_all = sh.count;
    __syncthreads();
    if (tid == 0) sh.count = 0;
    const int want = n_all < P.k ? n_all : P.k;
    unsigned T = 0;
    int need_eq = 0, n_eq = 0;
    unsigned long long Ti = 0;  // ties: the kept ones have ~index >= Ti
    bool all_ties = true;
    if (want > 0 && n_all > P.k) {
      T = block_select<unsigned, SEL_NE>(u, on, 32, want, &sh, &need_eq, &n_eq);
      if (need_eq < n_eq) {
        // more entries equal the k-th best than fit: the lowest document indices win
        unsigned long long ik[SEL_NE];
        bool tie[SEL_NE];
#pragma unroll
        for (int e = 0; e < SEL_NE; ++e) {
          tie[e] = on[e] && u[e] == T;
          const long long id = e < SEL_PER ? sl * SEL_SLAB + (long long)e * SEL_T + tid + P.index_offset : my_idx[e - SEL_PER];
          ik[e] = ~(unsigned long long)id;
        }
        int ne2 = 0, nn2 = 0;
        Ti = block_select<unsigned long long, SEL_NE>(ik, tie, 64, need_eq, &sh, &ne2, &nn2);
        all_ties = false;
      }
    }
    __syncthreads();  // everyone has read the kept list; it is rebuilt now
    // gather the kept elements (any order), pad, sort
    int my_pos[SEL_NE];
#pragma unroll
    for (int e = 0; e < SEL_NE; ++e) {
      bool take = on[e] && (n_all <= P.k || u[e] > T);
      if (on[e] && n_all > P.k && u[e] == T) {
        const long long id = e < SEL_PER ? sl * SEL_SLAB + (long long)e * SEL_T + tid + P.index_offset : my_idx[e - SEL_PER];
        take = all_ties || ~(unsigned long long)id >= Ti;
      }
      my_pos[e] = take ? atomicAdd(&sh.count, 1) : -1;
    }
    __syncthreads();
    const int n_kept = sh.count;
    __syncthreads();
    if (tid == 0) sh.count = 0;
#pragma unroll
    for (int e = 0; e < SEL_NE; ++e) {
      if (my_pos[e] >= 0 && my_pos[e] < P.KP) {
        top_k[my_pos[e]] = f[e];
        top_i[my_pos[e]] = e < SEL_PER ? sl * SEL_SLAB + (long long)e * SEL_T + tid + P.index_offset : my_idx[e - SEL_PER];
      }
    }
    for (int t = n_kept + tid; t < P.KP; t += SEL_T) {
      top_k[t] = -INFINITY;
      top_i[t] = kPadIdx;
    }
    __syncthreads();
    bitonic_sort(top_k, top_i, P.KP, tid, SEL_T);
    sorted = true;
    kth_key = (n_kept >= P.k) ? sel_key(top_k[P.k - 1]) : 0u;
  }
  for (int t = tid; t < P.k; t += SEL_T) {
    const bool pad = top_i[t] == kPadIdx;
    P.out_scores[row * P.k + t] = pad ? -sgn * INFINITY : sgn * top_k[t];
    P.out_index[row * P.k + t] = pad ? -1 : top_i[t];
  }
}

static int launch_topk(TopkParams& P, cudaStream_t st) {
  if (P.n_rows <= 0 || P.k <= 0) return LIK_OK;
  int KP = 1;
  while (KP < P.k) KP <<= 1;
  if (KP < 2) KP = 2;
  P.KP = KP;
  if (P.mode == 0) {
    const size_t smem = (size_t)KP * (sizeof(long long) + sizeof(float));
    if (P.k <= SEL_K_SMALL) {
      topk_select_kernel<256, 16, SEL_K_SMALL / 256, 3><<<(unsigned)P.n_rows, 256, smem, st>>>(P), ::lik::count_launch();
    } else {
      static bool raised[64] = {false};  // by device ordinal: the kept list of a large k needs more than 48 KB
      int dev = 0;
      LIK_CUDA_OK(cudaGetDevice(&dev));
      if (dev < 0 || dev >= 64 || !raised[dev]) {
        LIK_CUDA_OK(cudaFuncSetAttribute(topk_select_kernel<1024, 4, LIK_TOPK_MAX / 1024, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)((size_t)LIK_TOPK_MAX * (sizeof(long long) + sizeof(float)))));
        if (dev >= 0 && dev < 64) raised[dev] = true;
      }
      topk_select_kernel<1024, 4, LIK_TOPK_MAX / 1024, 1><<<(unsigned)P.n_rows, 1024, smem, st>>>(P), ::lik::count_launch();
    }
    LIK_CUDA_OK(cudaGetLastError());
    return LIK_OK;
  }
  size_t smem = (size_t)KP * 2 * (sizeof(long long) + sizeof(float));
  if (smem > 48 * 1024) {
    static bool raised[64] = {false};
    int dev = 0;
    LIK_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !raised[dev]) {
      LIK_CUDA_OK(cudaFuncSetAttribute(topk_kernel<1024, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)((size_t)LIK_TOPK_MAX * 2 * (sizeof(long long) + sizeof(float)))));
      if (dev >= 0 && dev < 64) raised[dev] = true;
    }
  }
  if (KP > 1024) topk_kernel<1024, 1><<<(unsigned)P.n_rows, 1024, smem, st>>>(P), ::lik::count_launch();
  else topk_kernel<256, 6><<<(unsigned)P.n_rows, 256, smem, st>>>(P), ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

}  // namespace lik

extern "C" int lik_topk_rows(const float* scores, int64_t n_rows, int64_t n_cols, int64_t ld, int32_t k, int32_t largest,
                             int64_t index_offset, int32_t merge, float* out_scores, int64_t* out_index,
                             lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(k > 0 && k <= LIK_TOPK_MAX, "k=%d outside [1, %d]", k, LIK_TOPK_MAX);
  LIK_REQUIRE(n_rows >= 0 && n_cols >= 0 && ld >= n_cols, "bad score matrix shape");
  LIK_REQUIRE(out_scores && out_index && (scores || n_cols == 0), "NULL pointer");
  TopkParams P{};
  P.mode = 0;
  P.scores = scores;
  P.n_cols = n_cols;
  P.ld = ld;
  P.index_offset = index_offset;
  P.n_rows = n_rows;
  P.k = k;
  P.largest = largest;
  P.merge = merge;
  P.out_scores = out_scores;
  P.out_index = (long long*)out_index;
  return launch_topk(P, (cudaStream_t)stream);
}

extern "C" int lik_topk_merge(const float* cand_scores, const int64_t* cand_index, int32_t n_lists, int64_t n_rows,
                              int32_t k, int32_t largest, float* out_scores, int64_t* out_index, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(k > 0 && k <= LIK_TOPK_MAX, "k=%d outside [1, %d]", k, LIK_TOPK_MAX);
  LIK_REQUIRE(n_lists >= 0 && n_rows >= 0, "negative size");
  LIK_REQUIRE(out_scores && out_index && ((cand_scores && cand_index) || n_lists == 0), "NULL pointer");
  TopkParams P{};
  P.mode = 1;
  P.cand_scores = cand_scores;
  P.cand_index = (const long long*)cand_index;
  P.n_lists = n_lists;
  P.n_rows = n_rows;
  P.k = k;
  P.largest = largest;
  P.merge = 0;
  P.out_scores = out_scores;
  P.out_index = (long long*)out_index;
  return launch_topk(P, (cudaStream_t)stream);
}
