// Blackwell tensor-core MaxSim forward (sm_100a: TMA + tcgen05.mma + TMEM).
//
// GEMM view: rows = query tokens (A operand, K-major, 128 per tile), columns = document tokens (B
// operand, K-major, up to 256 per tile), K = embedding width.  A CTA is persistent: it keeps one or
// two 128-row query tiles resident in shared memory and streams document tiles through a TMA ring.
// Every document tile feeds one MMA group per resident query tile; the fp32 accumulator of query
// tile m lives in TMEM columns [256 m, 256 m + 256).  A tile never spans two documents, so the
// epilogue is: per thread (= one query token = one TMEM lane) a running max over the tile's columns,
// carried across the tiles of a document; at the end of the document the 128 row maxima are summed
// per query (fixed order) into one score.  Scores for a (query, document) pair have exactly one
// writer, so the forward is bitwise reproducible.
//
// Warp roles (640 threads): warp 0 = producer (TMA; the only role that walks the work units, which it publishes in
// a small ring in shared memory); warp 1 = MMA issuer + TMEM owner, driven by one word per ring stage that the
// producer writes; warps 2-9 = epilogue group 0 (accumulator 0), warps 10-17 = epilogue group 1 (accumulator 1);
// warps 18-19 decode tokens beside warp 0 in the PLAID kernels and are idle otherwise (they also round the block up
// to the register-allocation granule).  An accumulator is single-buffered (two 256-column accumulators fill TMEM).
// What bounds the kernel is the chain of dependent steps an epilogue warp runs per (query tile, document): hand-shake,
// three or four TMEM round trips with their folds, the hand-over between the two halves of a group, the emit.  So the
// code on that chain is kept short and free of branches, and paths that are rare (documents whose mask has holes)
// get their own copy of the loop instead of a test inside the common one.
//
// The same kernel scores into a matrix, keeps the winners for the backward, or keeps a per-query top-k (candidate
// lists per CTA and query, merged by a second kernel); documents come from a matrix through TMA or are decoded
// from a PLAID index by the producer warps.
//
// Every mbarrier wait is bounded: on expiry the CTA raises LIK_DEV_WAIT_TIMEOUT in the status word,
// sets a shared abort flag, drains its TMA copies, frees TMEM and returns.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "lik_common.cuh"
#include "lik_plaid_row.cuh"
#include "lik_tc.cuh"
#include "lik_tc_ptx.cuh"

namespace lik {

namespace {

#ifndef LIK_TILE_N
#define LIK_TILE_N 256
#endif
constexpr int TILE_N = LIK_TILE_N;     // document tokens per TMA stage = columns of one accumulator
constexpr int ACC_COLS = 256;          // TMEM columns reserved per accumulator
static_assert(TILE_N <= ACC_COLS && TILE_N % 32 == 0, "a stage must fit one accumulator");
constexpr int BOX_ROWS = 64;        // granule of the document TMA boxes (64, 128, 192 or 256 rows)
constexpr int SLAB_BYTES_ROW = 128; // one swizzle span: 64 two-byte or 128 one-byte elements
constexpr int MAX_SLABS = 2;
constexpr int NUM_THREADS = 640;
constexpr int EPI_THREADS = 128;     // threads per half of an epilogue group (one per accumulator row)
constexpr int GROUP_WARPS = 8;
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;  // default limit of a wait: about 2 s at 2 GHz
constexpr int UNIT_RING = 8;                  // slots of the producer -> epilogue unit ring
constexpr int LONG_DOC_TOKENS = 2048;         // problems whose documents can be this long run the kernel with the lazy winner scan
constexpr int UNIT_LEN_MASK = 0xFFFFFF;       // unit_info.x: document length in the low 24 bits,
constexpr int UNIT_SLOT_SHIFT = 24;           // the multiplier slot of its first tile in bits 24..28, LEN_FLAG_MASKED above

// ---------------------------------------------------------------------------------------------
// Kernel parameters
// ---------------------------------------------------------------------------------------------
// Fused top-k (retrieve).  Instead of a score matrix the epilogue keeps candidate lists: one list per
// (CTA, query) for every query of the tile groups the CTA works on.  A CTA meets the documents of a
// group in ascending order, so a list is append-only in document order; a score enters when it beats the
// list's threshold (strictly: an equal score that arrives later has a higher index and loses the tie).
// A full list (TOPK_CAP entries) is cut back to its k best by the warp that owns it, which also raises
// the threshold to the k-th best.  The lists of a query are merged by lik::launch_topk_slots afterwards.
// List slot of (CTA c, group g) is c + g: a CTA works on a contiguous range of groups and the ranges of
// consecutive CTAs are ordered, so c + g is unique among the pairs that occur.
constexpr int TOPK_CAP = 256;  // entries per list: eight per lane of the owning warp
struct TopkOut {
  float* cand_key;  // [n_slots * qpg][TOPK_CAP]: score (negated when the smallest are wanted)
  int* cand_idx;    // same shape: document index
  int2* hdr;        // [n_slots * qpg]: x = entries in the list, y = threshold as an ordered key (0: none yet)
  int k;
  int qpg;          // lists per slot: two query tiles' worth
  int largest;
  int doc_base;     // added to the document index stored with a candidate
  int n_lists;      // lists allocated (the kernel checks every list number against it)
};

// One row of the pair-list table (LIK_PAIR_LIST): written by list_units_kernel, read by the producer.
//   x = query (0 for a pair that is out of range), y = first document row, z = document length, w = unused
struct TcParams {
  SeqView q, d;
  int pairing;       // CROSS, GROUPED or LIST
  int group;         // GROUPED: documents per query
  int n_q, n_d;
  int elt_bytes;     // 1 or 2
  int ab_format;     // instruction-descriptor operand format
  int n_slabs;       // 128-byte K slabs per row
  int k_steps;       // MMA K steps (32 bytes each)
  int stages;        // document ring depth
  int q_per_tile;    // whole queries per 128-row tile (when q_chunks == 1)
  int q_chunks;      // 128-row chunks per query (> 1: one query chunk per tile)
  int n_tiles;       // query tiles
  int mt;            // query tiles resident per CTA (1 or 2)
  int n_sb;          // CROSS: the documents are walked in n_sb super-blocks of sb_docs documents (L2-sized)
  int sb_docs;
  long long n_flat;  // GROUPED / LIST: number of units
  const int4* list_tab;  // LIST: one row per pair
  float* scores;
  float* partial;    // [n_tiles, n_d] when q_chunks > 1
  int* argmax;
  int argmax_stride;
  int* status;
  const int* tile_q0;  // packed queries: tile m holds queries [tile_q0[m], tile_q0[m+1]); tile_q0[-1] is the tile count
  int d_len_flagged;  // d.lens carries LEN_FLAG_MASKED on documents whose mask is not a plain prefix
  // Per-column multipliers that are one fp32 per document row (inverse norms, or per-token scales) and whose layout
  // allows it travel with the tile: the producer copies the tile's run of them into a slot of a small ring in shared
  // memory (bulk copy on the stage's barrier) instead of the epilogue fetching them from device memory per tile.
  const float* col_src;  // nullptr: the epilogue stages the multipliers itself
  // Two rings of sc_per = stages + 1 slots, one per accumulator (tiles that feed both use the first).  Slot n of an
  // accumulator's ring is refilled for its tile n + sc_per: by then the MMAs of one of the sc_per - 1 tiles between them
  // have completed (the producer is at most `stages` tiles ahead of the tensor pipe), which needed the accumulator
  // back from every earlier tile - and an epilogue gives it back only after its last read of the multipliers.
  int sc_per;
  int sc_slots;          // 2 * sc_per, or 0
  int d_full_count;   // arrivals that complete a ring stage: 1 (TMA) or the number of decompress warps
  TopkOut topk;       // cand_key == nullptr: scores are written instead
  PlaidSrc plaid;     // PLAID kernels: the compressed documents
  int plaid_f16;      // PLAID kernels: operand type fp16 instead of bf16
};

constexpr int PLAID_WARPS = 3;  // warps 0, 18 and 19 decode compressed tokens in the PLAID kernels

struct SharedCtl {
  unsigned long long q_full, q_empty;
  unsigned long long d_full[8], d_empty[8];
  unsigned long long acc_full[2], acc_empty[2];
  uint32_t stage_info[8];
  int4 unit_info[UNIT_RING];    // per work unit: x = document length | LEN_FLAG_MASKED, y = its first row, z = tile group, w = document
  volatile int units_posted;    // units published in unit_info so far
  volatile int units_total;     // all units of this CTA once the producer has walked them (INT_MAX until then)
  uint32_t tmem_base;
  volatile int abort_flag;
  long long wait_limit;         // cycles after which a wait gives up
  int seg_off[2][TILE_M], seg_len[2][TILE_M], seg_q[2][TILE_M];
  short row_seg[2][TILE_M];
  int n_seg[2];
  int warp_aligned[2];  // every query of the tile sits inside one warp's 32 rows, starting at its first row
  float emit[2][2][TILE_M];
  float xch_m[2][2][TILE_M];  // half 1 -> half 0: per-row running maximum and its column
  int xch_i[2][2][TILE_M];
  alignas(16) float col_scale[2][TILE_N];  // read as float4
  alignas(16) float col_bias[2][TILE_N];
  // fused top-k: state of the candidate list of every query of the resident tiles
  int seg_cnt[2][TILE_M];
  unsigned seg_thr[2][TILE_M];
  int seg_list[2][TILE_M];      // list number (slot * qpg + query within the group)
  float plaid_bw[256];          // PLAID kernels: the bucket weights
};

// Bounded wait.  Returns false when the CTA is aborting.  The first probe lets the hardware suspend
// the thread until the phase completes (or the hint expires), so the common case costs two
// instructions; everything else lives in one out-of-line function.
__device__ __noinline__ bool wait_bar_slow(uint32_t b, uint32_t parity, SharedCtl* ctl, int* status) {
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(b, parity)) return true;
    if (ctl->abort_flag) return false;
    if (clock64() - t0 > ctl->wait_limit) {
      ctl->abort_flag = 1;
      if (status) atomicOr(status, LIK_DEV_WAIT_TIMEOUT);
      return false;
    }
  }
}
__device__ __forceinline__ bool wait_bar(unsigned long long* bar, uint32_t parity, SharedCtl* ctl, int* status) {
  const uint32_t b = smem_u32(bar);
  if (mbar_try_wait(b, parity)) return true;
  return wait_bar_slow(b, parity, ctl, status);
}
// Bounded wait until the producer has published unit `uc` of this CTA in the unit ring.
// Returns 1 when the unit is there, 2 when the stream has ended before it, 0 when the CTA is aborting.
__device__ __noinline__ int wait_posted_slow(SharedCtl* ctl, int uc, int* status) {
  const long long t0 = clock64();
  while (true) {
    if (ctl->units_posted > uc) return 1;
    if (ctl->units_total <= uc) return 2;
    if (ctl->abort_flag) return 0;
    if (clock64() - t0 > ctl->wait_limit) {
      ctl->abort_flag = 1;
      if (status) atomicOr(status, LIK_DEV_WAIT_TIMEOUT);
      return 0;
    }
  }
}
__device__ __forceinline__ int wait_posted(SharedCtl* ctl, int uc, int* status) {
  if (ctl->units_posted > uc) return 1;
  return wait_posted_slow(ctl, uc, status);
}

// Query tiles of tile-group g: tiles [g*mt, min((g+1)*mt, n_tiles)).
struct TileInfo {
  int qa, qb;        // queries [qa, qb)
  int chunk;         // chunk index when q_chunks > 1
  long long row0;    // first matrix row of the tile
};

__device__ __forceinline__ TileInfo tile_info(const TcParams& P, int tile) {
  TileInfo t;
  if (P.tile_q0) {
    t.qa = P.tile_q0[tile];
    t.qb = P.tile_q0[tile + 1];
    t.chunk = 0;
  } else if (P.q_chunks == 1) {
    t.qa = tile * P.q_per_tile;
    t.qb = min(t.qa + P.q_per_tile, P.n_q);
    t.chunk = 0;
  } else {
    t.qa = tile / P.q_chunks;
    t.qb = t.qa + 1;
    t.chunk = tile - t.qa * P.q_chunks;
  }
  long long r0;
  int len;
  seq_bounds(P.q, t.qa, r0, len, nullptr);
  t.row0 = r0 + (long long)t.chunk * TILE_M;
  return t;
}

// ---------------------------------------------------------------------------------------------
// The units of a CTA, in the order every role walks them.
//   CROSS: the documents are cut into super-blocks (one unless the caller asked for more: a super-block is
//   sized to stay in L2 while every tile group passes over it); inside a super-block the units are (tile
//   group, document), group-major, and CTA c of G takes the c-th of G equal shares.  A CTA therefore sees
//   the same one to three groups in every super-block, each with an ascending document range.
//   GROUPED: unit = document, group = its query.  LIST: unit = pair, group = its query (from the table).
// `doc` is the global document index (LIST: the pair).
// ---------------------------------------------------------------------------------------------
struct UnitIter {
  int sb;               // super-block
  int doc_lo, doc_hi;   // its documents
  int left;             // units of this CTA's share of the super-block still to come, this one included
  int grp, doc, in_grp;
};

__device__ __forceinline__ bool iter_enter(const TcParams& P, int n_groups, UnitIter& it) {
  const long long c = blockIdx.x, G = gridDim.x;
  while (it.sb < P.n_sb) {
    long long units;
    if (P.pairing == LIK_PAIR_CROSS) {
      it.doc_lo = (int)min((long long)it.sb * P.sb_docs, (long long)P.n_d);
      it.doc_hi = (int)min((long long)it.doc_lo + P.sb_docs, (long long)P.n_d);
      units = (long long)n_groups * (it.doc_hi - it.doc_lo);
    } else {
      it.doc_lo = 0;
      it.doc_hi = P.n_d;
      units = P.n_flat;
    }
    const long long u = units * c / G, u_end = units * (c + 1) / G;
    if (u < u_end) {
      it.left = (int)(u_end - u);
      if (P.pairing == LIK_PAIR_CROSS) {
        const int nd_b = it.doc_hi - it.doc_lo;
        it.grp = (int)(u / nd_b);
        it.doc = it.doc_lo + (int)(u - (long long)it.grp * nd_b);
        it.in_grp = 0;
      } else if (P.pairing == LIK_PAIR_GROUPED) {
        it.doc = (int)u;
        it.grp = it.doc / P.group;
        it.in_grp = it.doc - it.grp * P.group;
      } else {
        it.doc = (int)u;
        it.grp = -1;  // comes from the table
        it.in_grp = 0;
      }
      return true;
    }
    ++it.sb;
  }
  return false;
}
__device__ __forceinline__ bool iter_begin(const TcParams& P, int n_groups, UnitIter& it) {
  it.sb = 0;
  return iter_enter(P, n_groups, it);
}
__device__ __forceinline__ bool iter_next(const TcParams& P, int n_groups, UnitIter& it) {
  if (--it.left > 0) {
    ++it.doc;
    if (P.pairing == LIK_PAIR_CROSS) {
      if (it.doc == it.doc_hi) {
        it.doc = it.doc_lo;
        ++it.grp;
      }
    } else if (P.pairing == LIK_PAIR_GROUPED) {
      if (++it.in_grp == P.group) {
        it.in_grp = 0;
        ++it.grp;
      }
    }
    return true;
  }
  ++it.sb;
  return iter_enter(P, n_groups, it);
}

// Length words of a unit's document, loaded one unit ahead of their use.
struct UnitRaw {
  int a, b, q;
};
__device__ __forceinline__ UnitRaw unit_fetch(const TcParams& P, int doc) {
  UnitRaw r{0, 0, 0};
  if (P.pairing == LIK_PAIR_LIST) {
    const int4 t = __ldg(P.list_tab + doc);
    r.q = t.x;
    r.a = t.y;
    r.b = t.z;
  } else if (P.d.cu) {
    r.a = P.d.cu[doc];
    r.b = P.d.cu[doc + 1];
  } else if (P.d.lens) {
    r.a = P.d.lens[doc];
  }
  return r;
}
// First row and column count of the fetched document; `masked` tells whether its mask has holes.
// Lengths come from the caller-validated views, clamped to the padded extent.
__device__ __forceinline__ void unit_resolve(const TcParams& P, int doc, const UnitRaw& r, long long& row0, int& len, bool& masked) {
  masked = false;
  if (P.pairing == LIK_PAIR_LIST) {
    row0 = r.a;
    len = r.b;
  } else if (P.d.cu) {
    const int a = r.a, b = r.b;
    row0 = a;
    len = b > a ? b - a : 0;
    if ((long long)a + len > P.d.n_rows) len = P.d.n_rows > a ? (int)(P.d.n_rows - a) : 0;
  } else {
    row0 = (long long)doc * P.d.seq_stride;
    len = P.d.max_len;
    if (P.d.lens) {
      int l = r.a;
      if (P.d_len_flagged) {
        masked = (l & LEN_FLAG_MASKED) != 0;
        l &= ~LEN_FLAG_MASKED;
      }
      len = l < 0 ? 0 : (l > P.d.max_len ? P.d.max_len : l);
    }
  }
}

struct DocMaps {
  CUtensorMap m[4];  // document boxes of 64, 128, 192 and 256 rows: one copy per K slab whatever the tile height
};

// Word the producer leaves beside every ring stage for the MMA issuer.
constexpr uint32_t STAGE_COLS_MASK = 0x1FFu;   // valid document rows in the stage
constexpr uint32_t STAGE_ACC0 = 1u << 16;      // feed accumulator 0 / 1
constexpr uint32_t STAGE_ACC1 = 1u << 17;
constexpr uint32_t STAGE_FIRST = 1u << 18;     // first stage of a query-tile group: wait for the tiles
constexpr uint32_t STAGE_LAST = 1u << 19;      // last stage of the group: hand the tiles back afterwards
constexpr uint32_t STAGE_END = 1u << 20;       // no more work

// Monotone map float -> unsigned (larger float, larger key); 0 is below every float.
__device__ __forceinline__ unsigned ordered_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Cut a full candidate list (TOPK_CAP entries, in arrival = ascending document order) back to its k best
// and return the k-th best as an ordered key.  One warp; lane l holds entries l, l + 32, ...  The k-th
// largest key is found by bisection on its bits (32 warp-wide counts); entries above it stay, and of the
// entries equal to it the earliest ones (lowest document indices), so that exactly k remain, in order.
__device__ __noinline__ unsigned topk_compact(float* keys, int* idx, int k, int lane) {
  constexpr int PER = TOPK_CAP / 32;
  unsigned uk[PER];
  float fk[PER];
  int id[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    fk[j] = keys[j * 32 + lane];
    id[j] = idx[j * 32 + lane];
    uk[j] = ordered_key(fk[j]);
  }
  unsigned kth = 0;
  for (int bit = 31; bit >= 0; --bit) {
    const unsigned cand = kth | (1u << bit);
    int c = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) c += uk[j] >= cand ? 1 : 0;
    c = __reduce_add_sync(0xffffffffu, c);
    if (c >= k) kth = cand;
  }
  int n_gt = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) n_gt += uk[j] > kth ? 1 : 0;
  n_gt = __reduce_add_sync(0xffffffffu, n_gt);
  const int need = k - n_gt;  // ties to keep (at least one)
  const unsigned lt = (1u << lane) - 1u;
  int out = 0, ties = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const bool eq = uk[j] == kth;
    const unsigned m_eq = __ballot_sync(0xffffffffu, eq);
    const bool keep = uk[j] > kth || (eq && ties + __popc(m_eq & lt) < need);
    const unsigned m_keep = __ballot_sync(0xffffffffu, keep);
    if (keep) {
      const int pos = out + __popc(m_keep & lt);
      keys[pos] = fk[j];
      idx[pos] = id[j];
    }
    out += __popc(m_keep);
    ties += __popc(m_eq);
  }
  __syncwarp();
  return kth;
}

// WINNERS: 0 = scores only, 1 = winners saved, 2 = winners saved and every document takes the lazy winner scan (launched
// for problems whose documents are long, so that the kernels for short documents carry no third copy of the tile loop)
template <bool FP8, int WINNERS, bool SCALED, bool PLAID>
__global__ void __launch_bounds__(NUM_THREADS, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ DocMaps d_maps, const TcParams P) {
  constexpr bool ARGMAX = WINNERS != 0;
  extern __shared__ unsigned char smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int q_tile_bytes = P.n_slabs * TILE_M * SLAB_BYTES_ROW;
  const int d_stage_bytes = P.n_slabs * TILE_N * SLAB_BYTES_ROW;
  unsigned char* q_smem = smem;                              // [2][n_slabs][128 rows][128 B]
  unsigned char* d_smem = smem + 2 * q_tile_bytes;           // [stages][n_slabs][256 rows][128 B]
  float* sc_ring = reinterpret_cast<float*>(d_smem + (size_t)P.stages * d_stage_bytes);  // [sc_slots][TILE_N] (kernels with multipliers)
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(d_smem + (size_t)P.stages * d_stage_bytes + (size_t)P.sc_slots * TILE_N * sizeof(float));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // greedy-packed query tiles are counted on the device (the count sits in front of the table)
  const int n_tiles = P.tile_q0 ? P.tile_q0[-1] : P.n_tiles;
  const int n_groups = (n_tiles + P.mt - 1) / P.mt;
  const bool list = P.pairing == LIK_PAIR_LIST;
  const bool topk = !ARGMAX && P.topk.cand_key != nullptr;  // the fused top-k never saves winners

  if (tid == 0) {
    mbar_init(smem_u32(&ctl->q_full), 1);
    mbar_init(smem_u32(&ctl->q_empty), 1);
    for (int s = 0; s < P.stages; ++s) {
      mbar_init(smem_u32(&ctl->d_full[s]), (uint32_t)P.d_full_count);
      mbar_init(smem_u32(&ctl->d_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), GROUP_WARPS);
    }
    ctl->abort_flag = 0;
    ctl->wait_limit = WAIT_LIMIT_CYCLES;
    ctl->units_posted = 0;
    ctl->units_total = 0x7fffffff;
    fence_barrier_init();
    prefetch_tmap(&q_map);
    if (!PLAID)
      for (int i = 0; i < 4; ++i) prefetch_tmap(&d_maps.m[i]);
  }
  if (PLAID)
    for (int b = tid; b < (1 << P.plaid.nbits); b += NUM_THREADS) ctl->plaid_bw[b] = P.plaid.bucket_weights[b];
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  const bool producer_warp = warp == 0 || (PLAID && warp >= 2 + 2 * GROUP_WARPS);
  if (producer_warp) {
    // =========================== producer ===========================
    // TMA kernels: one thread (warp 0, lane 0) walks the units, loads the query tiles and the document
    // stages with TMA and leaves the stage words and the unit ring.  PLAID kernels: three whole warps walk
    // the units in step; each decodes its share of every stage's tokens into the swizzled operand layout
    // (generic-proxy stores, fenced for the tensor core's reads), and arrives on the stage barrier; the
    // elected thread of warp 0 still does everything else.
    const bool elect = warp == 0 && lane == 0;
    if (PLAID || lane == 0) {
      const int pw = warp == 0 ? 0 : warp - (2 + 2 * GROUP_WARPS) + 1;  // decoder warp number 0..2
      int cur_grp = -1;
      uint32_t n_qload = 0, st = 0, ph = 0, n_dload = 0;
      int sc_cnt[2] = {0, 0};  // next slot in either accumulator's multiplier ring
      long long uc = 0;
      const int x_per_slab = SLAB_BYTES_ROW / P.elt_bytes;
      bool ok = true;
      int tiles_here = 0;
      // the iterator stands one unit ahead: that unit's length words are in flight while this one is produced
      UnitIter it;
      bool have = iter_begin(P, n_groups, it);
      int nx_grp = 0, nx_doc = 0;
      UnitRaw nx_raw{0, 0, 0};
      if (have) {
        nx_grp = it.grp;
        nx_doc = it.doc;
        nx_raw = unit_fetch(P, nx_doc);
      }
      while (have && ok) {
        const int doc = nx_doc;
        const int grp = list ? nx_raw.q : nx_grp;
        long long drow0;
        int dlen;
        bool dmasked;
        unit_resolve(P, doc, nx_raw, drow0, dlen, dmasked);
        have = iter_next(P, n_groups, it);
        int next_grp = -1;
        if (have) {
          nx_grp = it.grp;
          nx_doc = it.doc;
          nx_raw = unit_fetch(P, nx_doc);
          next_grp = list ? nx_raw.q : nx_grp;
        }
        const bool last_unit_of_grp = next_grp != grp;
        uint32_t first = 0;
        if (grp != cur_grp) {
          cur_grp = grp;
          first = STAGE_FIRST;
          const int t0 = grp * P.mt, t1 = min(t0 + P.mt, n_tiles);
          tiles_here = t1 - t0;
          if (elect) {
            // wait until the MMAs that read the previous query tiles are done
            ok = wait_bar(&ctl->q_empty, (n_qload & 1) ^ 1, ctl, P.status);
            if (ok) {
              mbar_arrive_expect_tx(smem_u32(&ctl->q_full), (uint32_t)((t1 - t0) * q_tile_bytes));
              for (int t = t0; t < t1; ++t) {
                TileInfo ti = tile_info(P, t);
                for (int sl = 0; sl < P.n_slabs; ++sl)
                  tma_load_2d(smem_u32(q_smem + (t - t0) * q_tile_bytes + sl * TILE_M * SLAB_BYTES_ROW), &q_map, sl * x_per_slab,
                              (int)ti.row0, smem_u32(&ctl->q_full));
              }
            }
          }
          ++n_qload;
          if (PLAID && warp == 0) ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
        }
        // which accumulators this unit feeds: both resident tiles, or (one tile) alternating with the unit count
        const uint32_t acc_bits = P.mt == 2 ? (tiles_here == 2 ? (STAGE_ACC0 | STAGE_ACC1) : STAGE_ACC0)
                                            : ((uc & 1) ? STAGE_ACC1 : STAGE_ACC0);
        const int sc_ring_id = (!SCALED || P.mt == 2 || !(uc & 1)) ? 0 : 1;  // the multiplier ring of the accumulator(s) this unit feeds
        // publish the unit for the epilogue groups, then its stages; an empty document still sends one
        // (empty) stage so that every unit passes through the same hand-shakes
        if (elect) {
          ctl->unit_info[uc & (UNIT_RING - 1)] = make_int4(
              (dlen & UNIT_LEN_MASK) | (SCALED ? (sc_ring_id * P.sc_per + sc_cnt[sc_ring_id]) << UNIT_SLOT_SHIFT : 0) |
                  (dmasked ? LEN_FLAG_MASKED : 0),
              (int)drow0, grp, doc);
          __threadfence_block();
          ctl->units_posted = (int)uc + 1;
        }
        int c0 = 0;
        do {
          const int ncols = max(0, min(TILE_N, dlen - c0));
          ok = wait_bar(&ctl->d_empty[st], ph ^ 1, ctl, P.status);
          if (!ok) break;
          const uint32_t full = smem_u32(&ctl->d_full[st]);
          if (elect) {
            uint32_t info = (uint32_t)ncols | acc_bits;
            if (c0 == 0) info |= first;
            if (last_unit_of_grp && c0 + TILE_N >= dlen) info |= STAGE_LAST;
            ctl->stage_info[st] = info;
          }
          if (PLAID) {
            // the stage's tokens in six equal runs, one per half-warp of the three decoder warps
            const int hl = lane & 15;
            const int hw6 = pw * 2 + (lane >> 4);
            const int per = (ncols + 2 * PLAID_WARPS - 1) / (2 * PLAID_WARPS);
            const int t_lo = min(hw6 * per, ncols), n_run = min(per, ncols - t_lo);
            unsigned char* stage = d_smem + (size_t)st * d_stage_bytes + (hl >> 3) * (TILE_N * SLAB_BYTES_ROW);
            const bool f16 = P.plaid_f16 != 0;
            auto sink = [&](int t, const float (&e)[8]) {
              const int row = t_lo + t;
              *reinterpret_cast<uint4*>(stage + row * SLAB_BYTES_ROW + (((hl & 7) ^ (row & 7)) << 4)) = plaid_pack16(e, f16);
            };
            if (P.plaid.centroid_dtype == LIK_F32)
              plaid_decode_range<true, 4>(P.plaid, ctl->plaid_bw, drow0 + c0 + t_lo, n_run, per, lane, hl * 8 < P.plaid.dim, P.status, sink);
            else
              plaid_decode_range<false, 8>(P.plaid, ctl->plaid_bw, drow0 + c0 + t_lo, n_run, per, lane, hl * 8 < P.plaid.dim, P.status, sink);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(full);
          } else {
            const int boxes = (ncols + BOX_ROWS - 1) / BOX_ROWS;
            if (boxes > 0) {
              // the tile's multipliers ride on the same barrier: whole groups of four floats, never past the array's end
              uint32_t sc_bytes = 0;
              if (SCALED && P.col_src) {
                const long long r = drow0 + c0;
                sc_bytes = (uint32_t)min((long long)((ncols + 3) & ~3), P.d.n_rows - r) * 4u;
              }
              mbar_arrive_expect_tx(full, (uint32_t)(boxes * BOX_ROWS * SLAB_BYTES_ROW * P.n_slabs) + sc_bytes);
              const CUtensorMap* map = &d_maps.m[boxes - 1];
              for (int sl = 0; sl < P.n_slabs; ++sl)
                tma_load_2d(smem_u32(d_smem + (size_t)st * d_stage_bytes + sl * TILE_N * SLAB_BYTES_ROW), map, sl * x_per_slab,
                            (int)(drow0 + c0), full);
              if (sc_bytes)
                bulk_load_1d(smem_u32(sc_ring + (sc_ring_id * P.sc_per + sc_cnt[sc_ring_id]) * TILE_N), P.col_src + drow0 + c0, sc_bytes, full);
            } else {
              mbar_arrive(full);
            }
          }
          ++n_dload;
          if (++st == (uint32_t)P.stages) { st = 0; ph ^= 1; }
          if (SCALED && ++sc_cnt[sc_ring_id] >= P.sc_per) sc_cnt[sc_ring_id] = 0;
          c0 += TILE_N;
        } while (c0 < dlen);
        ++uc;
      }
      if (ok && elect) {
        // tell the epilogue groups how many units there were
        __threadfence_block();
        ctl->units_total = (int)uc;
      }
      if (ok) {
        // tell the issuer that the stream has ended
        ok = wait_bar(&ctl->d_empty[st], ph ^ 1, ctl, P.status);
        if (ok) {
          if (elect) ctl->stage_info[st] = STAGE_END;
          if (lane == 0) mbar_arrive(smem_u32(&ctl->d_full[st]));
        }
      }
      if (!ok && elect) {
        // aborting: let the copies already issued land before the CTA goes away
        if (!PLAID) {
          for (uint32_t i = 1; i <= (uint32_t)P.stages && i <= n_dload; ++i) {
            const bool wrapped = i > st;  // that use lies before the last wrap of the ring
            const uint32_t slot = wrapped ? st + (uint32_t)P.stages - i : st - i;
            const uint32_t bar = smem_u32(&ctl->d_full[slot]);
            for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(bar, wrapped ? ph ^ 1 : ph); ++spin) {
            }
          }
        }
        if (n_qload) {
          const uint32_t bar = smem_u32(&ctl->q_full);
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(bar, (n_qload - 1) & 1); ++spin) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    // Driven by the stage words alone: between two MMA groups it runs a few dozen instructions, so the
    // tensor pipe's queue never drains while work is available.
    if (lane == 0) {
      uint32_t st = 0, ph = 0, q_ph = 0, acc_ph = 0;  // acc_ph: one phase bit per accumulator
      bool ok = true;
      const uint32_t q_tile_desc = (uint32_t)(q_tile_bytes >> 4);
      const uint32_t desc_hi = (uint32_t)(smem_desc_sw128(0) >> 32);
      const uint32_t a_desc0 = (uint32_t)smem_desc_sw128(smem_u32(q_smem));
      const uint32_t b_desc0 = (uint32_t)smem_desc_sw128(smem_u32(d_smem));
      const uint32_t stage_desc = (uint32_t)(d_stage_bytes >> 4);
      const uint32_t idesc0 = instr_desc(P.ab_format, 0);
      const int k_steps = P.k_steps, n_slabs = P.n_slabs;
      const uint32_t a_tile1 = P.mt == 2 ? q_tile_desc : 0u;  // descriptor offset of the second resident tile
      uint32_t a_lo0[8], a_lo1[8];  // the eight K steps of either resident tile never move
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        a_lo0[k] = a_desc0 + (uint32_t)((k & 3) * 2 + (k >> 2) * ((TILE_M * SLAB_BYTES_ROW) >> 4));
        a_lo1[k] = a_lo0[k] + a_tile1;
      }
      while (ok) {
        ok = wait_bar(&ctl->d_full[st], ph, ctl, P.status);
        if (!ok) break;
        const uint32_t info = ctl->stage_info[st];
        if (info & STAGE_END) break;
        if (info & STAGE_FIRST) {
          ok = wait_bar(&ctl->q_full, q_ph, ctl, P.status);
          if (!ok) break;
          q_ph ^= 1;
        }
        const uint32_t ncols = info & STAGE_COLS_MASK;
        {
          const uint32_t idesc = idesc0 | (((ncols + 15) >> 4) << 18);  // N / 8 in bits 17..22
          const uint32_t b_stage = b_desc0 + st * stage_desc;
          uint32_t b_lo[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) b_lo[k] = b_stage + (uint32_t)((k & 3) * 2 + (k >> 2) * ((TILE_N * SLAB_BYTES_ROW) >> 4));
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            if (!(info & (STAGE_ACC0 << a))) continue;
            ok = wait_bar(&ctl->acc_empty[a], ((acc_ph >> a) & 1u) ^ 1u, ctl, P.status);
            if (!ok) break;
            acc_ph ^= 1u << a;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(a * ACC_COLS);
            // descriptors differ only in the 16-byte-unit start address: add offsets to a base descriptor
            uint32_t a_desc = a_desc0 + a * a_tile1;
            uint32_t b_desc = b_stage;
            if (ncols == 0) {
              // empty document: the accumulator still changes hands so that both sides keep their phase
            } else if (k_steps == 8) {
              // the common width (128 two-byte or 256 one-byte elements): straight-line issue from
              // descriptor words prepared ahead of the accumulator wait
              const uint32_t* al = a ? a_lo1 : a_lo0;
              tc_mma<FP8>(d_tmem, al[0], b_lo[0], desc_hi, idesc, 0u);
              tc_mma<FP8>(d_tmem, al[1], b_lo[1], desc_hi, idesc, 1u);
              tc_mma<FP8>(d_tmem, al[2], b_lo[2], desc_hi, idesc, 1u);
              tc_mma<FP8>(d_tmem, al[3], b_lo[3], desc_hi, idesc, 1u);
              tc_mma<FP8>(d_tmem, al[4], b_lo[4], desc_hi, idesc, 1u);
              tc_mma<FP8>(d_tmem, al[5], b_lo[5], desc_hi, idesc, 1u);
              tc_mma<FP8>(d_tmem, al[6], b_lo[6], desc_hi, idesc, 1u);
              tc_mma<FP8>(d_tmem, al[7], b_lo[7], desc_hi, idesc, 1u);
            } else {
              int left = k_steps;
              uint32_t accum = 0;
              for (int sl = 0; sl < n_slabs; ++sl) {
                tc_mma<FP8>(d_tmem, a_desc, b_desc, desc_hi, idesc, accum);
                accum = 1;
                if (left > 1) tc_mma<FP8>(d_tmem, a_desc + 2, b_desc + 2, desc_hi, idesc, 1u);
                if (left > 2) tc_mma<FP8>(d_tmem, a_desc + 4, b_desc + 4, desc_hi, idesc, 1u);
                if (left > 3) tc_mma<FP8>(d_tmem, a_desc + 6, b_desc + 6, desc_hi, idesc, 1u);
                left -= 4;
                a_desc += (uint32_t)((TILE_M * SLAB_BYTES_ROW) >> 4);
                b_desc += (uint32_t)((TILE_N * SLAB_BYTES_ROW) >> 4);
              }
            }
            tc_commit(smem_u32(&ctl->acc_full[a]));
          }
          if (!ok) break;
        }
        tc_commit(smem_u32(&ctl->d_empty[st]));  // ring slot reusable once these MMAs retire
        if (info & STAGE_LAST) tc_commit(smem_u32(&ctl->q_empty));  // and so are the query tiles
        if (++st == (uint32_t)P.stages) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp < 2 + 2 * GROUP_WARPS) {
    // =========================== epilogue groups ===========================
    // Group g (eight warps) drains accumulator g.  Its two halves split the 32-column chunks of a tile
    // between them (even chunks / odd chunks); half 1 hands its per-row result to half 0, which sums
    // the rows of every query and writes the score.  (group, document) advance locally; a document's
    // length and first row come from the producer's unit ring.
    const int e = warp - 2;
    const int wg = e >> 3;                   // accumulator / epilogue group
    const int sub = (e >> 2) & 1;            // half of the group
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int wq = e & 3;                    // warp index inside the half
    const int row = quad * 32 + lane;        // accumulator row == query token slot in the tile
    const int et = wq * 32 + lane;           // thread index inside the half (0..127)
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(wg * ACC_COLS);
    const uint32_t acc_empty_bar = smem_u32(&ctl->acc_empty[wg]);
    int cur_grp = -1;
    uint32_t n_acc = 0, n_emit = 0, n_doc = 0;
    int uc = 0;
    bool ok = true;
    // per-row / per-warp state for the resident query tile
    bool have_tile = false, in_seg = false, row_ok = false, aligned = false;
    float my_qf = 1.f;
    int tile_id = 0;
    long long arg_off = -1;   // ARGMAX: offset of this row's slot for document 0 (-1: row stores nothing)
    long long warp_out = -1;  // aligned tiles: offset of this warp's query score for document 0
    int my_list = -1;         // top-k: the list whose state thread `et` (half 0) loaded into shared memory
    int warp_seg = -1;        // aligned tiles: the query (segment) of this warp's rows
    // Rendezvous of the whole group / of half 0 on hardware named barriers: a waiting warp issues
    // nothing.  Nobody waits on anything else between two of them, so every warp of the group always
    // arrives; the only bounded waits of a group (for a unit, for the accumulator) are done by its first warp,
    // which tells the others whether to go on through the rendezvous itself: a barrier that counts the
    // threads arriving with a true predicate (0: go on, 1: the wait gave up, 2: the stream has ended).
    const bool leader = (e & 7) == 0;
#define LIK_GRP_SYNC_COUNT(pred_, count_out_)                                                                        \
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %3, 0;\n\tbar.red.popc.u32 %0, %1, %2, q;\n\t}"              \
               : "=r"(count_out_) : "r"(1 + wg), "r"(2 * EPI_THREADS), "r"((int)(pred_)) : "memory")
#define LIK_GRP_SYNC() asm volatile("bar.sync %0, %1;" ::"r"(1 + wg), "r"(2 * EPI_THREADS) : "memory")
#define LIK_SUB_SYNC() asm volatile("bar.sync %0, %1;" ::"r"(3 + wg), "r"(EPI_THREADS) : "memory")
#define LIK_GROUP_WAIT_ACC()                                                         \
  do {                                                                               \
    bool gave_up_ = false;                                                           \
    if (leader) gave_up_ = !wait_bar(&ctl->acc_full[wg], n_acc & 1, ctl, P.status);  \
    int n_;                                                                          \
    LIK_GRP_SYNC_COUNT(gave_up_ && lane == 0, n_);                                   \
    ok = n_ == 0;                                                                    \
  } while (0)
    // top-k: write the state of the lists this thread loaded back to their headers
#define LIK_TOPK_STORE_BACK()                                                                          \
  do {                                                                                                 \
    if (topk && sub == 0 && my_list >= 0) {                                                            \
      P.topk.hdr[my_list] = make_int2(ctl->seg_cnt[wg][et], (int)ctl->seg_thr[wg][et]);                \
      my_list = -1;                                                                                    \
    }                                                                                                  \
  } while (0)
    // one (query, document) score: stored, or offered to the query's candidate list (warp-uniform)
#define LIK_EMIT_SCORE(sg_, value_, offset_)                                                           \
  do {                                                                                                 \
    if (!topk) {                                                                                       \
      if (lane == 0) P.scores[offset_] = (value_);                                                     \
    } else {                                                                                           \
      const float key_ = (P.topk.largest ? (value_) : -(value_)) + 0.f;                                \
      const unsigned ukey_ = ordered_key(key_);                                                        \
      if (ukey_ > ctl->seg_thr[wg][sg_]) {                                                             \
        int cnt_ = ctl->seg_cnt[wg][sg_];                                                              \
        if ((unsigned)cnt_ >= (unsigned)TOPK_CAP || (unsigned)ctl->seg_list[wg][sg_] >= (unsigned)P.topk.n_lists) {  \
          if (lane == 0 && P.status) atomicOr(P.status, LIK_DEV_INTERNAL);                             \
          break;                                                                                       \
        }                                                                                              \
        float* keys_ = P.topk.cand_key + (long long)ctl->seg_list[wg][sg_] * TOPK_CAP;                 \
        int* idx_ = P.topk.cand_idx + (long long)ctl->seg_list[wg][sg_] * TOPK_CAP;                    \
        if (lane == 0) {                                                                               \
          keys_[cnt_] = key_;                                                                          \
          idx_[cnt_] = doc + P.topk.doc_base;                                                          \
        }                                                                                              \
        ++cnt_;                                                                                        \
        __syncwarp();                                                                                  \
        if (cnt_ == TOPK_CAP) {                                                                        \
          const unsigned thr_ = topk_compact(keys_, idx_, P.topk.k, lane);                             \
          cnt_ = P.topk.k;                                                                             \
          if (lane == 0) ctl->seg_thr[wg][sg_] = thr_;                                                 \
        }                                                                                              \
        if (lane == 0) ctl->seg_cnt[wg][sg_] = cnt_;                                                   \
        __syncwarp();                                                                                  \
      }                                                                                                \
    }                                                                                                  \
  } while (0)

    const bool cross = P.pairing == LIK_PAIR_CROSS;
    const bool bulk = SCALED && P.col_src != nullptr;  // the multipliers of a tile arrive with it
    const bool every_group_full = P.mt == 1 || (n_tiles & 1) == 0;
    for (;; ++uc) {
      // with one resident tile the two groups take alternate units
      if (P.mt == 1 && (uc & 1) != wg) continue;
      // The unit (tile group, document, length, first row) comes from the producer's ring.  The group's first warp
      // waits for its publication and - in kernels without per-column multipliers, which have nothing to prepare
      // while the MMAs run - for the unit's first accumulator, when this group has a tile in the unit's tile group.
      int st_ = 1;
      if (leader) {
        st_ = wait_posted(ctl, uc, P.status);
        if (st_ == 1 && !SCALED) {
          // (only the last tile group can lack this group's tile, and only when the tile count is odd)
          const bool mine_ = every_group_full || ctl->unit_info[uc & (UNIT_RING - 1)].z * P.mt + wg < n_tiles;
          if (mine_ && !wait_bar(&ctl->acc_full[wg], n_acc & 1, ctl, P.status)) st_ = 0;
        }
      }
      {
        // the first warp arrives with one true predicate when its wait gave up, with two when the stream has ended
        int state_;
        LIK_GRP_SYNC_COUNT((st_ == 0 && lane == 0) || (st_ == 2 && lane < 2), state_);
        ok = state_ != 1;
        if (state_ != 0) break;
      }
      const int4 uinfo = ctl->unit_info[uc & (UNIT_RING - 1)];
      const int grp = uinfo.z;
      const int doc = uinfo.w;
      // (a group number out of range cannot index anything: its tile number fails the range check below)
      if (grp != cur_grp) {
        cur_grp = grp;
        // (re)build the segment table of this group's tile `wg` (mt == 2) or tile 0 (mt == 1: both groups)
        const int m = P.mt == 2 ? wg : 0;
        tile_id = grp * P.mt + m;
        have_tile = (unsigned)tile_id < (unsigned)n_tiles;
        LIK_GRP_SYNC();  // everyone in the group is done reading the old table
        LIK_TOPK_STORE_BACK();
        TileInfo ti{};
        int nseg = 0;
        if (have_tile) {
          ti = tile_info(P, tile_id);
          nseg = ti.qb - ti.qa;
          if (sub == 0) {
            ctl->row_seg[wg][et] = -1;
            if (et == 0) {
              ctl->n_seg[wg] = nseg;
              ctl->warp_aligned[wg] = P.q_chunks == 1 ? 1 : 0;
            }
          }
        }
        LIK_GRP_SYNC();
        if (have_tile && sub == 0 && et < nseg) {
          long long r0;
          int len;
          seq_bounds(P.q, ti.qa + et, r0, len, P.status);
          int off, l;
          if (P.q_chunks == 1) {
            off = (int)(r0 - ti.row0);
            l = len;
            if (off + l > TILE_M) {  // max_len was smaller than a real query: report, stay in bounds
              l = max(0, TILE_M - off);
              if (P.status) atomicOr(P.status, LIK_DEV_LEN_RANGE);
            }
          } else {
            off = 0;
            l = min(TILE_M, max(0, len - ti.chunk * TILE_M));
            if (len > P.q_chunks * TILE_M && P.status) atomicOr(P.status, LIK_DEV_LEN_RANGE);
          }
          // an empty query owns no accumulator row, so only the per-query pass below can write its zero
          if ((off & 31) != 0 || l > 32 || l == 0) ctl->warp_aligned[wg] = 0;
          if (ARGMAX && len > P.argmax_stride && P.status) atomicOr(P.status, LIK_DEV_ARGMAX_STRIDE);
          ctl->seg_off[wg][et] = off;
          ctl->seg_len[wg][et] = l;
          ctl->seg_q[wg][et] = ti.qa + et;
          for (int i = 0; i < l; ++i) ctl->row_seg[wg][off + i] = (short)et;
          if (topk) {
            // the candidate list of (this CTA, this group, this query)
            // (with one resident tile the two epilogue groups take alternate documents: a list each)
            my_list = ((int)blockIdx.x + grp) * P.topk.qpg + (P.mt == 2 ? m : wg) * P.q_per_tile + et;
            if ((unsigned)my_list >= (unsigned)P.topk.n_lists) {
              if (P.status) atomicOr(P.status, LIK_DEV_INTERNAL);
              my_list = 0;
            }
            const int2 hd = P.topk.hdr[my_list];
            ctl->seg_list[wg][et] = my_list;
            ctl->seg_cnt[wg][et] = hd.x;
            ctl->seg_thr[wg][et] = (unsigned)hd.y;
          }
        }
        LIK_GRP_SYNC();
        in_seg = false;
        row_ok = false;
        arg_off = -1;
        warp_out = -1;
        warp_seg = -1;
        aligned = have_tile && ctl->warp_aligned[wg] != 0;
        if (have_tile) {
          const int sg = ctl->row_seg[wg][row];
          if (sg >= 0) {
            in_seg = true;
            const int my_q = ctl->seg_q[wg][sg];
            const int my_s = row - ctl->seg_off[wg][sg] + ti.chunk * TILE_M;
            const long long qrow = ti.row0 + row;
            row_ok = row_valid(P.q, qrow);
            my_qf = row_factor(P.q, qrow);
            if (ARGMAX && my_s < P.argmax_stride)
              arg_off = (cross ? (long long)my_q * P.n_d : 0ll) * P.argmax_stride + my_s;
          }
          const int sg0 = ctl->row_seg[wg][quad * 32];
          if (aligned && sg0 >= 0) {
            warp_seg = sg0;
            warp_out = cross ? (long long)ctl->seg_q[wg][sg0] * P.n_d : 0ll;
          }
        }
      }
      // a tile group with an odd tile out: the second epilogue group has nothing in it
      if (!have_tile) continue;
      const int dlen = uinfo.x & UNIT_LEN_MASK;
      int sc_slot = SCALED ? (uinfo.x >> UNIT_SLOT_SHIFT) & 31 : 0;  // multiplier slot of the unit's first tile
      const int sc_base = SCALED && sc_slot >= P.sc_per ? P.sc_per : 0;  // first slot of its ring
      const long long drow0 = uinfo.y;
      const bool holes = (uinfo.x & LEN_FLAG_MASKED) != 0;  // the document's mask is not a plain prefix
      // where this unit's results go: CROSS / GROUPED index by document, LIST by pair (== unit)
      const long long out_col = doc;
      float run_m = -INFINITY;
      int run_i = -1;
      int c0 = 0;
      // The tiles of the document.  The body exists twice in the kernels without per-column multipliers: documents whose
      // mask is a plain prefix (nearly all) take the copy that has no column arrays in it, the others the general one -
      // the common path's time goes with its code size, so the rare one stays out of it.
      auto document_tiles = [&](auto general_, auto lazy_) {
      constexpr bool general = decltype(general_)::value;  // the document's mask has holes
      constexpr bool lazy = decltype(lazy_)::value;        // long document: winner scan only when some row of the warp needs it
      constexpr bool use_cols = SCALED || general;          // per-column multiplier / additive mask needed
      do {
        const int ncols = max(0, min(TILE_N, dlen - c0));
        // per-column arrays of this tile.  They may be written once the previous tile's readers are done with them (a
        // rendezvous, unless the one at the top of the unit already stands between), and read after one more rendezvous.
#define LIK_STAGE_COLUMNS(sync_before_)                                                                   \
  do {                                                                                                    \
    if (sync_before_) LIK_GRP_SYNC();                                                                     \
    for (int c = sub * EPI_THREADS + et; c < ((ncols + 31) & ~31); c += 2 * EPI_THREADS) {                \
      float sc = 1.f, bi = -INFINITY;                                                                     \
      if (c < ncols) {                                                                                    \
        const long long drow = drow0 + c0 + c;                                                            \
        sc = row_factor(P.d, drow);                                                                       \
        bi = row_valid(P.d, drow) ? 0.f : -INFINITY;                                                      \
      }                                                                                                   \
      ctl->col_scale[wg][c] = sc;                                                                         \
      ctl->col_bias[wg][c] = bi;                                                                          \
    }                                                                                                     \
  } while (0)
        // before the accumulator wait: overlaps the MMAs; the wait's rendezvous also publishes the columns
        // (not needed when the multipliers came with the tile and the mask has no holes)
        const bool staged = SCALED && (general || !bulk);
        if (staged) LIK_STAGE_COLUMNS(c0 > 0);
        if (SCALED || c0 > 0) {
          LIK_GROUP_WAIT_ACC();
          if (!ok) break;
        }
        ++n_acc;
        if (!SCALED && use_cols) {  // a document whose mask has holes: known only now
          LIK_STAGE_COLUMNS(true);
          LIK_GRP_SYNC();
        }
#undef LIK_STAGE_COLUMNS
        tc_fence_after();
        // the accumulator goes back to the issuer as soon as this warp's last columns sit in registers
#define LIK_RELEASE_ACC()                                          \
  do {                                                             \
    tc_fence_before();                                             \
    __syncwarp();                                                  \
    if (lane == 0) mbar_arrive(acc_empty_bar);                     \
  } while (0)
        // chunks of this half: cc, cc + 64, ...; only the tile's last chunk can be partial
        int cc = sub * 32;
        if (cc >= ncols) LIK_RELEASE_ACC();
        if (use_cols && general) {
          // a mask with holes: every chunk takes multiplier and additive mask
          for (; cc < ncols; cc += 64) {
            float v[32];
            tmem_ld32_issue(lane_addr + (uint32_t)cc, v);
            tmem_ld_wait(v);
            if (cc + 64 >= ncols) LIK_RELEASE_ACC();
            affine32(v, &ctl->col_scale[wg][cc], &ctl->col_bias[wg][cc]);  // bias is -inf past ncols and in holes
            fold32<ARGMAX, lazy>(v, c0 + cc, run_m, run_i);
          }
        } else if (use_cols) {
          // whole chunks are valid: multiplier only; the partial last chunk also takes the mask (-inf past ncols).
          // Multipliers that came with the tile sit in a ring slot that is refilled once the accumulator has changed
          // hands often enough: there the accumulator goes back after the last read of them, not before.
          const float* sc_arr = bulk ? sc_ring + sc_slot * TILE_N : ctl->col_scale[wg];
          for (; cc + 32 <= ncols; cc += 64) {
            float v[32];
            tmem_ld32_issue(lane_addr + (uint32_t)cc, v);
            tmem_ld_wait(v);
            if (!bulk && cc + 64 >= ncols) LIK_RELEASE_ACC();
            scale32(v, sc_arr + cc);
            if (bulk && cc + 64 >= ncols) LIK_RELEASE_ACC();
            fold32<ARGMAX, lazy>(v, c0 + cc, run_m, run_i);
          }
          if (cc < ncols) {
            float v[32];
            tmem_ld32_issue(lane_addr + (uint32_t)cc, v);
            tmem_ld_wait(v);
            if (bulk) {
              scale32_first(v, sc_arr + cc, ncols - cc);
              LIK_RELEASE_ACC();
            } else {
              LIK_RELEASE_ACC();
              affine32(v, &ctl->col_scale[wg][cc], &ctl->col_bias[wg][cc]);
            }
            fold32<ARGMAX, lazy>(v, c0 + cc, run_m, run_i);
          }
        } else {
          for (; cc + 32 <= ncols; cc += 64) {
            float v[32];
            tmem_ld32_issue(lane_addr + (uint32_t)cc, v);
            tmem_ld_wait(v);
            if (cc + 64 >= ncols) LIK_RELEASE_ACC();
            fold32<ARGMAX, lazy>(v, c0 + cc, run_m, run_i);
          }
          if (cc < ncols) {
            // partial chunk: pieces of 16, 8, 4, 2 and 1 columns as the bits of its width say, absent
            // pieces stay at -inf, so nothing needs masking
            const int lim = ncols - cc;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = -INFINITY;
            tmem_ld_tail(lane_addr + (uint32_t)cc, lim, v);
            LIK_RELEASE_ACC();
            const float cmax = max32(v);
            if (ARGMAX) {
              const int p = tail_first_match(v, cmax, lim);
              const bool better = cmax > run_m;
              run_i = better ? c0 + cc + p : run_i;
              run_m = better ? cmax : run_m;
            } else {
              run_m = fmaxf(run_m, cmax);
            }
          }
        }
#undef LIK_RELEASE_ACC
        c0 += TILE_N;
        if (SCALED && ++sc_slot >= sc_base + P.sc_per) sc_slot = sc_base;
      } while (c0 < dlen);
      };
      // (long documents, WINNERS == 2: most 32-column chunks past the first few hundred tokens hold no new maximum for any
      // of a warp's rows, and the scan for its column is skipped there)
      if (holes) document_tiles(std::true_type{}, std::false_type{});
      else document_tiles(std::false_type{}, std::integral_constant<bool, WINNERS == 2>{});
      if (!ok) break;
      // ---- end of document: half 1 hands over, half 0 merges (lower column wins a tie) ----
      float* xm = ctl->xch_m[wg][n_doc & 1];
      int* xi = ctl->xch_i[wg][n_doc & 1];
      ++n_doc;
      if (sub == 1) {
        xm[row] = run_m;
        if (ARGMAX) xi[row] = run_i;
      }
      LIK_GRP_SYNC();
      if (sub == 1) continue;
      {
        const float m1 = xm[row];
        if (ARGMAX) {
          const int i1 = xi[row];
          const bool take = (i1 >= 0) & ((run_i < 0) | (m1 > run_m) | ((m1 == run_m) & (i1 < run_i)));
          run_m = take ? m1 : run_m;
          run_i = take ? i1 : run_i;
        } else {
          run_m = fmaxf(run_m, m1);
        }
      }
      // one value per row, summed per query in a fixed order
      const bool has_winner = ARGMAX ? (run_i >= 0) : (run_m != -INFINITY);
      const float val = (in_seg && row_ok && has_winner) ? run_m * my_qf : 0.f;
      if (ARGMAX && arg_off >= 0) P.argmax[arg_off + out_col * P.argmax_stride] = has_winner ? run_i : -1;
      if (aligned) {
        // one query per warp: a shuffle tree (fixed order) replaces the shared-memory pass
        const float sum = warp_sum(val);
        if (warp_out >= 0) LIK_EMIT_SCORE(warp_seg, sum, warp_out + out_col);
        continue;
      }
      float* ebuf = ctl->emit[wg][n_emit & 1];
      ++n_emit;
      ebuf[row] = val;
      LIK_SUB_SYNC();
      const int nseg = ctl->n_seg[wg];
      for (int sg = wq; sg < nseg; sg += 4) {
        const int off = ctl->seg_off[wg][sg], len = ctl->seg_len[wg][sg];
        float sum = 0.f;
        for (int i = lane; i < len; i += 32) sum += ebuf[off + i];
        sum = warp_sum(sum);
        const int qq = ctl->seg_q[wg][sg];
        if (P.q_chunks == 1) {
          const long long o = cross ? (long long)qq * P.n_d + out_col : out_col;
          LIK_EMIT_SCORE(sg, sum, o);
        } else if (lane == 0) {
          P.partial[(long long)tile_id * P.n_d + doc] = sum;
        }
      }
    }
    // top-k: leave the lists' state where the next launch stage (the merge) finds it
    if (sub == 0) {
      LIK_SUB_SYNC();
      LIK_TOPK_STORE_BACK();
    }
#undef LIK_EMIT_SCORE
#undef LIK_TOPK_STORE_BACK
#undef LIK_GROUP_WAIT_ACC
#undef LIK_GRP_SYNC
#undef LIK_GRP_SYNC_COUNT
#undef LIK_SUB_SYNC
  }

  // ---- teardown (also reached when aborting: every wait above is bounded) ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// The bounded wait of the kernel above, alone: one thread waits on a barrier that nothing ever arrives at, with a
// limit the caller chooses.  It must give up after that many cycles, raise LIK_DEV_WAIT_TIMEOUT in the status word,
// set the abort flag and return - the path every role of the scoring kernel takes when a hand-shake never comes.
// result[0] = what the wait returned (0 = gave up), result[1] = the abort flag, result[2] = cycles spent.
__global__ void wait_probe_kernel(long long limit, int* status, int* result) {
  __shared__ SharedCtl ctl;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl.q_full), 1);
    ctl.abort_flag = 0;
    ctl.wait_limit = limit;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool got = wait_bar(&ctl.q_full, 0, &ctl, status);
    const long long dt = clock64() - t0;
    result[0] = got ? 1 : 0;
    result[1] = ctl.abort_flag;
    result[2] = dt > 0x7fffffffll ? 0x7fffffff : (int)dt;
  }
}

// One row of the pair-list table per pair: the query (0 when the pair is out of range, which is reported
// through the status word and scores 0 because its document is then empty), the first row and the length of
// the document.
__global__ void list_units_kernel(SeqView q, SeqView d, const int* __restrict__ pair_q, const int* __restrict__ pair_d,
                                  long long n_pairs, int4* __restrict__ tab, int* status) {
  const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  const int i = pair_q[p], j = pair_d[p];
  int4 t = make_int4(0, 0, 0, 0);
  if (i < 0 || i >= q.n_seq || j < 0 || j >= d.n_seq) {
    if (status) atomicOr(status, LIK_DEV_PAIR_RANGE);
  } else {
    long long r0;
    int len;
    seq_bounds(d, j, r0, len, status);
    t = make_int4(i, (int)r0, len, 0);
  }
  tab[p] = t;
}

// Effective length of every padded document under its token mask: 1 + index of the last valid
// token, tagged with LEN_FLAG_MASKED when the valid tokens are not exactly the prefix [0, length).
__global__ void mask_lens_kernel(const unsigned char* __restrict__ mask, const int* __restrict__ lens, int n_seq, int max_len,
                                 long long seq_stride, int* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (j >= n_seq) return;
  int len0 = max_len;
  if (lens) len0 = min(max(lens[j], 0), max_len);
  const unsigned char* m = mask + (long long)j * seq_stride;
  int last = -1, cnt = 0;
  for (int t = lane; t < len0; t += 32)
    if (m[t]) {
      last = t;
      ++cnt;
    }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
    cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  }
  if (lane == 0) out[j] = (last + 1) | (cnt != last + 1 ? LEN_FLAG_MASKED : 0);
}

constexpr int PACK_MAX_QUERIES = 8192;  // offsets are staged in shared memory; larger batches use fixed groups

// Greedy packing of ragged queries into 128-row tiles: a tile takes whole consecutive queries until the next
// one would not fit (or it holds 128 queries; empty ones take no rows).  out[0] = tile count, out[1 + m] =
// first query of tile m (out[1 + count] = n_q).  One CTA: the offsets go to shared memory, every thread finds
// by bisection where a tile starting at its query would end, then one thread follows those links.
__global__ void __launch_bounds__(256) pack_query_tiles_kernel(const int* __restrict__ cu, int n_q, int* __restrict__ out) {
  __shared__ int s_cu[PACK_MAX_QUERIES + 1];
  __shared__ unsigned char s_span[PACK_MAX_QUERIES];  // queries in the tile that starts at query i (1..128)
  for (int i = threadIdx.x; i <= n_q; i += blockDim.x) s_cu[i] = cu[i];
  __syncthreads();
  for (int i = threadIdx.x; i < n_q; i += blockDim.x) {
    int lo = i + 1, hi = min(i + TILE_M, n_q);  // the tile ends at some j in [lo, hi]; a lone long query still gets one
    const int base = s_cu[i];
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_cu[mid] - base <= TILE_M) lo = mid;
      else hi = mid - 1;
    }
    s_span[i] = (unsigned char)(lo - i - 1);  // stored minus one so that 128 fits a byte
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0, q = 0;
    out[1] = 0;
    while (q < n_q) {
      q += (int)s_span[q] + 1;
      ++tiles;
      out[1 + tiles] = q;
    }
    if (tiles == 0) {  // n_q == 0 cannot reach this kernel; keep the table well formed anyway
      tiles = 1;
      out[2] = n_q;
    }
    out[0] = tiles;
  }
}

// scores[q, j] = sum over the chunks of query q, in chunk order
__global__ void reduce_chunks_kernel(const float* __restrict__ partial, int n_q, int n_d, int q_chunks, float* __restrict__ scores) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_q * n_d) return;
  const int q = (int)(idx / n_d), j = (int)(idx - (long long)q * n_d);
  float s = 0.f;
  for (int c = 0; c < q_chunks; ++c) s += partial[((long long)q * q_chunks + c) * n_d + j];
  scores[idx] = s;
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int make_map(CUtensorMap* map, const lik_seqs& s, int dtype, int dim, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return LIK_ERR_CUDA;
  }
  const int eb = (int)dtype_size(dtype);
  CUtensorMapDataType dt = dtype == LIK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype == LIK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                              : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t gdim[2] = {(cuuint64_t)dim, (cuuint64_t)(s.n_rows > 0 ? s.n_rows : 1)};
  cuuint64_t gstride[1] = {(cuuint64_t)s.row_stride * eb};
  cuuint32_t box[2] = {(cuuint32_t)(SLAB_BYTES_ROW / eb), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(s.data), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return LIK_ERR_CUDA;
  }
  return LIK_OK;
}

constexpr size_t SB_WINDOW_BYTES = 48u << 20;   // documents of one super-block: stays in L2 while every group passes
// LIK_SB_WINDOW_MB overrides the window (a tuning knob; document sets below twice the window are walked as one block)
static size_t sb_window_bytes() {
  static size_t v = 0;
  if (!v) {
    const char* e = getenv("LIK_SB_WINDOW_MB");
    const long mb = e ? atol(e) : 0;
    v = mb > 0 ? (size_t)mb << 20 : SB_WINDOW_BYTES;
  }
  return v;
}

struct TcPlan {
  bool pack_tiles;  // ragged queries packed greedily into tiles by pack_query_tiles_kernel
  int q_per_tile, q_chunks, n_tiles, mt, n_slabs, k_steps, stages;
  int n_sb, sb_docs, n_groups;
  long long n_flat, n_units_total;
  int grid;
  size_t smem_bytes;
};

TcPlan plan_tc(const lik_fwd_args& a, const TcExtra& x) {
  TcPlan pl{};
  const int eb = (int)dtype_size(a.dtype);
  pl.n_slabs = (a.dim * eb + SLAB_BYTES_ROW - 1) / SLAB_BYTES_ROW;
  pl.k_steps = (a.dim * eb + 31) / 32;
  const int ml = a.q.max_len > 0 ? a.q.max_len : 1;
  pl.n_sb = 1;
  pl.sb_docs = a.d.n_seq > 0 ? a.d.n_seq : 1;
  if (a.pairing != LIK_PAIR_CROSS) {
    pl.q_per_tile = 1;
    pl.q_chunks = 1;
    pl.n_tiles = a.q.n_seq;
    pl.mt = 1;
    pl.n_groups = a.q.n_seq;
    pl.n_flat = a.pairing == LIK_PAIR_GROUPED ? a.d.n_seq : a.n_pairs;
    pl.n_units_total = pl.n_flat;
  } else {
    if (ml <= TILE_M) {
      pl.q_per_tile = TILE_M / ml;
      pl.q_chunks = 1;
      pl.n_tiles = (int)ceil_div(a.q.n_seq, pl.q_per_tile);
    } else {
      pl.q_per_tile = 1;
      pl.q_chunks = (int)ceil_div(ml, TILE_M);
      pl.n_tiles = a.q.n_seq * pl.q_chunks;
    }
    pl.mt = pl.n_tiles >= 2 ? 2 : 1;
    // packed queries shorter than the fixed slot: let the device pack them tightly (n_tiles becomes an upper bound)
    pl.pack_tiles = a.q.cu && ml < TILE_M && pl.q_per_tile > 1 && a.q.n_seq > 1 && a.q.n_seq <= PACK_MAX_QUERIES;
    pl.n_groups = (int)ceil_div(pl.n_tiles, pl.mt);
    pl.n_flat = 0;
    pl.n_units_total = (long long)pl.n_groups * a.d.n_seq;
    // large document sets are walked in L2-sized super-blocks (several tile groups read every document)
    const size_t row_bytes = x.plaid ? (size_t)(4 + x.plaid->packed_dim) : (size_t)a.dim * eb;
    const size_t d_bytes = (size_t)a.d.n_rows * row_bytes;
    if (a.d.n_seq > 0 && pl.n_groups > 1 && d_bytes > 2 * sb_window_bytes()) {
      const size_t per_doc = d_bytes / (size_t)a.d.n_seq + 1;
      long long sb = (long long)(sb_window_bytes() / per_doc);
      if (sb < 64) sb = 64;
      if (sb < a.d.n_seq) {
        pl.sb_docs = (int)sb;
        pl.n_sb = (int)ceil_div(a.d.n_seq, sb);
      }
    }
  }
  const long long g = pl.n_units_total < sm_count() ? pl.n_units_total : sm_count();
  pl.grid = (int)(g < 0 ? 0 : g);
  // the fused top-k numbers its candidate lists by CTA: the same grid whatever the piece of the corpus
  if (x.topk_k > 0 && pl.grid > 0) pl.grid = sm_count();
  const size_t q_bytes = 2 * (size_t)pl.n_slabs * TILE_M * SLAB_BYTES_ROW;
  const size_t stage = (size_t)pl.n_slabs * TILE_N * SLAB_BYTES_ROW;
  const size_t fixed = q_bytes + sizeof(SharedCtl) + 1024;
  const size_t budget = 227 * 1024;
  int st = (int)((budget - fixed) / stage);
  pl.stages = st > 8 ? 8 : st;
  pl.smem_bytes = fixed + (size_t)pl.stages * stage;
  return pl;
}

}  // namespace

// What the tcgen05 kernel takes.  `plaid`: the documents are a compressed index (a.d.data is NULL).
static bool tc_problem_ok(const lik_fwd_args& a, bool plaid) {
  // per device ordinal: a process may hold GPUs of different architectures
  static signed char dev_ok[64] = {0};  // 0 = not asked yet, 1 = usable, -1 = not usable
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (dev < 0 || dev >= 64) {
    if (!lik_device_supported()) return false;
  } else {
    if (dev_ok[dev] == 0) dev_ok[dev] = lik_device_supported() ? 1 : -1;
    if (dev_ok[dev] < 0) return false;
  }
  if (a.dtype != LIK_BF16 && a.dtype != LIK_F16 && a.dtype != LIK_E4M3) return false;
  if (plaid && a.dtype == LIK_E4M3) return false;
  if (a.pairing < LIK_PAIR_CROSS || a.pairing > LIK_PAIR_LIST) return false;
  const int eb = (int)dtype_size(a.dtype);
  if ((a.dim * eb) % 16 != 0 || a.dim * eb > MAX_SLABS * SLAB_BYTES_ROW) return false;
  if (a.q.n_seq <= 0 || a.d.n_seq <= 0 || a.q.n_rows <= 0 || a.d.n_rows <= 0) return false;
  if (a.q.max_len <= 0) return false;  // packed queries need their longest length to form tiles
  if (a.pairing != LIK_PAIR_CROSS && a.q.max_len > TILE_M) return false;  // one query per tile
  if (a.pairing == LIK_PAIR_LIST) {
    if (a.n_pairs <= 0 || a.n_pairs >= (1ll << 31) || !a.pair_q || !a.pair_d) return false;
    if (a.d.mask) return false;  // token masks with holes are not carried by the pair table
  }
  if ((a.q.row_stride * eb) % 16 != 0 || ((uintptr_t)a.q.data & 15)) return false;
  if (!plaid && ((a.d.row_stride * eb) % 16 != 0 || ((uintptr_t)a.d.data & 15))) return false;
  if (a.q.n_rows >= (1ll << 31) || a.d.n_rows >= (1ll << 31)) return false;
  if (a.argmax && a.argmax_stride < 0) return false;
  return get_encode_fn() != nullptr;
}

bool fwd_tc_supported(const lik_fwd_args& a) { return tc_problem_ok(a, false); }

// Helpers shared with the document-head kernel: a 128-byte-swizzled TMA map over the rows of a matrix whose box is
// one 128-byte K slab wide and `box_rows` high, and the effective document lengths under a token mask.
int make_tmap_rows(CUtensorMap* map, const void* data, int dtype, long long inner, long long n_rows, long long row_stride,
                   int box_rows) {
  lik_seqs s{};
  s.data = data;
  s.n_rows = n_rows;
  s.row_stride = row_stride;
  return make_map(map, s, dtype, (int)inner, box_rows);
}
bool tmap_available() { return get_encode_fn() != nullptr; }
int launch_mask_lens(const unsigned char* mask, const int* lens, int n_seq, int max_len, long long seq_stride, int* out,
                     cudaStream_t st) {
  if (n_seq <= 0) return LIK_OK;
  mask_lens_kernel<<<(unsigned)ceil_div(n_seq, 8), 256, 0, st>>>(mask, lens, n_seq, max_len, seq_stride, out), ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

// The fused top-k needs fixed query slots (padded queries of at most 128 tokens) and k within the list size.
bool fwd_tc_topk_supported(const lik_fwd_args& a, const TcExtra& x) {
  if (!tc_problem_ok(a, x.plaid != nullptr)) return false;
  if (a.pairing != LIK_PAIR_CROSS || a.q.cu || a.q.max_len > TILE_M || a.argmax) return false;
  return x.topk_k >= 1 && x.topk_k <= TOPK_CAP / 2;
}

bool fwd_tc_plaid_supported(const lik_fwd_args& a, const TcExtra& x) {
  if (!x.plaid || !tc_problem_ok(a, true)) return false;
  if (x.plaid->dim != a.dim || a.dim % 16 != 0 || a.dim > 128 || a.d.mask || a.d.scale) return false;
  return plaid_row16_ok(*x.plaid);
}

int topk_merge_parts(int n_ctas, int n_groups);

namespace {
struct TcWs {
  size_t partial, lens, tiles, list, hdr, keys, idx, merge, total;
  long long n_lists;
  int merge_parts;  // the lists of a query are merged in this many parts first (1: in one pass)
};
TcWs tc_ws_layout(const TcPlan& pl, const lik_fwd_args& a, const TcExtra& x) {
  TcWs w{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += align_up(bytes, 256);
    return o;
  };
  // the candidate lists first: their size depends on the queries and the machine only, so they keep their place
  // when the documents come in pieces
  w.n_lists = 0;
  if (x.topk_k > 0) {
    w.n_lists = (long long)(pl.grid + pl.n_groups) * 2 * pl.q_per_tile;
    w.hdr = take((size_t)w.n_lists * sizeof(int2));
    w.keys = take((size_t)w.n_lists * TOPK_CAP * sizeof(float));
    w.idx = take((size_t)w.n_lists * TOPK_CAP * sizeof(int));
    // few tile groups: a query has lists from many CTAs, which are merged in parts by as many CTAs first
    w.merge_parts = topk_merge_parts(pl.grid, pl.n_groups);
    w.merge = take(w.merge_parts > 1 ? (size_t)w.merge_parts * a.q.n_seq * x.topk_k * (sizeof(float) + sizeof(long long)) + 8 : 0);
  }
  w.partial = take(pl.q_chunks > 1 ? (size_t)pl.n_tiles * a.d.n_seq * sizeof(float) : 0);
  w.lens = take((a.d.mask && !a.d.cu) ? (size_t)a.d.n_seq * sizeof(int) : 0);
  w.tiles = take(pl.pack_tiles ? (size_t)(a.q.n_seq + 3) * sizeof(int) : 0);
  w.list = take(a.pairing == LIK_PAIR_LIST ? (size_t)a.n_pairs * sizeof(int4) : 0);
  w.total = off;
  return w;
}
}  // namespace

size_t fwd_tc_workspace(const lik_fwd_args& a, const TcExtra& x) { return tc_ws_layout(plan_tc(a, x), a, x).total; }

int launch_topk_slots(const float* keys, const int* idx, const int2* hdr, long long n_lists, int cap, int n_ctas, int n_groups,
                      int mt, int qpt, long long n_q, int k, int largest, long long index_offset, float* out_scores,
                      long long* out_index, int parts, void* part_buf, cudaStream_t st);

// Raise the kernel's dynamic shared memory limit once per device and size instead of on every launch (a host call
// of a microsecond or two that small problems feel).
template <bool F, int A, bool X, bool PL>
static cudaError_t allow_smem(size_t bytes) {
  static size_t allowed[64] = {0};  // by device ordinal
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && allowed[dev] >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(fwd_tc_kernel<F, A, X, PL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && dev >= 0 && dev < 64) allowed[dev] = bytes;
  return e;
}

int launch_fwd_tc(const lik_fwd_args& a, const float* qn, const float* dn, void* ws, size_t ws_bytes, cudaStream_t st,
                  const TcExtra& x) {
  TcPlan pl = plan_tc(a, x);
  if (pl.stages < 1) {
    set_error("not enough shared memory for the document ring");
    return LIK_ERR_UNSUPPORTED;
  }
  const TcWs w = tc_ws_layout(pl, a, x);
  if (ws_bytes < w.total || (w.total && !ws)) {  // before anything that writes into the workspace is enqueued
    set_error("tcgen05 forward: workspace too small");
    return LIK_ERR_WORKSPACE;
  }
  if (pl.grid < 1) return LIK_OK;
  const bool plaid = x.plaid != nullptr;
  CUtensorMap q_map;
  DocMaps d_maps;
  memset(&d_maps, 0, sizeof(d_maps));
  int rc = make_map(&q_map, a.q, a.dtype, a.dim, TILE_M);
  if (rc) return rc;
  if (!plaid) {
    for (int i = 0; i < 4; ++i) {
      rc = make_map(&d_maps.m[i], a.d, a.dtype, a.dim, (i + 1) * BOX_ROWS);
      if (rc) return rc;
    }
  }

  TcParams P{};
  P.q = make_view(a.q, qn);
  P.d = make_view(a.d, dn);
  P.pairing = a.pairing;
  P.group = a.group;
  P.n_q = a.q.n_seq;
  P.n_d = a.d.n_seq;
  P.elt_bytes = (int)dtype_size(a.dtype);
  P.ab_format = a.dtype == LIK_BF16 ? 1 : 0;  // kind::f16: F16 = 0, BF16 = 1; kind::f8f6f4: E4M3 = 0
  P.n_slabs = pl.n_slabs;
  P.k_steps = pl.k_steps;
  P.stages = pl.stages;
  P.q_per_tile = pl.q_per_tile;
  P.q_chunks = pl.q_chunks;
  P.n_tiles = pl.n_tiles;
  P.mt = pl.mt;
  P.n_sb = pl.n_sb;
  P.sb_docs = pl.sb_docs;
  P.n_flat = pl.n_flat;
  P.scores = a.scores;
  P.partial = pl.q_chunks > 1 ? (float*)((char*)ws + w.partial) : nullptr;
  P.d_len_flagged = 0;
  P.tile_q0 = nullptr;
  P.list_tab = nullptr;
  P.d_full_count = plaid ? PLAID_WARPS : 1;
  // Per-column multipliers that are exactly one fp32 array over the document rows (inverse norms or per-token scales,
  // not both) travel with the tiles when every tile's run of them starts on a 16-byte boundary and whole groups of four
  // stay inside the array: padded documents whose stride and row count are multiples of four.
  P.col_src = nullptr;
  P.sc_per = P.sc_slots = 0;
  if (!plaid && !a.d.cu && a.d.scale_scalar == 1.0f && ((a.d.scale != nullptr) != (dn != nullptr))) {
    const float* arr = a.d.scale ? a.d.scale : dn;
    if (((uintptr_t)arr & 15) == 0 && a.d.seq_stride % 4 == 0 && a.d.n_rows % 4 == 0) {
      const size_t stage = (size_t)pl.n_slabs * TILE_N * SLAB_BYTES_ROW;
      const size_t fixed = pl.smem_bytes - (size_t)pl.stages * stage;
      auto need = [&](int stages) { return fixed + (size_t)stages * stage + (size_t)2 * (stages + 1) * TILE_N * sizeof(float); };
      int stages = pl.stages;
      while (stages > 1 && need(stages) > (size_t)227 * 1024) --stages;
      if (need(stages) <= (size_t)227 * 1024) {
        pl.stages = stages;
        pl.smem_bytes = need(stages);
        P.stages = stages;
        P.col_src = arr;
        P.sc_per = stages + 1;
        P.sc_slots = 2 * P.sc_per;
      }
    }
  }
  if (plaid) {
    P.plaid = *x.plaid;
    P.plaid_f16 = a.dtype == LIK_F16;
  }
  if (pl.pack_tiles) {
    int* tbl = (int*)((char*)ws + w.tiles);
    pack_query_tiles_kernel<<<1, 256, 0, st>>>(a.q.cu, a.q.n_seq, tbl), ::lik::count_launch();
    LIK_CUDA_OK(cudaGetLastError());
    P.tile_q0 = tbl + 1;
  }
  if (a.d.mask && !a.d.cu) {
    // trim every document to its last valid token; only documents with holes pay for per-column masking
    int* eff = (int*)((char*)ws + w.lens);
    mask_lens_kernel<<<(unsigned)ceil_div(a.d.n_seq, 8), 256, 0, st>>>(a.d.mask, a.d.lens, a.d.n_seq, a.d.max_len, a.d.seq_stride, eff), ::lik::count_launch();
    LIK_CUDA_OK(cudaGetLastError());
    P.d.lens = eff;
    P.d_len_flagged = 1;
  }
  if (a.pairing == LIK_PAIR_LIST) {
    int4* tab = (int4*)((char*)ws + w.list);
    list_units_kernel<<<(unsigned)ceil_div(a.n_pairs, 256), 256, 0, st>>>(P.q, P.d, a.pair_q, a.pair_d, a.n_pairs, tab, a.status), ::lik::count_launch();
    LIK_CUDA_OK(cudaGetLastError());
    P.list_tab = tab;
  }
  P.argmax = a.argmax;
  P.argmax_stride = a.argmax_stride;
  P.status = a.status;
  if (x.topk_k > 0) {
    P.topk.hdr = (int2*)((char*)ws + w.hdr);
    P.topk.cand_key = (float*)((char*)ws + w.keys);
    P.topk.cand_idx = (int*)((char*)ws + w.idx);
    P.topk.k = x.topk_k;
    P.topk.qpg = 2 * pl.q_per_tile;
    P.topk.largest = x.topk_largest;
    P.topk.doc_base = x.topk_doc_base;
    P.topk.n_lists = (int)w.n_lists;
    if (!(x.topk_flags & LIK_TOPK_CONTINUE))
      LIK_CUDA_OK(cudaMemsetAsync(P.topk.hdr, 0, (size_t)w.n_lists * sizeof(int2), st));  // empty lists, no threshold
  }
  // positions of the saved argmax that no accumulator row covers (queries shorter than the stride)
  if (a.argmax && (a.q.cu || a.q.lens || a.argmax_stride > a.q.max_len))
    LIK_CUDA_OK(cudaMemsetAsync(a.argmax, 0xFF,
                                (size_t)n_scores_of(a.pairing, a.q.n_seq, a.d.n_seq, a.n_pairs) * a.argmax_stride * sizeof(int), st));

  const bool fp8 = a.dtype == LIK_E4M3;
  const bool argmax = a.argmax != nullptr;
  const bool affine = a.d.scale || dn;  // a per-column multiplier for every document
  dim3 grid((unsigned)pl.grid), block(NUM_THREADS);
#define LIK_TC_LAUNCH(F, A, X, PL)                                                                                     \
  do {                                                                                                                 \
    LIK_CUDA_OK((allow_smem<F, A, X, PL>(pl.smem_bytes)));                                                             \
    fwd_tc_kernel<F, A, X, PL><<<grid, block, pl.smem_bytes, st>>>(q_map, d_maps, P), ::lik::count_launch();           \
  } while (0)
  // LIK_LONG_DOC_TOKENS overrides the length from which the lazy winner scan is used (a tuning knob)
  static int long_doc_tokens = 0;
  if (!long_doc_tokens) {
    const char* e = getenv("LIK_LONG_DOC_TOKENS");
    const int v = e ? atoi(e) : 0;
    long_doc_tokens = v > 0 ? v : LONG_DOC_TOKENS;
  }
  const bool long_docs = argmax && a.d.max_len >= long_doc_tokens;
  if (plaid) {
    if (argmax) LIK_TC_LAUNCH(false, 1, false, true);
    else LIK_TC_LAUNCH(false, 0, false, true);
  } else if (fp8) {
    if (argmax && affine) LIK_TC_LAUNCH(true, 1, true, false);
    else if (argmax) LIK_TC_LAUNCH(true, 1, false, false);
    else if (affine) LIK_TC_LAUNCH(true, 0, true, false);
    else LIK_TC_LAUNCH(true, 0, false, false);
  } else {
    if (long_docs && affine) LIK_TC_LAUNCH(false, 2, true, false);
    else if (long_docs) LIK_TC_LAUNCH(false, 2, false, false);
    else if (argmax && affine) LIK_TC_LAUNCH(false, 1, true, false);
    else if (argmax) LIK_TC_LAUNCH(false, 1, false, false);
    else if (affine) LIK_TC_LAUNCH(false, 0, true, false);
    else LIK_TC_LAUNCH(false, 0, false, false);
  }
#undef LIK_TC_LAUNCH
  LIK_CUDA_OK(cudaGetLastError());
  if (pl.q_chunks > 1) {
    const long long n = (long long)a.q.n_seq * a.d.n_seq;
    reduce_chunks_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(P.partial, a.q.n_seq, a.d.n_seq, pl.q_chunks, a.scores), ::lik::count_launch();
    LIK_CUDA_OK(cudaGetLastError());
  }
  if (x.topk_k > 0 && !(x.topk_flags & LIK_TOPK_PARTIAL)) {
    rc = launch_topk_slots(P.topk.cand_key, P.topk.cand_idx, P.topk.hdr, w.n_lists, TOPK_CAP, pl.grid, pl.n_groups, pl.mt, pl.q_per_tile,
                           a.q.n_seq, x.topk_k, x.topk_largest, x.topk_index_offset, x.topk_scores, (long long*)x.topk_index,
                           w.merge_parts, w.merge_parts > 1 ? (char*)ws + w.merge : nullptr, st);
    if (rc) return rc;
  }
  return LIK_OK;
}

}  // namespace lik

extern "C" int lik_selftest_wait_timeout(int64_t limit_cycles, int32_t* status, int32_t* result, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(result != nullptr, "result is NULL");
  LIK_REQUIRE(limit_cycles > 0 && limit_cycles <= 200000000ll, "limit_cycles outside (0, 2e8]");
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((long long)limit_cycles, status, result), ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}
