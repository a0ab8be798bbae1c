// Document head chained into MaxSim on the tensor cores (sm_100a: TMA + tcgen05.mma + TMEM).
//
//   scores[i, j] = sum_s max_t < q[i, s], normalize(h[j, t] @ w^T + bias) >
//
// Two MMAs back to back per 128-token tile of a document.  The projection (rows = the tile's tokens, columns =
// d_out, K = d_model streamed in 128-byte slabs of h and w through a TMA ring) accumulates in tensor memory.  Four
// "converter" warps read it (one thread per token, so a token's whole projected row passes through one thread), add
// the bias, round to the operand type, sum the squares of the rounded values for the inverse norm, and store the
// row into shared memory in the swizzled K-major layout the scoring MMA reads as its B operand.  The scoring MMA
// (rows = query tokens of a resident query tile, columns = the tile's tokens, K = d_out) accumulates in tensor
// memory as well; its epilogue warps multiply every column by the token's inverse norm, add the token's mask
// (0 or -inf), and keep a running (max, argmax) per query token across the tiles of a document.  The projected
// tokens never reach device memory.
//
// Warp roles (448 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 = converters,
// warps 6-9 / 10-13 = scoring epilogue of query tile 0 / 1.  Tensor memory: projection accumulators at columns
// [0, 128) and [128, 256) (double-buffered), scoring accumulators at [256, 384) and [384, 512) (one per query
// tile).  The issuer queues the projection of tile n + 1 before it waits for the converted tile n, so the tensor
// pipe works on the next projection while the converters run.  A CTA owns a contiguous range of documents, so every
// score has one writer and the result is bitwise reproducible.
//
// What bounds it: DRAM traffic is the hidden states once (w comes back from L2 for every tile), streamed at about
// 0.8 of the copy bandwidth.  The hidden states wait in the ring for the tensor pipe rather than the other way round:
// a 128 x 128 x 16 MMA reads 8 KB of operands from shared memory per 64 cycles, all of its bandwidth, while TMA fills
// the ring and the converters store the operand tile.  Measured and dropped: a ring of its own for w (one more wait
// and commit per stage on the issuing thread cost more than the deeper hidden-state ring gave), and two token tiles per
// w slab with single-buffered projection accumulators (the tensor pipe idles while the converters run).
//
// Every mbarrier wait is bounded: on expiry the CTA raises LIK_DEV_WAIT_TIMEOUT in the status word, sets a shared
// abort flag, drains its TMA copies, frees TMEM and returns.
#include <cuda.h>

#include <cstring>

#include "lik_common.cuh"
#include "lik_tc.cuh"
#include "lik_tc_ptx.cuh"

namespace lik {

namespace {

constexpr int HD_TOK = 128;          // document tokens per tile
constexpr int HD_SLAB_ROW = 128;     // bytes of one K slab per row (one swizzle span)
constexpr int HD_SLAB = HD_TOK * HD_SLAB_ROW;  // bytes of a 128-row slab
constexpr int HD_THREADS = 448;
constexpr int HD_EPI_WARP0 = 6;  // warps 2..5 convert, warps 6.. score
constexpr int HD_MAX_STAGES = 6;
constexpr long long HD_WAIT_LIMIT = 4000000000ll;  // about 2 s at 2 GHz

struct HeadParams {
  int n_d, ld;
  long long seq_stride;        // rows between document starts
  const int* lens;             // effective lengths (LEN_FLAG_MASKED tagged when lens_flagged), or nullptr
  int lens_flagged;
  const unsigned char* mask;   // per row, or nullptr
  int d_model, d_out;
  int n_k;                     // 128-byte K slabs of the projection
  int n_s2;                    // 128-byte K slabs of the scoring MMA (d_out)
  int stages;
  int mt;                      // resident query tiles (1 or 2)
  int n_q, lq, q_per_tile;
  int q_last_rows;             // rows held of the last query tile (a multiple of 8): the rows behind them are never looked at
  int f16;
  int normalize;
  const void* bias;
  float* scores;
  int* argmax;
  int argmax_stride;
  int* status;
};

struct HeadCtl {
  unsigned long long q_full;
  unsigned long long ring_full[HD_MAX_STAGES], ring_empty[HD_MAX_STAGES];
  unsigned long long acc1_full[2], acc1_empty[2];
  unsigned long long p_full, p_empty;
  unsigned long long acc2_full[2], acc2_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  long long wait_limit;
  float bias[HD_TOK];
  alignas(16) float col_scale[2][HD_TOK];
  alignas(16) float col_bias[2][HD_TOK];
  float emit[2][2][TILE_M];
};

__device__ __noinline__ bool hd_wait_slow(uint32_t b, uint32_t parity, HeadCtl* ctl, int* status) {
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
__device__ __forceinline__ bool hd_wait(unsigned long long* bar, uint32_t parity, HeadCtl* ctl, int* status) {
  const uint32_t b = smem_u32(bar);
  if (mbar_try_wait(b, parity)) return true;
  return hd_wait_slow(b, parity, ctl, status);
}

// Tokens of document `doc` that take part (its tiles cover [0, len)).
__device__ __forceinline__ int hd_doc_len(const HeadParams& P, int doc) {
  if (!P.lens) return P.ld;
  int l = P.lens[doc];
  if (P.lens_flagged) l &= ~LEN_FLAG_MASKED;
  return l < 0 ? 0 : (l > P.ld ? P.ld : l);
}

// Round two projected values to the operand type, add their squares (as rounded) to ss, return the packed pair.
template <bool F16>
__device__ __forceinline__ uint32_t hd_pack2(float a, float b, float& ss) {
  if (F16) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 f = __half22float2(h);
    ss = fmaf(f.x, f.x, ss);
    ss = fmaf(f.y, f.y, ss);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const float2 f = __bfloat1622float2(h);
    ss = fmaf(f.x, f.x, ss);
    ss = fmaf(f.y, f.y, ss);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
}

// 32 projected values of one token (columns c .. c + 31 of its row) -> bias, rounding, four 16-byte stores into the
// swizzled operand tile.  `keep` is false for rows past the end of the document, which are stored as zeros.
template <bool F16>
__device__ __forceinline__ void hd_convert32(const float (&v)[32], const float* bias, bool keep, unsigned char* row_base, int unit0,
                                             int row, float& ss) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 o;
    o.x = hd_pack2<F16>(v[8 * j + 0] + bias[8 * j + 0], v[8 * j + 1] + bias[8 * j + 1], ss);
    o.y = hd_pack2<F16>(v[8 * j + 2] + bias[8 * j + 2], v[8 * j + 3] + bias[8 * j + 3], ss);
    o.z = hd_pack2<F16>(v[8 * j + 4] + bias[8 * j + 4], v[8 * j + 5] + bias[8 * j + 5], ss);
    o.w = hd_pack2<F16>(v[8 * j + 6] + bias[8 * j + 6], v[8 * j + 7] + bias[8 * j + 7], ss);
    if (!keep) o = make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(row_base + ((((unit0 + j) ^ (row & 7))) << 4)) = o;
  }
}

// The four K steps of one 128-byte slab as one block: the descriptors of steps 1..3 are the first one's plus 2, 4, 6
// (16-byte units).  The issuing thread is a serial bottleneck of this kernel (one MMA per 4 KB of hidden states), so
// the code between two MMAs is kept to the few instructions that build the descriptors.
__device__ __forceinline__ void tc_mma_slab_f16(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                                uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 da, db;\n\t.reg .b32 ta, tb;\n\t"
      "setp.ne.b32 p0, %5, 0;\n\tsetp.eq.b32 p1, %3, %3;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p0;\n\t"
      "add.u32 ta, %1, 2;\n\tadd.u32 tb, %2, 2;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p1;\n\t"
      "add.u32 ta, %1, 4;\n\tadd.u32 tb, %2, 4;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p1;\n\t"
      "add.u32 ta, %1, 6;\n\tadd.u32 tb, %2, 6;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p1;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate_first)
      : "memory");
}

template <bool ARGMAX>
__global__ void __launch_bounds__(HD_THREADS, 1)
head_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap h_map,
               const __grid_constant__ CUtensorMap w_map, const HeadParams P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int q_tile_bytes = P.n_s2 * HD_SLAB;
  unsigned char* q_smem = smem;                                     // [mt][n_s2][128 rows (last tile: q_last_rows)][128 B]
  // (the last query tile holds only the rows that queries occupy: the MMA still reads 128 rows, and what it reads
  // behind them - the next buffers - only reaches accumulator rows that nobody looks at)
  unsigned char* p_smem = q_smem + (P.mt - 1) * q_tile_bytes + P.n_s2 * P.q_last_rows * HD_SLAB_ROW;  // [n_s2][128 rows][128 B]
  unsigned char* ring = p_smem + P.n_s2 * HD_SLAB;                  // [stages]{h slab [128][128 B], w slab [d_out][128 B]}
  constexpr int STAGE_BYTES = 2 * HD_SLAB;
  HeadCtl* ctl = reinterpret_cast<HeadCtl*>(ring + (size_t)P.stages * STAGE_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(smem_u32(&ctl->q_full), 1);
    for (int s = 0; s < P.stages; ++s) {
      mbar_init(smem_u32(&ctl->ring_full[s]), 1);
      mbar_init(smem_u32(&ctl->ring_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc1_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc1_empty[a]), 4);
      mbar_init(smem_u32(&ctl->acc2_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc2_empty[a]), 4);
    }
    mbar_init(smem_u32(&ctl->p_full), 4);
    mbar_init(smem_u32(&ctl->p_empty), 1);
    ctl->abort_flag = 0;
    ctl->wait_limit = HD_WAIT_LIMIT;
    fence_barrier_init();
    prefetch_tmap(&q_map);
    prefetch_tmap(&h_map);
    prefetch_tmap(&w_map);
  }
  if (tid < HD_TOK) {
    float bv = 0.f;
    if (P.bias && tid < P.d_out)
      bv = P.f16 ? __half2float(reinterpret_cast<const __half*>(P.bias)[tid]) : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(P.bias)[tid]);
    ctl->bias[tid] = bv;
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  // this CTA's documents
  const int doc_lo = (int)((long long)P.n_d * blockIdx.x / gridDim.x);
  const int doc_hi = (int)((long long)P.n_d * (blockIdx.x + 1) / gridDim.x);
  const int ab_format = P.f16 ? 0 : 1;

  if (warp == 0) {
    // =========================== producer ===========================
    if (lane == 0) {
      uint32_t st = 0, ph = 0, n_load = 0;
      bool ok = true;
      // the query tiles stay for the whole kernel
      mbar_arrive_expect_tx(smem_u32(&ctl->q_full), (uint32_t)((P.mt - 1) * q_tile_bytes + P.n_s2 * P.q_last_rows * HD_SLAB_ROW));
      for (int m = 0; m < P.mt; ++m) {
        const int rows = m == P.mt - 1 ? P.q_last_rows : TILE_M;
        for (int sl = 0; sl < P.n_s2; ++sl)
          for (int r = 0; r < rows; r += 8)  // boxes of 8 rows (one swizzle atom)
            tma_load_2d(smem_u32(q_smem + m * q_tile_bytes + (sl * rows + r) * HD_SLAB_ROW), &q_map, sl * 64, m * P.q_per_tile * P.lq + r,
                        smem_u32(&ctl->q_full));
      }
      const uint32_t stage_tx = (uint32_t)(HD_SLAB + P.d_out * HD_SLAB_ROW);
      for (int doc = doc_lo; doc < doc_hi && ok; ++doc) {
        const int len = hd_doc_len(P, doc);
        const long long row0 = (long long)doc * P.seq_stride;
        for (int t0 = 0; t0 < len && ok; t0 += HD_TOK) {
          for (int ks = 0; ks < P.n_k; ++ks) {
            ok = hd_wait(&ctl->ring_empty[st], ph ^ 1, ctl, P.status);
            if (!ok) break;
            const uint32_t full = smem_u32(&ctl->ring_full[st]);
            unsigned char* stage = ring + (size_t)st * STAGE_BYTES;
            mbar_arrive_expect_tx(full, stage_tx);
            tma_load_2d(smem_u32(stage), &h_map, ks * 64, (int)(row0 + t0), full);
            tma_load_2d(smem_u32(stage + HD_SLAB), &w_map, ks * 64, 0, full);
            ++n_load;
            if (++st == (uint32_t)P.stages) { st = 0; ph ^= 1; }
          }
        }
      }
      // (a CTA whose documents are all empty never scores: the query tiles must still have landed before it leaves)
      if (ok) ok = hd_wait(&ctl->q_full, 0, ctl, P.status);
      if (!ok) {
        // aborting: let the copies already issued land before the CTA goes away
        for (uint32_t i = 1; i <= (uint32_t)P.stages && i <= n_load; ++i) {
          const bool wrapped = i > st;
          const uint32_t slot = wrapped ? st + (uint32_t)P.stages - i : st - i;
          const uint32_t bar = smem_u32(&ctl->ring_full[slot]);
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(bar, wrapped ? ph ^ 1 : ph); ++spin) {
          }
        }
        const uint32_t qbar = smem_u32(&ctl->q_full);
        for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(qbar, 0); ++spin) {
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      uint32_t st = 0, ph = 0, n1 = 0, n2 = 0;
      bool ok = true, have_pend = false;
      int pend_cols = 0;
      const uint32_t desc_hi = (uint32_t)(smem_desc_sw128(0) >> 32);
      const uint32_t ring_desc0 = (uint32_t)smem_desc_sw128(smem_u32(ring));
      const uint32_t q_desc0 = (uint32_t)smem_desc_sw128(smem_u32(q_smem));
      const uint32_t p_desc0 = (uint32_t)smem_desc_sw128(smem_u32(p_smem));
      const uint32_t idesc1 = instr_desc(ab_format, P.d_out);
      const uint32_t idesc2_0 = instr_desc(ab_format, 0);
      const int k2_steps = P.d_out / 16;
      const uint32_t full0 = smem_u32(&ctl->ring_full[0]), empty0 = smem_u32(&ctl->ring_empty[0]);
      const uint32_t last_q_slab = (uint32_t)((P.q_last_rows * HD_SLAB_ROW) >> 4);  // slab pitch of the last (trimmed) query tile
      // scoring MMA of the tile converted last: every resident query tile against the tile's tokens
      auto score_tile = [&](int ncols) -> bool {
        if (n2 == 0 && !hd_wait(&ctl->q_full, 0, ctl, P.status)) return false;
        if (!hd_wait(&ctl->p_full, n2 & 1, ctl, P.status)) return false;
        const uint32_t idesc2 = idesc2_0 | ((uint32_t)((ncols + 31) >> 5) << 19);  // N / 8 in bits 17..22, N a multiple of 32
        for (int m = 0; m < P.mt; ++m) {
          if (!hd_wait(&ctl->acc2_empty[m], (n2 & 1) ^ 1, ctl, P.status)) return false;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + 256u + (uint32_t)(m * HD_TOK);
          const uint32_t a0 = q_desc0 + (uint32_t)((m * q_tile_bytes) >> 4);
          const uint32_t a_slab = m == P.mt - 1 ? last_q_slab : (uint32_t)(HD_SLAB >> 4);
          if (k2_steps == 8) {
            tc_mma_slab_f16(d_tmem, a0, p_desc0, desc_hi, idesc2, 0u);
            tc_mma_slab_f16(d_tmem, a0 + a_slab, p_desc0 + (uint32_t)(HD_SLAB >> 4), desc_hi, idesc2, 1u);
          } else {
            for (int k = 0; k < k2_steps; ++k)
              tc_mma<false>(d_tmem, a0 + (uint32_t)((k & 3) * 2) + (uint32_t)(k >> 2) * a_slab,
                            p_desc0 + (uint32_t)((k & 3) * 2 + (k >> 2) * (HD_SLAB >> 4)), desc_hi, idesc2, k ? 1u : 0u);
          }
          tc_commit(smem_u32(&ctl->acc2_full[m]));
        }
        tc_commit(smem_u32(&ctl->p_empty));
        ++n2;
        return true;
      };
      for (int doc = doc_lo; doc < doc_hi && ok; ++doc) {
        const int len = hd_doc_len(P, doc);
        for (int t0 = 0; t0 < len && ok; t0 += HD_TOK) {
          const uint32_t a = n1 & 1;
          ok = hd_wait(&ctl->acc1_empty[a], ((n1 >> 1) & 1) ^ 1, ctl, P.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + a * (uint32_t)HD_TOK;
          for (int ks = 0; ks < P.n_k; ++ks) {
            // (data landed by TMA and consumed by the MMA: the barrier alone orders the two)
            if (!mbar_try_wait(full0 + 8u * st, ph)) {
              ok = hd_wait_slow(full0 + 8u * st, ph, ctl, P.status);
              if (!ok) break;
            }
            const uint32_t h_desc = ring_desc0 + st * (uint32_t)(STAGE_BYTES >> 4);
            tc_mma_slab_f16(d_tmem, h_desc, h_desc + (uint32_t)(HD_SLAB >> 4), desc_hi, idesc1, (uint32_t)ks);
            tc_commit(empty0 + 8u * st);
            if (++st == (uint32_t)P.stages) { st = 0; ph ^= 1; }
          }
          if (!ok) break;
          tc_commit(smem_u32(&ctl->acc1_full[a]));
          ++n1;
          if (have_pend) ok = score_tile(pend_cols);
          pend_cols = min(HD_TOK, len - t0);
          have_pend = true;
        }
      }
      if (ok && have_pend) ok = score_tile(pend_cols);
    }
  } else if (warp < HD_EPI_WARP0) {
    // =========================== converters ===========================
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // token of the tile == TMEM lane
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    unsigned char* row_base = p_smem + row * HD_SLAB_ROW;
    uint32_t n1 = 0;
    bool ok = true;
    for (int doc = doc_lo; doc < doc_hi && ok; ++doc) {
      const int len = hd_doc_len(P, doc);
      const long long row0 = (long long)doc * P.seq_stride;
      for (int t0 = 0; t0 < len; t0 += HD_TOK) {
        const uint32_t a = n1 & 1;
        const int ncols = min(HD_TOK, len - t0);
        const bool in_doc = row < ncols;
        bool valid = in_doc;
        if (in_doc && P.mask) valid = P.mask[row0 + t0 + row] != 0;
        ok = hd_wait(&ctl->acc1_full[a], (n1 >> 1) & 1, ctl, P.status) && hd_wait(&ctl->p_empty, (n1 & 1) ^ 1, ctl, P.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float ss = 0.f;
        for (int c = 0; c < P.d_out; c += 32) {
          float v[32];
          tmem_ld32_issue(lane_addr + a * (uint32_t)HD_TOK + (uint32_t)c, v);
          tmem_ld_wait(v);
          unsigned char* dst = row_base + (c >> 6) * HD_SLAB;
          if (P.f16) hd_convert32<true>(v, &ctl->bias[c], in_doc, dst, (c & 63) >> 3, row, ss);
          else hd_convert32<false>(v, &ctl->bias[c], in_doc, dst, (c & 63) >> 3, row, ss);
        }
        // the projection accumulator goes back to the issuer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->acc1_empty[a]));
        const float inv = P.normalize ? 1.0f / fmaxf(sqrtf(ss), 1e-12f) : 1.0f;
        ctl->col_scale[n1 & 1][row] = in_doc ? inv : 0.f;
        ctl->col_bias[n1 & 1][row] = valid ? 0.f : -INFINITY;
        fence_proxy_async();  // the operand stores above are read by the tensor core
        __threadfence_block();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full));
        ++n1;
      }
    }
  } else {
    // =========================== scoring epilogue ===========================
    const int e = warp - HD_EPI_WARP0;
    const int m = e >> 2;              // query tile
    const int wq = e & 3;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // query token slot in the tile == TMEM lane
    if (m < P.mt) {
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + 256u + (uint32_t)(m * HD_TOK);
      const int q_first = m * P.q_per_tile;
      const int q_here = max(0, min(P.q_per_tile, P.n_q - q_first));
      const int my_q = q_first + row / P.lq, my_s = row % P.lq;
      const bool in_q = row < q_here * P.lq;
      uint32_t n = 0, n_doc = 0;
      bool ok = true;
      for (int doc = doc_lo; doc < doc_hi && ok; ++doc) {
        const int len = hd_doc_len(P, doc);
        float run_m = -INFINITY;
        int run_i = -1;
        for (int t0 = 0; t0 < len; t0 += HD_TOK) {
          const int ncols = min(HD_TOK, len - t0);
          {
            // the tile's first warp waits; the rendezvous tells the other three whether it gave up, so that the four
            // always agree (they meet again at the end of the document)
            bool gave_up = false;
            if (wq == 0) gave_up = !hd_wait(&ctl->acc2_full[m], n & 1, ctl, P.status);
            int n_gave_up;
            asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %3, 0;\n\tbar.red.popc.u32 %0, %1, %2, q;\n\t}"
                         : "=r"(n_gave_up) : "r"(1 + m), "r"(128), "r"((int)(gave_up && lane == 0)) : "memory");
            ok = n_gave_up == 0;
          }
          if (!ok) break;
          tc_fence_after();
          const float* sc = ctl->col_scale[n & 1];
          const float* bi = ctl->col_bias[n & 1];
          for (int cc = 0; cc < ncols; cc += 32) {
            float v[32];
            tmem_ld32_issue(lane_addr + (uint32_t)cc, v);
            tmem_ld_wait(v);
            affine32(v, sc + cc, bi + cc);  // inverse norm of the token; -inf for masked tokens and past the document's end
            fold32<ARGMAX>(v, t0 + cc, run_m, run_i);
          }
          // (released after the per-column factors were read: the converters may overwrite them two tiles on)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl->acc2_empty[m]));
          ++n;
        }
        if (!ok) break;
        const bool has_winner = ARGMAX ? (run_i >= 0) : (run_m != -INFINITY);
        const float val = (in_q && has_winner) ? run_m : 0.f;
        if (ARGMAX && in_q && my_s < P.argmax_stride)
          P.argmax[((long long)my_q * P.n_d + doc) * P.argmax_stride + my_s] = has_winner ? run_i : -1;
        float* ebuf = ctl->emit[m][n_doc & 1];
        ++n_doc;
        ebuf[row] = val;
        asm volatile("bar.sync %0, %1;" ::"r"(1 + m), "r"(128) : "memory");
        // one value per query token, summed per query in a fixed order
        for (int qi = wq; qi < q_here; qi += 4) {
          float sum = 0.f;
          for (int i = lane; i < P.lq; i += 32) sum += ebuf[qi * P.lq + i];
          sum = warp_sum(sum);
          if (lane == 0) P.scores[(long long)(q_first + qi) * P.n_d + doc] = sum;
        }
      }
    }
  }

  // ---- teardown (also reached when aborting: every wait above is bounded) ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// Backward helpers: only winning tokens carry gradient, so the backward works on "compact" documents made of the
// distinct winners of each document, in ascending token order.
// ---------------------------------------------------------------------------------------------
// One CTA per document.  A bitmap over the document's tokens collects the winners of every (query, query token);
// the number of winners below a token is a prefix count per bitmap word plus a popcount inside the word.  Outputs:
// the winner positions inside the compact document (for the backward kernels), the row of the hidden states behind
// every compact slot (for the gather), the compact length, and the bitmap with its prefix counts (for the scatter).
__global__ void __launch_bounds__(256) hidden_winners_kernel(const int* __restrict__ argmax, int n_q, int n_d, int lq, int ld, int slots,
                                                             int words, int* __restrict__ compact_argmax, long long* __restrict__ rows,
                                                             int* __restrict__ counts, unsigned* __restrict__ bitmap,
                                                             int* __restrict__ prefix, int* status) {
  extern __shared__ unsigned hw_smem[];
  unsigned* bm = hw_smem;
  int* pre = reinterpret_cast<int*>(hw_smem + words);
  __shared__ int warp_sum_s[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = blockIdx.x;
  for (int w = tid; w < words; w += 256) bm[w] = 0u;
  __syncthreads();
  const int n_ent = n_q * lq;
  for (int e = tid; e < n_ent; e += 256) {
    const int i = e / lq, s = e - i * lq;
    const int t = argmax[((long long)i * n_d + j) * lq + s];
    if (t >= 0) {
      if (t < ld) atomicOr(&bm[t >> 5], 1u << (t & 31));
      else if (status) atomicOr(status, LIK_DEV_INTERNAL);  // a saved winner outside its document: ignored
    }
  }
  __syncthreads();
  // exclusive prefix of the words' popcounts: every thread owns a run of consecutive words
  const int per = (words + 255) / 256;
  const int w0 = min(words, tid * per), w1 = min(words, w0 + per);
  int mine = 0;
  for (int w = w0; w < w1; ++w) mine += __popc(bm[w]);
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_sum_s[warp] = incl;
  __syncthreads();
  int before = incl - mine, total = 0;
  for (int w = 0; w < 8; ++w) {
    if (w < warp) before += warp_sum_s[w];
    total += warp_sum_s[w];
  }
  for (int w = w0; w < w1; ++w) {
    pre[w] = before;
    before += __popc(bm[w]);
  }
  __syncthreads();
  if (total > slots) {  // cannot happen for slots >= min(n_q * lq, ld); keep every store in bounds anyway
    if (tid == 0 && status) atomicOr(status, LIK_DEV_INTERNAL);
    total = slots;
  }
  if (tid == 0) counts[j] = total;
  for (int w = tid; w < words; w += 256) {
    const unsigned bits = bm[w];
    bitmap[(long long)j * words + w] = bits;
    prefix[(long long)j * words + w] = pre[w];
    int pos = pre[w];
    for (unsigned b = bits; b; b &= b - 1) {
      if (pos < slots) rows[(long long)j * slots + pos] = (long long)j * ld + w * 32 + (__ffs(b) - 1);
      ++pos;
    }
  }
  for (int p = total + tid; p < slots; p += 256) rows[(long long)j * slots + p] = (long long)j * ld;  // unused slots: any row of the document
  for (int e = tid; e < n_ent; e += 256) {
    const int i = e / lq, s = e - i * lq;
    const long long o = ((long long)i * n_d + j) * lq + s;
    const int t = argmax[o];
    int c = -1;
    if (t >= 0 && t < ld) {
      c = pre[t >> 5] + __popc(bm[t >> 5] & ((1u << (t & 31)) - 1u));
      if (c >= slots) c = -1;
    }
    compact_argmax[o] = c;
  }
}

// grad_h, every row written once: the compact row of a winning token, zeros for all the others.  One warp per
// bitmap word (32 tokens); rows are copied in 16-byte pieces.
__global__ void __launch_bounds__(256) hidden_scatter_kernel(const uint4* __restrict__ compact, int row_vecs, int n_d, int ld, int slots,
                                                             int words, const unsigned* __restrict__ bitmap, const int* __restrict__ prefix,
                                                             uint4* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long n_words = (long long)n_d * words;
  for (long long gw = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); gw < n_words; gw += (long long)gridDim.x * 8) {
    const int j = (int)(gw / words), w = (int)(gw - (long long)j * words);
    const unsigned bits = bitmap[gw];
    const int base = prefix[gw];
    const int n_tok = min(32, ld - w * 32);
    for (int b = 0; b < n_tok; ++b) {
      uint4* dst = out + ((long long)j * ld + w * 32 + b) * row_vecs;
      if ((bits >> b) & 1u) {
        const int pos = base + __popc(bits & ((1u << b) - 1u));
        const uint4* src = compact + ((long long)j * slots + min(pos, slots - 1)) * row_vecs;
        for (int v = lane; v < row_vecs; v += 32) dst[v] = src[v];
      } else {
        for (int v = lane; v < row_vecs; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
}

struct HeadPlan {
  int n_k, n_s2, stages, mt, q_per_tile, q_last_rows, grid;
  size_t smem_bytes;
  size_t lens_off, total_ws;
};

bool head_plan(const lik_hidden_fwd_args& a, HeadPlan& pl) {
  if (a.dtype != LIK_BF16 && a.dtype != LIK_F16) return false;
  if (a.d_out < 32 || a.d_out > 128 || a.d_out % 32 != 0) return false;
  if (a.d_model < 8 || (a.d_model * 2) % 16 != 0) return false;
  if (a.q.cu || a.q.lens || a.q.mask || a.q.scale || a.q.scale_scalar != 1.0f) return false;
  if (a.h.cu || a.h.scale || a.h.scale_scalar != 1.0f) return false;
  if (a.q.n_seq <= 0 || a.h.n_seq <= 0 || a.q.max_len <= 0 || a.h.max_len <= 0 || a.q.max_len > TILE_M) return false;
  if (a.q.seq_stride != a.q.max_len) return false;  // query tokens are consecutive rows
  pl.q_per_tile = TILE_M / a.q.max_len;
  const long long n_tiles = ceil_div(a.q.n_seq, pl.q_per_tile);
  if (n_tiles > 2) return false;
  pl.mt = (int)n_tiles;
  if ((a.q.row_stride * 2) % 16 != 0 || (a.h.row_stride * 2) % 16 != 0 || (a.w_stride * 2) % 16 != 0) return false;
  if (((uintptr_t)a.q.data & 15) || ((uintptr_t)a.h.data & 15) || ((uintptr_t)a.w & 15)) return false;
  if (a.h.n_rows >= (1ll << 31) || a.q.n_rows >= (1ll << 31)) return false;
  if (a.argmax && a.argmax_stride < a.q.max_len) return false;
  pl.n_k = (a.d_model * 2 + HD_SLAB_ROW - 1) / HD_SLAB_ROW;
  pl.n_s2 = (a.d_out * 2 + HD_SLAB_ROW - 1) / HD_SLAB_ROW;
  const int last_queries = a.q.n_seq - (pl.mt - 1) * pl.q_per_tile;
  pl.q_last_rows = (last_queries * a.q.max_len + 7) & ~7;
  const size_t fixed = (size_t)pl.mt * pl.n_s2 * HD_SLAB + (size_t)pl.n_s2 * pl.q_last_rows * HD_SLAB_ROW + sizeof(HeadCtl) + 1024;
  const size_t budget = 227 * 1024;
  int st = (int)((budget - fixed) / (2 * HD_SLAB));
  pl.stages = st > HD_MAX_STAGES ? HD_MAX_STAGES : st;
  if (pl.stages < 2) return false;
  pl.smem_bytes = fixed + (size_t)pl.stages * 2 * HD_SLAB;
  pl.grid = a.h.n_seq < sm_count() ? a.h.n_seq : sm_count();
  pl.lens_off = 0;
  pl.total_ws = a.h.mask ? align_up((size_t)a.h.n_seq * sizeof(int), 256) : 0;
  return true;
}

}  // namespace

}  // namespace lik

extern "C" int lik_maxsim_hidden_fwd_supported(const lik_hidden_fwd_args* a) {
  using namespace lik;
  if (!a || !lik_device_supported() || !tmap_available()) return 0;
  HeadPlan pl{};
  return head_plan(*a, pl) ? 1 : 0;
}

extern "C" size_t lik_maxsim_hidden_fwd_workspace(const lik_hidden_fwd_args* a) {
  using namespace lik;
  HeadPlan pl{};
  if (!a || !head_plan(*a, pl)) return 0;
  return pl.total_ws;
}

extern "C" int lik_maxsim_hidden_fwd(const lik_hidden_fwd_args* args, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(args != nullptr, "args is NULL");
  const lik_hidden_fwd_args& a = *args;
  cudaStream_t st = (cudaStream_t)stream;
  LIK_REQUIRE(a.q.data && a.h.data && a.w && a.scores, "q, h, w and scores must not be NULL");
  LIK_REQUIRE(a.q.n_seq >= 0 && a.h.n_seq >= 0, "negative size");
  LIK_REQUIRE(a.normalize == LIK_NORM_NONE || a.normalize == LIK_NORM_D, "normalize must be LIK_NORM_NONE or LIK_NORM_D");
  LIK_REQUIRE((long long)(a.q.n_seq - 1) * a.q.seq_stride + a.q.max_len <= a.q.n_rows, "q: padded sequences exceed n_rows");
  LIK_REQUIRE((long long)(a.h.n_seq - 1) * a.h.seq_stride + a.h.max_len <= a.h.n_rows, "h: padded sequences exceed n_rows");
  HeadPlan pl{};
  if (!lik_device_supported() || !tmap_available() || !head_plan(a, pl)) {
    set_error("lik_maxsim_hidden_fwd: this problem is not taken by the chained kernel (see lik_maxsim_hidden_fwd_supported)");
    return LIK_ERR_UNSUPPORTED;
  }
  if (a.workspace_bytes < pl.total_ws || (pl.total_ws && !a.workspace)) {
    set_error("lik_maxsim_hidden_fwd: workspace too small");
    return LIK_ERR_WORKSPACE;
  }
  CUtensorMap q_map, h_map, w_map;
  int rc = make_tmap_rows(&q_map, a.q.data, a.dtype, a.d_out, a.q.n_rows, a.q.row_stride, 8);
  if (rc) return rc;
  rc = make_tmap_rows(&h_map, a.h.data, a.dtype, a.d_model, a.h.n_rows, a.h.row_stride, HD_TOK);
  if (rc) return rc;
  rc = make_tmap_rows(&w_map, a.w, a.dtype, a.d_model, a.d_out, a.w_stride, a.d_out);
  if (rc) return rc;

  HeadParams P{};
  P.n_d = a.h.n_seq;
  P.ld = a.h.max_len;
  P.seq_stride = a.h.seq_stride;
  P.lens = a.h.lens;
  P.lens_flagged = 0;
  P.mask = a.h.mask;
  if (a.h.mask) {
    int* eff = (int*)a.workspace;
    rc = launch_mask_lens(a.h.mask, a.h.lens, a.h.n_seq, a.h.max_len, a.h.seq_stride, eff, st);
    if (rc) return rc;
    P.lens = eff;
    P.lens_flagged = 1;
  }
  P.d_model = a.d_model;
  P.d_out = a.d_out;
  P.n_k = pl.n_k;
  P.n_s2 = pl.n_s2;
  P.stages = pl.stages;
  P.mt = pl.mt;
  P.n_q = a.q.n_seq;
  P.lq = a.q.max_len;
  P.q_per_tile = pl.q_per_tile;
  P.q_last_rows = pl.q_last_rows;
  P.f16 = a.dtype == LIK_F16;
  P.normalize = a.normalize == LIK_NORM_D;
  P.bias = a.bias;
  P.scores = a.scores;
  P.argmax = a.argmax;
  P.argmax_stride = a.argmax_stride;
  P.status = a.status;
  // positions of the saved winners that no accumulator row covers
  if (a.argmax && a.argmax_stride > a.q.max_len)
    LIK_CUDA_OK(cudaMemsetAsync(a.argmax, 0xFF, (size_t)a.q.n_seq * a.h.n_seq * a.argmax_stride * sizeof(int), st));
  static size_t allowed[2][64] = {{0}};
  int dev = 0;
  LIK_CUDA_OK(cudaGetDevice(&dev));
  const int v = a.argmax ? 1 : 0;
  if (dev < 0 || dev >= 64 || allowed[v][dev] < pl.smem_bytes) {
    if (v) LIK_CUDA_OK(cudaFuncSetAttribute(head_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem_bytes));
    else LIK_CUDA_OK(cudaFuncSetAttribute(head_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem_bytes));
    if (dev >= 0 && dev < 64) allowed[v][dev] = pl.smem_bytes;
  }
  if (v) head_tc_kernel<true><<<pl.grid, HD_THREADS, pl.smem_bytes, st>>>(q_map, h_map, w_map, P), ::lik::count_launch();
  else head_tc_kernel<false><<<pl.grid, HD_THREADS, pl.smem_bytes, st>>>(q_map, h_map, w_map, P), ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

extern "C" int lik_hidden_winners(const int32_t* argmax, int32_t n_q, int32_t n_d, int32_t lq, int32_t ld, int32_t slots,
                                  int32_t* compact_argmax, int64_t* rows, int32_t* counts, uint32_t* bitmap, int32_t* prefix,
                                  int32_t* status, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(n_q >= 0 && n_d >= 0 && lq > 0 && ld > 0 && slots > 0, "sizes must be positive");
  LIK_REQUIRE((long long)n_q * lq < (1ll << 31) && (long long)n_d * ld < (1ll << 40), "sizes out of range");
  if (n_d == 0) return LIK_OK;
  LIK_REQUIRE(argmax && compact_argmax && rows && counts && bitmap && prefix, "NULL pointer");
  const int words = (ld + 31) / 32;
  const size_t smem = (size_t)words * 8;
  LIK_REQUIRE(smem <= 48 * 1024, "documents longer than 196608 tokens are not supported");
  hidden_winners_kernel<<<n_d, 256, smem, (cudaStream_t)stream>>>(argmax, n_q, n_d, lq, ld, slots, words, compact_argmax,
                                                                   (long long*)rows, counts, bitmap, prefix, status),
      ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}

extern "C" int lik_hidden_scatter_rows(const void* compact_rows, int64_t row_bytes, int32_t n_d, int32_t ld, int32_t slots,
                                       const uint32_t* bitmap, const int32_t* prefix, void* grad_h, lik_stream_t stream) {
  using namespace lik;
  LIK_REQUIRE(n_d >= 0 && ld > 0 && slots > 0 && row_bytes > 0, "sizes must be positive");
  if (n_d == 0) return LIK_OK;
  LIK_REQUIRE(compact_rows && bitmap && prefix && grad_h, "NULL pointer");
  LIK_REQUIRE(row_bytes % 16 == 0 && row_bytes / 16 < (1ll << 31) && ((uintptr_t)compact_rows & 15) == 0 && ((uintptr_t)grad_h & 15) == 0,
              "rows must be 16-byte aligned and a multiple of 16 bytes long");
  const int words = (ld + 31) / 32;
  const long long n_words = (long long)n_d * words;
  long long grid = ceil_div(n_words, 8);
  const long long cap = (long long)sm_count() * 8;
  if (grid > cap) grid = cap;
  hidden_scatter_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)compact_rows, (int)(row_bytes / 16), n_d, ld, slots,
                                                                            words, bitmap, prefix, (uint4*)grad_h),
      ::lik::count_launch();
  LIK_CUDA_OK(cudaGetLastError());
  return LIK_OK;
}
