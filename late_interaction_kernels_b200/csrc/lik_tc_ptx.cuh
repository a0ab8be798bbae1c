// PTX wrappers and epilogue arithmetic shared by the tcgen05 kernels (sm_100a): mbarriers, TMA loads, tensor
// memory, the MMA issue, shared-memory and instruction descriptors, and the running (max, argmax) fold over
// accumulator columns.
#pragma once

#include <cuda.h>

#include "lik_common.cuh"

namespace lik {
namespace {

constexpr int TILE_M = 128;                   // accumulator rows (TMEM lanes) of every MMA
constexpr uint32_t TRY_WAIT_HINT_NS = 20000;  // how long one try_wait may keep the thread suspended

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(TRY_WAIT_HINT_NS)
      : "memory");
  return ok != 0;
}
// generic-proxy writes to shared memory become visible to the async proxy (the tensor core's operand reads)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// untiled bulk copy global -> shared (16-byte aligned on both sides, a multiple of 16 bytes), completing on an mbarrier
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Both operand descriptors share their upper word (stride, version, swizzle mode); only the 14-bit
// start-address field in the lower word moves, so the issuer carries 32-bit values and the 64-bit
// descriptors are put together next to the instruction.
template <bool FP8>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                       uint32_t accumulate) {
  if (FP8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 lanes x 32 consecutive fp32 columns of TMEM -> 32 registers per thread.  The load is
// asynchronous: the registers may only be read after tmem_ld_wait(), which takes them as in/out
// operands so that no use can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, float (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]), "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(float (&v)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]), "+f"(v[8]), "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15]), "+f"(v[16]), "+f"(v[17]), "+f"(v[18]), "+f"(v[19]), "+f"(v[20]), "+f"(v[21]), "+f"(v[22]), "+f"(v[23]), "+f"(v[24]), "+f"(v[25]), "+f"(v[26]), "+f"(v[27]), "+f"(v[28]), "+f"(v[29]), "+f"(v[30]), "+f"(v[31]) : : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// maximum of 32 values as a shallow tree of independent 3-input max operations
__device__ __forceinline__ float max32(const float (&v)[32]) {
  float a0 = max3(v[0], v[1], v[2]), a1 = max3(v[3], v[4], v[5]), a2 = max3(v[6], v[7], v[8]);
  float a3 = max3(v[9], v[10], v[11]), a4 = max3(v[12], v[13], v[14]), a5 = max3(v[15], v[16], v[17]);
  float a6 = max3(v[18], v[19], v[20]), a7 = max3(v[21], v[22], v[23]), a8 = max3(v[24], v[25], v[26]);
  float a9 = max3(v[27], v[28], v[29]);
  float b0 = max3(a0, a1, a2), b1 = max3(a3, a4, a5), b2 = max3(a6, a7, a8), b3 = max3(a9, v[30], v[31]);
  return fmaxf(max3(b0, b1, b2), b3);
}

__device__ __forceinline__ float min3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Position (0..31) of the first element of v that equals cmax, where cmax is the maximum of v.
// Compare / select / logic instructions share one half-rate pipe, which a per-element equality scan
// would saturate, so the scan is arithmetic instead: key_i = (cmax - v_i) * 2^154 + i is exactly i
// for a match and at least 32 (or +inf) otherwise, because two different floats never differ by
// less than 2^-149; the scaling is split in two exact powers of two that cannot overflow for
// |cmax| < 2^64.  The minimum key is the answer.
__device__ __forceinline__ int first_match32(const float (&v)[32], float cmax) {
  const float c2 = cmax * 0x1p64f;
  float k[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) k[i] = fmaf(fmaf(v[i], -0x1p64f, c2), 0x1p90f, (float)i);
  float a0 = min3(k[0], k[1], k[2]), a1 = min3(k[3], k[4], k[5]), a2 = min3(k[6], k[7], k[8]);
  float a3 = min3(k[9], k[10], k[11]), a4 = min3(k[12], k[13], k[14]), a5 = min3(k[15], k[16], k[17]);
  float a6 = min3(k[18], k[19], k[20]), a7 = min3(k[21], k[22], k[23]), a8 = min3(k[24], k[25], k[26]);
  float a9 = min3(k[27], k[28], k[29]);
  float b0 = min3(a0, a1, a2), b1 = min3(a3, a4, a5), b2 = min3(a6, a7, a8), b3 = min3(a9, k[30], k[31]);
  return (int)fminf(min3(b0, b1, b2), b3);
}

// Fold the maximum of one 32-column chunk into the running (max, argmax) of a row.  The column scan
// only runs when the chunk beats the running maximum (strict: an equal value in a later chunk never
// displaces an earlier winner) and returns the lowest matching column.
// LAZY: the scan is skipped when no row of the warp has a new maximum in this chunk - worth its branch only deep
// into a long document, where most chunks bring none.
template <bool ARGMAX, bool LAZY = false>
__device__ __forceinline__ void fold32(const float (&v)[32], int col0, float& run_m, int& run_i) {
  const float cmax = max32(v);
  if (ARGMAX) {
    // (unconditional by default: with 32 rows per warp some row nearly always has a new maximum in a document of a few
    // chunks, and a branch costs more than the scan)
    const bool better = cmax > run_m;
    if (!LAZY || __any_sync(0xffffffffu, better)) {
      const int p = first_match32(v, cmax);
      run_i = better ? col0 + p : run_i;
    }
    run_m = better ? cmax : run_m;
  } else {
    run_m = fmaxf(run_m, cmax);
  }
}
// v[i] *= scale[i]: per-column multiplier staged in shared memory
__device__ __forceinline__ void scale32(float (&v)[32], const float* scale) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 sc = *reinterpret_cast<const float4*>(scale + i);
    v[i + 0] *= sc.x;
    v[i + 1] *= sc.y;
    v[i + 2] *= sc.z;
    v[i + 3] *= sc.w;
  }
}
// v[i] = v[i] * scale[i] for the first `lim` columns, -inf for the others (whatever scale holds there)
__device__ __forceinline__ void scale32_first(float (&v)[32], const float* scale, int lim) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 sc = *reinterpret_cast<const float4*>(scale + i);
    v[i + 0] = i + 0 < lim ? v[i + 0] * sc.x : -INFINITY;
    v[i + 1] = i + 1 < lim ? v[i + 1] * sc.y : -INFINITY;
    v[i + 2] = i + 2 < lim ? v[i + 2] * sc.z : -INFINITY;
    v[i + 3] = i + 3 < lim ? v[i + 3] * sc.w : -INFINITY;
  }
}
// v[i] = v[i] * scale[i] + bias[i]: per-column multiplier and additive mask staged in shared memory
__device__ __forceinline__ void affine32(float (&v)[32], const float* scale, const float* bias) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 sc = *reinterpret_cast<const float4*>(scale + i);
    const float4 bi = *reinterpret_cast<const float4*>(bias + i);
    v[i + 0] = fmaf(v[i + 0], sc.x, bi.x);
    v[i + 1] = fmaf(v[i + 1], sc.y, bi.y);
    v[i + 2] = fmaf(v[i + 2], sc.z, bi.z);
    v[i + 3] = fmaf(v[i + 3], sc.w, bi.w);
  }
}

// Partial chunk of `lim` (1..31) columns: loaded as pieces of 16, 8, 4, 2 and 1 columns according to
// the bits of lim into v[0..15], v[16..23], v[24..27], v[28..29], v[30]; pieces that are absent keep
// the value the caller put there.  Piece n starts at column (lim with the bits below 2n cleared).
__device__ __forceinline__ void tmem_ld_tail(uint32_t taddr, int lim, float (&v)[32]) {
  if (lim & 16) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];" : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]), "+f"(v[8]), "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15]) : "r"(taddr + (uint32_t)(lim & 0)) : "memory");
  }
  if (lim & 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "+f"(v[16]), "+f"(v[17]), "+f"(v[18]), "+f"(v[19]), "+f"(v[20]), "+f"(v[21]), "+f"(v[22]), "+f"(v[23]) : "r"(taddr + (uint32_t)(lim & 16)) : "memory");
  }
  if (lim & 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "+f"(v[24]), "+f"(v[25]), "+f"(v[26]), "+f"(v[27]) : "r"(taddr + (uint32_t)(lim & 24)) : "memory");
  }
  if (lim & 2) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "+f"(v[28]), "+f"(v[29]) : "r"(taddr + (uint32_t)(lim & 28)) : "memory");
  }
  if (lim & 1) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "+f"(v[30]) : "r"(taddr + (uint32_t)(lim & 30)) : "memory");
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]), "+f"(v[8]), "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15]), "+f"(v[16]), "+f"(v[17]), "+f"(v[18]), "+f"(v[19]), "+f"(v[20]), "+f"(v[21]), "+f"(v[22]), "+f"(v[23]), "+f"(v[24]), "+f"(v[25]), "+f"(v[26]), "+f"(v[27]), "+f"(v[28]), "+f"(v[29]), "+f"(v[30]) : : "memory");
}
// Column (relative to the chunk) of the first element of a tmem_ld_tail() array that equals cmax.
__device__ __forceinline__ int tail_first_match(const float (&v)[32], float cmax, int lim) {
  const int p = first_match32(v, cmax);  // array position; pieces are stored in ascending column order
  if (p < 16) return p;
  if (p < 24) return (lim & 16) + (p - 16);
  if (p < 28) return (lim & 24) + (p - 24);
  if (p < 30) return (lim & 28) + (p - 28);
  return lim & 30;
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);  // start address
  d |= (uint64_t)1 << 16;                   // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
  return d;
}
// Instruction descriptor: fp32 accumulate, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc(int ab_format, int n) {
  return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(TILE_M >> 4) << 24);
}

}  // namespace
}  // namespace lik
