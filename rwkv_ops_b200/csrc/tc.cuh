// Blackwell (sm_100a) building blocks for the chunked RWKV7 kernels: shared-memory tile layout,
// UMMA descriptors, tcgen05 MMA / TMEM load-store, mbarriers with bounded waits, TMA and bulk copies.
//
// Tile convention.  Every matrix operand is a 64 x 64 bf16 tile stored row-major with 128-byte rows
// and the 128-byte swizzle (16-byte chunk index XOR (row & 7)); a tile is 8 KB and 1024-byte aligned.
// The same bytes serve as
//   * a K-major operand whose M/N index is the tile row and whose contraction index is the tile column, or
//   * an MN-major operand whose M/N index is the tile column and whose contraction index is the tile row,
// so X, X^T products need no transposes: only the descriptor changes.  Two tiles that are adjacent in
// shared memory form a 128-row K-major operand.
//
// TMEM accumulators.  An M=128 MMA puts row r on lane r.  An M=64 MMA puts row r on lane
// (r & 15) + 32 * (r >> 4), i.e. on the lower 16 lanes of each warp's 32-lane window; a second M=64
// accumulator at lane offset 16 fills the upper halves, so one 32x32b TMEM load hands a row of the
// first accumulator to threads 0-15 and a row of the second to threads 16-31 of every warp.
//
// Every wait is bounded: after WAIT_LIMIT polls the waiter records a status word and the kernel winds
// down (no trap, no endless spin).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rwkvb200 {
namespace tc {

constexpr int TILE = 64;
constexpr int TILE_BYTES = TILE * TILE * 2;     // 8192
constexpr uint32_t WAIT_LIMIT = 1u << 22;       // polls before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// byte offset of element (row, col) inside a swizzled 64x64 bf16 tile
__device__ __forceinline__ uint32_t tile_off(int row, int col) {
  return (uint32_t)(row * 128 + ((((col >> 3) ^ row) & 7) << 4) + ((col & 7) << 1));
}
// byte offset of the 16-byte chunk (8 elements starting at col8*8) of a row
__device__ __forceinline__ uint32_t tile_chunk_off(int row, int chunk) {
  return (uint32_t)(row * 128 + (((chunk ^ row) & 7) << 4));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; returns false (and records `code`) if the phase never completed.
// `status` is the library's device status word (0 = fine), see device_status_ptr().
// The result is made uniform over the threads of the warp that wait together, so that the
// warp-collective TMEM instructions that follow are never executed by part of a warp.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          uint32_t limit = WAIT_LIMIT) {
  bool done = false;
  for (uint32_t i = 0; i < limit && !done; ++i) done = mbar_try_wait(bar, parity);
  if (!done) atomicCAS(status, 0, code);
  return __all_sync(__activemask(), done) != 0;
}

// ---------------------------------------------------------------------------------------------
// proxies and fences
// ---------------------------------------------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (MMA operand reads, bulk stores)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// TMA (tiled, 4-D) and 1-D bulk copies.  No cluster multicast anywhere.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(void* dst_smem, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// Tiled store of one swizzled tile; rows past the end of the tensor are clipped by the hardware.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src_smem,
                                             int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src_smem)),
                 "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(src_gmem)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// ask for `bytes` (a multiple of 16) at src_gmem / for one box of a tensor map to be brought into L2
__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(src_gmem)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* tmap, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(dst_gmem)), "r"(smem_u32(src_smem)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed bulk stores have finished READING their shared-memory source
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the most recently committed group of bulk stores have finished reading shared memory
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// TMEM allocation (one warp executes these)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a swizzle-128B bf16 operand starting at `addr` (shared address).
//   bits [0,14) start address >> 4; [16,30) leading byte offset >> 4; [32,46) stride byte offset >> 4;
//   [46,48) version = 1; [61,64) layout type = 2 (128-byte swizzle).
// K-major : rows 128 B apart, 8-row groups SBO = 1024 B apart; a K=16 step advances the start by 32 B.
// MN-major: 64 M/N elements per 128-byte row; 8-row contraction groups SBO = 1024 B apart; the next
//           64 M/N elements (a second tile) are LBO = 8192 B further; a K=16 step advances by 2048 B.
// The descriptor is built from its two 32-bit halves (umma_desc_lo, UMMA_DESC_HI below).  For an MN-major operand
// `lbo` is the byte distance to the tile holding M/N elements 64..127 of a 128-wide operand.

// Instruction descriptor, kind::f16 with bf16 inputs and fp32 accumulation.
//   [4,6) D format 1 = f32; [7,10) A format 1 = bf16; [10,13) B format 1 = bf16;
//   bit 15 A major (1 = MN); bit 16 B major (1 = MN); [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread, from the two halves of each descriptor.  The issuing
// thread runs alone in its warp, one dependent instruction every few cycles, so what it computes per MMA is
// part of what a group of MMAs costs: here two additions
// (the lower words, by the caller) and the instruction itself; the upper word is the same for every operand
// (SBO 1024 B, version 1, 128-byte swizzle), and a literal accumulate flag folds into the predicate.
constexpr uint32_t UMMA_DESC_HI = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr & 0x3FFFF) >> 4) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
}
template <bool ACC>
__device__ __forceinline__ void umma_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  if constexpr (ACC) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(UMMA_DESC_HI) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(UMMA_DESC_HI) : "memory");
  }
}
// Make `bar` complete (one arrival) when all MMAs issued so far by this thread have finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// A product with a contraction length of 16*KSTEPS as K=16 steps.  A_MN / B_MN select the operand
// majors.  A 128-row K-major operand is two tiles adjacent in shared memory; a 128-wide MN-major operand
// is two tiles `a_lbo` / `b_lbo` bytes apart; an MN-major operand with KSTEPS = 8 continues into the
// tile that follows it (contraction rows 64..127).
template <int M, int N, int A_MN, int B_MN, int KSTEPS = 4>
__device__ __forceinline__ void umma_tile(uint32_t tmem_d, uint32_t a_addr, uint32_t b_addr, bool accumulate,
                                          uint32_t a_lbo = TILE_BYTES, uint32_t b_lbo = TILE_BYTES) {
  static_assert(KSTEPS == 4 || (A_MN && B_MN), "a K-major operand holds 64 contraction elements");
  constexpr uint32_t id = idesc_bf16(M, N, A_MN, B_MN);
  // lower descriptor words of step 0; a K=16 step advances the start address by 32 B (K-major) or 2048 B
  // (MN-major), i.e. the word by 2 or 128 (no carry out of the 14-bit field: shared addresses stay below 256 KB)
  const uint32_t a0 = umma_desc_lo(a_addr, A_MN ? a_lbo : 16u), b0 = umma_desc_lo(b_addr, B_MN ? b_lbo : 16u);
  constexpr uint32_t a_step = A_MN ? 128u : 2u, b_step = B_MN ? 128u : 2u;
  if (accumulate) umma_lo<true>(tmem_d, a0, b0, id); else umma_lo<false>(tmem_d, a0, b0, id);
#pragma unroll
  for (int ks = 1; ks < KSTEPS; ++ks) umma_lo<true>(tmem_d, a0 + a_step * ks, b0 + b_step * ks, id);
}

// ---------------------------------------------------------------------------------------------
// TMEM <-> registers: each thread of a warp moves 32 consecutive columns of its own lane
// (lane = 32 * (warp & 3) + laneid; the address carries the warp's lane base in bits [16,32)).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16 consecutive columns of the thread's lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// N = 16 or 32 consecutive columns
template <int N> __device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[N]);
template <> __device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address of (lane, column) relative to an allocation base
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// 2^x in one instruction.  The chunked kernels keep every decay sum in units of log 2 (g log2(e)), so that a
// scale factor e^{sum} costs this one instruction and no multiplication.
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------------------------
// small helpers for moving rows between registers and swizzled tiles
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// write 32 consecutive fp32 values (columns col0 .. col0+31, col0 a multiple of 8) of `row` as bf16
__device__ __forceinline__ void tile_store_row32(unsigned char* tile, int row, int col0, const float* x) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 u;
    u.x = pack_bf16(x[8 * c + 0], x[8 * c + 1]);
    u.y = pack_bf16(x[8 * c + 2], x[8 * c + 3]);
    u.z = pack_bf16(x[8 * c + 4], x[8 * c + 5]);
    u.w = pack_bf16(x[8 * c + 6], x[8 * c + 7]);
    *reinterpret_cast<uint4*>(tile + tile_chunk_off(row, (col0 >> 3) + c)) = u;
  }
}
// read 32 consecutive bf16 values of `row` as fp32
__device__ __forceinline__ void tile_load_row32(const unsigned char* tile, int row, int col0, float* x) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint4 u = *reinterpret_cast<const uint4*>(tile + tile_chunk_off(row, (col0 >> 3) + c));
    x[8 * c + 0] = bf16_lo(u.x); x[8 * c + 1] = bf16_hi(u.x);
    x[8 * c + 2] = bf16_lo(u.y); x[8 * c + 3] = bf16_hi(u.y);
    x[8 * c + 4] = bf16_lo(u.z); x[8 * c + 5] = bf16_hi(u.z);
    x[8 * c + 6] = bf16_lo(u.w); x[8 * c + 7] = bf16_hi(u.w);
  }
}

// the same for N = 16 or 32 consecutive values (col0 a multiple of 8)
template <int N>
__device__ __forceinline__ void tile_store_row(unsigned char* tile, int row, int col0, const float* x) {
#pragma unroll
  for (int c = 0; c < N / 8; ++c) {
    uint4 u;
    u.x = pack_bf16(x[8 * c + 0], x[8 * c + 1]);
    u.y = pack_bf16(x[8 * c + 2], x[8 * c + 3]);
    u.z = pack_bf16(x[8 * c + 4], x[8 * c + 5]);
    u.w = pack_bf16(x[8 * c + 6], x[8 * c + 7]);
    *reinterpret_cast<uint4*>(tile + tile_chunk_off(row, (col0 >> 3) + c)) = u;
  }
}
template <int N>
__device__ __forceinline__ void tile_load_row(const unsigned char* tile, int row, int col0, float* x) {
#pragma unroll
  for (int c = 0; c < N / 8; ++c) {
    const uint4 u = *reinterpret_cast<const uint4*>(tile + tile_chunk_off(row, (col0 >> 3) + c));
    x[8 * c + 0] = bf16_lo(u.x); x[8 * c + 1] = bf16_hi(u.x);
    x[8 * c + 2] = bf16_lo(u.y); x[8 * c + 3] = bf16_hi(u.y);
    x[8 * c + 4] = bf16_lo(u.z); x[8 * c + 5] = bf16_hi(u.z);
    x[8 * c + 6] = bf16_lo(u.w); x[8 * c + 7] = bf16_hi(u.w);
  }
}

}  // namespace tc

// Host side: encode a tensor map for a [B,T,H,64] / [B,H,T,64] 16-bit token tensor so that
// coordinates (0, t0, h, b) with box (64, 64, 1, 1) land one swizzled 64-token tile.
int make_token_tensor_map(CUtensorMap* out, const void* base, int B, int T, int H, int head_first);

// Device address (on the current device) of the status word that kernels set when a bounded wait
// ran out; nullptr if the lookup failed.  Read and cleared by rwkvb200_device_status().
int* device_status_ptr();

int make_row_tensor_map(CUtensorMap* out, const void* base, int B, int T, int H, int elem_bytes);

// Device buffer (>= 64 long long) that kernels fill with clock64() stamps at their phase boundaries (one
// designated CTA).  Only the developer build (-DRWKVB200_DEVTOOLS) can install one and only its kernels
// contain the stamping code; in the shipped library this is always nullptr.
long long* debug_stamp_buffer();

}  // namespace rwkvb200
