// Chunked RWKV7 backward on tcgen05 (bf16 token tensors).  Equations in rwkv7_chunked.cuh.
//
// Launch sequence (all on the caller's stream, tiles exchanged through the workspace):
//   1. forward intra kernel with keep_for_bwd (q~, k~, b~, a~, A_qk, A_ak, A_qb, Ainv, W, U, decay factors)
//   2. forward scan without output, keeping sa, h~0 and X of every chunk
//   3. r7c_bwd_pre_kernel    (parallel over chunks)   B2 = Ainv^T b~,  P2 = Ainv^T A_qb^T do
//   4. r7c_bwd_scan_kernel   (one CTA per (b,h), chunks in reverse)  dz, dh^ per chunk, d initial state
//   5. r7c_bwd_final_kernel  (parallel over chunks)   dq, dk, dv, da, db, dw
#include "rwkv7_chunked.cuh"

namespace rwkvb200 {
namespace r7c {

using namespace tc;
typedef __nv_bfloat16 bf16;

// decay sums are kept in units of log 2 (tc::ex2), as in the forward kernels; nothing is clamped
constexpr int NROW = 68;

__device__ __forceinline__ void store_row32_global(bf16* dst, const float* x) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 u;
    u.x = pack_bf16(x[j], x[j + 1]); u.y = pack_bf16(x[j + 2], x[j + 3]);
    u.z = pack_bf16(x[j + 4], x[j + 5]); u.w = pack_bf16(x[j + 6], x[j + 7]);
    *reinterpret_cast<uint4*>(dst + j) = u;
  }
}

// ---------------------------------------------------------------------------------------------
// 3. B2 = Ainv^T b~ and P2 = Ainv^T (A_qb^T do): persistent CTAs of 128 threads over the chunk-heads
// ---------------------------------------------------------------------------------------------
struct PreStage {
  unsigned char ainv[TILE_BYTES], bt[TILE_BYTES], aqb[TILE_BYTES], dout[TILE_BYTES];
};
struct PreSmem {
  PreStage st[2];             // the operand tiles of this chunk-head and of the next one
  unsigned char p1[TILE_BYTES], b2[TILE_BYTES], p2[TILE_BYTES];
  uint64_t bar_ld[2], bar_m1, bar_m2;
  uint32_t tmem_base;
};

// Two CTAs per SM walk over chunk-heads ch = blockIdx.x, blockIdx.x + gridDim.x, ...; the four operand tiles
// of the next chunk-head are requested before the current one is worked on, so that loads, the two dependent
// MMAs and the copies of the results overlap.
template <bool PACKED>
__global__ void __launch_bounds__(128)
r7c_bwd_pre_kernel(const __grid_constant__ CUtensorMap tmap_do, unsigned char* __restrict__ ws_tiles,
                   int tiles_per_chunk, SeqView sv, int H, int NT, int n_ch, int* status) {
  extern __shared__ unsigned char smem_raw[];
  PreSmem& sm = *reinterpret_cast<PreSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = 16 * warp + (lane & 15);
  const bool lo = lane < 16;

  if (tid == 0) {
    mbar_init(&sm.bar_ld[0], 1); mbar_init(&sm.bar_ld[1], 1); mbar_init(&sm.bar_m1, 1); mbar_init(&sm.bar_m2, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;

  auto empty = [&](const ChunkPos& p) {
    if constexpr (!PACKED) return false;
    return p.c * L >= sv.length<PACKED>(p.bi);      // a chunk slot past the end of a packed sequence
  };
  auto advance = [&](ChunkPos p) {
    do { chunk_step(p, gridDim.x, NT, H); } while (p.ch < n_ch && empty(p));
    return p;
  };
  auto issue_loads = [&](const ChunkPos& p, int s) {      // tid 0
    const unsigned char* tiles = ws_tiles + (size_t)p.ch * tiles_per_chunk * TILE_BYTES;
    PreStage& g = sm.st[s];
    mbar_expect_tx(&sm.bar_ld[s], 4 * TILE_BYTES);
    bulk_load(g.ainv, tiles + S_AINV * TILE_BYTES, TILE_BYTES, &sm.bar_ld[s]);
    bulk_load(g.bt, tiles + S_BT * TILE_BYTES, TILE_BYTES, &sm.bar_ld[s]);
    bulk_load(g.aqb, tiles + S_AQB * TILE_BYTES, TILE_BYTES, &sm.bar_ld[s]);
    tma_load_4d(g.dout, &tmap_do, &sm.bar_ld[s], 0, sv.first<PACKED>(p.bi) + p.c * L, p.hi, sv.row<PACKED>(p.bi));
  };
  ChunkPos cur = chunk_pos(blockIdx.x, NT, H);
  if (cur.ch < n_ch && empty(cur)) cur = advance(cur);
  if (cur.ch < n_ch && tid == 0) issue_loads(cur, 0);

  bool ok = true;
  int it = 0;
  for (ChunkPos nxt; cur.ch < n_ch && ok; cur = nxt, ++it) {
    const int s = it & 1;
    const uint32_t par = it & 1;
    PreStage& g = sm.st[s];
    unsigned char* tiles = ws_tiles + (size_t)cur.ch * tiles_per_chunk * TILE_BYTES;
    nxt = advance(cur);
    // the other stage was last read by the MMAs of the previous chunk-head, which have completed
    if (tid == 0 && nxt.ch < n_ch) issue_loads(nxt, s ^ 1);
    ok = mbar_wait(&sm.bar_ld[s], (it >> 1) & 1, status, 301);
    if (tid == 0 && ok) {
      bulk_wait_read();      // the copies of the previous B2 / P2 have left their tiles, which are rewritten below
      tc_fence_after();
      umma_tile<64, 64, 1, 1>(tmem_addr(tm, 0, 0), smem_u32(g.aqb), smem_u32(g.dout), false);   // A_qb^T do
      umma_tile<64, 64, 1, 1>(tmem_addr(tm, 16, 0), smem_u32(g.ainv), smem_u32(g.bt), false);   // Ainv^T b~
      umma_commit(&sm.bar_m1);
    }
    ok = mbar_wait(&sm.bar_m1, par, status, 302) && ok;
    tc_fence_after();
    if (ok) {
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, 32 * warp, 32 * part), r);
        tmem_ld_wait();
        float x[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]);
        tile_store_row32(lo ? sm.p1 : sm.b2, row, 32 * part, x);
      }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok) {
      tc_fence_after();
      umma_tile<64, 64, 1, 1>(tmem_addr(tm, 0, 64), smem_u32(g.ainv), smem_u32(sm.p1), false);   // Ainv^T P1
      umma_commit(&sm.bar_m2);
      bulk_store(tiles + S_B2 * TILE_BYTES, sm.b2, TILE_BYTES);
      bulk_commit();
    }
    ok = mbar_wait(&sm.bar_m2, par, status, 303) && ok;
    tc_fence_after();
    if (ok) {
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, 32 * warp, 64 + 32 * part), r);
        tmem_ld_wait();
        if (lo) {
          float x[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]);
          tile_store_row32(sm.p2, row, 32 * part, x);
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok) {
      bulk_store(tiles + S_P2 * TILE_BYTES, sm.p2, TILE_BYTES);
      bulk_commit();
    }
  }
  if (tid == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 128);
}

// ---------------------------------------------------------------------------------------------
// 4. reverse scan: grid = B*H, 256 threads (the two warps of a TMEM lane window take 32 columns each)
// ---------------------------------------------------------------------------------------------
struct BScanStage {
  unsigned char b2[TILE_BYTES], p2[TILE_BYTES];   // adjacent workspace slots: one bulk copy
  unsigned char at[TILE_BYTES], qt[TILE_BYTES], dout[TILE_BYTES];
};
struct BScanSmem {
  BScanStage st[2];
  unsigned char dhh[TILE_BYTES];    // dh^ as bf16, [k][v]
  unsigned char dz[TILE_BYTES];     // dz as bf16, [token][v]
  uint64_t bar_full[2], bar_m1, bar_m2;
  uint32_t tmem_base;
};

template <bool PACKED>
__global__ void __launch_bounds__(256, 2)
r7c_bwd_scan_kernel(const __grid_constant__ CUtensorMap tmap_do, unsigned char* __restrict__ ws_tiles,
                    const float* __restrict__ ws_aux, int tiles_per_chunk, const float* __restrict__ d_ht,
                    float* __restrict__ d_h0, SeqView sv, int H, int NT_slots, int spread, int* status) {
  extern __shared__ unsigned char smem_raw[];
  BScanSmem& sm = *reinterpret_cast<BScanSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int unit = blockIdx.x, bi = unit / H, hi = unit % H;
  const size_t ch0 = (size_t)unit * NT_slots;
  const int NT = (sv.length<PACKED>(bi) + L - 1) / L;      // chunks of this sequence
  const int tb = sv.first<PACKED>(bi), brow = sv.row<PACKED>(bi);
  const int wq = warp & 3, hsel = warp >> 2, c0 = 32 * hsel;
  const int row = 16 * wq + (lane & 15);
  const bool state_lane = lane < 16;
  // single-thread jobs side by side: thread 0 issues the MMAs (thread 96 one product of the first group, when
  // the CTA has the SM to itself), st_thread copies dh^ and dz out (and waits for
  // its own bulk-copy groups), ld_thread requests the operand tiles of the chunk after the next
  // (they share the SM with a second CTA when there are more sequences than SMs, and then stay with thread 0)
  const bool st_thread = tid == (spread ? 32 : 0), ld_thread = tid == (spread ? 64 : 0);

  if (tid == 0) {
    mbar_init(&sm.bar_full[0], 1); mbar_init(&sm.bar_full[1], 1);
    // with one CTA per SM the two products of the first MMA group have an issuing thread each
    mbar_init(&sm.bar_m1, spread ? 2 : 1); mbar_init(&sm.bar_m2, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 64);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;
  const uint32_t tm_w = tmem_addr(tm, 32 * wq, c0);

  auto issue_loads = [&](int n) {     // n-th chunk in reverse order
    const int c = NT - 1 - n;
    BScanStage& s = sm.st[n & 1];
    unsigned char* tiles = ws_tiles + (ch0 + c) * (size_t)tiles_per_chunk * TILE_BYTES;
    mbar_expect_tx(&sm.bar_full[n & 1], 5 * TILE_BYTES);
    bulk_load(s.b2, tiles + S_B2 * TILE_BYTES, 2 * TILE_BYTES, &sm.bar_full[n & 1]);
    bulk_load(s.at, tiles + S_AT * TILE_BYTES, TILE_BYTES, &sm.bar_full[n & 1]);
    bulk_load(s.qt, tiles + S_QT * TILE_BYTES, TILE_BYTES, &sm.bar_full[n & 1]);
    tma_load_4d(s.dout, &tmap_do, &sm.bar_full[n & 1], 0, tb + c * L, hi, brow);
  };
  if (tid == 0) {
    issue_loads(0);
    if (NT > 1) issue_loads(1);
  }

  // gradient of the state after the current chunk, row k of dh[k][v] = d_ht[v][k]
  float dh[32];        // columns c0 .. c0 + 31
  if (state_lane && d_ht) {
    const float* S = d_ht + (size_t)unit * 4096;
#pragma unroll
    for (int vv = 0; vv < 32; ++vv) dh[vv] = S[(c0 + vv) * 64 + row];
  } else {
#pragma unroll
    for (int vv = 0; vv < 32; ++vv) dh[vv] = 0.f;
  }

  // the two decay factors of a chunk are fetched one chunk ahead: they head the chain of a chunk
  float dc_next = 1.f, e0_next = 1.f;
  if (state_lane) {
    dc_next = ws_aux[(ch0 + NT - 1) * AUX_FLOATS + 64 + row];
    e0_next = ws_aux[(ch0 + NT - 1) * AUX_FLOATS + row];
  }
  bool ok = true;          // the same in every thread at the loop's head: the result of the last barrier
  bool tail_ok = true;     // this thread's wait at the end of the previous chunk
  for (int n = 0; n < NT && ok; ++n) {
    const int c = NT - 1 - n;
    BScanStage& s = sm.st[n & 1];
    unsigned char* tiles = ws_tiles + (ch0 + c) * (size_t)tiles_per_chunk * TILE_BYTES;
    const float dc = dc_next, e0 = e0_next;
    if (state_lane) {
#pragma unroll
      for (int vv = 0; vv < 32; ++vv) dh[vv] *= dc;      // dh^ = e^{glast-gref} dh_L
      tile_store_row32(sm.dhh, row, c0, dh);
      if (c > 0) {
        dc_next = ws_aux[(ch0 + c - 1) * AUX_FLOATS + 64 + row];
        e0_next = ws_aux[(ch0 + c - 1) * AUX_FLOATS + row];
      }
    }
    ok = tail_ok && mbar_wait(&sm.bar_full[n & 1], (n >> 1) & 1, status, 311);
    if (st_thread) bulk_wait_read();    // the copy of the previous chunk's dz has left its tile, rewritten below
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok) {
      tc_fence_after();
      umma_tile<64, 64, 0, 1>(tmem_addr(tm, 16, 0), smem_u32(s.b2), smem_u32(sm.dhh), false);   // B2 dh^
      if (!spread) umma_tile<64, 64, 1, 1>(tmem_addr(tm, 0, 0), smem_u32(s.qt), smem_u32(s.dout), false);    // q~^T do
      umma_commit(&sm.bar_m1);
    }
    if (spread && tid == 96 && ok) {
      tc_fence_after();
      umma_tile<64, 64, 1, 1>(tmem_addr(tm, 0, 0), smem_u32(s.qt), smem_u32(s.dout), false);    // q~^T do
      umma_commit(&sm.bar_m1);
    }
    if (st_thread && ok) {
      bulk_store(tiles + S_DHH * TILE_BYTES, sm.dhh, TILE_BYTES);
      bulk_commit();
    }
    ok = ok && mbar_wait(&sm.bar_m1, n & 1, status, 312);
    tc_fence_after();
    if (ok) {
      uint32_t r[32];
      tmem_ld32(tm_w, r);
      tmem_ld_wait();
      if (!state_lane) {      // dz = P2 + B2 dh^
        float x[32], p[32];
        tile_load_row32(s.p2, row, c0, p);
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]) + p[j];
        tile_store_row32(sm.dz, row, c0, x);
      }
    }
    if (st_thread) bulk_wait_read();    // the copy of dh^ has left its tile, rewritten at the top of the next chunk
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok) {
      tc_fence_after();
      umma_tile<64, 64, 1, 1>(tmem_addr(tm, 0, 0), smem_u32(s.at), smem_u32(sm.dz), true);      // += a~^T dz
      umma_commit(&sm.bar_m2);
    }
    if (st_thread && ok) {
      bulk_store(tiles + S_DZ * TILE_BYTES, sm.dz, TILE_BYTES);
      bulk_commit();
    }
    tail_ok = ok && mbar_wait(&sm.bar_m2, n & 1, status, 313);
    tc_fence_after();
    // this stage has been read: p2 by every thread before the last barrier, the rest by the two MMA groups
    if (ld_thread && tail_ok && n + 2 < NT) issue_loads(n + 2);
    if (tail_ok) {
      uint32_t r[32];
      tmem_ld32(tm_w, r);
      tmem_ld_wait();
      if (state_lane) {       // dh0 = e^{gref} (q~^T do + a~^T dz + dh^)
#pragma unroll
        for (int j = 0; j < 32; ++j) dh[j] = e0 * (__uint_as_float(r[j]) + dh[j]);
      }
    }
    // no barrier here: the next one (after dh^ of the next chunk is in its tile) orders these TMEM reads
    // before the MMAs that overwrite the accumulators
  }
  if (state_lane && d_h0 && ok && tail_ok) {
    float* S = d_h0 + (size_t)unit * 4096;
#pragma unroll
    for (int vv = 0; vv < 32; ++vv) S[(c0 + vv) * 64 + row] = dh[vv];
  }
  if (st_thread) bulk_wait_all();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 64);
}

// ---------------------------------------------------------------------------------------------
// 5. all token gradients of one chunk: persistent CTAs of 256 threads over the B*H*NT chunk-heads
// ---------------------------------------------------------------------------------------------
struct FinalSmem {
  // loaded per chunk, group A (free again once MMA group 2 has completed)
  unsigned char dout[TILE_BYTES], dz[TILE_BYTES];                 // [do; dz]
  unsigned char v[TILE_BYTES], sa[TILE_BYTES];                    // [v; sa]
  unsigned char aqk[TILE_BYTES], aak[TILE_BYTES];                 // adjacent workspace slots; aqk later stages dv
  unsigned char h0[TILE_BYTES], dhh[TILE_BYTES];
  // loaded per chunk, group B (read by the last epilogue, free after it)
  unsigned char qt[TILE_BYTES], at[TILE_BYTES], kt[TILE_BYTES], bt[TILE_BYTES];
  // computed
  unsigned char daqk[TILE_BYTES], daak[TILE_BYTES], daqb[TILE_BYTES], daab[TILE_BYTES];
  unsigned char red_pad[2048];    // the two fp32 scratch arrays that later overlay the dA tiles need 34 KB
  unsigned char dge[TILE_BYTES];  // da~ a~ as bf16
  unsigned char stage[5][TILE_BYTES];   // dq, dk, da, db, dw rows staged for TMA stores
  float gs[L * NROW];       // (gi - gref) log2(e): inclusive prefix of g inside the chunk, relative to the reference point
  float gg[L * NROW];       // g log2(e)
  float qtot[4][64];        // sums of g over the four quarters of the chunk
  float rqtot[4][64];       // sums of the decay-gradient terms over the four quarters
  float dgl[64];            // dglast
  uint64_t bar_lda, bar_ldb, bar_m1, bar_m2;
  uint32_t tmem_base;
};

// Persistent: one CTA per SM walks over chunk-heads ch = blockIdx.x, blockIdx.x + gridDim.x, ...; the
// tiles of the next chunk-head are requested as soon as the current one no longer needs them, and its w
// rows wait in registers, so only the first chunk-head of a CTA pays the load latency.
// 256 threads: warp w reads TMEM lanes 32*(w&3).. (its row), and the two warps that share a lane
// window split the columns (hsel = w>>2), so every elementwise phase is spread over 8 warps.
template <bool PACKED, bool FUSED>
__global__ void __launch_bounds__(256)
r7c_bwd_final_kernel(const bf16* __restrict__ w, const __grid_constant__ CUtensorMap tmap_do,
                     const __grid_constant__ CUtensorMap tmap_v, const unsigned char* __restrict__ ws_tiles,
                     int tiles_per_chunk, const __grid_constant__ CUtensorMap tmap_dq,
                     const __grid_constant__ CUtensorMap tmap_dw, const __grid_constant__ CUtensorMap tmap_dk,
                     const __grid_constant__ CUtensorMap tmap_dv, const __grid_constant__ CUtensorMap tmap_da,
                     const __grid_constant__ CUtensorMap tmap_db,
                     bf16* __restrict__ dq_rows, bf16* __restrict__ dw_rows, bf16* __restrict__ dk_rows,
                     bf16* __restrict__ dv_rows, bf16* __restrict__ da_rows, bf16* __restrict__ db_rows,
                     SeqView sv, int H, int NT, int n_ch, TokLayout lay, int* status, long long* dbg) {
#ifdef RWKVB200_DEVTOOLS
#define R7C_STAMP(n) do { if (dbg && tid == 0 && blockIdx.x == gridDim.x / 2 && it == 30) dbg[n] = clock64(); } while (0)
#else
#define R7C_STAMP(n) do {} while (0)
#endif
  extern __shared__ unsigned char smem_raw[];
  FinalSmem& sm = *reinterpret_cast<FinalSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wq = warp & 3, hsel = warp >> 2;

  if (tid == 0) {
    // each MMA group is issued by two threads (threads 0 and 32), one accumulator each, and completes with
    // the arrival of both: one thread issues an MMA about every 80 cycles, the tensor pipe takes them faster
    mbar_init(&sm.bar_lda, 1); mbar_init(&sm.bar_ldb, 1); mbar_init(&sm.bar_m1, 2); mbar_init(&sm.bar_m2, 2);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;

  auto coords = [&](const ChunkPos& p, int& bi, int& hi, int& t0) { bi = p.bi; hi = p.hi; t0 = p.c * L; };
  auto load_group_a = [&](const ChunkPos& p) {     // tid 0
    int bi, hi, t0; coords(p, bi, hi, t0);
    const unsigned char* tiles = ws_tiles + (size_t)p.ch * tiles_per_chunk * TILE_BYTES;
    mbar_expect_tx(&sm.bar_lda, 8 * TILE_BYTES);
    tma_load_4d(sm.dout, &tmap_do, &sm.bar_lda, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
    tma_load_4d(sm.v, &tmap_v, &sm.bar_lda, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
    bulk_load(sm.dz, tiles + S_DZ * TILE_BYTES, TILE_BYTES, &sm.bar_lda);
    bulk_load(sm.sa, tiles + S_SA * TILE_BYTES, TILE_BYTES, &sm.bar_lda);
    bulk_load(sm.aqk, tiles + S_AQK * TILE_BYTES, 2 * TILE_BYTES, &sm.bar_lda);
    bulk_load(sm.h0, tiles + S_H0 * TILE_BYTES, TILE_BYTES, &sm.bar_lda);
    bulk_load(sm.dhh, tiles + S_DHH * TILE_BYTES, TILE_BYTES, &sm.bar_lda);
  };
  auto load_group_b = [&](const ChunkPos& p) {     // tid 0
    const unsigned char* tiles = ws_tiles + (size_t)p.ch * tiles_per_chunk * TILE_BYTES;
    mbar_expect_tx(&sm.bar_ldb, 4 * TILE_BYTES);
    bulk_load(sm.qt, tiles + S_QT * TILE_BYTES, TILE_BYTES, &sm.bar_ldb);
    bulk_load(sm.at, tiles + S_AT * TILE_BYTES, TILE_BYTES, &sm.bar_ldb);
    bulk_load(sm.kt, tiles + S_KT * TILE_BYTES, TILE_BYTES, &sm.bar_ldb);
    bulk_load(sm.bt, tiles + S_BT * TILE_BYTES, TILE_BYTES, &sm.bar_ldb);
  };
  // Ask for everything a chunk-head will load to be brought into L2 (issued one chunk-head ahead of the
  // loads themselves, which then take an L2 round trip instead of a DRAM one).
  auto prefetch_l2 = [&](const ChunkPos& p) {      // one warp
    int bi, hi, t0; coords(p, bi, hi, t0);
    const unsigned char* tiles = ws_tiles + (size_t)p.ch * tiles_per_chunk * TILE_BYTES;
    if (lane == 0) {
      tma_prefetch_4d(&tmap_do, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
      tma_prefetch_4d(&tmap_v, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
      bulk_prefetch_l2(tiles + S_QT * TILE_BYTES, 3 * TILE_BYTES);     // q~, k~, b~
      bulk_prefetch_l2(tiles + S_AT * TILE_BYTES, 3 * TILE_BYTES);     // a~, A_qk, A_ak
      bulk_prefetch_l2(tiles + S_SA * TILE_BYTES, 3 * TILE_BYTES);     // sa, h~0, X
      bulk_prefetch_l2(tiles + S_DZ * TILE_BYTES, 2 * TILE_BYTES);     // dz, dh^
    }
    const int Tn = sv.length<PACKED>(bi);
    const long long base = sv.row<PACKED>(bi) * lay.sb + hi * lay.sh + sv.first<PACKED>(bi) * lay.st;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int tok = t0 + lane + 32 * n;
      if (tok < Tn) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + base + (long long)tok * lay.st));
    }
  };
  auto load_w = [&](const ChunkPos& p, uint4 (&rw)[2]) {   // all threads: 2 x 8 channels of the chunk's w rows
    int bi, hi, t0; coords(p, bi, hi, t0);
    const int Tn = sv.length<PACKED>(bi);
    const long long base = sv.row<PACKED>(bi) * lay.sb + hi * lay.sh + sv.first<PACKED>(bi) * lay.st;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int e = tid + 256 * n, row = e >> 3, cc = e & 7, tok = t0 + row;
      rw[n] = make_uint4(0u, 0u, 0u, 0u);
      if (tok < Tn) rw[n] = __ldg(reinterpret_cast<const uint4*>(w + base + (long long)tok * lay.st + 8 * cc));
    }
  };

  // chunk slots past the end of a (packed) sequence are skipped
  auto empty = [&](const ChunkPos& p) {
    if constexpr (!PACKED) return false;      // a dense batch has no empty slots
    return p.c * L >= sv.length<PACKED>(p.bi);
  };
  auto advance = [&](ChunkPos p) {
    do { chunk_step(p, gridDim.x, NT, H); } while (p.ch < n_ch && empty(p));
    return p;
  };
  ChunkPos cur = chunk_pos(blockIdx.x, NT, H);
  if (cur.ch < n_ch && empty(cur)) cur = advance(cur);
  ChunkPos nxt = cur;     // the chunk-head after `cur`, and the one after that (found once per iteration)
  if (cur.ch < n_ch) nxt = advance(cur);

  uint4 rw[2];
  if (cur.ch < n_ch) {
    if (tid == 0) { load_group_a(cur); load_group_b(cur); }
    load_w(cur, rw);
    if (warp == 1 && nxt.ch < n_ch) prefetch_l2(nxt);
  }

  bool ok = true;
  int it = 0;
  for (ChunkPos aft = nxt; cur.ch < n_ch && ok; cur = nxt, nxt = aft, ++it) {
    const int ch = cur.ch, next = nxt.ch;
    int bi, hi, t0; coords(cur, bi, hi, t0);
    const int Tn = sv.length<PACKED>(bi);
    // in a packed batch the last rows of a sequence's last chunk belong to the next sequence: such a chunk
    // is stored row by row instead of by TMA boxes
    const bool row_stores = PACKED && t0 + L > Tn;
    const long long out_base = sv.row<PACKED>(bi) * lay.sb + hi * lay.sh + (long long)(sv.first<PACKED>(bi) + t0) * lay.st;
    const unsigned char* tiles = ws_tiles + (size_t)ch * tiles_per_chunk * TILE_BYTES;
    const uint32_t par = it & 1;
    R7C_STAMP(16);

    // ---- g of every (token, channel), from the w rows already in registers
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int e = tid + 256 * n, row = e >> 3, cc = e & 7;
      const bool valid = t0 + row < Tn;
      const uint32_t u[4] = {rw[n].x, rw[n].y, rw[n].z, rw[n].w};
      float g[8];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        float w0 = bf16_lo(u[m]), w1 = bf16_hi(u[m]);
        if constexpr (FUSED) {      // the rows hold p: w = -e^{-1/2} sigmoid(p), as a bfloat16 value
          w0 = round_bf16(W_SCALE * sigmoidf_(w0));
          w1 = round_bf16(W_SCALE * sigmoidf_(w1));
        }
        g[2 * m] = valid ? -LOG2E * ex2(LOG2E * w0) : 0.f;
        g[2 * m + 1] = valid ? -LOG2E * ex2(LOG2E * w1) : 0.f;
      }
      *reinterpret_cast<float4*>(&sm.gg[row * NROW + 8 * cc]) = make_float4(g[0], g[1], g[2], g[3]);
      *reinterpret_cast<float4*>(&sm.gg[row * NROW + 8 * cc + 4]) = make_float4(g[4], g[5], g[6], g[7]);
    }
    if (tid == 0) bulk_wait_read();    // the TMA stores of the previous chunk-head have left the staging tiles
    R7C_STAMP(17);
    ok = mbar_wait(&sm.bar_lda, par, status, 321) && ok;
    ok = mbar_wait(&sm.bar_ldb, par, status, 324) && ok;
    ok = __syncthreads_and(ok);
    R7C_STAMP(18);

    // ---- MMA group 1: all four dA products, and dv
    if (tid == 0 && ok) {
      tc_fence_after();
      umma_tile<128, 128, 0, 0>(tmem_addr(tm, 0, 0), smem_u32(sm.dout), smem_u32(sm.v), false);        // [do;dz] [v;sa]^T
      umma_commit(&sm.bar_m1);
    }
    if (tid == 32 && ok) {
      tc_fence_after();
      umma_tile<64, 64, 1, 1, 8>(tmem_addr(tm, 0, 128), smem_u32(sm.aqk), smem_u32(sm.dout), false);   // A_qk^T do + A_ak^T dz
      umma_tile<64, 64, 0, 1>(tmem_addr(tm, 0, 128), smem_u32(sm.kt), smem_u32(sm.dhh), true);         // + k~ dh^
      umma_commit(&sm.bar_m1);
    }
    // ---- meanwhile: prefix sums of g over tokens, thread = (channel, quarter of the chunk)
    {
      const int c = tid & 63, quarter = tid >> 6;
      float gv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) gv[j] = sm.gg[(16 * quarter + j) * NROW + c];
      float run = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) { run += gv[j]; gv[j] = run; }
      sm.qtot[quarter][c] = run;
      __syncthreads();
      // gi - gref: the prefix inside the half; the first half lies before the reference point, the end of that half
      const float add = quarter == 0 ? -(run + sm.qtot[1][c]) : quarter == 1 ? -run : quarter == 3 ? sm.qtot[2][c] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) sm.gs[(16 * quarter + j) * NROW + c] = gv[j] + add;
    }
    // dglast[c] = sum_v dh^[c][v] X[c][v]  (X straight from the workspace)
    if (tid >= 128 && tid < 192 && ok) {
      const int c = tid - 128;
      float s_ = 0.f;
      const uint4* xr = reinterpret_cast<const uint4*>(tiles + S_X * TILE_BYTES);
#pragma unroll
      for (int cchunk = 0; cchunk < 8; ++cchunk) {
        const uint4 xa = __ldg(xr + (tile_chunk_off(c, cchunk) >> 4));
        const uint4 da_ = *reinterpret_cast<const uint4*>(sm.dhh + tile_chunk_off(c, cchunk));
        s_ += bf16_lo(xa.x) * bf16_lo(da_.x) + bf16_hi(xa.x) * bf16_hi(da_.x);
        s_ += bf16_lo(xa.y) * bf16_lo(da_.y) + bf16_hi(xa.y) * bf16_hi(da_.y);
        s_ += bf16_lo(xa.z) * bf16_lo(da_.z) + bf16_hi(xa.z) * bf16_hi(da_.z);
        s_ += bf16_lo(xa.w) * bf16_lo(da_.w) + bf16_hi(xa.w) * bf16_hi(da_.w);
      }
      sm.dgl[c] = s_;
    }
    ok = mbar_wait(&sm.bar_m1, par, status, 322) && ok;
    tc_fence_after();
    R7C_STAMP(19);
    if (ok) {
      const int r = 32 * wq + lane, i = r & 63;
      const bool lower = r >= 64;       // rows of dz: strictly lower; rows of do: lower incl. diagonal
      // The warp's 32 rows are i = 32*ihalf + lane, so which side of the diagonal a block of 32 columns lies on is
      // the same for the whole warp: left of the diagonal block every element is kept, right of it every element
      // is zero (TMEM is not read), and only the diagonal block takes a per-element choice.
      const int ihalf = wq & 1;
      unsigned char* dst = lower ? (hsel ? sm.daab : sm.daak) : (hsel ? sm.daqb : sm.daqk);
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        const int part = 2 * hsel + pp;   // hsel 0: products with v (dA_qk / dA_ak); hsel 1: with sa (dA_qb / dA_ab)
        const int j0 = 32 * pp;
        float x[32];
        if (pp > ihalf) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = 0.f;
          tile_store_row32(dst, i, j0, x);
          continue;
        }
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm, 32 * wq, 32 * part), rr);
        tmem_ld_wait();
        if (pp < ihalf) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
          tile_store_row32(dst, i, j0, x);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const bool keep = lower ? (j < lane) : (j <= lane);
            x[j] = keep ? __uint_as_float(rr[j]) : 0.f;
          }
          tile_store_row32(dst, i, j0, x);
        }
      }
      // dv rows sit on the lower lane halves of columns 128..191; each warp of a pair takes 32 columns.
      // Staged in the A_qk tile (dead: MMA group 1 has completed), stored by TMA below.
      const int row = 16 * wq + (lane & 15);
      uint32_t rr[32];
      tmem_ld32(tmem_addr(tm, 32 * wq, 128 + 32 * hsel), rr);
      tmem_ld_wait();
      if (lane < 16) {
        float x[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
        tile_store_row32(sm.aqk, row, 32 * hsel, x);
      }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    R7C_STAMP(20);

    // ---- MMA group 2: [dq~; da~] (columns 0..63) and [dk~; db~] (columns 64..127)
    if (tid == 32 && ok) {
      tc_fence_after();
      umma_tile<128, 64, 1, 1>(tmem_addr(tm, 0, 64), smem_u32(sm.daqk), smem_u32(sm.qt), false, 2 * TILE_BYTES);  // [dA_qk|dA_qb]^T q~
      umma_tile<128, 64, 1, 1>(tmem_addr(tm, 0, 64), smem_u32(sm.daak), smem_u32(sm.at), true, 2 * TILE_BYTES);   // + [dA_ak|dA_ab]^T a~
      umma_tile<128, 64, 0, 0>(tmem_addr(tm, 0, 64), smem_u32(sm.v), smem_u32(sm.dhh), true);          // + [v;sa] dh^^T
      umma_commit(&sm.bar_m2);
    }
    if (tid == 0 && ok) {
      tc_fence_after();
      umma_tile<128, 64, 0, 0>(tmem_addr(tm, 0, 0), smem_u32(sm.dout), smem_u32(sm.h0), false);        // [do;dz] h~0^T
      umma_tile<128, 64, 0, 1>(tmem_addr(tm, 0, 0), smem_u32(sm.daqk), smem_u32(sm.kt), true);         // + [dA_qk;dA_ak] k~
      umma_tile<128, 64, 0, 1>(tmem_addr(tm, 0, 0), smem_u32(sm.daqb), smem_u32(sm.bt), true);         // + [dA_qb;dA_ab] b~
      umma_commit(&sm.bar_m2);
      if (!row_stores) {
        tma_store_4d(&tmap_dv, sm.aqk, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
        bulk_commit();
      }
    }
    if (row_stores && ok) {
      store_tile_rows<256>(dv_rows + out_base, lay.st, sm.aqk, Tn - t0, tid);
      __syncthreads();      // the A_qk tile is loaded again below
    }
    ok = mbar_wait(&sm.bar_m2, par, status, 323) && ok;
    tc_fence_after();
    R7C_STAMP(21);
    // group A tiles are free: request the next chunk-head's, and fetch its w rows
    if (next < n_ch) {
      if (tid == 0 && ok) { bulk_wait_read(); load_group_a(nxt); }
      load_w(nxt, rw);
      aft = advance(nxt);
      if (warp == 1 && aft.ch < n_ch) prefetch_l2(aft);
    }

    // ---- epilogue.  Row r < 64 holds dq~_i and dk~_i (token i = r), row r >= 64 holds da~_i, db~_i; the
    // two warps of a lane window take 32 channels each.  Row owners read and write the fp32 scratch
    // arrays as float4 (conflict-free with the padded rows).  red1 = dq~ q~ - dk~ k~ and
    // red2 = da~ a~ - db~ b~ overlay the dA tiles (dead once MMA group 2 has completed).
    float* red1 = reinterpret_cast<float*>(sm.daqk);
    float* red2 = red1 + L * NROW;
    if (ok) {
      const int r = 32 * wq + lane, i = r & 63;
      const bool second = r >= 64;
      float* red = second ? red2 : red1;
      const int c0 = 32 * hsel;
      uint32_t r1[32], r2[32];
      tmem_ld32(tmem_addr(tm, 32 * wq, c0), r1);          // dq~ / da~
      tmem_ld32(tmem_addr(tm, 32 * wq, 64 + c0), r2);     // dk~ / db~
      tmem_ld_wait();
      float t1[32], t2[32], o1[32], o2[32], ge[32];
      tile_load_row32(second ? sm.at : sm.qt, i, c0, t1);
      tile_load_row32(second ? sm.bt : sm.kt, i, c0, t2);
#pragma unroll
      for (int j4 = 0; j4 < 32; j4 += 4) {
        const int c = c0 + j4;
        const float4 gs4 = *reinterpret_cast<const float4*>(&sm.gs[i * NROW + c]);
        const float4 gg4 = *reinterpret_cast<const float4*>(&sm.gg[i * NROW + c]);
        const float gsv[4] = {gs4.x, gs4.y, gs4.z, gs4.w}, ggv[4] = {gg4.x, gg4.y, gg4.z, gg4.w};
        float rd[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const int j = j4 + m;
          const float d1 = gsv[m];                                       // gi - gref
          const float x1 = __uint_as_float(r1[j]), x2 = __uint_as_float(r2[j]);
          o2[j] = x2 * ex2(-d1);                                         // dk / db
          o1[j] = x1 * ex2(second ? d1 - ggv[m] : d1);                   // da / dq
          ge[j] = x1 * t1[j];
          rd[m] = ge[j] - x2 * t2[j];
        }
        *reinterpret_cast<float4*>(&red[i * NROW + c]) = make_float4(rd[0], rd[1], rd[2], rd[3]);
      }
      if (second) tile_store_row32(sm.dge, i, c0, ge);
      tile_store_row32(sm.stage[second ? 2 : 0], i, c0, o1);    // da / dq
      tile_store_row32(sm.stage[second ? 3 : 1], i, c0, o2);    // db / dk
    }
    fence_async_smem();
    ok = __syncthreads_and(ok);
    R7C_STAMP(22);
    if (row_stores && ok) {
      store_tile_rows<256>(dq_rows + out_base, lay.st, sm.stage[0], Tn - t0, tid);
      store_tile_rows<256>(dk_rows + out_base, lay.st, sm.stage[1], Tn - t0, tid);
      store_tile_rows<256>(da_rows + out_base, lay.st, sm.stage[2], Tn - t0, tid);
      store_tile_rows<256>(db_rows + out_base, lay.st, sm.stage[3], Tn - t0, tid);
    }
    if (tid == 0 && ok) {
      if (!row_stores) {
        const int tt = sv.first<PACKED>(bi) + t0, br = sv.row<PACKED>(bi);
        tma_store_4d(&tmap_dq, sm.stage[0], 0, tt, hi, br);
        tma_store_4d(&tmap_dk, sm.stage[1], 0, tt, hi, br);
        tma_store_4d(&tmap_da, sm.stage[2], 0, tt, hi, br);
        tma_store_4d(&tmap_db, sm.stage[3], 0, tt, hi, br);
        bulk_commit();
      }
      if (next < n_ch) load_group_b(nxt);       // q~, a~, k~, b~ were last read by the epilogue above
    }
    // reverse inclusive prefix over tokens, per channel; thread = (channel, quarter)
    {
      const int c = tid & 63, quarter = tid >> 6;
      float rv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) rv[j] = red1[(16 * quarter + j) * NROW + c] + red2[(16 * quarter + j) * NROW + c];
      float run = 0.f;
#pragma unroll
      for (int j = 15; j >= 0; --j) { run += rv[j]; rv[j] = run; }
      sm.rqtot[quarter][c] = run;
      __syncthreads();
      float add = sm.dgl[c];
      for (int q2 = quarter + 1; q2 < 4; ++q2) add += sm.rqtot[q2][c];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int ii = 16 * quarter + j;
        const float e_ = __bfloat162float(*reinterpret_cast<const bf16*>(sm.dge + tile_off(ii, c)));
        const float dg = rv[j] + add - e_;
        // dw = dg g, with g = gg ln 2 (gg is in units of log 2)
        *reinterpret_cast<bf16*>(sm.stage[4] + tile_off(ii, c)) = __float2bfloat16_rn(dg * (LN2 * sm.gg[ii * NROW + c]));
      }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (row_stores) {
      if (ok) store_tile_rows<256>(dw_rows + out_base, lay.st, sm.stage[4], Tn - t0, tid);
    } else if (tid == 0 && ok) {
      tma_store_4d(&tmap_dw, sm.stage[4], 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
      bulk_commit();
    }
    R7C_STAMP(23);
  }
  if (tid == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 256);
#undef R7C_STAMP
}

// ---------------------------------------------------------------------------------------------
// 6. fused producers, backward: one 64-channel row per 8 threads (16 bytes each), in place
//      dp = dw W_SCALE s_p (1 - s_p),  s_p = sigmoid(p)
//      dkk = -da + db s_q,  s_q = sigmoid(q);   dq = db kk s_q (1 - s_q)
//      du = (dkk - kk (kk . dkk)) / |u|,  kk = u / |u|
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
r7c_producer_bwd_kernel(const bf16* __restrict__ p, const bf16* __restrict__ u, const bf16* __restrict__ q,
                        bf16* dw_dp, bf16* da_du, bf16* db_dq, long long n_rows) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = t >> 3;
  const bool live = row < n_rows;
  const long long off = (live ? row : 0) * 64 + 8 * (t & 7);
  float pv[8], uv[8], qv[8], dw[8], da[8], db[8];
  auto load8 = [&](const bf16* src, float* x) {
    const uint4 w4 = *reinterpret_cast<const uint4*>(src + off);
    const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) { x[2 * m] = bf16_lo(w[m]); x[2 * m + 1] = bf16_hi(w[m]); }
  };
  auto store8 = [&](bf16* dst, const float* x) {
    *reinterpret_cast<uint4*>(dst + off) = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]),
                                                      pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
  };
  load8(p, pv); load8(u, uv); load8(q, qv); load8(dw_dp, dw); load8(da_du, da); load8(db_dq, db);
  float ss = 0.f;
#pragma unroll
  for (int x = 0; x < 8; ++x) ss += uv[x] * uv[x];
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  const float inv = rsqrtf(fmaxf(ss, 1e-24f));      // 1 / max(|u|, 1e-12)
  float kk[8], dkk[8], dot = 0.f, dp[8], dq[8], du[8];
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const float sp = sigmoidf_(pv[x]), sq = sigmoidf_(qv[x]);
    kk[x] = uv[x] * inv;
    dp[x] = dw[x] * W_SCALE * sp * (1.f - sp);
    dkk[x] = -da[x] + db[x] * sq;
    dq[x] = db[x] * kk[x] * sq * (1.f - sq);
    dot += kk[x] * dkk[x];
  }
  dot += __shfl_xor_sync(0xffffffffu, dot, 1);
  dot += __shfl_xor_sync(0xffffffffu, dot, 2);
  dot += __shfl_xor_sync(0xffffffffu, dot, 4);
#pragma unroll
  for (int x = 0; x < 8; ++x) du[x] = (dkk[x] - kk[x] * dot) * inv;
  if (live) { store8(dw_dp, dp); store8(da_du, du); store8(db_dq, dq); }
}

}  // namespace r7c

int launch_rwkv7_producer_bwd(const void* p, const void* u, const void* q, void* dw_dp, void* da_du, void* db_dq,
                              long long n_rows, cudaStream_t st) {
  typedef __nv_bfloat16 bf16;
  ProfScope prof("r7c_producer_bwd_kernel", st);
  const long long threads = n_rows * 8;
  r7c::r7c_producer_bwd_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(
      (const bf16*)p, (const bf16*)u, (const bf16*)q, (bf16*)dw_dp, (bf16*)da_du, (bf16*)db_dq, n_rows);
  return check_launch();
}

int launch_rwkv7_chunked_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                             const float* h0, int n_state, const void* d_o, const float* d_ht,
                             void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                             void* workspace, int B, int Tn, int H, int head_first, bool kept, cudaStream_t st,
                             const int* seq_start, const int* seq_len, int T_total, bool fused, int phases) {
  using namespace r7c;
  if (fused && (seq_start || head_first)) return RWKVB200_E_UNSUPPORTED;
  typedef __nv_bfloat16 bf16;
  int e = RWKVB200_OK;
  if (!kept && (phases & PHASE_PREPARE)) {   // the workspace does not hold a forward pass yet: recompute it from the inputs
    e = launch_rwkv7_chunked_fwd(r, w, k, v, a, b, h0, n_state, nullptr, nullptr, workspace, B, Tn, H, head_first,
                                 true, st, seq_start, seq_len, T_total, fused);
    if (e) return e;
  }
  int* status = device_status_ptr();
  if (!status) { last_cuda_error_slot() = 99999; return RWKVB200_E_CUDA; }
  CUtensorMap tmap_do, tmap_v, tmap_out[6];
  const SeqView sv{seq_start, seq_len, Tn};
  const int mapB = seq_start ? 1 : B, mapT = seq_start ? T_total : Tn;   // shape of the token tensors
  e = make_token_tensor_map(&tmap_do, d_o, mapB, mapT, H, head_first);
  if (e) return e;
  e = make_token_tensor_map(&tmap_v, v, mapB, mapT, H, head_first);
  if (e) return e;
  void* outs[6] = {dr, dw, dk, dv, da, db};
  for (int i = 0; i < 6; ++i) {
    e = make_token_tensor_map(&tmap_out[i], outs[i], mapB, mapT, H, head_first);
    if (e) return e;
  }
  const int NT = num_chunks(Tn);
  Workspace ws = carve(workspace, B, Tn, H, ALL_TILES);
  TokLayout lay(mapT, H, head_first);
  // every kernel exists for dense batches and for packed variable-length ones
#define R7C_DISPATCH_PACKED(...) do { if (seq_start) { constexpr bool P = true; __VA_ARGS__; } else { constexpr bool P = false; __VA_ARGS__; } } while (0)
  if (phases & PHASE_PREPARE) {
    const int smem = (int)sizeof(PreSmem) + 1024;
    int dev = 0, sms = 0;
    if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))
      return RWKVB200_E_CUDA;
    const int pre_grid = B * H * NT < 2 * sms ? B * H * NT : 2 * sms;     // persistent: two CTAs per SM
    ProfScope prof("r7c_bwd_pre_kernel", st);
    R7C_DISPATCH_PACKED(
      if (cuda_ok(cudaFuncSetAttribute(r7c_bwd_pre_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
        return RWKVB200_E_CUDA;
      r7c_bwd_pre_kernel<P><<<pre_grid, 128, smem, st>>>(tmap_do, ws.tiles, ALL_TILES, sv, H, NT, B * H * NT, status));
  }
  e = check_launch();
  if (e) return e;
  if (phases & PHASE_SCAN) {
    const int smem = (int)sizeof(BScanSmem) + 1024;
    int dev = 0, sms = 0;
    if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))
      return RWKVB200_E_CUDA;
    ProfScope prof("r7c_bwd_scan_kernel", st);
    R7C_DISPATCH_PACKED(
      if (cuda_ok(cudaFuncSetAttribute(r7c_bwd_scan_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
        return RWKVB200_E_CUDA;
      r7c_bwd_scan_kernel<P><<<B * H, 256, smem, st>>>(tmap_do, ws.tiles, ws.aux, ALL_TILES, d_ht, d_h0, sv, H, NT,
                                                       B * H <= sms ? 1 : 0, status));
  }
  e = check_launch();
  if (e) return e;
  // Units the forward marked (decay beyond the range of the scaled operands, or a very short sequence): their
  // gradients come from the float32 recurrence instead.  Its state checkpoints (16 KB per 8 tokens = 128 KB per
  // chunk) go into the unit's own tile region of the workspace (144 KB per chunk), whose contents are void for
  // such a unit.
  auto exact_units = [&]() -> int {
    const long long unit_floats = (long long)NT * ALL_TILES * TILE_BYTES / (long long)sizeof(float);
    float* ckpt = reinterpret_cast<float*>(ws.tiles);
    const UnitSel sel{ws.flags, seq_start, seq_len, unit_floats};
    const int tt = seq_start ? T_total : 0;
    int e2 = launch_rwkv7_rec_fwd(r, w, k, v, a, b, h0, n_state, nullptr, nullptr, ckpt, R7_CKPT, B, Tn, H,
                                  RWKVB200_BF16, head_first, st, &sel, tt);
    if (e2) return e2;
    return launch_rwkv7_rec_bwd(r, w, k, v, a, b, d_o, d_ht, ckpt, dr, dw, dk, dv, da, db, d_h0, B, Tn, H,
                                RWKVB200_BF16, head_first, st, &sel, tt);
  };
  if (!(phases & PHASE_FINISH)) {
    // a scan-only call hands the gradient of the initial state to its caller (who passes it to the rank on the
    // left) before the token gradients exist: the marked units' share of it has to be exact already
    if ((phases & PHASE_SCAN) && !fused) return exact_units();
    return e;
  }
  {
    const int smem = (int)sizeof(FinalSmem) + 1024;
    ProfScope prof("r7c_bwd_final_kernel", st);
    const int n_ch = B * H * NT;
    int dev = 0, sms = 0;
    if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))
      return RWKVB200_E_CUDA;
    const int grid = n_ch < sms ? n_ch : sms;     // persistent: one CTA per SM
#define R7C_LAUNCH_FINAL(P, F)                                                                                    \
    do {                                                                                                          \
      if (cuda_ok(cudaFuncSetAttribute(r7c_bwd_final_kernel<P, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))) \
        return RWKVB200_E_CUDA;                                                                                   \
      r7c_bwd_final_kernel<P, F><<<grid, 256, smem, st>>>((const bf16*)w, tmap_do, tmap_v, ws.tiles, ALL_TILES,   \
          tmap_out[0], tmap_out[1], tmap_out[2], tmap_out[3], tmap_out[4], tmap_out[5], (bf16*)dr, (bf16*)dw,     \
          (bf16*)dk, (bf16*)dv, (bf16*)da, (bf16*)db, sv, H, NT, n_ch, lay, status, debug_stamp_buffer());        \
    } while (0)
    if (seq_start) R7C_LAUNCH_FINAL(true, false);
    else if (fused) R7C_LAUNCH_FINAL(false, true);
    else R7C_LAUNCH_FINAL(false, false);
#undef R7C_LAUNCH_FINAL
  }
#undef R7C_DISPATCH_PACKED
  if (fused) {      // dw, da, db -> gradients of the pre-activations, in place
    e = check_launch();
    if (e) return e;
    return launch_rwkv7_producer_bwd(w, a, b, dw, da, db, (long long)B * Tn * H, st);
  }
  e = check_launch();
  if (e) return e;
  return exact_units();
}


}  // namespace rwkvb200
