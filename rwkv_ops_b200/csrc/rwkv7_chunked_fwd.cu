// Chunked RWKV7 forward on tcgen05 (bf16 token tensors, fp32 state).  Equations and the
// two-kernel structure are described in rwkv7_chunked.cuh.
#include "rwkv7_chunked.cuh"

namespace rwkvb200 {
namespace r7c {

using namespace tc;
typedef __nv_bfloat16 bf16;

// All decay sums of this file are in units of log 2 (tc::ex2).  No exponent is clamped: inside DECAY_LIMIT every
// factor is a normal number, and a unit beyond it is recomputed by the float32 recurrence whatever the
// tensor-core kernels wrote for it.
constexpr float EXP2_FLOOR = -126.f;      // 2^x below this is flushed to zero anyway

// ---------------------------------------------------------------------------------------------
// intra-chunk kernel: persistent CTAs of 256 threads over the B*H*NT chunk-heads
// ---------------------------------------------------------------------------------------------
constexpr int NROW = 68;   // padded row of the fp32 copy of A_ab (keeps float4 alignment)

struct IntraSmem {
  unsigned char qt[TILE_BYTES], at[TILE_BYTES];     // [q~; a~]  (128-row A operand)
  unsigned char kt[TILE_BYTES], bt[TILE_BYTES];     // [k~; b~]  (128-row B operand)
  unsigned char aqk[TILE_BYTES], aak[TILE_BYTES];   // [A_qk; A_ak] (128-row A operand); aak later holds W
  unsigned char o1[TILE_BYTES];                     // A_qk v
  unsigned char aqb[TILE_BYTES];
  unsigned char v[TILE_BYTES];                      // TMA; later U
  unsigned char ainv[TILE_BYTES];
  unsigned char y[TILE_BYTES];                      // A_ak v
  float nmat[L * NROW];                             // stril(A_ab) in fp32
  float qtot[4][64];                                // sums of g over the four quarters of the chunk
  uint64_t bar_v, bar_w, bar_in, bar_ia, bar_m1, bar_m2, bar_m3, bar_m4, bar_m5;
  uint32_t tmem_base;
};

// Persistent: CTAs (two per SM) walk over chunk-heads ch = blockIdx.x, blockIdx.x + gridDim.x, ...  The
// raw q, k, a, b, w tiles of the next chunk-head are requested by TMA as soon as the tiles they land in
// (q~, k~, a~, b~, which are then scaled in place, and O1) have been copied out, its v tile as soon as
// MMA 2 has read the current one, and the rows of the one after that are asked into L2.
// 256 threads: warp w reads TMEM lanes 32*(w&3).. and the two warps that share a lane window split
// the columns (hsel = w>>2); the triangular solve runs on warps 0-1 while the other warps drain MMA 2.
template <bool PACKED, bool FUSED>
__global__ void __launch_bounds__(256, 2)
r7c_intra_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ w, const bf16* __restrict__ k,
                     const bf16* __restrict__ a, const bf16* __restrict__ b,
                     const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_w,
                     const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_v, unsigned char* __restrict__ ws_tiles,
                     float* __restrict__ ws_aux, int* __restrict__ ws_flags, int tiles_per_chunk,
                     int keep_for_bwd, SeqView sv, int H, int NT, int n_ch, TokLayout lay, int* status, long long* dbg) {
#ifdef RWKVB200_DEVTOOLS
#define R7C_STAMP(n) do { if (dbg && tid == 0 && blockIdx.x == gridDim.x / 2 && it == 30) dbg[n] = clock64(); } while (0)
#else
#define R7C_STAMP(n) do {} while (0)
#endif
  extern __shared__ unsigned char smem_raw[];
  IntraSmem& sm = *reinterpret_cast<IntraSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wq = warp & 3, hsel = warp >> 2;

  if (tid == 0) {
    mbar_init(&sm.bar_v, 1); mbar_init(&sm.bar_w, 1); mbar_init(&sm.bar_in, 1); mbar_init(&sm.bar_ia, 1); mbar_init(&sm.bar_m1, 1); mbar_init(&sm.bar_m2, 1); mbar_init(&sm.bar_m3, 1);
    mbar_init(&sm.bar_m4, 1); mbar_init(&sm.bar_m5, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;

  auto coords = [&](const ChunkPos& p, int& bi, int& hi, int& t0) { bi = p.bi; hi = p.hi; t0 = p.c * L; };
  // The raw tiles of a chunk-head (rows past the end of the sequence arrive as zeros).  w, needed first,
  // lands in the A_qk tile, free from the end of the triangular inverse to the first epilogue of the next
  // chunk-head; q, k, a, b, needed only after the prefix sums, land in the tiles that will hold their
  // scaled versions once those have been copied out.
  auto load_w = [&](const ChunkPos& p) {       // tid 0
    int bi, hi, t0; coords(p, bi, hi, t0);
    mbar_expect_tx(&sm.bar_w, TILE_BYTES);
    tma_load_4d(sm.aqk, &tmap_w, &sm.bar_w, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
  };
  // q, k, b land in tiles that only MMA 1 reads and are requested as soon as MMA 2 has completed (their
  // copies to the workspace have left shared memory by then); a lands in the tile MMA 3 reads and is requested
  // after it: both are on their way most of a chunk-head before the next one needs them.
  auto load_qkb = [&](const ChunkPos& p) {     // tid 0
    int bi, hi, t0; coords(p, bi, hi, t0);
    const int tt = sv.first<PACKED>(bi) + t0, br = sv.row<PACKED>(bi);
    mbar_expect_tx(&sm.bar_in, 3 * TILE_BYTES);
    tma_load_4d(sm.qt, &tmap_q, &sm.bar_in, 0, tt, hi, br);
    tma_load_4d(sm.kt, &tmap_k, &sm.bar_in, 0, tt, hi, br);
    tma_load_4d(sm.bt, &tmap_b, &sm.bar_in, 0, tt, hi, br);
  };
  auto load_a = [&](const ChunkPos& p) {       // tid 0
    int bi, hi, t0; coords(p, bi, hi, t0);
    mbar_expect_tx(&sm.bar_ia, TILE_BYTES);
    tma_load_4d(sm.at, &tmap_a, &sm.bar_ia, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
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
  // Ask for a chunk-head's token rows to be brought into L2, ahead of the TMA loads above.
  auto prefetch_rows = [&](const ChunkPos& p) {
    int bi, hi, t0; coords(p, bi, hi, t0);
    const int Tn = sv.length<PACKED>(bi);
    const long long base = sv.row<PACKED>(bi) * lay.sb + hi * lay.sh + sv.first<PACKED>(bi) * lay.st;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int e = tid + 256 * n, row = e >> 3, cc = e & 7, tok = t0 + row;
      if (tok < Tn && cc == 0) {      // one 128-byte row per request
        const long long off = base + (long long)tok * lay.st;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(w + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(q + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(k + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(b + off));
      }
    }
  };
  auto load_v = [&](const ChunkPos& p) {   // tid 0
    int bi, hi, t0; coords(p, bi, hi, t0);
    mbar_expect_tx(&sm.bar_v, TILE_BYTES);
    tma_load_4d(sm.v, &tmap_v, &sm.bar_v, 0, sv.first<PACKED>(bi) + t0, hi, sv.row<PACKED>(bi));
  };
  ChunkPos cur = chunk_pos(blockIdx.x, NT, H);
  if (cur.ch < n_ch && empty(cur)) cur = advance(cur);
  if (cur.ch < n_ch && tid == 0) { load_w(cur); load_qkb(cur); load_a(cur); load_v(cur); }
  // The two CTAs that share an SM would otherwise run their phases in lockstep and compete for the
  // same unit (shared-memory pipe during the triangular solve); start every other CTA half a
  // chunk-head late.
  if (blockIdx.x & 1) __nanosleep(6000);

  bool ok = true;
  int it = 0;
  for (ChunkPos nxt; cur.ch < n_ch && ok; cur = nxt, ++it) {
    const int ch = cur.ch;
    int bi, hi, t0; coords(cur, bi, hi, t0);
    const int Tn = sv.length<PACKED>(bi);
    unsigned char* out_tiles = ws_tiles + (size_t)ch * tiles_per_chunk * TILE_BYTES;
    const uint32_t par = it & 1;
    nxt = advance(cur);
    const int next = nxt.ch;

    R7C_STAMP(0);
    if (next < n_ch) prefetch_rows(nxt);
    // this thread's 2 x 16 bytes (8 channels of one token) of the raw w tile
    uint4 rw[2];
    ok = mbar_wait(&sm.bar_w, par, status, 206) && ok;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int e = tid + 256 * n;
      rw[n] = *reinterpret_cast<const uint4*>(sm.aqk + tile_chunk_off(e >> 3, e & 7));
    }
    // ---- phase A: decay prefix sums (in units of log 2) and the four scaled operands; the prefix sum over tokens goes
    // through shared memory (the fp32 area that later holds A_ab).
    {
      float* gs = sm.nmat;
      float gown[2][8];     // g of this thread's 2 x 8 (token, channel) entries
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int e = tid + 256 * n, row = e >> 3, cc = e & 7;
        const bool valid = t0 + row < Tn;
        const uint32_t u[4] = {rw[n].x, rw[n].y, rw[n].z, rw[n].w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          float w0 = bf16_lo(u[m]), w1 = bf16_hi(u[m]);
          if constexpr (FUSED) {      // the tile holds p: w = -e^{-1/2} sigmoid(p), as a bfloat16 value
            w0 = round_bf16(W_SCALE * sigmoidf_(w0));
            w1 = round_bf16(W_SCALE * sigmoidf_(w1));
          }
          gown[n][2 * m] = valid ? -LOG2E * ex2(LOG2E * w0) : 0.f;
          gown[n][2 * m + 1] = valid ? -LOG2E * ex2(LOG2E * w1) : 0.f;
        }
        *reinterpret_cast<float4*>(&gs[row * NROW + 8 * cc]) = make_float4(gown[n][0], gown[n][1], gown[n][2], gown[n][3]);
        *reinterpret_cast<float4*>(&gs[row * NROW + 8 * cc + 4]) = make_float4(gown[n][4], gown[n][5], gown[n][6], gown[n][7]);
      }
      __syncthreads();
      R7C_STAMP(1);
      {
        const int c = tid & 63, quarter = tid >> 6;
        float gv[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) gv[j] = gs[(16 * quarter + j) * NROW + c];
        float run = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { run += gv[j]; gv[j] = run; }
        sm.qtot[quarter][c] = run;
        __syncthreads();
        // gi - gref: the prefix inside the half; the reference point is the end of the first half
        const float add = quarter == 0 ? -(run + sm.qtot[1][c]) : quarter == 1 ? -run : quarter == 3 ? sm.qtot[2][c] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) gs[(16 * quarter + j) * NROW + c] = gv[j] + add;
      }
      __syncthreads();
      if (tid < 64) {
        const float tot0 = sm.qtot[0][tid] + sm.qtot[1][tid], tot1 = sm.qtot[2][tid] + sm.qtot[3][tid];
        ws_aux[(size_t)ch * AUX_FLOATS + tid] = ex2(fmaxf(tot0, EXP2_FLOOR));        // e^{gref}
        ws_aux[(size_t)ch * AUX_FLOATS + 64 + tid] = ex2(fmaxf(tot1, EXP2_FLOOR));   // e^{glast-gref}
        // a half-chunk decay sum beyond the limit: the unit is recomputed by the float32 recurrence
        if (fminf(tot0, tot1) < -DECAY_LIMIT * LOG2E || Tn < SHORT_SEQ) ws_flags[bi * H + hi] = 1;
      }
      // the raw q, k, a, b: each thread scales its own 2 x 16 bytes in place (the previous chunk-head's W, U,
      // A_qb, O1 copies may still be reading their tiles: those are rewritten only after MMA 1)
      uint4 rq[2], rk[2], ra[2], rb[2];
      ok = mbar_wait(&sm.bar_in, par, status, 207) && ok;
      ok = mbar_wait(&sm.bar_ia, par, status, 208) && ok;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int e = tid + 256 * n;
        const uint32_t off = tile_chunk_off(e >> 3, e & 7);
        rq[n] = *reinterpret_cast<const uint4*>(sm.qt + off);
        rk[n] = *reinterpret_cast<const uint4*>(sm.kt + off);
        ra[n] = *reinterpret_cast<const uint4*>(sm.at + off);
        rb[n] = *reinterpret_cast<const uint4*>(sm.bt + off);
        if (PACKED && t0 + (e >> 3) >= Tn) {      // in a packed batch these rows belong to the next sequence
          rq[n] = make_uint4(0u, 0u, 0u, 0u); rk[n] = rq[n]; ra[n] = rq[n]; rb[n] = rq[n];
        }
        if constexpr (FUSED) {      // the a / b tiles hold u and q: a = -kk, b = kk sigmoid(q), kk = u / |u|
          const uint32_t uu[4] = {ra[n].x, ra[n].y, ra[n].z, ra[n].w}, qq[4] = {rb[n].x, rb[n].y, rb[n].z, rb[n].w};
          float uv[8], ss = 0.f;
#pragma unroll
          for (int m = 0; m < 4; ++m) { uv[2 * m] = bf16_lo(uu[m]); uv[2 * m + 1] = bf16_hi(uu[m]); }
#pragma unroll
          for (int x = 0; x < 8; ++x) ss += uv[x] * uv[x];
          ss += __shfl_xor_sync(0xffffffffu, ss, 1);      // the 8 threads of a token row are neighbouring lanes
          ss += __shfl_xor_sync(0xffffffffu, ss, 2);
          ss += __shfl_xor_sync(0xffffffffu, ss, 4);
          const float inv = rsqrtf(fmaxf(ss, 1e-24f));      // 1 / max(|u|, 1e-12)
          uint32_t na[4], nb[4];
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            const float k0 = uv[2 * m] * inv, k1 = uv[2 * m + 1] * inv;
            na[m] = pack_bf16(-k0, -k1);
            nb[m] = pack_bf16(k0 * sigmoidf_(bf16_lo(qq[m])), k1 * sigmoidf_(bf16_hi(qq[m])));
          }
          ra[n] = make_uint4(na[0], na[1], na[2], na[3]);
          rb[n] = make_uint4(nb[0], nb[1], nb[2], nb[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int e = tid + 256 * n, row = e >> 3, cc = e & 7;
        float gl[8];
        *reinterpret_cast<float4*>(gl) = *reinterpret_cast<const float4*>(&gs[row * NROW + 8 * cc]);
        *reinterpret_cast<float4*>(gl + 4) = *reinterpret_cast<const float4*>(&gs[row * NROW + 8 * cc + 4]);
        const uint32_t uq[4] = {rq[n].x, rq[n].y, rq[n].z, rq[n].w};
        const uint32_t uk[4] = {rk[n].x, rk[n].y, rk[n].z, rk[n].w};
        const uint32_t ua[4] = {ra[n].x, ra[n].y, ra[n].z, ra[n].w};
        const uint32_t ub[4] = {rb[n].x, rb[n].y, rb[n].z, rb[n].w};
        uint32_t oq[4], ok_[4], oa[4], ob[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          float eq[2], ek[2], ea[2];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int x = 2 * m + hh;
            const float d1 = gl[x];                                         // gi - gref
            eq[hh] = ex2(d1); ek[hh] = ex2(-d1); ea[hh] = ex2(d1 - gown[n][x]);
          }
          oq[m] = pack_bf16(bf16_lo(uq[m]) * eq[0], bf16_hi(uq[m]) * eq[1]);
          ok_[m] = pack_bf16(bf16_lo(uk[m]) * ek[0], bf16_hi(uk[m]) * ek[1]);
          oa[m] = pack_bf16(bf16_lo(ua[m]) * ea[0], bf16_hi(ua[m]) * ea[1]);
          ob[m] = pack_bf16(bf16_lo(ub[m]) * ek[0], bf16_hi(ub[m]) * ek[1]);
        }
        const uint32_t off = tile_chunk_off(row, cc);
        *reinterpret_cast<uint4*>(sm.qt + off) = make_uint4(oq[0], oq[1], oq[2], oq[3]);
        *reinterpret_cast<uint4*>(sm.kt + off) = make_uint4(ok_[0], ok_[1], ok_[2], ok_[3]);
        *reinterpret_cast<uint4*>(sm.at + off) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
        *reinterpret_cast<uint4*>(sm.bt + off) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
      }
    }
    fence_async_smem();
    __syncthreads();

    R7C_STAMP(2);
    // ---- MMA 1: [q~; a~] [k~; b~]^T  ->  TMEM columns 0..127, row r on lane r
    if (tid == 0) {
      bulk_wait_read();      // the previous W, U copies are done: the epilogue below rewrites their tiles
      tc_fence_after();
      umma_tile<128, 128, 0, 0>(tm, smem_u32(sm.qt), smem_u32(sm.kt), false);
      umma_commit(&sm.bar_m1);
    }
    ok = mbar_wait(&sm.bar_m1, par, status, 201) && ok;
    tc_fence_after();
    R7C_STAMP(3);
    if (tid == 0 && ok) {      // MMA 1 was the last reader of q~, k~, b~ in shared memory: copy them out now
      bulk_store(out_tiles + S_QT * TILE_BYTES, sm.qt, TILE_BYTES);
      bulk_store(out_tiles + S_KT * TILE_BYTES, sm.kt, TILE_BYTES);
      bulk_store(out_tiles + S_BT * TILE_BYTES, sm.bt, TILE_BYTES);
      bulk_commit();
    }
    if (ok) {
      const int r = 32 * wq + lane, i = r & 63;
      const bool lower = r >= 64;       // rows of a~: strictly lower triangle; rows of q~: lower incl. diagonal
      // The warp's 32 rows are i = 32*ihalf + lane, so which side of the diagonal a block of 32 columns lies on is
      // the same for the whole warp: left of the diagonal block every element is kept, right of it every element
      // is zero (TMEM is not read), and only the diagonal block takes a per-element choice.
      const int ihalf = wq & 1;
      auto emit = [&](const float (&x)[32], int j0) {
        if (!lower) {
          tile_store_row32(hsel ? sm.aqb : sm.aqk, i, j0, x);
        } else if (!hsel) {
          tile_store_row32(sm.aak, i, j0, x);
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(&sm.nmat[i * NROW + j0 + j]) = make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
        }
      };
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        const int j0 = 32 * pp;
        float x[32];
        if (pp > ihalf) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = 0.f;
          emit(x, j0);
          continue;
        }
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm, 32 * wq, 64 * hsel + 32 * pp), rr);   // hsel 0: products with k~, 1: with b~
        tmem_ld_wait();
        if (pp < ihalf) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
          emit(x, j0);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const bool keep = lower ? (j < lane) : (j <= lane);
            x[j] = keep ? __uint_as_float(rr[j]) : 0.f;
          }
          emit(x, j0);
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);

    R7C_STAMP(4);
    // ---- MMA 2: [A_qk; A_ak] v  ->  TMEM columns 128..191 (rows 0..63 = O1, 64..127 = Y)
    if (tid == 0) {
      ok = mbar_wait(&sm.bar_v, par, status, 202) && ok;
      tc_fence_after();
      umma_tile<128, 64, 0, 1>(tmem_addr(tm, 0, 128), smem_u32(sm.aqk), smem_u32(sm.v), false);
      umma_commit(&sm.bar_m2);
      if (keep_for_bwd) {   // A_qk, A_ak, a~ are operands of the backward: copy them out before they are overwritten
        bulk_store(out_tiles + S_AQK * TILE_BYTES, sm.aqk, TILE_BYTES);
        bulk_store(out_tiles + S_AAK * TILE_BYTES, sm.aak, TILE_BYTES);
        bulk_store(out_tiles + S_AT * TILE_BYTES, sm.at, TILE_BYTES);
        bulk_commit();
      }
    }
    // ---- rows of MMA 2 (warps 2-7), then Ainv = X = (I - N)^-1, N = stril(A_ab), by two levels of block
    // inversion:
    //   D. the four 16 x 16 diagonal blocks D_I = (I - N_II)^-1 in fp32, one column per thread, row by row --
    //      the only substitutions, all four side by side (in place in nmat);
    //   1. the two 32 x 32 diagonal blocks in fp32: X_10 = D_1 (N_10 D_0) and X_32 = D_3 (N_32 D_2), 64 threads
    //      each (in place; P = N_IJ D_J passes through the A_qk tile, free once MMA 2 has read it);
    //   2., 3. the last block X_BA = X_B N_BA X_A (A = rows 0..31, B = rows 32..63) as two tensor-core products.
    {
      const int c = tid & 63, I = tid >> 6;
      float* scratch = reinterpret_cast<float*>(sm.aqk);
      if ((c >> 4) == I) {       // step D (while MMA 2 runs)
        float xb[16];
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) xb[rr] = (rr == (c & 15)) ? 1.f : 0.f;
#pragma unroll
        for (int rr = 1; rr < 16; ++rr) {
          const float* nrow = &sm.nmat[(16 * I + rr) * NROW + 16 * I];
          float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;   // entries at or right of the diagonal are 0
#pragma unroll
          for (int jj = 0; jj < (rr + 3) / 4; ++jj) {
            const float4 n = *reinterpret_cast<const float4*>(nrow + 4 * jj);
            p0 += n.x * xb[4 * jj];
            if (4 * jj + 1 < rr) p1 += n.y * xb[4 * jj + 1];
            if (4 * jj + 2 < rr) p2 += n.z * xb[4 * jj + 2];
            if (4 * jj + 3 < rr) p3 += n.w * xb[4 * jj + 3];
          }
          xb[rr] += (p0 + p1) + (p2 + p3);
        }
        __syncwarp((c & 16) ? 0xffff0000u : 0x0000ffffu);   // the 16 columns of a block share a half-warp
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) sm.nmat[(16 * I + rr) * NROW + c] = xb[rr];
      }
      if (warp >= 2) {
        // warps 4-5 take O1 (both column halves), warps 2-3 and 6-7 take Y (one column half each)
        ok = mbar_wait(&sm.bar_m2, par, status, 203) && ok;
        tc_fence_after();
        const int i = (32 * wq + lane) & 63;
        if (wq < 2) {        // warps 4, 5
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            uint32_t rr[32];
            tmem_ld32(tmem_addr(tm, 32 * wq, 128 + 32 * part), rr);
            tmem_ld_wait();
            float x[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
            tile_store_row32(sm.o1, i, 32 * part, x);
          }
        } else {             // warps 2, 3, 6, 7
          uint32_t rr[32];
          tmem_ld32(tmem_addr(tm, 32 * wq, 128 + 32 * hsel), rr);
          tmem_ld_wait();
          float x[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
          tile_store_row32(sm.y, i, 32 * hsel, x);
        }
      }
      // the scratch area: MMA 2 (and the copies of A_qk / A_ak kept for the backward) must be done with it
      ok = mbar_wait(&sm.bar_m2, par, status, 205) && ok;
      if (tid == 0) {
        bulk_wait_read();                  // q~, k~, b~ (and the tiles kept for the backward) have left shared memory
        if (next < n_ch) { load_v(nxt); load_qkb(nxt); }      // MMA 2 has read the v tile; nothing reads q~, k~, b~ any more
      }
      __syncthreads();
      R7C_STAMP(10);
      if (I & 1) {               // step 1: row block I, column block I - 1
        const int cl = tid & 15, r0 = ((tid & 63) >> 4) * 4;
        const int rb = 16 * I, cbk = 16 * (I - 1);
        float* P = scratch + (I >> 1) * 256;
        float col[16], acc[4];
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) col[kk] = sm.nmat[(cbk + kk) * NROW + cbk + cl];     // D_J[:, cl]
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float* nrow = &sm.nmat[(rb + r0 + q) * NROW + cbk];
          float s_ = 0.f;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const float4 n = *reinterpret_cast<const float4*>(nrow + 4 * jj);
            s_ += n.x * col[4 * jj] + n.y * col[4 * jj + 1] + n.z * col[4 * jj + 2] + n.w * col[4 * jj + 3];
          }
          acc[q] = s_;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) P[(r0 + q) * 16 + cl] = acc[q];
        if (I == 1) asm volatile("bar.sync 1, 64;" ::: "memory");
        else        asm volatile("bar.sync 2, 64;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) col[kk] = P[kk * 16 + cl];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float* drow = &sm.nmat[(rb + r0 + q) * NROW + rb];       // D_I is stored in full (zeros above)
          float s_ = 0.f;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const float4 n = *reinterpret_cast<const float4*>(drow + 4 * jj);
            s_ += n.x * col[4 * jj] + n.y * col[4 * jj + 1] + n.z * col[4 * jj + 2] + n.w * col[4 * jj + 3];
          }
          acc[q] = s_;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) sm.nmat[(rb + r0 + q) * NROW + cbk + cl] = acc[q];
      }
      __syncthreads();
      R7C_STAMP(11);
      // steps 2 and 3 on the tensor cores.  With P = diag(X_A, X_B) (the two finished 32 x 32 blocks) and
      // Q = [0 0; N_BA 0], the missing block is X_BA = (P Q P)_BA: T = Q P, then P T, two 64x64x64 products
      // of bf16 operands (N_BA is a small correction: rounding it, X_A, X_B and T to bf16 changes the rounded
      // inverse by less than the rounding of the inverse itself).  P is the Ainv tile with a zero BA
      // quadrant; Q and T pass through the A_qk / A_ak tiles, free since MMA 2.
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int e = tid + 256 * n, row = e >> 3, cc = e & 7;
        const float4 f0 = *reinterpret_cast<const float4*>(&sm.nmat[row * NROW + 8 * cc]);
        const float4 f1 = *reinterpret_cast<const float4*>(&sm.nmat[row * NROW + 8 * cc + 4]);
        const uint4 val = make_uint4(pack_bf16(f0.x, f0.y), pack_bf16(f0.z, f0.w), pack_bf16(f1.x, f1.y), pack_bf16(f1.z, f1.w));
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const bool ba = row >= 32 && cc < 4;
        *reinterpret_cast<uint4*>(sm.ainv + tile_chunk_off(row, cc)) = ba ? zero : val;
        *reinterpret_cast<uint4*>(sm.aqk + tile_chunk_off(row, cc)) = ba ? val : zero;
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      R7C_STAMP(12);
      if (tid == 0) {
        tc_fence_after();
        umma_tile<64, 64, 0, 1>(tmem_addr(tm, 0, 128), smem_u32(sm.aqk), smem_u32(sm.ainv), false);     // T = Q P
        umma_commit(&sm.bar_m4);
      }
      ok = mbar_wait(&sm.bar_m4, par, status, 209) && ok;
      tc_fence_after();
      if (ok) {
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm, 32 * wq, 128 + 32 * hsel), rr);
        tmem_ld_wait();
        if (lane < 16) {        // an M = 64 accumulator lives on the lower 16 lanes of every warp's window
          float x[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
          tile_store_row32(sm.aak, 16 * wq + lane, 32 * hsel, x);
        }
      }
      fence_async_smem();
      tc_fence_before();
      ok = __syncthreads_and(ok);
      if (tid == 0 && ok) {
        tc_fence_after();
        umma_tile<64, 64, 0, 1>(tmem_addr(tm, 0, 128), smem_u32(sm.ainv), smem_u32(sm.aak), false);     // P T
        umma_commit(&sm.bar_m5);
      }
      ok = mbar_wait(&sm.bar_m5, par, status, 210) && ok;
      tc_fence_after();
      if (ok && hsel == 0) {      // rows 32..63, columns 0..31: the BA quadrant of Ainv
        uint32_t rr[32];
        tmem_ld32(tmem_addr(tm, 32 * wq, 128), rr);
        tmem_ld_wait();
        if (lane < 16 && wq >= 2) {
          float x[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
          tile_store_row32(sm.ainv, 16 * wq + lane, 0, x);
        }
      }
      R7C_STAMP(13);
    }
    R7C_STAMP(5);
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);

    R7C_STAMP(6);
    // ---- MMA 3: W = Ainv a~ (lower lane halves), U = Ainv Y (upper lane halves) -> TMEM columns 0..63
    if (tid == 0) {
      if (ok && next < n_ch) load_w(nxt);      // the scratch area in the A_qk tile is free again
      tc_fence_after();
      umma_tile<64, 64, 0, 1>(tmem_addr(tm, 0, 0), smem_u32(sm.ainv), smem_u32(sm.at), false);
      umma_tile<64, 64, 0, 1>(tmem_addr(tm, 16, 0), smem_u32(sm.ainv), smem_u32(sm.y), false);
      umma_commit(&sm.bar_m3);
      bulk_store(out_tiles + S_AQB * TILE_BYTES, sm.aqb, TILE_BYTES);
      bulk_store(out_tiles + S_O1 * TILE_BYTES, sm.o1, TILE_BYTES);
      if (keep_for_bwd) bulk_store(out_tiles + S_AINV * TILE_BYTES, sm.ainv, TILE_BYTES);
      bulk_commit();
    }
    ok = mbar_wait(&sm.bar_m3, par, status, 204) && ok;
    tc_fence_after();
    R7C_STAMP(7);

    {
      // W -> the A_ak tile (free since MMA 2), U -> the Y tile (free: MMA 3 has completed)
      const int i = 16 * wq + (lane & 15);
      unsigned char* dst = lane < 16 ? sm.aak : sm.y;
      uint32_t rr[32];
      tmem_ld32(tmem_addr(tm, 32 * wq, 32 * hsel), rr);
      tmem_ld_wait();
      float x[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(rr[j]);
      tile_store_row32(dst, i, 32 * hsel, x);
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    R7C_STAMP(8);
    if (tid == 0 && ok) {
      bulk_store(out_tiles + S_W * TILE_BYTES, sm.aak, TILE_BYTES);
      bulk_store(out_tiles + S_U * TILE_BYTES, sm.y, TILE_BYTES);
      bulk_commit();
      // MMA 3 has read a~ (and its copy for the backward left shared memory long ago): the next raw a may land
      if (next < n_ch) load_a(nxt);
    }
    R7C_STAMP(9);
  }
  if (tid == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 256);
#undef R7C_STAMP
}

// ---------------------------------------------------------------------------------------------
// scan kernel: grid = B*H, 256 threads, chunks in order, fp32 state in TMEM.  Warp w reads TMEM lanes
// 32*(w&3)..; the two warps that share a lane window take 32 of the 64 columns each (hsel = w>>2).
// ---------------------------------------------------------------------------------------------
// Operand tiles come in two groups, each requested again the moment the MMAs that read it have completed.
// STAGES = 1 (single-buffered, 11 tiles = 88 KB): two CTAs (two sequences) share an SM, the choice when
// there are more sequences than SMs; U and O1, which are only added row by row, do not enter shared
// memory: every thread fetches its row into registers at the top of a chunk.  STAGES = 2 (21 tiles): one
// CTA per SM with the groups of chunk c + 2 requested during chunk c and U, O1 staged with group 1, for
// the case of few sequences, where nothing else on the SM covers a load latency.
template <int STAGES> struct ScanGroup1 {
  unsigned char qt[TILE_BYTES], kt[TILE_BYTES];   // read by step a: q~, k~ (adjacent slots)
  unsigned char w[TILE_BYTES], v[TILE_BYTES];     //                 W, v (TMA)
};
template <> struct ScanGroup1<2> {
  unsigned char qt[TILE_BYTES], kt[TILE_BYTES];
  unsigned char o1[TILE_BYTES], w[TILE_BYTES], u[TILE_BYTES];   // adjacent slots O1, W, U: one copy
  unsigned char v[TILE_BYTES];
};
struct ScanGroup2 {
  unsigned char bt[TILE_BYTES], aqb[TILE_BYTES];  // read by step c: b~, A_qb (adjacent slots)
};
template <int STAGES>
struct ScanSmem {
  ScanGroup1<STAGES> g1[STAGES];
  ScanGroup2 g2[STAGES];
  unsigned char ht[TILE_BYTES];             // h~0 as bf16, [k][v]
  unsigned char sa[TILE_BYTES];             // sa as bf16, [token][v]
  unsigned char xt[TILE_BYTES];             // X = h~0 + k~^T v + b~^T sa as bf16 (kept for the backward)
  unsigned char ot[2][TILE_BYTES];          // output rows of a chunk, staged for a TMA store
  uint64_t bar_g1[STAGES], bar_g2[STAGES], bar_a, bar_c;
  uint32_t tmem_base;
};

template <int STAGES, bool PACKED>
__global__ void __launch_bounds__(256, 3 - STAGES)
r7c_scan_fwd_kernel(const __grid_constant__ CUtensorMap tmap_v, const unsigned char* __restrict__ ws_tiles,
                    const float* __restrict__ ws_aux, int tiles_per_chunk, unsigned char* __restrict__ bwd_tiles,
                    const float* __restrict__ h0, int n_state, const __grid_constant__ CUtensorMap tmap_o,
                    int write_o, float* __restrict__ ht, bf16* __restrict__ o_rows, SeqView sv, int H, int NT_slots,
                    TokLayout lay, int* status, long long* dbg) {
#ifdef RWKVB200_DEVTOOLS
#define R7C_STAMP(n) do { if (dbg && tid == 0 && blockIdx.x == gridDim.x / 2 && c == 2) dbg[n] = clock64(); } while (0)
#else
#define R7C_STAMP(n) do {} while (0)
#endif
  extern __shared__ unsigned char smem_raw[];
  ScanSmem<STAGES>& sm =
      *reinterpret_cast<ScanSmem<STAGES>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wq = warp & 3, hsel = warp >> 2, c0 = 32 * hsel;
  const int unit = blockIdx.x, bi = unit / H, hi = unit % H;
  const size_t ch0 = (size_t)unit * NT_slots;
  const int Tn = sv.length<PACKED>(bi), tb = sv.first<PACKED>(bi), brow = sv.row<PACKED>(bi);
  const int NT = (Tn + L - 1) / L;           // chunks of this sequence (at least one)
  const int row = 16 * wq + (lane & 15);     // state row k (lanes 0-15) or token row i (lanes 16-31)
  const bool state_lane = lane < 16;
  // With one CTA per SM the single-thread jobs of a chunk lie on the chain from chunk to chunk, and each
  // bulk copy costs its issuing thread about a hundred cycles: they go to the first threads of four warps and
  // run side by side (-12 % per chunk).  Thread 0 issues the MMAs (with the first threads of warps 1 and 2, one
  // accumulator each), ld_thread requests operand tiles,
  // st_thread copies sa and h~0 out for the backward, out_thread copies X and the output rows out.  Bulk-copy
  // groups belong to the thread that committed them, so each storing thread waits for its own copies.  With
  // two CTAs per SM the other CTA fills such gaps and thread 0 keeps all four jobs.
  constexpr bool SPREAD = STAGES == 2;
  const bool ld_thread = tid == (SPREAD ? 32 : 0), st_thread = tid == (SPREAD ? 64 : 0),
             out_thread = tid == (SPREAD ? 96 : 0);

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&sm.bar_g1[i], 1); mbar_init(&sm.bar_g2[i], 1); }
    // with one CTA per SM each accumulator of an MMA group has its own issuing thread (one thread issues an
    // MMA about every 80 cycles, the tensor pipe takes them faster), and a group completes with all arrivals
    mbar_init(&sm.bar_a, SPREAD ? 3 : 1); mbar_init(&sm.bar_c, SPREAD ? 2 : 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;
  const uint32_t tm_p1 = tmem_addr(tm, 32 * wq, c0), tm_p2 = tmem_addr(tm, 32 * wq, 64 + c0);

  auto issue_g1 = [&](int c) {      // ld_thread (thread 0 for the first chunks)
    const unsigned char* tiles = ws_tiles + (ch0 + c) * (size_t)tiles_per_chunk * TILE_BYTES;
    ScanGroup1<STAGES>& g = sm.g1[c % STAGES];
    uint64_t* bar = &sm.bar_g1[c % STAGES];
    mbar_expect_tx(bar, (STAGES == 2 ? 6 : 4) * TILE_BYTES);
    bulk_load(g.qt, tiles + S_QT * TILE_BYTES, 2 * TILE_BYTES, bar);
    if constexpr (STAGES == 2) bulk_load(g.o1, tiles + S_O1 * TILE_BYTES, 3 * TILE_BYTES, bar);
    else                       bulk_load(g.w, tiles + S_W * TILE_BYTES, TILE_BYTES, bar);
    tma_load_4d(g.v, &tmap_v, bar, 0, tb + c * L, hi, brow);
  };
  auto issue_g2 = [&](int c) {      // ld_thread (thread 0 for the first chunks)
    const unsigned char* tiles = ws_tiles + (ch0 + c) * (size_t)tiles_per_chunk * TILE_BYTES;
    uint64_t* bar = &sm.bar_g2[c % STAGES];
    mbar_expect_tx(bar, 2 * TILE_BYTES);
    bulk_load(sm.g2[c % STAGES].bt, tiles + S_BT * TILE_BYTES, 2 * TILE_BYTES, bar);
  };
  if (tid == 0) {
    for (int c = 0; c < STAGES && c < NT; ++c) { issue_g1(c); issue_g2(c); }
  }

  // ---- initial state: h~0 = e^{gref(chunk 0)} h0, fp32 into TMEM (lower lane halves of P2), bf16 into ht
  {
    float x[32];
#pragma unroll
    for (int vv = 0; vv < 32; ++vv) x[vv] = 0.f;
    if (state_lane) {
      const float e0 = ws_aux[ch0 * AUX_FLOATS + row];
      if (n_state > 0) {
        const float* S = h0 + (size_t)(n_state == 1 ? hi : unit) * 4096;   // S[v][k], h[k][v] = S[v][k]
#pragma unroll
        for (int vv = 0; vv < 32; ++vv) x[vv] = e0 * S[(c0 + vv) * 64 + row];
      }
      tile_store_row32(sm.ht, row, c0, x);
    }
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(x[j]);
    tmem_st32(tm_p2, r);
    tmem_st_wait();
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  bool ok = true;
  for (int c = 0; c < NT && ok; ++c) {
    const int t0 = c * L;
    R7C_STAMP(48);
    // this thread's row of U (state lanes) or O1 (token lanes), straight from the workspace
    uint4 addrow[4];
    if constexpr (STAGES == 1) {
      const unsigned char* tile = ws_tiles + ((ch0 + c) * (size_t)tiles_per_chunk + (state_lane ? S_U : S_O1)) * TILE_BYTES;
#pragma unroll
      for (int q = 0; q < 4; ++q) addrow[q] = __ldg(reinterpret_cast<const uint4*>(tile + tile_chunk_off(row, 4 * hsel + q)));
      if (c + 1 < NT && hsel == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(tile + (size_t)tiles_per_chunk * TILE_BYTES + row * 128));
    }
    // decay factors needed at the end of this chunk, fetched early
    // (applied one after the other: their product can underflow float32 where neither factor does)
    float scale = 1.f, scale_next = 1.f;
    if (state_lane) {
      scale = ws_aux[(ch0 + c) * AUX_FLOATS + 64 + row];                       // e^{glast-gref} of this chunk
      if (c + 1 < NT) scale_next = ws_aux[(ch0 + c + 1) * AUX_FLOATS + row];    // e^{gref} of the next chunk
    }
    // (a) SA = W h~0, QH = q~ h~0 (P1);  H += k~^T v (P2 lower)
    if (lane == 0 && warp < (SPREAD ? 3 : 1)) {
      ScanGroup1<STAGES>& g = sm.g1[c % STAGES];
      ok = mbar_wait(&sm.bar_g1[c % STAGES], (c / STAGES) & 1, status, 211);
      R7C_STAMP(49);
      if (ok) {
        tc_fence_after();
        if (!SPREAD || warp == 0) umma_tile<64, 64, 0, 1>(tmem_addr(tm, 0, 0), smem_u32(g.w), smem_u32(sm.ht), false);
        if (!SPREAD || warp == 1) umma_tile<64, 64, 0, 1>(tmem_addr(tm, 16, 0), smem_u32(g.qt), smem_u32(sm.ht), false);
        if (!SPREAD || warp == 2) umma_tile<64, 64, 1, 1>(tmem_addr(tm, 0, 64), smem_u32(g.kt), smem_u32(g.v), true);
        umma_commit(&sm.bar_a);
      }
    }
    ok = ok && mbar_wait(&sm.bar_a, c & 1, status, 212);
    tc_fence_after();
    R7C_STAMP(50);
    // group 1 has been read by the MMAs: request the next (the staged O1 / U rows are still to be read)
    if (STAGES == 1 && ld_thread && ok && c + STAGES < NT) issue_g1(c + STAGES);
    float keep[32];     // token lanes: q~ h~0 + O1
    if constexpr (STAGES == 2) {      // the staged O1 / U rows: observe the arrival of group 1 before reading them
      ok = ok && mbar_wait(&sm.bar_g1[c % STAGES], (c / STAGES) & 1, status, 215);
      const unsigned char* tile = state_lane ? sm.g1[c % STAGES].u : sm.g1[c % STAGES].o1;
#pragma unroll
      for (int q = 0; q < 4; ++q) addrow[q] = *reinterpret_cast<const uint4*>(tile + tile_chunk_off(row, 4 * hsel + q));
    }
    if (ok) {
      uint32_t r[32];
      tmem_ld32(tm_p1, r);
      tmem_ld_wait();
      float add[32];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 u = addrow[q];
        add[8 * q + 0] = bf16_lo(u.x); add[8 * q + 1] = bf16_hi(u.x);
        add[8 * q + 2] = bf16_lo(u.y); add[8 * q + 3] = bf16_hi(u.y);
        add[8 * q + 4] = bf16_lo(u.z); add[8 * q + 5] = bf16_hi(u.z);
        add[8 * q + 6] = bf16_lo(u.w); add[8 * q + 7] = bf16_hi(u.w);
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) keep[j] = __uint_as_float(r[j]) + add[j];
      if (state_lane) tile_store_row32(sm.sa, row, c0, keep);   // sa = W h~0 + U
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (STAGES == 2 && ld_thread && ok && c + STAGES < NT) issue_g1(c + STAGES);
    if (bwd_tiles && st_thread && ok) {   // the backward needs sa and h~0 of every chunk
      unsigned char* dst = bwd_tiles + (ch0 + c) * (size_t)tiles_per_chunk * TILE_BYTES;
      bulk_store(dst + S_SA * TILE_BYTES, sm.sa, TILE_BYTES);
      bulk_store(dst + S_H0 * TILE_BYTES, sm.ht, TILE_BYTES);
      bulk_commit();
    }
    // (c) H += b~^T sa (P2 lower);  OQ = A_qb sa (P2 upper)
    R7C_STAMP(51);
    if (lane == 0 && warp < (SPREAD ? 2 : 1) && ok) {
      ScanGroup2& g = sm.g2[c % STAGES];
      ok = mbar_wait(&sm.bar_g2[c % STAGES], (c / STAGES) & 1, status, 214);
      R7C_STAMP(52);
      if (ok) {
        tc_fence_after();
        if (!SPREAD || warp == 0) umma_tile<64, 64, 1, 1>(tmem_addr(tm, 0, 64), smem_u32(g.bt), smem_u32(sm.sa), true);
        if (!SPREAD || warp == 1) umma_tile<64, 64, 0, 1>(tmem_addr(tm, 16, 64), smem_u32(g.aqb), smem_u32(sm.sa), false);
        umma_commit(&sm.bar_c);
      }
    }
    ok = ok && mbar_wait(&sm.bar_c, c & 1, status, 213);
    tc_fence_after();
    R7C_STAMP(53);
    if (ld_thread && ok && c + STAGES < NT) issue_g2(c + STAGES);     // group 2 has been read
    if (bwd_tiles) {                                  // ht / sa are rewritten below and in the next chunk
      if (st_thread) bulk_wait_read();
      __syncthreads();
    }
    R7C_STAMP(54);
    if (ok) {
      const bool last = c + 1 == NT;
      uint32_t r[32];
      tmem_ld32(tm_p2, r);
      tmem_ld_wait();
      float x[32];
      if (state_lane) {
        if (bwd_tiles) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]);
          tile_store_row32(sm.xt, row, c0, x);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) { x[j] = (__uint_as_float(r[j]) * scale) * scale_next; r[j] = __float_as_uint(x[j]); }
        if (!last) {
          tile_store_row32(sm.ht, row, c0, x);
        } else if (ht) {
          float* S = ht + (size_t)unit * 4096;
#pragma unroll
          for (int j = 0; j < 32; ++j) S[(c0 + j) * 64 + row] = x[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]) + keep[j];
        if (write_o) tile_store_row32(sm.ot[c & 1], row, c0, x);
      }
      tmem_st32(tm_p2, r);   // state lanes: rescaled state; token lanes: unchanged
      tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    R7C_STAMP(55);
    if (bwd_tiles && out_thread && ok) {
      bulk_store(bwd_tiles + ((ch0 + c) * (size_t)tiles_per_chunk + S_X) * TILE_BYTES, sm.xt, TILE_BYTES);
      bulk_commit();
    }
    if (write_o && ok) {
      if (PACKED && t0 + L > Tn) {  // the last rows of the box belong to the next sequence: row by row
        store_tile_rows<256>(o_rows + brow * lay.sb + hi * lay.sh + (long long)(tb + t0) * lay.st, lay.st,
                             sm.ot[c & 1], Tn - t0, tid);
      } else if (out_thread) {           // rows past the end of the tensor are clipped by the TMA store
        tma_store_4d(&tmap_o, sm.ot[c & 1], 0, tb + t0, hi, brow);
        bulk_commit();
        bulk_wait_read_1();              // the buffer of the previous chunk is free again
      }
    }
    R7C_STAMP(56);
  }
#undef R7C_STAMP
  if (st_thread || out_thread) bulk_wait_all();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 128);
}

}  // namespace r7c

int launch_rwkv7_chunked_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                             const float* h0, int n_state, void* o, float* ht, void* workspace,
                             int B, int Tn, int H, int head_first, bool keep_for_bwd, cudaStream_t st,
                             const int* seq_start, const int* seq_len, int T_total, bool fused, int phases) {
  using namespace r7c;
  typedef __nv_bfloat16 bf16;
  if (fused && seq_start) return RWKVB200_E_UNSUPPORTED;
  const SeqView sv{seq_start, seq_len, Tn};
  const int mapB = seq_start ? 1 : B, mapT = seq_start ? T_total : Tn;   // shape of the token tensors
  int* status = device_status_ptr();
  if (!status) { last_cuda_error_slot() = 99999; return RWKVB200_E_CUDA; }
  CUtensorMap tmap_v, tmap_o;
  int e = make_token_tensor_map(&tmap_v, v, mapB, mapT, H, head_first);
  if (e) return e;
  e = make_token_tensor_map(&tmap_o, o ? o : v, mapB, mapT, H, head_first);   // unused when o is NULL
  if (e) return e;
  CUtensorMap tmap_in[5];
  const void* ins[5] = {r, w, k, a, b};
  for (int i = 0; i < 5; ++i) {
    e = make_token_tensor_map(&tmap_in[i], ins[i], mapB, mapT, H, head_first);
    if (e) return e;
  }
  const int NT = num_chunks(Tn);
  const int tpc = keep_for_bwd ? (int)ALL_TILES : (int)FWD_TILES;
  Workspace ws = carve(workspace, B, Tn, H, tpc);
  TokLayout lay(mapT, H, head_first);
  if (phases & PHASE_PREPARE) {
    if (cuda_ok(cudaMemsetAsync(ws.flags, 0, (size_t)B * H * sizeof(int), st))) return RWKVB200_E_CUDA;
    const int smem = (int)sizeof(IntraSmem) + 1024;
    ProfScope prof("r7c_intra_fwd_kernel", st);
    const int n_ch = B * H * NT;
    int dev = 0, sms = 0;
    if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))
      return RWKVB200_E_CUDA;
    const int grid = n_ch < 2 * sms ? n_ch : 2 * sms;     // persistent: two CTAs per SM
#define R7C_LAUNCH_INTRA(P, F)                                                                                     \
    do {                                                                                                           \
      if (cuda_ok(cudaFuncSetAttribute(r7c_intra_fwd_kernel<P, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))) \
        return RWKVB200_E_CUDA;                                                                                    \
      r7c_intra_fwd_kernel<P, F><<<grid, 256, smem, st>>>((const bf16*)r, (const bf16*)w, (const bf16*)k,         \
          (const bf16*)a, (const bf16*)b, tmap_in[0], tmap_in[1], tmap_in[2], tmap_in[3], tmap_in[4], tmap_v,      \
          ws.tiles, ws.aux, ws.flags, tpc, keep_for_bwd ? 1 : 0, sv, H, NT, n_ch, lay, status,                    \
          debug_stamp_buffer());                                                                                   \
    } while (0)
    if (seq_start) R7C_LAUNCH_INTRA(true, false);
    else if (fused) R7C_LAUNCH_INTRA(false, true);
    else R7C_LAUNCH_INTRA(false, false);
#undef R7C_LAUNCH_INTRA
  }
  e = check_launch();
  if (e || !(phases & PHASE_SCAN)) return e;
  {
    int dev = 0, sms = 0;
    if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))
      return RWKVB200_E_CUDA;
    ProfScope prof("r7c_scan_fwd_kernel", st);
    // more sequences than SMs: two single-buffered CTAs per SM; else one double-buffered CTA per SM
#define R7C_LAUNCH_SCAN(S, P)                                                                                      \
    do {                                                                                                           \
      const int smem = (int)sizeof(ScanSmem<S>) + 1024;                                                            \
      if (cuda_ok(cudaFuncSetAttribute(r7c_scan_fwd_kernel<S, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))) \
        return RWKVB200_E_CUDA;                                                                                    \
      r7c_scan_fwd_kernel<S, P><<<B * H, 256, smem, st>>>(tmap_v, ws.tiles, ws.aux, tpc,                           \
          keep_for_bwd ? ws.tiles : nullptr, h0, n_state, tmap_o, o ? 1 : 0, ht, (bf16*)o, sv, H, NT, lay, status, \
          debug_stamp_buffer());                                                                                   \
    } while (0)
    if (B * H > sms) { if (seq_start) R7C_LAUNCH_SCAN(1, true); else R7C_LAUNCH_SCAN(1, false); }
    else             { if (seq_start) R7C_LAUNCH_SCAN(2, true); else R7C_LAUNCH_SCAN(2, false); }
#undef R7C_LAUNCH_SCAN
  }
  e = check_launch();
  if (e || fused) return e;      // fused producers bound |g| by e^{-1/2}: no unit can be marked
  // units whose decay left the range of the scaled operands: exact float32 recurrence over them (the
  // kernel's other CTAs leave at once)
  if (o || ht) {
    const UnitSel sel{ws.flags, seq_start, seq_len, 0};
    e = launch_rwkv7_rec_fwd(r, w, k, v, a, b, h0, n_state, o, ht, nullptr, R7_CKPT, B, Tn, H, RWKVB200_BF16,
                             head_first, st, &sel, seq_start ? T_total : 0);
  }
  return e;
}

}  // namespace rwkvb200
