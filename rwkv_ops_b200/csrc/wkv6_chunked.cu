// RWKV6 wkv on tcgen05: chunked forward and backward with split-precision operands.
//
// Maths (one (batch, head), chunk of L = 64 tokens, S is the [K][V] state; reference:
// rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:63-80):
//   g = -exp(w), gi / ge inclusive / exclusive prefix sums of g inside the chunk, gref = gi at token 31,
//   glast = gi at token 63,  r~ = r e^{ge-gref},  k~ = k e^{gref-gi},  S~0 = diag(e^{gref}) S0
//   A = stril(r~ k~^T) + diag(sum_k r u k)
//   y   = r~ S~0 + A v
//   S_L = diag(e^{glast-gref}) (S~0 + k~^T v)
// Backward (dy, dS_L given; dS^ = diag(e^{glast-gref}) dS_L):
//   dv = A^T dy + k~ dS^        dA = dy v^T (strictly lower part -> r~, k~; diagonal -> the u term)
//   dr~ = dy S~0^T + stril(dA) k~      dk~ = stril(dA)^T r~ + v dS^^T      dS0 = diag(e^{gref}) (r~^T dy + dS^)
//   dge = dr~ r~,  dgi = -dk~ k~,  dglast = sum_v dS_L S_L,  dg_j = sum_{i>j} dge_i + sum_{i>=j} dgi_i + dglast
//   (computed without the cancellation between dglast and the state part of dgi: with X = v dS^^T,
//    dg_j = sum_{i>j} dge_i - sum_{i>=j} (stril(dA)^T r~)_i k~_i + sum_v dS^ S~0 + sum_{i<j} X_i k~_i)
//   dw = dg g;   with dd_i = dy_i . v_i:  dr += dd u k,  dk += dd r u,  du += sum_i dd r k
//
// Precision.  The parity bar for float32 inputs is 1e-4, which bf16 operands cannot meet, so every
// operand X is split as X = hi + lo (two bf16 tiles) and every product is the three tensor-core
// products hi*hi + hi*lo + lo*hi accumulated in fp32 TMEM (relative error ~2^-16 per term).
//
// One CTA of 256 threads per (batch, head) walks the chunks in order; the fp32 state (its gradient in the
// backward) lives in the registers of the threads that own its rows, the products in TMEM, and nothing but
// the inputs and outputs touches HBM in the forward pass (plus, for the backward, the fp32 state at every
// chunk boundary).  The raw rows of the next chunk arrive by TMA while the current chunk is worked on.
// Tile and TMEM conventions are those of tc.cuh.
#include "common.cuh"
#include "tc.cuh"

namespace rwkvb200 {
namespace w6c {

using namespace tc;
typedef __nv_bfloat16 bf16;

constexpr int L = 64;
constexpr int NROW = 68;
// All decay sums are kept in units of log 2 (tc::ex2: a scale factor is one instruction); nothing is clamped.
constexpr float EXP2_FLOOR = -126.f;      // 2^x below this is flushed to zero anyway
// The scaled operands carry e^{+-(gi - gref)}, whose exponent reaches the sum of |g| over half a chunk.  Range
// alone would allow about 60 (every factor, and the low half of every split operand, stays a normal number),
// but the decay gradient is a difference of prefix sums that cancel the more the faster the state decays:
// measured against a float64 oracle with every channel decaying at the same rate, its relative error grows
// from 2e-5 at |g| = 0.3 per token to 1e-4 (the parity bar) at |g| = 1.55.  DECAY_LIMIT = 45 (|g| <= 1.4 per
// token, w <= 0.34) keeps it below the bar.  A (batch, head) unit that exceeds the limit in any channel of any
// chunk is marked by the forward kernel and recomputed by the float32 recurrence (wkv6.cu), forward and
// backward, so that no value computed from a clamped exponent is ever returned.
constexpr float DECAY_LIMIT = 45.f;
// Sequences shorter than this take the recurrence as well (marked in the same flags): with two or three tokens and
// fast decays the decay gradient is the small remainder of pair sums that cancel (every pair of tokens enters the
// row sums of dr~ r~ and the column sums of dk~ k~ with opposite signs, computed by different tensor-core
// products), and the 2^-17 roundings of the split operands reached 5e-4 of dw there; the recurrence costs nothing
// at that length.
constexpr int SHORT_SEQ = 8;

// two values as packed bf16 pairs hi and lo with x = hi + lo (+ an error of about 2^-17 |x|)
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x0, x1);
  lo = pack_bf16(x0 - bf16_lo(hi), x1 - bf16_hi(hi));
}
// write 4 consecutive values (columns col .. col+3, col a multiple of 4) of `row` into a hi and a lo tile
__device__ __forceinline__ void store_split4(unsigned char* hi_t, unsigned char* lo_t, int row, int col, float4 x) {
  uint2 h, l;
  split_pair(x.x, x.y, h.x, l.x);
  split_pair(x.z, x.w, h.y, l.y);
  const uint32_t off = tile_off(row, col);
  *reinterpret_cast<uint2*>(hi_t + off) = h;
  *reinterpret_cast<uint2*>(lo_t + off) = l;
}
// write 32 consecutive fp32 values of `row` (columns col0 .., col0 a multiple of 8) into a hi and a lo tile
__device__ __forceinline__ void store_split_row32(unsigned char* hi_t, unsigned char* lo_t, int row, int col0,
                                                  const float* x) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 h, l;
    split_pair(x[8 * c + 0], x[8 * c + 1], h.x, l.x);
    split_pair(x[8 * c + 2], x[8 * c + 3], h.y, l.y);
    split_pair(x[8 * c + 4], x[8 * c + 5], h.z, l.z);
    split_pair(x[8 * c + 6], x[8 * c + 7], h.w, l.w);
    const uint32_t off = tile_chunk_off(row, (col0 >> 3) + c);
    *reinterpret_cast<uint4*>(hi_t + off) = h;
    *reinterpret_cast<uint4*>(lo_t + off) = l;
  }
}

// D (+)= X Y with X = xh + xl, Y = yh + yl (lo tile = hi tile + TILE_BYTES): hi*hi + hi*lo + lo*hi
template <int M, int N, int A_MN, int B_MN>
__device__ __forceinline__ void umma_split(uint32_t tmem_d, uint32_t a_hi, uint32_t b_hi, bool accumulate) {
  umma_tile<M, N, A_MN, B_MN>(tmem_d, a_hi, b_hi, accumulate);
  umma_tile<M, N, A_MN, B_MN>(tmem_d, a_hi, b_hi + TILE_BYTES, true);
  umma_tile<M, N, A_MN, B_MN>(tmem_d, a_hi + TILE_BYTES, b_hi, true);
}

// Row `lr` (0..15) of a warp's 16 x 32 block of a 64 x 64 product that is kept strictly below the diagonal, the
// diagonal itself set to `diag`, split and stored.  Where the diagonal crosses the block depends on the warp alone:
// left of column JLO (of the block's 32) every element is kept, from JLO + 16 on every element is zero, and only
// the 16 columns between take a per-element choice.  JLO = 32: the whole block is kept; JLO = -16: all zero
// (`rr` is not read).
template <int JLO>
__device__ __forceinline__ void store_masked_row(const uint32_t (&rr)[32], int lr, float diag, unsigned char* hi_t,
                                                 int row, int col0) {
  float x[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (j < JLO) x[j] = __uint_as_float(rr[j]);
    else if (j >= JLO + 16) x[j] = 0.f;
    else x[j] = (j - JLO) < lr ? __uint_as_float(rr[j]) : ((j - JLO) == lr ? diag : 0.f);
  }
  store_split_row32(hi_t, hi_t + TILE_BYTES, row, col0, x);
}
// the same for a warp whose rows are 16*wq .. and whose columns are 32*hsel ..; all lanes of the warp call it
__device__ __forceinline__ void load_store_masked_row(uint32_t taddr, int wq, int hsel, int lr, float diag,
                                                      unsigned char* hi_t, int row, bool active) {
  const int jlo = 16 * wq - 32 * hsel;
  uint32_t rr[32];
  if (jlo < 0) {
    if (active) store_masked_row<-16>(rr, lr, diag, hi_t, row, 32 * hsel);
    return;
  }
  tmem_ld32(taddr, rr);
  tmem_ld_wait();
  if (!active) return;
  if (jlo >= 32) store_masked_row<32>(rr, lr, diag, hi_t, row, 32 * hsel);
  else if (jlo == 16) store_masked_row<16>(rr, lr, diag, hi_t, row, 32 * hsel);
  else store_masked_row<0>(rr, lr, diag, hi_t, row, 32 * hsel);
}

__device__ __forceinline__ long long state_row(const int32_t* smap, int n_state, int bi) {
  if (n_state == 1) return 0;
  if (!smap) return bi;
  int m = smap[bi];
  return m < 0 ? 0 : (m >= n_state ? n_state - 1 : m);
}

// Where the tokens of a unit's sequence lie.  Dense batches: row bi of [B][T][H][64], Tn tokens.  Packed batches
// (PACKED): the sequences lie end to end in one row [1][total][H][64]; sequence bi is tokens start[bi] ..
// start[bi] + len[bi] - 1, and the rows of a chunk past the end of the sequence belong to the next one: they are
// read as zeros and never stored.
struct Seqs {
  const int32_t* start;
  const int32_t* len;
  int nts;      // chunk-boundary state slots per unit in `states` (chunks of the longest sequence + 1)
};

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
struct FwdSmem {
  unsigned char rt[2][TILE_BYTES];    // r~ hi, lo      [token][k]
  unsigned char kt[2][TILE_BYTES];    // k~ hi, lo      [token][k]
  unsigned char vt[2][TILE_BYTES];    // v hi, lo       [token][v]
  unsigned char at[2][TILE_BYTES];    // A hi, lo       [token i][token j]
  unsigned char st[2][TILE_BYTES];    // S~0 hi, lo     [k][v]
  float gs[L * NROW];                 // gi - gref (prefix of g relative to the reference point); later the staged y rows
  float qtot[4][64];
  float dgs[64];                      // sum_k r u k per token
  uint64_t bar_1, bar_2, bar_in;
  uint32_t tmem_base;
  int handoff_ok, next_item;
};

// The raw r, k, v, w rows of a chunk (64 rows of 64 elements each) arrive by TMA in the space of the tile
// pairs they are turned into (r -> rt, k -> kt, v -> vt, w -> at), requested for the next chunk as soon as
// the last MMA of the current one has read those tiles; a thread reads its elements, all threads meet at a
// barrier, and then the split tiles are written over the raw rows.
// S0 of every chunk (and the final state) goes to `states` [B*H][NT+1][64][64] when it is not NULL.
template <typename T, bool PACKED>
__global__ void __launch_bounds__(256, 2)
wkv6c_fwd_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ w,
                 const float* __restrict__ u, const float* __restrict__ s0, int n_state,
                 const int32_t* __restrict__ smap, T* __restrict__ y, float* __restrict__ sT,
                 float* __restrict__ states, int* __restrict__ flags, const __grid_constant__ CUtensorMap tmap_r,
                 const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                 const __grid_constant__ CUtensorMap tmap_w, int Tn_dense, int H, Seqs seqs, int n_units, int parts,
                 float* __restrict__ handoff, int* __restrict__ handoff_flags, int* status, long long* dbg) {
#ifdef RWKVB200_DEVTOOLS
#define W6C_STAMP(n) do { if (dbg && tid == 0 && item == gridDim.x / 2 && c == 2) dbg[n] = clock64(); } while (0)
#else
#define W6C_STAMP(n) do {} while (0)
#endif
  extern __shared__ unsigned char smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wq = warp & 3, hsel = warp >> 2;
  const long long tstride = (long long)H * HS;
  const int srow = 16 * wq + (lane & 15);     // state row k (upper lane halves) / token row (lower lane halves)
  const bool tok_lane = lane < 16;            // lower lane halves hold token rows, upper halves state rows

  if (tid == 0) {
    // MMA batch 1 has three accumulators and three issuing threads (0, 32, 64) and completes with all arrivals
    mbar_init(&sm.bar_1, 3); mbar_init(&sm.bar_2, 1); mbar_init(&sm.bar_in, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;
  // TMEM: columns 0..63 lower halves = r~ k~^T; columns 64..127 lower halves = y, upper halves = k~^T v
  const uint32_t tm_a = tmem_addr(tm, 32 * wq, 32 * hsel);
  const uint32_t tm_ys = tmem_addr(tm, 32 * wq, 64 + 32 * hsel);

  const int c4 = tid & 15;
  const T* raw_r = reinterpret_cast<const T*>(sm.rt[0]);
  const T* raw_k = reinterpret_cast<const T*>(sm.kt[0]);
  const T* raw_v = reinterpret_cast<const T*>(sm.vt[0]);
  const T* raw_w = reinterpret_cast<const T*>(sm.at[0]);

  // Work items.  parts == 1: an item is a (batch, head) unit and the grid has one CTA per unit.  parts > 1 (more
  // units than the two CTAs per SM can hold at once): every unit is `parts` items, consecutive stretches of its
  // chunks, on a persistent grid whose free CTAs take the next item from a counter (handoff_flags[n_units]); all
  // first stretches come first in that order, so when a stretch is taken the one before it has been taken
  // already, by a CTA that is running, and the state travels between them through `handoff` (handoff_flags[unit]
  // counts the stretches of the unit that are done).  Shorter items even out the last round of CTAs (512 units
  // on 296 slots: 1.75 unit times instead of 2).
  const int n_items = parts * n_units;
  bool ok = true;
  uint32_t n_done = 0;      // chunks this CTA has worked on: every barrier completes once per chunk
  for (bool first = true; ok; first = false) {
  if (parts > 1) {
    if (tid == 0) sm.next_item = atomicAdd(handoff_flags + n_units, 1);
    __syncthreads();
  } else if (!first) {
    break;
  }
  const int item = parts > 1 ? sm.next_item : (int)blockIdx.x;
  if (item >= n_items) break;
  const int unit = item % n_units, part = item / n_units;
  const int bi = unit / H, hi = unit % H;
  const int Tn = PACKED ? seqs.len[bi] : Tn_dense;
  const int tok0 = PACKED ? seqs.start[bi] : 0;       // first token row of the sequence in its batch row
  const int brow = PACKED ? 0 : bi;
  const long long base = (((long long)brow * Tn_dense + tok0) * H + hi) * HS;   // Tn_dense: rows per batch row
  const int NT = (Tn + L - 1) / L;
  const size_t nts = PACKED ? (size_t)seqs.nts : (size_t)(NT + 1);
  // this item's chunks: c_lo .. c_hi - 1; the unit's last item is the one that reaches NT
  const int c_lo = (int)((long long)NT * part / parts), c_hi = (int)((long long)NT * (part + 1) / parts);
  const bool last_part = part == parts - 1;
  // (a stretch without a chunk, in a sequence shorter than `parts` chunks, just passes the state on)
  // per-thread slice of u (4 channels) for the diagonal term
  const float4 u4 = *reinterpret_cast<const float4*>(u + hi * HS + 4 * c4);

  // ---- state at the item's first chunk: rows k on the upper lane halves, this warp's 32 columns
  float sreg[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) sreg[j] = 0.f;
  if (part > 0) {
    // wait for the stretch before this one (taken before this item, by a CTA that is running): bounded
    if (tid == 0) {
      uint32_t polls = 0;
      int seen = 0;
      while (true) {
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(handoff_flags + unit) : "memory");
        if (seen >= part || ++polls > (WAIT_LIMIT << 2)) break;
        __nanosleep(200);
      }
      if (seen < part) { atomicExch(status, 405); sm.handoff_ok = 0; } else { sm.handoff_ok = 1; }
    }
    __syncthreads();
    ok = sm.handoff_ok != 0;
    if (!tok_lane && ok) {
      const float* S = handoff + (((size_t)unit * HS) + srow) * HS + 32 * hsel;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 fv = __ldcg(reinterpret_cast<const float4*>(S + j));
        sreg[j] = fv.x; sreg[j + 1] = fv.y; sreg[j + 2] = fv.z; sreg[j + 3] = fv.w;
      }
    }
  } else if (!tok_lane && s0 && n_state > 0) {
    const float* S = s0 + ((state_row(smap, n_state, bi) * H + hi) * HS + srow) * HS + 32 * hsel;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 fv = *reinterpret_cast<const float4*>(S + j);
      sreg[j] = fv.x; sreg[j + 1] = fv.y; sreg[j + 2] = fv.z; sreg[j + 3] = fv.w;
    }
  }

  auto load_in = [&](int c) {      // tid 0; rows past the end of the sequence arrive as zeros
    mbar_expect_tx(&sm.bar_in, 4 * 64 * 64 * (uint32_t)sizeof(T));
    tma_load_4d(sm.at[0], &tmap_w, &sm.bar_in, 0, tok0 + c * L, hi, brow);
    tma_load_4d(sm.vt[0], &tmap_v, &sm.bar_in, 0, tok0 + c * L, hi, brow);
    tma_load_4d(sm.rt[0], &tmap_r, &sm.bar_in, 0, tok0 + c * L, hi, brow);
    tma_load_4d(sm.kt[0], &tmap_k, &sm.bar_in, 0, tok0 + c * L, hi, brow);
  };
  if (tid == 0 && ok && c_lo < c_hi) load_in(c_lo);

  for (int c = c_lo; c < c_hi && ok; ++c, ++n_done) {
    const int t0 = c * L;
    const uint32_t par = n_done & 1;
    W6C_STAMP(0);
    // ---- the raw rows of the chunk have landed: this thread's w and v elements
    ok = mbar_wait(&sm.bar_in, par, status, 403) && ok;
    float4 gw[4], vv4[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4;
      gw[n] = load4_shared(raw_w + row * 64 + 4 * c4);
      vv4[n] = load4_shared(raw_v + row * 64 + 4 * c4);
      if (PACKED && t0 + row >= Tn) vv4[n] = make_float4(0.f, 0.f, 0.f, 0.f);      // the next sequence's row
    }
    __syncthreads();      // every raw v element is in registers: the split v tiles may overwrite the rows
    // ---- pass W: g and its prefix sums; pass V
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4, tok = t0 + row;
      float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tok < Tn)
        f = make_float4(-LOG2E * ex2(LOG2E * gw[n].x), -LOG2E * ex2(LOG2E * gw[n].y), -LOG2E * ex2(LOG2E * gw[n].z),
                        -LOG2E * ex2(LOG2E * gw[n].w));
      gw[n] = f;
      *reinterpret_cast<float4*>(&sm.gs[row * NROW + 4 * c4]) = f;
      store_split4(sm.vt[0], sm.vt[1], row, 4 * c4, vv4[n]);
    }
    __syncthreads();
    W6C_STAMP(1);
    {
      const int ch = tid & 63, quarter = tid >> 6;
      float gv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) gv[j] = sm.gs[(16 * quarter + j) * NROW + ch];
      float run = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) { run += gv[j]; gv[j] = run; }
      sm.qtot[quarter][ch] = run;
      __syncthreads();
      // gi - gref: the prefix inside the half; the reference point is the end of the first half
      const float add = quarter == 0 ? -(run + sm.qtot[1][ch]) : quarter == 1 ? -run : quarter == 3 ? sm.qtot[2][ch] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) sm.gs[(16 * quarter + j) * NROW + ch] = gv[j] + add;
    }
    __syncthreads();
    W6C_STAMP(2);
    // decay factors of the state rows: e^{gref} of this chunk scales the incoming state, e^{glast-gref} the outgoing
    float e0 = 1.f, dlast = 1.f;
    if (!tok_lane) {
      const float tot0 = sm.qtot[0][srow] + sm.qtot[1][srow], tot1 = sm.qtot[2][srow] + sm.qtot[3][srow];
      e0 = ex2(fmaxf(tot0, EXP2_FLOOR));
      dlast = ex2(fmaxf(tot1, EXP2_FLOOR));
      // a half-chunk decay sum beyond the limit: the unit is recomputed by the float32 recurrence
      if (hsel == 0 && (fminf(tot0, tot1) < -DECAY_LIMIT * LOG2E || Tn < SHORT_SEQ)) flags[unit] = 1;
    }
    // ---- S~0 = e^{gref} S0 stays in registers (fp32); hi/lo bf16 tiles for the r~ S~0 product
    if (!tok_lane) {
      if (states) {
        float* dst = states + (((size_t)unit * nts + c) * HS + srow) * HS + 32 * hsel;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(sreg[j], sreg[j + 1], sreg[j + 2], sreg[j + 3]);
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) sreg[j] *= e0;
      store_split_row32(sm.st[0], sm.st[1], srow, 32 * hsel, sreg);
    }
    W6C_STAMP(3);
    // ---- pass RK: scaled r, k (split hi/lo) and the diagonal term
    float4 rr4[4], kk4[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int row = (tid + 256 * n) >> 4;
      rr4[n] = load4_shared(raw_r + row * 64 + 4 * c4);
      kk4[n] = load4_shared(raw_k + row * 64 + 4 * c4);
      if (PACKED && t0 + row >= Tn) { rr4[n] = make_float4(0.f, 0.f, 0.f, 0.f); kk4[n] = rr4[n]; }
    }
    __syncthreads();      // every raw r, k element is in registers
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4;
      const float4 r4 = rr4[n], k4 = kk4[n];
      const float4 gp = *reinterpret_cast<const float4*>(&sm.gs[row * NROW + 4 * c4]);
      const float d1x = gp.x, d1y = gp.y, d1z = gp.z, d1w = gp.w;   // gi - gref
      const float4 rs = make_float4(r4.x * ex2(d1x - gw[n].x), r4.y * ex2(d1y - gw[n].y),
                                    r4.z * ex2(d1z - gw[n].z), r4.w * ex2(d1w - gw[n].w));
      const float4 ks = make_float4(k4.x * ex2(-d1x), k4.y * ex2(-d1y), k4.z * ex2(-d1z), k4.w * ex2(-d1w));
      store_split4(sm.rt[0], sm.rt[1], row, 4 * c4, rs);
      store_split4(sm.kt[0], sm.kt[1], row, 4 * c4, ks);
      float dg = r4.x * u4.x * k4.x + r4.y * u4.y * k4.y + r4.z * u4.z * k4.z + r4.w * u4.w * k4.w;
#pragma unroll
      for (int m = 8; m >= 1; m >>= 1) dg += __shfl_xor_sync(0xffffffffu, dg, m);
      if (c4 == 0) sm.dgs[row] = dg;
    }
    // ask for the next chunk's rows to be brought into L2 while this chunk is in its MMA phases
    if (tid == 0 && c + 1 < c_hi) {
      tma_prefetch_4d(&tmap_w, 0, tok0 + t0 + L, hi, brow);
      tma_prefetch_4d(&tmap_v, 0, tok0 + t0 + L, hi, brow);
      tma_prefetch_4d(&tmap_r, 0, tok0 + t0 + L, hi, brow);
      tma_prefetch_4d(&tmap_k, 0, tok0 + t0 + L, hi, brow);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    W6C_STAMP(4);
    // ---- batch 1: r~ k~^T (columns 0..63), y = r~ S~0 (columns 64.., lower), k~^T v (upper)
    if (lane == 0 && warp < 3) {
      tc_fence_after();
      if (warp == 0)      umma_split<64, 64, 0, 0>(tmem_addr(tm, 0, 0), smem_u32(sm.rt[0]), smem_u32(sm.kt[0]), false);
      else if (warp == 1) umma_split<64, 64, 0, 1>(tmem_addr(tm, 0, 64), smem_u32(sm.rt[0]), smem_u32(sm.st[0]), false);
      else                umma_split<64, 64, 1, 1>(tmem_addr(tm, 16, 64), smem_u32(sm.kt[0]), smem_u32(sm.vt[0]), false);
      umma_commit(&sm.bar_1);
    }
    ok = mbar_wait(&sm.bar_1, par, status, 401) && ok;
    tc_fence_after();
    W6C_STAMP(5);
    if (ok) {
      // A rows (lower halves of columns 0..63): strictly lower part plus the diagonal term, split hi/lo
      uint32_t rr[32];
      load_store_masked_row(tm_a, wq, hsel, lane & 15, tok_lane ? sm.dgs[srow] : 0.f, sm.at[0], srow, tok_lane);
      // state rows (k~^T v on the upper halves of columns 64..127): S_L = e^{glast-gref} (S~0 + k~^T v)
      tmem_ld32(tm_ys, rr);
      tmem_ld_wait();
      if (!tok_lane) {
#pragma unroll
        for (int j = 0; j < 32; ++j) sreg[j] = (sreg[j] + __uint_as_float(rr[j])) * dlast;
      }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);

    W6C_STAMP(6);
    // ---- batch 2: y += A v
    if (tid == 0 && ok) {
      tc_fence_after();
      umma_split<64, 64, 0, 1>(tmem_addr(tm, 0, 64), smem_u32(sm.at[0]), smem_u32(sm.vt[0]), true);
      umma_commit(&sm.bar_2);
    }
    ok = mbar_wait(&sm.bar_2, par, status, 402) && ok;
    tc_fence_after();
    W6C_STAMP(7);
    if (tid == 0 && ok && c + 1 < c_hi) load_in(c + 1);      // the tiles of this chunk have been read for the last time
    if (ok) {
      uint32_t rr[32];
      tmem_ld32(tm_ys, rr);
      tmem_ld_wait();
      if (tok_lane) {     // stage the y rows (fp32) in the prefix-sum area, then store them coalesced
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(&sm.gs[srow * NROW + 32 * hsel + j]) =
              make_float4(__uint_as_float(rr[j]), __uint_as_float(rr[j + 1]), __uint_as_float(rr[j + 2]),
                          __uint_as_float(rr[j + 3]));
      }
    }
    tc_fence_before();
    ok = __syncthreads_and(ok);
    W6C_STAMP(8);
    if (y && ok) {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int e = tid + 256 * n, row = e >> 4, tok = t0 + row;
        if (tok < Tn)
          store4(y + base + (long long)tok * tstride + 4 * c4,
                 *reinterpret_cast<const float4*>(&sm.gs[row * NROW + 4 * c4]));
      }
    }
    __syncthreads();
    W6C_STAMP(9);
  }
#undef W6C_STAMP
  // ---- the state after the item's last chunk: the unit's final state, or what its next stretch starts from
  if (!tok_lane && ok) {
    if (last_part) {
      if (sT) {
        float* dst = sT + (((size_t)unit * HS) + srow) * HS + 32 * hsel;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(sreg[j], sreg[j + 1], sreg[j + 2], sreg[j + 3]);
      }
      if (states) {
        float* dst = states + (((size_t)unit * nts + NT) * HS + srow) * HS + 32 * hsel;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(sreg[j], sreg[j + 1], sreg[j + 2], sreg[j + 3]);
      }
    } else {
      float* dst = handoff + (((size_t)unit * HS) + srow) * HS + 32 * hsel;
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(sreg[j], sreg[j + 1], sreg[j + 2], sreg[j + 3]);
    }
  }
  if (!last_part) {
    __threadfence();
    __syncthreads();
    if (tid == 0 && ok)
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(handoff_flags + unit), "r"(part + 1) : "memory");
  }
  __syncthreads();      // the tiles and next_item are the next item's
  }   // items
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 128);
}

// ---------------------------------------------------------------------------------------------
// backward: one CTA per (batch, head), chunks in reverse; `states` holds the forward state at every
// chunk boundary (written by the forward kernel)
// ---------------------------------------------------------------------------------------------
struct BwdSmem {
  unsigned char rt[2][TILE_BYTES];    // r~            [token][k]
  unsigned char kt[2][TILE_BYTES];    // k~            [token][k]
  // the twelve tiles below are dead once MMA batch 2 has completed; the fp32 staging arrays overlay them
  unsigned char vt[2][TILE_BYTES];    // v             [token][v]
  unsigned char dyt[2][TILE_BYTES];   // dy            [token][v]
  unsigned char at[2][TILE_BYTES];    // A             [i][j]
  unsigned char dat[2][TILE_BYTES];   // stril(dA)     [i][j]
  unsigned char st[2][TILE_BYTES];    // S~0           [k][v]
  unsigned char dst[2][TILE_BYTES];   // dS^           [k][v]
  float gs[L * NROW];                 // gi - gref (prefix of g relative to the reference point)
  float gg[L * NROW];                 // g log2(e)
  float red_e[L * NROW];              // dr~ r~
  float qtot[4][64];
  float rqtot[4][64];
  float pqtot[4][64];
  float dgs[64];                      // sum_k r u k per token
  float dds[64];                      // dy_i . v_i per token
  float dgl[2][64];                   // sum_v dS^ S~0, one partial per column half
  float du_s[64];
  // raw rows of the next chunk, requested by TMA a chunk ahead: w and dy (needed first) here; r and k land
  // in the space of rt / kt once the last epilogue has read those, v in red_e once the decay gradient has
  alignas(128) unsigned char raw_w[L * 64 * 4];
  alignas(128) unsigned char raw_dy[L * 64 * 4];
  uint64_t bar_1, bar_2, bar_2a, bar_in_a, bar_in_b, bar_in_c;
  uint32_t tmem_base;
  int handoff_ok, next_item;
};
static_assert(sizeof(BwdSmem) + 1024 <= 227 * 1024, "backward shared memory");

template <typename T, bool PACKED>
__global__ void __launch_bounds__(256)
wkv6c_bwd_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ w,
                 const float* __restrict__ u, const T* __restrict__ d_y, const float* __restrict__ d_sT,
                 const float* __restrict__ states, T* __restrict__ dr, T* __restrict__ dk, T* __restrict__ dv,
                 T* __restrict__ dw, float* __restrict__ du_partial, float* __restrict__ d_s0,
                 const __grid_constant__ CUtensorMap tmap_r, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ CUtensorMap tmap_dy, int Tn_dense, int H, Seqs seqs, int n_units,
                 int split, float* __restrict__ handoff, int* __restrict__ handoff_flags, int* status,
                 long long* dbg) {
#ifdef RWKVB200_DEVTOOLS
#define W6C_STAMP(n) do { if (dbg && tid == 0 && item == gridDim.x / 2 && c == NT - 2) dbg[n] = clock64(); } while (0)
#else
#define W6C_STAMP(n) do {} while (0)
#endif
  extern __shared__ unsigned char smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wq = warp & 3, hsel = warp >> 2;
  const long long tstride = (long long)H * HS;
  const int srow = 16 * wq + (lane & 15);
  const bool lower = lane < 16;
  const int c4 = tid & 15;
  // fp32 arrays that overlay the dead tiles after MMA batch 2
  float* stage_dr = reinterpret_cast<float*>(sm.vt[0]);
  float* stage_dk = stage_dr + L * NROW;
  float* stage_dv = stage_dk + L * NROW;
  float* stage_dw = stage_dv + L * NROW;
  float* red_i = stage_dw + L * NROW;          // 5 x 17408 B = 87040 B <= 12 tiles
  float* red_x = stage_dw;                     // X k~ per (token, channel), read before dw is staged over it

  if (tid == 0) {
    // every MMA batch is issued by two threads (threads 0 and 32, each with accumulators of its own) and completes
    // with the arrival of both: one thread issues an MMA about every 55 cycles, the tensor pipe takes them faster
    mbar_init(&sm.bar_1, 2); mbar_init(&sm.bar_2, 2); mbar_init(&sm.bar_2a, 2);
    mbar_init(&sm.bar_in_a, 1); mbar_init(&sm.bar_in_b, 1); mbar_init(&sm.bar_in_c, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;
  const uint32_t tm_c0 = tmem_addr(tm, 32 * wq, 32 * hsel);          // A (lower), dA (upper)
  const uint32_t tm_c1 = tmem_addr(tm, 32 * wq, 64 + 32 * hsel);     // dk~ (lower), dr~ (upper)
  const uint32_t tm_c2 = tmem_addr(tm, 32 * wq, 128 + 32 * hsel);    // dv (lower), dS~0 (upper)
  const uint32_t tm_c3 = tmem_addr(tm, 32 * wq, 192 + 32 * hsel);    // X = v dS^^T (lower): the state part of dk~

  constexpr uint32_t RAW_BYTES = 64 * 64 * (uint32_t)sizeof(T);
  const T* raw_w = reinterpret_cast<const T*>(sm.raw_w);
  const T* raw_dy = reinterpret_cast<const T*>(sm.raw_dy);
  const T* raw_v = reinterpret_cast<const T*>(sm.red_e);
  const T* raw_r = reinterpret_cast<const T*>(sm.rt[0]);
  const T* raw_k = reinterpret_cast<const T*>(sm.kt[0]);

  // Work items.  Without `split` an item is a (batch, head) unit and the grid has one CTA per unit.  With it
  // (more units than SMs) every unit is two items, the later half of its chunks and the earlier half, and the
  // grid is one persistent CTA per SM; a CTA that is free takes the next item from a counter (handoff_flags
  // [n_units]).  All later halves come first in that order, so when an earlier half is taken its later half has
  // been taken before, by a CTA that is running, and the state gradient travels between them through `handoff` (a
  // flag per unit says it is there).  Halves of units instead of whole units even out the last round of CTAs
  // (512 units on 148 SMs: 3.5 unit times instead of 4).
  const int n_items = split ? 2 * n_units : n_units;
  bool ok = true;
  uint32_t n_done = 0;      // chunks this CTA has worked on: every barrier completes once per chunk
  for (bool first = true; ok; first = false) {
  if (split) {
    if (tid == 0) sm.next_item = atomicAdd(handoff_flags + n_units, 1);
    __syncthreads();
  } else if (!first) {
    break;
  }
  const int item = split ? sm.next_item : (int)blockIdx.x;
  if (item >= n_items) break;
  const int unit = split ? item % n_units : item;
  const bool early_half = split && item >= n_units;
  const int bi = unit / H, hi = unit % H;
  const int Tn = PACKED ? seqs.len[bi] : Tn_dense;
  const int tok0 = PACKED ? seqs.start[bi] : 0;
  const int brow = PACKED ? 0 : bi;
  const long long base = (((long long)brow * Tn_dense + tok0) * H + hi) * HS;
  const int NT = (Tn + L - 1) / L;
  const size_t nts = PACKED ? (size_t)seqs.nts : (size_t)(NT + 1);
  const int mid = split ? NT / 2 : 0;                 // the later half is chunks mid .. NT-1, the earlier 0 .. mid-1
  const int c_hi = early_half ? mid - 1 : NT - 1;     // first chunk of this item (chunks go in reverse)
  const int c_lo = early_half ? 0 : mid;              // last chunk of this item
  if (c_hi < c_lo) {                                  // an earlier half with nothing in it (a one-chunk sequence)
    if (tid < 64) du_partial[(size_t)item * HS + tid] = 0.f;
    __syncthreads();      // next_item is rewritten at the top
    continue;
  }
  const float4 u4 = *reinterpret_cast<const float4*>(u + hi * HS + 4 * c4);
  if (tid < 64) sm.du_s[tid] = 0.f;

  // gradient of the state after the current chunk: row k = srow (upper lane halves), 32 columns
  float dsreg[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) dsreg[j] = 0.f;
  if (early_half) {
    // wait for the later half of this unit (taken before this item, by a CTA that is running): bounded
    if (tid == 0) {
      uint32_t polls = 0;
      int seen = 0;
      while (true) {
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(handoff_flags + unit) : "memory");
        if (seen || ++polls > (WAIT_LIMIT << 2)) break;
        __nanosleep(200);
      }
      if (!seen) { atomicExch(status, 417); sm.handoff_ok = 0; } else { sm.handoff_ok = 1; }
    }
    __syncthreads();
    ok = sm.handoff_ok != 0;
    if (!lower && ok) {
      const float* S = handoff + (((size_t)unit * HS) + srow) * HS + 32 * hsel;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 f = __ldcg(reinterpret_cast<const float4*>(S + j));
        dsreg[j] = f.x; dsreg[j + 1] = f.y; dsreg[j + 2] = f.z; dsreg[j + 3] = f.w;
      }
    }
  } else if (!lower && d_sT) {
    const float* S = d_sT + (((size_t)unit * HS) + srow) * HS + 32 * hsel;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 f = *reinterpret_cast<const float4*>(S + j);
      dsreg[j] = f.x; dsreg[j + 1] = f.y; dsreg[j + 2] = f.z; dsreg[j + 3] = f.w;
    }
  }
  float4 du_acc = make_float4(0.f, 0.f, 0.f, 0.f);

  auto load_in_a = [&](int c) {      // tid 0; rows past the end of the sequence arrive as zeros
    mbar_expect_tx(&sm.bar_in_a, 2 * RAW_BYTES);
    tma_load_4d(sm.raw_w, &tmap_w, &sm.bar_in_a, 0, tok0 + c * L, hi, brow);
    tma_load_4d(sm.raw_dy, &tmap_dy, &sm.bar_in_a, 0, tok0 + c * L, hi, brow);
  };
  auto load_in_b = [&](int c) {
    mbar_expect_tx(&sm.bar_in_b, 2 * RAW_BYTES);
    tma_load_4d(sm.rt[0], &tmap_r, &sm.bar_in_b, 0, tok0 + c * L, hi, brow);
    tma_load_4d(sm.kt[0], &tmap_k, &sm.bar_in_b, 0, tok0 + c * L, hi, brow);
  };
  auto load_in_c = [&](int c) {
    mbar_expect_tx(&sm.bar_in_c, RAW_BYTES);
    tma_load_4d(sm.red_e, &tmap_v, &sm.bar_in_c, 0, tok0 + c * L, hi, brow);
  };
  if (tid == 0 && ok) { load_in_a(c_hi); load_in_c(c_hi); load_in_b(c_hi); }

  for (int c = c_hi; c >= c_lo && ok; --c, ++n_done) {
    const int t0 = c * L;
    const uint32_t par = n_done & 1;
    W6C_STAMP(32);
    // ---- r and k are read at pass RK and stay in registers until the u-term gradients at the end of the chunk
    float4 gw[4], rr4[4], kk4[4];
    {
      ok = mbar_wait(&sm.bar_in_a, par, status, 413) && ok;
      // ---- pass W: g; pass DY: split tiles
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int e = tid + 256 * n, row = e >> 4, tok = t0 + row;
        const float4 w4 = load4_shared(raw_w + row * 64 + 4 * c4);
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tok < Tn)
          f = make_float4(-LOG2E * ex2(LOG2E * w4.x), -LOG2E * ex2(LOG2E * w4.y), -LOG2E * ex2(LOG2E * w4.z),
                          -LOG2E * ex2(LOG2E * w4.w));
        gw[n] = f;
        *reinterpret_cast<float4*>(&sm.gg[row * NROW + 4 * c4]) = f;
        float4 y4 = load4_shared(raw_dy + row * 64 + 4 * c4);
        if (PACKED && tok >= Tn) y4 = make_float4(0.f, 0.f, 0.f, 0.f);      // the next sequence's row
        store_split4(sm.dyt[0], sm.dyt[1], row, 4 * c4, y4);
      }
    }
    __syncthreads();
    W6C_STAMP(33);

    {
      const int ch = tid & 63, quarter = tid >> 6;
      float gv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) gv[j] = sm.gg[(16 * quarter + j) * NROW + ch];
      float run = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) { run += gv[j]; gv[j] = run; }
      sm.qtot[quarter][ch] = run;
      __syncthreads();
      // gi - gref: the prefix inside the half; the reference point is the end of the first half
      const float add = quarter == 0 ? -(run + sm.qtot[1][ch]) : quarter == 1 ? -run : quarter == 3 ? sm.qtot[2][ch] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) sm.gs[(16 * quarter + j) * NROW + ch] = gv[j] + add;
    }
    __syncthreads();
    W6C_STAMP(34);
    W6C_STAMP(35);
    // ---- pass RK: scaled r, k (split, written over the raw rows once every thread has its elements) and
    // the diagonal term
    ok = mbar_wait(&sm.bar_in_b, par, status, 415) && ok;
    ok = mbar_wait(&sm.bar_in_c, par, status, 414) && ok;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int row = (tid + 256 * n) >> 4;
      rr4[n] = load4_shared(raw_r + row * 64 + 4 * c4);
      kk4[n] = load4_shared(raw_k + row * 64 + 4 * c4);
      // pass V: split tiles and dd_i = dy_i . v_i
      float4 v4 = load4_shared(raw_v + row * 64 + 4 * c4), y4 = load4_shared(raw_dy + row * 64 + 4 * c4);
      if (PACKED && t0 + row >= Tn) {
        v4 = make_float4(0.f, 0.f, 0.f, 0.f); y4 = v4; rr4[n] = v4; kk4[n] = v4;
      }
      store_split4(sm.vt[0], sm.vt[1], row, 4 * c4, v4);
      float dd = v4.x * y4.x + v4.y * y4.y + v4.z * y4.z + v4.w * y4.w;
#pragma unroll
      for (int m = 8; m >= 1; m >>= 1) dd += __shfl_xor_sync(0xffffffffu, dd, m);
      if (c4 == 0) sm.dds[row] = dd;
    }
    __syncthreads();
    if (tid == 0 && ok && c > c_lo) load_in_a(c - 1);      // every thread has taken its w and dy elements
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4;
      const float4 r4 = rr4[n], k4 = kk4[n];
      const float4 gp = *reinterpret_cast<const float4*>(&sm.gs[row * NROW + 4 * c4]);
      const float d1x = gp.x, d1y = gp.y, d1z = gp.z, d1w = gp.w;   // gi - gref
      const float4 rs = make_float4(r4.x * ex2(d1x - gw[n].x), r4.y * ex2(d1y - gw[n].y),
                                    r4.z * ex2(d1z - gw[n].z), r4.w * ex2(d1w - gw[n].w));
      const float4 ks = make_float4(k4.x * ex2(-d1x), k4.y * ex2(-d1y), k4.z * ex2(-d1z), k4.w * ex2(-d1w));
      store_split4(sm.rt[0], sm.rt[1], row, 4 * c4, rs);
      store_split4(sm.kt[0], sm.kt[1], row, 4 * c4, ks);
      float dg = r4.x * u4.x * k4.x + r4.y * u4.y * k4.y + r4.z * u4.z * k4.z + r4.w * u4.w * k4.w;
#pragma unroll
      for (int m = 8; m >= 1; m >>= 1) dg += __shfl_xor_sync(0xffffffffu, dg, m);
      if (c4 == 0) sm.dgs[row] = dg;
    }
    // the row of S0 (both lanes of a pair: the lower one for S~0, the upper one for sum_v dS^ S~0) is requested
    // here and used under MMA batch 1 (requested a phase earlier, the loads held the pass above up instead)
    float4 srow4[8];
    {
      const float* Srow = states + (((size_t)unit * nts + c) * HS + srow) * HS + 32 * hsel;
#pragma unroll
      for (int j = 0; j < 8; ++j) srow4[j] = *reinterpret_cast<const float4*>(Srow + 4 * j);
    }
    if (tid == 0 && c > c_lo) {   // bring the previous chunk's rows into L2 while this chunk is in its MMA phases
      tma_prefetch_4d(&tmap_w, 0, tok0 + t0 - L, hi, brow);
      tma_prefetch_4d(&tmap_dy, 0, tok0 + t0 - L, hi, brow);
      tma_prefetch_4d(&tmap_v, 0, tok0 + t0 - L, hi, brow);
      tma_prefetch_4d(&tmap_r, 0, tok0 + t0 - L, hi, brow);
      tma_prefetch_4d(&tmap_k, 0, tok0 + t0 - L, hi, brow);
      // and the chunk-boundary state the previous chunk starts from
      bulk_prefetch_l2(states + ((size_t)unit * nts + c - 1) * HS * HS, HS * HS * (uint32_t)sizeof(float));
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    W6C_STAMP(36);
    // ---- batch 1: r~ k~^T (lower halves) and dy v^T (upper halves), columns 0..63
    if (tid == 0) {
      tc_fence_after();
      umma_split<64, 64, 0, 0>(tmem_addr(tm, 0, 0), smem_u32(sm.rt[0]), smem_u32(sm.kt[0]), false);
      umma_commit(&sm.bar_1);
    }
    if (tid == 32) {
      tc_fence_after();
      umma_split<64, 64, 0, 0>(tmem_addr(tm, 16, 0), smem_u32(sm.dyt[0]), smem_u32(sm.vt[0]), false);
      umma_commit(&sm.bar_1);
    }
    // decay factors of state row k = srow (both lanes of a pair work on that row below)
    const float e0 = ex2(fmaxf(sm.qtot[0][srow] + sm.qtot[1][srow], EXP2_FLOOR));
    const float dlast = ex2(fmaxf(sm.qtot[2][srow] + sm.qtot[3][srow], EXP2_FLOOR));
    // ---- state rows, while MMA batch 1 runs (it reads neither of the two tiles written here): the upper lane of a
    // pair holds dS and takes sum_v dS^ S~0 (the part of dglast that nothing
    // cancels) and dS^ = e^{glast-gref} dS_L, the lower lane takes S~0 = e^{gref} S0; one split-and-store call
    // serves both
    {
      float x[32];
      if (!lower) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 f = srow4[j >> 2];
          acc += dsreg[j] * f.x + dsreg[j + 1] * f.y + dsreg[j + 2] * f.z + dsreg[j + 3] * f.w;
        }
        sm.dgl[hsel][srow] = acc * (e0 * dlast);      // sum_v dS^ S~0 = e^{gref} e^{glast-gref} sum_v dS_L S0
#pragma unroll
        for (int j = 0; j < 32; ++j) { dsreg[j] *= dlast; x[j] = dsreg[j]; }     // dsreg now holds dS^
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 f = srow4[j >> 2];
          x[j] = f.x * e0; x[j + 1] = f.y * e0; x[j + 2] = f.z * e0; x[j + 3] = f.w * e0;
        }
      }
      unsigned char* hi_t = lower ? sm.st[0] : sm.dst[0];
      store_split_row32(hi_t, hi_t + TILE_BYTES, srow, 32 * hsel, x);
    }
    ok = mbar_wait(&sm.bar_1, par, status, 411) && ok;
    tc_fence_after();
    W6C_STAMP(37);
    if (ok) {
      const float dgi = lower ? sm.dgs[srow] : 0.f;     // the diagonal of A carries the u term; dA's does not
      // one call: both lane halves run the same code
      load_store_masked_row(tm_c0, wq, hsel, lane & 15, dgi, lower ? sm.at[0] : sm.dat[0], srow, true);
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);

    W6C_STAMP(38);
    // ---- batch 2, committed in two parts: the products the heavier part of the read-out needs first, so that its
    // arithmetic runs while the tensor pipe works on the rest (its results stay in registers until then: the
    // staging arrays lie over operand tiles of the products still running)
    if (tid == 0 && ok) {
      tc_fence_after();
      // dr~ = dy S~0^T + stril(dA) k~               (upper halves, columns 64..127)
      umma_split<64, 64, 0, 0>(tmem_addr(tm, 16, 64), smem_u32(sm.dyt[0]), smem_u32(sm.st[0]), false);
      umma_split<64, 64, 0, 1>(tmem_addr(tm, 16, 64), smem_u32(sm.dat[0]), smem_u32(sm.kt[0]), true);
      umma_commit(&sm.bar_2a);
      // dv = A^T dy + k~ dS^                        (lower halves, columns 128..191)
      umma_split<64, 64, 1, 1>(tmem_addr(tm, 0, 128), smem_u32(sm.at[0]), smem_u32(sm.dyt[0]), false);
      umma_split<64, 64, 0, 1>(tmem_addr(tm, 0, 128), smem_u32(sm.kt[0]), smem_u32(sm.dst[0]), true);
      umma_commit(&sm.bar_2);
    }
    if (tid == 32 && ok) {
      tc_fence_after();
      // the part of dk~ from inside the chunk, stril(dA)^T r~   (lower halves, columns 64..127: beside dr~, so
      // that one piece of code scales both in the epilogue)
      umma_split<64, 64, 1, 1>(tmem_addr(tm, 0, 64), smem_u32(sm.dat[0]), smem_u32(sm.rt[0]), false);
      // its state part X = v dS^^T apart (lower halves, columns 192..255): the decay gradient takes the two
      // parts of dk~ k~ in different sums
      umma_split<64, 64, 0, 0>(tmem_addr(tm, 0, 192), smem_u32(sm.vt[0]), smem_u32(sm.dst[0]), false);
      umma_commit(&sm.bar_2a);
      // dS~0 = r~^T dy                              (upper halves, columns 128..191)
      umma_split<64, 64, 1, 1>(tmem_addr(tm, 16, 128), smem_u32(sm.rt[0]), smem_u32(sm.dyt[0]), false);
      umma_commit(&sm.bar_2);
    }
    ok = mbar_wait(&sm.bar_2a, par, status, 416) && ok;
    tc_fence_after();
    const int c0 = 32 * hsel;
    float o[32], rd[32], rs[32];
    if (ok) {
      // r1: the part of dk~ from inside the chunk (lower halves) / dr~ (upper halves), row of token srow; rx: the
      // state part of dk~ (lower halves only)
      uint32_t r1[32], rx[32];
      tmem_ld32(tm_c1, r1);
      tmem_ld32(tm_c3, rx);
      tmem_ld_wait();
      float th[32], tl[32];
      tile_load_row32(lower ? sm.kt[0] : sm.rt[0], srow, c0, th);
      tile_load_row32(lower ? sm.kt[1] : sm.rt[1], srow, c0, tl);
#pragma unroll
      for (int j4 = 0; j4 < 32; j4 += 4) {
        const int cc = c0 + j4;
        const float4 gs4 = *reinterpret_cast<const float4*>(&sm.gs[srow * NROW + cc]);
        const float4 gg4 = *reinterpret_cast<const float4*>(&sm.gg[srow * NROW + cc]);
        const float gsv[4] = {gs4.x, gs4.y, gs4.z, gs4.w}, ggv[4] = {gg4.x, gg4.y, gg4.z, gg4.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const int j = j4 + m;
          const float d1 = gsv[m];                                   // gi - gref
          const float tt = th[j] + tl[j];                            // k~ (lower) / r~ (upper)
          const float x = __uint_as_float(r1[j]);
          const float xs = lower ? __uint_as_float(rx[j]) : 0.f;
          o[j] = (x + xs) * ex2(lower ? -d1 : d1 - ggv[m]);          // dk = dk~ e^{gref-gi},  dr = dr~ e^{ge-gref}
          rd[j] = lower ? -x * tt : x * tt;                          // -(stril(dA)^T r~) k~,  dge = dr~ r~
          rs[j] = xs * tt;                                           // X k~
        }
      }
    }
    ok = mbar_wait(&sm.bar_2, par, status, 412) && ok;
    tc_fence_after();
    W6C_STAMP(39);
    if (ok) {
      float* so = lower ? stage_dk : stage_dr;
      float* sd = lower ? red_i : sm.red_e;
#pragma unroll
      for (int j4 = 0; j4 < 32; j4 += 4) {
        const int cc = c0 + j4;
        *reinterpret_cast<float4*>(&so[srow * NROW + cc]) = make_float4(o[j4], o[j4 + 1], o[j4 + 2], o[j4 + 3]);
        *reinterpret_cast<float4*>(&sd[srow * NROW + cc]) = make_float4(rd[j4], rd[j4 + 1], rd[j4 + 2], rd[j4 + 3]);
        if (lower)
          *reinterpret_cast<float4*>(&red_x[srow * NROW + cc]) = make_float4(rs[j4], rs[j4 + 1], rs[j4 + 2], rs[j4 + 3]);
      }
      // dv row of token srow (lower halves) / dS~0 row k = srow (upper halves)
      uint32_t r2[32];
      tmem_ld32(tm_c2, r2);
      tmem_ld_wait();
      if (!lower) {
#pragma unroll
        for (int j = 0; j < 32; ++j) dsreg[j] = e0 * (__uint_as_float(r2[j]) + dsreg[j]);   // dS0 = e^{gref}(r~^T dy + dS^)
      } else {
#pragma unroll
        for (int j4 = 0; j4 < 32; j4 += 4)
          *reinterpret_cast<float4*>(&stage_dv[srow * NROW + c0 + j4]) =
              make_float4(__uint_as_float(r2[j4]), __uint_as_float(r2[j4 + 1]), __uint_as_float(r2[j4 + 2]),
                          __uint_as_float(r2[j4 + 3]));
      }
    }
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok && c > c_lo) load_in_b(c - 1);      // the epilogue above was the last reader of rt / kt
    W6C_STAMP(40);
    // ---- decay gradient, with I_i = -(stril(dA)^T r~)_i k~_i and X_i k~_i the two parts of dgi_i = -dk~_i k~_i:
    // dg_j = sum_{i>j} (dge_i + I_i) + I_j + sum_v dS^ S~0 + sum_{i<j} X_i k~_i;   dw = dg g.
    // (dglast = sum_v dS_L S_L contains sum_i X_i k~_i; taking the sum over i < j instead of dglast minus the
    // sum over i >= j keeps the two large, nearly equal terms from cancelling.)
    {
      const int ch = tid & 63, quarter = tid >> 6;
      float rv[16], px[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        rv[j] = red_i[(16 * quarter + j) * NROW + ch] + sm.red_e[(16 * quarter + j) * NROW + ch];
        px[j] = red_x[(16 * quarter + j) * NROW + ch];
      }
      float run = 0.f, prun = 0.f;
#pragma unroll
      for (int j = 15; j >= 0; --j) { const float t = rv[j]; rv[j] = run; run += t; }      // sums over i > j
#pragma unroll
      for (int j = 0; j < 16; ++j) { const float t = px[j]; px[j] = prun; prun += t; }      // sums over i < j
      sm.rqtot[quarter][ch] = run;
      sm.pqtot[quarter][ch] = prun;
      __syncthreads();
      float add = sm.dgl[0][ch] + sm.dgl[1][ch];
      for (int q2 = quarter + 1; q2 < 4; ++q2) add += sm.rqtot[q2][ch];
      for (int q2 = 0; q2 < quarter; ++q2) add += sm.pqtot[q2][ch];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int ii = 16 * quarter + j;
        const float dg = (rv[j] + px[j]) + add + red_i[ii * NROW + ch];
        // stage_dw lies over red_x: this thread has read its 16 entries above and writes the same 16
        stage_dw[ii * NROW + ch] = dg * (LN2 * sm.gg[ii * NROW + ch]);      // dw = dg g, g = gg ln 2
      }
    }
    __syncthreads();
    if (tid == 0 && ok && c > c_lo) load_in_c(c - 1);      // red_e has been read for the last time
    W6C_STAMP(41);
    // ---- outputs, coalesced, plus the u-term parts of dr, dk and du
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4, tok = t0 + row;
      if (tok < Tn) {
        const long long off = base + (long long)tok * tstride + 4 * c4;
        const float4 r4 = rr4[n], k4 = kk4[n];
        const float dd = sm.dds[row];
        float4 a = *reinterpret_cast<const float4*>(&stage_dr[row * NROW + 4 * c4]);
        a.x += dd * u4.x * k4.x; a.y += dd * u4.y * k4.y; a.z += dd * u4.z * k4.z; a.w += dd * u4.w * k4.w;
        store4(dr + off, a);
        float4 b = *reinterpret_cast<const float4*>(&stage_dk[row * NROW + 4 * c4]);
        b.x += dd * r4.x * u4.x; b.y += dd * r4.y * u4.y; b.z += dd * r4.z * u4.z; b.w += dd * r4.w * u4.w;
        store4(dk + off, b);
        store4(dv + off, *reinterpret_cast<const float4*>(&stage_dv[row * NROW + 4 * c4]));
        store4(dw + off, *reinterpret_cast<const float4*>(&stage_dw[row * NROW + 4 * c4]));
        du_acc.x += dd * r4.x * k4.x; du_acc.y += dd * r4.y * k4.y;
        du_acc.z += dd * r4.z * k4.z; du_acc.w += dd * r4.w * k4.w;
      }
    }
    __syncthreads();
    W6C_STAMP(42);
  }
#undef W6C_STAMP
  // ---- du of this item and the gradient of the state at its first token: the initial state's, or what the
  // earlier half of the unit starts from
  atomicAdd(&sm.du_s[4 * c4], du_acc.x); atomicAdd(&sm.du_s[4 * c4 + 1], du_acc.y);
  atomicAdd(&sm.du_s[4 * c4 + 2], du_acc.z); atomicAdd(&sm.du_s[4 * c4 + 3], du_acc.w);
  __syncthreads();
  if (tid < 64) du_partial[(size_t)item * HS + tid] = sm.du_s[tid];
  const bool hand_on = split && !early_half && mid > 0;
  float* dS_out = hand_on ? handoff : d_s0;
  if (!lower && dS_out && ok) {
    float* dst = dS_out + (((size_t)unit * HS) + srow) * HS + 32 * hsel;
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      *reinterpret_cast<float4*>(dst + j) = make_float4(dsreg[j], dsreg[j + 1], dsreg[j + 2], dsreg[j + 3]);
  }
  if (hand_on) {
    __threadfence();
    __syncthreads();
    if (tid == 0 && ok) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(handoff_flags + unit), "r"(1) : "memory");
  }
  __syncthreads();      // du_s and the tiles are the next item's
  }   // items
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 256);
}

}  // namespace w6c

int launch_wkv6_chunked_fwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                            const float* s0, int n_state, const int32_t* smap, void* y, float* sT,
                            float* states, int* flags, float* handoff, int* hflags, int B, int Tn, int H,
                            int dtype, cudaStream_t st, const int32_t* seq_start, const int32_t* seq_len,
                            int T_total) {
  using namespace w6c;
  // a packed batch: B sequences (the longest of Tn tokens) end to end in one row of T_total tokens
  const bool packed = seq_start != nullptr;
  const int mapB = packed ? 1 : B, mapT = packed ? T_total : Tn;
  const Seqs seqs{seq_start, seq_len, (Tn + L - 1) / L + 1};
  if (cuda_ok(cudaMemsetAsync(flags, 0, (size_t)B * H * sizeof(int), st))) return RWKVB200_E_CUDA;
  int* status = device_status_ptr();
  if (!status) { last_cuda_error_slot() = 99999; return RWKVB200_E_CUDA; }
  const int smem = (int)sizeof(FwdSmem) + 1024;
  const int esz = dtype == RWKVB200_F32 ? 4 : 2;
  CUtensorMap tm_r, tm_k, tm_v, tm_w;
  int e = make_row_tensor_map(&tm_r, r, mapB, mapT, H, esz);
  if (!e) e = make_row_tensor_map(&tm_k, k, mapB, mapT, H, esz);
  if (!e) e = make_row_tensor_map(&tm_v, v, mapB, mapT, H, esz);
  if (!e) e = make_row_tensor_map(&tm_w, w, mapB, mapT, H, esz);
  if (e) return e;
#define W6C_DISPATCH_PACKED(...) do { if (packed) { constexpr bool P = true; __VA_ARGS__; } else { constexpr bool P = false; __VA_ARGS__; } } while (0)
  {
    // more units than the two CTAs per SM hold at once: every unit as 2 or 4 stretches of its chunks on a
    // persistent grid, whichever evens out the last round best (see the kernel); else one CTA per unit
    int dev = 0, sms = 0;
    if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))
      return RWKVB200_E_CUDA;
    const int n_units = B * H, slots = 2 * sms, NTmax = (Tn + L - 1) / L;
    int parts = 1;
    if (n_units > slots) {
      double best = (double)((n_units + slots - 1) / slots);      // rounds, in unit times
      for (int p2 = 2; p2 <= 4 && NTmax >= 4 * p2; p2 *= 2) {
        const double rounds = (double)(((long long)n_units * p2 + slots - 1) / slots) / p2;
        if (rounds < best - 1e-9) { best = rounds; parts = p2; }
      }
    }
    const int grid = parts > 1 ? slots : n_units;
    if (parts > 1 && cuda_ok(cudaMemsetAsync(hflags, 0, ((size_t)n_units + 1) * sizeof(int), st))) return RWKVB200_E_CUDA;
    ProfScope prof("wkv6c_fwd_kernel", st);
    RWKVB200_DISPATCH_DTYPE(dtype, W6C_DISPATCH_PACKED(
      if (cuda_ok(cudaFuncSetAttribute(wkv6c_fwd_kernel<T, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
        return RWKVB200_E_CUDA;
      wkv6c_fwd_kernel<T, P><<<grid, 256, smem, st>>>((const T*)r, (const T*)k, (const T*)v, (const T*)w, u, s0,
                                                       n_state, smap, (T*)y, sT, states, flags, tm_r, tm_k, tm_v, tm_w,
                                                       mapT, H, seqs, n_units, parts, handoff, hflags, status,
                                                       debug_stamp_buffer())));
  }
  e = check_launch();
  if (e) return e;
  // the marked units again, exactly: outputs, final state and (for the backward) the chunk-boundary states
  const long long unit_floats = (long long)seqs.nts * HS * HS;
  const UnitSel sel{flags, seq_start, seq_len, states ? unit_floats : 0};
  return launch_wkv6_fwd(r, k, v, w, u, s0, n_state, smap, y, sT, states, B, Tn, H, dtype, st, &sel, L);
}

}  // namespace rwkvb200

namespace rwkvb200 {

// workspace of the backward: [chunk-boundary states | du rows, two per unit | du rows of the recurrent
// fallback, four per unit | unit flags | state gradients handed from the later to the earlier half of a unit |
// their flags]; the forward fills the states and the unit flags
namespace {
struct W6Workspace { float* states; float* du_partial; float* du_partial_rec; int* flags; float* handoff; int* hflags; };
inline size_t a256(size_t x) { return (x + 255) & ~size_t(255); }
inline size_t w6_states_bytes(int B, int Tn, int H) {
  const size_t nt = (size_t)(Tn + w6c::L - 1) / w6c::L;
  return a256((size_t)B * H * (nt + 1) * HS * HS * sizeof(float));
}
inline W6Workspace w6_carve(void* workspace, int B, int Tn, int H) {
  char* p = reinterpret_cast<char*>(workspace);
  W6Workspace w;
  w.states = reinterpret_cast<float*>(p);
  p += w6_states_bytes(B, Tn, H);
  w.du_partial = reinterpret_cast<float*>(p);
  p += a256((size_t)B * H * 2 * HS * sizeof(float));
  w.du_partial_rec = reinterpret_cast<float*>(p);
  p += a256((size_t)B * H * 4 * HS * sizeof(float));
  w.flags = reinterpret_cast<int*>(p);
  p += a256((size_t)B * H * sizeof(int));
  w.handoff = reinterpret_cast<float*>(p);
  p += a256((size_t)B * H * HS * HS * sizeof(float));
  w.hflags = reinterpret_cast<int*>(p);      // one flag per unit, then the item counter
  return w;
}
}  // namespace

size_t wkv6_chunked_flags_bytes(int B, int H) { return a256((size_t)B * H * sizeof(int)); }

// scratch of a forward that keeps nothing for a backward: [unit flags | state hand-off | its flags and counter]
size_t wkv6_chunked_fwd_scratch_bytes(int B, int H) {
  return wkv6_chunked_flags_bytes(B, H) + a256((size_t)B * H * HS * HS * sizeof(float)) +
         a256(((size_t)B * H + 1) * sizeof(int));
}
void wkv6_chunked_fwd_scratch(void* workspace, int B, int H, int** flags, float** handoff, int** hflags) {
  char* p = reinterpret_cast<char*>(workspace);
  *flags = reinterpret_cast<int*>(p);
  p += wkv6_chunked_flags_bytes(B, H);
  *handoff = reinterpret_cast<float*>(p);
  p += a256((size_t)B * H * HS * HS * sizeof(float));
  *hflags = reinterpret_cast<int*>(p);
}
// the same three parts inside the backward's workspace (a forward that keeps its chunk-boundary states)
void wkv6_chunked_workspace_parts(void* workspace, int B, int Tn, int H, int** flags, float** handoff, int** hflags) {
  const W6Workspace w = w6_carve(workspace, B, Tn, H);
  *flags = w.flags; *handoff = w.handoff; *hflags = w.hflags;
}

size_t wkv6_chunked_bwd_workspace_bytes(int B, int Tn, int H) {
  return w6_states_bytes(B, Tn, H) + a256((size_t)B * H * 2 * HS * sizeof(float)) +
         a256((size_t)B * H * 4 * HS * sizeof(float)) + wkv6_chunked_flags_bytes(B, H) +
         a256((size_t)B * H * HS * HS * sizeof(float)) + a256(((size_t)B * H + 1) * sizeof(int));
}


int launch_wkv6_chunked_bwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                            const float* s0, int n_state, const int32_t* smap, const void* d_y, const float* d_sT,
                            void* dr, void* dk, void* dv, void* dw, float* du, float* d_s0, void* workspace,
                            int B, int Tn, int H, int dtype, bool kept, cudaStream_t st,
                            const int32_t* seq_start, const int32_t* seq_len, int T_total) {
  using namespace w6c;
  const bool packed = seq_start != nullptr;
  const int mapB = packed ? 1 : B, mapT = packed ? T_total : Tn;
  const Seqs seqs{seq_start, seq_len, (Tn + L - 1) / L + 1};
  const W6Workspace ws = w6_carve(workspace, B, Tn, H);
  float* states = ws.states;
  float* du_partial = ws.du_partial;
  int e = RWKVB200_OK;
  if (!kept) {   // the workspace does not hold the chunk-boundary states yet: run the forward for them
    e = launch_wkv6_chunked_fwd(r, k, v, w, u, s0, n_state, smap, nullptr, nullptr, states, ws.flags, ws.handoff,
                                ws.hflags, B, Tn, H, dtype, st, seq_start, seq_len, T_total);
    if (e) return e;
  }
  int* status = device_status_ptr();
  if (!status) { last_cuda_error_slot() = 99999; return RWKVB200_E_CUDA; }
  const int smem = (int)sizeof(BwdSmem) + 1024;
  bool split = false;
  {
    const int esz = dtype == RWKVB200_F32 ? 4 : 2;
    CUtensorMap tm_r, tm_k, tm_v, tm_w, tm_dy;
    e = make_row_tensor_map(&tm_r, r, mapB, mapT, H, esz);
    if (!e) e = make_row_tensor_map(&tm_k, k, mapB, mapT, H, esz);
    if (!e) e = make_row_tensor_map(&tm_v, v, mapB, mapT, H, esz);
    if (!e) e = make_row_tensor_map(&tm_w, w, mapB, mapT, H, esz);
    if (!e) e = make_row_tensor_map(&tm_dy, d_y, mapB, mapT, H, esz);
    if (e) return e;
    // more units than SMs: every unit as two half-length items on one persistent CTA per SM, which evens out
    // the last round (see the kernel); else one CTA per unit
    int dev = 0, sms = 0;
    if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))
      return RWKVB200_E_CUDA;
    const int n_units = B * H;
    split = n_units > sms && (Tn + L - 1) / L >= 4;
    const int grid = split ? sms : n_units;
    if (split && cuda_ok(cudaMemsetAsync(ws.hflags, 0, ((size_t)n_units + 1) * sizeof(int), st))) return RWKVB200_E_CUDA;
    ProfScope prof("wkv6c_bwd_kernel", st);
    RWKVB200_DISPATCH_DTYPE(dtype, W6C_DISPATCH_PACKED(
      if (cuda_ok(cudaFuncSetAttribute(wkv6c_bwd_kernel<T, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
        return RWKVB200_E_CUDA;
      wkv6c_bwd_kernel<T, P><<<grid, 256, smem, st>>>((const T*)r, (const T*)k, (const T*)v, (const T*)w, u,
                                                       (const T*)d_y, d_sT, states, (T*)dr, (T*)dk, (T*)dv, (T*)dw,
                                                       du_partial, d_s0, tm_r, tm_k, tm_v, tm_w, tm_dy, mapT, H, seqs,
                                                       n_units, split ? 1 : 0, ws.handoff, ws.hflags, status,
                                                       debug_stamp_buffer())));
  }
  e = check_launch();
  if (e) return e;
  // the units the forward marked: gradients from the float32 recurrence, which restarts from the (exact)
  // chunk-boundary states the fallback forward left in the workspace
  {
    const UnitSel sel{ws.flags, seq_start, seq_len, (long long)seqs.nts * HS * HS};
    e = launch_wkv6_bwd_coarse(r, k, v, w, u, d_y, d_sT, states, dr, dk, dv, dw, ws.du_partial_rec, d_s0, B, Tn, H,
                               dtype, st, &sel);
    if (e) return e;
  }
  return launch_wkv6_du_reduce_mixed(du_partial, ws.du_partial_rec, ws.flags, du, B, H, st, split ? 2 : 1);
}

}  // namespace rwkvb200
