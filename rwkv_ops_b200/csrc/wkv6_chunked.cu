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
//   dw = dg g;   with dd_i = dy_i . v_i:  dr += dd u k,  dk += dd r u,  du += sum_i dd r k
//
// Precision.  The parity bar for float32 inputs is 1e-4, which bf16 operands cannot meet, so every
// operand X is split as X = hi + lo (two bf16 tiles) and every product is the three tensor-core
// products hi*hi + hi*lo + lo*hi accumulated in fp32 TMEM (relative error ~2^-16 per term).
//
// One CTA of 256 threads per (batch, head) walks the chunks in order; the state lives in TMEM (fp32)
// and nothing but the inputs and outputs touches HBM in the forward pass (plus, for the backward, the
// fp32 state at every chunk boundary).  Tile and TMEM conventions are those of tc.cuh.
#include "common.cuh"
#include "tc.cuh"

namespace rwkvb200 {
namespace w6c {

using namespace tc;
typedef __nv_bfloat16 bf16;

constexpr int L = 64;
constexpr int NROW = 68;
constexpr float EXP_CLAMP = 80.f;
__device__ __forceinline__ float cexp(float x) { return __expf(fminf(fmaxf(x, -EXP_CLAMP), EXP_CLAMP)); }

__device__ __forceinline__ void split2(float x, float& hi, float& lo) {
  hi = __bfloat162float(__float2bfloat16_rn(x));
  lo = x - hi;
}
// write 4 consecutive values (columns col .. col+3, col a multiple of 4) of `row` into a hi and a lo tile
__device__ __forceinline__ void store_split4(unsigned char* hi_t, unsigned char* lo_t, int row, int col, float4 x) {
  float h[4], l[4];
  split2(x.x, h[0], l[0]); split2(x.y, h[1], l[1]); split2(x.z, h[2], l[2]); split2(x.w, h[3], l[3]);
  const uint32_t off = tile_off(row, col);
  *reinterpret_cast<uint2*>(hi_t + off) = make_uint2(pack_bf16(h[0], h[1]), pack_bf16(h[2], h[3]));
  *reinterpret_cast<uint2*>(lo_t + off) = make_uint2(pack_bf16(l[0], l[1]), pack_bf16(l[2], l[3]));
}
// write 32 consecutive fp32 values of `row` into a hi and a lo tile
__device__ __forceinline__ void store_split_row32(unsigned char* hi_t, unsigned char* lo_t, int row, int col0,
                                                  const float* x) {
  float h[32], l[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) split2(x[j], h[j], l[j]);
  tile_store_row32(hi_t, row, col0, h);
  tile_store_row32(lo_t, row, col0, l);
}

// D (+)= X Y with X = xh + xl, Y = yh + yl (lo tile = hi tile + TILE_BYTES): hi*hi + hi*lo + lo*hi
template <int M, int N, int A_MN, int B_MN>
__device__ __forceinline__ void umma_split(uint32_t tmem_d, uint32_t a_hi, uint32_t b_hi, bool accumulate) {
  umma_tile<M, N, A_MN, B_MN>(tmem_d, a_hi, b_hi, accumulate);
  umma_tile<M, N, A_MN, B_MN>(tmem_d, a_hi, b_hi + TILE_BYTES, true);
  umma_tile<M, N, A_MN, B_MN>(tmem_d, a_hi + TILE_BYTES, b_hi, true);
}

__device__ __forceinline__ long long state_row(const int32_t* smap, int n_state, int bi) {
  if (n_state == 1) return 0;
  if (!smap) return bi;
  int m = smap[bi];
  return m < 0 ? 0 : (m >= n_state ? n_state - 1 : m);
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
struct FwdSmem {
  unsigned char rt[2][TILE_BYTES];    // r~ hi, lo      [token][k]
  unsigned char kt[2][TILE_BYTES];    // k~ hi, lo      [token][k]
  unsigned char vt[2][TILE_BYTES];    // v hi, lo       [token][v]
  unsigned char at[2][TILE_BYTES];    // A hi, lo       [token i][token j]
  unsigned char st[2][TILE_BYTES];    // S~0 hi, lo     [k][v]
  float gs[L * NROW];                 // prefix of g inside each half; later the staged y rows
  float qtot[4][64];
  float dgs[64];                      // sum_k r u k per token
  uint64_t bar_1, bar_2;
  uint32_t tmem_base;
};

// S0 of every chunk (and the final state) goes to `states` [B*H][NT+1][64][64] when it is not NULL.
template <typename T>
__global__ void __launch_bounds__(256)
wkv6c_fwd_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ w,
                 const float* __restrict__ u, const float* __restrict__ s0, int n_state,
                 const int32_t* __restrict__ smap, T* __restrict__ y, float* __restrict__ sT,
                 float* __restrict__ states, int Tn, int H, int* status) {
  extern __shared__ unsigned char smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wq = warp & 3, hsel = warp >> 2;
  const int unit = blockIdx.x, bi = unit / H, hi = unit % H;
  const long long tstride = (long long)H * HS;
  const long long base = ((long long)bi * Tn * H + hi) * HS;
  const int NT = (Tn + L - 1) / L;
  const int srow = 16 * wq + (lane & 15);     // state row k (upper lane halves) / token row (lower lane halves)
  const bool tok_lane = lane < 16;            // lower lane halves hold token rows, upper halves state rows

  if (tid == 0) {
    mbar_init(&sm.bar_1, 1); mbar_init(&sm.bar_2, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sm.tmem_base;
  // TMEM: columns 0..63 lower halves = r~ k~^T; columns 64..127 lower halves = y, upper halves = state
  const uint32_t tm_a = tmem_addr(tm, 32 * wq, 32 * hsel);
  const uint32_t tm_ys = tmem_addr(tm, 32 * wq, 64 + 32 * hsel);

  // per-thread slice of u (4 channels) for the diagonal term
  const int c4 = tid & 15;
  const float4 u4 = *reinterpret_cast<const float4*>(u + hi * HS + 4 * c4);

  // ---- initial state: rows k on the upper lane halves, this warp's 32 columns
  float sreg[32];
  {
    if (!tok_lane) {
      if (s0 && n_state > 0) {
        const float* S = s0 + ((state_row(smap, n_state, bi) * H + hi) * HS + srow) * HS + 32 * hsel;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 f = *reinterpret_cast<const float4*>(S + j);
          sreg[j] = f.x; sreg[j + 1] = f.y; sreg[j + 2] = f.z; sreg[j + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) sreg[j] = 0.f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) sreg[j] = 0.f;
    }
  }

  bool ok = true;
  for (int c = 0; c < NT && ok; ++c) {
    const int t0 = c * L;
    const uint32_t par = c & 1;
    // ---- pass W: g and its prefix sums
    float4 gw[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4, tok = t0 + row;
      float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tok < Tn) {
        f = load4(w + base + (long long)tok * tstride + 4 * c4);
        f = make_float4(-__expf(f.x), -__expf(f.y), -__expf(f.z), -__expf(f.w));
      }
      gw[n] = f;
      *reinterpret_cast<float4*>(&sm.gs[row * NROW + 4 * c4]) = f;
    }
    __syncthreads();
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
      const float add = (quarter & 1) ? sm.qtot[quarter - 1][ch] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) sm.gs[(16 * quarter + j) * NROW + ch] = gv[j] + add;   // prefix inside each half
    }
    __syncthreads();
    // decay factors of the state rows: e^{gref} of this chunk scales the incoming state, e^{glast-gref} the outgoing
    float e0 = 1.f, dlast = 1.f;
    if (!tok_lane) {
      e0 = __expf(fmaxf(sm.qtot[0][srow] + sm.qtot[1][srow], -EXP_CLAMP));
      dlast = __expf(fmaxf(sm.qtot[2][srow] + sm.qtot[3][srow], -EXP_CLAMP));
    }
    // ---- S~0 = e^{gref} S0: fp32 into TMEM (upper lane halves), hi/lo bf16 tiles for the r~ S~0 product
    {
      if (!tok_lane && states) {
        float* dst = states + (((size_t)unit * (NT + 1) + c) * HS + srow) * HS + 32 * hsel;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(sreg[j], sreg[j + 1], sreg[j + 2], sreg[j + 3]);
      }
      uint32_t rr[32];
      float x[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) { x[j] = sreg[j] * e0; rr[j] = __float_as_uint(x[j]); }
      if (!tok_lane) store_split_row32(sm.st[0], sm.st[1], srow, 32 * hsel, x);
      tmem_st32(tm_ys, rr);            // lower halves (y) get zeros: overwritten by the first product
      tmem_st_wait();
    }
    // ---- pass RK: scaled r, k (split hi/lo) and the diagonal term
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4, tok = t0 + row;
      float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f), k4 = r4;
      if (tok < Tn) {
        const long long off = base + (long long)tok * tstride + 4 * c4;
        r4 = load4(r + off); k4 = load4(k + off);
      }
      const float4 gp = *reinterpret_cast<const float4*>(&sm.gs[row * NROW + 4 * c4]);
      const float4 ta = *reinterpret_cast<const float4*>(&sm.qtot[0][4 * c4]);
      const float4 tb = *reinterpret_cast<const float4*>(&sm.qtot[1][4 * c4]);
      const bool fh = row < 32;
      const float d1x = gp.x - (fh ? ta.x + tb.x : 0.f), d1y = gp.y - (fh ? ta.y + tb.y : 0.f);
      const float d1z = gp.z - (fh ? ta.z + tb.z : 0.f), d1w = gp.w - (fh ? ta.w + tb.w : 0.f);   // gi - gref
      const float4 rs = make_float4(r4.x * cexp(d1x - gw[n].x), r4.y * cexp(d1y - gw[n].y),
                                    r4.z * cexp(d1z - gw[n].z), r4.w * cexp(d1w - gw[n].w));
      const float4 ks = make_float4(k4.x * cexp(-d1x), k4.y * cexp(-d1y), k4.z * cexp(-d1z), k4.w * cexp(-d1w));
      store_split4(sm.rt[0], sm.rt[1], row, 4 * c4, rs);
      store_split4(sm.kt[0], sm.kt[1], row, 4 * c4, ks);
      float dg = r4.x * u4.x * k4.x + r4.y * u4.y * k4.y + r4.z * u4.z * k4.z + r4.w * u4.w * k4.w;
#pragma unroll
      for (int m = 8; m >= 1; m >>= 1) dg += __shfl_xor_sync(0xffffffffu, dg, m);
      if (c4 == 0) sm.dgs[row] = dg;
    }
    // ---- pass V
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int e = tid + 256 * n, row = e >> 4, tok = t0 + row;
      float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tok < Tn) v4 = load4(v + base + (long long)tok * tstride + 4 * c4);
      store_split4(sm.vt[0], sm.vt[1], row, 4 * c4, v4);
    }
    // ask for the next chunk's rows to be brought into L2 while this chunk is in its MMA phases
    if (t0 + L < Tn && c4 == 0) {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int tok = t0 + L + ((tid + 256 * n) >> 4);
        if (tok < Tn) {
          const long long off = base + (long long)tok * tstride;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(w + off));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(r + off));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(k + off));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(v + off));
          if (sizeof(T) == 4) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(w + off + 32));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(r + off + 32));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(k + off + 32));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(v + off + 32));
          }
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- batch 1: r~ k~^T (columns 0..63), y = r~ S~0 (columns 64.., lower), state += k~^T v (upper)
    if (tid == 0) {
      tc_fence_after();
      umma_split<64, 64, 0, 0>(tmem_addr(tm, 0, 0), smem_u32(sm.rt[0]), smem_u32(sm.kt[0]), false);
      umma_split<64, 64, 0, 1>(tmem_addr(tm, 0, 64), smem_u32(sm.rt[0]), smem_u32(sm.st[0]), false);
      umma_split<64, 64, 1, 1>(tmem_addr(tm, 16, 64), smem_u32(sm.kt[0]), smem_u32(sm.vt[0]), true);
      umma_commit(&sm.bar_1);
    }
    ok = mbar_wait(&sm.bar_1, par, status, 401) && ok;
    tc_fence_after();
    if (ok) {
      // A rows (lower halves of columns 0..63): strictly lower part plus the diagonal term, split hi/lo
      uint32_t rr[32];
      tmem_ld32(tm_a, rr);
      tmem_ld_wait();
      if (tok_lane) {
        float x[32];
        const float dgi = sm.dgs[srow];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int jj = 32 * hsel + j;
          x[j] = jj < srow ? __uint_as_float(rr[j]) : (jj == srow ? dgi : 0.f);
        }
        store_split_row32(sm.at[0], sm.at[1], srow, 32 * hsel, x);
      }
      // state rows (upper halves of columns 64..127): S_L = e^{glast-gref} (S~0 + k~^T v)
      tmem_ld32(tm_ys, rr);
      tmem_ld_wait();
      if (!tok_lane) {
#pragma unroll
        for (int j = 0; j < 32; ++j) sreg[j] = __uint_as_float(rr[j]) * dlast;
      }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);

    // ---- batch 2: y += A v
    if (tid == 0 && ok) {
      tc_fence_after();
      umma_split<64, 64, 0, 1>(tmem_addr(tm, 0, 64), smem_u32(sm.at[0]), smem_u32(sm.vt[0]), true);
      umma_commit(&sm.bar_2);
    }
    ok = mbar_wait(&sm.bar_2, par, status, 402) && ok;
    tc_fence_after();
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
  }
  // ---- final state
  if (!tok_lane && ok) {
    if (sT) {
      float* dst = sT + (((size_t)unit * HS) + srow) * HS + 32 * hsel;
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(sreg[j], sreg[j + 1], sreg[j + 2], sreg[j + 3]);
    }
    if (states) {
      float* dst = states + (((size_t)unit * (NT + 1) + NT) * HS + srow) * HS + 32 * hsel;
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(sreg[j], sreg[j + 1], sreg[j + 2], sreg[j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 128);
}

}  // namespace w6c

int launch_wkv6_chunked_fwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                            const float* s0, int n_state, const int32_t* smap, void* y, float* sT,
                            float* states, int B, int Tn, int H, int dtype, cudaStream_t st) {
  using namespace w6c;
  int* status = device_status_ptr();
  if (!status) { last_cuda_error_slot() = 99999; return RWKVB200_E_CUDA; }
  const int smem = (int)sizeof(FwdSmem) + 1024;
  ProfScope prof("wkv6c_fwd_kernel", st);
  RWKVB200_DISPATCH_DTYPE(dtype,
    if (cuda_ok(cudaFuncSetAttribute(wkv6c_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
      return RWKVB200_E_CUDA;
    wkv6c_fwd_kernel<T><<<B * H, 256, smem, st>>>((const T*)r, (const T*)k, (const T*)v, (const T*)w, u, s0, n_state,
                                                   smap, (T*)y, sT, states, Tn, H, status));
  return check_launch();
}

}  // namespace rwkvb200
