// RWKV6 wkv operator, float32 arithmetic, forward and backward.
//
// Maths of the reference's native operator (rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:63-80):
//   d_t = exp(-exp(w_t));  y_t[v] = sum_k r_t[k] (u[k] k_t[k] v_t[v] + S_{t-1}[k][v]);  S_t = diag(d_t) S_{t-1} + k_t v_t^T
// with S[k][v] and S_0 = s0[state_map[b]] or zero.
//
// Column v of S never mixes with another column, so the N value columns (N = head size: 32, 64 or 128) are
// split over N/16 CTAs of 16 columns each: grid (B*H, N/16), N threads.  In the "value role" thread
// (vl = tid / NKQ, kq = tid % NKQ, NKQ = N/16) holds S[16*kq .. 16*kq+15][vl] in registers; the reduction
// over k takes log2(NKQ) shuffles.  In the "key role" thread kc = tid owns key channel kc.
//
// Backward, with G the gradient of the state flowing from the future and dyv = sum_v dy_t[v] v_t[v]:
//   dr_t[k] = u[k] k_t[k] dyv + sum_v S_{t-1}[k][v] dy_t[v]      dk_t[k] = r_t[k] u[k] dyv + sum_v G[k][v] v_t[v]
//   dv_t[v] = dy_t[v] sum_k r u k + sum_k G[k][v] k_t[k]         dd_t[k] = sum_v G[k][v] S_{t-1}[k][v]
//   du[k]  += r_t[k] k_t[k] dyv                                  G <- diag(d_t) G + r_t dy_t^T
//   dw_t = dd_t * d_t * (-exp(w_t))
// S_{t-1} is needed per token: the forward sweep stores the state every W6_CKPT tokens (the workspace)
// and the backward kernel re-runs each chunk forward into shared memory before sweeping it backward.
// Sums over v need all CTAs of a (batch, head): they form a thread-block cluster and exchange
// per-chunk partial sums through distributed shared memory in a fixed order (deterministic).
#include <cooperative_groups.h>

#include <type_traits>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace rwkvb200 {

namespace {

constexpr int VS = 16;
// A staged vector of N key channels is kept as segments of 16 with 4 floats of padding between them: the lanes
// of a quarter warp read the same 16 bytes of N/16 different segments, which 64 bytes apart would share banks.
__host__ __device__ constexpr int padk(int k) { return k + ((k >> 4) << 2); }
template <int N> __host__ __device__ constexpr int NP() { return N + N / 4; }
constexpr int TL = 16;
constexpr int CK = W6_CKPT;
constexpr int SCOL = VS + 1;   // padded row (one key, 16 values) of a state slab in shared memory

__device__ __forceinline__ long long state_row(const int32_t* smap, int n_state, int bi) {
  if (n_state == 1) return 0;
  if (!smap) return bi;
  int m = smap[bi];
  return m < 0 ? 0 : (m >= n_state ? n_state - 1 : m);
}

// sum over the NKQ lanes that share a value column
template <int NKQ>
__device__ __forceinline__ float sum_kq(float x) {
#pragma unroll
  for (int m = 1; m < NKQ; m <<= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}

template <typename T, int N>
__global__ void __launch_bounds__(N)
wkv6_fwd_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                const T* __restrict__ w, const float* __restrict__ u,
                const float* __restrict__ s0, int n_state, const int32_t* __restrict__ smap,
                T* __restrict__ yout, float* __restrict__ sT, float* __restrict__ ckpt, int ckpt_every,
                int Tn_dense, int H, UnitSel sel) {
  constexpr int NKQ = N / VS, QUADS = N / 4;
  __shared__ __align__(16) float tile[TL][4][NP<N>()];   // r, d, k, r*u*k
  __shared__ __align__(16) float vt[TL][VS];
  __shared__ __align__(16) float yt[TL][VS];

  const int unit = blockIdx.x, y = blockIdx.y, tid = threadIdx.x;
  if (sel.flags && sel.flags[unit] == 0) return;      // only the selected units run
  const int bi = unit / H, hi = unit % H;
  const int vl = tid / NKQ, kq = tid % NKQ;
  // a packed batch keeps its sequences end to end in batch row 0
  const int Tn = sel.seq_len ? sel.seq_len[bi] : Tn_dense;
  const long long base = sel.seq_start ? ((long long)sel.seq_start[bi] * H + hi) * N
                                       : ((long long)bi * Tn_dense * H + hi) * N;   // + t*H*N
  const long long tstride = (long long)H * N;
  const long long ckpt_unit = sel.ckpt_unit_stride ? sel.ckpt_unit_stride
                                                   : (long long)((Tn_dense + ckpt_every - 1) / ckpt_every) * N * N;
  const float4 u4 = *reinterpret_cast<const float4*>(u + hi * N + 4 * (tid % QUADS));

  float S[16];
  if (s0 && n_state > 0) {
    const float* p = s0 + ((state_row(smap, n_state, bi) * H + hi) * N + 16 * kq) * N + y * VS + vl;
#pragma unroll
    for (int j = 0; j < 16; ++j) S[j] = p[j * N];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) S[j] = 0.f;
  }

  // The inputs of a tile travel global memory -> registers -> shared memory, and the loads of tile i + 1 are
  // issued before the tokens of tile i are worked on: few warps share an SM here, so a load that is waited for
  // where it is issued costs its full latency every time.
  constexpr int PER = TL / 4;                      // (token, quad) pairs per thread per tile: TL x N/4 over N threads
  constexpr int VPER = (TL * 4 + N - 1) / N;       // float4 of v per thread per tile (16 values per token)
  float4 rbuf[PER], kbuf[PER], wbuf[PER], vbuf[VPER];
  const int quad = tid % QUADS, rq = tid / QUADS;      // this thread's quad of channels; its tokens are rq + 4 m
  auto fetch = [&](int t0) {
    const int nt = min(TL, Tn - t0);
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int tl = rq + 4 * m;
      const long long off = base + (long long)(t0 + tl) * tstride + 4 * quad;
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      rbuf[m] = tl < nt ? load4(r + off) : z;
      kbuf[m] = tl < nt ? load4(k + off) : z;
      wbuf[m] = tl < nt ? load4(w + off) : z;
    }
#pragma unroll
    for (int m = 0; m < VPER; ++m) {
      const int i = tid + m * N;
      vbuf[m] = i < nt * 4 ? load4(v + base + (long long)(t0 + (i >> 2)) * tstride + y * VS + 4 * (i & 3))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int tl = rq + 4 * m;
      const float4 r4 = rbuf[m], k4 = kbuf[m], w4 = wbuf[m];
      *reinterpret_cast<float4*>(&tile[tl][0][padk(4 * quad)]) = r4;
      *reinterpret_cast<float4*>(&tile[tl][1][padk(4 * quad)]) =
          make_float4(decay_of(w4.x), decay_of(w4.y), decay_of(w4.z), decay_of(w4.w));
      *reinterpret_cast<float4*>(&tile[tl][2][padk(4 * quad)]) = k4;
      *reinterpret_cast<float4*>(&tile[tl][3][padk(4 * quad)]) =
          make_float4(r4.x * u4.x * k4.x, r4.y * u4.y * k4.y, r4.z * u4.z * k4.z, r4.w * u4.w * k4.w);
    }
#pragma unroll
    for (int m = 0; m < VPER; ++m) {
      const int i = tid + m * N;
      if (i < TL * 4) *reinterpret_cast<float4*>(&vt[i >> 2][4 * (i & 3)]) = vbuf[m];
    }
  };
  if (Tn > 0) fetch(0);
  for (int t0 = 0; t0 < Tn; t0 += TL) {
    const int nt = min(TL, Tn - t0);
    stash();
    __syncthreads();
    if (t0 + TL < Tn) fetch(t0 + TL);
    for (int tl = 0; tl < nt; ++tl) {
      const int t = t0 + tl;
      if (ckpt && (t % ckpt_every) == 0) {
        float* p = ckpt + unit * ckpt_unit + (((long long)(t / ckpt_every) * N) + 16 * kq) * N + y * VS + vl;
#pragma unroll
        for (int j = 0; j < 16; ++j) p[j * N] = S[j];
      }
      const float* tr = &tile[tl][0][20 * kq];
      const float* td = &tile[tl][1][20 * kq];
      const float* tk = &tile[tl][2][20 * kq];
      const float* tq = &tile[tl][3][20 * kq];
      const float vv = vt[tl][vl];
      float y0 = 0.f, y1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        y0 += tr[j] * S[j]; y1 += tr[j + 1] * S[j + 1];
        q0 += tq[j]; q1 += tq[j + 1];
        S[j] = td[j] * S[j] + tk[j] * vv;
        S[j + 1] = td[j + 1] * S[j + 1] + tk[j + 1] * vv;
      }
      const float yy = sum_kq<NKQ>((y0 + y1) + vv * (q0 + q1));
      if (kq == 0) yt[tl][vl] = yy;
    }
    __syncthreads();
    if (yout) {
      for (int i = tid; i < nt * 4; i += N) {
        const int tl = i >> 2, quad = i & 3;
        store4(yout + base + (long long)(t0 + tl) * tstride + y * VS + 4 * quad,
               *reinterpret_cast<const float4*>(&yt[tl][4 * quad]));
      }
    }
  }
  if (sT) {
    float* p = sT + (((long long)unit * N) + 16 * kq) * N + y * VS + vl;
#pragma unroll
    for (int j = 0; j < 16; ++j) p[j * N] = S[j];
  }
}

template <int N> struct BwdSmem {
  float tile[CK][6][NP<N>()];           // r, d, exp(w), k, r*u, u*k
  float ruk[CK];                  // sum_k r u k
  float vt[CK][VS];
  float dyt[CK][VS];
  float dvt[CK][VS];
  float Sbuf[CK][N][SCOL];        // state before token i of the chunk
  float part[2][CK][3][N];        // partial dr, dk, dd over this CTA's 16 value columns
  float pdyv[2][CK];              // partial sum_v dy v
};
// COARSE variant: the checkpoints lie 64 tokens apart (the chunk-boundary states of the chunked path); the
// states at the start of the eight 8-token groups of a 64-token stretch are recomputed into `sub`.
template <int N> struct BwdSmemCoarse : BwdSmem<N> {
  float sub[8][N][VS];
};

// launched with a cluster of (1, N/16, 1): the CTAs of one unit
template <typename T, int N, bool COARSE>
__global__ void __launch_bounds__(N)
wkv6_bwd_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                const T* __restrict__ w, const float* __restrict__ u,
                const T* __restrict__ d_y, const float* __restrict__ d_sT, const float* __restrict__ ckpt,
                T* __restrict__ dr, T* __restrict__ dk, T* __restrict__ dv, T* __restrict__ dw,
                float* __restrict__ du_partial, float* __restrict__ d_s0, int Tn_dense, int H, UnitSel sel) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int NKQ = N / VS, NQ = N / VS, QUADS = N / 4;
  typedef typename std::conditional<COARSE, BwdSmemCoarse<N>, BwdSmem<N>>::type Smem;
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();

  const int unit = blockIdx.x, y = blockIdx.y, tid = threadIdx.x;
  if (sel.flags && sel.flags[unit] == 0) return;      // the CTAs of a cluster share the unit: all leave
  const int bi = unit / H, hi = unit % H;
  const int vl = tid / NKQ, kq = tid % NKQ;   // value role
  const int kc = tid;                      // key role
  const int Tn = sel.seq_len ? sel.seq_len[bi] : Tn_dense;
  const long long base = sel.seq_start ? ((long long)sel.seq_start[bi] * H + hi) * N
                                       : ((long long)bi * Tn_dense * H + hi) * N;
  const long long tstride = (long long)H * N;
  const int NC = (Tn + CK - 1) / CK;
  const long long ckpt_unit = sel.ckpt_unit_stride ? sel.ckpt_unit_stride
                                                   : (long long)((Tn_dense + CK - 1) / CK) * N * N;
  const float4 u4 = *reinterpret_cast<const float4*>(u + hi * N + 4 * (tid % QUADS));

  float Gv[16], Gk[VS];   // value-role copy G[16kq+j][vl], key-role copy G[kc][i]
  if (d_sT) {
#pragma unroll
    for (int j = 0; j < 16; ++j) Gv[j] = d_sT[(((long long)unit * N) + 16 * kq + j) * N + y * VS + vl];
#pragma unroll
    for (int i = 0; i < VS; ++i) Gk[i] = d_sT[(((long long)unit * N) + kc) * N + y * VS + i];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) Gv[j] = 0.f;
#pragma unroll
    for (int i = 0; i < VS; ++i) Gk[i] = 0.f;
  }
  float du_acc = 0.f;

  // The inputs of chunk c - 1 (and, from checkpoints one chunk apart, its starting state) are requested into
  // registers before chunk c is worked on, and written to shared memory when chunk c is done: see the forward
  // kernel.
  constexpr int PER = CK / 4;                      // (token, quad) pairs per thread per chunk
  constexpr int VPER = (CK * 4 + N - 1) / N;       // float4 of v (and of dy) per thread per chunk
  float4 rbuf[PER], kbuf[PER], wbuf[PER], vbuf[VPER], dybuf[VPER];
  float Snext[16];
  const int quad = tid % QUADS, rq = tid / QUADS;
  auto fetch = [&](int c) {
    const int t0 = c * CK, nt = min(CK, Tn - t0);
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int tl = rq + 4 * m;
      const long long off = base + (long long)(t0 + tl) * tstride + 4 * quad;
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      rbuf[m] = tl < nt ? load4(r + off) : z;
      kbuf[m] = tl < nt ? load4(k + off) : z;
      wbuf[m] = tl < nt ? load4(w + off) : z;
    }
#pragma unroll
    for (int m = 0; m < VPER; ++m) {
      const int i = tid + m * N;
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      const long long off = base + (long long)(t0 + (i >> 2)) * tstride + y * VS + 4 * (i & 3);
      vbuf[m] = i < nt * 4 ? load4(v + off) : z;
      dybuf[m] = i < nt * 4 ? load4(d_y + off) : z;
    }
    if constexpr (!COARSE) {
      const float* p = ckpt + unit * ckpt_unit + (((long long)c * N) + 16 * kq) * N + y * VS + vl;
#pragma unroll
      for (int j = 0; j < 16; ++j) Snext[j] = p[j * N];
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int tl = rq + 4 * m;
      const float4 r4 = rbuf[m], k4 = kbuf[m], w4 = wbuf[m];
      *reinterpret_cast<float4*>(&sm.tile[tl][0][padk(4 * quad)]) = r4;
      *reinterpret_cast<float4*>(&sm.tile[tl][1][padk(4 * quad)]) =
          make_float4(decay_of(w4.x), decay_of(w4.y), decay_of(w4.z), decay_of(w4.w));
      *reinterpret_cast<float4*>(&sm.tile[tl][2][padk(4 * quad)]) = make_float4(expf(w4.x), expf(w4.y), expf(w4.z), expf(w4.w));
      *reinterpret_cast<float4*>(&sm.tile[tl][3][padk(4 * quad)]) = k4;
      *reinterpret_cast<float4*>(&sm.tile[tl][4][padk(4 * quad)]) = make_float4(r4.x * u4.x, r4.y * u4.y, r4.z * u4.z, r4.w * u4.w);
      *reinterpret_cast<float4*>(&sm.tile[tl][5][padk(4 * quad)]) = make_float4(u4.x * k4.x, u4.y * k4.y, u4.z * k4.z, u4.w * k4.w);
    }
#pragma unroll
    for (int m = 0; m < VPER; ++m) {
      const int i = tid + m * N;
      if (i < CK * 4) {
        *reinterpret_cast<float4*>(&sm.vt[i >> 2][4 * (i & 3)]) = vbuf[m];
        *reinterpret_cast<float4*>(&sm.dyt[i >> 2][4 * (i & 3)]) = dybuf[m];
      }
    }
  };
  if (NC > 0) fetch(NC - 1);
  for (int c = NC - 1; c >= 0; --c) {
    const int t0 = c * CK, nt = min(CK, Tn - t0), pb = c & 1;
    if constexpr (COARSE) {
      // entering a 64-token stretch (from its end): re-run it forward from its checkpoint, keeping the
      // state at the start of each of its 8-token groups
      if (c == NC - 1 || (c & 7) == 7) {
        const int c64 = c >> 3;
        float S0[16];
        {
          const float* p = ckpt + unit * ckpt_unit + (((long long)c64 * N) + 16 * kq) * N + y * VS + vl;
#pragma unroll
          for (int j = 0; j < 16; ++j) S0[j] = p[j * N];
        }
        for (int g = 8 * c64; g <= c; ++g) {
          const int tg0 = g * CK, ntg = min(CK, Tn - tg0);
          for (int i = tid; i < ntg * QUADS; i += N) {
            const int quad = i % QUADS, tl = i / QUADS;
            const long long off = base + (long long)(tg0 + tl) * tstride + 4 * quad;
            const float4 k4 = load4(k + off), w4 = load4(w + off);
            *reinterpret_cast<float4*>(&sm.tile[tl][1][padk(4 * quad)]) =
                make_float4(decay_of(w4.x), decay_of(w4.y), decay_of(w4.z), decay_of(w4.w));
            *reinterpret_cast<float4*>(&sm.tile[tl][3][padk(4 * quad)]) = k4;
          }
          for (int i = tid; i < ntg * 4; i += N) {
            const int tl = i >> 2, quad = i & 3;
            *reinterpret_cast<float4*>(&sm.vt[tl][4 * quad]) =
                load4(v + base + (long long)(tg0 + tl) * tstride + y * VS + 4 * quad);
          }
          __syncthreads();
#pragma unroll
          for (int j = 0; j < 16; ++j) sm.sub[g & 7][16 * kq + j][vl] = S0[j];
          for (int tl = 0; tl < ntg; ++tl) {
            const float* td = &sm.tile[tl][1][20 * kq];
            const float* tk = &sm.tile[tl][3][20 * kq];
            const float vv = sm.vt[tl][vl];
#pragma unroll
            for (int j = 0; j < 16; ++j) S0[j] = td[j] * S0[j] + tk[j] * vv;
          }
          __syncthreads();      // the tile is staged again for the next group
        }
      }
    }
    // ---- the chunk's inputs, and the state at its start (value role) for the forward re-run
    stash();
    float S[16];
    if constexpr (COARSE) {
#pragma unroll
      for (int j = 0; j < 16; ++j) S[j] = sm.sub[c & 7][16 * kq + j][vl];
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) S[j] = Snext[j];
    }
    __syncthreads();
    if (c > 0) fetch(c - 1);
    // sum_k r u k per token (threads 0..nt-1, one token each)
    if (tid < nt) {
      float s = 0.f;
      for (int j = 0; j < N; ++j) s += sm.tile[tid][4][padk(j)] * sm.tile[tid][3][padk(j)];
      sm.ruk[tid] = s;
    }
    // re-run the chunk forward (value role), keeping the state before every token
    for (int tl = 0; tl < nt; ++tl) {
      const float* td = &sm.tile[tl][1][20 * kq];
      const float* tk = &sm.tile[tl][3][20 * kq];
      const float vv = sm.vt[tl][vl];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        sm.Sbuf[tl][16 * kq + j][vl] = S[j];
        S[j] = td[j] * S[j] + tk[j] * vv;
      }
    }
    __syncthreads();

    for (int tl = nt - 1; tl >= 0; --tl) {
      // value role: dv = dy * sum(ruk) + sum_k G[k][v] k[k]
      const float* tr = &sm.tile[tl][0][20 * kq];
      const float* td = &sm.tile[tl][1][20 * kq];
      const float* tk = &sm.tile[tl][3][20 * kq];
      const float dyr = sm.dyt[tl][vl];
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        a0 += Gv[j] * tk[j]; a1 += Gv[j + 1] * tk[j + 1];
        Gv[j] = td[j] * Gv[j] + tr[j] * dyr;
        Gv[j + 1] = td[j + 1] * Gv[j + 1] + tr[j + 1] * dyr;
      }
      const float dvv = sum_kq<NKQ>(a0 + a1);
      if (kq == 0) sm.dvt[tl][vl] = dvv + dyr * sm.ruk[tl];
      // key role
      const float rk = sm.tile[tl][0][padk(kc)], dk_ = sm.tile[tl][1][padk(kc)];
      float p_dr = 0.f, p_dk = 0.f, p_dd = 0.f, p_dyv = 0.f;
#pragma unroll
      for (int i = 0; i < VS; ++i) {
        const float sp = sm.Sbuf[tl][kc][i];
        const float dyi = sm.dyt[tl][i], vi = sm.vt[tl][i];
        p_dr += sp * dyi;
        p_dk += Gk[i] * vi;
        p_dd += Gk[i] * sp;
        p_dyv += dyi * vi;
        Gk[i] = dk_ * Gk[i] + rk * dyi;
      }
      sm.part[pb][tl][0][kc] = p_dr;
      sm.part[pb][tl][1][kc] = p_dk;
      sm.part[pb][tl][2][kc] = p_dd;
      if (kc == 0) sm.pdyv[pb][tl] = p_dyv;
    }
    __syncthreads();
    for (int i = tid; i < nt * VS; i += N) {
      const int tl = i >> 4, vi = i & 15;
      dv[base + (long long)(t0 + tl) * tstride + y * VS + vi] = from_f32<T>(sm.dvt[tl][vi]);
    }
    cluster.sync();
    for (int tl = y; tl < nt; tl += NQ) {
      float acc[3] = {0.f, 0.f, 0.f}, dyv = 0.f;
#pragma unroll
      for (int rk_ = 0; rk_ < NQ; ++rk_) {
        const float* rp = cluster.map_shared_rank(&sm.part[pb][tl][0][0], rk_);
        const float* rd = cluster.map_shared_rank(&sm.pdyv[pb][0], rk_);
#pragma unroll
        for (int qn = 0; qn < 3; ++qn) acc[qn] += rp[qn * N + kc];
        dyv += rd[tl];
      }
      const long long off = base + (long long)(t0 + tl) * tstride + kc;
      dr[off] = from_f32<T>(acc[0] + sm.tile[tl][5][padk(kc)] * dyv);
      dk[off] = from_f32<T>(acc[1] + sm.tile[tl][4][padk(kc)] * dyv);
      dw[off] = from_f32<T>(acc[2] * sm.tile[tl][1][padk(kc)] * (-sm.tile[tl][2][padk(kc)]));
      du_acc += sm.tile[tl][0][padk(kc)] * sm.tile[tl][3][padk(kc)] * dyv;
    }
    __syncthreads();
  }
  du_partial[((long long)unit * NQ + y) * N + kc] = du_acc;
  if (d_s0) {
#pragma unroll
    for (int j = 0; j < 16; ++j) d_s0[(((long long)unit * N) + 16 * kq + j) * N + y * VS + vl] = Gv[j];
  }
  cluster.sync();
}

// du[h][k] = sum over batch rows and the CTAs of a unit, in a fixed order (one thread per key channel).
__global__ void __launch_bounds__(128)
wkv6_du_reduce_kernel(const float* __restrict__ du_partial, float* __restrict__ du, int B, int H) {
  const int hi = blockIdx.x, kc = threadIdx.x, n = blockDim.x, nq = n / VS;
  float s = 0.f;
  for (int bi = 0; bi < B; ++bi)
    for (int q = 0; q < nq; ++q) s += du_partial[(((long long)bi * H + hi) * nq + q) * n + kc];
  du[hi * n + kc] = s;
}

// The same for the chunked path with its recurrent fallback: a unit contributes `rows` rows of `part_chunked`
// [rows][B*H][64] (two when its chunks were worked on as two halves), or, when the forward marked it (flags),
// its four rows of `part_rec` [B*H][4][64].
__global__ void __launch_bounds__(64)
wkv6_du_reduce_mixed_kernel(const float* __restrict__ part_chunked, const float* __restrict__ part_rec,
                            const int* __restrict__ flags, float* __restrict__ du, int B, int H, int rows) {
  constexpr int NQ = HS / VS;
  const int hi = blockIdx.x, kc = threadIdx.x;
  float s = 0.f;
  for (int bi = 0; bi < B; ++bi) {
    const long long unit = (long long)bi * H + hi;
    if (flags[unit]) {
      for (int q = 0; q < NQ; ++q) s += part_rec[(unit * NQ + q) * HS + kc];
    } else {
      for (int q = 0; q < rows; ++q) s += part_chunked[((long long)q * B * H + unit) * HS + kc];
    }
  }
  du[hi * HS + kc] = s;
}

}  // namespace

// head size 32, 64 or 128
#define RWKVB200_DISPATCH_HEAD6(hs, ...)                          \
  switch (hs) {                                                   \
    case 32:  { constexpr int N = 32;  __VA_ARGS__; break; }      \
    case 64:  { constexpr int N = 64;  __VA_ARGS__; break; }      \
    case 128: { constexpr int N = 128; __VA_ARGS__; break; }      \
    default: return RWKVB200_E_UNSUPPORTED;                       \
  }

int launch_wkv6_fwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                    const float* s0, int n_state, const int32_t* smap, void* y, float* sT,
                    float* ckpt, int B, int Tn, int H, int dtype, cudaStream_t st, const UnitSel* sel_,
                    int ckpt_every, int head_size) {
  const UnitSel sel = sel_ ? *sel_ : UnitSel{nullptr, nullptr, nullptr, 0};
  ProfScope prof("wkv6_fwd_kernel", st);
  RWKVB200_DISPATCH_HEAD6(head_size,
    dim3 grid(B * H, N / VS);
    RWKVB200_DISPATCH_DTYPE(dtype,
      wkv6_fwd_kernel<T, N><<<grid, N, 0, st>>>((const T*)r, (const T*)k, (const T*)v, (const T*)w, u, s0, n_state,
                                                smap, (T*)y, sT, ckpt, ckpt_every ? ckpt_every : CK, Tn, H, sel)));
  return check_launch();
}

namespace {
// the backward kernel over a cluster of the N/16 CTAs of a unit
template <typename T, int N, bool COARSE>
int launch_bwd_cluster(const void* r, const void* k, const void* v, const void* w, const float* u, const void* d_y,
                       const float* d_sT, const float* ckpt, void* dr, void* dk, void* dv, void* dw,
                       float* du_partial, float* d_s0, int B, int Tn, int H, cudaStream_t st, const UnitSel& sel) {
  typedef typename std::conditional<COARSE, BwdSmemCoarse<N>, BwdSmem<N>>::type Smem;
  const int smem = (int)sizeof(Smem);
  if (cuda_ok(cudaFuncSetAttribute(wkv6_bwd_kernel<T, N, COARSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
    return RWKVB200_E_CUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(B * H, N / VS);
  cfg.blockDim = dim3(N);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;      // the CTAs of a unit exchange partial sums
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = N / VS; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cuda_ok(cudaLaunchKernelEx(&cfg, wkv6_bwd_kernel<T, N, COARSE>, (const T*)r, (const T*)k, (const T*)v,
                                 (const T*)w, u, (const T*)d_y, d_sT, ckpt, (T*)dr, (T*)dk, (T*)dv, (T*)dw,
                                 du_partial, d_s0, Tn, H, sel)))
    return RWKVB200_E_CUDA;
  return RWKVB200_OK;
}
}  // namespace

// The backward over the units marked in sel->flags, from checkpoints 64 tokens apart (sel->ckpt_unit_stride
// floats between units); du_partial receives four rows per unit.  No reduction of du.  Head size 64.
int launch_wkv6_bwd_coarse(const void* r, const void* k, const void* v, const void* w, const float* u,
                           const void* d_y, const float* d_sT, const float* ckpt,
                           void* dr, void* dk, void* dv, void* dw, float* du_partial, float* d_s0,
                           int B, int Tn, int H, int dtype, cudaStream_t st, const UnitSel* sel) {
  ProfScope prof("wkv6_bwd_kernel", st);
  RWKVB200_DISPATCH_DTYPE(dtype,
    const int e = launch_bwd_cluster<T, HS, true>(r, k, v, w, u, d_y, d_sT, ckpt, dr, dk, dv, dw, du_partial, d_s0,
                                                  B, Tn, H, st, *sel);
    if (e) return e);
  return check_launch();
}

int launch_wkv6_du_reduce_mixed(const float* part_chunked, const float* part_rec, const int* flags, float* du,
                                int B, int H, cudaStream_t st, int rows) {
  ProfScope prof("wkv6_du_reduce_kernel", st);
  wkv6_du_reduce_mixed_kernel<<<H, 64, 0, st>>>(part_chunked, part_rec, flags, du, B, H, rows);
  return check_launch();
}

int launch_wkv6_bwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                    const void* d_y, const float* d_sT, const float* ckpt,
                    void* dr, void* dk, void* dv, void* dw, float* du_partial, float* du, float* d_s0,
                    int B, int Tn, int H, int dtype, cudaStream_t st, int head_size) {
  {
    ProfScope prof("wkv6_bwd_kernel", st);
    const UnitSel none{nullptr, nullptr, nullptr, 0};
    RWKVB200_DISPATCH_HEAD6(head_size,
      RWKVB200_DISPATCH_DTYPE(dtype,
        const int e = launch_bwd_cluster<T, N, false>(r, k, v, w, u, d_y, d_sT, ckpt, dr, dk, dv, dw, du_partial,
                                                      d_s0, B, Tn, H, st, none);
        if (e) return e));
  }
  int e = check_launch();
  if (e) return e;
  ProfScope prof("wkv6_du_reduce_kernel", st);
  wkv6_du_reduce_kernel<<<H, head_size, 0, st>>>(du_partial, du, B, H);
  return check_launch();
}

}  // namespace rwkvb200
