// RWKV7 generalized delta rule, token-by-token in float32 (forward and backward).
//
// This is the float32-exact path: the same arithmetic as the reference's native operator
// (rwkv_ops/rwkv7_kernel/native_keras_op.py:80-91), used for float32 token tensors and as the
// on-device cross-check of the chunked tensor-core path.
//
//   d_t = exp(-exp(w_t));  sa_t = S_{t-1} a_t;  S_t = S_{t-1} diag(d_t) + sa_t b_t^T + v_t k_t^T;  o_t = S_t r_t
//
// with S[v][k].  Row v of S never mixes with another row, so the 64 value rows are split over
// four CTAs (16 rows each): grid (B*H, 4), 64 threads.  In the "row role" thread (vl = tid>>2,
// kq = tid&3) holds S[vl][16*kq .. 16*kq+15] in registers and reductions over k take two shuffles.
//
// Backward.  With dS the gradient of the state flowing from the future,
//   dS += do_t r_t^T;  dr_t = S_t^T do_t;  dv_t = dS k_t;  dk_t = dS^T v_t;  dsa = dS b_t;  db_t = dS^T sa_t;
//   dd_t[k] = sum_v dS[v,k] S_{t-1}[v,k];  da_t = S_{t-1}^T dsa;  dS <- dS diag(d_t) + dsa a_t^T;
//   dw_t = dd_t * d_t * (-exp(w_t)).
// It needs S_{t-1} and S_t for every token: a first forward sweep stores the state every R7_CKPT
// tokens (the workspace), and the backward kernel walks the chunks in reverse, re-running each chunk
// forward into shared memory before sweeping it backward.  Reductions over v (dr, dk, db, da, dd) need
// all 64 rows: each thread also keeps a "column role" copy dS[0..15][k = tid] of the CTA's slab, the
// four CTAs of a (batch, head) form a thread-block cluster, and after each chunk every CTA sums the
// four partial results of a quarter of the chunk's tokens through distributed shared memory, in a
// fixed order (deterministic, no atomics, no scratch beyond the checkpoints).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace rwkvb200 {

namespace {

constexpr int VS = 16;        // value rows per CTA
// A staged vector of N key channels is kept as segments of 16 with 4 floats of padding between them: the lanes
// of a quarter warp read the same 16 bytes of N/16 different segments, which 64 bytes apart would share banks.
__host__ __device__ constexpr int padk(int k) { return k + ((k >> 4) << 2); }
template <int N> __host__ __device__ constexpr int NP() { return N + N / 4; }
constexpr int CK = R7_CKPT;   // chunk of the backward = checkpoint interval
// The kernels are templates over the head size N (64 or 128): N / 16 CTAs per (batch, head), N threads per
// CTA, N / 16 lanes share a state row (16 key columns each).

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
template <typename T, int N>
__global__ void __launch_bounds__(N)
rwkv7_rec_fwd_kernel(const T* __restrict__ r, const T* __restrict__ w, const T* __restrict__ k,
                     const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                     const float* __restrict__ h0, int n_state, T* __restrict__ o, float* __restrict__ ht,
                     float* __restrict__ ckpt, int ckpt_every, int Tn_dense, int H, TokLayout lay, UnitSel sel) {
  constexpr int TL = N > 64 ? 8 : 16;   // tokens staged per tile (the static shared memory holds 16 only up to N = 64)
  __shared__ __align__(16) float tile[TL][5][NP<N>()];   // r, d, k, a, b
  __shared__ __align__(16) float vt[TL][VS];
  __shared__ __align__(16) float ot[TL][VS];

  const int unit = blockIdx.x, y = blockIdx.y, tid = threadIdx.x;
  if (sel.flags && sel.flags[unit] == 0) return;      // only the selected units run
  const int bi = unit / H, hi = unit % H;
  constexpr int KSEG = N / 16;      // lanes per state row
  const int vl = tid / KSEG, kq = tid % KSEG;
  // a packed batch keeps its sequences end to end in batch row 0
  const int Tn = sel.seq_len ? sel.seq_len[bi] : Tn_dense;
  const long long base = sel.seq_start ? hi * lay.sh + sel.seq_start[bi] * lay.st : bi * lay.sb + hi * lay.sh;
  const long long ckpt_unit = sel.ckpt_unit_stride ? sel.ckpt_unit_stride
                                                   : (long long)((Tn_dense + ckpt_every - 1) / ckpt_every) * N * N;

  float S[16];
  if (h0 && n_state > 0) {
    const float* p = h0 + ((long long)(n_state == 1 ? hi : unit) * N + (y * VS + vl)) * N + 16 * kq;
#pragma unroll
    for (int j = 0; j < 16; j += 4) {
      float4 f = *reinterpret_cast<const float4*>(p + j);
      S[j] = f.x; S[j + 1] = f.y; S[j + 2] = f.z; S[j + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) S[j] = 0.f;
  }

  // The inputs of a tile travel global memory -> registers -> shared memory, and the loads of tile i + 1 are
  // issued before the tokens of tile i are worked on: few warps share an SM here (the grid is B*H*N/16 CTAs of N
  // threads), so a load that is waited for where it is issued costs its full latency every time.
  constexpr int PER = TL * 5 / 4;      // float4 per thread per tile: TL tokens x 5 vectors x N/4 quads over N threads
  float4 buf[PER], vbuf = make_float4(0.f, 0.f, 0.f, 0.f);
  const int quad = tid % (N / 4), rq = tid / (N / 4);      // this thread's quad of channels; its rows are rq + 4 m
  auto fetch = [&](int t0) {
    const int nt = min(TL, Tn - t0);
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int row = rq + 4 * m, tl = row / 5, which = row % 5;
      const T* src = which == 0 ? r : which == 1 ? w : which == 2 ? k : which == 3 ? a : b;
      buf[m] = tl < nt ? load4(src + base + (long long)(t0 + tl) * lay.st + 4 * quad) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (tid < nt * 4)
      vbuf = load4(v + base + (long long)(t0 + (tid >> 2)) * lay.st + y * VS + 4 * (tid & 3));
  };
  auto stash = [&]() {
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int row = rq + 4 * m, tl = row / 5, which = row % 5;
      float4 f = buf[m];
      if (which == 1) f = make_float4(decay_of(f.x), decay_of(f.y), decay_of(f.z), decay_of(f.w));
      *reinterpret_cast<float4*>(&tile[tl][which][padk(4 * quad)]) = f;
    }
    if (tid < TL * 4) *reinterpret_cast<float4*>(&vt[tid >> 2][4 * (tid & 3)]) = vbuf;
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
        float* p = ckpt + unit * ckpt_unit + (((long long)(t / ckpt_every) * N) + (y * VS + vl)) * N + 16 * kq;
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(p + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
      }
      const float* tr = &tile[tl][0][20 * kq];
      const float* td = &tile[tl][1][20 * kq];
      const float* tk = &tile[tl][2][20 * kq];
      const float* ta = &tile[tl][3][20 * kq];
      const float* tb = &tile[tl][4][20 * kq];
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        s0 += S[j] * ta[j]; s1 += S[j + 1] * ta[j + 1]; s2 += S[j + 2] * ta[j + 2]; s3 += S[j + 3] * ta[j + 3];
      }
      float sa = (s0 + s1) + (s2 + s3);
#pragma unroll
      for (int m = 1; m < KSEG; m <<= 1) sa += __shfl_xor_sync(0xffffffffu, sa, m);
      const float vv = vt[tl][vl];
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        S[j]     = S[j]     * td[j]     + sa * tb[j]     + vv * tk[j];
        S[j + 1] = S[j + 1] * td[j + 1] + sa * tb[j + 1] + vv * tk[j + 1];
        S[j + 2] = S[j + 2] * td[j + 2] + sa * tb[j + 2] + vv * tk[j + 2];
        S[j + 3] = S[j + 3] * td[j + 3] + sa * tb[j + 3] + vv * tk[j + 3];
        o0 += S[j] * tr[j]; o1 += S[j + 1] * tr[j + 1]; o2 += S[j + 2] * tr[j + 2]; o3 += S[j + 3] * tr[j + 3];
      }
      float oo = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int m = 1; m < KSEG; m <<= 1) oo += __shfl_xor_sync(0xffffffffu, oo, m);
      if (kq == 0) ot[tl][vl] = oo;
    }
    __syncthreads();
    if (o && tid < nt * 4) {
      const int tl = tid >> 2, quad = tid & 3;
      store4(o + base + (long long)(t0 + tl) * lay.st + y * VS + 4 * quad,
             *reinterpret_cast<const float4*>(&ot[tl][4 * quad]));
    }
    // the next tile's staging writes tile/vt only after every thread has passed the barrier
    // above; ot is rewritten only after the next barrier pair
  }
  if (ht) {
    float* p = ht + ((long long)unit * N + (y * VS + vl)) * N + 16 * kq;
#pragma unroll
    for (int j = 0; j < 16; j += 4)
      *reinterpret_cast<float4*>(p + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
  }
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
template <int N>
struct BwdSmem {
  float tile[CK][6][NP<N>()];         // r, d, exp(w), k, a, b
  float vt[CK][VS];
  float dot[CK][VS];
  float sa[CK][VS];
  float dvt[CK][VS];
  float dsa[2][VS];
  float Sbuf[CK + 1][VS][N + 1]; // state before token i of the chunk (i = nt: after the last), padded rows
  float part[2][CK][5][N];      // per-chunk partial dr, dk, db, da, dd of this CTA's 16 rows
};

// launched as clusters of N / 16 CTAs along y (one per 16 value rows of a unit)
template <typename T, int N>
__global__ void __launch_bounds__(N)
rwkv7_rec_bwd_kernel(const T* __restrict__ r, const T* __restrict__ w, const T* __restrict__ k,
                     const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                     const T* __restrict__ d_o, const float* __restrict__ d_ht, const float* __restrict__ ckpt,
                     T* __restrict__ dr, T* __restrict__ dw, T* __restrict__ dk, T* __restrict__ dv,
                     T* __restrict__ da, T* __restrict__ db, float* __restrict__ d_h0,
                     int Tn_dense, int H, TokLayout lay, UnitSel sel) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  BwdSmem<N>& sm = *reinterpret_cast<BwdSmem<N>*>(smem_raw);
  constexpr int KSEG = N / 16, NQ = N / VS;
  cg::cluster_group cluster = cg::this_cluster();

  const int unit = blockIdx.x, y = blockIdx.y, tid = threadIdx.x;
  if (sel.flags && sel.flags[unit] == 0) return;      // the four CTAs of a cluster share the unit: all leave
  const int bi = unit / H, hi = unit % H;
  const int vl = tid / KSEG, kq = tid % KSEG;   // row role
  const int kc = tid;                      // column role
  const int Tn = sel.seq_len ? sel.seq_len[bi] : Tn_dense;
  const long long base = sel.seq_start ? hi * lay.sh + sel.seq_start[bi] * lay.st : bi * lay.sb + hi * lay.sh;
  const int NC = (Tn + CK - 1) / CK;
  const long long ckpt_unit = sel.ckpt_unit_stride ? sel.ckpt_unit_stride
                                                   : (long long)((Tn_dense + CK - 1) / CK) * N * N;

  float dSr[16], dSc[VS];
  if (d_ht) {
    const float* p = d_ht + ((long long)unit * N + (y * VS + vl)) * N + 16 * kq;
#pragma unroll
    for (int j = 0; j < 16; ++j) dSr[j] = p[j];
#pragma unroll
    for (int i = 0; i < VS; ++i) dSc[i] = d_ht[((long long)unit * N + (y * VS + i)) * N + kc];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) dSr[j] = 0.f;
#pragma unroll
    for (int i = 0; i < VS; ++i) dSc[i] = 0.f;
  }

  // The inputs and the checkpoint of chunk c - 1 are requested (into registers) before chunk c is worked on,
  // and written to shared memory when chunk c is done: see the forward kernel.
  constexpr int PER = CK * 5 / 4;      // float4 per thread per chunk: CK tokens x (r, w, k, a, b) x N/4 quads
  float4 buf[PER], vbuf = make_float4(0.f, 0.f, 0.f, 0.f), dobuf = vbuf, Snext[4];
  const int quad = tid % (N / 4), rq = tid / (N / 4);
  auto fetch = [&](int c) {
    const int t0 = c * CK, nt = min(CK, Tn - t0);
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int row = rq + 4 * m, tl = row / 5, which = row % 5;
      const T* src = which == 0 ? r : which == 1 ? w : which == 2 ? k : which == 3 ? a : b;
      buf[m] = tl < nt ? load4(src + base + (long long)(t0 + tl) * lay.st + 4 * quad) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (tid < nt * 4) {
      const long long off = base + (long long)(t0 + (tid >> 2)) * lay.st + y * VS + 4 * (tid & 3);
      vbuf = load4(v + off);
      dobuf = load4(d_o + off);
    }
    const float* p = ckpt + unit * ckpt_unit + (((long long)c * N) + (y * VS + vl)) * N + 16 * kq;
#pragma unroll
    for (int j = 0; j < 4; ++j) Snext[j] = *reinterpret_cast<const float4*>(p + 4 * j);
  };
  // tile rows: 0 r, 1 d, 2 exp(w), 3 k, 4 a, 5 b
  auto stash = [&]() {
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int row = rq + 4 * m, tl = row / 5, which = row % 5;
      const float4 f = buf[m];
      if (which == 1) {
        *reinterpret_cast<float4*>(&sm.tile[tl][1][padk(4 * quad)]) =
            make_float4(decay_of(f.x), decay_of(f.y), decay_of(f.z), decay_of(f.w));
        *reinterpret_cast<float4*>(&sm.tile[tl][2][padk(4 * quad)]) = make_float4(expf(f.x), expf(f.y), expf(f.z), expf(f.w));
      } else {
        *reinterpret_cast<float4*>(&sm.tile[tl][which == 0 ? 0 : which + 1][padk(4 * quad)]) = f;
      }
    }
    if (tid < CK * 4) {
      *reinterpret_cast<float4*>(&sm.vt[tid >> 2][4 * (tid & 3)]) = vbuf;
      *reinterpret_cast<float4*>(&sm.dot[tid >> 2][4 * (tid & 3)]) = dobuf;
    }
  };
  if (NC > 0) fetch(NC - 1);
  for (int c = NC - 1; c >= 0; --c) {
    const int t0 = c * CK, nt = min(CK, Tn - t0), pb = c & 1;
    // ---- the chunk's inputs, and its checkpoint (row role) for the forward re-run
    stash();
    float S[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) { S[4 * j] = Snext[j].x; S[4 * j + 1] = Snext[j].y; S[4 * j + 2] = Snext[j].z; S[4 * j + 3] = Snext[j].w; }
    __syncthreads();
    if (c > 0) fetch(c - 1);
    for (int tl = 0; tl < nt; ++tl) {
      const float* td = &sm.tile[tl][1][20 * kq];
      const float* tk = &sm.tile[tl][3][20 * kq];
      const float* ta = &sm.tile[tl][4][20 * kq];
      const float* tb = &sm.tile[tl][5][20 * kq];
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        sm.Sbuf[tl][vl][16 * kq + j] = S[j];
        sm.Sbuf[tl][vl][16 * kq + j + 1] = S[j + 1];
        s0 += S[j] * ta[j]; s1 += S[j + 1] * ta[j + 1];
      }
      float sa = s0 + s1;
#pragma unroll
      for (int m = 1; m < KSEG; m <<= 1) sa += __shfl_xor_sync(0xffffffffu, sa, m);
      if (kq == 0) sm.sa[tl][vl] = sa;
      const float vv = sm.vt[tl][vl];
#pragma unroll
      for (int j = 0; j < 16; ++j) S[j] = S[j] * td[j] + sa * tb[j] + vv * tk[j];
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) sm.Sbuf[nt][vl][16 * kq + j] = S[j];
    __syncthreads();

    // ---- sweep the chunk backward
    float St[VS], Sp[VS];
#pragma unroll
    for (int i = 0; i < VS; ++i) St[i] = sm.Sbuf[nt][i][kc];
    for (int tl = nt - 1; tl >= 0; --tl) {
      const int buf = tl & 1;
      const float rk = sm.tile[tl][0][padk(kc)], dk_ = sm.tile[tl][1][padk(kc)], ak = sm.tile[tl][4][padk(kc)];
      const float* tr = &sm.tile[tl][0][20 * kq];
      const float* td = &sm.tile[tl][1][20 * kq];
      const float* tk = &sm.tile[tl][3][20 * kq];
      const float* ta = &sm.tile[tl][4][20 * kq];
      const float* tb = &sm.tile[tl][5][20 * kq];
      // row role: dS += do r^T ; dv = dS k ; dsa = dS b
      const float dor = sm.dot[tl][vl];
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        dSr[j] += dor * tr[j]; dSr[j + 1] += dor * tr[j + 1];
        a0 += dSr[j] * tk[j]; a1 += dSr[j + 1] * tk[j + 1];
        b0 += dSr[j] * tb[j]; b1 += dSr[j + 1] * tb[j + 1];
      }
      float dvv = a0 + a1, dsa = b0 + b1;
#pragma unroll
      for (int m = 1; m < KSEG; m <<= 1) {
        dvv += __shfl_xor_sync(0xffffffffu, dvv, m);
        dsa += __shfl_xor_sync(0xffffffffu, dsa, m);
      }
      if (kq == 0) { sm.dvt[tl][vl] = dvv; sm.dsa[buf][vl] = dsa; }
      // column role, part 1 (does not need dsa)
      float p_dr = 0.f, p_dk = 0.f, p_db = 0.f, p_dd = 0.f;
#pragma unroll
      for (int i = 0; i < VS; ++i) {
        Sp[i] = sm.Sbuf[tl][i][kc];
        const float doi = sm.dot[tl][i];
        dSc[i] += doi * rk;
        p_dr += St[i] * doi;
        p_dk += dSc[i] * sm.vt[tl][i];
        p_db += dSc[i] * sm.sa[tl][i];
        p_dd += dSc[i] * Sp[i];
      }
      __syncthreads();   // dsa of this token visible to every thread
      float p_da = 0.f;
#pragma unroll
      for (int i = 0; i < VS; ++i) {
        const float ds = sm.dsa[buf][i];
        p_da += Sp[i] * ds;
        dSc[i] = dSc[i] * dk_ + ds * ak;
        St[i] = Sp[i];
      }
      const float dsr = sm.dsa[buf][vl];
#pragma unroll
      for (int j = 0; j < 16; ++j) dSr[j] = dSr[j] * td[j] + dsr * ta[j];
      sm.part[pb][tl][0][kc] = p_dr;
      sm.part[pb][tl][1][kc] = p_dk;
      sm.part[pb][tl][2][kc] = p_db;
      sm.part[pb][tl][3][kc] = p_da;
      sm.part[pb][tl][4][kc] = p_dd;
    }
    // ---- dv rows of this CTA
    __syncthreads();
    for (int i = tid; i < nt * VS; i += N) {
      const int tl = i >> 4, vi = i & 15;
      dv[base + (long long)(t0 + tl) * lay.st + y * VS + vi] = from_f32<T>(sm.dvt[tl][vi]);
    }
    // ---- sum the four CTAs' partial column results; this CTA finishes tokens tl = y, y+NQ, ...
    cluster.sync();
    for (int tl = y; tl < nt; tl += NQ) {
      float acc[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int rk_ = 0; rk_ < NQ; ++rk_) {
        const float* rp = cluster.map_shared_rank(&sm.part[pb][tl][0][0], rk_);
#pragma unroll
        for (int qn = 0; qn < 5; ++qn) acc[qn] += rp[qn * N + kc];
      }
      const long long off = base + (long long)(t0 + tl) * lay.st + kc;
      dr[off] = from_f32<T>(acc[0]);
      dk[off] = from_f32<T>(acc[1]);
      db[off] = from_f32<T>(acc[2]);
      da[off] = from_f32<T>(acc[3]);
      dw[off] = from_f32<T>(acc[4] * sm.tile[tl][1][padk(kc)] * (-sm.tile[tl][2][padk(kc)]));
    }
    // part[pb] is rewritten two chunks later, after the next chunk's cluster.sync(); the tile is
    // rewritten by the next chunk's staging, which only this CTA reads
    __syncthreads();
  }
  if (d_h0) {
    float* p = d_h0 + ((long long)unit * N + (y * VS + vl)) * N + 16 * kq;
#pragma unroll
    for (int j = 0; j < 16; ++j) p[j] = dSr[j];
  }
  cluster.sync();   // no CTA leaves while a peer may still read its shared memory
}

}  // namespace

// head size 64 or 128
#define RWKVB200_DISPATCH_HEAD(hs, ...)                           \
  switch (hs) {                                                   \
    case 64:  { constexpr int N = 64;  __VA_ARGS__; break; }      \
    case 128: { constexpr int N = 128; __VA_ARGS__; break; }      \
    default: return RWKVB200_E_UNSUPPORTED;                       \
  }

int launch_rwkv7_rec_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                         const float* h0, int n_state, void* o, float* ht, float* ckpt, int ckpt_every,
                         int B, int Tn, int H, int dtype, int head_first, cudaStream_t st, const UnitSel* sel_,
                         int T_total, int head_size) {
  TokLayout lay(T_total ? T_total : Tn, H, head_first, head_size);
  const UnitSel sel = sel_ ? *sel_ : UnitSel{nullptr, nullptr, nullptr, 0};
  ProfScope prof("rwkv7_rec_fwd_kernel", st);
  RWKVB200_DISPATCH_HEAD(head_size,
    dim3 grid(B * H, N / VS);
    RWKVB200_DISPATCH_DTYPE(dtype,
      rwkv7_rec_fwd_kernel<T, N><<<grid, N, 0, st>>>((const T*)r, (const T*)w, (const T*)k, (const T*)v, (const T*)a,
                                                     (const T*)b, h0, n_state, (T*)o, ht, ckpt, ckpt_every, Tn, H,
                                                     lay, sel)));
  return check_launch();
}

int launch_rwkv7_rec_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                         const void* d_o, const float* d_ht, const float* ckpt,
                         void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                         int B, int Tn, int H, int dtype, int head_first, cudaStream_t st, const UnitSel* sel_,
                         int T_total, int head_size) {
  TokLayout lay(T_total ? T_total : Tn, H, head_first, head_size);
  const UnitSel sel = sel_ ? *sel_ : UnitSel{nullptr, nullptr, nullptr, 0};
  ProfScope prof("rwkv7_rec_bwd_kernel", st);
  RWKVB200_DISPATCH_HEAD(head_size,
    const int smem = (int)sizeof(BwdSmem<N>);
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
    RWKVB200_DISPATCH_DTYPE(dtype,
      if (cuda_ok(cudaFuncSetAttribute(rwkv7_rec_bwd_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
        return RWKVB200_E_CUDA;
      if (cuda_ok(cudaLaunchKernelEx(&cfg, rwkv7_rec_bwd_kernel<T, N>, (const T*)r, (const T*)w, (const T*)k,
                                     (const T*)v, (const T*)a, (const T*)b, (const T*)d_o, d_ht, ckpt, (T*)dr, (T*)dw,
                                     (T*)dk, (T*)dv, (T*)da, (T*)db, d_h0, Tn, H, lay, sel)))
        return RWKVB200_E_CUDA));
  return check_launch();
}

}  // namespace rwkvb200
