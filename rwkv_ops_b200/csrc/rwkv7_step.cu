// RWKV7 single-token decode step: the recurrence of the reference's native operator
// (rwkv_ops/rwkv7_kernel/native_keras_op.py:80-91) for one t, as a bandwidth-bound kernel.
//
// Per (batch, head): read the float32 state S[v][k] (16 KB), the six 64-vectors, write the new
// state (16 KB) and o (64 values).  Algorithmic bytes per unit: 2*64*64*4 + 6*64*e + 64*e
// (e = element size of the token tensors).
//
// One CTA per unit.  A thread owns four rows v = rg + 16*j and 16 bytes of each (four float32 or eight
// bfloat16 consecutive key columns), so a warp's load covers whole state rows and all four loads are in
// flight before first use.  The two dot products over k (S a and S' r) reduce over the lanes that
// share a row.
//
// The state element type ST is float (the reference's state type) or bfloat16 (an option for decode
// loops that keep their state on the device: half the bytes per step, bf16 rounding of the state
// after every token).  The arithmetic is float32 either way.
#include "common.cuh"

namespace rwkvb200 {

// KQ consecutive state values as float32: one 16-byte access either way
__device__ __forceinline__ void load_state(const float* p, float (&x)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  x[0] = f.x; x[1] = f.y; x[2] = f.z; x[3] = f.w;
}
__device__ __forceinline__ void load_state(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { x[2 * i] = __uint_as_float(w[i] << 16); x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
__device__ __forceinline__ void store_state(float* p, const float (&x)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
__device__ __forceinline__ void store_state(__nv_bfloat16* p, const float (&x)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&t);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// KQ = consecutive key columns per thread: 4 for a float32 state (16 lanes per row, 256 threads per
// unit), 8 for a bfloat16 state (8 lanes per row, 128 threads per unit), so that a thread always has
// four 16-byte state loads in flight.
template <typename T, typename ST, int KQ>
__global__ void __launch_bounds__(1024 / KQ, KQ == 4 ? 6 : 8)
rwkv7_step_kernel(const T* __restrict__ r, const T* __restrict__ w, const T* __restrict__ k,
                  const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                  const ST* s_in, int n_state, ST* s_out, T* __restrict__ o, int H) {
  constexpr int LR = HS / KQ;                  // lanes that share a state row
  const int tid = threadIdx.x;
  const int q = tid % LR;                      // key group
  const int rg = tid / LR;                     // row group, 0..15
  __shared__ __align__(16) float vec[5][HS];
  auto load_unit = [&](int unit, float (&X)[4][KQ]) {
    const long long sbase = (n_state == 1 ? (long long)(unit % H) : (long long)unit) * (HS * HS);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (s_in) {
        load_state(s_in + sbase + (rg + 16 * j) * HS + KQ * q, X[j]);
      } else {
#pragma unroll
        for (int c = 0; c < KQ; ++c) X[j][c] = 0.f;
      }
    }
  };
  const int unit = blockIdx.x;                 // b*H + h
  float S[4][KQ];
  load_unit(unit, S);
  ST* Sout = s_out + (long long)unit * (HS * HS);
  const long long vbase = (long long)unit * HS;
  // the five key-indexed vectors go through shared memory (as float32, w already as the decay): held in
  // registers they would cost 5 * KQ registers per thread and with them the CTAs per SM that keep
  // enough state loads in flight
  if (tid < HS) {
    vec[0][tid] = to_f32(r[vbase + tid]);
    vec[1][tid] = decay_of(to_f32(w[vbase + tid]));
    vec[2][tid] = to_f32(k[vbase + tid]);
    vec[3][tid] = to_f32(a[vbase + tid]);
    vec[4][tid] = to_f32(b[vbase + tid]);
  }
  float vv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) vv[j] = to_f32(v[vbase + rg + 16 * j]);

  __syncthreads();
  float sa[4];
  {
    float av[KQ];
#pragma unroll
    for (int c = 0; c < KQ; c += 4) *reinterpret_cast<float4*>(av + c) = *reinterpret_cast<const float4*>(&vec[3][KQ * q + c]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float t = 0.f;
#pragma unroll
      for (int c = 0; c < KQ; ++c) t += S[j][c] * av[c];
      sa[j] = t;
    }
  }
#pragma unroll
  for (int m = LR / 2; m >= 1; m >>= 1)
#pragma unroll
    for (int j = 0; j < 4; ++j) sa[j] += __shfl_xor_sync(0xffffffffu, sa[j], m);

  float oo[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < KQ; c += 4) {
    const float4 r4 = *reinterpret_cast<const float4*>(&vec[0][KQ * q + c]);
    const float4 d4 = *reinterpret_cast<const float4*>(&vec[1][KQ * q + c]);
    const float4 k4 = *reinterpret_cast<const float4*>(&vec[2][KQ * q + c]);
    const float4 b4 = *reinterpret_cast<const float4*>(&vec[4][KQ * q + c]);
    const float rv[4] = {r4.x, r4.y, r4.z, r4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
    const float kv[4] = {k4.x, k4.y, k4.z, k4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        S[j][c + m] = S[j][c + m] * dv[m] + sa[j] * bv[m] + vv[j] * kv[m];
        oo[j] += S[j][c + m] * rv[m];
      }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) store_state(Sout + (rg + 16 * j) * HS + KQ * q, S[j]);
#pragma unroll
  for (int m = LR / 2; m >= 1; m >>= 1)
#pragma unroll
    for (int j = 0; j < 4; ++j) oo[j] += __shfl_xor_sync(0xffffffffu, oo[j], m);
  if (q == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) o[vbase + rg + 16 * j] = from_f32<T>(oo[j]);
  }
}

// The bfloat16-state step.  A unit moves half the bytes of the float32 case, so twice as many bytes per thread
// have to be in flight to keep the memory system as busy: a thread owns EIGHT rows v = rg + 8*j and 16 bytes
// (eight key columns) of each, 64 threads per unit, two units per CTA.  The eight rows stay packed in
// registers (32 of them) and are unpacked twice, once for S a and once for the update, instead of living
// unpacked in 64 registers: that is what lets five such CTAs share an SM (80 KB of state loads in flight;
// a bound of six CTAs spills and measured slower, 61 against 55 us at B 256 x H 64).
template <typename T>
__global__ void __launch_bounds__(128, 5)
rwkv7_step_bf16state_kernel(const T* __restrict__ r, const T* __restrict__ w, const T* __restrict__ k,
                            const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                            __nv_bfloat16* state, T* __restrict__ o, int n_units) {
  constexpr int ROWS = 8, KQ = 8, LR = HS / KQ;      // 8 lanes share a state row
  const int tid = threadIdx.x, usel = tid >> 6, tu = tid & 63;
  const int q = tu % LR, rg = tu / LR;                 // key group, row group 0..7
  __shared__ __align__(16) float vec[2][6][HS];   // r, decay, k, a, b, v
  const int unit = 2 * blockIdx.x + usel;
  const bool live = unit < n_units;
  __nv_bfloat16* S = state + (long long)(live ? unit : 0) * (HS * HS);
  const long long vbase = (long long)(live ? unit : 0) * HS;
  uint4 P[ROWS];
#pragma unroll
  for (int j = 0; j < ROWS; ++j)
    P[j] = live ? *reinterpret_cast<const uint4*>(S + (rg + 8 * j) * HS + KQ * q) : make_uint4(0u, 0u, 0u, 0u);
  if (live) {      // tu = 0..63: one element of each key-indexed vector
    vec[usel][0][tu] = to_f32(r[vbase + tu]);
    vec[usel][1][tu] = decay_of(to_f32(w[vbase + tu]));
    vec[usel][2][tu] = to_f32(k[vbase + tu]);
    vec[usel][3][tu] = to_f32(a[vbase + tu]);
    vec[usel][4][tu] = to_f32(b[vbase + tu]);
    vec[usel][5][tu] = to_f32(v[vbase + tu]);
  }
  __syncthreads();

  // Both passes walk the eight columns as four packed pairs (word c of every row), with only that pair's
  // vector entries in registers; the second pass overwrites the packed words in place.
  auto word = [](uint4& u, int c) -> uint32_t& { return c == 0 ? u.x : c == 1 ? u.y : c == 2 ? u.z : u.w; };
  float sa[ROWS], oo[ROWS];
#pragma unroll
  for (int j = 0; j < ROWS; ++j) { sa[j] = 0.f; oo[j] = 0.f; }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float2 a2 = *reinterpret_cast<const float2*>(&vec[usel][3][KQ * q + 2 * c]);
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
      const uint32_t u = word(P[j], c);
      sa[j] += __uint_as_float(u << 16) * a2.x + __uint_as_float(u & 0xffff0000u) * a2.y;
    }
  }
#pragma unroll
  for (int m = LR / 2; m >= 1; m >>= 1)
#pragma unroll
    for (int j = 0; j < ROWS; ++j) sa[j] += __shfl_xor_sync(0xffffffffu, sa[j], m);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float2 r2 = *reinterpret_cast<const float2*>(&vec[usel][0][KQ * q + 2 * c]);
    const float2 d2 = *reinterpret_cast<const float2*>(&vec[usel][1][KQ * q + 2 * c]);
    const float2 k2 = *reinterpret_cast<const float2*>(&vec[usel][2][KQ * q + 2 * c]);
    const float2 b2 = *reinterpret_cast<const float2*>(&vec[usel][4][KQ * q + 2 * c]);
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
      const uint32_t u = word(P[j], c);
      const float vj = vec[usel][5][rg + 8 * j];
      const float s0 = __uint_as_float(u << 16) * d2.x + sa[j] * b2.x + vj * k2.x;
      const float s1 = __uint_as_float(u & 0xffff0000u) * d2.y + sa[j] * b2.y + vj * k2.y;
      // the output uses the float32 value of the new state, as the float32-state kernel does; the stored
      // state is its bfloat16 rounding
      oo[j] += s0 * r2.x + s1 * r2.y;
      const __nv_bfloat162 pk = __floats2bfloat162_rn(s0, s1);
      word(P[j], c) = *reinterpret_cast<const uint32_t*>(&pk);
    }
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < ROWS; ++j) *reinterpret_cast<uint4*>(S + (rg + 8 * j) * HS + KQ * q) = P[j];
  }
#pragma unroll
  for (int m = LR / 2; m >= 1; m >>= 1)
#pragma unroll
    for (int j = 0; j < ROWS; ++j) oo[j] += __shfl_xor_sync(0xffffffffu, oo[j], m);
  if (q == 0 && live) {
#pragma unroll
    for (int j = 0; j < ROWS; ++j) o[vbase + rg + 8 * j] = from_f32<T>(oo[j]);
  }
}

int launch_rwkv7_step(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                      const float* s_in, int n_state, float* s_out, void* o, int B, int H, int dtype,
                      cudaStream_t st) {
  ProfScope prof("rwkv7_step_kernel", st);
  RWKVB200_DISPATCH_DTYPE(dtype,
    rwkv7_step_kernel<T, float, 4><<<B * H, 256, 0, st>>>(
        (const T*)r, (const T*)w, (const T*)k, (const T*)v, (const T*)a, (const T*)b, s_in, n_state, s_out, (T*)o, H));
  return check_launch();
}

// in place on a state the caller keeps on the device: [B][H][64][64], float32 or bfloat16
int launch_rwkv7_decode_step(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                             void* state, int state_dtype, void* o, int B, int H, int dtype, cudaStream_t st) {
  ProfScope prof("rwkv7_step_kernel", st);
  if (state_dtype == RWKVB200_BF16) {
    RWKVB200_DISPATCH_DTYPE(dtype,
      rwkv7_step_bf16state_kernel<T><<<(B * H + 1) / 2, 128, 0, st>>>(
          (const T*)r, (const T*)w, (const T*)k, (const T*)v, (const T*)a, (const T*)b, (__nv_bfloat16*)state, (T*)o,
          B * H));
  } else {
    RWKVB200_DISPATCH_DTYPE(dtype,
      rwkv7_step_kernel<T, float, 4><<<B * H, 256, 0, st>>>(
          (const T*)r, (const T*)w, (const T*)k, (const T*)v, (const T*)a, (const T*)b, (const float*)state, B,
          (float*)state, (T*)o, H));
  }
  return check_launch();
}

}  // namespace rwkvb200
