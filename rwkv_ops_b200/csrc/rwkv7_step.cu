// RWKV7 single-token decode step: the recurrence of the reference's native operator
// (rwkv_ops/rwkv7_kernel/native_keras_op.py:80-91) for one t, as a bandwidth-bound kernel.
//
// Per (batch, head): read the float32 state S[v][k] (16 KB), the six 64-vectors, write the new
// state (16 KB) and o (64 values).  Algorithmic bytes per unit: 2*64*64*4 + 6*64*e + 64*e
// (e = element size of the token tensors).
//
// One CTA of 256 threads per unit.  A thread owns four rows v = (tid>>4) + 16*j and four
// consecutive key columns k = 4*(tid&15).., i.e. one float4 of each of its rows, so a warp's
// load covers two whole 256-byte state rows and all four loads are in flight before first use.
// The two dot products over k (S a and S' r) reduce over the 16 lanes that share a row.
#include "common.cuh"

namespace rwkvb200 {

template <typename T>
__global__ void __launch_bounds__(256)
rwkv7_step_kernel(const T* __restrict__ r, const T* __restrict__ w, const T* __restrict__ k,
                  const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                  const float* s_in, int n_state, float* s_out, T* __restrict__ o, int H) {
  const int unit = blockIdx.x;                 // b*H + h
  const int tid = threadIdx.x;
  const int q = tid & 15;                      // key quad
  const int rg = tid >> 4;                     // row group
  const int h = unit % H;
  const long long sbase = (n_state == 1 ? (long long)h : (long long)unit) * (HS * HS);
  const float* Sin = s_in ? s_in + sbase : nullptr;
  float* Sout = s_out + (long long)unit * (HS * HS);
  const long long vbase = (long long)unit * HS;

  float4 S[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int row = rg + 16 * j;
    S[j] = Sin ? *reinterpret_cast<const float4*>(Sin + row * HS + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float4 r4 = load4(r + vbase + 4 * q);
  const float4 w4 = load4(w + vbase + 4 * q);
  const float4 k4 = load4(k + vbase + 4 * q);
  const float4 a4 = load4(a + vbase + 4 * q);
  const float4 b4 = load4(b + vbase + 4 * q);
  float vv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) vv[j] = to_f32(v[vbase + rg + 16 * j]);
  const float4 d4 = make_float4(decay_of(w4.x), decay_of(w4.y), decay_of(w4.z), decay_of(w4.w));

  float sa[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) sa[j] = S[j].x * a4.x + S[j].y * a4.y + S[j].z * a4.z + S[j].w * a4.w;
#pragma unroll
  for (int m = 8; m >= 1; m >>= 1)
#pragma unroll
    for (int j = 0; j < 4; ++j) sa[j] += __shfl_xor_sync(0xffffffffu, sa[j], m);

  float oo[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    S[j].x = S[j].x * d4.x + sa[j] * b4.x + vv[j] * k4.x;
    S[j].y = S[j].y * d4.y + sa[j] * b4.y + vv[j] * k4.y;
    S[j].z = S[j].z * d4.z + sa[j] * b4.z + vv[j] * k4.z;
    S[j].w = S[j].w * d4.w + sa[j] * b4.w + vv[j] * k4.w;
    oo[j] = S[j].x * r4.x + S[j].y * r4.y + S[j].z * r4.z + S[j].w * r4.w;
    *reinterpret_cast<float4*>(Sout + (rg + 16 * j) * HS + 4 * q) = S[j];
  }
#pragma unroll
  for (int m = 8; m >= 1; m >>= 1)
#pragma unroll
    for (int j = 0; j < 4; ++j) oo[j] += __shfl_xor_sync(0xffffffffu, oo[j], m);
  if (q == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) o[vbase + rg + 16 * j] = from_f32<T>(oo[j]);
  }
}

int launch_rwkv7_step(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                      const float* s_in, int n_state, float* s_out, void* o, int B, int H, int dtype,
                      cudaStream_t st) {
  ProfScope prof("rwkv7_step_kernel", st);
  RWKVB200_DISPATCH_DTYPE(dtype,
    rwkv7_step_kernel<T><<<B * H, 256, 0, st>>>((const T*)r, (const T*)w, (const T*)k, (const T*)v,
                                                (const T*)a, (const T*)b, s_in, n_state, s_out, (T*)o, H));
  return check_launch();
}

}  // namespace rwkvb200
