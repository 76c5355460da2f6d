// Shared helpers for the rwkv_ops_b200 kernels: element-type conversion, vector loads,
// argument checks.  Everything computes in float32; token tensors may be f32, bf16 or f16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rwkv_ops_b200.h"

namespace rwkvb200 {

constexpr int HS = 64;  // head size (key and value)

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Load four consecutive elements (16-byte aligned for f32, 8-byte for 16-bit types) as float4.
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
  float4 f;
  f.x = __uint_as_float(u.x << 16);
  f.y = __uint_as_float(u.x & 0xffff0000u);
  f.z = __uint_as_float(u.y << 16);
  f.w = __uint_as_float(u.y & 0xffff0000u);
  return f;
}
template <> __device__ __forceinline__ float4 load4<__half>(const __half* p) {
  uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
  __half2 h0 = *reinterpret_cast<__half2*>(&u.x), h1 = *reinterpret_cast<__half2*>(&u.y);
  float2 a = __half22float2(h0), b = __half22float2(h1);
  return make_float4(a.x, a.y, b.x, b.y);
}

// The same from shared memory (load4 reads through the read-only global path and must not be given a
// shared-memory address).
template <typename T> __device__ __forceinline__ float4 load4_shared(const T* p);
template <> __device__ __forceinline__ float4 load4_shared<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <> __device__ __forceinline__ float4 load4_shared<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
template <> __device__ __forceinline__ float4 load4_shared<__half>(const __half* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// Store four consecutive elements from a float4 (same alignment rule as load4).
template <typename T> __device__ __forceinline__ void store4(T* p, float4 f);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 f) {
  *reinterpret_cast<float4*>(p) = f;
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 f) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
template <> __device__ __forceinline__ void store4<__half>(__half* p, float4 f) {
  __half2 lo = __floats2half2_rn(f.x, f.y), hi = __floats2half2_rn(f.z, f.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

// The decay every operator applies to its w input.
__device__ __forceinline__ float decay_of(float w) { return expf(-expf(w)); }

// Strides (in elements) of a [B,T,H,64] or [B,H,T,64] token tensor.
struct TokLayout {
  long long sb, st, sh;
  __host__ __device__ TokLayout(int T, int H, int head_first, int hs = HS) {
    sb = (long long)T * H * hs;
    if (head_first) { sh = (long long)T * hs; st = hs; }
    else            { sh = hs;                st = (long long)H * hs; }
  }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Last CUDA runtime error seen by this library (cudaSuccess if none); see rwkvb200_last_cuda_error().
int& last_cuda_error_slot();

inline int cuda_ok(cudaError_t e) {
  if (e == cudaSuccess) return RWKVB200_OK;
  last_cuda_error_slot() = (int)e;
  return RWKVB200_E_CUDA;
}

inline int check_launch() { return cuda_ok(cudaGetLastError()); }

// Brackets one kernel launch with timing events when profiling is on (see profile.cu).
struct ProfScope {
  ProfScope(const char* name, cudaStream_t st);
  ~ProfScope();
  cudaStream_t st_;
  int idx_;
};

// Host-side dispatch on the dtype code.
#define RWKVB200_DISPATCH_DTYPE(dtype, ...)                                  \
  switch (dtype) {                                                           \
    case RWKVB200_F32:  { using T = float;          __VA_ARGS__; break; }    \
    case RWKVB200_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; }    \
    case RWKVB200_F16:  { using T = __half;         __VA_ARGS__; break; }    \
    default: return RWKVB200_E_DTYPE;                                        \
  }

// Which (batch, head) units a recurrent kernel works on, and where their tokens and checkpoints lie.  The
// recurrent kernels double as the exact fallback of the chunked tensor-core paths: a chunked kernel marks
// the units whose decay leaves the range its scaled operands can represent, and the recurrent kernel is
// then launched over all units with `flags` set, so that only the marked ones run.
struct UnitSel {
  const int* flags;             // one entry per unit, nonzero = run it; nullptr = run every unit
  const int* seq_start;         // packed variable-length batch: first token and length of every sequence
  const int* seq_len;           //   (all in batch row 0); nullptr = dense batch
  long long ckpt_unit_stride;   // floats between the checkpoint regions of consecutive units; 0 = dense
};

// Kernel launchers implemented in the .cu files (internal linkage across the library only).
int launch_rwkv7_decode_step(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                             void* state, int state_dtype, void* o, int B, int H, int dtype, cudaStream_t st);
int launch_rwkv7_step(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                      const float* s_in, int n_state, float* s_out, void* o, int B, int H, int dtype,
                      cudaStream_t st);

// Recurrent (token-by-token) RWKV7 forward.  ckpt (may be NULL) receives the state before every
// ckpt_every-th token as [B,H,ceil(T/ckpt_every),64,64]; o and ht may be NULL.
int launch_rwkv7_rec_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                         const float* h0, int n_state, void* o, float* ht, float* ckpt, int ckpt_every,
                         int B, int Tn, int H, int dtype, int head_first, cudaStream_t st,
                         const UnitSel* sel = nullptr, int T_total = 0, int head_size = HS);
int launch_rwkv7_rec_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                         const void* d_o, const float* d_ht, const float* ckpt,
                         void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                         int B, int Tn, int H, int dtype, int head_first, cudaStream_t st,
                         const UnitSel* sel = nullptr, int T_total = 0, int head_size = HS);
constexpr int R7_CKPT = 8;   // tokens between state checkpoints of the recurrent backward

int launch_wkv6_fwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                    const float* s0, int n_state, const int32_t* smap, void* y, float* sT,
                    float* ckpt, int B, int Tn, int H, int dtype, cudaStream_t st, const UnitSel* sel = nullptr,
                    int ckpt_every = 0, int head_size = HS);
int launch_wkv6_bwd_coarse(const void* r, const void* k, const void* v, const void* w, const float* u,
                           const void* d_y, const float* d_sT, const float* ckpt,
                           void* dr, void* dk, void* dv, void* dw, float* du_partial, float* d_s0,
                           int B, int Tn, int H, int dtype, cudaStream_t st, const UnitSel* sel);
int launch_wkv6_du_reduce_mixed(const float* part_chunked, const float* part_rec, const int* flags, float* du,
                                int B, int H, cudaStream_t st, int rows = 1);
int launch_wkv6_bwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                    const void* d_y, const float* d_sT, const float* ckpt,
                    void* dr, void* dk, void* dv, void* dw, float* du_partial, float* du, float* d_s0,
                    int B, int Tn, int H, int dtype, cudaStream_t st, int head_size = HS);
constexpr int W6_CKPT = 8;

// Chunked tcgen05 wkv6 (wkv6_chunked.cu).  `states` (may be NULL) receives the fp32 state at every chunk
// boundary, [B*H][ceil(T/64)+1][64][64].
int launch_wkv6_chunked_fwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                            const float* s0, int n_state, const int32_t* smap, void* y, float* sT,
                            float* states, int* flags, float* handoff, int* hflags, int B, int Tn, int H, int dtype,
                            cudaStream_t st, const int32_t* seq_start = nullptr, const int32_t* seq_len = nullptr,
                            int T_total = 0);
size_t wkv6_chunked_fwd_scratch_bytes(int B, int H);
void wkv6_chunked_fwd_scratch(void* workspace, int B, int H, int** flags, float** handoff, int** hflags);
void wkv6_chunked_workspace_parts(void* workspace, int B, int Tn, int H, int** flags, float** handoff, int** hflags);
size_t wkv6_chunked_bwd_workspace_bytes(int B, int Tn, int H);
size_t wkv6_chunked_flags_bytes(int B, int H);
int launch_wkv6_chunked_bwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                            const float* s0, int n_state, const int32_t* smap, const void* d_y, const float* d_sT,
                            void* dr, void* dk, void* dv, void* dw, float* du, float* d_s0, void* workspace,
                            int B, int Tn, int H, int dtype, bool kept, cudaStream_t st,
                            const int32_t* seq_start = nullptr, const int32_t* seq_len = nullptr, int T_total = 0);

}  // namespace rwkvb200
