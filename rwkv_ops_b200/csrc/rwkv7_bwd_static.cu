// rwkvb200_rwkv7_bwd_static: the recurrent RWKV7 backward for callers that cannot allocate.
//
// The regular backward entry point needs a caller-provided workspace for its state checkpoints.
// Some hosts cannot provide one: an operator plugin whose enqueue hook is handed only its input and
// output buffers and is forbidden to call cudaMalloc (the call synchronises the whole device and the
// host framework owns the memory budget), or a serving process that reserved all device memory at
// start-up.  For them the checkpoints live in a fixed array in the library's own device image.
//
// Cost and limits: the array below is part of the module, so every GPU that loads this library
// holds RWKVB200_STATIC_SCRATCH_BYTES of device memory until the process exits.  A call whose
// checkpoints do not fit returns RWKVB200_E_TOO_LARGE.  All calls share the one array: it keeps
// whatever the previous call left in it, and two calls that overlap on the GPU (different streams,
// or different host threads) overwrite each other's checkpoints and race.  Nothing in it has to start
// at zero: the forward sweep rewrites every checkpoint the backward sweep reads.
#include <mutex>

#include "common.cuh"

using namespace rwkvb200;

namespace {

constexpr size_t STATIC_SCRATCH_BYTES = RWKVB200_STATIC_SCRATCH_BYTES;
constexpr int MAX_DEVICES = 64;

// In host code this name is only a handle for the runtime's symbol table, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

std::mutex g_mu;
float* g_scratch_ptr[MAX_DEVICES] = {};

// Device address of the array on the current device, looked up once per device.
int static_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return RWKVB200_E_CUDA;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) {
      cudaGetLastError();
      return RWKVB200_E_CUDA;
    }
    g_scratch_ptr[dev] = reinterpret_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return RWKVB200_OK;
}

}  // namespace

extern "C" {

size_t rwkvb200_rwkv7_bwd_static_capacity_bytes(void) { return STATIC_SCRATCH_BYTES; }

int rwkvb200_rwkv7_bwd_static(const void* r, const void* w, const void* k, const void* v,
                              const void* a, const void* b,
                              const float* h0, int n_state,
                              const void* d_o, const float* d_ht,
                              void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                              int B, int T, int H, int head_size, int dtype, int head_first,
                              void* stream) {
  if (B <= 0 || T <= 0 || H <= 0) return RWKVB200_E_SHAPE;
  if (head_size != HS) return RWKVB200_E_UNSUPPORTED;
  if (dtype != RWKVB200_F32 && dtype != RWKVB200_BF16 && dtype != RWKVB200_F16) return RWKVB200_E_DTYPE;
  if (!r || !w || !k || !v || !a || !b || !d_o || !dr || !dw || !dk || !dv || !da || !db) return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != B) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !h0) return RWKVB200_E_NULL;
  const void* ps[] = {r, w, k, v, a, b, h0, d_o, d_ht, dr, dw, dk, dv, da, db, d_h0};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  // same checkpoint volume as rwkvb200_rwkv7_bwd_workspace_bytes(..., RWKVB200_ALGO_RECURRENT)
  const size_t need = (size_t)B * H * ((size_t)(T + R7_CKPT - 1) / R7_CKPT) * HS * HS * sizeof(float);
  if (need > STATIC_SCRATCH_BYTES) return RWKVB200_E_TOO_LARGE;
  float* ckpt = nullptr;
  int e = static_scratch(&ckpt);
  if (e) return e;
  cudaStream_t st = (cudaStream_t)stream;
  e = launch_rwkv7_rec_fwd(r, w, k, v, a, b, n_state ? h0 : nullptr, n_state, nullptr, nullptr, ckpt, R7_CKPT,
                           B, T, H, dtype, head_first, st);
  if (e) return e;
  return launch_rwkv7_rec_bwd(r, w, k, v, a, b, d_o, d_ht, ckpt, dr, dw, dk, dv, da, db, d_h0,
                              B, T, H, dtype, head_first, st);
}

}  // extern "C"
