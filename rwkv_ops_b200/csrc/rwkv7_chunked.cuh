// Chunked RWKV7 delta rule on tcgen05: shared definitions of the forward and backward kernels.
//
// Notation (one (batch, head), one chunk of L = 64 tokens, h = S^T is the [K][V] state):
//   g = -exp(w) per token and channel, gi / ge its inclusive / exclusive prefix sums inside the chunk,
//   gref = gi at token 31 (the reference point that keeps every exponent within +-32 |g|max),
//   glast = gi at token 63.
//   q~ = q e^{gi-gref}   k~ = k e^{gref-gi}   a~ = a e^{ge-gref}   b~ = b e^{gref-gi}
//   A_qk = tril(q~ k~^T)  A_qb = tril(q~ b~^T)  A_ak = stril(a~ k~^T)  A_ab = stril(a~ b~^T)
//   Ainv = (I - A_ab)^-1,  W = Ainv a~,  U = Ainv A_ak v,  O1 = A_qk v
//   with h~0 = diag(e^{gref}) h0:
//     sa  = W h~0 + U                       (rows a_i^T h_{i-1})
//     o   = q~ h~0 + O1 + A_qb sa
//     h_L = diag(e^{glast-gref}) (h~0 + k~^T v + b~^T sa)
// These are the chunk equations of the reference's kernels (rwkv_ops/rwkv7_kernel/triton_kernel/
// chunk_A_fwd.py:111-165, wy_fast_fwd.py:57-62,273-321, chunk_h_fwd.py:140-150, chunk_o_fwd.py:82-136)
// rewritten around one reference point per chunk so that all four A matrices come out of a single
// 128x128x64 tensor-core product of pre-scaled bf16 operands.
//
// Two kernels per direction: an "intra" kernel, parallel over (batch, head, chunk), that produces the
// state-independent tiles, and a "scan" kernel, one CTA per (batch, head), that walks the chunks in
// order with the fp32 state resident in TMEM.  Tiles travel between them through the caller's
// workspace as raw 8 KB images of the swizzled shared-memory layout (tc.cuh), moved by bulk copies.
#pragma once

#include "common.cuh"
#include "tc.cuh"

namespace rwkvb200 {
namespace r7c {

constexpr int L = 64;                 // chunk length
// tiles of one chunk in the workspace, in this order (the first FWD_TILES feed the forward scan)
enum Slot { S_QT = 0, S_KT, S_BT, S_AQB, S_O1, S_W, S_U, FWD_TILES,
            S_AT = FWD_TILES, S_AQK, S_AAK, S_AINV, S_SA, S_H0, ALL_TILES };
constexpr int AUX_FLOATS = 128;       // per chunk: e^{gref}[64], e^{glast-gref}[64]

inline int num_chunks(int T) { return (T + L - 1) / L; }

struct Workspace {
  unsigned char* tiles;   // [n_chunks_total][tiles_per_chunk][8192]
  float* aux;             // [n_chunks_total][128]
  int tiles_per_chunk;
};

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

inline size_t fwd_workspace_bytes(int B, int T, int H, int tiles_per_chunk) {
  const size_t n = (size_t)B * H * num_chunks(T);
  return align256(n * tiles_per_chunk * tc::TILE_BYTES) + align256(n * AUX_FLOATS * sizeof(float)) + 1024;
}

inline Workspace carve(void* ws, int B, int T, int H, int tiles_per_chunk) {
  const size_t n = (size_t)B * H * num_chunks(T);
  Workspace w;
  uintptr_t p = (reinterpret_cast<uintptr_t>(ws) + 1023) & ~uintptr_t(1023);
  w.tiles = reinterpret_cast<unsigned char*>(p);
  w.aux = reinterpret_cast<float*>(p + align256(n * tiles_per_chunk * tc::TILE_BYTES));
  w.tiles_per_chunk = tiles_per_chunk;
  return w;
}

}  // namespace r7c

int launch_rwkv7_chunked_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                             const float* h0, int n_state, void* o, float* ht, void* workspace,
                             int B, int Tn, int H, int head_first, bool keep_for_bwd, cudaStream_t st);

}  // namespace rwkvb200
