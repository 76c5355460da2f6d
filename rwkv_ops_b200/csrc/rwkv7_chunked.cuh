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
// Backward (do = grad of o, dh_L = grad of the state after the chunk, gref held constant: the result
// does not depend on it):
//     dh^  = diag(e^{glast-gref}) dh_L
//     dz   = Ainv^T (A_qb^T do + b~ dh^)  = P2 + B2 dh^          (z = a~ h~0 + A_ak v,  sa = Ainv z)
//     dh~0 = q~^T do + a~^T dz + dh^,   dh0 = diag(e^{gref}) dh~0
//     dv   = A_qk^T do + A_ak^T dz + k~ dh^
//     dA_qk = tril(do v^T)  dA_qb = tril(do sa^T)  dA_ak = stril(dz v^T)  dA_ab = stril(dz sa^T)
//     dq~ = do h~0^T + dA_qk k~ + dA_qb b~        da~ = dz h~0^T + dA_ak k~ + dA_ab b~
//     dk~ = dA_qk^T q~ + dA_ak^T a~ + v dh^^T     db~ = dA_qb^T q~ + dA_ab^T a~ + sa dh^^T
//     dq = dq~ e^{gi-gref} ...;  dgi = dq~ q~ - dk~ k~ - db~ b~;  dge = da~ a~;  dglast = sum_v dh^ X
//     dg_j = sum_{i>=j} (dgi_i + dge_i) - dge_j + dglast;   dw = dg g
// (reference: chunk_o_bwd.py:111-113,246-277,364-381, chunk_h_bwd.py:141-157, wy_fast_bwd.py:99-193,
// chunk_A_bwd.py:146-250,318-320 under rwkv_ops/rwkv7_kernel/triton_kernel/).
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
            // kept for the backward: a~, A_qk, A_ak, Ainv (intra kernel); sa, h~0 and
            // X = h~0 + k~^T v + b~^T sa (forward scan)
            S_AT = FWD_TILES, S_AQK, S_AAK, S_AINV, S_SA, S_H0, S_X,
            // backward intermediates: B2 = Ainv^T b~, P2 = Ainv^T A_qb^T do (adjacent), then
            // dz = Ainv^T dsa and dh^ = e^{glast-gref} dh_L written by the reverse scan
            S_B2, S_P2, S_DZ, S_DHH, ALL_TILES };
constexpr int AUX_FLOATS = 128;       // per chunk: e^{gref}[64], e^{glast-gref}[64]

inline int num_chunks(int T) { return (T + L - 1) / L; }

// Which tokens a sequence occupies.  A dense batch has B sequences of Tn tokens, sequence bi in batch row
// bi of the token tensors.  A packed variable-length batch (start != nullptr) has its sequences laid end
// to end in ONE batch row; sequence bi is tokens start[bi] .. start[bi] + len[bi] - 1 of that row and Tn is
// the longest length: every sequence owns ceil(Tn / 64) chunk slots of the workspace and uses the first
// ceil(len / 64) of them.
// The kernels are compiled for both cases (template parameter PACKED), so that the dense case pays nothing.
struct SeqView {
  const int* start;   // device pointers, one entry per sequence, or nullptr
  const int* len;
  int Tn;
  template <bool PACKED> __device__ __forceinline__ int first(int bi) const {
    if constexpr (PACKED) return __ldg(start + bi); else return 0;
  }
  template <bool PACKED> __device__ __forceinline__ int length(int bi) const {
    if constexpr (PACKED) return __ldg(len + bi); else return Tn;
  }
  template <bool PACKED> __device__ __forceinline__ int row(int bi) const {
    if constexpr (PACKED) return 0; else return bi;
  }
};

// Position of a persistent CTA in the list of chunk slots: slot index, sequence, head, chunk within the
// sequence.  Stepping by the grid size updates it without the divisions of the direct formula.
struct ChunkPos { int ch, bi, hi, c; };
__device__ __forceinline__ ChunkPos chunk_pos(int ch, int NT, int H) {
  ChunkPos p;
  const int unit = ch / NT;
  p.ch = ch; p.c = ch % NT; p.bi = unit / H; p.hi = unit % H;
  return p;
}
__device__ __forceinline__ void chunk_step(ChunkPos& p, int stride, int NT, int H) {
  if (stride >= 4 * NT) {      // short sequences: a step crosses many of them, divide after all
    p = chunk_pos(p.ch + stride, NT, H);
    return;
  }
  p.ch += stride;
  p.c += stride;
  while (p.c >= NT) {
    p.c -= NT;
    if (++p.hi == H) { p.hi = 0; ++p.bi; }
  }
}

// Fused producers (template parameter FUSED of the intra and final kernels).  The three inputs w, a, b of
// the delta rule are then computed on the fly from pre-activations p, u, q of the same shape,
//   w = -e^{-1/2} sigmoid(p),   kk = u / max(|u|_2, 1e-12) over the 64 channels of a head,
//   a = -kk,   b = kk sigmoid(q),
// the elementwise tail of an RWKV7 time-mix block; each is rounded to bfloat16 exactly as if it had been
// materialised as a bfloat16 tensor, so the fused and the unfused operator return the same bits.
constexpr float W_SCALE = -0.60653065971263342f;
__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Rows 0 .. n_rows-1 of a swizzled bf16 tile to token rows `dst`, `dst + st`, ... (st in elements), by all
// NTHREADS threads of the CTA: the store of a chunk whose last rows belong to the next packed sequence,
// which a TMA store of the whole box would overwrite.
// (Kept out of line: it runs for one chunk per sequence and would only lengthen the persistent loops.)
template <int NTHREADS>
__device__ __noinline__ void store_tile_rows(__nv_bfloat16* dst, long long st, const unsigned char* tile,
                                                int n_rows, int tid) {
  for (int e = tid; e < 512; e += NTHREADS) {
    const int row = e >> 3, cc = e & 7;
    if (row < n_rows)
      *reinterpret_cast<uint4*>(dst + row * st + 8 * cc) = *reinterpret_cast<const uint4*>(tile + tc::tile_chunk_off(row, cc));
  }
}

struct Workspace {
  unsigned char* tiles;   // [n_chunks_total][tiles_per_chunk][8192]
  float* aux;             // [n_chunks_total][128]
  int* flags;             // [B*H] nonzero: the unit's decay left the range of the scaled operands (DECAY_LIMIT)
  int tiles_per_chunk;
};

// The scaled operands carry e^{+-(gi - gref)}: with the reference point in the middle of the chunk the
// exponent of a channel reaches the sum of |g| over half a chunk.  Up to DECAY_LIMIT every factor and every
// scaled state entry stays a normal bfloat16 / float32 number and the chunk equations are exact; a
// (batch, head) unit with a larger half-chunk sum in any channel is marked in Workspace::flags by the intra
// kernel and recomputed afterwards by the float32 recurrence (rwkv7_recurrent.cu), so the operator never
// returns values computed from clamped exponents.  |g| <= 1.875 per token never reaches the limit; RWKV7's
// own parametrisation keeps |g| below 0.61.
constexpr float DECAY_LIMIT = 60.f;
// Sequences shorter than this are recomputed by the recurrence as well (marked in the same flags): with one or
// two tokens the decay gradient is what is left of sums over the whole chunk that cancel almost completely
// (exactly zero for one token and no initial state), so the bfloat16 roundings of the chunk products would be all
// there is in dw; the recurrence costs nothing at that length.
constexpr int SHORT_SEQ = 8;

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

inline size_t fwd_workspace_bytes(int B, int T, int H, int tiles_per_chunk) {
  const size_t n = (size_t)B * H * num_chunks(T);
  return align256(n * tiles_per_chunk * tc::TILE_BYTES) + align256(n * AUX_FLOATS * sizeof(float)) +
         align256((size_t)B * H * sizeof(int)) + 1024;
}

inline Workspace carve(void* ws, int B, int T, int H, int tiles_per_chunk) {
  const size_t n = (size_t)B * H * num_chunks(T);
  Workspace w;
  uintptr_t p = (reinterpret_cast<uintptr_t>(ws) + 1023) & ~uintptr_t(1023);
  w.tiles = reinterpret_cast<unsigned char*>(p);
  w.aux = reinterpret_cast<float*>(p + align256(n * tiles_per_chunk * tc::TILE_BYTES));
  w.flags = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(w.aux) + align256(n * AUX_FLOATS * sizeof(float)));
  w.tiles_per_chunk = tiles_per_chunk;
  return w;
}

}  // namespace r7c

// Phases of a forward / backward call (bit mask).  A whole call runs all of them in order; a caller that splits
// a sequence over several GPUs runs the state-independent phase on every GPU at once and only the scans one GPU
// after the other (the workspace carries everything from one phase to the next).
//   forward:  PREPARE = intra-chunk kernel;            SCAN = state scan over the chunks (+ exact fallback)
//   backward: PREPARE = (forward recomputation and) the state-independent products of the reverse scan;
//             SCAN = reverse scan (gradient of the state);   FINISH = token gradients (+ exact fallback)
enum Phase { PHASE_PREPARE = 1, PHASE_SCAN = 2, PHASE_FINISH = 4, PHASE_ALL = 7 };

// Backward of the chunked path; `workspace` must hold fwd_workspace_bytes(B, T, H, ALL_TILES).
// Packed variable-length batches: seq_start / seq_len are device arrays of B entries, Tn the longest length
// and T_total the number of tokens in the one batch row; dense batches pass nullptr, nullptr, 0.
// `fused`: w, a, b are the pre-activations p, u, q (dense batches only).
int launch_rwkv7_chunked_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                             const float* h0, int n_state, const void* d_o, const float* d_ht,
                             void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                             void* workspace, int B, int Tn, int H, int head_first, bool kept, cudaStream_t st,
                             const int* seq_start = nullptr, const int* seq_len = nullptr, int T_total = 0,
                             bool fused = false, int phases = PHASE_ALL);

int launch_rwkv7_chunked_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                             const float* h0, int n_state, void* o, float* ht, void* workspace,
                             int B, int Tn, int H, int head_first, bool keep_for_bwd, cudaStream_t st,
                             const int* seq_start = nullptr, const int* seq_len = nullptr, int T_total = 0,
                             bool fused = false, int phases = PHASE_ALL);

// Fused producers, backward: dw, da, db (in place in the three buffers) -> dp, du, dq.
int launch_rwkv7_producer_bwd(const void* p, const void* u, const void* q, void* dw_dp, void* da_du, void* db_dq,
                              long long n_rows, cudaStream_t st);

}  // namespace rwkvb200
