// extern "C" entry points of librwkv_ops_b200.so: argument checks and dispatch.
// The contract of every function is in include/rwkv_ops_b200.h.
#include "common.cuh"
#include "rwkv7_chunked.cuh"

using namespace rwkvb200;

namespace {

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// head sizes: 64 everywhere; 128 for the RWKV7 operator through the float32 recurrence (big_heads)
inline int check_common(int B, int T, int H, int head_size, int dtype, bool big_heads = false) {
  if (B <= 0 || T <= 0 || H <= 0) return RWKVB200_E_SHAPE;
  if (head_size != HS && !(big_heads && head_size == 128)) return RWKVB200_E_UNSUPPORTED;
  if (dtype != RWKVB200_F32 && dtype != RWKVB200_BF16 && dtype != RWKVB200_F16) return RWKVB200_E_DTYPE;
  return RWKVB200_OK;
}

// AUTO: bf16 token tensors take the chunked tensor-core path; float32 (whose parity bar of 1e-4 a
// bf16-operand path cannot meet) and float16 (whose range the scaled operands exceed) take the
// float32 recurrence.
inline int resolve_r7_algo(int algo, int dtype, int head_size = HS) {
  algo &= 0xff;
  if (algo == RWKVB200_ALGO_AUTO)
    return dtype == RWKVB200_BF16 && head_size == HS ? RWKVB200_ALGO_CHUNKED : RWKVB200_ALGO_RECURRENT;
  return algo;
}

// phase bits of the algo argument (chunked path); none set = the whole call
inline int phases_of(int algo) {
  int p = 0;
  if (algo & RWKVB200_ALGO_PHASE_PREPARE) p |= PHASE_PREPARE;
  if (algo & RWKVB200_ALGO_PHASE_SCAN) p |= PHASE_SCAN;
  if (algo & RWKVB200_ALGO_PHASE_FINISH) p |= PHASE_FINISH;
  return p ? p : (int)PHASE_ALL;
}

// wkv6: AUTO = chunked tensor-core path (its split-precision operands keep float32-grade accuracy).
// head sizes 32 and 128 run the float32 recurrence (the tensor-core path is built for head size 64)
inline int resolve_w6_algo(int algo, int head_size = HS) {
  algo &= 0xff;
  if (head_size != HS) return RWKVB200_ALGO_RECURRENT;
  return algo == RWKVB200_ALGO_RECURRENT ? RWKVB200_ALGO_RECURRENT : RWKVB200_ALGO_CHUNKED;
}
inline int check_w6(int B, int T, int H, int head_size, int dtype, int algo) {
  if (B <= 0 || T <= 0 || H <= 0) return RWKVB200_E_SHAPE;
  if (head_size != 32 && head_size != HS && head_size != 128) return RWKVB200_E_UNSUPPORTED;
  if (head_size != HS && (algo & 0xff) == RWKVB200_ALGO_CHUNKED) return RWKVB200_E_UNSUPPORTED;
  if (dtype != RWKVB200_F32 && dtype != RWKVB200_BF16 && dtype != RWKVB200_F16) return RWKVB200_E_DTYPE;
  return RWKVB200_OK;
}

inline size_t r7_ckpt_bytes(int B, int T, int H, int head_size = HS) {
  const size_t nc = (size_t)(T + R7_CKPT - 1) / R7_CKPT;
  return align256((size_t)B * H * nc * head_size * head_size * sizeof(float));
}

inline size_t w6_ckpt_bytes(int B, int T, int H, int head_size = HS) {
  const size_t nc = (size_t)(T + W6_CKPT - 1) / W6_CKPT;
  return align256((size_t)B * H * nc * head_size * head_size * sizeof(float));
}

}  // namespace

extern "C" {

int rwkvb200_abi_version(void) { return RWKVB200_ABI_VERSION; }

const char* rwkvb200_strerror(int code) {
  switch (code) {
    case RWKVB200_OK: return "ok";
    case RWKVB200_E_SHAPE: return "bad shape: a size is <= 0 or inconsistent";
    case RWKVB200_E_DTYPE: return "bad dtype code";
    case RWKVB200_E_ALIGN: return "pointer not 16-byte aligned";
    case RWKVB200_E_NULL: return "required pointer is NULL";
    case RWKVB200_E_WORKSPACE: return "workspace too small";
    case RWKVB200_E_UNSUPPORTED: return "unsupported head size or mode";
    case RWKVB200_E_CUDA: return "CUDA runtime error at launch";
    case RWKVB200_E_STATE_MAP: return "state_map entry out of range";
    case RWKVB200_E_TOO_LARGE: return "size beyond this entry point's fixed capacity";
    default: return "unknown error code";
  }
}

int rwkvb200_rwkv7_step(const void* r, const void* w, const void* k, const void* v,
                        const void* a, const void* b,
                        const float* state_in, int n_state, float* state_out, void* o,
                        int B, int H, int head_size, int dtype, void* stream) {
  int e = check_common(B, 1, H, head_size, dtype, true);
  if (e) return e;
  if (!r || !w || !k || !v || !a || !b || !state_out || !o) return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != B) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !state_in) return RWKVB200_E_NULL;
  const void* ps[] = {r, w, k, v, a, b, state_in, state_out, o};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  if (head_size != HS)      // one token of the float32 recurrence
    return launch_rwkv7_rec_fwd(r, w, k, v, a, b, n_state ? state_in : nullptr, n_state, o, state_out, nullptr,
                                R7_CKPT, B, 1, H, dtype, 0, (cudaStream_t)stream, nullptr, 0, head_size);
  return launch_rwkv7_step(r, w, k, v, a, b, n_state ? state_in : nullptr, n_state, state_out, o, B, H, dtype,
                           (cudaStream_t)stream);
}

int rwkvb200_rwkv7_decode_step(const void* r, const void* w, const void* k, const void* v,
                               const void* a, const void* b, void* state, int state_dtype, void* o,
                               int B, int H, int head_size, int dtype, void* stream) {
  int e = check_common(B, 1, H, head_size, dtype);
  if (e) return e;
  if (state_dtype != RWKVB200_F32 && state_dtype != RWKVB200_BF16) return RWKVB200_E_DTYPE;
  if (!r || !w || !k || !v || !a || !b || !state || !o) return RWKVB200_E_NULL;
  const void* ps[] = {r, w, k, v, a, b, state, o};
  for (const void* p : ps) if (!aligned16(p)) return RWKVB200_E_ALIGN;
  return launch_rwkv7_decode_step(r, w, k, v, a, b, state, state_dtype, o, B, H, dtype, (cudaStream_t)stream);
}

size_t rwkvb200_rwkv7_fwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo) {
  if (check_common(B, T, H, head_size, dtype, true)) return 0;
  if (head_size == HS && resolve_r7_algo(algo, dtype, head_size) == RWKVB200_ALGO_CHUNKED)
    return r7c::fwd_workspace_bytes(B, T, H, (algo & RWKVB200_ALGO_KEEP) ? r7c::ALL_TILES : r7c::FWD_TILES);
  return 0;
}

int rwkvb200_rwkv7_fwd(const void* r, const void* w, const void* k, const void* v,
                       const void* a, const void* b,
                       const float* h0, int n_state, void* o, float* ht,
                       void* workspace, size_t workspace_bytes,
                       int B, int T, int H, int head_size, int dtype, int head_first, int algo,
                       void* stream) {
  int e = check_common(B, T, H, head_size, dtype, true);
  if (e) return e;
  if (head_size != HS && resolve_r7_algo(algo, dtype, head_size) != RWKVB200_ALGO_RECURRENT)
    return RWKVB200_E_UNSUPPORTED;      // the tensor-core path is built for head size 64
  const int phases = phases_of(algo);
  if (!r || !w || !k || !v || !a || !b || (!o && (phases & PHASE_SCAN))) return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != B) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !h0) return RWKVB200_E_NULL;
  const void* ps[] = {r, w, k, v, a, b, h0, o, ht, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  const size_t need = rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, head_size, dtype, algo);
  if (workspace_bytes < need || (need && !workspace)) return RWKVB200_E_WORKSPACE;
  if (phases != PHASE_ALL && resolve_r7_algo(algo, dtype, head_size) != RWKVB200_ALGO_CHUNKED)
    return RWKVB200_E_UNSUPPORTED;
  switch (resolve_r7_algo(algo, dtype, head_size)) {
    case RWKVB200_ALGO_RECURRENT:
      return launch_rwkv7_rec_fwd(r, w, k, v, a, b, n_state ? h0 : nullptr, n_state, o, ht, nullptr, R7_CKPT,
                                  B, T, H, dtype, head_first, (cudaStream_t)stream, nullptr, 0, head_size);
    case RWKVB200_ALGO_CHUNKED:
      if (dtype != RWKVB200_BF16) return RWKVB200_E_UNSUPPORTED;
      return launch_rwkv7_chunked_fwd(r, w, k, v, a, b, n_state ? h0 : nullptr, n_state, o, ht, workspace,
                                      B, T, H, head_first, (algo & RWKVB200_ALGO_KEEP) != 0, (cudaStream_t)stream,
                                      nullptr, nullptr, 0, false, phases);
    default:
      return RWKVB200_E_UNSUPPORTED;
  }
}

size_t rwkvb200_rwkv7_bwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo) {
  if (check_common(B, T, H, head_size, dtype, true)) return 0;
  switch (resolve_r7_algo(algo, dtype, head_size)) {
    case RWKVB200_ALGO_RECURRENT: return r7_ckpt_bytes(B, T, H, head_size);
    case RWKVB200_ALGO_CHUNKED: return head_size == HS ? r7c::fwd_workspace_bytes(B, T, H, r7c::ALL_TILES) : 0;
    default: return 0;
  }
}

int rwkvb200_rwkv7_bwd(const void* r, const void* w, const void* k, const void* v,
                       const void* a, const void* b,
                       const float* h0, int n_state,
                       const void* d_o, const float* d_ht,
                       void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                       void* workspace, size_t workspace_bytes,
                       int B, int T, int H, int head_size, int dtype, int head_first, int algo,
                       void* stream) {
  int e = check_common(B, T, H, head_size, dtype, true);
  if (e) return e;
  if (head_size != HS && resolve_r7_algo(algo, dtype, head_size) != RWKVB200_ALGO_RECURRENT)
    return RWKVB200_E_UNSUPPORTED;
  if (!r || !w || !k || !v || !a || !b || !d_o || !dr || !dw || !dk || !dv || !da || !db) return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != B) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !h0) return RWKVB200_E_NULL;
  const void* ps[] = {r, w, k, v, a, b, h0, d_o, d_ht, dr, dw, dk, dv, da, db, d_h0, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  const size_t need = rwkvb200_rwkv7_bwd_workspace_bytes(B, T, H, head_size, dtype, algo);
  if (workspace_bytes < need || (need && !workspace)) return RWKVB200_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (phases_of(algo) != PHASE_ALL && resolve_r7_algo(algo, dtype, head_size) != RWKVB200_ALGO_CHUNKED)
    return RWKVB200_E_UNSUPPORTED;
  switch (resolve_r7_algo(algo, dtype, head_size)) {
    case RWKVB200_ALGO_RECURRENT: {
      float* ckpt = reinterpret_cast<float*>(workspace);
      e = launch_rwkv7_rec_fwd(r, w, k, v, a, b, n_state ? h0 : nullptr, n_state, nullptr, nullptr, ckpt, R7_CKPT,
                               B, T, H, dtype, head_first, st, nullptr, 0, head_size);
      if (e) return e;
      return launch_rwkv7_rec_bwd(r, w, k, v, a, b, d_o, d_ht, ckpt, dr, dw, dk, dv, da, db, d_h0,
                                  B, T, H, dtype, head_first, st, nullptr, 0, head_size);
    }
    case RWKVB200_ALGO_CHUNKED:
      if (dtype != RWKVB200_BF16) return RWKVB200_E_UNSUPPORTED;
      return launch_rwkv7_chunked_bwd(r, w, k, v, a, b, n_state ? h0 : nullptr, n_state, d_o, d_ht,
                                      dr, dw, dk, dv, da, db, d_h0, workspace, B, T, H, head_first,
                                      (algo & RWKVB200_ALGO_KEEP) != 0, st, nullptr, nullptr, 0, false,
                                      phases_of(algo));
    default:
      return RWKVB200_E_UNSUPPORTED;
  }
}

// ---- packed variable-length batches (chunked bf16 path only)
size_t rwkvb200_rwkv7_varlen_workspace_bytes(int n_seq, int max_len, int H, int head_size, int keep) {
  if (check_common(n_seq, max_len, H, head_size, RWKVB200_BF16)) return 0;
  return r7c::fwd_workspace_bytes(n_seq, max_len, H, keep ? r7c::ALL_TILES : r7c::FWD_TILES);
}

int rwkvb200_rwkv7_fwd_varlen(const void* r, const void* w, const void* k, const void* v,
                              const void* a, const void* b,
                              const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                              const float* h0, int n_state, void* o, float* ht,
                              void* workspace, size_t workspace_bytes,
                              int H, int head_size, int dtype, int keep, void* stream) {
  int e = check_common(n_seq, max_len, H, head_size, dtype);
  if (e) return e;
  if (dtype != RWKVB200_BF16) return RWKVB200_E_UNSUPPORTED;
  if (total_len < max_len) return RWKVB200_E_SHAPE;
  if (!r || !w || !k || !v || !a || !b || !o || !seq_start || !seq_len) return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != n_seq) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !h0) return RWKVB200_E_NULL;
  const void* ps[] = {r, w, k, v, a, b, h0, o, ht, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  const size_t need = rwkvb200_rwkv7_varlen_workspace_bytes(n_seq, max_len, H, head_size, keep);
  if (workspace_bytes < need || !workspace) return RWKVB200_E_WORKSPACE;
  return launch_rwkv7_chunked_fwd(r, w, k, v, a, b, n_state ? h0 : nullptr, n_state, o, ht, workspace,
                                  n_seq, max_len, H, 0, keep != 0, (cudaStream_t)stream, seq_start, seq_len, total_len);
}

int rwkvb200_rwkv7_bwd_varlen(const void* r, const void* w, const void* k, const void* v,
                              const void* a, const void* b,
                              const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                              const float* h0, int n_state, const void* d_o, const float* d_ht,
                              void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                              void* workspace, size_t workspace_bytes,
                              int H, int head_size, int dtype, int kept, void* stream) {
  int e = check_common(n_seq, max_len, H, head_size, dtype);
  if (e) return e;
  if (dtype != RWKVB200_BF16) return RWKVB200_E_UNSUPPORTED;
  if (total_len < max_len) return RWKVB200_E_SHAPE;
  if (!r || !w || !k || !v || !a || !b || !d_o || !dr || !dw || !dk || !dv || !da || !db || !seq_start || !seq_len)
    return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != n_seq) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !h0) return RWKVB200_E_NULL;
  const void* ps[] = {r, w, k, v, a, b, h0, d_o, d_ht, dr, dw, dk, dv, da, db, d_h0, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  const size_t need = rwkvb200_rwkv7_varlen_workspace_bytes(n_seq, max_len, H, head_size, 1);
  if (workspace_bytes < need || !workspace) return RWKVB200_E_WORKSPACE;
  return launch_rwkv7_chunked_bwd(r, w, k, v, a, b, n_state ? h0 : nullptr, n_state, d_o, d_ht,
                                  dr, dw, dk, dv, da, db, d_h0, workspace, n_seq, max_len, H, 0, kept != 0,
                                  (cudaStream_t)stream, seq_start, seq_len, total_len);
}

// ---- fused producers (chunked bf16 path, dense [B,T,H,64] batches)
int rwkvb200_rwkv7_fused_fwd(const void* r, const void* w_pre, const void* k, const void* v,
                             const void* kk_pre, const void* a_pre,
                             const float* h0, int n_state, void* o, float* ht,
                             void* workspace, size_t workspace_bytes,
                             int B, int T, int H, int head_size, int dtype, int keep, void* stream) {
  int e = check_common(B, T, H, head_size, dtype);
  if (e) return e;
  if (dtype != RWKVB200_BF16) return RWKVB200_E_UNSUPPORTED;
  if (!r || !w_pre || !k || !v || !kk_pre || !a_pre || !o) return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != B) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !h0) return RWKVB200_E_NULL;
  const void* ps[] = {r, w_pre, k, v, kk_pre, a_pre, h0, o, ht, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  const size_t need = r7c::fwd_workspace_bytes(B, T, H, keep ? r7c::ALL_TILES : r7c::FWD_TILES);
  if (workspace_bytes < need || !workspace) return RWKVB200_E_WORKSPACE;
  return launch_rwkv7_chunked_fwd(r, w_pre, k, v, kk_pre, a_pre, n_state ? h0 : nullptr, n_state, o, ht, workspace,
                                  B, T, H, 0, keep != 0, (cudaStream_t)stream, nullptr, nullptr, 0, true);
}

int rwkvb200_rwkv7_fused_bwd(const void* r, const void* w_pre, const void* k, const void* v,
                             const void* kk_pre, const void* a_pre,
                             const float* h0, int n_state, const void* d_o, const float* d_ht,
                             void* dr, void* dw_pre, void* dk, void* dv, void* dkk_pre, void* da_pre, float* d_h0,
                             void* workspace, size_t workspace_bytes,
                             int B, int T, int H, int head_size, int dtype, int kept, void* stream) {
  int e = check_common(B, T, H, head_size, dtype);
  if (e) return e;
  if (dtype != RWKVB200_BF16) return RWKVB200_E_UNSUPPORTED;
  if (!r || !w_pre || !k || !v || !kk_pre || !a_pre || !d_o || !dr || !dw_pre || !dk || !dv || !dkk_pre || !da_pre)
    return RWKVB200_E_NULL;
  if (n_state != 0 && n_state != 1 && n_state != B) return RWKVB200_E_SHAPE;
  if (n_state != 0 && !h0) return RWKVB200_E_NULL;
  const void* ps[] = {r, w_pre, k, v, kk_pre, a_pre, h0, d_o, d_ht, dr, dw_pre, dk, dv, dkk_pre, da_pre, d_h0, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  const size_t need = r7c::fwd_workspace_bytes(B, T, H, r7c::ALL_TILES);
  if (workspace_bytes < need || !workspace) return RWKVB200_E_WORKSPACE;
  return launch_rwkv7_chunked_bwd(r, w_pre, k, v, kk_pre, a_pre, n_state ? h0 : nullptr, n_state, d_o, d_ht,
                                  dr, dw_pre, dk, dv, dkk_pre, da_pre, d_h0, workspace, B, T, H, 0, kept != 0,
                                  (cudaStream_t)stream, nullptr, nullptr, 0, true);
}

size_t rwkvb200_wkv6_fwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo) {
  if (check_w6(B, T, H, head_size, dtype, algo)) return 0;
  if (resolve_w6_algo(algo, head_size) != RWKVB200_ALGO_CHUNKED) return 0;
  return (algo & RWKVB200_ALGO_KEEP) ? wkv6_chunked_bwd_workspace_bytes(B, T, H) : wkv6_chunked_fwd_scratch_bytes(B, H);
}

int rwkvb200_wkv6_fwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                      const float* s0, int n_state, const int32_t* state_map,
                      void* y, float* sT, void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int head_size, int dtype, int algo, void* stream) {
  int e = check_w6(B, T, H, head_size, dtype, algo);
  if (e) return e;
  if (!r || !k || !v || !w || !u || !y) return RWKVB200_E_NULL;
  if (n_state < 0) return RWKVB200_E_SHAPE;
  if (n_state > 0 && !s0) return RWKVB200_E_NULL;
  if (n_state > 1 && !state_map && n_state != B) return RWKVB200_E_STATE_MAP;
  const void* ps[] = {r, k, v, w, u, s0, y, sT};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  if (resolve_w6_algo(algo, head_size) == RWKVB200_ALGO_CHUNKED) {
    if (!workspace || !aligned16(workspace) ||
        workspace_bytes < rwkvb200_wkv6_fwd_workspace_bytes(B, T, H, head_size, dtype, algo))
      return RWKVB200_E_WORKSPACE;
    float* states = nullptr;
    float* handoff = nullptr;
    int* flags = nullptr;
    int* hflags = nullptr;
    if (algo & RWKVB200_ALGO_KEEP) {
      states = reinterpret_cast<float*>(workspace);
      wkv6_chunked_workspace_parts(workspace, B, T, H, &flags, &handoff, &hflags);
    } else {
      wkv6_chunked_fwd_scratch(workspace, B, H, &flags, &handoff, &hflags);
    }
    return launch_wkv6_chunked_fwd(r, k, v, w, u, n_state ? s0 : nullptr, n_state, state_map, y, sT, states, flags,
                                   handoff, hflags, B, T, H, dtype, (cudaStream_t)stream);
  }
  return launch_wkv6_fwd(r, k, v, w, u, n_state ? s0 : nullptr, n_state, state_map, y, sT, nullptr,
                         B, T, H, dtype, (cudaStream_t)stream, nullptr, 0, head_size);
}

size_t rwkvb200_wkv6_bwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo) {
  if (check_w6(B, T, H, head_size, dtype, algo)) return 0;
  if (resolve_w6_algo(algo, head_size) == RWKVB200_ALGO_CHUNKED) return wkv6_chunked_bwd_workspace_bytes(B, T, H);
  // checkpoints, and one row of du per CTA (head_size / 16 of them per unit)
  return w6_ckpt_bytes(B, T, H, head_size) + align256((size_t)B * H * (head_size / 16) * head_size * sizeof(float));
}

int rwkvb200_wkv6_bwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                      const float* s0, int n_state, const int32_t* state_map,
                      const void* d_y, const float* d_sT,
                      void* dr, void* dk, void* dv, void* dw, float* du, float* d_s0,
                      void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int head_size, int dtype, int algo, void* stream) {
  int e = check_w6(B, T, H, head_size, dtype, algo);
  if (e) return e;
  if (!r || !k || !v || !w || !u || !d_y || !dr || !dk || !dv || !dw || !du) return RWKVB200_E_NULL;
  if (n_state < 0) return RWKVB200_E_SHAPE;
  if (n_state > 0 && !s0) return RWKVB200_E_NULL;
  if (n_state > 1 && !state_map && n_state != B) return RWKVB200_E_STATE_MAP;
  const void* ps[] = {r, k, v, w, u, s0, d_y, d_sT, dr, dk, dv, dw, du, d_s0, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  if (!workspace || workspace_bytes < rwkvb200_wkv6_bwd_workspace_bytes(B, T, H, head_size, dtype, algo))
    return RWKVB200_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (resolve_w6_algo(algo, head_size) == RWKVB200_ALGO_CHUNKED)
    return launch_wkv6_chunked_bwd(r, k, v, w, u, n_state ? s0 : nullptr, n_state, state_map, d_y, d_sT,
                                   dr, dk, dv, dw, du, d_s0, workspace, B, T, H, dtype,
                                   (algo & RWKVB200_ALGO_KEEP) != 0, st);
  float* ckpt = reinterpret_cast<float*>(workspace);
  float* du_partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + w6_ckpt_bytes(B, T, H, head_size));
  e = launch_wkv6_fwd(r, k, v, w, u, n_state ? s0 : nullptr, n_state, state_map, nullptr, nullptr, ckpt,
                      B, T, H, dtype, st, nullptr, 0, head_size);
  if (e) return e;
  return launch_wkv6_bwd(r, k, v, w, u, d_y, d_sT, ckpt, dr, dk, dv, dw, du_partial, du, d_s0, B, T, H, dtype, st,
                         head_size);
}

size_t rwkvb200_wkv6_varlen_workspace_bytes(int n_seq, int max_len, int H, int head_size, int dtype, int keep) {
  if (check_common(n_seq, max_len, H, head_size, dtype)) return 0;
  return keep ? wkv6_chunked_bwd_workspace_bytes(n_seq, max_len, H) : wkv6_chunked_fwd_scratch_bytes(n_seq, H);
}

int rwkvb200_wkv6_fwd_varlen(const void* r, const void* k, const void* v, const void* w, const float* u,
                             const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                             const float* s0, int n_state, const int32_t* state_map,
                             void* y, float* sT, void* workspace, size_t workspace_bytes,
                             int H, int head_size, int dtype, int keep, void* stream) {
  int e = check_common(n_seq, max_len, H, head_size, dtype);
  if (e) return e;
  if (total_len < max_len) return RWKVB200_E_SHAPE;
  if (!r || !k || !v || !w || !u || !y || !seq_start || !seq_len) return RWKVB200_E_NULL;
  if (n_state < 0) return RWKVB200_E_SHAPE;
  if (n_state > 0 && !s0) return RWKVB200_E_NULL;
  if (n_state > 1 && !state_map && n_state != n_seq) return RWKVB200_E_STATE_MAP;
  const void* ps[] = {r, k, v, w, u, s0, y, sT, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  if (!workspace || workspace_bytes < rwkvb200_wkv6_varlen_workspace_bytes(n_seq, max_len, H, head_size, dtype, keep))
    return RWKVB200_E_WORKSPACE;
  float* states = nullptr;
  float* handoff = nullptr;
  int* flags = nullptr;
  int* hflags = nullptr;
  if (keep) {
    states = reinterpret_cast<float*>(workspace);
    wkv6_chunked_workspace_parts(workspace, n_seq, max_len, H, &flags, &handoff, &hflags);
  } else {
    wkv6_chunked_fwd_scratch(workspace, n_seq, H, &flags, &handoff, &hflags);
  }
  return launch_wkv6_chunked_fwd(r, k, v, w, u, n_state ? s0 : nullptr, n_state, state_map, y, sT, states, flags,
                                 handoff, hflags, n_seq, max_len, H, dtype, (cudaStream_t)stream, seq_start, seq_len,
                                 total_len);
}

int rwkvb200_wkv6_bwd_varlen(const void* r, const void* k, const void* v, const void* w, const float* u,
                             const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                             const float* s0, int n_state, const int32_t* state_map,
                             const void* d_y, const float* d_sT,
                             void* dr, void* dk, void* dv, void* dw, float* du, float* d_s0,
                             void* workspace, size_t workspace_bytes,
                             int H, int head_size, int dtype, int kept, void* stream) {
  int e = check_common(n_seq, max_len, H, head_size, dtype);
  if (e) return e;
  if (total_len < max_len) return RWKVB200_E_SHAPE;
  if (!r || !k || !v || !w || !u || !d_y || !dr || !dk || !dv || !dw || !du || !seq_start || !seq_len)
    return RWKVB200_E_NULL;
  if (n_state < 0) return RWKVB200_E_SHAPE;
  if (n_state > 0 && !s0) return RWKVB200_E_NULL;
  if (n_state > 1 && !state_map && n_state != n_seq) return RWKVB200_E_STATE_MAP;
  const void* ps[] = {r, k, v, w, u, s0, d_y, d_sT, dr, dk, dv, dw, du, d_s0, workspace};
  for (const void* p : ps) if (p && !aligned16(p)) return RWKVB200_E_ALIGN;
  if (!workspace || workspace_bytes < rwkvb200_wkv6_varlen_workspace_bytes(n_seq, max_len, H, head_size, dtype, 1))
    return RWKVB200_E_WORKSPACE;
  return launch_wkv6_chunked_bwd(r, k, v, w, u, n_state ? s0 : nullptr, n_state, state_map, d_y, d_sT,
                                 dr, dk, dv, dw, du, d_s0, workspace, n_seq, max_len, H, dtype, kept != 0,
                                 (cudaStream_t)stream, seq_start, seq_len, total_len);
}

}  // extern "C"
