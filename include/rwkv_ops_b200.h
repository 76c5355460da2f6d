/*
 * rwkv_ops_b200 -- C ABI of the sm_100a CUDA library behind the RWKV7
 * generalized delta rule and the RWKV6 wkv operator.
 *
 * Every entry point takes plain device pointers and sizes; the caller owns all
 * memory (inputs, outputs, workspace) and the stream.  Nothing here allocates,
 * frees or keeps a pointer after it returns, and all work is enqueued on the
 * given stream without synchronising it.  Return value: 0 on success, a negative
 * RWKVB200_E_* code otherwise (rwkvb200_strerror names it).  Nothing traps or
 * asserts on the device.
 *
 * Conventions shared by all entry points
 *   dtype        RWKVB200_F32 / RWKVB200_BF16 / RWKVB200_F16: element type of the
 *                token tensors (inputs, outputs and their gradients).  Arithmetic
 *                and all states are float32.
 *   head size    64 (key and value) on every entry point; the dense RWKV7 forward / backward / step also
 *                take 128 and the wkv6 forward / backward 32 and 128, through the float32 recurrence
 *                (RWKVB200_ALGO_AUTO or _RECURRENT).  Other sizes return RWKVB200_E_UNSUPPORTED.
 *   decay        every operator applies exp(-exp(w)) to its w input, as the
 *                reference does (rwkv_ops/rwkv7_kernel/native_keras_op.py:58,
 *                rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:63).
 *   alignment    token tensors 16-byte aligned, states 16-byte aligned.
 */
#ifndef RWKV_OPS_B200_H
#define RWKV_OPS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RWKVB200_ABI_VERSION 1

enum {
  RWKVB200_F32 = 0,
  RWKVB200_BF16 = 1,
  RWKVB200_F16 = 2
};

enum {
  RWKVB200_OK = 0,
  RWKVB200_E_SHAPE = -1,        /* a size is <= 0 or inconsistent */
  RWKVB200_E_DTYPE = -2,        /* unknown dtype code */
  RWKVB200_E_ALIGN = -3,        /* a pointer is not 16-byte aligned */
  RWKVB200_E_NULL = -4,         /* a required pointer is NULL */
  RWKVB200_E_WORKSPACE = -5,    /* workspace smaller than *_workspace_bytes() */
  RWKVB200_E_UNSUPPORTED = -6,  /* head size / mode not built */
  RWKVB200_E_CUDA = -7,         /* the CUDA runtime reported an error at launch */
  RWKVB200_E_STATE_MAP = -8,    /* a state_map entry is outside [0, n_state) */
  RWKVB200_E_TOO_LARGE = -9     /* size beyond a fixed-capacity entry point's limit */
};

/* algo argument of the RWKV7 entry points */
enum {
  RWKVB200_ALGO_AUTO = 0,       /* chunked tensor-core path for bf16 tokens, recurrent for f32 and f16 */
  RWKVB200_ALGO_RECURRENT = 1,  /* token-by-token float32 recurrence (float32-exact) */
  /* Chunked tcgen05 path (bf16 tokens).  Its scaled operands are exact while the sum of exp(w) over any 32
   * consecutive tokens of a channel stays below 60 (always true for w <= 0.62; RWKV7's own
   * parametrisation keeps exp(w) below 0.61).  A (batch, head) unit beyond that is detected on the device
   * and recomputed, forward and backward, by the float32 recurrence inside the same call: results hold
   * for any w, such units just run at the recurrent path's speed. */
  RWKVB200_ALGO_CHUNKED = 2,
  /* Flag, OR-ed into algo (chunked path only).  Forward: also leave the per-chunk tiles the backward
   * needs in the workspace (size it with the flag set).  Backward: the workspace still holds what that
   * forward call left there, so skip the recomputation.  Without the flag the backward recomputes the
   * forward from the inputs, as the reference does (rwkv_ops/rwkv7_kernel/torch_op.py:163-183). */
  RWKVB200_ALGO_KEEP = 0x100,
  /* Flags, OR-ed into algo (chunked path of rwkvb200_rwkv7_fwd / _bwd only): run part of the call.  None set
   * = the whole call.  The parts of one call must run in order on the same workspace with the same
   * arguments.  Forward: PREPARE does everything that does not depend on the initial state (h0, o and ht
   * are not touched and o may be NULL), SCAN walks the state through the chunks and writes o and ht.
   * Backward: PREPARE does what does not depend on d_ht, SCAN carries the state gradient back through the
   * chunks and writes d_h0, FINISH writes the six token gradients (pass the same gradient buffers to every
   * part: for units beyond the decay range SCAN already runs the recurrence, which writes into them, so that
   * their share of d_h0 is exact when SCAN returns).  A caller that splits one sequence over
   * several GPUs runs PREPARE / FINISH on all of them at once and only the SCAN parts one GPU after the
   * other, passing ht (forward) and d_h0 (backward) to the neighbour.  No counterpart in the reference,
   * which has no multi-device mode (README.md:179). */
  RWKVB200_ALGO_PHASE_PREPARE = 0x1000,
  RWKVB200_ALGO_PHASE_SCAN = 0x2000,
  RWKVB200_ALGO_PHASE_FINISH = 0x4000
};

int rwkvb200_abi_version(void);
const char* rwkvb200_strerror(int code);
/* Text of the last CUDA runtime error behind a RWKVB200_E_CUDA return ("no error" if none). */
const char* rwkvb200_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * RWKV7 generalized delta rule.
 * Replaces generalized_delta_rule of the reference
 * (native: rwkv_ops/rwkv7_kernel/native_keras_op.py:23-95; GPU: rwkv_ops/rwkv7_kernel/torch_op.py:458-490)
 * and the kernel sequence it launches (chunk_dplr_fwd, torch_op.py:46-120; chunk_dplr_bwd, :123-265).
 *
 * Token tensors r,w,k,v,a,b,o (and gradients) hold B*T*H*64 elements, laid out [B,T,H,64] when
 * head_first == 0 and [B,H,T,64] when head_first != 0.  States are float32 [n,H,64,64] with the
 * VALUE index before the KEY index (the native operator's layout, native_keras_op.py:85-88).
 *   h0 / n_state   initial state: n_state = 0 (h0 ignored, zero state), 1 (one state broadcast over
 *                  the batch, native_keras_op.py:62-63) or B.
 *   ht             final state [B,H,64,64], may be NULL.
 * ---------------------------------------------------------------------------------------- */

/* One decode step (T == 1): token tensors are [B,H,64]; state_out may alias state_in when
 * n_state == B.  Maths of native_keras_op.py:80-91 for a single t. */
int rwkvb200_rwkv7_step(const void* r, const void* w, const void* k, const void* v,
                        const void* a, const void* b,
                        const float* state_in, int n_state, float* state_out, void* o,
                        int B, int H, int head_size, int dtype, void* stream);

/* Packed variable-length batches (bfloat16 token tensors only).  The n_seq sequences lie end to end in
 * token tensors of shape [1, total_len, H, 64]; sequence i is tokens seq_start[i] .. seq_start[i] +
 * seq_len[i] - 1 (device arrays of n_seq int32, every length >= 1, no overlap) and max_len is the longest
 * length.  States are per sequence: h0 [n_state, H, 64, 64] with n_state 0, 1 or n_seq, ht and d_h0
 * [n_seq, H, 64, 64].  keep / kept as RWKVB200_ALGO_KEEP in the dense entry points; the workspace is
 * sized by rwkvb200_rwkv7_varlen_workspace_bytes (every sequence owns ceil(max_len / 64) chunk slots).
 * The reference carries cu_seqlens plumbing for this but has it disabled (torch_op.py:283,299;
 * triton_kernel/chunk_A_fwd.py:47-56); the result equals running each sequence on its own. */
size_t rwkvb200_rwkv7_varlen_workspace_bytes(int n_seq, int max_len, int H, int head_size, int keep);

int rwkvb200_rwkv7_fwd_varlen(const void* r, const void* w, const void* k, const void* v,
                              const void* a, const void* b,
                              const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                              const float* h0, int n_state, void* o, float* ht,
                              void* workspace, size_t workspace_bytes,
                              int H, int head_size, int dtype, int keep, void* stream);

int rwkvb200_rwkv7_bwd_varlen(const void* r, const void* w, const void* k, const void* v,
                              const void* a, const void* b,
                              const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                              const float* h0, int n_state, const void* d_o, const float* d_ht,
                              void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                              void* workspace, size_t workspace_bytes,
                              int H, int head_size, int dtype, int kept, void* stream);

/* The delta rule with its three elementwise producers fused in (bfloat16, dense [B,T,H,64] batches):
 *   w = -exp(-1/2) * sigmoid(w_pre),  kk = kk_pre / max(|kk_pre|_2, 1e-12) over the 64 channels of a head,
 *   a = -kk,  b = kk * sigmoid(a_pre),
 * each rounded to bfloat16 as a materialised tensor would be, then rwkvb200_rwkv7_fwd / _bwd on
 * (r, w, k, v, a, b): same results, without w, a, b (forward) or their gradients (backward) ever being
 * written to or read from memory.  The backward returns the gradients of the pre-activations.  Workspace
 * as rwkvb200_rwkv7_fwd_workspace_bytes / _bwd_workspace_bytes with the chunked algorithm (keep / kept as
 * RWKVB200_ALGO_KEEP).  These producers are not part of the reference; they are what its callers compute
 * right before the operator (the input distributions of its value test, test_script/test_rwkv7_value.py). */
int rwkvb200_rwkv7_fused_fwd(const void* r, const void* w_pre, const void* k, const void* v,
                             const void* kk_pre, const void* a_pre,
                             const float* h0, int n_state, void* o, float* ht,
                             void* workspace, size_t workspace_bytes,
                             int B, int T, int H, int head_size, int dtype, int keep, void* stream);

int rwkvb200_rwkv7_fused_bwd(const void* r, const void* w_pre, const void* k, const void* v,
                             const void* kk_pre, const void* a_pre,
                             const float* h0, int n_state, const void* d_o, const float* d_ht,
                             void* dr, void* dw_pre, void* dk, void* dv, void* dkk_pre, void* da_pre, float* d_h0,
                             void* workspace, size_t workspace_bytes,
                             int B, int T, int H, int head_size, int dtype, int kept, void* stream);

/* One decode step in place on a state the caller keeps on the device across steps:
 * state [B,H,64,64] (value index before key index, like the reference's final_state), element type
 * state_dtype = RWKVB200_F32 (the reference's state type; same arithmetic as rwkvb200_rwkv7_step) or
 * RWKVB200_BF16 (half the state traffic; the state is rounded to bfloat16 after every token, which the
 * reference does not do).  Token tensors [B,H,64] of `dtype`.  No counterpart in the reference, whose
 * T == 1 call allocates a new state every step (native_keras_op.py:60-95). */
int rwkvb200_rwkv7_decode_step(const void* r, const void* w, const void* k, const void* v,
                               const void* a, const void* b, void* state, int state_dtype, void* o,
                               int B, int H, int head_size, int dtype, void* stream);

size_t rwkvb200_rwkv7_fwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo);

int rwkvb200_rwkv7_fwd(const void* r, const void* w, const void* k, const void* v,
                       const void* a, const void* b,
                       const float* h0, int n_state, void* o, float* ht,
                       void* workspace, size_t workspace_bytes,
                       int B, int T, int H, int head_size, int dtype, int head_first, int algo,
                       void* stream);

size_t rwkvb200_rwkv7_bwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo);

/* Backward.  Recomputes the forward from the inputs (the reference's autograd node also saves
 * only the inputs, torch_op.py:298).  d_o is the gradient of o; d_ht (may be NULL) the gradient of
 * the final state.  Writes dr,dw,dk,dv,da,db (token layout, dtype) and, when d_h0 is not NULL,
 * the float32 gradient of the per-batch-row initial state [B,H,64,64] (a caller that broadcast one
 * state sums it over the batch).  dw is the gradient of the w INPUT (chain rule through
 * exp(-exp(w)) included; the reference leaves that step to autograd, torch_op.py:434). */
int rwkvb200_rwkv7_bwd(const void* r, const void* w, const void* k, const void* v,
                       const void* a, const void* b,
                       const float* h0, int n_state,
                       const void* d_o, const float* d_ht,
                       void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                       void* workspace, size_t workspace_bytes,
                       int B, int T, int H, int head_size, int dtype, int head_first, int algo,
                       void* stream);

/* Backward without a workspace argument, for callers that cannot allocate device memory.
 * No counterpart in the reference.  It is the float32 recurrent backward (RWKVB200_ALGO_RECURRENT)
 * with the same inputs, outputs and results as rwkvb200_rwkv7_bwd, but its state checkpoints live in
 * a fixed array inside the library's device image instead of a caller workspace.  Meant for hosts
 * that hand an operator only its input and output buffers and forbid cudaMalloc in the call
 * (operator plugins of inference runtimes, servers that reserved all device memory at start-up).
 *   - Every GPU that loads the library holds RWKVB200_STATIC_SCRATCH_BYTES for the life of the process.
 *   - B*H*ceil(T/8)*16 KiB must fit in that array, else RWKVB200_E_TOO_LARGE.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call before any stream capture begins.
 *   - The array is shared by all calls and keeps the previous call's contents (nothing in it needs
 *     to start at zero).  Calls that overlap on the GPU race on it: issue them on one stream.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine. */
#define RWKVB200_STATIC_SCRATCH_BYTES (32u << 20)
size_t rwkvb200_rwkv7_bwd_static_capacity_bytes(void);
int rwkvb200_rwkv7_bwd_static(const void* r, const void* w, const void* k, const void* v,
                              const void* a, const void* b,
                              const float* h0, int n_state,
                              const void* d_o, const float* d_ht,
                              void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* d_h0,
                              int B, int T, int H, int head_size, int dtype, int head_first,
                              void* stream);

/* ------------------------------------------------------------------------------------------
 * RWKV6 wkv.
 * Replaces RWKVKernelOperator.__call__ of the reference
 * (native: rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:10-86; GPU: rwkv_ops/rwkv6_kernel/torch_rwkv_kernel.py:214-304
 * with kernels rwkv_ops/rwkv6_kernel/torch_kernel/wkv6_cuda.cu:13-357).
 *
 * r,k,v,w,y are [B,T,C], C = H*64; u is float32 [H,64].  States are float32 [n,H,64,64] with the KEY
 * index before the VALUE index (ops_rwkv_kernel.py:71-77).
 *   s0 / n_state / state_map   initial-state table [n_state,H,64,64] (n_state = 0: zero state) and a
 *                  DEVICE int32 array [B] choosing one table row per batch row; NULL means row b for
 *                  batch row b (then n_state must be B) or row 0 when n_state == 1.  The range of
 *                  state_map is the caller's to check on the host (the Python layer does, before the
 *                  launch); out-of-range entries are clamped on the device instead of trapping.
 *   sT             final state [B,H,64,64], may be NULL.
 *   algo           RWKVB200_ALGO_AUTO / _RECURRENT (token-by-token float32) / _CHUNKED (tcgen05 with
 *                  split-precision bf16 operands, float32-grade accuracy for every dtype); AUTO = chunked.
 *                  With RWKVB200_ALGO_KEEP (chunked only) the forward also writes the state at every chunk
 *                  boundary into `workspace`, and a backward called with the same flag and workspace
 *                  skips its recomputation of the forward.
 *   workspace      rwkvb200_wkv6_fwd_workspace_bytes(...) bytes: with KEEP the backward's workspace
 *                  (rwkvb200_wkv6_bwd_workspace_bytes, the two are equal), without it 16 KiB and a few
 *                  bytes per (batch, head) for the chunked path (decay-range marks, and the state handed
 *                  between the stretches a unit is worked on in when the units outnumber the SMs' CTA
 *                  slots) and none for the recurrent one.
 * Head sizes 32 and 128 (the reference's operator takes the head size in its constructor,
 * rwkv_ops/rwkv6_kernel/__init__.py:37-50) run the recurrent path whatever `algo` says, except that an
 * explicit RWKVB200_ALGO_CHUNKED returns RWKVB200_E_UNSUPPORTED; states are [head_size][head_size].
 * Sequences shorter than 8 tokens are computed by the float32 recurrence as well (same mechanism as below).
 * Decay range of the chunked path: it holds the 1e-4 parity bar while the sum of exp(w) over the 32 tokens
 * of a half chunk stays below 45 in every channel (always true for w <= 0.34).  A (batch, head) unit that
 * exceeds this is detected on the device and recomputed, forward and backward, by the float32 recurrence
 * inside the same call: results are exact for any w, such units just run at the recurrent path's speed.
 * ---------------------------------------------------------------------------------------- */
size_t rwkvb200_wkv6_fwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo);

int rwkvb200_wkv6_fwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                      const float* s0, int n_state, const int32_t* state_map,
                      void* y, float* sT, void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int head_size, int dtype, int algo, void* stream);

size_t rwkvb200_wkv6_bwd_workspace_bytes(int B, int T, int H, int head_size, int dtype, int algo);

/* Backward of wkv6, including the gradient paths the reference's GPU operator lacks (initial state,
 * final-state gradient; wkv6_cuda.cu:291,316 hard-zero them).  d_y: gradient of y; d_sT (may be NULL):
 * gradient of the final state.  Writes dr,dk,dv,dw [B,T,C] (dtype; dw is the gradient of the w input),
 * du float32 [H,64] summed over batch and time, and, when d_s0 is not NULL, the float32 gradient of the
 * per-batch-row initial state [B,H,64,64] (the caller scatters rows through state_map). */
int rwkvb200_wkv6_bwd(const void* r, const void* k, const void* v, const void* w, const float* u,
                      const float* s0, int n_state, const int32_t* state_map,
                      const void* d_y, const float* d_sT,
                      void* dr, void* dk, void* dv, void* dw, float* du, float* d_s0,
                      void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int head_size, int dtype, int algo, void* stream);

/* wkv6 on packed variable-length batches (head size 64, every dtype; the chunked tensor-core path with its
 * recurrent fallback).  The n_seq sequences lie end to end in token tensors of shape [1, total_len, H*64];
 * sequence i is tokens seq_start[i] .. seq_start[i] + seq_len[i] - 1 (device arrays of n_seq int32, every
 * length >= 1, no overlap), max_len is the longest length.  Initial states as in the dense entry points with
 * the sequence in the place of the batch row (s0 [n_state, H, 64, 64], state_map [n_seq] or NULL); sT and
 * d_s0 are [n_seq, H, 64, 64].  keep / kept as RWKVB200_ALGO_KEEP in the dense entry points; the workspace
 * is sized by rwkvb200_wkv6_varlen_workspace_bytes (the backward always needs the keep = 1 size).
 * No counterpart in the reference: its wkv6 operator takes dense [B, T, C] batches only
 * (rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:10-21); the result equals running each sequence on its own. */
size_t rwkvb200_wkv6_varlen_workspace_bytes(int n_seq, int max_len, int H, int head_size, int dtype, int keep);

int rwkvb200_wkv6_fwd_varlen(const void* r, const void* k, const void* v, const void* w, const float* u,
                             const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                             const float* s0, int n_state, const int32_t* state_map,
                             void* y, float* sT, void* workspace, size_t workspace_bytes,
                             int H, int head_size, int dtype, int keep, void* stream);

int rwkvb200_wkv6_bwd_varlen(const void* r, const void* k, const void* v, const void* w, const float* u,
                             const int32_t* seq_start, const int32_t* seq_len, int n_seq, int max_len, int total_len,
                             const float* s0, int n_state, const int32_t* state_map,
                             const void* d_y, const float* d_sT,
                             void* dr, void* dk, void* dv, void* dw, float* du, float* d_s0,
                             void* workspace, size_t workspace_bytes,
                             int H, int head_size, int dtype, int kept, void* stream);


/* ------------------------------------------------------------------------------------------
 * Diagnostics of the tensor-core path (no counterpart in the reference).
 * rwkvb200_device_status: every wait inside a tensor-core kernel (on an mbarrier that a TMA copy or
 *   an MMA completes) gives up after a fixed number of polls, records a non-zero code in a status word
 *   on the device and lets the kernel finish; this call synchronises the device, returns the word
 *   (0 = no wait ever ran out) and clears it when reset != 0.  The Python layer reads it after every
 *   operator call when RWKV_OPS_B200_CHECK_STATUS=1 is set (a debugging aid: it synchronises).
 * ---------------------------------------------------------------------------------------- */
int rwkvb200_device_status(int reset);

/* ------------------------------------------------------------------------------------------
 * Per-kernel timing for benchmarks (no counterpart in the reference, which ships no timing code).
 * When enabled, each kernel launch of the library is bracketed by CUDA events on its stream.
 * rwkvb200_profile_get synchronises on the recorded events and returns, for kernel name index i in
 * [0, rwkvb200_profile_count()), the name, the summed duration in milliseconds and the launch count.
 * ---------------------------------------------------------------------------------------- */
void rwkvb200_profile_enable(int on);
void rwkvb200_profile_reset(void);
int rwkvb200_profile_count(void);
int rwkvb200_profile_get(int i, char* name, int name_len, float* total_ms, int* launches);

#ifdef __cplusplus
}
#endif
#endif /* RWKV_OPS_B200_H */
