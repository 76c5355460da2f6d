// Host-side helpers of the tensor-core path: tensor-map encoding (driver entry point looked up at run
// time, so the library does not link libcuda), the device status word, and a self-test entry point that
// exercises every tcgen05 / TMA building block of tc.cuh on known data.
#include <mutex>

#include "common.cuh"
#include "tc.cuh"
#ifdef RWKVB200_DEVTOOLS
#include "../../include/rwkv_ops_b200_devtools.h"
#endif

namespace rwkvb200 {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static __device__ int g_status_word;
std::mutex g_mu;
int* g_status_ptr[64] = {};

}  // namespace

int make_token_tensor_map(CUtensorMap* out, const void* base, int B, int T, int H, int head_first) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { last_cuda_error_slot() = 100000; return RWKVB200_E_CUDA; }
  // dims, fastest first: (64 channels, T, H, B); strides in bytes of dims 1..3
  const cuuint64_t row = HS * 2;
  cuuint64_t dims[4] = {(cuuint64_t)HS, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3];
  if (head_first) { strides[0] = row; strides[1] = row * T; }
  else            { strides[0] = row * H; strides[1] = row; }
  strides[2] = row * (cuuint64_t)T * H;
  cuuint32_t box[4] = {(cuuint32_t)HS, 64, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  // The driver entry point needs the device's primary context current on THIS host thread; a thread
  // that has only been handed the device by its framework (e.g. an autograd worker) may not have it yet.
  int dev = 0;
  if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaSetDevice(dev))) return RWKVB200_E_CUDA;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) return RWKVB200_OK;
  last_cuda_error_slot() = 100000 + (int)r;   // driver-API result, reported by rwkvb200_last_cuda_error()
  return RWKVB200_E_CUDA;
}

// [B][T][H][64] rows of 2- or 4-byte elements, box = 64 rows x 64 elements of one (batch, head), no swizzle:
// the box lands in shared memory as 64 consecutive rows of 64 * elem_bytes bytes
int make_row_tensor_map(CUtensorMap* out, const void* base, int B, int T, int H, int elem_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { last_cuda_error_slot() = 100000; return RWKVB200_E_CUDA; }
  const cuuint64_t row = (cuuint64_t)HS * elem_bytes;
  cuuint64_t dims[4] = {(cuuint64_t)HS, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {row * H, row, row * (cuuint64_t)T * H};
  cuuint32_t box[4] = {(cuuint32_t)HS, 64, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  int dev = 0;
  if (cuda_ok(cudaGetDevice(&dev)) || cuda_ok(cudaSetDevice(dev))) return RWKVB200_E_CUDA;
  CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 4,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) return RWKVB200_OK;
  last_cuda_error_slot() = 100000 + (int)r;
  return RWKVB200_E_CUDA;
}

#ifdef RWKVB200_DEVTOOLS
static long long* g_stamp_buffer = nullptr;
long long* debug_stamp_buffer() { return g_stamp_buffer; }
#else
long long* debug_stamp_buffer() { return nullptr; }
#endif

int* device_status_ptr() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    g_status_ptr[dev] = reinterpret_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

#ifdef RWKVB200_DEVTOOLS
// ---------------------------------------------------------------------------------------------
// self-test kernel: one CTA, 128 threads
// ---------------------------------------------------------------------------------------------
namespace {

using namespace tc;

struct SelfTestSmem {
  unsigned char tiles[6][TILE_BYTES];   // 1024-byte aligned
  uint64_t bar_mma, bar_tma, bar_bulk;
  uint32_t tmem_base;
};

// copy a row-major 64x64 bf16 matrix from global into a swizzled tile (all threads)
__device__ void load_tile_plain(unsigned char* tile, const __nv_bfloat16* src, int ld) {
  for (int i = threadIdx.x; i < 64 * 8; i += blockDim.x) {
    const int row = i >> 3, chunk = i & 7;
    *reinterpret_cast<uint4*>(tile + tile_chunk_off(row, chunk)) =
        *reinterpret_cast<const uint4*>(src + (long long)row * ld + chunk * 8);
  }
}

// mode 0: D[128x128] = [X;Y] [Z;W]^T                      (M=128, N=128, both K-major)
// mode 1: lanes' lower halves: X * Z  (A K-major, B MN-major, M=64,N=64)
//         lanes' upper halves: X^T * W (A MN-major, B MN-major), written at lane offset 16;
//         the whole 128-lane x 64-column TMEM block is dumped to out[128][64]
// mode 2: TMA tiled load of the token tile (b,t0,h) of `tok` into a tile, bulk-store its raw image to
//         img[0..4095], bulk-load that image back into a second tile and store it again to img[4096..]
__global__ void __launch_bounds__(128)
tc_selftest_kernel(int mode, const __nv_bfloat16* X, const __nv_bfloat16* Y, const __nv_bfloat16* Z,
                   const __nv_bfloat16* W, float* out, const __grid_constant__ CUtensorMap tmap,
                   int b, int t0, int h, __nv_bfloat16* img, int* status) {
  extern __shared__ unsigned char smem_raw[];
  SelfTestSmem& sm = *reinterpret_cast<SelfTestSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&sm.bar_mma, 1);
    mbar_init(&sm.bar_tma, 1);
    mbar_init(&sm.bar_bulk, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sm.tmem_base;
  bool ok = true;

  if (mode == 5) {
    // nothing ever arrives on this barrier: the bounded wait must give up and report
    ok = mbar_wait(&sm.bar_bulk, 0, status, 105, 1000u);
    if (ok && out) out[0] = 1.f;      // (would mean that the wait returned as if completed)
  } else if (mode == 0 || mode == 1 || mode == 3 || mode == 4) {
    load_tile_plain(sm.tiles[0], X, 64);
    load_tile_plain(sm.tiles[1], Y, 64);
    load_tile_plain(sm.tiles[2], Z, 64);
    load_tile_plain(sm.tiles[3], W, 64);
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      if (mode == 0) {
        umma_tile<128, 128, 0, 0>(tbase, smem_u32(sm.tiles[0]), smem_u32(sm.tiles[2]), false);
      } else if (mode == 3) {
        // [X^T; Y^T] Z : 128-wide MN-major A (second half one tile further), MN-major B
        umma_tile<128, 64, 1, 1>(tbase, smem_u32(sm.tiles[0]), smem_u32(sm.tiles[2]), false, TILE_BYTES);
      } else if (mode == 4) {
        // X^T Z + Y^T W as one product with a contraction length of 128 (both operands MN-major)
        umma_tile<64, 64, 1, 1, 8>(tbase, smem_u32(sm.tiles[0]), smem_u32(sm.tiles[2]), false);
      } else {
        umma_tile<64, 64, 0, 1>(tmem_addr(tbase, 0, 0), smem_u32(sm.tiles[0]), smem_u32(sm.tiles[2]), false);
        umma_tile<64, 64, 1, 1>(tmem_addr(tbase, 16, 0), smem_u32(sm.tiles[0]), smem_u32(sm.tiles[3]), false);
      }
      umma_commit(&sm.bar_mma);
    }
    ok = mbar_wait(&sm.bar_mma, 0, status, 101);
    tc_fence_after();
    if (ok) {
      const int ncol = mode == 0 ? 128 : 64;   // modes 1, 3, 4 dump 128 lanes x 64 columns
      for (int c0 = 0; c0 < ncol; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tbase, 32 * warp, c0), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) out[(long long)tid * ncol + c0 + j] = __uint_as_float(r[j]);
      }
    }
  } else {
    if (tid == 0) {
      mbar_expect_tx(&sm.bar_tma, TILE_BYTES);
      tma_load_4d(sm.tiles[0], &tmap, &sm.bar_tma, 0, t0, h, b);
    }
    ok = mbar_wait(&sm.bar_tma, 0, status, 102);
    if (ok && tid == 0) {
      bulk_store(img, sm.tiles[0], TILE_BYTES);
      bulk_commit();
      bulk_wait_all();
      mbar_expect_tx(&sm.bar_bulk, TILE_BYTES);
      bulk_load(sm.tiles[1], img, TILE_BYTES, &sm.bar_bulk);
    }
    if (ok) ok = mbar_wait(&sm.bar_bulk, 0, status, 103);
    if (ok && tid == 0) {
      bulk_store(img + 4096, sm.tiles[1], TILE_BYTES);
      bulk_commit();
      bulk_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 128);
}

}  // namespace
#endif  // RWKVB200_DEVTOOLS
}  // namespace rwkvb200

using namespace rwkvb200;

extern "C" {

#ifdef RWKVB200_DEVTOOLS
void rwkvb200_debug_stamps(void* device_buffer) { g_stamp_buffer = reinterpret_cast<long long*>(device_buffer); }
#endif

int rwkvb200_device_status(int reset) {
  int* p = device_status_ptr();
  if (!p) return RWKVB200_E_CUDA;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return RWKVB200_E_CUDA;
  if (reset && v != 0) {
    int z = 0;
    if (cudaMemcpy(p, &z, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return RWKVB200_E_CUDA;
  }
  return v;
}

#ifdef RWKVB200_DEVTOOLS
int rwkvb200_tc_selftest(int mode, const void* X, const void* Y, const void* Z, const void* W, float* out,
                         const void* tok, int B, int T, int H, int b, int t0, int h, void* img, void* stream) {
  if (mode < 0 || mode > 5) return RWKVB200_E_SHAPE;
  int* status = device_status_ptr();
  if (!status) { last_cuda_error_slot() = 99999; return RWKVB200_E_CUDA; }
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  if (mode == 2) {
    if (!tok || !img) return RWKVB200_E_NULL;
    int e = make_token_tensor_map(&tmap, tok, B, T, H, 0);
    if (e) return e;
  } else if (mode != 5 && (!X || !Y || !Z || !W || !out)) {
    return RWKVB200_E_NULL;
  }
  const int smem = (int)sizeof(SelfTestSmem) + 1024;
  if (cuda_ok(cudaFuncSetAttribute(tc_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))) return RWKVB200_E_CUDA;
  tc_selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(
      mode, (const __nv_bfloat16*)X, (const __nv_bfloat16*)Y, (const __nv_bfloat16*)Z, (const __nv_bfloat16*)W, out,
      tmap, b, t0, h, (__nv_bfloat16*)img, status);
  return check_launch();
}
#endif  // RWKVB200_DEVTOOLS

}  // extern "C"
