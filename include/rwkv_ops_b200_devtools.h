/* Developer entry points of librwkv_ops_b200_dev.so, the build of the library with -DRWKVB200_DEVTOOLS.
 * The shipped library (librwkv_ops_b200.so) does not contain them: it keeps no pointer after a call returns and
 * its kernels carry no instrumentation.  No counterpart in the reference.
 */
#ifndef RWKV_OPS_B200_DEVTOOLS_H
#define RWKV_OPS_B200_DEVTOOLS_H

#include "rwkv_ops_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* While device_buffer (>= 64 int64, caller-owned) is installed, one CTA of each tensor-core kernel writes
 * clock64() stamps at its phase boundaries into it; NULL switches it off. */
void rwkvb200_debug_stamps(void* device_buffer);

/*
 * rwkvb200_tc_selftest: runs one building block on caller data so a test can compare with a plain
 *   matrix product.  mode 0: out[128][128] = [X;Y] [Z;W]^T (X..W are 64x64 bf16, row-major);
 *   mode 1: dumps the 128-lane x 64-column accumulator block holding X*Z (lower lane halves) and
 *   X^T*W (upper lane halves) to out[128][64]; mode 2: TMA-loads the 64-token tile (b,t0,h) of the
 *   [B,T,H,64] bf16 tensor tok, and writes its shared-memory image twice to img (2 x 4096 bf16), the
 *   second copy after a bulk load of the first; mode 3: out[128][64] = [X^T; Y^T] Z (128-wide
 *   transposed A operand); mode 4: lanes' lower halves of out[128][64] = X^T Z + Y^T W (contraction
 *   length 128 over two adjacent tiles).
 *   mode 5: every thread waits, with a limit of a thousand polls, on an mbarrier that nothing ever
 *   completes: the wait gives up, the kernel returns normally and rwkvb200_device_status() reports code 105
 *   (the path a lost TMA copy or MMA would take, exercised without faulting or hanging anything). */
int rwkvb200_tc_selftest(int mode, const void* X, const void* Y, const void* Z, const void* W, float* out,
                         const void* tok, int B, int T, int H, int b, int t0, int h, void* img, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RWKV_OPS_B200_DEVTOOLS_H */
