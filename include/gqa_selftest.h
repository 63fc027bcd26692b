/*
 * gqa_selftest.h -- C ABI of the diagnostics library (libgqa_b200_selftest.so) that accompanies
 * libgqa_b200.so: building-block self tests, an issue-rate probe, CUDA-core checker kernels and a
 * self test of the bounded-wait give-up path.  The test-suite uses it; no product entry point does,
 * and the product library does not depend on it.  Status codes and gqa_stream_t come from gqa.h.
 */
#ifndef GQA_B200_SELFTEST_H_
#define GQA_B200_SELFTEST_H_

#include "gqa.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Building-block self test: one 128 x N x 128 bf16 UMMA product from two
 * 128 x 128 bf16 matrices X and Y (row-major) into C[128, N] fp32.
 *   mode 0: C = X  * Y^T   (A K-major,  B K-major)
 *   mode 1: C = X  * Y     (A K-major,  B MN-major)
 *   mode 2: C = X^T * Y^T  (A MN-major, B K-major)
 *   mode 3: C = X^T * Y    (A MN-major, B MN-major)
 *   mode 4: C = X  * Y^T   (A from tensor memory, B K-major)
 *   mode 5: C = X  * Y     (A from tensor memory, B MN-major)
 *   mode 6: C = X  * Y^T + X[:, :16] * Y[:, :16]^T  (mode 0 plus one K step read through
 *           un-swizzled 16-byte-row column panels)
 * N is 64 or 128 (for N = 64 only the first 64 rows/columns of Y are used).
 * use_tma != 0 stages X and Y with TMA tile loads, otherwise threads write the
 * swizzled layout themselves.  Synchronises `stream`.  No counterpart in the
 * reference (its kernels are wgmma-based); used by the test-suite only.
 */
int gqa_selftest_umma(const void* X, const void* Y, float* C, int N, int mode, int use_tma,
                      gqa_stream_t stream);

/*
 * Issue-rate probe over arrangements 0-5: reps x 8 back-to-back K = 16 products into one
 * accumulator, issued by one warp or (two_issuers != 0) by two warps on separate accumulators;
 * *cycles_per_product (host memory) receives the SM cycles per product per issuing warp.
 * C is scratch.  Synchronises `stream`.  No counterpart in the reference.
 */
int gqa_selftest_umma_cycles(const void* X, const void* Y, float* C, int N, int mode, int reps,
                             int two_issuers, float* cycles_per_product, gqa_stream_t stream);

/*
 * CUDA-core checker kernels (diagnostics): a slow, simple restatement of forward
 * and backward on the device, used by the tests to cross-check the tensor-core
 * kernels at sizes where the CPU oracle takes too long.  No product entry point
 * dispatches to them.  Same tensor contract as above, any S, D <= 128;
 * `delta_scratch` is B*Hq*S floats of device memory.  They follow the reference's
 * per-head loops (precision/baseline_gqa.py:169-197).
 */
int gqa_checker_fwd_simt(const void* Q, const void* K, const void* V, void* O, float* LSE,
                         int B, int Hq, int Hkv, int S, int D, int causal, float scale,
                         gqa_stream_t stream);
int gqa_checker_bwd_simt(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                         const float* LSE, void* dQ, void* dK, void* dV, float* delta_scratch,
                         int B, int Hq, int Hkv, int S, int D, int causal, float scale,
                         gqa_stream_t stream);

/*
 * Self test of the path a kernel takes when one of its bounded waits gives up.  The reference's waits spin
 * without limit (src/attention/GQA_bwd_baseline.cu:85-93), so it has no counterpart there.  Launches
 * `blocks` thread blocks (1..1024, one per SM at a time) in which one warp waits for `limit_cycles` SM cycles
 * (1..2e8, i.e. at most a tenth of a second) on a barrier that nothing arrives at; the wait runs out, the
 * thread block records wait site 7 and its block index in status_word[0], raises its abort flag, the other
 * warps leave their waits through the flag, and the block frees its tensor memory and exits -- the same
 * functions, status encoding and teardown the attention kernels use.  Thread blocks that start after the
 * word has been set return at once and count themselves in status_word[1].  `status_word` is device memory
 * of at least 8 bytes, 8-byte aligned; pass it to gqa_check_status() afterwards, which returns
 * GQA_ERR_DEVICE_TIMEOUT and leaves the decoded site and block in gqa_last_cuda_error().  The device stays
 * usable: nothing faults, traps or waits without a limit.
 */
int gqa_selftest_timeout(void* status_word, long long limit_cycles, int blocks, gqa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GQA_B200_SELFTEST_H_ */
