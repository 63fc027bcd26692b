// Entry points of the diagnostics library (libgqa_b200_selftest.so): the CUDA-core checker kernels, the
// status area of the self tests and the time-out self test.  None of this is on a product path; the
// product library (libgqa_b200.so) does not depend on it.
#include <mutex>

#include "../../include/gqa_selftest.h"
#include "gqa_kernels.cuh"
#include "selftest_common.cuh"
#include "sm100_ptx.cuh"

namespace gqa_selftest {

static __device__ __align__(256) unsigned int g_selftest_status[64];

int status_area(unsigned int** out) {
    constexpr int kMaxDev = 64;
    static unsigned int* areas[kMaxDev] = {};
    static std::mutex mu;
    int dev = 0;
    GQA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) return GQA_ERR_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lock(mu);
    if (!areas[dev]) {
        void* p = nullptr;  // the array's name is a host-side handle; kernels need the looked-up address
        GQA_CUDA_TRY(cudaGetSymbolAddress(&p, g_selftest_status));
        if (!p) return GQA_ERR_CUDA;
        areas[dev] = static_cast<unsigned int*>(p);
    }
    *out = areas[dev];
    return GQA_OK;
}

}  // namespace gqa_selftest

namespace {

using namespace sm100;

// The give-up path of the product kernels, run on purpose: same mbarrier wait, same abort flag, same
// status word, same teardown (barrier, grace period, TMEM release).  Warp 1 waits on a barrier that nothing
// ever arrives at, with a short limit; warps 2 and 3 wait (with the product limit of about a second) on a
// barrier that warp 1 would arrive at after its own wait, so they leave through the abort flag; warp 0 owns
// the tensor-memory allocation.  Nothing here faults, traps or spins without a limit.
constexpr uint32_t kSiteNeverArrives = 7, kSiteDependent = 8;

// 200 KB of (unused) dynamic shared memory keep it to one thread block per SM, as the product kernels run, so a
// launch of more blocks than SMs has later waves that find the status word set.
constexpr int kTimeoutSmemBytes = 200 * 1024;

__global__ void __launch_bounds__(128, 1) timeout_selftest_kernel(unsigned int* status, long long limit_cycles) {
    extern __shared__ uint8_t unused_smem[];
    (void)unused_smem;
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5;
    AbortCtx ctx{abort_flag, status};
    if (threadIdx.x == 0) {
        *abort_flag = (*reinterpret_cast<volatile unsigned int*>(status) != 0u) ? 98u : 0u;
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 32);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (*abort_flag != 0) {  // an earlier block of this launch has given up: leave at once, as the product kernels do
        if (warp == 0) tmem_dealloc(tmem, 32);
        if (threadIdx.x == 0) atomicAdd(status + 1, 1u);  // counted for the test
        return;
    }
    if (warp == 1) {
        if (mbar_wait_limit(&bars[0], 0, ctx, kSiteNeverArrives, limit_cycles) && (threadIdx.x & 31) == 0)
            mbar_arrive(&bars[1]);
    } else if (warp >= 2) {
        mbar_wait(&bars[1], 0, ctx, kSiteDependent);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        if (*abort_flag != 0) abort_grace_period();
        tmem_dealloc(tmem, 32);
    }
}

}  // namespace

extern "C" int gqa_selftest_timeout(void* status_word, long long limit_cycles, int blocks, gqa_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!status_word || (reinterpret_cast<uintptr_t>(status_word) & 7u)) return GQA_ERR_BAD_ARGUMENT;
    // the wait is meant to run out: keep it to at most a tenth of a second, and the launch to a few waves
    if (limit_cycles < 1 || limit_cycles > 200000000LL || blocks < 1 || blocks > 1024) return GQA_ERR_BAD_ARGUMENT;
    GQA_CUDA_TRY(cudaMemsetAsync(status_word, 0, 2 * sizeof(unsigned int), stream));
    GQA_CUDA_TRY(cudaFuncSetAttribute(timeout_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kTimeoutSmemBytes));
    timeout_selftest_kernel<<<blocks, 128, kTimeoutSmemBytes, stream>>>(static_cast<unsigned int*>(status_word),
                                                                        limit_cycles);
    gqa::count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

extern "C" int gqa_checker_fwd_simt(const void* Q, const void* K, const void* V, void* O, float* LSE, int B, int Hq,
                                    int Hkv, int S, int D, int causal, float scale, gqa_stream_t stream) {
    if (!Q || !K || !V || !O) return GQA_ERR_BAD_ARGUMENT;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || D <= 0 || D > 128 || Hq % Hkv) return GQA_ERR_UNSUPPORTED;
    const gqa::Shape s{B, Hq, Hkv, S, D, causal ? 1 : 0, scale};
    return gqa::launch_fwd_simt(Q, K, V, O, LSE, s, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int gqa_checker_bwd_simt(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                                    const float* LSE, void* dQ, void* dK, void* dV, float* delta_scratch, int B,
                                    int Hq, int Hkv, int S, int D, int causal, float scale, gqa_stream_t stream_) {
    if (!Q || !K || !V || !O || !dO || !LSE || !dQ || !dK || !dV || !delta_scratch) return GQA_ERR_BAD_ARGUMENT;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || (D != 64 && D != 128) || Hq % Hkv) return GQA_ERR_UNSUPPORTED;
    const gqa::Shape s{B, Hq, Hkv, S, D, causal ? 1 : 0, scale};
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    int rc = gqa::launch_bwd_preprocess(O, dO, nullptr, 0.f, delta_scratch, nullptr, nullptr, nullptr, s.q_rows(), D,
                                        stream);
    if (rc) return rc;
    return gqa::launch_bwd_simt(Q, K, V, dO, LSE, delta_scratch, dQ, dK, dV, s, stream);
}
