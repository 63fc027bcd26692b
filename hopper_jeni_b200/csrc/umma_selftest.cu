// Building-block self test and issue-rate probe: one CTA stages two 128x128 bf16 matrices as
// 128-byte-swizzled panels (by TMA or by hand), runs a 128 x N x 128 UMMA product in one of the
// operand arrangements the attention kernels use and writes the fp32 result.  It exercises exactly
// the descriptor helpers of sm100_ptx.cuh.
#include "../../include/gqa_selftest.h"
#include "selftest_common.cuh"
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int kPanelBytes = 128 * 128;    // 128 rows x 128 B
constexpr int kColPanelBytes = 128 * 16;  // 128 rows x 16 B (un-swizzled column panel)
constexpr int kOffBars = 4 * kPanelBytes;
constexpr int kOffCol = kOffBars + 256;
constexpr int kSmemBytes = 1024 /*align*/ + kOffCol + 4 * kColPanelBytes;

struct SelftestArgs {
    const __nv_bfloat16* X;
    const __nv_bfloat16* Y;
    float* C;
    unsigned int* status;
    long long* cycles;  // null for the correctness run
    int N, mode, use_tma, reps, two_issuers;
};

// Descriptor of K step k (16 contraction elements) of a 128x128 operand held as two swizzled panels.
__device__ __forceinline__ uint64_t operand_desc(uint32_t base, int k, bool mn_major) {
    return mn_major ? make_sdesc_sw128(base + k * 2048, kPanelBytes, 1024)
                    : make_sdesc_sw128(base + (k >> 2) * kPanelBytes + (k & 3) * 32, 16, 1024);
}

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY,
                     const SelftestArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sX = smem;
    uint8_t* sY = smem + 2 * kPanelBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
    uint64_t* bar_load = bars + 0;
    uint64_t* bar_mma = bars + 1;  // [2]: one per issuing warp
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 4);
    uint8_t* sCol = smem + kOffCol;  // mode 6: X cols 0-7 | X cols 8-15 | Y cols 0-7 | Y cols 8-15

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int N = a.N, mode = a.mode;
    AbortCtx ctx{abort_flag, a.status};

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar_load, 1);
        mbar_init(&bar_mma[0], 1);
        mbar_init(&bar_mma[1], 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // ---- stage the operands --------------------------------------------------------------------
    bool ok = true;
    if (a.use_tma) {
        if (tid == 0) {
            mbar_expect_tx(bar_load, 4 * kPanelBytes);
            tma_load_2d(sX, &mapX, bar_load, 0, 0);
            tma_load_2d(sX + kPanelBytes, &mapX, bar_load, 64, 0);
            tma_load_2d(sY, &mapY, bar_load, 0, 0);
            tma_load_2d(sY + kPanelBytes, &mapY, bar_load, 64, 0);
        }
        ok = mbar_wait(bar_load, 0, ctx, 1);
    } else {
        // thread = row; 16 chunks of 16 B per 256-byte row, two panels, chunk c of row r at c ^ (r & 7)
        const uint4* gx = reinterpret_cast<const uint4*>(a.X + (size_t)tid * 128);
        const uint4* gy = reinterpret_cast<const uint4*>(a.Y + (size_t)tid * 128);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const uint32_t off = (c >> 3) * kPanelBytes + tid * 128 + (((c & 7) ^ (tid & 7)) << 4);
            *reinterpret_cast<uint4*>(sX + off) = gx[c];
            *reinterpret_cast<uint4*>(sY + off) = gy[c];
        }
    }
    if (mode == 6) {  // first 16 columns of X and Y again, as un-swizzled column panels (thread = row)
        const uint4* gx = reinterpret_cast<const uint4*>(a.X + (size_t)tid * 128);
        const uint4* gy = reinterpret_cast<const uint4*>(a.Y + (size_t)tid * 128);
        *reinterpret_cast<uint4*>(sCol + 0 * kColPanelBytes + tid * 16) = gx[0];
        *reinterpret_cast<uint4*>(sCol + 1 * kColPanelBytes + tid * 16) = gx[1];
        *reinterpret_cast<uint4*>(sCol + 2 * kColPanelBytes + tid * 16) = gy[0];
        *reinterpret_cast<uint4*>(sCol + 3 * kColPanelBytes + tid * 16) = gy[1];
    }
    fence_proxy_async_smem();
    const uint32_t tmem_a = tmem + 256;  // columns [256,320): bf16 A operand for the TMEM modes
    if (mode == 4 || mode == 5) {
        const uint32_t* gx = reinterpret_cast<const uint32_t*>(a.X + (size_t)tid * 128);
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = gx[c * 32 + i];
            tmem_st32(tmem_a + lane_base + c * 32, r);
        }
        tmem_wait_st();
    }
    tc_fence_before_sync();
    __syncthreads();

    // ---- issue: the whole warp runs the loop, one elected lane issues ----------------------------
    if ((warp == 0 || (warp == 1 && a.two_issuers)) && ok) {
        tc_fence_after_sync();
        const uint32_t leader = elect_one() ? 1u : 0u;
        const bool a_mn = (mode == 2 || mode == 3);
        const bool b_mn = (mode == 1 || mode == 3 || mode == 5);
        const uint32_t idesc = make_idesc_bf16(128, N, a_mn, b_mn);
        const uint32_t ax = smem_u32(sX), bx = smem_u32(sY), cx = smem_u32(sCol);
        const uint32_t td = tmem + (warp == 1 ? 128u : 0u);  // a second issuer works on its own accumulator
        uint64_t ad[8], bd[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            ad[k] = operand_desc(ax, k, a_mn);
            bd[k] = operand_desc(bx, k, b_mn);
        }
        const long long t_issue = clock64();
#pragma unroll 1
        for (int rep = 0; rep < a.reps; ++rep) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t acc = (k > 0 || rep > 0) ? 1u : 0u;
                if (mode == 4 || mode == 5) umma_ts_pred(leader, td, tmem_a + k * 8, bd[k], idesc, acc);
                else umma_ss_pred(leader, td, ad[k], bd[k], idesc, acc);
            }
        }
        if (mode == 6)  // once more over columns 0-15, read through the un-swizzled descriptors
            umma_ss_pred(leader, td, make_sdesc_noswizzle(cx, kColPanelBytes, 128),
                         make_sdesc_noswizzle(cx + 2 * kColPanelBytes, kColPanelBytes, 128), idesc, 1u);
        umma_commit_pred(leader, &bar_mma[warp]);
        if (a.cycles) {  // issue-rate probe: time from first issue to completion of the last product
            mbar_wait(&bar_mma[warp], 0, ctx, 3);
            if ((tid & 31) == 0) a.cycles[warp] = clock64() - t_issue;
        }
    }
    if (warp <= 1) __syncwarp();
    if (ok) ok = mbar_wait(&bar_mma[0], 0, ctx, 2);
    tc_fence_after_sync();
    if (ok && !a.cycles) {
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        for (int c = 0; c < N; c += 32) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_base + c, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) a.C[(size_t)tid * N + c + i] = __uint_as_float(r[i]);
        }
    }
    if (a.two_issuers && ok) mbar_wait(&bar_mma[1], 0, ctx, 4);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

int run_selftest(const void* X, const void* Y, float* C, int N, int mode, int use_tma, int reps, int two_issuers,
                 long long* dcycles, unsigned int* status, cudaStream_t stream) {
    CUtensorMap mx, my;
    int rc = gqa::make_panel_tmap(&mx, X, 128, 128, 128);
    if (rc) return rc;
    rc = gqa::make_panel_tmap(&my, Y, 128, 128, 128);
    if (rc) return rc;
    GQA_CUDA_TRY(cudaMemsetAsync(status, 0, 64, stream));
    GQA_CUDA_TRY(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    SelftestArgs a{static_cast<const __nv_bfloat16*>(X), static_cast<const __nv_bfloat16*>(Y), C, status, dcycles,
                   N, mode, use_tma, reps, two_issuers};
    umma_selftest_kernel<<<1, 128, kSmemBytes, stream>>>(mx, my, a);
    gqa::count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

}  // namespace

extern "C" int gqa_selftest_umma(const void* X, const void* Y, float* C, int N, int mode, int use_tma,
                                 gqa_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!X || !Y || !C) return GQA_ERR_BAD_ARGUMENT;
    if ((N != 64 && N != 128) || mode < 0 || mode > 6) return GQA_ERR_UNSUPPORTED;
    if (!gqa::aligned16(X) || !gqa::aligned16(Y) || !gqa::aligned16(C)) return GQA_ERR_BAD_ARGUMENT;
    unsigned int* status = nullptr;
    int rc = gqa_selftest::status_area(&status);
    if (rc) return rc;
    rc = run_selftest(X, Y, C, N, mode, use_tma, 1, 0, nullptr, status, stream);
    if (rc) return rc;
    return gqa_check_status(status, stream_);
}

// Issue-rate probe for arrangements 0-5: `reps` x 8 back-to-back K = 16 products accumulating into one
// TMEM tile, issued by one warp (two_issuers = 0) or by two warps on separate accumulators; reports the
// SM cycles per product per issuing warp.  Synchronises `stream`.
extern "C" int gqa_selftest_umma_cycles(const void* X, const void* Y, float* C, int N, int mode, int reps,
                                        int two_issuers, float* cycles_per_product, gqa_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    // one CTA runs reps x 8 products back to back with no wait inside the loop: keep it to a few milliseconds
    if (!X || !Y || !C || !cycles_per_product || reps < 1 || reps > 65536) return GQA_ERR_BAD_ARGUMENT;
    if ((N != 64 && N != 128) || mode < 0 || mode > 5) return GQA_ERR_UNSUPPORTED;
    unsigned int* status = nullptr;
    int rc = gqa_selftest::status_area(&status);
    if (rc) return rc;
    long long* dcycles = reinterpret_cast<long long*>(status + 2);  // the status area is 256 bytes
    rc = run_selftest(X, Y, C, N, mode, 1, reps, two_issuers ? 1 : 0, dcycles, status, stream);
    if (rc) return rc;
    long long h[2] = {0, 0};
    GQA_CUDA_TRY(cudaMemcpyAsync(h, dcycles, sizeof h, cudaMemcpyDeviceToHost, stream));
    GQA_CUDA_TRY(cudaStreamSynchronize(stream));
    *cycles_per_product = (float)(h[0] > h[1] ? h[0] : h[1]) / (8.0f * reps);
    return gqa_check_status(status, stream_);
}
