// Building-block self test: one CTA stages two 128x128 bf16 matrices as
// 128-byte-swizzled panels (by TMA or by hand), runs a 128 x N x 128 UMMA product
// in one of six operand arrangements and writes the fp32 result.  It exercises
// exactly the descriptor helpers the attention kernels use.
#include "gqa_common.cuh"
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int kPanelBytes = 128 * 128;  // 128 rows x 128 B
constexpr int kSmemBytes = 4 * kPanelBytes + 1024 /*align*/ + 256 /*barriers*/;

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY,
                     const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ Y, float* __restrict__ C,
                     int N, int mode, int use_tma, unsigned int* status, int reps, long long* cycles, int variant) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sX = smem;
    uint8_t* sY = smem + 2 * kPanelBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 4 * kPanelBytes);
    uint64_t* bar_load = bars + 0;
    uint64_t* bar_mma = bars + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 3);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    AbortCtx ctx{abort_flag, status};

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar_load, 1);
        mbar_init(bar_mma, 1);
        mbar_init(bars + 4, 1);
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

    bool ok = true;
    if (use_tma) {
        if (tid == 0) {
            mbar_expect_tx(bar_load, 4 * kPanelBytes);
            tma_load_2d(sX, &mapX, bar_load, 0, 0);
            tma_load_2d(sX + kPanelBytes, &mapX, bar_load, 64, 0);
            tma_load_2d(sY, &mapY, bar_load, 0, 0);
            tma_load_2d(sY + kPanelBytes, &mapY, bar_load, 64, 0);
        }
        ok = mbar_wait(bar_load, 0, ctx, 1);
    } else {
        // thread = row; 16 chunks of 16 B per 256-byte row, two panels
        const uint4* gx = reinterpret_cast<const uint4*>(X + (size_t)tid * 128);
        const uint4* gy = reinterpret_cast<const uint4*>(Y + (size_t)tid * 128);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const uint32_t off = (c >> 3) * kPanelBytes + tid * 128 + (((c & 7) ^ (tid & 7)) << 4);
            *reinterpret_cast<uint4*>(sX + off) = gx[c];
            *reinterpret_cast<uint4*>(sY + off) = gy[c];
        }
        fence_proxy_async_smem();
    }
    const uint32_t tmem_a = tmem + 256;  // columns [256,320): bf16 A operand for the TMEM modes
    if (mode >= 4) {
        const uint32_t* gx = reinterpret_cast<const uint32_t*>(X + (size_t)tid * 128);
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

    if ((warp == 0 || (warp == 1 && (variant & 64))) && ok) {  // a whole warp runs the issue loop; an elected lane issues
        tc_fence_after_sync();
        const bool a_mn = (mode == 2 || mode == 3);
        const bool b_mn = (mode == 1 || mode == 3 || mode == 5);
        const uint32_t idesc = make_idesc_bf16(128, N, a_mn, b_mn);
        const uint32_t ax = smem_u32(sX), bx = smem_u32(sY);
        const long long t_issue = clock64();
        if (variant & 8) {  // lean loop: descriptors precomputed, nothing but the issue in the body
            uint64_t ad[8], bd[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t off = (N == 256 ? 0 : (k >> 2) * kPanelBytes) + (k & 3) * 32;
                ad[k] = make_sdesc_sw128(ax + off, 16, 1024);
                bd[k] = make_sdesc_sw128(bx + off, 16, 1024);
            }
            const uint32_t leader = elect_one() ? 1u : 0u;
            // a second issuing warp (variant bit 6) works on its own accumulator and barrier
            const uint32_t td = tmem + (warp == 1 ? 128u : 0u);
            const uint32_t ta = tmem_a;
#pragma unroll 1
            for (int rep = 0; rep < reps; ++rep) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (variant & 16) {
                        if (mode >= 4) umma_ts_pred(leader, td, ta + k * 8, bd[k], idesc, 1u);
                        else umma_ss_pred(leader, td, ad[k], bd[k], idesc, 1u);
                    } else {
                        if (mode >= 4) umma_ts_warp(td, ta + k * 8, bd[k], idesc, 1u);
                        else umma_ss_warp(td, ad[k], bd[k], idesc, 1u);
                    }
                }
            }
        } else
#pragma unroll 1
        for (int rep = 0; rep < reps; ++rep)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t kmaj_off = (k >> 2) * kPanelBytes + (k & 3) * 32;
            const uint32_t mn_off = k * 2048;
            const uint64_t bdesc = b_mn ? make_sdesc_sw128(bx + mn_off, kPanelBytes, 1024)
                                        : make_sdesc_sw128(bx + kmaj_off, 16, 1024);
            const uint32_t acc = (variant & 2) ? 0u : uint32_t((k > 0) || (rep > 0));
            const uint32_t d = tmem + ((variant & 1) ? (k & 1) * 64 : 0);
            if (mode >= 4) {
                umma_ts_warp(d, tmem_a + k * 8, bdesc, idesc, acc);
            } else {
                const uint64_t adesc = a_mn ? make_sdesc_sw128(ax + mn_off, kPanelBytes, 1024)
                                            : make_sdesc_sw128(ax + kmaj_off, 16, 1024);
                umma_ss_warp(d, adesc, bdesc, idesc, acc);
            }
        }
        uint64_t* done_bar = (warp == 1) ? (bars + 4) : bar_mma;
        umma_commit_warp(done_bar);
        if (cycles) {  // throughput probe: time from first issue to completion of the last product
            mbar_wait(done_bar, 0, ctx, 3);
            if ((tid & 31) == 0) cycles[warp] = clock64() - t_issue;
        }
    }
    if (warp <= 1) __syncwarp();  // keep lanes 1-31 from spinning on the barrier while lane 0 still issues
    if (variant & 4) {            // probe variant: nobody polls the barrier while the products run
        __syncthreads();
    }
    if (ok) ok = mbar_wait(bar_mma, 0, ctx, 2);
    tc_fence_after_sync();
    if (ok) {
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        for (int c = 0; c < N; c += 32) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_base + c, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) C[(size_t)tid * N + c + i] = __uint_as_float(r[i]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

extern "C" int gqa_selftest_umma(const void* X, const void* Y, float* C, int N, int mode, int use_tma,
                                 gqa_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!X || !Y || !C) return GQA_ERR_BAD_ARGUMENT;
    if ((N != 64 && N != 128) || mode < 0 || mode > 5) return GQA_ERR_UNSUPPORTED;
    if (!gqa::aligned16(X) || !gqa::aligned16(Y) || !gqa::aligned16(C)) return GQA_ERR_BAD_ARGUMENT;
    CUtensorMap mx, my;
    int rc = gqa::make_panel_tmap(&mx, X, 128, 128, 128);
    if (rc) return rc;
    rc = gqa::make_panel_tmap(&my, Y, 128, 128, 128);
    if (rc) return rc;
    unsigned int* status = nullptr;
    rc = gqa::forward_status_word(&status);
    if (rc) return rc;
    GQA_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(unsigned int), stream));
    GQA_CUDA_TRY(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    umma_selftest_kernel<<<1, 128, kSmemBytes, stream>>>(mx, my, static_cast<const __nv_bfloat16*>(X),
                                                         static_cast<const __nv_bfloat16*>(Y), C, N, mode, use_tma,
                                                         status, 1, nullptr, 0);
    gqa::count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return gqa_check_status(nullptr, stream_);
}

// Throughput probe for the same six operand arrangements: `reps` x 8 back-to-back K = 16 products
// accumulating into one TMEM tile; reports the average tensor-pipe cycles per product.  Values of C
// are meaningless for reps > 1 (the sum is repeated).  Synchronises `stream`.
extern "C" int gqa_selftest_umma_cycles(const void* X, const void* Y, float* C, int N, int mode, int reps,
                                        float* cycles_per_product, gqa_stream_t stream_) {
    const int variant = mode >> 8;  // development knobs in the high bits (0 = the documented behaviour)
    mode &= 0xff;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!X || !Y || !C || !cycles_per_product || reps < 1) return GQA_ERR_BAD_ARGUMENT;
    if ((N != 64 && N != 128 && !(variant && N == 256)) || mode < 0 || mode > 5) return GQA_ERR_UNSUPPORTED;
    CUtensorMap mx, my;
    int rc = gqa::make_panel_tmap(&mx, X, 128, 128, 128);
    if (rc) return rc;
    rc = gqa::make_panel_tmap(&my, Y, 128, 128, 128);
    if (rc) return rc;
    unsigned int* status = nullptr;
    rc = gqa::forward_status_word(&status);
    if (rc) return rc;
    long long* dcycles = reinterpret_cast<long long*>(status + 2);  // the status allocation is 256 bytes
    GQA_CUDA_TRY(cudaMemsetAsync(status, 0, 64, stream));
    GQA_CUDA_TRY(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    umma_selftest_kernel<<<1, 128, kSmemBytes, stream>>>(mx, my, static_cast<const __nv_bfloat16*>(X),
                                                         static_cast<const __nv_bfloat16*>(Y), C, N, mode, 1, status,
                                                         reps, dcycles, variant);
    gqa::count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    long long h[2] = {0, 0};
    GQA_CUDA_TRY(cudaMemcpyAsync(h, dcycles, sizeof h, cudaMemcpyDeviceToHost, stream));
    GQA_CUDA_TRY(cudaStreamSynchronize(stream));
    *cycles_per_product = (float)(h[0] > h[1] ? h[0] : h[1]) / (8.0f * reps);
    return gqa_check_status(nullptr, stream_);
}
