// GQA backward, the alternative dQ path for sm_100a: a separate query-parallel pass.
//
// One CTA owns one 128-row query tile of one (batch, query head) and streams the KV head's 128-row key/value
// blocks through TMA rings, as the forward does.  It recomputes, in the natural orientation (a TMEM lane is a
// query row),
//   S  = Q K^T,  dP = dO V^T        (both operands K-major from TMA panels, one 64-key half-block at a time)
//   P  = exp2(scale*log2e * S - LSE*log2e)  -> rounded to bf16
//   dS = bf16(P * (dP - Delta))             -> packed into the head of the S half-block buffer in TMEM
//   dQ += dS K                              (A from TMEM, B = the key block read MN-major)
// and writes dQ = bf16(scale * sum) once.  dQ needs no accumulator in global memory, no zeroing, no finalise pass,
// and its summation order is fixed: it is bit-reproducible by construction.  The price is that S and dP are
// computed a second time (the KV-parallel main kernel still needs them for dK and dV) -- 3 products here plus 4
// there instead of 5 -- and with them a second set of exponentials.
//
// Roles (10 warps):
//   warps 0-7  two elementwise warpgroups; both cover all 128 query rows (thread = row = TMEM lane), warpgroup w
//              handles key columns [32w, 32w+32) of every 64-key half-block
//   warp  8    TMA producer (Q and dO once, K and V rings)
//   warp  9    UMMA issuer (one thread: the products into the one dQ accumulator stay ordered)
// S and dP have two half-block buffers each (2 x 64 + 2 x 64 TMEM columns, dQ D more): while the warpgroups work
// on half-block j the issuer has already produced S and dP of half-block j+1.
//
// The reference's first generations are built this way (a dQ kernel per query tile looping over key tiles beside a
// dK/dV kernel per key tile: src/attention/GQA_bwd.cu:29, :415, :1416); its shipped kernel accumulates dQ with
// TMA reduce-add instead (src/attention/GQA_bwd_baseline.cu:360-365), as this library's default path does.
#include "gqa_common.cuh"
#include "gqa_kernels.cuh"
#include "sm100_ptx.cuh"

namespace gqa {
namespace {

using namespace sm100;

constexpr int kTile = 128;             // query rows per tile and key rows per block
constexpr int kPanel = kTile * 128;    // bytes of one 64-column panel of a 128-row tile
constexpr int kHalf = 64;              // keys per half-block
constexpr int kEwThreads = 256;
constexpr int kWarpTma = 8, kWarpMma = 9;
constexpr int kThreads = 10 * 32;
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct DqCfg {
    static constexpr int kPanels = D / 64;
    static constexpr int kTileBytes = kPanels * kPanel;  // one 128 x D bf16 tile
    static constexpr int kStages = (D == 64) ? 4 : 2;
    static constexpr int kOffQ = 0;
    static constexpr int kOffDO = kOffQ + kTileBytes;
    static constexpr int kOffK = kOffDO + kTileBytes;
    static constexpr int kOffV = kOffK + kStages * kTileBytes;
    static constexpr int kOffBars = kOffV + kStages * kTileBytes;
    static constexpr int kSmemTotal = kOffBars + 512;  // the dynamic window must start 1024-byte aligned (checked)
    static constexpr uint32_t kTmemCols = 512;
    static constexpr uint32_t kColS = 0, kColDP = 128, kColDQ = 256;  // S and dP: two 64-column half-block buffers each
    static_assert(256 + D <= 512, "TMEM budget");
    static_assert(kSmemTotal <= 227 * 1024, "shared memory budget");
    static_assert(kSmemTotal > 114 * 1024, "one CTA per SM is assumed by the 512-column TMEM allocation");
};

struct DqParams {
    __nv_bfloat16* dQ;
    const float* lse;    // [B*Hq*S] natural log
    const float* delta;  // [B*Hq*S] rowsum(dO * O)
    unsigned int* status;
    int Hq, Hkv, S, causal, n_qtiles, bshd, d_real;
    float scale, scale_log2;
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
gqa_bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapDO,
                        const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                        const DqParams p) {
    using Cfg = DqCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // swizzled panels need 1024-byte alignment; report instead of computing garbage
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, 0x80000000u | (99u << 20));
        return;
    }
    uint8_t* sQ = smem + Cfg::kOffQ;
    uint8_t* sDO = smem + Cfg::kOffDO;
    uint8_t* sK = smem + Cfg::kOffK;
    uint8_t* sV = smem + Cfg::kOffV;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
    uint64_t* qdo_full = bars;              // TMA: Q and dO tiles
    uint64_t* dq_full = bars + 1;           // issuer: every product complete
    uint64_t* sdp_full = bars + 2;          // [2] per half-block buffer: S(j) and dP(j) written
    uint64_t* ds_ready = bars + 4;          // [2] per buffer: dS(j) stored by the warpgroups (S(j), dP(j) consumed)
    uint64_t* dq_done = bars + 6;           // [2] per buffer: dS(j) K completed
    uint64_t* k_full = bars + 8;            // [kStages]
    uint64_t* k_empty = k_full + Cfg::kStages;
    uint64_t* v_full = k_empty + Cfg::kStages;
    uint64_t* v_empty = v_full + Cfg::kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_empty + Cfg::kStages);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    AbortCtx ctx{abort_flag, p.status};

    // ---- work decode ------------------------------------------------------------
    const int qt = p.causal ? (p.n_qtiles - 1 - (int)blockIdx.x) : (int)blockIdx.x;  // heavy causal tiles first
    const int hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int q0 = qt * kTile;
    const int n_blocks_all = (p.S + kTile - 1) / kTile;
    const int n_blk = p.causal ? qt + 1 : n_blocks_all;
    const int total = 2 * n_blk;  // half-blocks
    // Tensor-map coordinates (x = column, y = position in the sequence, z = matrix), as in the other kernels.
    const int q_x = p.bshd ? hq * D : 0, q_z = p.bshd ? b : b * p.Hq + hq;
    const int kv_x = p.bshd ? hkv * D : 0, kv_z = p.bshd ? b : b * p.Hkv + hkv;

    // ---- setup ------------------------------------------------------------------
    if (tid == 0) {
        *abort_flag = (*reinterpret_cast<volatile unsigned int*>(p.status) != 0u) ? 98u : 0u;  // see the main kernel
        mbar_init(qdo_full, 1);
        mbar_init(dq_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sdp_full[i], 1);
            mbar_init(&ds_ready[i], kEwThreads);
            mbar_init(&dq_done[i], 1);
        }
        for (int i = 0; i < Cfg::kStages; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        fence_mbar_init();
    }
    if (warp == kWarpMma) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (*abort_flag != 0) {  // uniform: every thread reads the flag after the barrier
        if (warp == kWarpMma) tmem_dealloc(tmem, Cfg::kTmemCols);
        return;
    }

    if (warp == kWarpTma) {
        // ======================= TMA producer =======================
        if (elect_one()) {
            tma_prefetch_desc(&mapQ);
            tma_prefetch_desc(&mapDO);
            tma_prefetch_desc(&mapK);
            tma_prefetch_desc(&mapV);
            mbar_expect_tx(qdo_full, 2 * Cfg::kTileBytes);
            for (int pn = 0; pn < Cfg::kPanels; ++pn) {
                tma_load_3d(sQ + pn * kPanel, &mapQ, qdo_full, q_x + pn * 64, q0, q_z);
                tma_load_3d(sDO + pn * kPanel, &mapDO, qdo_full, q_x + pn * 64, q0, q_z);
            }
            for (int n = 0; n < n_blk; ++n) {
                const int st = n % Cfg::kStages;
                const uint32_t use = n / Cfg::kStages;
                if (use > 0 && !mbar_wait(&k_empty[st], (use - 1) & 1, ctx, 10)) break;
                mbar_expect_tx(&k_full[st], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_3d(sK + st * Cfg::kTileBytes + pn * kPanel, &mapK, &k_full[st], kv_x + pn * 64, n * kTile, kv_z);
                if (use > 0 && !mbar_wait(&v_empty[st], (use - 1) & 1, ctx, 11)) break;
                mbar_expect_tx(&v_full[st], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_3d(sV + st * Cfg::kTileBytes + pn * kPanel, &mapV, &v_full[st], kv_x + pn * 64, n * kTile, kv_z);
            }
        }
    } else if (warp == kWarpMma) {
        // ======================= issuer: S(j), dP(j) per half-block, dQ += dS(j) K(j) =======================
        // The whole warp runs the loop (uniform control flow); `leader` marks the one lane that issues.
        const uint32_t leader = elect_one() ? 1u : 0u;
        const uint32_t idesc_sdp = make_idesc_bf16(128, kHalf, false, false);
        const uint32_t idesc_dq = make_idesc_bf16(128, D, false, true);
        const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
        bool ok = mbar_wait(qdo_full, 0, ctx, 20);
        // S(j) and dP(j): rows 64h.. of key / value block n = j/2 are the B operands (K-major panels, 64 rows = 8192 B down)
        auto issue_sdp = [&](int j) -> bool {
            const int n = j >> 1, h = j & 1, st = n % Cfg::kStages;
            if (h == 0 && !(mbar_wait(&k_full[st], (n / Cfg::kStages) & 1, ctx, 21) &&
                            mbar_wait(&v_full[st], (n / Cfg::kStages) & 1, ctx, 22)))
                return false;
            tc_fence_after_sync();
            const uint32_t kb = k_addr + st * Cfg::kTileBytes + h * (kHalf * 128);
            const uint32_t vb = v_addr + st * Cfg::kTileBytes + h * (kHalf * 128);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk >> 2) * kPanel + (kk & 3) * 32;
                umma_ss_pred(leader, tmem + Cfg::kColS + h * kHalf, make_sdesc_sw128(q_addr + off, 16, 1024),
                             make_sdesc_sw128(kb + off, 16, 1024), idesc_sdp, kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk >> 2) * kPanel + (kk & 3) * 32;
                umma_ss_pred(leader, tmem + Cfg::kColDP + h * kHalf, make_sdesc_sw128(do_addr + off, 16, 1024),
                             make_sdesc_sw128(vb + off, 16, 1024), idesc_sdp, kk > 0);
            }
            umma_commit_pred(leader, &sdp_full[h]);
            if (h == 1) umma_commit_pred(leader, &v_empty[st]);  // the value block is only read by dP
            return true;
        };
        if (ok) ok = issue_sdp(0);
        for (int j = 0; j < total && ok; ++j) {
            const int n = j >> 1, h = j & 1, st = n % Cfg::kStages;
            if (j + 1 < total) {
                // S(j+1) goes where dS(j-1) lives: that product must have completed
                if (j >= 1) ok = mbar_wait(&dq_done[h ^ 1], ((j - 1) >> 1) & 1, ctx, 23);
                if (ok) ok = issue_sdp(j + 1);
                if (!ok) break;
            }
            ok = mbar_wait(&ds_ready[h], n & 1, ctx, 24);
            if (!ok) break;
            tc_fence_after_sync();
            // dS(j) (64 keys as packed bf16, 16 columns at the head of each warpgroup's 32 S columns) times rows 64h.. of
            // the key block read MN-major
            const uint32_t b0 = k_addr + st * Cfg::kTileBytes + h * (kHalf / 16) * 2048;
#pragma unroll
            for (int kk = 0; kk < kHalf / 16; ++kk)
                umma_ts_pred(leader, tmem + Cfg::kColDQ, tmem + Cfg::kColS + h * kHalf + (kk >> 1) * 32 + (kk & 1) * 8,
                             make_sdesc_sw128(b0 + kk * 2048, kPanel, 1024), idesc_dq, (j > 0 || kk > 0));
            umma_commit_pred(leader, &dq_done[h]);
            if (h == 1) umma_commit_pred(leader, &k_empty[st]);
            if (j + 1 == total) umma_commit_pred(leader, dq_full);
        }
    } else {
        // ======================= elementwise warpgroups =======================
        const int w = warp >> 2;                      // which 32 key columns of every half-block
        const int r = (warp & 3) * 32 + lane;         // query row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const size_t row = (size_t)(b * p.Hq + hq) * p.S + q0 + r;  // in [B,Hq,S] order
        const bool row_ok = q0 + r < p.S;
        const float c = p.scale_log2;
        const float nlse2 = row_ok ? -p.lse[row] * kLog2e : 0.f;   // rows beyond S: finite garbage, never stored
        const float delta = row_ok ? p.delta[row] : 0.f;
        bool ok = true;
        for (int j = 0; j < total; ++j) {
            const int n = j >> 1, h = j & 1;
            ok = mbar_wait(&sdp_full[h], n & 1, ctx, 30);
            if (!ok) break;
            tc_fence_after_sync();
            // last visible key column of this row inside the 128-key block: the causal diagonal and / or the end of S
            const bool diag = p.causal && (n == qt);
            const int s_left = p.S - n * kTile;
            const bool masked = diag || s_left < kTile;
            const int lim = min(diag ? r : kTile - 1, s_left - 1);
            const int col0 = h * kHalf + w * 32;  // column of v[0] inside the block
            uint32_t vs[32], vd[32];
            tmem_ld32(tmem + lane_addr + Cfg::kColS + h * kHalf + w * 32, vs);
            tmem_ld32(tmem + lane_addr + Cfg::kColDP + h * kHalf + w * 32, vd);
            tmem_wait_ld();
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float e0 = ex2_approx(fmaf(__uint_as_float(vs[2 * i]), c, nlse2));
                float e1 = ex2_approx(fmaf(__uint_as_float(vs[2 * i + 1]), c, nlse2));
                if (masked) {
                    if (col0 + 2 * i > lim) e0 = 0.f;
                    if (col0 + 2 * i + 1 > lim) e1 = 0.f;
                }
                // P rounded to bf16 first (what the dV product of the main kernel uses), then one fp32 product, one rounding
                const uint32_t pb = pack_bf16x2(e0, e1);
                const float p_lo = __uint_as_float(pb << 16), p_hi = __uint_as_float(pb & 0xffff0000u);
                pk[i] = pack_bf16x2(p_lo * (__uint_as_float(vd[2 * i]) - delta), p_hi * (__uint_as_float(vd[2 * i + 1]) - delta));
            }
            // dS of these 32 keys = 16 packed columns, stored over the head of this warpgroup's OWN S columns (which it
            // has just read), so the two warpgroups never touch each other's columns: K step kk of the dQ product
            // (16 keys) finds its A operand at column 32 * (kk / 2) + 8 * (kk % 2) of the buffer
            tmem_st16(tmem + lane_addr + Cfg::kColS + h * kHalf + w * 32, pk);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&ds_ready[h]);
        }
        // ---- epilogue: dQ = bf16(scale * sum), half of the columns per warpgroup
        if (ok) ok = mbar_wait(dq_full, 0, ctx, 31);
        if (ok) {
            tc_fence_after_sync();
            constexpr int kColsPerWg = D / 2;
            __nv_bfloat16* out = p.bshd ? p.dQ + ((size_t)(b * p.S + q0 + r) * p.Hq + hq) * D : p.dQ + row * p.d_real;
#pragma unroll
            for (int ch = 0; ch < kColsPerWg / 32; ++ch) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_addr + Cfg::kColDQ + w * kColsPerWg + ch * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 o;
                    o.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * p.scale, __uint_as_float(v[8 * i + 1]) * p.scale);
                    o.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * p.scale, __uint_as_float(v[8 * i + 3]) * p.scale);
                    o.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * p.scale, __uint_as_float(v[8 * i + 5]) * p.scale);
                    o.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * p.scale, __uint_as_float(v[8 * i + 7]) * p.scale);
                    const int col = w * kColsPerWg + ch * 32 + i * 8;
                    if (row_ok && col < p.d_real) *reinterpret_cast<uint4*>(out + col) = o;
                }
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kWarpMma) {
        if (*abort_flag != 0) abort_grace_period();  // in-flight copies and MMAs land before TMEM is released
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

template <int D>
int launch_dq_t(const void* Q, const void* K, const void* V, const void* dO, const float* lse, const float* delta,
                void* dQ, const Shape& s, unsigned int* status, cudaStream_t stream) {
    using Cfg = DqCfg<D>;
    CUtensorMap mq, mdo, mk, mv;
    const uint64_t S = s.S, qc = s.bshd ? (uint64_t)s.Hq * D : s.D, kc = s.bshd ? (uint64_t)s.Hkv * D : s.D;
    const uint64_t nq = s.bshd ? s.B : (uint64_t)s.B * s.Hq, nkv = s.bshd ? s.B : (uint64_t)s.B * s.Hkv;
    int rc = make_tile3_tmap(&mq, Q, qc, S, nq, S * qc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mdo, dO, qc, S, nq, S * qc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mk, K, kc, S, nkv, S * kc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mv, V, kc, S, nkv, S * kc, kTile);
    if (rc) return rc;
    GQA_CUDA_TRY(cudaFuncSetAttribute(gqa_bwd_dq_sm100_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg::kSmemTotal));
    DqParams p;
    p.dQ = static_cast<__nv_bfloat16*>(dQ);
    p.lse = lse;
    p.delta = delta;
    p.status = status;
    p.Hq = s.Hq;
    p.Hkv = s.Hkv;
    p.S = s.S;
    p.causal = s.causal;
    p.bshd = s.bshd;
    p.d_real = s.D;
    p.n_qtiles = (s.S + kTile - 1) / kTile;
    p.scale = s.scale;
    p.scale_log2 = s.scale * kLog2e;
    dim3 grid(p.n_qtiles, s.Hq, s.B);
    gqa_bwd_dq_sm100_kernel<D><<<grid, kThreads, Cfg::kSmemTotal, stream>>>(mq, mdo, mk, mv, p);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

}  // namespace

int launch_bwd_dq_sm100(const void* Q, const void* K, const void* V, const void* dO, const float* lse,
                        const float* delta, void* dQ, const Shape& s, unsigned int* status, cudaStream_t stream) {
    if (s.Dp() == 64) return launch_dq_t<64>(Q, K, V, dO, lse, delta, dQ, s, status, stream);
    return launch_dq_t<128>(Q, K, V, dO, lse, delta, dQ, s, status, stream);
}

}  // namespace gqa
