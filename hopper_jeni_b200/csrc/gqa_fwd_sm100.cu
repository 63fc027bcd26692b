// GQA forward for sm_100a: O = softmax(scale * Q K^T [+ causal]) V, LSE.
//
// One CTA owns two 128-row query tiles of one (batch, query head) and streams the
// KV head's 128-row key/value blocks through a TMA ring.  Roles:
//   warps 0-3  softmax warpgroup for query tile 0 (thread = query row = TMEM lane)
//   warps 4-7  softmax warpgroup for query tile 1
//   warp  8    TMA producer (Q once, K and V rings)
//   warp  9    UMMA issuer for S = Q K^T (both tiles)
//   warps 10,11 UMMA issuers for O += P V of tile 0 / tile 1 (P read from TMEM)
// One issuing warp sustains a product with A in TMEM only every ~78 cycles, and the three GEMM
// streams wait on different producers, hence three issuers (warp-uniform loops, one elected lane).  The two query tiles ping-pong: while one warpgroup runs its softmax (the exp unit is
// the bound at D = 64), the tensor core works on the other tile.  S lives in TMEM (128 fp32 columns per tile), P
// overwrites the first 64 columns of S as packed bf16, O accumulates in TMEM.
// The running maximum is only refreshed when it grows by more than 2^8, so O is
// rescaled rarely; the final division by the row sum uses the same maximum.
//
// Replaces gqa62::gqa_v62 / launch_gqa_v62 (src/attention/GQA_fwd_ref.cu:336-651):
// same inputs/outputs, LSE = natural-log of the scaled-logit sum (:611-614).
#include "gqa_common.cuh"
#include "gqa_kernels.cuh"
#include "sm100_ptx.cuh"

namespace gqa {
namespace {

using namespace sm100;

// Optional timeline tracing (development builds only): block 0 stamps clock64 at a few points per key block.
#ifdef GQA_FWD_TRACE
__device__ long long g_fwd_trace[3][64][4];
#define GQA_FTRACE(role, it, slot)                                                                 \
    do {                                                                                           \
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (it) < 64 && (threadIdx.x & 31) == 0) \
            g_fwd_trace[role][it][slot] = clock64();                                               \
    } while (0)
#else
#define GQA_FTRACE(role, it, slot) \
    do {                           \
    } while (0)
#endif

constexpr int kTile = 128;             // query rows per tile and key rows per block
constexpr int kPanel = kTile * 128;    // bytes of one 64-column panel of a 128-row tile
constexpr int kFwdThreads = 384;
constexpr int kWarpTma = 8, kWarpQK = 9, kWarpPV0 = 10;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units

template <int D>
struct FwdCfg {
    static constexpr int kPanels = D / 64;
    static constexpr int kTileBytes = kPanels * kPanel;  // one 128 x D bf16 tile
    static constexpr int kStages = (D == 64) ? 4 : 2;
    static constexpr int kSmemQ = 2 * kTileBytes;
    static constexpr int kSmemKV = 2 * kStages * kTileBytes;
    static constexpr int kBarBytes = 512;
    static constexpr int kSmemTotal = kSmemQ + kSmemKV + kBarBytes;  // the dynamic window must start 1024-byte aligned (checked)
    static constexpr uint32_t kTmemCols = 512;
    static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 256 + D;
    static_assert(256 + 2 * D <= 512, "TMEM budget");
    static_assert(kSmemTotal <= 227 * 1024, "shared memory budget");
    static_assert(kSmemTotal > 114 * 1024, "one CTA per SM is assumed by the 512-column TMEM allocation");
};

struct FwdParams {
    __nv_bfloat16* O;
    float* LSE;
    unsigned int* status;
    int Hq, Hkv, S, causal, n_pairs;
    float scale_log2;  // scale * log2(e)
};

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
gqa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                     const __grid_constant__ CUtensorMap mapV, const FwdParams p) {
    using Cfg = FwdCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // swizzled panels need 1024-byte alignment; report instead of computing garbage
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, 0x80000000u | (99u << 20));
        return;
    }
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + Cfg::kSmemQ;
    uint8_t* sV = sK + Cfg::kStages * Cfg::kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + Cfg::kStages * Cfg::kTileBytes);
    uint64_t* q_full = bars;                       // [2]
    uint64_t* s_full = bars + 2;                   // [2]
    uint64_t* p_full = bars + 4;                   // [2]
    uint64_t* o_full = bars + 6;                   // [2]
    uint64_t* pv_done = bars + 8;                  // [2] PV issuer t -> QK issuer: P_t consumed, S_t may be rewritten
    uint64_t* turn = bars + 10;                    // [2] softmax warpgroup t finished the exp phase of a block
    uint64_t* k_full = bars + 12;                  // [kStages]
    uint64_t* k_empty = k_full + Cfg::kStages;     // [kStages]
    uint64_t* v_full = k_empty + Cfg::kStages;     // [kStages]
    uint64_t* v_empty = v_full + Cfg::kStages;     // [kStages]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_empty + Cfg::kStages);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    AbortCtx ctx{abort_flag, p.status};

    // ---- work decode ------------------------------------------------------------
    const int pair = p.causal ? (p.n_pairs - 1 - (int)blockIdx.x) : (int)blockIdx.x;  // heavy causal tiles first
    const int hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int q0 = pair * 2 * kTile;
    const int n_tiles = (q0 + kTile < p.S) ? 2 : 1;
    const int n_blocks_all = p.S / kTile;
    int n_blk[2];
    n_blk[0] = p.causal ? (q0 / kTile + 1) : n_blocks_all;
    n_blk[1] = (n_tiles == 2) ? (p.causal ? (q0 / kTile + 2) : n_blocks_all) : 0;
    const int n_max = n_blk[1] > n_blk[0] ? n_blk[1] : n_blk[0];
    const int q_row0 = (b * p.Hq + hq) * p.S + q0;   // row in the flattened [B*Hq*S, D] view
    const int kv_row0 = (b * p.Hkv + hkv) * p.S;

    // ---- setup ------------------------------------------------------------------
    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&o_full[i], 1);
            mbar_init(&pv_done[i], 1);
            mbar_init(&turn[i], 128);
        }
        for (int i = 0; i < Cfg::kStages; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], n_tiles);  // one commit per PV issuer that uses the block
        }
        fence_mbar_init();
    }
    if (warp == kWarpQK) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == kWarpTma) {
        // ======================= TMA producer =======================
        if (elect_one()) {
            tma_prefetch_desc(&mapQ);
            tma_prefetch_desc(&mapK);
            tma_prefetch_desc(&mapV);
            for (int t = 0; t < n_tiles; ++t) {
                mbar_expect_tx(&q_full[t], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_2d(sQ + t * Cfg::kTileBytes + pn * kPanel, &mapQ, &q_full[t], pn * 64, q_row0 + t * kTile);
            }
            for (int n = 0; n < n_max; ++n) {
                const int st = n % Cfg::kStages;
                const uint32_t use = n / Cfg::kStages;
                if (use > 0 && !mbar_wait(&k_empty[st], (use - 1) & 1, ctx, 10)) break;
                mbar_expect_tx(&k_full[st], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_2d(sK + st * Cfg::kTileBytes + pn * kPanel, &mapK, &k_full[st], pn * 64, kv_row0 + n * kTile);
                if (use > 0 && !mbar_wait(&v_empty[st], (use - 1) & 1, ctx, 11)) break;
                mbar_expect_tx(&v_full[st], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_2d(sV + st * Cfg::kTileBytes + pn * kPanel, &mapV, &v_full[st], pn * 64, kv_row0 + n * kTile);
            }
        }
    } else if (warp == kWarpQK) {
        // ======================= issuer: S_t(n) = Q_t K(n)^T for both tiles =======================
        // The whole warp runs the loop (uniform control flow); `leader` marks the one lane that issues.
        const uint32_t leader = elect_one() ? 1u : 0u;
        const uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
        const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK);
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; ++t) ok = mbar_wait(&q_full[t], 0, ctx, 20);
        for (int n = 0; n < n_max && ok; ++n) {
            const int st = n % Cfg::kStages;
            ok = mbar_wait(&k_full[st], (n / Cfg::kStages) & 1, ctx, 21);
            for (int t = 0; t < n_tiles && ok; ++t) {
                if (n >= n_blk[t]) continue;
                if (n > 0) ok = mbar_wait(&pv_done[t], (n - 1) & 1, ctx, 22);  // P_t(n-1) lives in the S_t columns
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t a0 = q_addr + t * Cfg::kTileBytes, b0 = k_addr + st * Cfg::kTileBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kPanel + (kk & 3) * 32;
                    umma_ss_pred(leader, tmem + (t ? Cfg::kColS1 : Cfg::kColS0), make_sdesc_sw128(a0 + off, 16, 1024),
                                 make_sdesc_sw128(b0 + off, 16, 1024), idesc_qk, kk > 0);
                }
                umma_commit_pred(leader, &s_full[t]);
                if (t == 0) GQA_FTRACE(1, n, 0);
            }
            if (ok) umma_commit_pred(leader, &k_empty[st]);
        }
    } else if (warp >= kWarpPV0) {
        // ======================= issuers: O_t += P_t(n) V(n)  (A = P_t from TMEM, B = V read MN-major) =======================
        const int t = warp - kWarpPV0;
        if (t < n_tiles) {
            const uint32_t leader = elect_one() ? 1u : 0u;
            const uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
            const uint32_t v_addr = smem_u32(sV);
            const uint32_t colS = t ? Cfg::kColS1 : Cfg::kColS0, colO = t ? Cfg::kColO1 : Cfg::kColO0;
            bool ok = true;
            for (int n = 0; n < n_blk[t] && ok; ++n) {
                const int st = n % Cfg::kStages;
                ok = mbar_wait(&v_full[st], (n / Cfg::kStages) & 1, ctx, 23) && mbar_wait(&p_full[t], n & 1, ctx, 24);
                if (!ok) break;
                tc_fence_after_sync();
                if (t == 0) GQA_FTRACE(1, n, 1);
                const uint32_t b0 = v_addr + st * Cfg::kTileBytes;
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)
                    umma_ts_pred(leader, tmem + colO, tmem + colS + kk * 8, make_sdesc_sw128(b0 + kk * 2048, kPanel, 1024),
                                 idesc_pv, (n > 0 || kk > 0));
                umma_commit_pred(leader, &pv_done[t]);
                umma_commit_pred(leader, &v_empty[st]);
                if (n + 1 == n_blk[t]) umma_commit_pred(leader, &o_full[t]);
                if (t == 0) GQA_FTRACE(1, n, 2);
            }
        }
    } else {
        // ======================= softmax warpgroups =======================
        const int t = warp >> 2;                      // query tile owned by this warpgroup
        const int r = (warp & 3) * 32 + lane;         // row inside the tile == TMEM lane
        if (t < n_tiles) {
            const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
            const uint32_t tS = tmem + lane_addr + (t == 0 ? Cfg::kColS0 : Cfg::kColS1);
            const uint32_t tO = tmem + lane_addr + (t == 0 ? Cfg::kColO0 : Cfg::kColO1);
            const float c = p.scale_log2;
            const int n_mine = n_blk[t];
            const int diag_block = (q0 + t * kTile) / kTile;  // only this block needs the causal mask
            float m_run = -INFINITY;  // running maximum of the raw logits that P is measured against
            float l_run = 0.f;
            bool ok = true;
            for (int n = 0; n < n_mine; ++n) {
                ok = mbar_wait(&s_full[t], n & 1, ctx, 30);
                if (!ok) break;
                tc_fence_after_sync();
                if (warp == 0) GQA_FTRACE(0, n, 0);
                if (warp == 4) GQA_FTRACE(2, n, 0);
                const bool masked = p.causal && (n == diag_block);
                // the whole 128-column row of S into registers (one TMEM round trip), then the row maximum
                // with four independent partial maxima (a single chain of 128 dependent max ops is slow)
                uint32_t v[128];
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) tmem_ld32p(tS + ch * 32, v + ch * 32);
                tmem_wait_ld();
                float mx;
                {
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < 128; ++i)
                            m4[i & 3] = (i > r) ? m4[i & 3] : fmaxf(m4[i & 3], __uint_as_float(v[i]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 128; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v[i]));
                    }
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                }
                if (warp == 0) GQA_FTRACE(0, n, 1);
                const float m_new = fmaxf(m_run, mx);
                const bool grow = (m_new - m_run) * c > kRescaleThreshold;  // true on the first block (m_run = -inf)
                if (__any_sync(0xffffffffu, grow)) {
                    const float m_next = grow ? m_new : m_run;
                    const float alpha = ex2_approx((m_run - m_next) * c);
                    l_run *= alpha;
                    m_run = m_next;
                    if (n > 0) {
#pragma unroll 1
                        for (int ch = 0; ch < D / 32; ++ch) {
                            uint32_t v[32];
                            tmem_ld32(tO + ch * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                            tmem_st32(tO + ch * 32, v);
                        }
                    }
                }
                // The exp unit is the shared bottleneck, so the two tiles are kept out of phase: one tile's exps
                // then overlap the other tile's tensor-core round trip instead of both idling together.
                // D = 128 (tensor and exp work balanced): strict turns 0,1,0,1,... in the exp phase.
                // D = 64 (exp-bound): only the first exp phase of tile 1 is delayed until tile 0 finished its own;
                // measured, strict turns cost 5 % there and gain 25 % at D = 128.
                if constexpr (D == 128) {
                    if (t == 1) {
                        if (n < n_blk[0]) ok = mbar_wait(&turn[0], n & 1, ctx, 35);
                    } else if (n > 0 && n - 1 < n_blk[1]) {
                        ok = mbar_wait(&turn[1], (n - 1) & 1, ctx, 36);
                    }
                } else {
                    if (t == 1 && n == 0 && n_blk[0] > 0) ok = mbar_wait(&turn[0], 0, ctx, 35);
                }
                if (!ok) break;
                // P = exp2(c*s - c*m), row sum (four partial sums), packed bf16 back into the first 64 S columns
                const float mc = m_run * c;
                float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float e0 = ex2_approx(fmaf(__uint_as_float(v[ch * 32 + 2 * i]), c, -mc));
                        float e1 = ex2_approx(fmaf(__uint_as_float(v[ch * 32 + 2 * i + 1]), c, -mc));
                        if (masked) {
                            if (ch * 32 + 2 * i > r) e0 = 0.f;
                            if (ch * 32 + 2 * i + 1 > r) e1 = 0.f;
                        }
                        l4[i & 3] += e0 + e1;
                        pk[i] = pack_bf16x2(e0, e1);
                    }
                    tmem_st16(tS + ch * 16, pk);
                }
                l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
                if (D == 128 || (t == 0 && n == 0)) mbar_arrive(&turn[t]);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&p_full[t]);
                if (warp == 0) GQA_FTRACE(0, n, 2);
                if (warp == 4) GQA_FTRACE(2, n, 2);
            }
            // epilogue: O / l -> bf16, LSE
            if (ok) ok = mbar_wait(&o_full[t], 0, ctx, 31);
            if (ok) {
                tc_fence_after_sync();
                const float inv_l = 1.0f / l_run;
                const size_t grow_ = (size_t)q_row0 + t * kTile + r;
                __nv_bfloat16* orow = p.O + grow_ * D;
#pragma unroll 1
                for (int ch = 0; ch < D / 32; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(tO + ch * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * inv_l, __uint_as_float(v[8 * i + 1]) * inv_l);
                        o.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * inv_l, __uint_as_float(v[8 * i + 3]) * inv_l);
                        o.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * inv_l, __uint_as_float(v[8 * i + 5]) * inv_l);
                        o.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * inv_l, __uint_as_float(v[8 * i + 7]) * inv_l);
                        *reinterpret_cast<uint4*>(orow + ch * 32 + i * 8) = o;
                    }
                }
                if (p.LSE) p.LSE[grow_] = (m_run * c + log2f(l_run)) * kLn2;
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kWarpQK) {
        if (*abort_flag != 0) __nanosleep(20000);  // let in-flight copies and MMAs drain before TMEM is released
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

template <int D>
int launch_fwd_t(const void* Q, const void* K, const void* V, void* O, float* LSE, const Shape& s, unsigned int* status,
                 cudaStream_t stream) {
    using Cfg = FwdCfg<D>;
    CUtensorMap mq, mk, mv;
    int rc = make_panel_tmap(&mq, Q, s.q_rows(), D, kTile);
    if (rc) return rc;
    rc = make_panel_tmap(&mk, K, s.kv_rows(), D, kTile);
    if (rc) return rc;
    rc = make_panel_tmap(&mv, V, s.kv_rows(), D, kTile);
    if (rc) return rc;
    GQA_CUDA_TRY(cudaFuncSetAttribute(gqa_fwd_sm100_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg::kSmemTotal));
    FwdParams p;
    p.O = static_cast<__nv_bfloat16*>(O);
    p.LSE = LSE;
    p.status = status;
    p.Hq = s.Hq;
    p.Hkv = s.Hkv;
    p.S = s.S;
    p.causal = s.causal;
    p.n_pairs = (s.S + 2 * kTile - 1) / (2 * kTile);
    p.scale_log2 = s.scale * kLog2e;
    dim3 grid(p.n_pairs, s.Hq, s.B);
    gqa_fwd_sm100_kernel<D><<<grid, kFwdThreads, Cfg::kSmemTotal, stream>>>(mq, mk, mv, p);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

}  // namespace

#ifdef GQA_FWD_TRACE
extern "C" int gqa_debug_copy_fwd_trace(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, g_fwd_trace, sizeof(g_fwd_trace));
}
#endif

int launch_fwd_sm100(const void* Q, const void* K, const void* V, void* O, float* LSE, const Shape& s,
                     unsigned int* status, cudaStream_t stream) {
    GQA_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(unsigned int), stream));
    if (s.D == 64) return launch_fwd_t<64>(Q, K, V, O, LSE, s, status, stream);
    return launch_fwd_t<128>(Q, K, V, O, LSE, s, status, stream);
}

}  // namespace gqa
