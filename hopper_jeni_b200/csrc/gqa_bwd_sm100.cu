// GQA backward, stage 2 of 3, for sm_100a: the KV-tile-parallel main kernel.
//
// One CTA owns one 128-row key/value tile of one (batch, KV head) and loops over
// all G query heads of the group and over the 128-row query tiles that see the
// tile (all of them, or the ones at and below the diagonal when causal).  dK and
// dV therefore accumulate in tensor memory across the whole GQA group and are
// written exactly once: no atomics, bit-reproducible.  dQ tiles are reduced into
// an fp32 accumulator with vector reductions (order-dependent in the last bits).
//
// Everything is computed in the transposed orientation so that a TMEM lane is a
// key row:  S^T = K Q^T,  dP^T = V dO^T  (both operands K-major from TMA panels),
//   P^T  = exp2(S^T * scale*log2e - LSE*log2e)   -> bf16 into TMEM (A operand of dV)
//   dS^T = P^T * (dP^T - Delta)                   -> bf16 into swizzled shared memory
//   dV  += P^T dO      (A from TMEM,  B = dO panel read MN-major)
//   dK  += dS^T Q      (A = dS^T K-major, B = Q panel read MN-major)
//   dQ   = dS K        (A = dS^T read MN-major, B = K panel read MN-major)
// Roles: warps 0-3 drain dQ, warps 4-7 / 8-11 are the two elementwise warpgroups
// (each owns 64 query columns of the tile pair), warp 12 is the TMA producer and
// warp 13 issues every UMMA.
//
// Replaces gqa_bwd_vj1d (src/attention/GQA_bwd_baseline.cu:405-547) in the
// G-loop-inside-the-CTA form of gqa_bwd_vz2_wgmma (src/attention/GQA_bwd.cu:15207-15342);
// roundings follow the reference: P and dS are rounded to bf16 before the GEMMs that
// consume them, dK and dQ are scaled in fp32 (GQA_bwd_baseline.cu:243-255, :320-326, :530-534).
#include "gqa_common.cuh"
#include "gqa_kernels.cuh"
#include "sm100_ptx.cuh"

namespace gqa {
namespace {

using namespace sm100;

// Optional timeline tracing (development builds only): block 0 stamps clock64 at a few points per iteration.
#ifdef GQA_BWD_TRACE
__device__ long long g_bwd_trace[3][64][4];
#define GQA_TRACE(role, it, slot)                                                              \
    do {                                                                                       \
        if (blockIdx.x == 0 && (it) < 64 && (threadIdx.x & 31) == 0 && (((role) != 0) || warp == 4)) \
            g_bwd_trace[role][it][slot] = clock64();                                           \
    } while (0)
#else
#define GQA_TRACE(role, it, slot) \
    do {                          \
    } while (0)
#endif

constexpr int kTile = 128;
constexpr int kPanel = kTile * 128;  // bytes of one 64-column panel of a 128-row tile
constexpr int kBwdThreads = 448;

template <int D>
struct BwdCfg {
    static constexpr int kPanels = D / 64;
    static constexpr int kTileBytes = kPanels * kPanel;
    static constexpr int kQStages = 2;
    static constexpr int kDOStages = (D == 64) ? 2 : 1;
    static constexpr int kVecBytes = kTile * 4;  // 128 floats of LSE*log2e or Delta
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kOffK + kTileBytes;
    static constexpr int kOffQ = kOffV + kTileBytes;
    static constexpr int kOffDO = kOffQ + kQStages * kTileBytes;
    static constexpr int kOffDS = kOffDO + kDOStages * kTileBytes;
    static constexpr int kOffLse = kOffDS + 2 * kPanel;
    static constexpr int kOffDelta = kOffLse + kQStages * kVecBytes;
    static constexpr int kOffBars = kOffDelta + kQStages * kVecBytes;
    static constexpr int kSmemTotal = 1024 + kOffBars + 256;
    static constexpr uint32_t kTmemCols = 512;
    static constexpr uint32_t kColS = 0, kColDP = 128;
    static constexpr uint32_t kColDQ = (D == 64) ? 256 : 128;  // D = 128: dQ reuses the dP columns
    static constexpr uint32_t kColDV = (D == 64) ? 320 : 256;
    static constexpr uint32_t kColDK = kColDV + D;
    static constexpr bool kDqAliasesDp = (D != 64);
    static_assert(kColDK + D <= 512, "TMEM budget");
    static_assert(kSmemTotal <= 227 * 1024, "shared memory budget");
    static_assert(kSmemTotal > 114 * 1024, "one CTA per SM is assumed by the 512-column TMEM allocation");
};

struct BwdParams {
    const float* lse2;   // [B*Hq*S] LSE * log2(e)
    const float* delta;  // [B*Hq*S]
    float* dq_accum;     // [B*Hq*S, D] fp32, zeroed by the preprocess stage
    __nv_bfloat16* dK;
    __nv_bfloat16* dV;
    unsigned int* status;
    int Hq, Hkv, S, causal, n_tiles, G;
    float scale, scale_log2;
};

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
gqa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                     const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                     const BwdParams p) {
    using Cfg = BwdCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem + Cfg::kOffK;
    uint8_t* sV = smem + Cfg::kOffV;
    uint8_t* sQ = smem + Cfg::kOffQ;
    uint8_t* sDO = smem + Cfg::kOffDO;
    uint8_t* sDS = smem + Cfg::kOffDS;
    float* sLse = reinterpret_cast<float*>(smem + Cfg::kOffLse);
    float* sDelta = reinterpret_cast<float*>(smem + Cfg::kOffDelta);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
    uint64_t* kv_full = bars + 0;
    uint64_t* s_full = bars + 1;
    uint64_t* dp_full = bars + 2;
    uint64_t* p_ready = bars + 3;
    uint64_t* ds_ready = bars + 4;
    uint64_t* ds_free = bars + 5;
    uint64_t* dq_full = bars + 6;
    uint64_t* dq_empty = bars + 7;
    uint64_t* acc_full = bars + 8;
    uint64_t* q_full = bars + 9;                     // [kQStages]
    uint64_t* q_empty = q_full + Cfg::kQStages;      // [kQStages]
    uint64_t* do_full = q_empty + Cfg::kQStages;     // [kDOStages]
    uint64_t* do_empty = do_full + Cfg::kDOStages;   // [kDOStages]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(do_empty + Cfg::kDOStages);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    AbortCtx ctx{abort_flag, p.status};

    // ---- work decode: KV tile is the slow index so the longest causal items start first ----
    const int groups = gridDim.x / p.n_tiles;  // B * Hkv
    const int kt = blockIdx.x / groups;
    const int grp = blockIdx.x % groups;
    const int b = grp / p.Hkv, hkv = grp % p.Hkv;
    const int qt0 = p.causal ? kt : 0;
    const int n_qt = p.n_tiles - qt0;
    const int n_iter = p.G * n_qt;
    const int kv_row0 = (b * p.Hkv + hkv) * p.S + kt * kTile;
    const int q_head0 = b * p.Hq + hkv * p.G;  // first query head of the group
    auto q_row_of = [&](int it) { return (q_head0 + it / n_qt) * p.S + (qt0 + it % n_qt) * kTile; };

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(kv_full, 1);
        mbar_init(s_full, 1);
        mbar_init(dp_full, 1);
        mbar_init(p_ready, 256);
        mbar_init(ds_ready, 256);
        mbar_init(ds_free, 1);
        mbar_init(dq_full, 1);
        mbar_init(dq_empty, 128);
        mbar_init(acc_full, 1);
        for (int i = 0; i < Cfg::kQStages; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&q_empty[i], 1);
        }
        for (int i = 0; i < Cfg::kDOStages; ++i) {
            mbar_init(&do_full[i], 1);
            mbar_init(&do_empty[i], 1);
        }
        fence_mbar_init();
    }
    if (warp == 13) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 12) {
        // ======================= TMA producer =======================
        if (elect_one()) {
            tma_prefetch_desc(&mapQ);
            tma_prefetch_desc(&mapK);
            tma_prefetch_desc(&mapV);
            tma_prefetch_desc(&mapDO);
            mbar_expect_tx(kv_full, 2 * Cfg::kTileBytes);
            for (int pn = 0; pn < Cfg::kPanels; ++pn) {
                tma_load_2d(sK + pn * kPanel, &mapK, kv_full, pn * 64, kv_row0);
                tma_load_2d(sV + pn * kPanel, &mapV, kv_full, pn * 64, kv_row0);
            }
            for (int it = 0; it < n_iter; ++it) {
                const int row = q_row_of(it);
                {
                    const int st = it % Cfg::kQStages;
                    const uint32_t use = it / Cfg::kQStages;
                    if (use > 0 && !mbar_wait(&q_empty[st], (use - 1) & 1, ctx, 10)) break;
                    // LSE and Delta ride with Q: their buffers are released with the Q stage, i.e. only
                    // after the elementwise warpgroups have finished the iteration that reads them
                    mbar_expect_tx(&q_full[st], Cfg::kTileBytes + 2 * Cfg::kVecBytes);
                    for (int pn = 0; pn < Cfg::kPanels; ++pn)
                        tma_load_2d(sQ + st * Cfg::kTileBytes + pn * kPanel, &mapQ, &q_full[st], pn * 64, row);
                    bulk_load_1d(sLse + st * kTile, p.lse2 + row, Cfg::kVecBytes, &q_full[st]);
                    bulk_load_1d(sDelta + st * kTile, p.delta + row, Cfg::kVecBytes, &q_full[st]);
                }
                {
                    const int st = it % Cfg::kDOStages;
                    const uint32_t use = it / Cfg::kDOStages;
                    if (use > 0 && !mbar_wait(&do_empty[st], (use - 1) & 1, ctx, 11)) break;
                    mbar_expect_tx(&do_full[st], Cfg::kTileBytes);
                    for (int pn = 0; pn < Cfg::kPanels; ++pn)
                        tma_load_2d(sDO + st * Cfg::kTileBytes + pn * kPanel, &mapDO, &do_full[st], pn * 64, row);
                }
            }
        }
    } else if (warp == 13) {
        // ======================= UMMA issuer =======================
        if (elect_one()) {
            const uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);  // S^T, dP^T
            const uint32_t idesc_dv = make_idesc_bf16(128, D, false, true);    // A K-major (TMEM or dS), B MN-major
            const uint32_t idesc_dq = make_idesc_bf16(128, D, true, true);     // A = dS^T read MN-major
            const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ);
            const uint32_t do_addr = smem_u32(sDO), ds_addr = smem_u32(sDS);
            bool ok = true;

            // S^T / dP^T: A = K or V tile (rows = keys), B = Q or dO tile (rows = queries), contraction over D
            auto issue_kmajor_pair = [&](uint32_t col, uint32_t a0, uint32_t b0) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kPanel + (kk & 3) * 32;
                    umma_ss(tmem + col, make_sdesc_sw128(a0 + off, 16, 1024), make_sdesc_sw128(b0 + off, 16, 1024),
                            idesc_s, kk > 0);
                }
            };

            ok = mbar_wait(kv_full, 0, ctx, 20) && mbar_wait(&q_full[0], 0, ctx, 21);
            if (ok) {
                tc_fence_after_sync();
                issue_kmajor_pair(Cfg::kColS, k_addr, q_addr);
                umma_commit(s_full);
                ok = mbar_wait(&do_full[0], 0, ctx, 22);
            }
            if (ok) {
                tc_fence_after_sync();
                issue_kmajor_pair(Cfg::kColDP, v_addr, do_addr);
                umma_commit(dp_full);
            }

            for (int it = 0; it < n_iter && ok; ++it) {
                const int qs = it % Cfg::kQStages, dos = it % Cfg::kDOStages;
                const uint32_t q_cur = q_addr + qs * Cfg::kTileBytes, do_cur = do_addr + dos * Cfg::kTileBytes;
                const bool more = it + 1 < n_iter;
                // ---- dV += P^T dO(it): A = P^T in TMEM; query rows 0-63 sit in S columns [0,32), 64-127 in [64,96)
                ok = mbar_wait(p_ready, it & 1, ctx, 23);
                if (!ok) break;
                GQA_TRACE(1, it, 0);
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t a_col = Cfg::kColS + (kk >> 2) * 64 + (kk & 3) * 8;
                    umma_ts(tmem + Cfg::kColDV, tmem + a_col, make_sdesc_sw128(do_cur + kk * 2048, kPanel, 1024),
                            idesc_dv, (it > 0 || kk > 0));
                }
                umma_commit(&do_empty[dos]);
                // ---- S^T(it+1)
                if (more) {
                    const int qn = (it + 1) % Cfg::kQStages;
                    ok = mbar_wait(&q_full[qn], ((it + 1) / Cfg::kQStages) & 1, ctx, 24);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_kmajor_pair(Cfg::kColS, k_addr, q_addr + qn * Cfg::kTileBytes);
                    umma_commit(s_full);
                }
                // ---- dK += dS^T Q(it)
                ok = mbar_wait(ds_ready, it & 1, ctx, 25);
                if (!ok) break;
                GQA_TRACE(1, it, 1);
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t a_off = (kk >> 2) * kPanel + (kk & 3) * 32;
                    umma_ss(tmem + Cfg::kColDK, make_sdesc_sw128(ds_addr + a_off, 16, 1024),
                            make_sdesc_sw128(q_cur + kk * 2048, kPanel, 1024), idesc_dv, (it > 0 || kk > 0));
                }
                umma_commit(&q_empty[qs]);
                // ---- dQ(it) = dS K
                if (it > 0) {
                    ok = mbar_wait(dq_empty, (it - 1) & 1, ctx, 26);
                    if (!ok) break;
                    tc_fence_after_sync();
                    GQA_TRACE(1, it, 2);
                }
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    umma_ss(tmem + Cfg::kColDQ, make_sdesc_sw128(ds_addr + kk * 2048, kPanel, 1024),
                            make_sdesc_sw128(k_addr + kk * 2048, kPanel, 1024), idesc_dq, kk > 0);
                }
                umma_commit(dq_full);
                umma_commit(ds_free);
                // ---- dP^T(it+1)
                if (more) {
                    const int dn = (it + 1) % Cfg::kDOStages;
                    ok = mbar_wait(&do_full[dn], ((it + 1) / Cfg::kDOStages) & 1, ctx, 27);
                    if (ok && Cfg::kDqAliasesDp) ok = mbar_wait(dq_empty, it & 1, ctx, 28);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_kmajor_pair(Cfg::kColDP, v_addr, do_addr + dn * Cfg::kTileBytes);
                    umma_commit(dp_full);
                    GQA_TRACE(1, it, 3);
                }
            }
            if (ok) umma_commit(acc_full);
        }
    } else if (warp < 4) {
        // ======================= dQ drain warpgroup =======================
        const int r = warp * 32 + lane;  // query row inside the tile == TMEM lane
        const uint32_t tDQ = tmem + ((uint32_t)(warp * 32) << 16) + Cfg::kColDQ;
        for (int it = 0; it < n_iter; ++it) {
            if (!mbar_wait(dq_full, it & 1, ctx, 40)) break;
            tc_fence_after_sync();
            GQA_TRACE(2, it, 0);
            float* dst = p.dq_accum + ((size_t)q_row_of(it) + r) * D;
            if constexpr (D == 64) {
                uint32_t v0[32], v1[32];
                tmem_ld32(tDQ, v0);
                tmem_ld32(tDQ + 32, v1);
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(dq_empty);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * i), "r"(v0[4 * i]),
                                 "r"(v0[4 * i + 1]), "r"(v0[4 * i + 2]), "r"(v0[4 * i + 3])
                                 : "memory");
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 32 + 4 * i),
                                 "r"(v1[4 * i]), "r"(v1[4 * i + 1]), "r"(v1[4 * i + 2]), "r"(v1[4 * i + 3])
                                 : "memory");
            } else {
#pragma unroll 1
                for (int ch = 0; ch < D / 32; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(tDQ + ch * 32, v);
                    tmem_wait_ld();
                    if (ch == D / 32 - 1) {
                        tc_fence_before_sync();
                        mbar_arrive(dq_empty);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + ch * 32 + 4 * i),
                                     "r"(v[4 * i]), "r"(v[4 * i + 1]), "r"(v[4 * i + 2]), "r"(v[4 * i + 3])
                                     : "memory");
                }
            }
        }
    } else {
        // ======================= elementwise warpgroups (P^T and dS^T) =======================
        const int h = (warp - 4) >> 2;            // which 64 query columns of the tile pair
        const int j = (warp & 3) * 32 + lane;     // key row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_addr + Cfg::kColS + h * 64;    // this half's S^T columns; P^T goes to the first 32
        const uint32_t tDP = tmem + lane_addr + Cfg::kColDP + h * 64;
        uint8_t* ds_row = sDS + h * kPanel + j * 128;
        const float c = p.scale_log2;
        bool ok = true;
        for (int it = 0; it < n_iter; ++it) {
            const int qs = it % Cfg::kQStages;
            const float* lse = sLse + qs * kTile + h * 64;
            const float* dlt = sDelta + qs * kTile + h * 64;
            const bool masked = p.causal && (it % n_qt == 0);  // the diagonal query tile
            uint32_t pk[32];  // P^T of this thread: 64 query columns, packed bf16 pairs
            // the Q barrier also carries the LSE and Delta rows of this query tile
            ok = mbar_wait(&q_full[qs], (it / Cfg::kQStages) & 1, ctx, 29) && mbar_wait(s_full, it & 1, ctx, 30);
            if (!ok) break;
            tc_fence_after_sync();
            GQA_TRACE(0, it, 0);
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t v[32];
                tmem_ld32(tS + ch * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int col = ch * 32 + 2 * i;
                    const float2 l2 = *reinterpret_cast<const float2*>(lse + col);
                    float e0 = ex2_approx(fmaf(__uint_as_float(v[2 * i]), c, -l2.x));
                    float e1 = ex2_approx(fmaf(__uint_as_float(v[2 * i + 1]), c, -l2.y));
                    if (masked) {  // key j is visible to query i iff j <= i
                        if (j > h * 64 + col) e0 = 0.f;
                        if (j > h * 64 + col + 1) e1 = 0.f;
                    }
                    pk[ch * 16 + i] = pack_bf16x2(e0, e1);
                }
                uint32_t out[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) out[i] = pk[ch * 16 + i];
                tmem_st16(tS + ch * 16, out);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(p_ready);
            GQA_TRACE(0, it, 1);

            ok = mbar_wait(dp_full, it & 1, ctx, 31);
            if (ok && it > 0) ok = mbar_wait(ds_free, (it - 1) & 1, ctx, 32);
            if (!ok) break;
            GQA_TRACE(0, it, 2);
            tc_fence_after_sync();
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t v[32];
                tmem_ld32(tDP + ch * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {  // 8 query columns = one 16-byte chunk of the dS^T row
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int col = ch * 32 + q4 * 8 + 2 * i;
                        const float2 d2 = *reinterpret_cast<const float2*>(dlt + col);
                        const uint32_t pp = pk[(col >> 1)];
                        const float s0 = bf16_lo_to_f32(pp) * (__uint_as_float(v[q4 * 8 + 2 * i]) - d2.x);
                        const float s1 = bf16_hi_to_f32(pp) * (__uint_as_float(v[q4 * 8 + 2 * i + 1]) - d2.y);
                        w[i] = pack_bf16x2(s0, s1);
                    }
                    const int chunk = ch * 4 + q4;
                    *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (j & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(ds_ready);
            GQA_TRACE(0, it, 3);
        }
        // ---- epilogue: dV and scale*dK of this key row, half of the columns per warpgroup ----
        if (ok) ok = mbar_wait(acc_full, 0, ctx, 33);
        if (ok) {
            tc_fence_after_sync();
            constexpr int kHalf = D / 2;
            const size_t grow = (size_t)kv_row0 + j;
#pragma unroll 1
            for (int which = 0; which < 2; ++which) {
                const uint32_t tA = tmem + lane_addr + (which == 0 ? Cfg::kColDV : Cfg::kColDK) + h * kHalf;
                __nv_bfloat16* dst = (which == 0 ? p.dV : p.dK) + grow * D + h * kHalf;
                const float mul = which == 0 ? 1.0f : p.scale;
#pragma unroll 1
                for (int ch = 0; ch < kHalf / 32; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(tA + ch * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * mul, __uint_as_float(v[8 * i + 1]) * mul);
                        o.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * mul, __uint_as_float(v[8 * i + 3]) * mul);
                        o.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * mul, __uint_as_float(v[8 * i + 5]) * mul);
                        o.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * mul, __uint_as_float(v[8 * i + 7]) * mul);
                        *reinterpret_cast<uint4*>(dst + ch * 32 + i * 8) = o;
                    }
                }
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 13) {
        if (*abort_flag != 0) __nanosleep(20000);  // let in-flight copies and MMAs drain before TMEM is released
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

template <int D>
int launch_bwd_t(const void* Q, const void* K, const void* V, const void* dO, const float* lse2, const float* delta,
                 float* dq_accum, void* dK, void* dV, const Shape& s, unsigned int* status, cudaStream_t stream) {
    using Cfg = BwdCfg<D>;
    CUtensorMap mq, mk, mv, mdo;
    int rc = make_panel_tmap(&mq, Q, s.q_rows(), D, kTile);
    if (rc) return rc;
    rc = make_panel_tmap(&mk, K, s.kv_rows(), D, kTile);
    if (rc) return rc;
    rc = make_panel_tmap(&mv, V, s.kv_rows(), D, kTile);
    if (rc) return rc;
    rc = make_panel_tmap(&mdo, dO, s.q_rows(), D, kTile);
    if (rc) return rc;
    GQA_CUDA_TRY(cudaFuncSetAttribute(gqa_bwd_sm100_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg::kSmemTotal));
    BwdParams p;
    p.lse2 = lse2;
    p.delta = delta;
    p.dq_accum = dq_accum;
    p.dK = static_cast<__nv_bfloat16*>(dK);
    p.dV = static_cast<__nv_bfloat16*>(dV);
    p.status = status;
    p.Hq = s.Hq;
    p.Hkv = s.Hkv;
    p.S = s.S;
    p.causal = s.causal;
    p.n_tiles = s.S / kTile;
    p.G = s.G();
    p.scale = s.scale;
    p.scale_log2 = s.scale * 1.4426950408889634f;
    const unsigned grid = (unsigned)(p.n_tiles * s.B * s.Hkv);
    gqa_bwd_sm100_kernel<D><<<grid, kBwdThreads, Cfg::kSmemTotal, stream>>>(mq, mk, mv, mdo, p);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

}  // namespace

#ifdef GQA_BWD_TRACE
extern "C" int gqa_debug_copy_bwd_trace(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, g_bwd_trace, sizeof(g_bwd_trace));
}
#endif

int launch_bwd_main_sm100(const void* Q, const void* K, const void* V, const void* dO, const float* lse2,
                          const float* delta, float* dq_accum, void* dK, void* dV, const Shape& s,
                          unsigned int* status, cudaStream_t stream) {
    if (s.D == 64) return launch_bwd_t<64>(Q, K, V, dO, lse2, delta, dq_accum, dK, dV, s, status, stream);
    return launch_bwd_t<128>(Q, K, V, dO, lse2, delta, dq_accum, dK, dV, s, status, stream);
}

}  // namespace gqa
