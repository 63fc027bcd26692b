// GQA forward for sm_100a: O = softmax(scale * Q K^T [+ causal]) V, LSE.
//
// One CTA owns two 128-row query tiles of one (batch, query head) and streams the
// KV head's 128-row key/value blocks through a TMA ring.  Roles:
//   warps 0-3  softmax warpgroup for query tile 0 (thread = query row = TMEM lane)
//   warps 4-7  softmax warpgroup for query tile 1
//   warp  8    TMA producer (Q once, K and V rings)
//   warps 9,10 UMMA issuers, one per query tile: S = Q K^T and O += P V (P read from TMEM)
// Every key block is handled as two half-blocks of 64 keys, and the 128 fp32 S columns of a tile are two
// 64-column buffers: while the softmax warpgroup works on half-block j, the issuer has already produced
// S(j+1) in the other buffer, so the warpgroup never waits for the tensor core in steady state (with one
// 128-column S buffer per tile the chain softmax -> P V -> Q K^T -> softmax was serial and set the period).
// P(j) overwrites the first 32 columns of its own S buffer as packed bf16; S(j+2) may overwrite it only after
// P(j) V has completed (pv_done barrier; different accumulators, so issue order alone guarantees nothing).
// The running maximum is only refreshed when it grows by more than 2^8, so O is rescaled rarely (and then
// only after the previous P V has completed); the final division by the row sum uses the same maximum.
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
__device__ long long g_fwd_trace[6][64][4];
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
constexpr int kHalf = 64;               // keys per half-block
constexpr int kFwdThreads = 352;
constexpr int kWarpTma = 8, kWarpMma0 = 9;
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
    int Hq, Hkv, S, causal, n_pairs, bshd;
    const int* cu;     // packed variable-length batch: sequence starts (blockIdx.z = sequence), else null
    int d_real;        // head dimension of the tensors (<= D of the kernel; the columns beyond it read as zeros)
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
    uint64_t* q_full = bars;                       // [2]  per tile
    uint64_t* o_full = bars + 2;                   // [2]  per tile
    uint64_t* s_full = bars + 4;                   // [4]  per (tile, S buffer): S(j) written
    uint64_t* p_full = bars + 8;                   // [4]  per (tile, S buffer): P(j) written by the warpgroup
    uint64_t* pv_done = bars + 12;                 // [4]  per (tile, S buffer): P(j) V completed
    uint64_t* k_full = bars + 16;                  // [kStages]
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
    const int hq = blockIdx.y;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int q0 = pair * 2 * kTile;
    // Packed variable-length batch: the sequence is a row range [y0, y0 + len) of the one [T, H*D] matrix; rows past
    // its end belong to the next sequence (or read as zeros past T): as keys they are masked like keys beyond S,
    // as queries they are computed and not stored.  The grid covers max_seqlen: blocks beyond this sequence leave
    // here, before anything is set up.
    int b = blockIdx.z, y0 = 0, len = p.S;
    if (p.cu) {
        y0 = p.cu[b];
        len = p.cu[b + 1] - y0;
        b = 0;
        if (q0 >= len) return;
    }
    const int n_tiles = (q0 + kTile < len) ? 2 : 1;
    const int n_blocks_all = (len + kTile - 1) / kTile;  // the last block may be partial: keys at and beyond len are masked
    int n_blk[2];
    n_blk[0] = p.causal ? (q0 / kTile + 1) : n_blocks_all;
    n_blk[1] = (n_tiles == 2) ? (p.causal ? (q0 / kTile + 2) : n_blocks_all) : 0;
    const int n_max = n_blk[1] > n_blk[0] ? n_blk[1] : n_blk[0];
    const int q_row0 = (b * p.Hq + hq) * p.S + y0 + q0;   // row in [B,Hq,S] order (LSE)
    // Tensor-map coordinates (x = column, y = position in the sequence, z = matrix).  [B,H,S,D] is B*H matrices
    // [S, D]; [B,S,H,D] is B matrices [S, H*D] with the head at x = head * D.  Rows at y >= S read as zeros.
    const int q_x = p.bshd ? hq * D : 0, q_z = p.bshd ? b : b * p.Hq + hq;
    const int kv_x = p.bshd ? hkv * D : 0, kv_z = p.bshd ? b : b * p.Hkv + hkv;

    // ---- setup ------------------------------------------------------------------
    if (tid == 0) {
        // a non-zero status word (a bounded wait gave up earlier and nobody has read the report yet) makes
        // every later thread block skip its work, so a wedged launch drains in one wave
        *abort_flag = (*reinterpret_cast<volatile unsigned int*>(p.status) != 0u) ? 98u : 0u;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&o_full[i], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&pv_done[i], 1);
        }
        for (int i = 0; i < Cfg::kStages; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], n_tiles);  // one commit per issuer that uses the block
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], n_tiles);
        }
        fence_mbar_init();
    }
    if (warp == kWarpMma0) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (*abort_flag != 0) {  // uniform: every thread reads the flag after the barrier
        if (warp == kWarpMma0) tmem_dealloc(tmem, Cfg::kTmemCols);
        return;
    }

    if (warp == kWarpTma) {
        // ======================= TMA producer =======================
        if (elect_one()) {
            tma_prefetch_desc(&mapQ);
            tma_prefetch_desc(&mapK);
            tma_prefetch_desc(&mapV);
            for (int t = 0; t < n_tiles; ++t) {
                mbar_expect_tx(&q_full[t], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_3d(sQ + t * Cfg::kTileBytes + pn * kPanel, &mapQ, &q_full[t], q_x + pn * 64, y0 + q0 + t * kTile, q_z);
            }
            for (int n = 0; n < n_max; ++n) {
                const int st = n % Cfg::kStages;
                const uint32_t use = n / Cfg::kStages;
                if (use > 0 && !mbar_wait(&k_empty[st], (use - 1) & 1, ctx, 10)) break;
                mbar_expect_tx(&k_full[st], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_3d(sK + st * Cfg::kTileBytes + pn * kPanel, &mapK, &k_full[st], kv_x + pn * 64, y0 + n * kTile, kv_z);
                if (use > 0 && !mbar_wait(&v_empty[st], (use - 1) & 1, ctx, 11)) break;
                mbar_expect_tx(&v_full[st], Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn)
                    tma_load_3d(sV + st * Cfg::kTileBytes + pn * kPanel, &mapV, &v_full[st], kv_x + pn * 64, y0 + n * kTile, kv_z);
            }
        }
    } else if (warp >= kWarpMma0) {
        // ======================= issuer of tile t: S(j) = Q K(j)^T per half-block, O += P(j) V(j) =======================
        // The whole warp runs the loop (uniform control flow); `leader` marks the one lane that issues.
        const int t = warp - kWarpMma0;
        if (t < n_tiles) {
            const uint32_t leader = elect_one() ? 1u : 0u;
            const uint32_t idesc_qk = make_idesc_bf16(128, kHalf, false, false);
            const uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
            const uint32_t q_addr = smem_u32(sQ) + t * Cfg::kTileBytes, k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            const uint32_t colS = tmem + (t ? Cfg::kColS1 : Cfg::kColS0), colO = tmem + (t ? Cfg::kColO1 : Cfg::kColO0);
            const int total = 2 * n_blk[t];
            bool ok = mbar_wait(&q_full[t], 0, ctx, 20);
            // S(j): rows 64h.. of key block n = j/2 are the B operand (K-major panels, 64 rows = 8192 bytes down)
            auto issue_qk = [&](int j) -> bool {
                const int n = j >> 1, h = j & 1, st = n % Cfg::kStages;
                if (h == 0 && !mbar_wait(&k_full[st], (n / Cfg::kStages) & 1, ctx, 21)) return false;
                tc_fence_after_sync();
                const uint32_t b0 = k_addr + st * Cfg::kTileBytes + h * (kHalf * 128);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kPanel + (kk & 3) * 32;
                    umma_ss_pred(leader, colS + h * kHalf, make_sdesc_sw128(q_addr + off, 16, 1024),
                                 make_sdesc_sw128(b0 + off, 16, 1024), idesc_qk, kk > 0);
                }
                umma_commit_pred(leader, &s_full[t * 2 + h]);
                if (h == 1) umma_commit_pred(leader, &k_empty[st]);
                if (t == 0) GQA_FTRACE(1, j, 0);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < total && ok; ++j) {
                const int n = j >> 1, h = j & 1, st = n % Cfg::kStages;
                if (j + 1 < total) {
                    // S(j+1) goes where P(j-1) lives: that product must have completed
                    if (j >= 1) ok = mbar_wait(&pv_done[t * 2 + (h ^ 1)], ((j - 1) >> 1) & 1, ctx, 22);
                    if (ok) ok = issue_qk(j + 1);
                    if (!ok) break;
                }
                if (h == 0) ok = mbar_wait(&v_full[st], (n / Cfg::kStages) & 1, ctx, 23);
                if (ok) ok = mbar_wait(&p_full[t * 2 + h], n & 1, ctx, 24);
                if (!ok) break;
                tc_fence_after_sync();
                if (t == 0) GQA_FTRACE(1, j, 1);
                const uint32_t b0 = v_addr + st * Cfg::kTileBytes + h * (kHalf / 16) * 2048;
#pragma unroll
                for (int kk = 0; kk < kHalf / 16; ++kk)
                    umma_ts_pred(leader, colO, colS + h * kHalf + kk * 8, make_sdesc_sw128(b0 + kk * 2048, kPanel, 1024),
                                 idesc_pv, (j > 0 || kk > 0));
                umma_commit_pred(leader, &pv_done[t * 2 + h]);
                if (h == 1) umma_commit_pred(leader, &v_empty[st]);
                if (j + 1 == total) umma_commit_pred(leader, &o_full[t]);
                if (t == 0) GQA_FTRACE(1, j, 2);
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
            const uint64_t c2 = pack_f32x2(c, c);
            const int total = 2 * n_blk[t];
            const int diag_block = (q0 + t * kTile) / kTile;  // only this block needs the causal mask
            float m_run = -INFINITY;  // running maximum of the raw logits that P is measured against
            float l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < total; ++j) {
                const int n = j >> 1, h = j & 1;
                ok = mbar_wait(&s_full[t * 2 + h], n & 1, ctx, 30);
                if (!ok) break;
                tc_fence_after_sync();
                if (warp == 0) GQA_FTRACE(0, j, 0);
                if (warp == 4) GQA_FTRACE(2, j, 0);
                if (t == 0) GQA_FTRACE(4, j, warp & 3);
                // last valid column of this row inside the 128-key block: the causal diagonal and / or the end of S
                const bool diag = p.causal && (n == diag_block);
                const int s_left = len - n * kTile;  // keys of this block that exist
                const bool masked = diag || s_left < kTile;
                const int lim = min(diag ? r : kTile - 1, s_left - 1);
                const int col0 = h * kHalf;  // column of v[0] inside the 128-key block
                // the 64-column half row of S into registers (one TMEM round trip), then the row maximum with
                // four independent chains of three-input maxima
                uint32_t v[kHalf];
                tmem_ld32p(tS + col0, v);
                tmem_ld32p(tS + col0 + 32, v + 32);
                tmem_wait_ld();
                float mx;
                {
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < kHalf; ++i)
                            m4[i & 3] = (col0 + i > lim) ? m4[i & 3] : fmaxf(m4[i & 3], __uint_as_float(v[i]));
                    } else {
#pragma unroll
                        for (int i = 0; i < kHalf; i += 2)
                            m4[(i >> 1) & 3] = max3_f32(m4[(i >> 1) & 3], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                    }
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                }
                if (warp == 0) GQA_FTRACE(0, j, 1);
                const float m_new = fmaxf(m_run, mx);
                const bool grow = (m_new - m_run) * c > kRescaleThreshold;  // true on the first half-block (m_run = -inf)
                if (__any_sync(0xffffffffu, grow)) {
                    const float m_next = grow ? m_new : m_run;
                    const float alpha = ex2_approx((m_run - m_next) * c);
                    l_run *= alpha;
                    m_run = m_next;
                    if (j > 0) {
                        // O holds P(0..j-1) V; the last of those products may still be running
                        ok = mbar_wait(&pv_done[t * 2 + (h ^ 1)], ((j - 1) >> 1) & 1, ctx, 32);
                        if (!ok) break;
                        tc_fence_after_sync();
#pragma unroll 1
                        for (int ch = 0; ch < D / 32; ++ch) {
                            uint32_t w[32];
                            tmem_ld32(tO + ch * 32, w);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * alpha);
                            tmem_st32(tO + ch * 32, w);
                        }
                    }
                }
                // P = exp2(c*s - c*m) (packed fma), row sum (two packed partial sums), packed bf16 into the first
                // 32 columns of this S buffer
                const float mc = m_run * c;
                float l_add;
                if (!masked) {
                    const uint64_t nmc2 = pack_f32x2(-mc, -mc);
                    uint64_t l2[2] = {0ull, 0ull};
#pragma unroll
                    for (int ch = 0; ch < 2; ++ch) {
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint64_t x = fma_f32x2(
                                pack_f32x2(__uint_as_float(v[ch * 32 + 2 * i]), __uint_as_float(v[ch * 32 + 2 * i + 1])), c2, nmc2);
                            float x0, x1;
                            unpack_f32x2(x, x0, x1);
                            const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
                            l2[i & 1] = add_f32x2(l2[i & 1], pack_f32x2(e0, e1));
                            pk[i] = pack_bf16x2(e0, e1);
                        }
                        tmem_st16(tS + col0 + ch * 16, pk);
                    }
                    float a0, a1, b0, b1;
                    unpack_f32x2(l2[0], a0, a1);
                    unpack_f32x2(l2[1], b0, b1);
                    l_add = (a0 + a1) + (b0 + b1);
                } else {
                    float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int ch = 0; ch < 2; ++ch) {
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int cc = col0 + ch * 32 + 2 * i;
                            float e0 = ex2_approx(fmaf(__uint_as_float(v[ch * 32 + 2 * i]), c, -mc));
                            float e1 = ex2_approx(fmaf(__uint_as_float(v[ch * 32 + 2 * i + 1]), c, -mc));
                            if (cc > lim) e0 = 0.f;
                            if (cc + 1 > lim) e1 = 0.f;
                            l4[i & 3] += e0 + e1;
                            pk[i] = pack_bf16x2(e0, e1);
                        }
                        tmem_st16(tS + col0 + ch * 16, pk);
                    }
                    l_add = (l4[0] + l4[1]) + (l4[2] + l4[3]);
                }
                l_run += l_add;
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&p_full[t * 2 + h]);
                if (warp == 0) GQA_FTRACE(0, j, 2);
                if (warp == 4) GQA_FTRACE(2, j, 2);
                GQA_FTRACE(t == 0 ? 3 : 5, j, warp & 3);
            }
            // epilogue: O / l -> bf16, LSE
            if (ok) ok = mbar_wait(&o_full[t], 0, ctx, 31);
            if (ok) {
                tc_fence_after_sync();
                // rows beyond the end of the sequence are not stored (the TMEM loads below are warp-wide
                // instructions: every lane runs them, only the stores are guarded)
                const bool row_ok = q0 + t * kTile + r < len;
                const float inv_l = 1.0f / l_run;
                const size_t grow_ = (size_t)q_row0 + t * kTile + r;
                __nv_bfloat16* orow = p.bshd ? p.O + ((size_t)(b * p.S + y0 + q0 + t * kTile + r) * p.Hq + hq) * D
                                             : p.O + grow_ * p.d_real;
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
                        if (row_ok && ch * 32 + i * 8 < p.d_real) *reinterpret_cast<uint4*>(orow + ch * 32 + i * 8) = o;
                    }
                }
                if (p.LSE && row_ok) p.LSE[grow_] = (m_run * c + log2f(l_run)) * kLn2;
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kWarpMma0) {
        if (*abort_flag != 0) abort_grace_period();  // in-flight copies and MMAs land before TMEM is released
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

template <int D>
int launch_fwd_t(const void* Q, const void* K, const void* V, void* O, float* LSE, const Shape& s, unsigned int* status,
                 cudaStream_t stream) {
    using Cfg = FwdCfg<D>;
    CUtensorMap mq, mk, mv;
    // see the coordinates in the kernel
    // (the matrices are s.D columns wide; a box that reaches beyond them reads zeros there)
    const uint64_t S = s.S, qc = s.bshd ? (uint64_t)s.Hq * D : s.D, kc = s.bshd ? (uint64_t)s.Hkv * D : s.D;
    const uint64_t nq = s.bshd ? s.B : (uint64_t)s.B * s.Hq, nkv = s.bshd ? s.B : (uint64_t)s.B * s.Hkv;
    int rc = make_tile3_tmap(&mq, Q, qc, S, nq, S * qc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mk, K, kc, S, nkv, S * kc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mv, V, kc, S, nkv, S * kc, kTile);
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
    p.bshd = s.bshd;
    p.d_real = s.D;
    p.cu = s.cu_seqlens;
    p.n_pairs = ((s.cu_seqlens ? s.max_seqlen : s.S) + 2 * kTile - 1) / (2 * kTile);
    p.scale_log2 = s.scale * kLog2e;
    dim3 grid(p.n_pairs, s.Hq, s.cu_seqlens ? s.n_seqs : s.B);
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
    if (s.Dp() == 64) return launch_fwd_t<64>(Q, K, V, O, LSE, s, status, stream);
    return launch_fwd_t<128>(Q, K, V, O, LSE, s, status, stream);
}

}  // namespace gqa
