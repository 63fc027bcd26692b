// GQA forward for sm_100a at head dimension 64: O = softmax(scale * Q K^T [+ causal]) V, LSE.
//
// At D = 64 a 128 x 128 tile needs 16 384 exponentials (1 024 cycles of the SM's exp unit) against 512 cycles
// of tensor math, and a softmax warp that works alone on its scheduler partition cannot keep the exp unit busy:
// its own TMEM loads, maxima, conversions and barrier hand-overs sit between its exponentials.  This kernel
// therefore runs FOUR softmax warpgroups per SM (four warps per scheduler partition) instead of two:
// one CTA owns two 128-row query tiles of one (batch, query head), and the keys of every 128-row block are split
// between two independent streams per tile -- stream 0 takes keys 0-63 of each block, stream 1 keys 64-127.
// Each stream is a complete online softmax of its own: own running maximum and row sum, own 64-column S buffer
// (P overwrites its head as packed bf16) and own 64-column O accumulator in tensor memory (4 x 64 + 4 x 64 = 512
// columns).  The two partial results of a tile are merged once, in the epilogue:
//     m = max(m0, m1),  a_w = exp2((m_w - m) * c),  O = (a0 O0 + a1 O1) / (a0 l0 + a1 l1).
// Roles (21 warps):
//   warps 0-15   softmax warpgroups g = 2 * tile + stream (thread = query row = TMEM lane)
//   warp  16     TMA producer (Q once, K and V rings)
//   warps 17-20  UMMA issuers, one per stream: S = Q K_half^T and O += P V_half (P read from TMEM)
// A stream's S buffer is single: S(n+1) is issued when P(n) V has completed, and while that stream waits for its
// two products the other three warps of the partition own the exp unit.  The softmax runs in two passes over the
// 64 columns (row maximum, then exponentials) with 32 values in registers at a time, so that 24 resident warps
// fit the register file.  The running maximum is only refreshed when it grows by more than 2^8.
//
// Replaces gqa62::gqa_v62 / launch_gqa_v62 (src/attention/GQA_fwd_ref.cu:336-651) for D = 64:
// same inputs/outputs, LSE = natural-log of the scaled-logit sum (:611-614).
#include "gqa_common.cuh"
#include "gqa_kernels.cuh"
#include "sm100_ptx.cuh"

namespace gqa {
namespace {

using namespace sm100;

constexpr int kD = 64;
constexpr int kTile = 128;             // query rows per tile and key rows per block
constexpr int kPanel = kTile * 128;    // bytes of one 128-row x 64-column bf16 tile (one swizzled panel)
constexpr int kHalf = 64;              // keys per stream and block
constexpr int kStages = 4;
constexpr int kWarpTma = 16, kWarpMma0 = 17;
constexpr int kThreads = 21 * 32;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units

constexpr int kOffQ = 0;                           // two query tiles
constexpr int kOffK = kOffQ + 2 * kPanel;          // kStages key blocks
constexpr int kOffV = kOffK + kStages * kPanel;    // kStages value blocks
constexpr int kOffMl = kOffV + kStages * kPanel;   // [2 tiles][2 streams][128 rows] (m, l) for the merge
constexpr int kOffBars = kOffMl + 2 * 2 * kTile * 8;
constexpr int kSmemTotal = kOffBars + 512;         // the dynamic window must start 1024-byte aligned (checked)
static_assert(kSmemTotal <= 227 * 1024, "shared memory budget");
static_assert(kSmemTotal > 114 * 1024, "one CTA per SM is assumed by the 512-column TMEM allocation");
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;         // + 64 * g

struct Fwd64Params {
    __nv_bfloat16* O;
    float* LSE;
    unsigned int* status;
    int Hq, Hkv, S, causal, n_pairs, bshd;
    float scale_log2;  // scale * log2(e)
};

__global__ void __launch_bounds__(kThreads, 1)
gqa_fwd64_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                       const __grid_constant__ CUtensorMap mapV, const Fwd64Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // swizzled panels need 1024-byte alignment; report instead of computing garbage
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, 0x80000000u | (99u << 20));
        return;
    }
    uint8_t* sQ = smem + kOffQ;
    uint8_t* sK = smem + kOffK;
    uint8_t* sV = smem + kOffV;
    float2* sMl = reinterpret_cast<float2*>(smem + kOffMl);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
    uint64_t* q_full = bars;                // [2]  per tile
    uint64_t* s_full = bars + 2;            // [4]  per stream: S(n) written
    uint64_t* p_full = bars + 6;            // [4]  per stream: P(n) written by the warpgroup (and S(n) consumed)
    uint64_t* pv_done = bars + 10;          // [4]  per stream: P(n) V completed
    uint64_t* ml_full = bars + 14;          // [2]  per tile: both streams have published (m, l)
    uint64_t* k_full = bars + 16;           // [kStages]
    uint64_t* k_empty = k_full + kStages;   // [kStages]
    uint64_t* v_full = k_empty + kStages;   // [kStages]
    uint64_t* v_empty = v_full + kStages;   // [kStages]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_empty + kStages);
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
    const int n_blocks_all = (p.S + kTile - 1) / kTile;  // the last block may be partial: keys at and beyond S are masked
    int n_blk[2];
    n_blk[0] = p.causal ? (q0 / kTile + 1) : n_blocks_all;
    n_blk[1] = (n_tiles == 2) ? (p.causal ? (q0 / kTile + 2) : n_blocks_all) : 0;
    const int n_max = n_blk[1] > n_blk[0] ? n_blk[1] : n_blk[0];
    const int q_row0 = (b * p.Hq + hq) * p.S + q0;   // row in [B,Hq,S] order (LSE)
    // Tensor-map coordinates (x = column, y = position in the sequence, z = matrix).  [B,H,S,D] is B*H matrices
    // [S, D]; [B,S,H,D] is B matrices [S, H*D] with the head at x = head * D.  Rows at y >= S read as zeros.
    const int q_x = p.bshd ? hq * kD : 0, q_z = p.bshd ? b : b * p.Hq + hq;
    const int kv_x = p.bshd ? hkv * kD : 0, kv_z = p.bshd ? b : b * p.Hkv + hkv;

    // ---- setup ------------------------------------------------------------------
    if (tid == 0) {
        // a non-zero status word (a bounded wait gave up earlier and nobody has read the report yet) makes
        // every later thread block skip its work, so a wedged launch drains in one wave
        *abort_flag = (*reinterpret_cast<volatile unsigned int*>(p.status) != 0u) ? 98u : 0u;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&ml_full[i], 2 * kTile);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], kTile);
            mbar_init(&pv_done[i], 1);
        }
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 2 * n_tiles);  // one commit per issuer that reads the block
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 2 * n_tiles);
        }
        fence_mbar_init();
    }
    if (warp == kWarpMma0) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (*abort_flag != 0) {  // uniform: every thread reads the flag after the barrier
        if (warp == kWarpMma0) tmem_dealloc(tmem, kTmemCols);
        return;
    }

    if (warp == kWarpTma) {
        // ======================= TMA producer =======================
        if (elect_one()) {
            tma_prefetch_desc(&mapQ);
            tma_prefetch_desc(&mapK);
            tma_prefetch_desc(&mapV);
            for (int t = 0; t < n_tiles; ++t) {
                mbar_expect_tx(&q_full[t], kPanel);
                tma_load_3d(sQ + t * kPanel, &mapQ, &q_full[t], q_x, q0 + t * kTile, q_z);
            }
            for (int n = 0; n < n_max; ++n) {
                const int st = n % kStages;
                const uint32_t use = n / kStages;
                if (use > 0 && !mbar_wait(&k_empty[st], (use - 1) & 1, ctx, 10)) break;
                mbar_expect_tx(&k_full[st], kPanel);
                tma_load_3d(sK + st * kPanel, &mapK, &k_full[st], kv_x, n * kTile, kv_z);
                if (use > 0 && !mbar_wait(&v_empty[st], (use - 1) & 1, ctx, 11)) break;
                mbar_expect_tx(&v_full[st], kPanel);
                tma_load_3d(sV + st * kPanel, &mapV, &v_full[st], kv_x, n * kTile, kv_z);
            }
        }
    } else if (warp >= kWarpMma0) {
        // ======================= issuer of stream g: S(n) = Q K_half(n)^T, O += P(n) V_half(n) =======================
        // The whole warp runs the loop (uniform control flow); `leader` marks the one lane that issues.
        const int g = warp - kWarpMma0, t = g >> 1, w = g & 1;
        if (t < n_tiles) {
            const uint32_t leader = elect_one() ? 1u : 0u;
            const uint32_t idesc_qk = make_idesc_bf16(128, kHalf, false, false);
            const uint32_t idesc_pv = make_idesc_bf16(128, kD, false, true);
            const uint32_t q_addr = smem_u32(sQ) + t * kPanel, k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            const uint32_t colS = tmem + kColS + g * 64, colO = tmem + kColO + g * 64;
            const int total = n_blk[t];
            bool ok = mbar_wait(&q_full[t], 0, ctx, 20);
            // (causal: tile 0 stops one block before tile 1; the release of that last block is never waited for)
            for (int n = 0; n < total && ok; ++n) {
                const int st = n % kStages;
                const uint32_t ph = (n / kStages) & 1;
                // S(n) overwrites the buffer that holds P(n-1): that product must have completed
                ok = mbar_wait(&k_full[st], ph, ctx, 21);
                if (ok && n > 0) ok = mbar_wait(&pv_done[g], (n - 1) & 1, ctx, 22);
                if (!ok) break;
                tc_fence_after_sync();
                {   // rows 64w.. of the key block are the B operand (K-major panel, 64 rows = 8192 bytes down)
                    const uint32_t b0 = k_addr + st * kPanel + w * (kHalf * 128);
#pragma unroll
                    for (int kk = 0; kk < kD / 16; ++kk)
                        umma_ss_pred(leader, colS, make_sdesc_sw128(q_addr + kk * 32, 16, 1024),
                                     make_sdesc_sw128(b0 + kk * 32, 16, 1024), idesc_qk, kk > 0);
                    umma_commit_pred(leader, &s_full[g]);
                    umma_commit_pred(leader, &k_empty[st]);
                }
                ok = mbar_wait(&v_full[st], ph, ctx, 23) && mbar_wait(&p_full[g], n & 1, ctx, 24);
                if (!ok) break;
                tc_fence_after_sync();
                {   // P(n) (64 keys = 32 packed columns at the head of the S buffer) times rows 64w.. of the value block
                    const uint32_t b0 = v_addr + st * kPanel + w * (kHalf / 16) * 2048;
#pragma unroll
                    for (int kk = 0; kk < kHalf / 16; ++kk)
                        umma_ts_pred(leader, colO, colS + kk * 8, make_sdesc_sw128(b0 + kk * 2048, kPanel, 1024), idesc_pv,
                                     (n > 0 || kk > 0));
                    umma_commit_pred(leader, &pv_done[g]);
                    umma_commit_pred(leader, &v_empty[st]);
                }
            }
        }
    } else {
        // ======================= softmax warpgroups =======================
        const int g = warp >> 2, t = g >> 1, w = g & 1;   // stream g: tile t, key half w
        const int r = (warp & 3) * 32 + lane;             // row inside the tile == TMEM lane
        if (t < n_tiles) {
            const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
            const uint32_t tS = tmem + lane_addr + kColS + g * 64;
            const uint32_t tO = tmem + lane_addr + kColO + g * 64;
            const float c = p.scale_log2;
            const uint64_t c2 = pack_f32x2(c, c);
            const int total = n_blk[t];
            const int diag_block = (q0 + t * kTile) / kTile;  // only this block needs the causal mask
            const int col0 = w * kHalf;                       // column of this stream's first key inside a block
            float m_run = -INFINITY;  // running maximum of the raw logits that P is measured against
            float l_run = 0.f;
            bool ok = true;
            for (int n = 0; n < total; ++n) {
                ok = mbar_wait(&s_full[g], n & 1, ctx, 30);
                if (!ok) break;
                tc_fence_after_sync();
                // last valid column of this row inside the 128-key block: the causal diagonal and / or the end of S
                const bool diag = p.causal && (n == diag_block);
                const int s_left = p.S - n * kTile;  // keys of this block that exist
                const bool masked = diag || s_left < kTile;
                const int lim = min(diag ? r : kTile - 1, s_left - 1);
                uint32_t v[32];
                // ---- pass 1: row maximum of the 64 columns
                float mx = -INFINITY;
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    tmem_ld32(tS + ch * 32, v);
                    tmem_wait_ld();
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            m4[i & 3] = (col0 + ch * 32 + i > lim) ? m4[i & 3] : fmaxf(m4[i & 3], __uint_as_float(v[i]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 2)
                            m4[(i >> 1) & 3] = max3_f32(m4[(i >> 1) & 3], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                    }
                    mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
                }
                // A stream may not have seen a visible key yet (causal rows above its key half, keys beyond S):
                // its maximum is then still -inf and every difference of maxima below is guarded against inf - inf.
                const float m_new = fmaxf(m_run, mx);
                const bool grow = (m_new > m_run) && ((m_run == -INFINITY) || (m_new - m_run) * c > kRescaleThreshold);
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = grow ? ((m_run == -INFINITY) ? 0.f : ex2_approx((m_run - m_new) * c)) : 1.f;
                    l_run *= alpha;
                    if (grow) m_run = m_new;
                    if (n > 0) {
                        // O holds P(0..n-1) V; the last of those products may still be running
                        ok = mbar_wait(&pv_done[g], (n - 1) & 1, ctx, 32);
                        if (!ok) break;
                        tc_fence_after_sync();
#pragma unroll 1
                        for (int ch = 0; ch < kD / 32; ++ch) {
                            uint32_t o32[32];
                            tmem_ld32(tO + ch * 32, o32);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o32[i] = __float_as_uint(__uint_as_float(o32[i]) * alpha);
                            tmem_st32(tO + ch * 32, o32);
                        }
                    }
                }
                // ---- pass 2: P = exp2(c*s - c*m) (packed fma), row sum, packed bf16 into the first 32 columns of the
                // S buffer (chunk 0 lands on columns 0-15, which it has just read; chunk 1 on 16-31, read by chunk 0)
                const float mc = (m_run == -INFINITY) ? 0.f : m_run * c;  // a row without a visible key: every P is masked to 0
                float l_add = 0.f;
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    tmem_ld32(tS + ch * 32, v);
                    tmem_wait_ld();
                    uint32_t pk[16];
                    if (!masked) {
                        const uint64_t nmc2 = pack_f32x2(-mc, -mc);
                        uint64_t l2[2] = {0ull, 0ull};
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), c2, nmc2);
                            float x0, x1;
                            unpack_f32x2(x, x0, x1);
                            const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
                            l2[i & 1] = add_f32x2(l2[i & 1], pack_f32x2(e0, e1));
                            pk[i] = pack_bf16x2(e0, e1);
                        }
                        float a0, a1, b0, b1;
                        unpack_f32x2(l2[0], a0, a1);
                        unpack_f32x2(l2[1], b0, b1);
                        l_add += (a0 + a1) + (b0 + b1);
                    } else {
                        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int cc = col0 + ch * 32 + 2 * i;
                            float e0 = ex2_approx(fmaf(__uint_as_float(v[2 * i]), c, -mc));
                            float e1 = ex2_approx(fmaf(__uint_as_float(v[2 * i + 1]), c, -mc));
                            if (cc > lim) e0 = 0.f;
                            if (cc + 1 > lim) e1 = 0.f;
                            l4[i & 3] += e0 + e1;
                            pk[i] = pack_bf16x2(e0, e1);
                        }
                        l_add += (l4[0] + l4[1]) + (l4[2] + l4[3]);
                    }
                    tmem_st16(tS + ch * 16, pk);
                }
                l_run += l_add;
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&p_full[g]);
            }
            // ---- epilogue: merge the two streams of the tile.  Each thread publishes (m, l) of its row, then reads
            // both; stream w writes output columns [32w, 32w+32) from both accumulators (a warp reaches the TMEM
            // lanes of its own quarter in every column, so no accumulator has to travel through shared memory).
            if (ok) {
                sMl[(t * 2 + w) * kTile + r] = make_float2(m_run, l_run);
                mbar_arrive(&ml_full[t]);
                ok = mbar_wait(&ml_full[t], 0, ctx, 33);
            }
            // both accumulators complete: the last product of either stream
            if (ok) ok = mbar_wait(&pv_done[t * 2], (total - 1) & 1, ctx, 31) && mbar_wait(&pv_done[t * 2 + 1], (total - 1) & 1, ctx, 34);
            if (ok) {
                tc_fence_after_sync();
                const float2 ml0 = sMl[(t * 2 + 0) * kTile + r], ml1 = sMl[(t * 2 + 1) * kTile + r];
                const float m = fmaxf(ml0.x, ml1.x);  // finite: stream 0 always sees key 0 of the first block
                const float a0 = (ml0.x == -INFINITY) ? 0.f : ex2_approx((ml0.x - m) * c);
                const float a1 = (ml1.x == -INFINITY) ? 0.f : ex2_approx((ml1.x - m) * c);
                const float l = a0 * ml0.y + a1 * ml1.y;
                const float inv_l = 1.0f / l;
                const float f0 = a0 * inv_l, f1 = a1 * inv_l;
                // rows beyond the end of the sequence are not stored (the TMEM loads below are warp-wide
                // instructions: every lane runs them, only the stores are guarded)
                const bool row_ok = q0 + t * kTile + r < p.S;
                const size_t grow_ = (size_t)q_row0 + t * kTile + r;
                __nv_bfloat16* orow = p.bshd ? p.O + ((size_t)(b * p.S + q0 + t * kTile + r) * p.Hq + hq) * kD : p.O + grow_ * kD;
                uint32_t x0[32], x1[32];
                tmem_ld32(tmem + lane_addr + kColO + (t * 2 + 0) * 64 + w * 32, x0);
                tmem_ld32(tmem + lane_addr + kColO + (t * 2 + 1) * 64 + w * 32, x1);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t o4[4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int e = 8 * i + 2 * jj;
                        o4[jj] = pack_bf16x2(fmaf(__uint_as_float(x0[e]), f0, __uint_as_float(x1[e]) * f1),
                                             fmaf(__uint_as_float(x0[e + 1]), f0, __uint_as_float(x1[e + 1]) * f1));
                    }
                    if (row_ok) *reinterpret_cast<uint4*>(orow + w * 32 + i * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                }
                if (w == 0 && p.LSE && row_ok) p.LSE[grow_] = (m * c + log2f(l)) * kLn2;
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kWarpMma0) {
        if (*abort_flag != 0) abort_grace_period();  // in-flight copies and MMAs land before TMEM is released
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace

int launch_fwd64_sm100(const void* Q, const void* K, const void* V, void* O, float* LSE, const Shape& s,
                       unsigned int* status, cudaStream_t stream) {
    CUtensorMap mq, mk, mv;
    // see the coordinates in the kernel
    const uint64_t S = s.S, qc = s.bshd ? (uint64_t)s.Hq * kD : kD, kc = s.bshd ? (uint64_t)s.Hkv * kD : kD;
    const uint64_t nq = s.bshd ? s.B : (uint64_t)s.B * s.Hq, nkv = s.bshd ? s.B : (uint64_t)s.B * s.Hkv;
    int rc = make_tile3_tmap(&mq, Q, qc, S, nq, S * qc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mk, K, kc, S, nkv, S * kc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mv, V, kc, S, nkv, S * kc, kTile);
    if (rc) return rc;
    GQA_CUDA_TRY(cudaFuncSetAttribute(gqa_fwd64_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    Fwd64Params p;
    p.O = static_cast<__nv_bfloat16*>(O);
    p.LSE = LSE;
    p.status = status;
    p.Hq = s.Hq;
    p.Hkv = s.Hkv;
    p.S = s.S;
    p.causal = s.causal;
    p.bshd = s.bshd;
    p.n_pairs = (s.S + 2 * kTile - 1) / (2 * kTile);
    p.scale_log2 = s.scale * kLog2e;
    dim3 grid(p.n_pairs, s.Hq, s.B);
    gqa_fwd64_sm100_kernel<<<grid, kThreads, kSmemTotal, stream>>>(mq, mk, mv, p);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

}  // namespace gqa
