// GQA backward, stage 2 of 3, for sm_100a: the KV-tile-parallel main kernel.
//
// A work item is one 128-row key/value tile of one (batch, KV head): the thread block that takes it loops over
// all G query heads of the group and over the 128-row query tiles that see the
// tile (all of them, or the ones at and below the diagonal when causal).  dK and
// dV therefore accumulate in tensor memory across the whole GQA group and are
// written exactly once: no atomics, bit-reproducible.  dQ tiles are reduced into
// an fp32 accumulator with vector reductions (order-dependent in the last bits).
// The thread blocks are persistent (one per SM) and claim items from a counter, the work of the reference's
// persistent launchers with an atomic tile counter (src/attention/GQA_bwd.cu:14269-14278, :14351-14376).
//
// Everything is computed in the transposed orientation so that a TMEM lane is a
// key row:  S^T = K Q^T,  dP^T = V dO^T  (both operands K-major from TMA panels),
//   P^T  = exp2(scale*log2e * (S^T - LSE/scale))  -> bf16 into TMEM (A operand of dV)
//   dS^T = P^T * (dP^T - Delta)                   -> bf16 into swizzled shared memory
// The two subtractions are done by the tensor core: -LSE/scale and -Delta of every query row are split
// into three bf16 terms by the preprocess kernel and enter S^T and dP^T as one extra K step against a
// constant "ones" operand.  That removes the per-element broadcast loads of LSE and Delta from shared
// memory, whose bandwidth is what bounds this kernel.
//   dV  += P^T dO      (A from TMEM,  B = dO panel read MN-major)
//   dK  += dS^T Q      (A = dS^T K-major, B = Q panel read MN-major)
//   dQ   = dS K        (A = dS^T read MN-major, B = K panel read MN-major)
//
// Roles at D = 64 (24 warps; D = 128 uses 16: two elementwise warpgroups):
//   warps 0-3    drain dQ tiles from TMEM into the fp32 accumulator
//   warps 4-19   four elementwise warpgroups; each owns 32 query columns of the tile pair
//   warp  20     TMA producer
//   warps 21-23  UMMA issuers: [S^T, dP^T] | dV | [dK, dQ]
// The five GEMMs wait on different producers, and one issuing warp sustains a 128x64x16 product
// only every 57 cycles (78 when A comes from TMEM) against 32 cycles of tensor math, so they are
// issued by three warps in parallel, each a warp-uniform loop with one elected lane; mbarriers
// carry every cross-warp dependency.  Registers are granted in steps of four warps, so 24 warps
// get 80 registers per thread where 25 got 72 (dK and dQ both wait for dS^T and share a warp).
//
// Replaces gqa_bwd_vj1d (src/attention/GQA_bwd_baseline.cu:405-547) in the
// G-loop-inside-the-CTA form of gqa_bwd_vz2_wgmma (src/attention/GQA_bwd.cu:15207-15342);
// roundings follow the reference: P is rounded to bf16 before dV and before the dS product,
// dS = bf16(P_bf16 * (dP - Delta)) with the product in fp32, dK and dQ are scaled in fp32
// (GQA_bwd_baseline.cu:243-255, :320-326, :530-534).
#include <type_traits>

#include "gqa_common.cuh"
#include "gqa_kernels.cuh"
#include "sm100_ptx.cuh"

namespace gqa {
namespace {

using namespace sm100;

// Optional timeline tracing (development builds only): block 0 stamps clock64 at a few points per iteration.
#ifdef GQA_BWD_TRACE
#ifndef GQA_BWD_TRACE_BLOCK
#define GQA_BWD_TRACE_BLOCK 0
#endif
__device__ long long g_bwd_trace[5][64][4];
__device__ long long g_bwd_marks[16];
__device__ long long g_bwd_items[4096][6];  // per work item: block, SM, start and end (globaltimer, ns), start and end (clock64)
__device__ __forceinline__ long long trace_globaltimer() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ int trace_smid() {
    int v;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
    return v;
}
#define GQA_ITEM_BEGIN(idx)                                  \
    do {                                                     \
        if ((idx) < 4096) {                                  \
            g_bwd_items[idx][0] = blockIdx.x;                \
            g_bwd_items[idx][1] = trace_smid();              \
            g_bwd_items[idx][2] = trace_globaltimer();       \
            g_bwd_items[idx][4] = clock64();                 \
        }                                                    \
    } while (0)
#define GQA_ITEM_END(idx)                                          \
    do {                                                           \
        if ((idx) < 4096) { g_bwd_items[idx][3] = trace_globaltimer(); g_bwd_items[idx][5] = clock64(); } \
    } while (0)
#define GQA_MARK(slot)                                                                            \
    do {                                                                                           \
        if (blockIdx.x == GQA_BWD_TRACE_BLOCK && (threadIdx.x & 31) == 0) g_bwd_marks[slot] = clock64(); \
    } while (0)
#define GQA_TRACE(role, it, slot)                                                                  \
    do {                                                                                           \
        if (blockIdx.x == GQA_BWD_TRACE_BLOCK && (it) >= 0 && (it) < 64 && (threadIdx.x & 31) == 0) g_bwd_trace[role][it][slot] = clock64(); \
    } while (0)
#else
#define GQA_TRACE(role, it, slot) \
    do {                          \
    } while (0)
#define GQA_MARK(slot) \
    do {               \
    } while (0)
#define GQA_ITEM_BEGIN(idx) \
    do {                    \
    } while (0)
#define GQA_ITEM_END(idx) \
    do {                  \
    } while (0)
#endif

constexpr int kTile = 128;
constexpr int kPanel = kTile * 128;  // bytes of one 64-column panel of a 128-row tile
constexpr int kWarpEw0 = 4;  // warps 0-3 drain dQ, the elementwise warpgroups follow

template <int D>
struct BwdCfg {
    static constexpr int kPanels = D / 64;
    static constexpr int kTileBytes = kPanels * kPanel;
    // Elementwise warpgroups: four at D = 64 (32 query columns per thread).  At D = 128 two (64 columns per
    // thread): the tensor work per tile pair doubles while the elementwise work does not, and the smaller CTA
    // (16 instead of 24 warps) leaves 128 registers per thread, which the dQ drain needs (see kDrainEarlyRelease).
    static constexpr int kEwGroups = (D == 64) ? 4 : 2;
    static constexpr int kCols = kTile / kEwGroups;       // query columns per elementwise thread
    static constexpr int kHalves = kCols / 16;            // 16-column steps per thread and stage
    static constexpr int kEwThreads = kEwGroups * 128;
    // dK and dQ (both wait for dS^T) are issued by one warp, which makes the CTA 24 / 16 warps.
    static constexpr int kWarpTma = kWarpEw0 + 4 * kEwGroups, kWarpMmaS = kWarpTma + 1, kWarpMmaDV = kWarpTma + 2,
                         kWarpMmaDK = kWarpTma + 3;
    static constexpr int kThreads = (kWarpMmaDK + 1) * 32;
    // D = 128: dQ sits in the dP^T columns, so the next dP^T product waits for the drain.  The drain warps
    // therefore pull the tile into registers as fast as TMEM delivers it (three 32-column chunks at once, the
    // fourth as soon as the first is staged) and hand the columns back before the copy engine has taken anything.
    static constexpr bool kDrainEarlyRelease = (D == 128);
    // Stages of the Q and dO rings.  A stage is released late in an iteration (Q by dK(it), dO by dV(it)) and a tile
    // takes 1 000-1 700 cycles to arrive, so with two stages S^T(it+2) / dP^T(it+2) waited for their operands (seen on
    // the clock64 timeline); D = 64 has the room for three.
    static constexpr int kQStages = (D == 64) ? 3 : 2;
    static constexpr int kDOStages = (D == 64) ? 3 : 1;
    static constexpr int kColPanel = kTile * 16;  // 128 rows x 16 B: an un-swizzled 8-column operand panel
    static constexpr int kDqBoxes = (D == 64) ? 2 : 1;  // 32-column fp32 boxes staged per drain round and warp
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kOffK + kTileBytes;
    static constexpr int kOffQ = kOffV + kTileBytes;
    static constexpr int kOffDO = kOffQ + kQStages * kTileBytes;
    static constexpr int kOffDS = kOffDO + kDOStages * kTileBytes;
    // (a second dS^T staging buffer, dQ(it) reading one while dS^T(it+1) is written into the other, was measured
    // at D = 64 and changed nothing)
    static constexpr int kOffDQ = kOffDS + 2 * kPanel;   // dQ staging: 4 drain warps x kDqBoxes x (32 rows x 128 B)
    static constexpr int kOffOnes = kOffDQ + 4 * kDqBoxes * 4096;   // constant A operand of the extra K step
    static constexpr int kOffLseCol = kOffOnes + kColPanel;         // [kQStages] -LSE/scale columns of the query tile
    static constexpr int kOffDltCol = kOffLseCol + kQStages * kColPanel;  // [kDOStages] -Delta columns
    static constexpr int kOffZero = kOffDltCol + kDOStages * kColPanel;   // all-zero panel (columns 8-15 of every one)
    static constexpr int kOffBars = kOffZero + kColPanel;
    static constexpr int kSmemTotal = kOffBars + 384;  // the dynamic window must start 1024-byte aligned (checked)
    static constexpr uint32_t kTmemCols = 512;
    // fp32 column map.  D = 64: every tile has its own columns.  D = 128: P^T overwrites the S^T columns
    // and dQ reuses the dP^T columns; the p_free / dq_empty barriers guard the reuse.
    static constexpr bool kPAliasesS = (D != 64);
    static constexpr bool kDqAliasesDp = (D != 64);
    // D = 64: dS^T is also stored as bf16 over the first half of each warpgroup's dP^T columns, so that dK reads
    // its A operand from TMEM instead of shared memory (shared-memory bandwidth is what bounds this kernel).
    static constexpr bool kDsInTmem = (D == 64);
    static constexpr uint32_t kColS = 0, kColDP = 128;
    static constexpr uint32_t kColDQ = (D == 64) ? 256 : 128;
    static constexpr uint32_t kColDV = (D == 64) ? 320 : 256;
    static constexpr uint32_t kColDK = kColDV + D;
    static constexpr uint32_t kColP = (D == 64) ? 448 : 0;
    static_assert(kColDK + D + (kPAliasesS ? 0 : 64) <= 512, "TMEM budget");
    static_assert(kSmemTotal <= 227 * 1024, "shared memory budget");
    static_assert(kSmemTotal > 114 * 1024, "one CTA per SM is assumed by the 512-column TMEM allocation");
};

struct BwdParams {
    float* dq_accum;     // [B*Hq*S, D] fp32, zeroed by the preprocess stage
    __nv_bfloat16* dK;
    __nv_bfloat16* dV;
    unsigned int* status;
    unsigned int* dq_turn;  // deterministic mode: one counter per 32 query rows (zeroed), else nullptr
    // Head split: with `parts` > 1 a KV tile's work is cut over `parts` thread blocks, each looping over G / parts
    // of the group's query heads and storing its dK / dV sums as fp32 into `partial` ([part][dV, dK][key row][D of
    // the kernel]); a fixed-order sum over the parts then rounds once (dkdv_reduce_kernel).  Used when there are too
    // few KV tiles to fill the SMs evenly (a long-context problem sharded down to one KV head per GPU).
    float* partial;
    int parts;
    int groups;   // B * Hkv
    const int* cu;  // packed variable-length batch: sequence starts (n_seqs + 1), else null
    int sg;       // causal order: (batch, KV head) groups per super-group (see the work-item comment)
    int n_items;  // n_tiles * groups * parts: work items, each handled by one thread block at a time
    int Hq, Hkv, S, causal, n_tiles, G, bshd;
    int d_real;  // head dimension of the tensors (<= D of the kernel; the columns beyond it read as zeros)
    float scale, scale_log2;
};

// TMEM column of the bf16 P^T block that holds query columns [16*kk, 16*kk+16) (one K step of dV).
template <int D>
__device__ __forceinline__ uint32_t p_col_of_kstep(int kk) {
    using Cfg = BwdCfg<D>;
    if constexpr (Cfg::kPAliasesS)  // inside its owner's S columns
        return Cfg::kColS + (kk / Cfg::kHalves) * Cfg::kCols + (kk % Cfg::kHalves) * 8;
    else return Cfg::kColP + kk * 8;
}

// kVarlen: packed variable-length batch (see the work-item decode): the items of the list that lie beyond their
// sequence are skipped by the producer, the rows beyond a sequence's end are masked in P^T.
// kWithDQ = false: the variant that leaves dQ to the separate query-parallel pass (gqa_bwd_dq_sm100.cu): no dQ
// product, idle drain warps, and at D = 64 no dS^T in shared memory at all (dK reads its copy in TMEM).
template <int D, bool kWithDQ, bool kVarlen>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, 1)
gqa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                     const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                     const __grid_constant__ CUtensorMap mapDQ, const __grid_constant__ CUtensorMap mapLseCol,
                     const __grid_constant__ CUtensorMap mapDltCol, const BwdParams p) {
    using Cfg = BwdCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // swizzled panels need 1024-byte alignment; report instead of computing garbage
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, 0x80000000u | (99u << 20));
        return;
    }
    if (threadIdx.x == 0) GQA_MARK(0);
    uint8_t* sK = smem + Cfg::kOffK;
    uint8_t* sV = smem + Cfg::kOffV;
    uint8_t* sQ = smem + Cfg::kOffQ;
    uint8_t* sDO = smem + Cfg::kOffDO;
    uint8_t* sDS = smem + Cfg::kOffDS;
    uint8_t* sDQ = smem + Cfg::kOffDQ;
    uint8_t* sOnes = smem + Cfg::kOffOnes;
    uint8_t* sLseCol = smem + Cfg::kOffLseCol;
    uint8_t* sDltCol = smem + Cfg::kOffDltCol;
    uint8_t* sZero = smem + Cfg::kOffZero;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
    // Every group of products is followed by ONE commit (a commit is not free: it takes a slot in the tensor core's
    // queue like a small product), to a barrier that serves all the consumers of that group; the barriers that
    // release a Q or dO stage are kept per stage, so that the TMA producer, which lags by one use, can wait on them
    // by parity like everybody else.
    uint64_t* kv_full = bars + 0;    // TMA: K and V tiles
    uint64_t* p_ready = bars + 1;    // elementwise -> issuers: P^T(it) stored, S^T(it) consumed
    uint64_t* ds_ready = bars + 2;   // elementwise -> issuers: dS^T(it) stored, dP^T(it) consumed
    uint64_t* ds_free = bars + 3;    // after dQ(it) (covers dK(it), same thread): dS^T(it) consumed, dQ(it) complete
    uint64_t* dq_empty = bars + 4;   // drain warps -> issuers: dQ columns free
    uint64_t* acc_full = bars + 5;   // issuers dV + dK after the last products of a work item -> epilogue
    uint64_t* acc_empty = bars + 6;  // elementwise -> issuers dV + dK: the accumulators of the item have been read
    uint64_t* kv_empty = bars + 7;   // issuer dK/dQ after the last product of an item: K and V may be overwritten
    uint64_t* s_full = bars + 8;                     // [kQStages] after S^T(it): -> elementwise
    uint64_t* dk_done = s_full + Cfg::kQStages;      // [kQStages] after dK(it): Q stage free (S^T(it) finished long before),
                                                     //            and the dS^T copy in the dP^T columns has been read
    uint64_t* q_full = dk_done + Cfg::kQStages;      // [kQStages] TMA: Q tile + -LSE/scale columns
    uint64_t* dp_full = q_full + Cfg::kQStages;      // [kDOStages] after dP^T(it): -> elementwise; dO stage read by dP^T
    uint64_t* p_free = dp_full + Cfg::kDOStages;     // [kDOStages] after dV(it): P^T(it) consumed; dO stage read by dV
    uint64_t* do_full = p_free + Cfg::kDOStages;     // [kDOStages] TMA: dO tile + -Delta columns
    uint64_t* item_full = do_full + Cfg::kDOStages;  // [kItemSlots] TMA producer -> everybody: the block's next work item
    constexpr int kItemSlots = 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(item_full + kItemSlots);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
    volatile int* item_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [kItemSlots]
    static_assert((8 + 3 * Cfg::kQStages + 3 * Cfg::kDOStages + kItemSlots) * 8 + 8 + kItemSlots * 4 <= 384, "barrier area");

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    AbortCtx ctx{abort_flag, p.status};

    // ---- work items.  The grid is persistent (one thread block per SM, fewer when there is less work).  A block
    // starts with item blockIdx.x and then takes the next unclaimed item of the list below from a counter in global
    // memory, one after the other, with every barrier and ring simply carrying on, so that the head of an item (K/V
    // load, first S^T) overlaps the tail of the previous one (epilogue, last dQ drains).  The claim is dynamic and made
    // late (see the producer), so that the items are handed out in list order as the blocks become free, like thread
    // blocks by the hardware: neighbours in the list then run side by side and share their Q/dO tiles in L2.  A fixed
    // share per block (items c, c + gridDim.x, ... in snake order) broke that and was 19 % slower at the 32k-token
    // causal shape.  Launched with one block per item the same code is the classic one-item-per-block kernel and never
    // touches the counter.
    // Order of the list.  Non-causal: the KV tiles of one (batch, KV head) group are neighbours, so the blocks that
    // run at the same time share their Q/dO tiles and dQ accumulator rows in L2 (measured +6.7 % at the headline
    // shape).  Causal: super-groups of (batch, KV head) groups, inside them the KV tile is the slow index, longest items
    // first (list scheduling in that order; the size of a super-group is chosen on the host).  The
    // deterministic mode also takes the KV tile as the slow index: the blocks of one group that run at the same time
    // must reduce one after the other, and this order keeps only a few of them in flight together.  It is launched
    // with one block per item: its blocks wait for one another, and a block that waits must never hold the SM that
    // the block it waits for needs (blocks are dispatched in index order, and a block only waits for lower ones).
    struct WorkItem {
        int kt, grp, part, b, hkv, qt0, n_qt, n_iter, kv_x, kv_z;
        int shift;  // the item's loop over the query tiles of a head starts at tile qt0 + shift and wraps around
        int y0, len;  // first row and length of the sequence in the tensors' row coordinate (0 and S unless packed)
    };
    const bool kt_major = p.causal || p.dq_turn != nullptr;
    const int g_local = p.G / p.parts;  // query heads a work item loops over
    // The j-th item of this block, published by the TMA producer in a small ring of slots; -1 = no more (or give up).
    // A slot is rewritten four items later, when every role has long read it (the producer publishes item j after
    // it has issued the loads of item j-1, which needs the products of item j-2 complete and with them the drains
    // inside item j-3 at the least).
    auto fetch_item = [&](int j) -> int {
        if (!mbar_wait(&item_full[j & (kItemSlots - 1)], (j / kItemSlots) & 1, ctx, 14)) return -1;
        return item_slot[j & (kItemSlots - 1)];
    };
    auto decode = [&](int idx) -> WorkItem {
        WorkItem w;
        w.part = idx % p.parts;  // the parts of a tile are neighbours
        const int item = idx / p.parts;
        if (kt_major) {  // super-group, then KV tile, then group inside the super-group
            const int per_sg = p.n_tiles * p.sg;
            const int r = item % per_sg;
            w.kt = r / p.sg;
            w.grp = (item / per_sg) * p.sg + r % p.sg;
        } else {
            w.kt = item % p.n_tiles;
            w.grp = item / p.n_tiles;
        }
        w.b = w.grp / p.Hkv;
        w.hkv = w.grp % p.Hkv;
        w.y0 = 0;
        w.len = p.S;
        int n_tiles = p.n_tiles;
        if constexpr (kVarlen) {
            // Packed batch: "batch" w.b of the list is a sequence, a row range of the one [T, H*D] matrix (matrix
            // index 0).  The list is laid out for max_seqlen: an item whose KV tile lies beyond its sequence comes out
            // with n_iter <= 0 and is skipped.  Rows past the end of the sequence are another sequence's (or zeros
            // past T): the elementwise warps zero P^T there, which zeroes dS^T and with it every contribution.
            w.y0 = p.cu[w.b];
            w.len = p.cu[w.b + 1] - w.y0;
            n_tiles = (w.len + kTile - 1) / kTile;
            w.b = 0;
        }
        w.qt0 = p.causal ? w.kt : 0;
        w.n_qt = n_tiles - w.qt0;
        w.n_iter = g_local * w.n_qt;
        // Non-causal: the blocks of one (batch, KV head) group start together; rotated by their KV tile index they
        // are on different query tiles at any time, so their dQ reductions do not queue on the same lines in L2 (all
        // starting at tile 0, the first waves ran 10-15 % slower per tile pair than the later, drifted-apart ones).
        // Causal blocks are staggered already (block kt starts at query tile kt); the deterministic mode wants its
        // blocks on the same tile one after the other.
        w.shift = kt_major ? 0 : w.kt;
        w.kv_x = p.bshd ? w.hkv * D : 0;
        w.kv_z = p.bshd ? w.b : w.b * p.Hkv + w.hkv;
        return w;
    };
    // Tensor-map coordinates (x = column, y = position in the sequence, z = matrix).  [B,H,S,D] is B*H matrices
    // [S, D]; [B,S,H,D] is B matrices [S, H*D] with the head at x = head * D.  The workspace arrays are B*Hq
    // matrices [S, .].  Rows at y >= S read as zeros and are skipped by the reductions, so S may be any length:
    // keys beyond S give zero rows of K and V (their dK / dV rows are not stored and their dS meets a zero row of
    // K in dQ), queries beyond S give zero rows of Q, dO and of the -LSE / -Delta columns (P = 1, dS = 0).
    auto head_of = [&](const WorkItem& w, int it) { return w.hkv * p.G + w.part * g_local + it / w.n_qt; };
    auto q_y_of = [&](const WorkItem& w, int it) {  // first query position
        return w.y0 + (w.qt0 + (it % w.n_qt + w.shift) % w.n_qt) * kTile;
    };
    auto q_x_of = [&](const WorkItem& w, int it) { return p.bshd ? head_of(w, it) * D : 0; };
    auto q_z_of = [&](const WorkItem& w, int it) { return p.bshd ? w.b : w.b * p.Hq + head_of(w, it); };
    auto ws_z_of = [&](const WorkItem& w, int it) { return w.b * p.Hq + head_of(w, it); };

    if (tid == 0) {
        // a thread block of this launch that has already given up leaves a non-zero status word: the blocks that
        // start after it skip their work (see below), so a wedged launch drains in one wave
        *abort_flag = (*reinterpret_cast<volatile unsigned int*>(p.status) != 0u) ? 98u : 0u;
        mbar_init(kv_full, 1);
        mbar_init(p_ready, Cfg::kEwThreads);
        mbar_init(ds_ready, Cfg::kEwThreads);
        mbar_init(ds_free, 1);
        mbar_init(dq_empty, 128);
        mbar_init(acc_full, 2);
        mbar_init(acc_empty, Cfg::kEwThreads);
        mbar_init(kv_empty, 1);
        for (int i = 0; i < Cfg::kQStages; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&dk_done[i], 1);
            mbar_init(&q_full[i], 1);
        }
        for (int i = 0; i < kItemSlots; ++i) mbar_init(&item_full[i], 1);
        for (int i = 0; i < Cfg::kDOStages; ++i) {
            mbar_init(&dp_full[i], 1);
            mbar_init(&p_free[i], 1);
            mbar_init(&do_full[i], 1);
        }
        fence_mbar_init();
    }
    if (warp == Cfg::kWarpMmaS) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    if (tid < kTile) {  // constant operands: ones in columns 0-2 (one per bf16 term of the split), zeros elsewhere
        *reinterpret_cast<uint4*>(sOnes + tid * 16) = make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u);
        *reinterpret_cast<uint4*>(sZero + tid * 16) = make_uint4(0u, 0u, 0u, 0u);
        fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (*abort_flag != 0) {  // uniform: every thread reads the flag after the barrier
        if (warp == Cfg::kWarpMmaS) tmem_dealloc(tmem, Cfg::kTmemCols);
        return;
    }
    if (threadIdx.x == 0) GQA_MARK(1);
    const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ);
    const uint32_t do_addr = smem_u32(sDO), ds_addr = smem_u32(sDS);

    if (warp == Cfg::kWarpTma) {
        // ======================= TMA producer =======================
        if (elect_one()) {
            tma_prefetch_desc(&mapQ);
            tma_prefetch_desc(&mapK);
            tma_prefetch_desc(&mapV);
            tma_prefetch_desc(&mapDO);
            tma_prefetch_desc(&mapDQ);
            tma_prefetch_desc(&mapLseCol);
            tma_prefetch_desc(&mapDltCol);
            unsigned int* work_counter = p.status + 16;  // zeroed with the status word before every launch
            int gi = 0;  // iterations issued so far, over all items: the rings and their barriers carry on across items
            auto claim = [&]() -> int {  // the next unclaimed item of the list that has work, -1 when there is none
                for (;;) {
                    if ((int)gridDim.x >= p.n_items) return -1;
                    const int next = (int)gridDim.x + (int)atomicAdd(work_counter, 1u);
                    if (next >= p.n_items) return -1;
                    if (!kVarlen || decode(next).n_iter > 0) return next;
                }
            };
            int idx = blockIdx.x;
            if constexpr (kVarlen) {
                if (decode(idx).n_iter <= 0) idx = claim();
            }
            bool ok = true;
            for (int j = 0; ok; ++j) {
                item_slot[j & (kItemSlots - 1)] = idx;
                mbar_arrive(&item_full[j & (kItemSlots - 1)]);
                if (idx < 0) break;
                const WorkItem w = decode(idx);
                if (j > 0) {
                    // a block of this launch that gave up has left a non-zero status word: stop taking items
                    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0u) {
                        *abort_flag = 98u;
                        break;
                    }
                    if (!mbar_wait(kv_empty, (j - 1) & 1, ctx, 13)) break;  // the previous item's last readers of K, V
                }
                mbar_expect_tx(kv_full, 2 * Cfg::kTileBytes);
                for (int pn = 0; pn < Cfg::kPanels; ++pn) {
                    tma_load_3d(sK + pn * kPanel, &mapK, kv_full, w.kv_x + pn * 64, w.y0 + w.kt * kTile, w.kv_z);
                    tma_load_3d(sV + pn * kPanel, &mapV, kv_full, w.kv_x + pn * 64, w.y0 + w.kt * kTile, w.kv_z);
                }
                int next = -1;
                for (int it = 0; it < w.n_iter; ++it, ++gi) {
                    // Claim the next item while the last tile pair of this one is loaded: late, so that the items
                    // are handed out in the order in which the blocks become free, as the hardware hands out thread
                    // blocks (neighbouring items then run side by side and share their Q/dO tiles in L2: claimed a
                    // whole item early, the 32k-token causal shape went to HBM for them, drew 13 % more energy
                    // per tile pair and ran that much slower under the power cap); the round trip to the counter hides
                    // behind the tile pairs that are still in the rings.
                    if (it == w.n_iter - 1) next = claim();
                    const int qx = q_x_of(w, it), qy = q_y_of(w, it), qz = q_z_of(w, it), wz = ws_z_of(w, it);
                    {
                        const int st = gi % Cfg::kQStages;
                        const uint32_t use = gi / Cfg::kQStages;
                        // the stage's last reader is dK of its previous use
                        if (use > 0 && !mbar_wait(&dk_done[st], (use - 1) & 1, ctx, 10)) { ok = false; break; }
                        // the -LSE/scale columns of the tile ride with Q (both are operands of S^T)
                        mbar_expect_tx(&q_full[st], Cfg::kTileBytes + Cfg::kColPanel);
                        for (int pn = 0; pn < Cfg::kPanels; ++pn)
                            tma_load_3d(sQ + st * Cfg::kTileBytes + pn * kPanel, &mapQ, &q_full[st], qx + pn * 64, qy, qz);
                        tma_load_3d(sLseCol + st * Cfg::kColPanel, &mapLseCol, &q_full[st], 0, qy, wz);
                    }
                    {
                        const int st = gi % Cfg::kDOStages;
                        const uint32_t use = gi / Cfg::kDOStages;
                        // the stage's readers are dP^T and dV of its previous use (neither implies the other)
                        if (use > 0 && !(mbar_wait(&dp_full[st], (use - 1) & 1, ctx, 11) && mbar_wait(&p_free[st], (use - 1) & 1, ctx, 12))) { ok = false; break; }
                        // the -Delta columns ride with dO (both are operands of dP^T)
                        mbar_expect_tx(&do_full[st], Cfg::kTileBytes + Cfg::kColPanel);
                        for (int pn = 0; pn < Cfg::kPanels; ++pn)
                            tma_load_3d(sDO + st * Cfg::kTileBytes + pn * kPanel, &mapDO, &do_full[st], qx + pn * 64, qy, qz);
                        tma_load_3d(sDltCol + st * Cfg::kColPanel, &mapDltCol, &do_full[st], 0, qy, wz);
                    }
                }
                idx = next;
            }
        }
    } else if (warp == Cfg::kWarpMmaS) {
        // ======================= issuer: S^T(it) = K Q^T, dP^T(it) = V dO^T =======================
        // The whole warp runs the loop (uniform control flow); `leader` marks the one lane that issues.
        const uint32_t leader = elect_one() ? 1u : 0u;
        const uint32_t idesc = make_idesc_bf16(128, 128, false, false);
        // A operand of the extra K step: ones in columns 0-2 (un-swizzled column panel), columns 8-15 = the zero panel
        const uint32_t ones_addr = smem_u32(sOnes), zero_addr = smem_u32(sZero);
        const uint64_t ones_desc = make_sdesc_noswizzle(ones_addr, zero_addr - ones_addr, 128);
        auto issue = [&](uint32_t col, uint32_t a0, uint32_t b0, uint32_t cols_addr) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk >> 2) * kPanel + (kk & 3) * 32;
                umma_ss_pred(leader, tmem + col, make_sdesc_sw128(a0 + off, 16, 1024),
                             make_sdesc_sw128(b0 + off, 16, 1024), idesc, kk > 0);
            }
            // + 1 * (hi + mid + lo) of the per-query-row term (-LSE/scale or -Delta)
            umma_ss_pred(leader, tmem + col, ones_desc, make_sdesc_noswizzle(cols_addr, zero_addr - cols_addr, 128), idesc,
                         1u);
        };
        int gi = 0;  // iteration index over all items of this block (parities and ring stages carry on across items)
        bool ok = true;
        for (int j = 0; ok; ++j) {
            const int idx = fetch_item(j);
            if (idx < 0) break;
            const int n_iter = decode(idx).n_iter;
            ok = mbar_wait(kv_full, j & 1, ctx, 20);
            for (int it = 0; it < n_iter && ok; ++it, ++gi) {
                const int qs = gi % Cfg::kQStages, dos = gi % Cfg::kDOStages;
                ok = mbar_wait(&q_full[qs], (gi / Cfg::kQStages) & 1, ctx, 21);
                if (ok && gi > 0) ok = mbar_wait(p_ready, (gi - 1) & 1, ctx, 22);                        // S^T columns read
                if (ok && gi > 0 && Cfg::kPAliasesS)                                                     // P^T consumed
                    ok = mbar_wait(&p_free[(gi - 1) % Cfg::kDOStages], ((gi - 1) / Cfg::kDOStages) & 1, ctx, 23);
                if (!ok) break;
                tc_fence_after_sync();
                GQA_TRACE(1, gi, 0);
                issue(Cfg::kColS, k_addr, q_addr + qs * Cfg::kTileBytes, smem_u32(sLseCol) + qs * Cfg::kColPanel);
                umma_commit_pred(leader, &s_full[qs]);
                GQA_TRACE(1, gi, 1);
                ok = mbar_wait(&do_full[dos], (gi / Cfg::kDOStages) & 1, ctx, 24);
                if (ok && gi > 0) ok = mbar_wait(ds_ready, (gi - 1) & 1, ctx, 25);                       // dP^T columns read
                if (ok && gi > 0 && Cfg::kDqAliasesDp && kWithDQ) ok = mbar_wait(dq_empty, (gi - 1) & 1, ctx, 26);  // dQ drained
                if (ok && gi > 0 && Cfg::kDsInTmem)                                                      // dK read dS^T
                    ok = mbar_wait(&dk_done[(gi - 1) % Cfg::kQStages], ((gi - 1) / Cfg::kQStages) & 1, ctx, 27);
                if (!ok) break;
                tc_fence_after_sync();
                GQA_TRACE(1, gi, 2);
                issue(Cfg::kColDP, v_addr, do_addr + dos * Cfg::kTileBytes, smem_u32(sDltCol) + dos * Cfg::kColPanel);
                umma_commit_pred(leader, &dp_full[dos]);
                GQA_TRACE(1, gi, 3);
            }
        }
    } else if (warp == Cfg::kWarpMmaDV) {
        // ======================= issuer: dV += P^T dO(it)  (A from TMEM, B = dO read MN-major) =======================
        const uint32_t leader = elect_one() ? 1u : 0u;
        const uint32_t idesc = make_idesc_bf16(128, D, false, true);
        int gi = 0;
        bool ok = true;
        for (int j = 0; ok; ++j) {
            const int idx = fetch_item(j);
            if (idx < 0) break;
            const int n_iter = decode(idx).n_iter;
            if (j > 0) ok = mbar_wait(acc_empty, (j - 1) & 1, ctx, 37);  // the epilogue has read the previous item's dV
            for (int it = 0; it < n_iter && ok; ++it, ++gi) {
                const int dos = gi % Cfg::kDOStages;
                ok = mbar_wait(&do_full[dos], (gi / Cfg::kDOStages) & 1, ctx, 30) && mbar_wait(p_ready, gi & 1, ctx, 31);
                if (!ok) break;
                tc_fence_after_sync();
                GQA_TRACE(3, gi, 0);
                const uint32_t b0 = do_addr + dos * Cfg::kTileBytes;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    umma_ts_pred(leader, tmem + Cfg::kColDV, tmem + p_col_of_kstep<D>(kk),
                                 make_sdesc_sw128(b0 + kk * 2048, kPanel, 1024), idesc, (it > 0 || kk > 0));
                umma_commit_pred(leader, &p_free[dos]);
                GQA_TRACE(3, gi, 1);
            }
            if (ok) umma_commit_pred(leader, acc_full);
        }
    } else if (warp == Cfg::kWarpMmaDK) {
        // ======================= issuer: dK += dS^T Q(it)  (A = dS^T K-major, B = Q read MN-major), then dQ(it) =======================
        const uint32_t leader = elect_one() ? 1u : 0u;
        const uint32_t idesc = make_idesc_bf16(128, D, false, true);
        int gi = 0;
        bool ok = true;
        for (int j = 0; ok; ++j) {
            const int idx = fetch_item(j);
            if (idx < 0) break;
            const int n_iter = decode(idx).n_iter;
            ok = mbar_wait(kv_full, j & 1, ctx, 34);
            if (ok && j > 0) ok = mbar_wait(acc_empty, (j - 1) & 1, ctx, 38);  // the epilogue has read the previous item's dK
            for (int it = 0; it < n_iter && ok; ++it, ++gi) {
                const int qs = gi % Cfg::kQStages;
                ok = mbar_wait(&q_full[qs], (gi / Cfg::kQStages) & 1, ctx, 32) && mbar_wait(ds_ready, gi & 1, ctx, 33);
                if (!ok) break;
                tc_fence_after_sync();
                GQA_TRACE(4, gi, 0);
                const uint32_t b0 = q_addr + qs * Cfg::kTileBytes;
                const uint32_t ds_buf = ds_addr;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    if constexpr (Cfg::kDsInTmem)  // A = bf16 dS^T in the dP^T columns: query columns [16kk, 16kk+16)
                        umma_ts_pred(leader, tmem + Cfg::kColDK, tmem + Cfg::kColDP + (kk / Cfg::kHalves) * Cfg::kCols + (kk % Cfg::kHalves) * 8,
                                     make_sdesc_sw128(b0 + kk * 2048, kPanel, 1024), idesc, (it > 0 || kk > 0));
                    else
                        umma_ss_pred(leader, tmem + Cfg::kColDK,
                                     make_sdesc_sw128(ds_buf + (kk >> 2) * kPanel + (kk & 3) * 32, 16, 1024),
                                     make_sdesc_sw128(b0 + kk * 2048, kPanel, 1024), idesc, (it > 0 || kk > 0));
                }
                umma_commit_pred(leader, &dk_done[qs]);
                GQA_TRACE(4, gi, 1);
                if constexpr (!kWithDQ) {
                    umma_commit_pred(leader, ds_free);  // dK(it) was the last reader of dS^T(it)
                } else {  // dQ(it) = dS K  (A = dS^T read MN-major, B = K read MN-major)
                    if (gi > 0) ok = mbar_wait(dq_empty, (gi - 1) & 1, ctx, 36);
                    if (!ok) break;
                    tc_fence_after_sync();
                    GQA_TRACE(4, gi, 2);
                    const uint32_t idesc_dq = make_idesc_bf16(128, D, true, true);
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        umma_ss_pred(leader, tmem + Cfg::kColDQ, make_sdesc_sw128(ds_buf + kk * 2048, kPanel, 1024),
                                     make_sdesc_sw128(k_addr + kk * 2048, kPanel, 1024), idesc_dq, kk > 0);
                    umma_commit_pred(leader, ds_free);
                    GQA_TRACE(4, gi, 3);
                }
            }
            if (ok) {
                umma_commit_pred(leader, acc_full);
                umma_commit_pred(leader, kv_empty);  // every product of the item that reads K (dQ) or V (dP^T, ordered before
                                                     // dK by ds_ready) has finished when this fires
            }
        }
    } else if (warp < kWarpEw0) {
        if constexpr (kWithDQ) {
        // ======================= dQ drain warps =======================
        // Each warp owns 32 query rows: TMEM -> registers -> its own swizzled staging boxes -> TMA reduce-add
        // into the fp32 accumulator.  The reductions run on the copy engine, off the load/store pipe.
        const uint32_t tDQ = tmem + ((uint32_t)(warp * 32) << 16) + Cfg::kColDQ;
        constexpr int kWarpStage = Cfg::kDqBoxes * 4096;
        uint8_t* stage = sDQ + warp * kWarpStage + lane * 128;
        const int sw = lane & 7;
        // The loop exists twice, with and without the deterministic mode's bookkeeping (the `det` tag below): the role
        // is short of registers, and the default path should not carry the turn state.
        auto drain_items = [&](auto det) {
        constexpr bool kDet = decltype(det)::value;
        // Deterministic mode: the reductions into one 32-row slice of the accumulator are applied in KV-tile order.
        // The CTA of KV tile kt waits until the slice's counter reads kt (its predecessors run or have run: they
        // have smaller block indices), and hands on with kt + 1 once its own reductions have completed.
        // Fill cost: CTA kt starts its first reduction kt hand-overs late; after that the stagger persists.
        auto turn_acquire = [&](unsigned int* turn, unsigned int early, int kt) -> bool {
            uint32_t good = 1;
            if (lane == 0) {
                const long long t0 = clock64();
                uint32_t polls = 0;
                while (early != (unsigned)kt && ld_acquire_gpu(turn) != (unsigned)kt) {
                    if ((++polls & 0x3fu) == 0) {
                        if (*abort_flag != 0) { good = 0; break; }
                        if (clock64() - t0 > kWaitLimitCycles) {
                            *abort_flag = 41;
                            atomicCAS(p.status, 0u, 0x80000000u | (41u << 20) | (blockIdx.x & 0xfffffu));
                            good = 0;
                            break;
                        }
                    }
                }
                fence_proxy_async_global();  // our reductions (async proxy) are ordered after the acquire
            }
            return __shfl_sync(0xffffffffu, good, 0) != 0;
        };
        // The turn of a tile is handed on one iteration later, just before the next tile's reductions are issued:
        // by then the reductions have had a TMEM round trip and a staging pass to land, so the wait for their
        // completion is short.  (Holding the turns of three tiles instead was slower: the hand-over delay, not the
        // wait, is what the CTAs of a group queue on.)
        unsigned int* held = nullptr;  // slice whose turn this warp still holds
        unsigned int held_next = 0;    // the value that hands it on: 1 + the KV tile it was taken for
        auto release_held = [&]() {
            if (kDet && held) {
                if (lane == 0) {
                    bulk_wait_all();  // completed: the sums are visible to this thread
                    st_release_gpu(held, held_next);
                }
                __syncwarp();
                held = nullptr;
            }
        };
        int gi = 0;
        bool going = true;
        for (int j = 0; going; ++j) {
        // per item only what the loop needs, kept as running coordinates (registers are short in this role)
        int kt, n_left, n_qt, row0, row, wz;
        {
            const int idx = fetch_item(j);
            if (idx < 0) break;
            const WorkItem w = decode(idx);
            kt = w.kt;
            n_left = w.n_iter;
            n_qt = w.n_qt;
            row0 = w.y0 + w.qt0 * kTile + warp * 32;  // first query position of this warp's slice in the item's lowest tile
            row = q_y_of(w, 0) + warp * 32;    // ... and in the tile its loop starts with
            wz = ws_z_of(w, 0);
        }
        const int row_end = row0 + n_qt * kTile;
        int qi = 0;  // tiles done in the current query head
        for (; n_left > 0; --n_left, ++gi) {
            unsigned int* turn = kDet ? p.dq_turn + ((size_t)wz * p.n_tiles + row / kTile) * 4 + warp : nullptr;
            bool turn_mine = !kDet;  // becomes true once this warp may reduce into the slice
            // first look at the counter now: its round trip to L2 hides behind the TMEM loads and the staging
            const unsigned int early = (kDet && lane == 0) ? ld_acquire_gpu(turn) : 0xffffffffu;
            if (!mbar_wait(ds_free, gi & 1, ctx, 40)) { going = false; break; }  // dQ(it) complete
            tc_fence_after_sync();
            GQA_TRACE(2, gi, 0);
            constexpr int kRounds = D / (32 * Cfg::kDqBoxes);
            if constexpr (Cfg::kDrainEarlyRelease) {
                static_assert(!Cfg::kDrainEarlyRelease || (D == 128 && Cfg::kDqBoxes == 1), "four 32-column chunks, one box");
                auto stage_box = [&](const uint32_t (&v)[32]) {
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8)
                        *reinterpret_cast<uint4*>(stage + ((c8 ^ sw) << 4)) =
                            make_uint4(v[4 * c8], v[4 * c8 + 1], v[4 * c8 + 2], v[4 * c8 + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                };
                auto reduce_box = [&](int chunk) {  // then wait until the box may be overwritten
                    if (turn_mine && lane == 0) {
                        tma_reduce_add_3d(&mapDQ, sDQ + warp * kWarpStage, chunk * 32, row, wz);
                        bulk_commit_group();
                        bulk_wait_read_all();
                    }
                    __syncwarp();
                };
                uint32_t va[32], vb[32], vc[32];
                tmem_ld32(tDQ, va);
                tmem_ld32(tDQ + 32, vb);
                tmem_ld32(tDQ + 64, vc);
                tmem_wait_ld();
                stage_box(va);
                tmem_ld32(tDQ + 96, va);  // chunk 0 is in shared memory: its registers take chunk 3
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(dq_empty);     // the dP^T columns are free after two TMEM round trips
                release_held();
                if (kDet && !turn_mine) turn_mine = turn_acquire(turn, early, kt);
                reduce_box(0);
                stage_box(vb);
                reduce_box(1);
                stage_box(vc);
                reduce_box(2);
                stage_box(va);
                reduce_box(3);
                if (kDet && turn_mine) { held = turn; held_next = (unsigned)kt + 1u; }
            } else {
    #pragma unroll 1
                for (int rnd = 0; rnd < kRounds; ++rnd) {
                    // (Plain stores whose order against the TMEM loads is left to the compiler.  Measured alternatives,
                    // all slower at D = 64 although they remove the ~100 bytes per thread that this form spills under the
                    // kernel's 80 registers: the box loop not unrolled, 10 %; 16-column chunks with the next load in
                    // flight, 1-3 %; the second box's load issued by hand before the first box is staged, 4 %; the same
                    // boxes with the staging addresses recomputed per tile pair instead of kept in registers, 0.7 %.)
    #pragma unroll
                    for (int bx = 0; bx < Cfg::kDqBoxes; ++bx) {
                        uint32_t v[32];
                        tmem_ld32(tDQ + (rnd * Cfg::kDqBoxes + bx) * 32, v);
                        tmem_wait_ld();
                        if (rnd == kRounds - 1 && bx == Cfg::kDqBoxes - 1) {  // every column is in registers: hand the TMEM tile back
                            tc_fence_before_sync();
                            mbar_arrive(dq_empty);
                        }
    #pragma unroll
                        for (int c8 = 0; c8 < 8; ++c8)
                            *reinterpret_cast<uint4*>(stage + bx * 4096 + ((c8 ^ sw) << 4)) =
                                make_uint4(v[4 * c8], v[4 * c8 + 1], v[4 * c8 + 2], v[4 * c8 + 3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    release_held();
                    GQA_TRACE(2, gi, 2);
                    if (kDet && !turn_mine) turn_mine = turn_acquire(turn, early, kt);
                    GQA_TRACE(2, gi, 3);
                    if (turn_mine && lane == 0) {
    #pragma unroll
                        for (int bx = 0; bx < Cfg::kDqBoxes; ++bx)
                            tma_reduce_add_3d(&mapDQ, sDQ + warp * kWarpStage + bx * 4096, (rnd * Cfg::kDqBoxes + bx) * 32, row, wz);
                        bulk_commit_group();
                        bulk_wait_read_all();  // staging boxes may be overwritten after this
                    }
                    __syncwarp();
                }
                if (kDet && turn_mine) { held = turn; held_next = (unsigned)kt + 1u; }
            }
            if (!turn_mine) { going = false; break; }  // a bounded wait gave up: the abort flag is set
            GQA_TRACE(2, gi, 1);
            row += kTile;  // next tile of the head (the loop wraps around at the head's last tile) ...
            if (row == row_end) row = row0;
            if (++qi == n_qt) {  // ... or the same start tile of the next head
                qi = 0;
                ++wz;
            }
        }
        }
        if (warp == 0) GQA_MARK(7);
        release_held();
        };
        if (p.dq_turn)
            drain_items(std::true_type{});
        else
            drain_items(std::false_type{});
        if (lane == 0) bulk_wait_all();
        if (warp == 0) GQA_MARK(8);
        }
    } else if (warp < Cfg::kWarpTma) {
        // ======================= elementwise warpgroups (P^T and dS^T) =======================
        // Per tile pair: S^T(it) -> P^T(it), then dP^T(it) -> dS^T(it); P^T is carried in registers as packed bf16
        // (the rounded values the dV product uses) between the two phases.
        constexpr int C = Cfg::kCols, H = Cfg::kHalves;
        const int w = (warp - kWarpEw0) >> 2;     // which C query columns of the tile pair
        const int j = (warp & 3) * 32 + lane;     // key row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_addr + Cfg::kColS + w * C;
        const uint32_t tDP = tmem + lane_addr + Cfg::kColDP + w * C;
        const uint32_t tP = tmem + lane_addr + (Cfg::kPAliasesS ? (Cfg::kColS + w * C) : (Cfg::kColP + w * (C / 2)));
        // dS^T row j, query columns [C*w, C*w+C): 64-column panel (C*w)/64, 16-byte chunks from ((C*w) % 64)/8 on
        uint8_t* ds_row0 = sDS + ((w * C) >> 6) * kPanel + j * 128;
        const int chunk0 = ((w * C) & 63) >> 3;
        const float c = p.scale_log2;
        const bool trace_me = (warp == kWarpEw0);
        (void)trace_me;
        bool ok = true;
        uint32_t pk_cur[C / 2];  // P^T(it) of this thread: C query columns as packed bf16 pairs

        // P^T of 16 columns [16*hf, 16*hf+16) from the S^T values v (which already hold S - LSE/scale) -> packed pairs
        // (masked: the query columns outside [c_lo, c_hi) of this key row are zeroed: c_lo = j on the causal diagonal
        // tile; packed batches also cut at the end of the sequence, in the query and in the key direction)
        auto p_half = [&](const uint32_t (&v)[16], int hf, bool masked, int c_lo, int c_hi, uint32_t* out) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float e0 = ex2_approx(__uint_as_float(v[4 * i + 0]) * c);
                float e1 = ex2_approx(__uint_as_float(v[4 * i + 1]) * c);
                float e2 = ex2_approx(__uint_as_float(v[4 * i + 2]) * c);
                float e3 = ex2_approx(__uint_as_float(v[4 * i + 3]) * c);
                if (masked) {
                    const int col = w * C + hf * 16 + 4 * i;
                    if constexpr (kVarlen) {
                        if (col + 0 < c_lo || col + 0 >= c_hi) e0 = 0.f;
                        if (col + 1 < c_lo || col + 1 >= c_hi) e1 = 0.f;
                        if (col + 2 < c_lo || col + 2 >= c_hi) e2 = 0.f;
                        if (col + 3 < c_lo || col + 3 >= c_hi) e3 = 0.f;
                    } else {  // causal diagonal tile: key j is visible to query i iff j <= i
                        if (j > col + 0) e0 = 0.f;
                        if (j > col + 1) e1 = 0.f;
                        if (j > col + 2) e2 = 0.f;
                        if (j > col + 3) e3 = 0.f;
                    }
                }
                out[2 * i + 0] = pack_bf16x2(e0, e1);
                out[2 * i + 1] = pack_bf16x2(e2, e3);
            }
        };
        // dS^T of 16 columns from the dP^T values v (which already hold dP - Delta) and the packed P^T pairs
        // -> two 16-byte chunks of the dS^T row (and the same packed values for the TMEM copy)
        auto ds_half = [&](const uint32_t (&v)[16], int hf, const uint32_t* pk, uint32_t* dsp, uint8_t* ds_row) {
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2) {
                const uint32_t* pp = pk + q2 * 4;
                uint32_t o4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#ifdef GQA_BWD_PACKED_DS
                    // shortcut (not the default): (dP - Delta) rounded to bf16 first, one packed bf16 product;
                    // two roundings instead of one, about 3 % faster
                    o4[i] = mul_bf16x2(pp[i], pack_bf16x2(__uint_as_float(v[q2 * 8 + 2 * i]), __uint_as_float(v[q2 * 8 + 2 * i + 1])));
#else
                    // dS = bf16(P_bf16 * (dP - Delta)): the product in fp32, one rounding, as the reference does
                    const float p_lo = __uint_as_float(pp[i] << 16), p_hi = __uint_as_float(pp[i] & 0xffff0000u);
                    o4[i] = pack_bf16x2(p_lo * __uint_as_float(v[q2 * 8 + 2 * i]), p_hi * __uint_as_float(v[q2 * 8 + 2 * i + 1]));
#endif
                }
                const uint4 o = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                const int chunk = chunk0 + hf * 2 + q2;
                // shared-memory copy: read by dQ, and by dK where it does not have the TMEM copy
                if constexpr (kWithDQ || !Cfg::kDsInTmem) *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (j & 7)) << 4)) = o;
                dsp[q2 * 4 + 0] = o.x;
                dsp[q2 * 4 + 1] = o.y;
                dsp[q2 * 4 + 2] = o.z;
                dsp[q2 * 4 + 3] = o.w;
            }
        };
        auto publish_p = [&](const uint32_t* pk) {
#pragma unroll
            for (int ch = 0; ch < C / 32; ++ch) {
                uint32_t t16[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) t16[i] = pk[ch * 16 + i];
                tmem_st16(tP + ch * 16, t16);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(p_ready);
        };

        // S^T(g) -> P^T(g), published for dV
        // diag: the tile on the causal diagonal; q_valid / kv_valid: query columns / key rows of the tile pair that
        // belong to the sequence (packed batches only; >= kTile when the tile is whole)
        auto make_p = [&](int g, bool diag, int q_valid, int kv_valid) -> bool {
            bool masked = diag;
            int c_lo = 0, c_hi = kTile;
            if constexpr (kVarlen) {
                masked = diag || q_valid < kTile || kv_valid < kTile;
                c_lo = diag ? j : 0;
                c_hi = (j < kv_valid) ? q_valid : 0;
            }
            if (!mbar_wait(&s_full[g % Cfg::kQStages], (g / Cfg::kQStages) & 1, ctx, 51)) return false;
            tc_fence_after_sync();
            if (trace_me) GQA_TRACE(0, g - 1, 2);
#pragma unroll
            for (int hf = 0; hf < H; ++hf) {
                uint32_t vs[16];
                tmem_ld16(tS + hf * 16, vs);
                tmem_wait_ld();
                p_half(vs, hf, masked, c_lo, c_hi, pk_cur + hf * 8);
            }
            if constexpr (!Cfg::kPAliasesS) {
                if (g > 0) {  // dV(g-1) has consumed P^T(g-1): its columns can be rewritten
                    if (!mbar_wait(&p_free[(g - 1) % Cfg::kDOStages], ((g - 1) / Cfg::kDOStages) & 1, ctx, 52)) return false;
                    tc_fence_after_sync();
                }
            }
            publish_p(pk_cur);
            if (trace_me) GQA_TRACE(0, g - 1, 3);
            return true;
        };
        // dV and scale*dK of this key row of work item wi (its j-th of this block), a quarter of the columns per warpgroup
        auto epilogue = [&](int jj) -> bool {
            // read and decoded again here (the slot is still valid): nothing of it stays live across the loop over the tile pairs
            const WorkItem wi = decode(item_slot[jj & (kItemSlots - 1)]);
            if (trace_me) GQA_MARK(4);
            if (!mbar_wait(acc_full, jj & 1, ctx, 55)) return false;
            if (trace_me) GQA_MARK(5);
            tc_fence_after_sync();
            // key rows beyond the end of the sequence are not stored (the TMEM loads below are warp-wide
            // instructions: every lane runs them, only the stores are guarded)
            const bool row_ok = wi.kt * kTile + j < wi.len;
            constexpr int kQuarter = D / Cfg::kEwGroups;  // columns of dV / dK per warpgroup
            // element offset of this key row in dK / dV
            const size_t kv_pos = (size_t)wi.y0 + wi.kt * kTile + j;
            const size_t kv_elem = p.bshd ? (((size_t)wi.b * p.S + kv_pos) * p.Hkv + wi.hkv) * D
                                          : (((size_t)wi.b * p.Hkv + wi.hkv) * p.S + kv_pos) * p.d_real;
#pragma unroll 1
            for (int which = 0; which < 2; ++which) {
                const uint32_t tA = tmem + lane_addr + (which == 0 ? Cfg::kColDV : Cfg::kColDK) + w * kQuarter;
                __nv_bfloat16* dst = (which == 0 ? p.dV : p.dK) + kv_elem + w * kQuarter;
                // head split: fp32 sums of this part, [part][which][key row in [B,Hkv,S] order][D]
                float* pdst = p.parts > 1 ? p.partial + (((size_t)(wi.part * 2 + which) * ((size_t)p.groups * p.S)) +
                                                         (size_t)wi.grp * p.S + kv_pos) * D + w * kQuarter
                                          : nullptr;
                const float mul = which == 0 ? 1.0f : p.scale;
#pragma unroll
                for (int ch = 0; ch < kQuarter / 16; ++ch) {
                    uint32_t v[16];
                    tmem_ld16(tA + ch * 16, v);
                    tmem_wait_ld();
                    if (p.parts > 1) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (row_ok)
                                *reinterpret_cast<float4*>(pdst + ch * 16 + i * 4) =
                                    make_float4(__uint_as_float(v[4 * i + 0]) * mul, __uint_as_float(v[4 * i + 1]) * mul,
                                                __uint_as_float(v[4 * i + 2]) * mul, __uint_as_float(v[4 * i + 3]) * mul);
                        continue;
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * mul, __uint_as_float(v[8 * i + 1]) * mul);
                        o.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * mul, __uint_as_float(v[8 * i + 3]) * mul);
                        o.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * mul, __uint_as_float(v[8 * i + 5]) * mul);
                        o.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * mul, __uint_as_float(v[8 * i + 7]) * mul);
                        if (row_ok && w * kQuarter + ch * 16 + i * 8 < p.d_real) *reinterpret_cast<uint4*>(dst + ch * 16 + i * 8) = o;
                    }
                }
            }
            // every accumulator value is in registers or on its way to memory: the next item's products may overwrite them
            tc_fence_before_sync();
            mbar_arrive(acc_empty);
            return true;
        };

        int gi = 0;  // iteration index over all items of this block
        for (int jj = 0; ok; ++jj) {
            int n_iter, n_qt;
            int qi = 0;  // position of the tile pair's query tile in its head: 0 is the diagonal tile when causal, n_qt - 1
                         // the sequence's last (possibly partial) one; the loop starts at the item's rotation
            int kv_valid = kTile, q_tail = kTile;  // packed batches: key rows of the KV tile / query rows of the
                                                   // sequence's last query tile that belong to the sequence
            {
                const int idx = fetch_item(jj);
                if (idx < 0) break;
                const WorkItem wi = decode(idx);
                n_iter = wi.n_iter;
                n_qt = wi.n_qt;
                qi = wi.shift;
                if constexpr (kVarlen) {
                    kv_valid = wi.len - wi.kt * kTile;
                    q_tail = wi.len - (wi.qt0 + wi.n_qt - 1) * kTile;
                }
                if (warp == kWarpEw0 && lane == 0) GQA_ITEM_BEGIN(idx);
            }
            // One pass per tile pair: P^T(it) from S^T(it), then dS^T(it) from dP^T(it) and the P^T(it) kept in registers.
            // (One copy of each phase in the instruction stream: this loop is the bulk of the kernel's code, and the
            // roles of an SM already miss in the instruction cache.)
            for (int it = 0; it < n_iter && ok; ++it, ++gi) {
                ok = make_p(gi, p.causal && qi == 0, qi == n_qt - 1 ? q_tail : kTile, kv_valid);
                if (++qi == n_qt) qi = 0;
                if (!ok) break;
                ok = mbar_wait(&dp_full[gi % Cfg::kDOStages], (gi / Cfg::kDOStages) & 1, ctx, 53);
                if (ok && gi > 0) ok = mbar_wait(ds_free, (gi - 1) & 1, ctx, 54);  // dK and dQ of the iteration before have read its dS^T
                if (!ok) break;
                tc_fence_after_sync();
                if (trace_me) GQA_TRACE(0, gi, 0);
                {
                    uint32_t dsp[C / 2];
#pragma unroll
                    for (int hf = 0; hf < H; ++hf) {
                        uint32_t vd[16];
                        tmem_ld16(tDP + hf * 16, vd);
                        tmem_wait_ld();
                        ds_half(vd, hf, pk_cur + hf * 8, dsp + hf * 8, ds_row0);
                    }
                    if constexpr (Cfg::kDsInTmem) {
                        static_assert(!Cfg::kDsInTmem || C == 32, "the TMEM copy of dS^T is written as one 16-column store");
                        uint32_t t16[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) t16[i] = dsp[i];
                        tmem_st16(tDP, t16);  // over this thread's own, already consumed, dP^T columns
                        tmem_wait_st();
                    }
                }
                if constexpr (kWithDQ || !Cfg::kDsInTmem) fence_proxy_async_smem();
                tc_fence_before_sync();
                mbar_arrive(ds_ready);
                if (trace_me) GQA_TRACE(0, gi, 1);
            }
            // ---- epilogue, before the next item's first P^T: the issuers need the accumulators back for its products
            if (ok) ok = epilogue(jj);
            if (warp == kWarpEw0 && lane == 0) GQA_ITEM_END(item_slot[jj & (kItemSlots - 1)]);
        }
    }

    // ---- teardown ---------------------------------------------------------------
    if (warp == kWarpEw0) GQA_MARK(6);
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) GQA_MARK(9);
    if (warp == Cfg::kWarpMmaS) {
        if (*abort_flag != 0) abort_grace_period();  // in-flight copies and MMAs land before TMEM is released
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

// Thread blocks of the main kernel that run at the same time: one per SM (shared memory and TMEM allow no second).
int resident_blocks() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    if (dev != cached_dev) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) return 1;
        cached = sms;
        cached_dev = dev;
    }
    return cached;
}

// Causal order: how many (batch, KV head) groups form a super-group (the list runs super-group by super-group, KV
// tile by KV tile inside, longest items first).  Few groups at a time means many KV tiles of the same group in
// flight together, all streaming that group's Q/dO tiles through L2 at nearly the same time, so HBM is read fewer
// times (measured: 7 % at B4 Hq32 Hkv8 S8192 D128, 3 % at the headline shape with a causal mask, 2 % at S = 32768).
// The bound keeps the end of the launch balanced: a super-group must last about as long as its longest item
// (n_tiles tile pairs per head against sg * n_tiles * (n_tiles + 1) / 2 spread over the SMs), or the long items of
// the last super-group would start too late for the others to level them out.
int causal_super_group(int groups, int n_tiles, int sms) {
    const int bound = (2 * sms + n_tiles) / (n_tiles + 1);  // ceil(2 * sms / (n_tiles + 1))
    for (int d = 1; d <= groups; ++d)
        if (groups % d == 0 && d >= bound) return d;
    return groups;
}

// dq_accum == nullptr selects the variant without the dQ part.
template <int D>
int launch_bwd_t(const void* Q, const void* K, const void* V, const void* dO, const void* lse_cols,
                 const void* delta_cols, float* dq_accum, unsigned int* dq_turn, void* dK, void* dV, const Shape& s,
                 unsigned int* status, int parts, float* partial, cudaStream_t stream) {
    using Cfg = BwdCfg<D>;
    CUtensorMap mq, mk, mv, mdo;
    // see the coordinates in the kernel
    // (the matrices are s.D columns wide; a box that reaches beyond them reads zeros there)
    const uint64_t S = s.S, qc = s.bshd ? (uint64_t)s.Hq * D : s.D, kc = s.bshd ? (uint64_t)s.Hkv * D : s.D;
    const uint64_t nq = s.bshd ? s.B : (uint64_t)s.B * s.Hq, nkv = s.bshd ? s.B : (uint64_t)s.B * s.Hkv;
    const uint64_t nws = (uint64_t)s.B * s.Hq;
    int rc = make_tile3_tmap(&mq, Q, qc, S, nq, S * qc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mk, K, kc, S, nkv, S * kc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mv, V, kc, S, nkv, S * kc, kTile);
    if (rc) return rc;
    rc = make_tile3_tmap(&mdo, dO, qc, S, nq, S * qc, kTile);
    if (rc) return rc;
    CUtensorMap mlse, mdlt;
    rc = make_col8_3_tmap(&mlse, lse_cols, S, nws, kTile);
    if (rc) return rc;
    rc = make_col8_3_tmap(&mdlt, delta_cols, S, nws, kTile);
    if (rc) return rc;
    CUtensorMap mdq = mlse;  // unused without the dQ part
    if (dq_accum) {
        rc = make_f32box3_tmap(&mdq, dq_accum, D, S, nws, 32);
        if (rc) return rc;
    }
    const bool varlen = s.cu_seqlens != nullptr;
    if (varlen && (!dq_accum || dq_turn || parts != 1 || !s.bshd || s.B != 1)) return GQA_ERR_BAD_ARGUMENT;
    auto kernel = varlen     ? gqa_bwd_sm100_kernel<D, true, true>
                  : dq_accum ? gqa_bwd_sm100_kernel<D, true, false>
                             : gqa_bwd_sm100_kernel<D, false, false>;
    GQA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemTotal));
    BwdParams p;
    p.dq_accum = dq_accum;
    p.dK = static_cast<__nv_bfloat16*>(dK);
    p.dV = static_cast<__nv_bfloat16*>(dV);
    p.status = status;
    p.dq_turn = dq_turn;
    p.partial = partial;
    p.parts = parts;
    p.Hq = s.Hq;
    p.Hkv = s.Hkv;
    p.S = s.S;
    p.causal = s.causal;
    p.bshd = s.bshd;
    p.d_real = s.D;
    p.cu = s.cu_seqlens;
    // packed batch: the item list is laid out for max_seqlen; the kernel skips what lies beyond a sequence
    p.n_tiles = ((varlen ? s.max_seqlen : s.S) + kTile - 1) / kTile;
    p.G = s.G();
    p.scale = s.scale;
    p.scale_log2 = s.scale * 1.4426950408889634f;
    p.groups = (varlen ? s.n_seqs : s.B) * s.Hkv;
    p.sg = dq_turn ? p.groups : causal_super_group(p.groups, p.n_tiles, resident_blocks());
    p.n_items = p.n_tiles * p.groups * parts;
    // persistent, except in the deterministic mode (see the work-item comment in the kernel)
    const unsigned grid = (unsigned)(dq_turn ? p.n_items : std::min(p.n_items, resident_blocks()));
    kernel<<<grid, Cfg::kThreads, Cfg::kSmemTotal, stream>>>(mq, mk, mv, mdo, mdq, mlse, mdlt, p);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

}  // namespace

#ifdef GQA_BWD_TRACE
extern "C" int gqa_debug_copy_bwd_trace(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, g_bwd_trace, sizeof(g_bwd_trace));
}
extern "C" int gqa_debug_copy_bwd_items(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, g_bwd_items, sizeof(g_bwd_items));
}
extern "C" int gqa_debug_copy_bwd_marks(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, g_bwd_marks, sizeof(g_bwd_marks));
}
#endif

int launch_bwd_main_sm100(const void* Q, const void* K, const void* V, const void* dO, const void* lse_cols,
                          const void* delta_cols, float* dq_accum, unsigned int* dq_turn, void* dK, void* dV,
                          const Shape& s, unsigned int* status, int parts, float* partial, cudaStream_t stream) {
    if (parts < 1 || s.G() % parts != 0 || (parts > 1 && !partial)) return GQA_ERR_BAD_ARGUMENT;
    if (s.Dp() == 64)
        return launch_bwd_t<64>(Q, K, V, dO, lse_cols, delta_cols, dq_accum, dq_turn, dK, dV, s, status, parts, partial,
                                stream);
    return launch_bwd_t<128>(Q, K, V, dO, lse_cols, delta_cols, dq_accum, dq_turn, dK, dV, s, status, parts, partial,
                             stream);
}

}  // namespace gqa
