// Internal launcher declarations (one per kernel role).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace gqa {

struct Shape {
    int B, Hq, Hkv, S, D, causal;
    float scale;
    // 0: Q,O,dO,dQ [B,Hq,S,D] and K,V,dK,dV [B,Hkv,S,D] (the reference's layout); 1: [B,S,H,D] for all of them.
    // LSE and the workspace arrays are always in [B,Hq,S] row order.
    int bshd = 0;
    // Variable-length batch (packed): B = 1, S = the total number of tokens, bshd = 1, i.e. Q [T,Hq,D], K/V [T,Hkv,D],
    // LSE [Hq,T]; sequence i owns the rows cu_seqlens[i] .. cu_seqlens[i+1]-1 (n_seqs + 1 int32 in device memory)
    // and attends only to itself; max_seqlen bounds every length (it sizes the grid).
    const int* cu_seqlens = nullptr;
    int n_seqs = 0, max_seqlen = 0;
    int G() const { return Hq / Hkv; }
    // Head dimensions other than 64 and 128 run on the kernel of the next size up: the tensor maps describe the real
    // D columns, the 64-column boxes read zeros beyond them (out-of-bounds fill), zero columns add nothing to any
    // product, and the epilogues store only the real columns.
    int Dp() const { return D <= 64 ? 64 : 128; }
    size_t q_rows() const { return (size_t)B * Hq * S; }
    size_t kv_rows() const { return (size_t)B * Hkv * S; }
};

// Workspace carve-up for the backward (offsets in bytes, 256-byte aligned).
struct BwdWorkspace {
    // lse_cols / delta_cols: per query row eight bf16 (16 bytes): a three-way bf16 split of -LSE/scale and of
    // -Delta in the first three, zeros after; they enter the S^T and dP^T products as one extra K step.
    // dq_turn: one counter per 32-row slice of a query tile, used only by the deterministic mode (order of the dQ
    // reductions).
    // delta_f32: Delta as fp32, one per query row, for the separate dQ pass (which subtracts it in registers).
    size_t status_off, lse_cols_off, delta_cols_off, delta_f32_off, dq_turn_off, dq_turn_bytes, dq_accum_off, partial_off,
        partial_bytes, total;
    explicit BwdWorkspace(const Shape& s, int parts = 1) {
        auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
        status_off = 0;
        lse_cols_off = 256;
        delta_cols_off = lse_cols_off + up(s.q_rows() * 16);
        delta_f32_off = delta_cols_off + up(s.q_rows() * 16);
        dq_turn_off = delta_f32_off + up(s.q_rows() * sizeof(float));
        dq_turn_bytes = (size_t)s.B * s.Hq * ((s.S + 127) / 128) * 4 * sizeof(unsigned int);  // per tile and drain warp
        dq_accum_off = dq_turn_off + up(dq_turn_bytes);
        partial_off = dq_accum_off + up(s.q_rows() * (size_t)s.Dp() * sizeof(float));  // accumulator rows are Dp wide
        // head split: [part][dV, dK][key rows][Dp] fp32
        partial_bytes = parts > 1 ? up((size_t)parts * 2 * s.kv_rows() * s.Dp() * sizeof(float)) : 0;
        total = partial_off + partial_bytes;
    }
};

// Stage 1 of the backward: Delta = rowsum(dO*O); with `delta` it is stored as fp32, with the column arrays
// the bf16 splits of -LSE*inv_scale and -Delta are stored (16 bytes per row each) and, if given, the dQ
// accumulator is zeroed.
// `S_bshd` / `H_bshd`: 0 when O, dO are in [B,H,S,D] order, else S and Hq of the [B,S,H,D] layout they are in.
int launch_bwd_preprocess(const void* O, const void* dO, const float* lse, float inv_scale, float* delta,
                          void* lse_cols, void* delta_cols, float* dq_accum, size_t rows, int D, cudaStream_t stream,
                          int S_bshd = 0, int H_bshd = 0);
// Stage 3 of the backward: dQ = bf16(scale * dq_accum) (dQ in [B,S,H,D] order when S_bshd / H_bshd are given).
// `rows` rows of Dp fp32 accumulator columns -> rows of D bf16 columns.
int launch_dq_finalise(const float* dq_accum, void* dQ, size_t rows, float scale, cudaStream_t stream,
                       int D, int S_bshd = 0, int H_bshd = 0);

// Tensor-core forward (tcgen05 + TMEM + TMA).
int launch_fwd_sm100(const void* Q, const void* K, const void* V, void* O, float* LSE, const Shape& s,
                     unsigned int* status, cudaStream_t stream);
// Stage 2 of the backward: KV-tile-parallel main kernel (tcgen05 + TMEM + TMA); dK/dV written
// once per element, dQ accumulated into dq_accum with fp32 reductions.
// With dq_turn (zeroed counters, one per 32 query rows) the reductions of every dQ tile are applied in KV-tile
// order, which makes dQ bit-reproducible; nullptr = unordered.  dq_accum == nullptr launches the variant without the
// dQ part (dK and dV only), for use with launch_bwd_dq_sm100.
// With parts > 1 (a divisor of G) every KV tile is handled by `parts` thread blocks over disjoint query heads; their
// fp32 dK / dV sums go to `partial` (BwdWorkspace::partial_bytes) and launch_dkdv_reduce adds them in a fixed order.
int launch_bwd_main_sm100(const void* Q, const void* K, const void* V, const void* dO, const void* lse_cols,
                          const void* delta_cols, float* dq_accum, unsigned int* dq_turn, void* dK, void* dV,
                          const Shape& s, unsigned int* status, int parts, float* partial, cudaStream_t stream);
// The alternative dQ path: a separate query-parallel pass that recomputes S and dP and writes dQ once (no accumulator,
// no finalise, bit-reproducible).  `delta` is rowsum(dO * O) as fp32 per query row.
int launch_bwd_dq_sm100(const void* Q, const void* K, const void* V, const void* dO, const float* lse,
                        const float* delta, void* dQ, const Shape& s, unsigned int* status, cudaStream_t stream);
// dK, dV = bf16(sum over the parts of the fp32 partial sums), in part order: the counterpart of gqa_dkdv_greduce
// (src/attention/GQA_bwd_baseline.cu:385-403), on fp32 partials and only when the head split is in use.
int launch_dkdv_reduce(const float* partial, void* dK, void* dV, const Shape& s, int parts, cudaStream_t stream);
// How many thread blocks share a KV tile for this shape (1 = no split): a pure function of the shape, so that the
// workspace query and the launch agree.
int bwd_head_parts(const Shape& s);

// CUDA-core checker kernels (slow, simple; fp32 math on bf16 inputs).
int launch_fwd_simt(const void* Q, const void* K, const void* V, void* O, float* LSE, const Shape& s,
                    cudaStream_t stream);
int launch_bwd_simt(const void* Q, const void* K, const void* V, const void* dO, const float* LSE, const float* delta,
                    void* dQ, void* dK, void* dV, const Shape& s, cudaStream_t stream);

}  // namespace gqa
