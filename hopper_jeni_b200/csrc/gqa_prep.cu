// Memory-bound helper kernels around the tensor-core backward:
//   * preprocess: Delta = rowsum(dO * O), the bf16 column splits of -LSE/scale and -Delta that the
//     main kernel folds into its S^T and dP^T products, and zeroing of the fp32 dQ accumulator, in
//     one pass (stage 1 of the backward);
//   * finalise:   dQ = bf16(scale * dq_accum) (stage 3).
// Algorithmic traffic per query row (D bf16 elements): preprocess reads 2*D*2 B and writes
// D*4 + 32 B; finalise reads D*4 B and writes D*2 B.
#include <algorithm>
#include <functional>
#include <queue>
#include <vector>

#include "gqa_common.cuh"
#include "gqa_kernels.cuh"

namespace gqa {

namespace {

// x as hi + mid + lo with each part a bf16: exact to about 2^-24 relative; returned as {hi|mid<<16, lo}.
__device__ __forceinline__ uint2 split3_bf16(float x) {
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    return make_uint2((uint32_t)__bfloat16_as_ushort(hi) | ((uint32_t)__bfloat16_as_ushort(mid) << 16),
                      (uint32_t)__bfloat16_as_ushort(lo));
}

// One group of D/8 lanes per row; each lane owns 8 consecutive elements (one 16-byte load
// from O and one from dO).  A warp covers 256/D rows per step.  D is the padded head dimension (64 or 128, the
// width of an accumulator row); O and dO rows hold `d_real` <= D columns.
template <int D>
__global__ void __launch_bounds__(256)
bwd_preprocess_kernel(const uint4* __restrict__ O, const uint4* __restrict__ dO, const float* __restrict__ lse,
                      float inv_scale, float* __restrict__ delta, uint4* __restrict__ lse_cols,
                      uint4* __restrict__ delta_cols, float4* __restrict__ dq_accum, size_t rows, int S_bshd, int H_bshd,
                      int d_real) {
    constexpr int kLanesPerRow = D / 8;
    const int real8 = d_real / 8;  // 16-byte groups per O / dO row
    constexpr int kRowsPerWarp = 32 / kLanesPerRow;
    const int lane = threadIdx.x & 31;
    const size_t warp_global = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t n_warps = (size_t)gridDim.x * (blockDim.x >> 5);
    const int sub = lane / kLanesPerRow, part = lane % kLanesPerRow;
    for (size_t base = warp_global * kRowsPerWarp; base < rows; base += n_warps * kRowsPerWarp) {
        const size_t row = base + sub;
        float acc = 0.f;
        if (row < rows) {
            // `row` counts in [B,H,S] order (LSE, Delta, accumulator); O and dO may be stored [B,S,H,D]
            size_t src = row;
            if (S_bshd) {
                const size_t s_ = row % S_bshd, bh = row / S_bshd;
                src = ((bh / H_bshd) * S_bshd + s_) * H_bshd + bh % H_bshd;
            }
            const bool in_row = part < real8;
            const uint4 a = in_row ? O[src * real8 + part] : make_uint4(0u, 0u, 0u, 0u);
            const uint4 b = in_row ? dO[src * real8 + part] : make_uint4(0u, 0u, 0u, 0u);
            const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc = fmaf(__uint_as_float(av[i] << 16), __uint_as_float(bv[i] << 16), acc);
                acc = fmaf(__uint_as_float(av[i] & 0xffff0000u), __uint_as_float(bv[i] & 0xffff0000u), acc);
            }
            if (dq_accum) {
                const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                dq_accum[(row * kLanesPerRow + part) * 2 + 0] = z;
                dq_accum[(row * kLanesPerRow + part) * 2 + 1] = z;
            }
        }
#pragma unroll
        for (int off = kLanesPerRow / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (row < rows && part == 0) {
            if (delta) delta[row] = acc;
            if (lse_cols) {
                const uint2 l = split3_bf16(-lse[row] * inv_scale), d = split3_bf16(-acc);
                lse_cols[row] = make_uint4(l.x, l.y, 0u, 0u);
                delta_cols[row] = make_uint4(d.x, d.y, 0u, 0u);
            }
        }
    }
}

// n8 groups of eight output elements; per8 = D / 8 groups per dQ row, acc8 = groups per accumulator row (the padded
// head dimension / 8).  The accumulator is in [B,H,S] row order, dQ may be stored [B,S,H,D] (S_bshd, H_bshd non-zero).
__global__ void __launch_bounds__(256)
dq_finalise_kernel(const float4* __restrict__ acc, uint4* __restrict__ dq, size_t n8, float scale, int per8, int acc8,
                   int S_bshd, int H_bshd) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t src = (i / per8) * acc8 + i % per8;
        const float4 a = acc[2 * src], b = acc[2 * src + 1];
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x * scale, a.y * scale);
        __nv_bfloat162 p1 = __floats2bfloat162_rn(a.z * scale, a.w * scale);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x * scale, b.y * scale);
        __nv_bfloat162 p3 = __floats2bfloat162_rn(b.z * scale, b.w * scale);
        uint4 o;
        o.x = *reinterpret_cast<uint32_t*>(&p0);
        o.y = *reinterpret_cast<uint32_t*>(&p1);
        o.z = *reinterpret_cast<uint32_t*>(&p2);
        o.w = *reinterpret_cast<uint32_t*>(&p3);
        size_t dst = i;
        if (S_bshd) {
            const size_t row = i / per8, s_ = row % S_bshd, bh = row / S_bshd;
            dst = (((bh / H_bshd) * S_bshd + s_) * H_bshd + bh % H_bshd) * per8 + i % per8;
        }
        dq[dst] = o;
    }
}

// out = bf16(sum over the parts, in part order, of the fp32 partial sums); n8 groups of eight output elements,
// per8 = D / 8 groups per output row, acc8 = groups per partial row, part_stride8 = groups between two parts' copies of
// one tensor.
__global__ void __launch_bounds__(256)
dkdv_reduce_kernel(const float4* __restrict__ partial, uint4* __restrict__ out, size_t n8, int per8, int acc8, int parts,
                   size_t part_stride8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t src = (i / per8) * acc8 + i % per8;
        float4 a = partial[2 * src], b = partial[2 * src + 1];
        for (int p = 1; p < parts; ++p) {
            const float4 c = partial[2 * (src + p * part_stride8)], d = partial[2 * (src + p * part_stride8) + 1];
            a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
            b.x += d.x; b.y += d.y; b.z += d.z; b.w += d.w;
        }
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
        uint4 o;
        o.x = *reinterpret_cast<uint32_t*>(&p0);
        o.y = *reinterpret_cast<uint32_t*>(&p1);
        o.z = *reinterpret_cast<uint32_t*>(&p2);
        o.w = *reinterpret_cast<uint32_t*>(&p3);
        out[i] = o;
    }
}

int grid_for(size_t work_items, int per_block) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t want = (work_items + per_block - 1) / per_block;
    size_t cap = (size_t)sms * 16;  // a multiple of the SM count; grid-stride loops cover the rest
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    return (int)want;
}

}  // namespace

int launch_bwd_preprocess(const void* O, const void* dO, const float* lse, float inv_scale, float* delta,
                          void* lse_cols, void* delta_cols, float* dq_accum, size_t rows, int D, cudaStream_t stream,
                          int S_bshd, int H_bshd) {
    const int Dp = D <= 64 ? 64 : 128;
    const int rows_per_block = (256 / 32) * (256 / Dp);
    const int grid = grid_for(rows, rows_per_block);
    if (Dp == 64)
        bwd_preprocess_kernel<64><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(O), static_cast<const uint4*>(dO),
                                                            lse, inv_scale, delta, static_cast<uint4*>(lse_cols),
                                                            static_cast<uint4*>(delta_cols),
                                                            reinterpret_cast<float4*>(dq_accum), rows, S_bshd, H_bshd, D);
    else
        bwd_preprocess_kernel<128><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(O), static_cast<const uint4*>(dO),
                                                             lse, inv_scale, delta, static_cast<uint4*>(lse_cols),
                                                            static_cast<uint4*>(delta_cols),
                                                            reinterpret_cast<float4*>(dq_accum), rows, S_bshd, H_bshd, D);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

int launch_dq_finalise(const float* dq_accum, void* dQ, size_t rows, float scale, cudaStream_t stream, int D,
                       int S_bshd, int H_bshd) {
    const size_t n8 = rows * (size_t)(D / 8);
    const int grid = grid_for(n8, 256);
    dq_finalise_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(dq_accum), static_cast<uint4*>(dQ), n8,
                                                 scale, D / 8, (D <= 64 ? 64 : 128) / 8, S_bshd, H_bshd);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

int launch_dkdv_reduce(const float* partial, void* dK, void* dV, const Shape& s, int parts, cudaStream_t stream) {
    const size_t rows = s.kv_rows(), n8 = rows * (size_t)(s.D / 8);
    const int acc8 = s.Dp() / 8;
    const size_t tensor_stride8 = rows * acc8;  // [part][dV, dK][rows][Dp]: the two tensors of a part are neighbours
    const int grid = grid_for(n8, 256);
    for (int which = 0; which < 2; ++which) {
        dkdv_reduce_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(partial) + 2 * which * tensor_stride8,
                                                     static_cast<uint4*>(which == 0 ? dV : dK), n8, s.D / 8, acc8, parts,
                                                     2 * tensor_stride8);
        count_launch();
    }
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

int bwd_head_parts(const Shape& s) {
    constexpr int kSms = 148;  // the library is sm_100a-only: B200
    const int G = s.G(), n_tiles = (s.S + 127) / 128;
    const long items = (long)n_tiles * s.B * s.Hkv;
    if (G == 1 || s.bshd || items >= 2 * kSms) return 1;
    // This runs on the host in front of every call that passes the flag: the answer for the last shape is kept.
    static thread_local int memo_key[6] = {-1, -1, -1, -1, -1, -1}, memo_parts = 1;
    const int key[6] = {s.B, s.Hq, s.Hkv, s.S, s.D, s.causal};
    if (std::equal(key, key + 6, memo_key)) return memo_parts;
    // Estimated makespan (in tile pairs) of list scheduling, longest item first, on the SMs, for every divisor of G;
    // every item also pays a fixed start/finish cost worth about four tile pairs.  The split is taken only when it
    // shortens the estimate by more than 8 %: the partial sums and their reduction are not free.
    auto makespan = [&](int parts) -> double {
        const int g_local = G / parts;
        const long per_tile = (long)s.B * s.Hkv * parts;  // items of equal length
        if (!s.causal) return (double)((items * parts + kSms - 1) / kSms) * (g_local * n_tiles + 4.0);
        std::priority_queue<double, std::vector<double>, std::greater<double>> load;  // the least loaded SM on top
        for (int i = 0; i < kSms; ++i) load.push(0.0);
        double worst = 0;
        for (int kt = 0; kt < n_tiles; ++kt) {
            const double len = (double)g_local * (n_tiles - kt) + 4.0;
            for (long rep = 0; rep < per_tile; ++rep) {
                const double l = load.top() + len;
                load.pop();
                load.push(l);
                worst = l > worst ? l : worst;
            }
        }
        return worst;
    };
    int best_parts = 1;
    double best = makespan(1);
    for (int parts = 2; parts <= G; ++parts) {
        if (G % parts) continue;
        const double m = makespan(parts);
        if (m < 0.92 * best) {
            best = m;
            best_parts = parts;
        }
    }
    std::copy(key, key + 6, memo_key);
    memo_parts = best_parts;
    return best_parts;
}

}  // namespace gqa

extern "C" int gqa_bwd_delta(const void* O, const void* dO, float* delta, size_t rows, int D, gqa_stream_t stream) {
    if (!O || !dO || !delta || rows == 0) return GQA_ERR_BAD_ARGUMENT;
    if (D < 8 || D > 128 || D % 8 != 0) return GQA_ERR_UNSUPPORTED;
    if (!gqa::aligned16(O) || !gqa::aligned16(dO)) return GQA_ERR_BAD_ARGUMENT;
    return gqa::launch_bwd_preprocess(O, dO, nullptr, 0.f, delta, nullptr, nullptr, nullptr, rows, D,
                                      reinterpret_cast<cudaStream_t>(stream));
}
