// CUDA-core checker kernels: a deliberately simple restatement of the attention
// forward and backward on the GPU (one block per row, fp32 math on bf16 inputs).
// They exist so that the tensor-core kernels can be cross-checked on the device at
// sizes where the CPU oracle takes too long; they are not a product path and no
// product entry point dispatches to them.
//
// Math follows the reference's per-head loops (precision/baseline_gqa.py:169-197):
//   p = exp(scale*q.k - LSE), dp = dO.v, ds = p*(dp - Delta),
//   dq = scale*ds k, dk = scale*ds^T q, dv = p^T dO, summed over the G heads of a group.
#include "gqa_common.cuh"
#include "gqa_kernels.cuh"

namespace gqa {
namespace {

constexpr int kThreads = 128;

__device__ __forceinline__ float bf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

__device__ float block_reduce(float v, bool is_max, float* scratch) {
    for (int o = 16; o > 0; o >>= 1) {
        float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, w) : v + w;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch[0];
    for (int w = 1; w < kThreads / 32; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
    return r;
}

// grid = B*Hq*S blocks, one query row each; dynamic smem = S floats.
__global__ void __launch_bounds__(kThreads)
fwd_simt_kernel(const __nv_bfloat16* Q, const __nv_bfloat16* K, const __nv_bfloat16* V, __nv_bfloat16* O, float* LSE,
                int Hq, int Hkv, int S, int D, int causal, float scale) {
    extern __shared__ float sc[];
    __shared__ float red[kThreads / 32];
    __shared__ float qrow[128];
    const size_t row = blockIdx.x;
    const int i = (int)(row % S);
    const int hq = (int)((row / S) % Hq);
    const int b = (int)(row / ((size_t)S * Hq));
    const int hkv = hq / (Hq / Hkv);
    const __nv_bfloat16* kb = K + ((size_t)b * Hkv + hkv) * S * D;
    const __nv_bfloat16* vb = V + ((size_t)b * Hkv + hkv) * S * D;
    for (int d = threadIdx.x; d < D; d += kThreads) qrow[d] = bf(Q, row * D + d);
    __syncthreads();
    const int n = causal ? i + 1 : S;
    float m = -INFINITY;
    for (int j = threadIdx.x; j < n; j += kThreads) {
        float s = 0.f;
        for (int d = 0; d < D; ++d) s = fmaf(qrow[d], bf(kb, (size_t)j * D + d), s);
        s *= scale;
        sc[j] = s;
        m = fmaxf(m, s);
    }
    m = block_reduce(m, true, red);
    float l = 0.f;
    for (int j = threadIdx.x; j < n; j += kThreads) {
        const float e = expf(sc[j] - m);
        sc[j] = e;
        l += e;
    }
    l = block_reduce(l, false, red);
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += kThreads) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) acc = fmaf(sc[j], bf(vb, (size_t)j * D + d), acc);
        O[row * D + d] = __float2bfloat16(acc / l);
    }
    if (threadIdx.x == 0 && LSE) LSE[row] = m + logf(l);
}

// grid = B*Hq*S blocks, one query row each: dQ.
__global__ void __launch_bounds__(kThreads)
bwd_dq_simt_kernel(const __nv_bfloat16* Q, const __nv_bfloat16* K, const __nv_bfloat16* V, const __nv_bfloat16* dO,
                   const float* LSE, const float* delta, __nv_bfloat16* dQ, int Hq, int Hkv, int S, int D, int causal,
                   float scale) {
    extern __shared__ float ds[];
    __shared__ float qrow[128], dorow[128];
    const size_t row = blockIdx.x;
    const int i = (int)(row % S);
    const int hq = (int)((row / S) % Hq);
    const int b = (int)(row / ((size_t)S * Hq));
    const int hkv = hq / (Hq / Hkv);
    const __nv_bfloat16* kb = K + ((size_t)b * Hkv + hkv) * S * D;
    const __nv_bfloat16* vb = V + ((size_t)b * Hkv + hkv) * S * D;
    for (int d = threadIdx.x; d < D; d += kThreads) {
        qrow[d] = bf(Q, row * D + d);
        dorow[d] = bf(dO, row * D + d);
    }
    __syncthreads();
    const int n = causal ? i + 1 : S;
    const float lse = LSE[row], dl = delta[row];
    for (int j = threadIdx.x; j < n; j += kThreads) {
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < D; ++d) {
            s = fmaf(qrow[d], bf(kb, (size_t)j * D + d), s);
            dp = fmaf(dorow[d], bf(vb, (size_t)j * D + d), dp);
        }
        const float p = expf(s * scale - lse);
        ds[j] = p * (dp - dl);
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += kThreads) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) acc = fmaf(ds[j], bf(kb, (size_t)j * D + d), acc);
        dQ[row * D + d] = __float2bfloat16(acc * scale);
    }
}

// grid = B*Hkv*S blocks, one key row each: dK and dV, summed over the G heads in order.
// dynamic smem = 2*S floats (p and ds of the current head).
__global__ void __launch_bounds__(kThreads)
bwd_dkdv_simt_kernel(const __nv_bfloat16* Q, const __nv_bfloat16* K, const __nv_bfloat16* V, const __nv_bfloat16* dO,
                     const float* LSE, const float* delta, __nv_bfloat16* dK, __nv_bfloat16* dV, int Hq, int Hkv,
                     int S, int D, int causal, float scale) {
    extern __shared__ float buf[];
    float* ps = buf;
    float* dss = buf + S;
    __shared__ float krow[128], vrow[128];
    const size_t row = blockIdx.x;
    const int j = (int)(row % S);
    const int hkv = (int)((row / S) % Hkv);
    const int b = (int)(row / ((size_t)S * Hkv));
    const int G = Hq / Hkv;
    for (int d = threadIdx.x; d < D; d += kThreads) {
        krow[d] = bf(K, row * D + d);
        vrow[d] = bf(V, row * D + d);
    }
    float dk_acc = 0.f, dv_acc = 0.f;  // thread d owns column d (D <= 128 = kThreads)
    const int i0 = causal ? j : 0;
    for (int g = 0; g < G; ++g) {
        const int hq = hkv * G + g;
        const size_t qbase = ((size_t)b * Hq + hq) * S;
        __syncthreads();
        for (int i = i0 + threadIdx.x; i < S; i += kThreads) {
            float s = 0.f, dp = 0.f;
            for (int d = 0; d < D; ++d) {
                s = fmaf(bf(Q, (qbase + i) * D + d), krow[d], s);
                dp = fmaf(bf(dO, (qbase + i) * D + d), vrow[d], dp);
            }
            const float p = expf(s * scale - LSE[qbase + i]);
            ps[i] = p;
            dss[i] = p * (dp - delta[qbase + i]);
        }
        __syncthreads();
        if (threadIdx.x < D) {
            const int d = threadIdx.x;
            for (int i = i0; i < S; ++i) {
                dv_acc = fmaf(ps[i], bf(dO, (qbase + i) * D + d), dv_acc);
                dk_acc = fmaf(dss[i], bf(Q, (qbase + i) * D + d), dk_acc);
            }
        }
    }
    if (threadIdx.x < D) {
        dK[row * D + threadIdx.x] = __float2bfloat16(dk_acc * scale);
        dV[row * D + threadIdx.x] = __float2bfloat16(dv_acc);
    }
}

}  // namespace

int launch_fwd_simt(const void* Q, const void* K, const void* V, void* O, float* LSE, const Shape& s,
                    cudaStream_t stream) {
    const size_t smem = (size_t)s.S * sizeof(float);
    if (smem > 200 * 1024) return GQA_ERR_UNSUPPORTED;
    GQA_CUDA_TRY(cudaFuncSetAttribute(fwd_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    fwd_simt_kernel<<<(unsigned)s.q_rows(), kThreads, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(Q), static_cast<const __nv_bfloat16*>(K), static_cast<const __nv_bfloat16*>(V),
        static_cast<__nv_bfloat16*>(O), LSE, s.Hq, s.Hkv, s.S, s.D, s.causal, s.scale);
    count_launch();
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

int launch_bwd_simt(const void* Q, const void* K, const void* V, const void* dO, const float* LSE, const float* delta,
                    void* dQ, void* dK, void* dV, const Shape& s, cudaStream_t stream) {
    const size_t smem1 = (size_t)s.S * sizeof(float), smem2 = 2 * smem1;
    if (smem2 > 200 * 1024) return GQA_ERR_UNSUPPORTED;
    GQA_CUDA_TRY(cudaFuncSetAttribute(bwd_dq_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
    GQA_CUDA_TRY(cudaFuncSetAttribute(bwd_dkdv_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    auto q = static_cast<const __nv_bfloat16*>(Q);
    auto k = static_cast<const __nv_bfloat16*>(K);
    auto v = static_cast<const __nv_bfloat16*>(V);
    auto d_o = static_cast<const __nv_bfloat16*>(dO);
    bwd_dq_simt_kernel<<<(unsigned)s.q_rows(), kThreads, smem1, stream>>>(
        q, k, v, d_o, LSE, delta, static_cast<__nv_bfloat16*>(dQ), s.Hq, s.Hkv, s.S, s.D, s.causal, s.scale);
    bwd_dkdv_simt_kernel<<<(unsigned)s.kv_rows(), kThreads, smem2, stream>>>(
        q, k, v, d_o, LSE, delta, static_cast<__nv_bfloat16*>(dK), static_cast<__nv_bfloat16*>(dV), s.Hq, s.Hkv, s.S,
        s.D, s.causal, s.scale);
    count_launch(2);
    GQA_CUDA_TRY(cudaGetLastError());
    return GQA_OK;
}

}  // namespace gqa
