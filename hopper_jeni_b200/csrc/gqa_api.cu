// C-ABI entry points: argument validation, workspace carve-up and the launch
// sequence of each operator.  Nothing here allocates device memory.
#include <mutex>

#include "gqa_common.cuh"
#include "gqa_kernels.cuh"

namespace {

using gqa::Shape;

int check_device() {
    static thread_local int cached_dev = -1;
    static thread_local int cached_rc = GQA_OK;
    int dev = 0;
    GQA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev == cached_dev) return cached_rc;
    int major = 0;
    GQA_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    cached_dev = dev;
    cached_rc = (major == 10) ? GQA_OK : GQA_ERR_ARCH;
    return cached_rc;
}

// scale enters as 1/scale (the folded LSE term of the backward) and as the sign convention of the forward's
// running maximum: it must be finite and positive.
bool scale_ok(float scale) { return scale > 0.f && scale < INFINITY; }

int check_shape(int B, int Hq, int Hkv, int S, int D) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || D <= 0) return GQA_ERR_BAD_ARGUMENT;
    if (D < 8 || D > 128 || D % 8 != 0) return GQA_ERR_UNSUPPORTED;  // rows must be multiples of 16 bytes (TMA)
    if (Hq % Hkv != 0) return GQA_ERR_UNSUPPORTED;  // S may be any length: partial tiles are masked
    if ((size_t)B * Hq * S >= (size_t)1 << 31) return GQA_ERR_UNSUPPORTED;  // TMA row coordinate is 32-bit
    return GQA_OK;
}

}  // namespace

namespace {

// A packed variable-length batch as the kernels see it: one [total, H*D] matrix per tensor (B = 1, S = total,
// sequence-major) plus the sequence starts.  Only the two head dimensions with native kernels.
struct Packed {
    const int* cu_seqlens;
    int n_seqs, max_seqlen;
};

int check_packed(const int* cu_seqlens, int n_seqs, int total_tokens, int max_seqlen, int D) {
    if (!cu_seqlens || n_seqs <= 0 || total_tokens <= 0 || max_seqlen <= 0 || max_seqlen > total_tokens)
        return GQA_ERR_BAD_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(cu_seqlens) & 3u) return GQA_ERR_BAD_ARGUMENT;
    if (D != 64 && D != 128) return GQA_ERR_UNSUPPORTED;
    return GQA_OK;
}

int run_fwd(const void* Q, const void* K, const void* V, void* O, float* LSE, int B, int Hq, int Hkv, int S, int D,
            int causal, float scale, cudaStream_t stream, unsigned int flags, const Packed* packed = nullptr) {
    if (flags & ~(unsigned)GQA_LAYOUT_BSHD) return GQA_ERR_BAD_ARGUMENT;
    if (!Q || !K || !V || !O || !scale_ok(scale)) return GQA_ERR_BAD_ARGUMENT;
    int rc = check_shape(B, Hq, Hkv, S, D);
    if (rc) return rc;
    // [B,S,H,D]: a head's columns are followed by the next head's, so nothing reads as zero padding
    if ((flags & GQA_LAYOUT_BSHD) && D != 64 && D != 128) return GQA_ERR_UNSUPPORTED;
    if (!gqa::aligned16(Q) || !gqa::aligned16(K) || !gqa::aligned16(V) || !gqa::aligned16(O) ||
        (LSE && !gqa::aligned16(LSE)))
        return GQA_ERR_BAD_ARGUMENT;
    rc = check_device();
    if (rc) return rc;
    unsigned int* status = nullptr;
    rc = gqa::forward_status_word(&status);
    if (rc) return rc;
    Shape s{B, Hq, Hkv, S, D, causal ? 1 : 0, scale};
    s.bshd = (flags & GQA_LAYOUT_BSHD) ? 1 : 0;
    if (packed) {
        s.cu_seqlens = packed->cu_seqlens;
        s.n_seqs = packed->n_seqs;
        s.max_seqlen = packed->max_seqlen;
    }
    return gqa::launch_fwd_sm100(Q, K, V, O, LSE, s, status, stream);
}

}  // namespace

extern "C" int gqa_fwd(const void* Q, const void* K, const void* V, void* O, float* LSE, int B, int Hq, int Hkv, int S,
                       int D, int causal, float scale, gqa_stream_t stream) {
    return run_fwd(Q, K, V, O, LSE, B, Hq, Hkv, S, D, causal, scale, reinterpret_cast<cudaStream_t>(stream), 0u);
}

extern "C" int gqa_fwd_ex(const void* Q, const void* K, const void* V, void* O, float* LSE, int B, int Hq, int Hkv,
                          int S, int D, int causal, float scale, gqa_stream_t stream, unsigned int flags) {
    return run_fwd(Q, K, V, O, LSE, B, Hq, Hkv, S, D, causal, scale, reinterpret_cast<cudaStream_t>(stream), flags);
}

extern "C" int launch_gqa(const void* Q, const void* K, const void* V, void* O, float* LSE, int B, int Hq, int Hkv,
                          int S, int D, int causal, float scale, gqa_stream_t stream) {
    return gqa_fwd(Q, K, V, O, LSE, B, Hq, Hkv, S, D, causal, scale, stream);
}

extern "C" int gqa_fwd_varlen(const void* Q, const void* K, const void* V, void* O, float* LSE, const int* cu_seqlens,
                              int n_seqs, int total_tokens, int max_seqlen, int Hq, int Hkv, int D, int causal,
                              float scale, gqa_stream_t stream) {
    const int rc = check_packed(cu_seqlens, n_seqs, total_tokens, max_seqlen, D);
    if (rc) return rc;
    const Packed packed{cu_seqlens, n_seqs, max_seqlen};
    return run_fwd(Q, K, V, O, LSE, 1, Hq, Hkv, total_tokens, D, causal, scale, reinterpret_cast<cudaStream_t>(stream),
                   GQA_LAYOUT_BSHD, &packed);
}

extern "C" size_t gqa_bwd_varlen_workspace_bytes(int total_tokens, int Hq, int Hkv, int D) {
    if (D != 64 && D != 128) return 0;
    return gqa_bwd_workspace_bytes(1, Hq, Hkv, total_tokens, D, 0);
}

extern "C" size_t gqa_bwd_workspace_bytes(int B, int Hq, int Hkv, int S, int D, int causal) {
    (void)causal;
    if (check_shape(B, Hq, Hkv, S, D) != GQA_OK) return 0;
    (void)causal;
    const Shape s{B, Hq, Hkv, S, D, 0, 0.f};
    return gqa::BwdWorkspace(s).total;
}

extern "C" size_t gqa_bwd_workspace_bytes_ex(int B, int Hq, int Hkv, int S, int D, int causal, unsigned int flags) {
    if (check_shape(B, Hq, Hkv, S, D) != GQA_OK) return 0;
    if (flags & ~(unsigned)(GQA_BWD_DETERMINISTIC | GQA_LAYOUT_BSHD | GQA_BWD_SPLIT_HEADS | GQA_BWD_DQ_SEPARATE)) return 0;
    Shape s{B, Hq, Hkv, S, D, causal ? 1 : 0, 0.f};
    s.bshd = (flags & GQA_LAYOUT_BSHD) ? 1 : 0;
    return gqa::BwdWorkspace(s, (flags & GQA_BWD_SPLIT_HEADS) ? gqa::bwd_head_parts(s) : 1).total;
}

namespace {

// Shared body of gqa_bwd and gqa_bwd_stage_times; `ev` is null or four events recorded around the stages.
int run_bwd(const void* Q, const void* K, const void* V, const void* O, const void* dO, const float* LSE, void* dQ,
            void* dK, void* dV, int B, int Hq, int Hkv, int S, int D, int causal, float scale, void* workspace,
            size_t workspace_bytes, cudaStream_t stream, cudaEvent_t* ev, unsigned int flags = 0,
            const Packed* packed = nullptr) {
    if (flags & ~(unsigned)(GQA_BWD_DETERMINISTIC | GQA_LAYOUT_BSHD | GQA_BWD_SPLIT_HEADS | GQA_BWD_DQ_SEPARATE))
        return GQA_ERR_BAD_ARGUMENT;
    if (packed && flags != GQA_LAYOUT_BSHD) return GQA_ERR_BAD_ARGUMENT;  // no ordered mode, head split or separate dQ pass
    if (!Q || !K || !V || !O || !dO || !LSE || !dQ || !dK || !dV || !scale_ok(scale)) return GQA_ERR_BAD_ARGUMENT;
    int rc = check_shape(B, Hq, Hkv, S, D);
    if (rc) return rc;
    if ((flags & GQA_LAYOUT_BSHD) && D != 64 && D != 128) return GQA_ERR_UNSUPPORTED;  // see the forward
    const void* ptrs[] = {Q, K, V, O, dO, LSE, dQ, dK, dV};
    for (const void* p : ptrs)
        if (!gqa::aligned16(p)) return GQA_ERR_BAD_ARGUMENT;
    Shape s{B, Hq, Hkv, S, D, causal ? 1 : 0, scale};
    s.bshd = (flags & GQA_LAYOUT_BSHD) ? 1 : 0;
    if (packed) {
        s.cu_seqlens = packed->cu_seqlens;
        s.n_seqs = packed->n_seqs;
        s.max_seqlen = packed->max_seqlen;
    }
    const int parts = (flags & GQA_BWD_SPLIT_HEADS) ? gqa::bwd_head_parts(s) : 1;
    const gqa::BwdWorkspace ws(s, parts);
    if (!workspace || workspace_bytes < ws.total) {
        gqa::note_text("backward workspace: need %zu bytes, got %zu", ws.total, workspace ? workspace_bytes : (size_t)0);
        return GQA_ERR_WORKSPACE;
    }
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return GQA_ERR_BAD_ARGUMENT;
    rc = check_device();
    if (rc) return rc;
    char* w = static_cast<char*>(workspace);
    unsigned int* status = reinterpret_cast<unsigned int*>(w + ws.status_off);
    void* lse_cols = w + ws.lse_cols_off;
    void* delta_cols = w + ws.delta_cols_off;
    float* dq_accum = reinterpret_cast<float*>(w + ws.dq_accum_off);
    float* delta_f32 = reinterpret_cast<float*>(w + ws.delta_f32_off);
    // The dQ path.  Default: fp32 TMA reduce-add of the main kernel's dQ tiles into the accumulator: measured faster
    // than the separate query-parallel pass at every benchmark shape (1.3-1.7x), and so is its ordered (deterministic)
    // form except at one shape, so the separate pass is taken only when asked for.
    const bool dq_separate = (flags & GQA_BWD_DQ_SEPARATE) != 0;
    unsigned int* dq_turn = nullptr;
    if ((flags & GQA_BWD_DETERMINISTIC) && !dq_separate) {
        dq_turn = reinterpret_cast<unsigned int*>(w + ws.dq_turn_off);
        GQA_CUDA_TRY(cudaMemsetAsync(dq_turn, 0, ws.dq_turn_bytes, stream));
    }

    GQA_CUDA_TRY(cudaMemsetAsync(status, 0, 256, stream));
    if (ev) GQA_CUDA_TRY(cudaEventRecord(ev[0], stream));
    rc = gqa::launch_bwd_preprocess(O, dO, LSE, 1.0f / scale, dq_separate ? delta_f32 : nullptr, lse_cols, delta_cols,
                                    dq_separate ? nullptr : dq_accum, s.q_rows(), D, stream, s.bshd ? S : 0,
                                    s.bshd ? Hq : 0);
    if (rc) return rc;
    if (ev) GQA_CUDA_TRY(cudaEventRecord(ev[1], stream));
    float* partial = parts > 1 ? reinterpret_cast<float*>(w + ws.partial_off) : nullptr;
    rc = gqa::launch_bwd_main_sm100(Q, K, V, dO, lse_cols, delta_cols, dq_separate ? nullptr : dq_accum, dq_turn, dK, dV,
                                    s, status, parts, partial, stream);
    if (rc) return rc;
    if (ev) GQA_CUDA_TRY(cudaEventRecord(ev[2], stream));
    if (parts > 1) {
        rc = gqa::launch_dkdv_reduce(partial, dK, dV, s, parts, stream);
        if (rc) return rc;
    }
    if (dq_separate)
        rc = gqa::launch_bwd_dq_sm100(Q, K, V, dO, LSE, delta_f32, dQ, s, status, stream);
    else
        rc = gqa::launch_dq_finalise(dq_accum, dQ, s.q_rows(), scale, stream, D, s.bshd ? S : 0, s.bshd ? Hq : 0);
    if (rc) return rc;
    if (ev) GQA_CUDA_TRY(cudaEventRecord(ev[3], stream));
    return GQA_OK;
}

}  // namespace

extern "C" int gqa_bwd(const void* Q, const void* K, const void* V, const void* O, const void* dO, const float* LSE,
                       void* dQ, void* dK, void* dV, int B, int Hq, int Hkv, int S, int D, int causal, float scale,
                       void* workspace, size_t workspace_bytes, gqa_stream_t stream) {
    return run_bwd(Q, K, V, O, dO, LSE, dQ, dK, dV, B, Hq, Hkv, S, D, causal, scale, workspace, workspace_bytes,
                   reinterpret_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int gqa_bwd_ex(const void* Q, const void* K, const void* V, const void* O, const void* dO, const float* LSE,
                          void* dQ, void* dK, void* dV, int B, int Hq, int Hkv, int S, int D, int causal, float scale,
                          void* workspace, size_t workspace_bytes, gqa_stream_t stream, unsigned int flags) {
    return run_bwd(Q, K, V, O, dO, LSE, dQ, dK, dV, B, Hq, Hkv, S, D, causal, scale, workspace, workspace_bytes,
                   reinterpret_cast<cudaStream_t>(stream), nullptr, flags);
}

extern "C" int gqa_bwd_varlen(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                              const float* LSE, void* dQ, void* dK, void* dV, const int* cu_seqlens, int n_seqs,
                              int total_tokens, int max_seqlen, int Hq, int Hkv, int D, int causal, float scale,
                              void* workspace, size_t workspace_bytes, gqa_stream_t stream) {
    const int rc = check_packed(cu_seqlens, n_seqs, total_tokens, max_seqlen, D);
    if (rc) return rc;
    const Packed packed{cu_seqlens, n_seqs, max_seqlen};
    return run_bwd(Q, K, V, O, dO, LSE, dQ, dK, dV, 1, Hq, Hkv, total_tokens, D, causal, scale, workspace,
                   workspace_bytes, reinterpret_cast<cudaStream_t>(stream), nullptr, GQA_LAYOUT_BSHD, &packed);
}

extern "C" int gqa_bwd_stage_times(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                                   const float* LSE, void* dQ, void* dK, void* dV, int B, int Hq, int Hkv, int S,
                                   int D, int causal, float scale, void* workspace, size_t workspace_bytes,
                                   gqa_stream_t stream_, float* stage_ms) {
    if (!stage_ms) return GQA_ERR_BAD_ARGUMENT;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    for (auto& e : ev) GQA_CUDA_TRY(cudaEventCreate(&e));
    int rc = run_bwd(Q, K, V, O, dO, LSE, dQ, dK, dV, B, Hq, Hkv, S, D, causal, scale, workspace, workspace_bytes,
                     stream, ev);
    if (rc == GQA_OK) {
        cudaError_t e = cudaEventSynchronize(ev[3]);
        for (int i = 0; i < 3 && e == cudaSuccess; ++i) e = cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
        if (e != cudaSuccess) rc = gqa::note_cuda_error(e, "stage timing");
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return rc;
}

// ---- backward for callers that must not allocate --------------------------------------------
// The scratch that gqa_bwd takes from its caller lives here in a fixed device array instead.
// Every GPU that loads this library keeps these bytes resident until the process exits.
#define GQA_STATIC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[GQA_STATIC_SCRATCH_BYTES];

namespace {

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can use.
// The device address is looked up once per device, with that device current, and cached.
int static_scratch_address(void** out) {
    constexpr int kMaxDev = 64;
    static void* addr[kMaxDev] = {};
    static std::mutex mu;
    int dev = 0;
    GQA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) return GQA_ERR_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        GQA_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return GQA_ERR_CUDA;
        addr[dev] = p;
    }
    *out = addr[dev];
    return GQA_OK;
}

}  // namespace

extern "C" size_t gqa_bwd_static_scratch_bytes(void) { return GQA_STATIC_SCRATCH_BYTES; }

extern "C" int gqa_bwd_static_scratch(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                                      const float* LSE, void* dQ, void* dK, void* dV, int B, int Hq, int Hkv, int S,
                                      int D, int causal, float scale, gqa_stream_t stream) {
    int rc = check_shape(B, Hq, Hkv, S, D);
    if (rc) return rc;
    const Shape s{B, Hq, Hkv, S, D, causal ? 1 : 0, scale};
    const size_t need = gqa::BwdWorkspace(s).total;
    if (need > GQA_STATIC_SCRATCH_BYTES) {
        gqa::note_text("gqa_bwd_static_scratch: this shape needs %zu bytes of scratch, the built-in array holds %zu",
                       need, (size_t)GQA_STATIC_SCRATCH_BYTES);
        return GQA_ERR_WORKSPACE;
    }
    // the argument and device checks of run_bwd come first, so that a wrong device reports GQA_ERR_ARCH and
    // not the failed symbol look-up
    if (!Q || !K || !V || !O || !dO || !LSE || !dQ || !dK || !dV || !scale_ok(scale)) return GQA_ERR_BAD_ARGUMENT;
    rc = check_device();
    if (rc) return rc;
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc) return rc;
    // run_bwd clears the status word and the preprocess stage zeroes the dQ accumulator, so nothing
    // left in the array by an earlier call is read.
    return run_bwd(Q, K, V, O, dO, LSE, dQ, dK, dV, B, Hq, Hkv, S, D, causal, scale, scratch, need,
                   reinterpret_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int gqa_check_status(const void* workspace, gqa_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const unsigned int* word = static_cast<const unsigned int*>(workspace);
    unsigned int* forward_word = nullptr;
    if (!word) {
        int rc = gqa::forward_status_word(&forward_word);
        if (rc) return rc;
        word = forward_word;
    }
    unsigned int host = 0;
    GQA_CUDA_TRY(cudaMemcpyAsync(&host, word, sizeof host, cudaMemcpyDeviceToHost, stream));
    GQA_CUDA_TRY(cudaStreamSynchronize(stream));
    if (host == 0) return GQA_OK;
    // the forward's report is sticky: reading it re-arms the device
    if (forward_word) GQA_CUDA_TRY(cudaMemsetAsync(forward_word, 0, sizeof(unsigned int), stream));
    return gqa::note_device_timeout(host);
}
