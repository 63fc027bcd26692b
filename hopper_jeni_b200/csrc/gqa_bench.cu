// C++ host driver for the C ABI, in the shape of the reference's drivers
// (src/attention/GQA_bwd_baseline.cu:608-692, src/attention/GQA_fwd_v62.cu:39-131):
//   load data/gqa_*.bin (raw fp32, bf16-representable) -> H2D -> gqa_fwd / gqa_bwd -> D2H ->
//   reportPrecision + checkResult(2e-2, 2e-2) -> determinism probe -> benchmarkKernel -> displayStats.
// Unlike the reference it returns a non-zero exit code when a gate fails, takes S, D and
// causal from the command line and prints one JSON line per run.
//
//   gqa_bench B Hq Hkv [S=4096] [D=64] [causal=0] [--data DIR] [--synthetic] [--iters N] [--warmup N] [--runs N]
//
// Golden files are produced by oracle/make_ref.py (PyTorch fp32 SDPA autograd on the same
// seeded inputs).  With --synthetic the inputs are generated here and only timing,
// finiteness and determinism are reported.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "gqa.h"
#include "gqa_harness.hpp"

#define CK(call)                                                                                     \
    do {                                                                                             \
        cudaError_t e__ = (call);                                                                    \
        if (e__ != cudaSuccess) {                                                                    \
            std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e__), __FILE__, __LINE__); \
            return 2;                                                                                \
        }                                                                                            \
    } while (0)
#define GQ(call)                                                                                               \
    do {                                                                                                       \
        int s__ = (call);                                                                                      \
        if (s__ != GQA_OK) {                                                                                   \
            std::fprintf(stderr, "%s -> %s | %s\n", #call, gqa_status_string(s__), gqa_last_cuda_error());     \
            return 3;                                                                                          \
        }                                                                                                      \
    } while (0)

namespace {

struct Tensor {
    std::vector<float> host;      // fp32 view (bf16-representable for inputs)
    __nv_bfloat16* dev = nullptr;
    size_t n = 0;
};

bool upload_bf16(Tensor& t) {
    std::vector<__nv_bfloat16> tmp(t.n);
    for (size_t i = 0; i < t.n; ++i) tmp[i] = __float2bfloat16(t.host[i]);
    if (cudaMalloc(&t.dev, t.n * sizeof(__nv_bfloat16)) != cudaSuccess) return false;
    return cudaMemcpy(t.dev, tmp.data(), t.n * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice) == cudaSuccess;
}

bool download_bf16(const __nv_bfloat16* dev, size_t n, std::vector<float>& out) {
    std::vector<__nv_bfloat16> tmp(n);
    if (cudaMemcpy(tmp.data(), dev, n * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost) != cudaSuccess) return false;
    out.resize(n);
    for (size_t i = 0; i < n; ++i) out[i] = __bfloat162float(tmp[i]);
    return true;
}

void fill_normal(std::vector<float>& v, unsigned seed, float mul) {
    std::mt19937 gen(seed);
    std::normal_distribution<float> dist(0.f, 1.f);
    for (float& x : v) x = __bfloat162float(__float2bfloat16(dist(gen) * mul));
}

}  // namespace

int main(int argc, char** argv) {
    int pos[6] = {8, 12, 4, 4096, 64, 0};
    int npos = 0, iters = 100, warmup = 10, runs = 3;
    std::string data = "data";
    bool synthetic = false;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        if (a == "--data" && i + 1 < argc) data = argv[++i];
        else if (a == "--synthetic") synthetic = true;
        else if (a == "--iters" && i + 1 < argc) iters = std::atoi(argv[++i]);
        else if (a == "--warmup" && i + 1 < argc) warmup = std::atoi(argv[++i]);
        else if (a == "--runs" && i + 1 < argc) runs = std::atoi(argv[++i]);
        else if (npos < 6) pos[npos++] = std::atoi(argv[i]);
    }
    const int B = pos[0], Hq = pos[1], Hkv = pos[2], S = pos[3], D = pos[4], causal = pos[5];
    const float scale = 1.0f / std::sqrt((float)D);
    const size_t nq = (size_t)B * Hq * S * D, nkv = (size_t)B * Hkv * S * D, nl = (size_t)B * Hq * S;
    std::printf("GQA bench: B=%d Hq=%d Hkv=%d (G=%d) S=%d D=%d causal=%d  lib %s\n", B, Hq, Hkv, Hkv ? Hq / Hkv : 0, S,
                D, causal, gqa_version());

    Tensor q, k, v, d_o;
    q.n = d_o.n = nq;
    k.n = v.n = nkv;
    for (Tensor* t : {&q, &k, &v, &d_o}) t->host.resize(t->n);
    std::vector<float> ref_o, ref_lse, ref_dq, ref_dk, ref_dv;
    bool have_ref = false;
    if (!synthetic) {
        auto path = [&](const char* name) { return data + "/gqa_" + name + ".bin"; };
        bool ok = loadBin(path("q").c_str(), q.host.data(), nq) && loadBin(path("k").c_str(), k.host.data(), nkv) &&
                  loadBin(path("v").c_str(), v.host.data(), nkv) && loadBin(path("do").c_str(), d_o.host.data(), nq);
        if (!ok) {
            std::fprintf(stderr, "missing inputs under %s: run `python oracle/make_ref.py %d %d %d %d %d %d` or pass --synthetic\n",
                         data.c_str(), B, Hq, Hkv, S, D, causal);
            return 1;
        }
        ref_o.resize(nq); ref_lse.resize(nl); ref_dq.resize(nq); ref_dk.resize(nkv); ref_dv.resize(nkv);
        have_ref = loadBin(path("o").c_str(), ref_o.data(), nq) && loadBin(path("lse").c_str(), ref_lse.data(), nl) &&
                   loadBin(path("dq").c_str(), ref_dq.data(), nq) && loadBin(path("dk").c_str(), ref_dk.data(), nkv) &&
                   loadBin(path("dv").c_str(), ref_dv.data(), nkv);
        if (!have_ref) return 1;
    } else {
        fill_normal(q.host, 42, 1.f);
        fill_normal(k.host, 43, 1.f);
        fill_normal(v.host, 44, 1.f);
        fill_normal(d_o.host, 45, 1.f);
    }
    for (Tensor* t : {&q, &k, &v, &d_o})
        if (!upload_bf16(*t)) return 2;

    __nv_bfloat16 *o = nullptr, *dq = nullptr, *dk = nullptr, *dv = nullptr;
    float* lse = nullptr;
    void* ws = nullptr;
    const size_t ws_bytes = gqa_bwd_workspace_bytes(B, Hq, Hkv, S, D, causal);
    if (ws_bytes == 0) {
        std::fprintf(stderr, "unsupported shape\n");
        return 1;
    }
    CK(cudaMalloc(&o, nq * 2));
    CK(cudaMalloc(&dq, nq * 2));
    CK(cudaMalloc(&dk, nkv * 2));
    CK(cudaMalloc(&dv, nkv * 2));
    CK(cudaMalloc(&lse, nl * 4));
    CK(cudaMalloc(&ws, ws_bytes));

    auto fwd = [&]() { return gqa_fwd(q.dev, k.dev, v.dev, o, lse, B, Hq, Hkv, S, D, causal, scale, nullptr); };
    auto bwd = [&]() {
        return gqa_bwd(q.dev, k.dev, v.dev, o, d_o.dev, lse, dq, dk, dv, B, Hq, Hkv, S, D, causal, scale, ws, ws_bytes,
                       nullptr);
    };

    GQ(fwd());
    GQ(gqa_check_status(nullptr, nullptr));
    GQ(bwd());
    GQ(gqa_check_status(ws, nullptr));
    CK(cudaDeviceSynchronize());

    bool pass = true;
    std::vector<float> h_o, h_dq, h_dk, h_dv, h_lse(nl);
    if (!download_bf16(o, nq, h_o) || !download_bf16(dq, nq, h_dq) || !download_bf16(dk, nkv, h_dk) ||
        !download_bf16(dv, nkv, h_dv))
        return 2;
    CK(cudaMemcpy(h_lse.data(), lse, nl * 4, cudaMemcpyDeviceToHost));
    PrecisionReport rep[5];
    if (have_ref) {
        std::printf("\n=== precision vs fp32 SDPA autograd (gate |d| <= 2e-2 + 2e-2|ref|) ===\n");
        rep[0] = reportPrecision("O  ", ref_o.data(), h_o.data(), nq);
        pass &= checkResult(ref_o.data(), h_o.data(), nq, 2e-2f, 2e-2f);
        rep[1] = reportPrecision("LSE", ref_lse.data(), h_lse.data(), nl);
        pass &= checkResult(ref_lse.data(), h_lse.data(), nl, 2e-2f, 2e-2f);
        rep[2] = reportPrecision("dQ ", ref_dq.data(), h_dq.data(), nq);
        pass &= checkResult(ref_dq.data(), h_dq.data(), nq, 2e-2f, 2e-2f);
        rep[3] = reportPrecision("dK ", ref_dk.data(), h_dk.data(), nkv);
        pass &= checkResult(ref_dk.data(), h_dk.data(), nkv, 2e-2f, 2e-2f);
        rep[4] = reportPrecision("dV ", ref_dv.data(), h_dv.data(), nkv);
        pass &= checkResult(ref_dv.data(), h_dv.data(), nkv, 2e-2f, 2e-2f);
    } else {
        for (const std::vector<float>* t : {&h_o, &h_dq, &h_dk, &h_dv})
            for (float x : *t)
                if (!std::isfinite(x)) pass = false;
        std::printf("synthetic inputs: outputs %s\n", pass ? "finite" : "NOT finite");
    }

    // determinism probe: same inputs, 8 runs (precision/vj1d_determinism_probe.cu:32-48)
    bool dkdv_identical = true;
    double dq_max_delta = 0;
    {
        std::vector<float> a, b2, c2;
        for (int r = 0; r < 8; ++r) {
            GQ(bwd());
            CK(cudaDeviceSynchronize());
            if (!download_bf16(dq, nq, a) || !download_bf16(dk, nkv, b2) || !download_bf16(dv, nkv, c2)) return 2;
            if (std::memcmp(b2.data(), h_dk.data(), nkv * 4) || std::memcmp(c2.data(), h_dv.data(), nkv * 4))
                dkdv_identical = false;
            for (size_t i = 0; i < nq; ++i) dq_max_delta = std::max(dq_max_delta, (double)std::fabs(a[i] - h_dq[i]));
        }
        std::printf("\ndeterminism over 8 runs: dK/dV %s, dQ max|delta| = %.3e\n",
                    dkdv_identical ? "bit-identical" : "DIFFER", dq_max_delta);
    }

    // timing: whole gqa_bwd call (preprocess + main + dQ finalise), L2 flushed before every rep
    double f = 4.0 * B * Hq * (double)S * S * D * (causal ? 0.5 : 1.0);
    const long long flops_fwd = (long long)f, flops_bwd = (long long)(4.0 * f);
    const size_t bytes_bwd = 4 * nq * 2 + 4 * nkv * 2 + nl * 4, bytes_fwd = 2 * nq * 2 + 2 * nkv * 2 + nl * 4;
    std::vector<float> med_b, med_f;
    KernelStats sb, sf;
    for (int r = 0; r < runs; ++r) {
        sb = benchmarkKernel([&] { bwd(); }, iters, warmup, flops_bwd, bytes_bwd);
        sf = benchmarkKernel([&] { fwd(); }, iters, warmup, flops_fwd, bytes_fwd);
        if (!sb.valid || !sf.valid) return 2;
        med_b.push_back(sb.median_ms);
        med_f.push_back(sf.median_ms);
    }
    GQ(gqa_check_status(ws, nullptr));
    std::sort(med_b.begin(), med_b.end());
    std::sort(med_f.begin(), med_f.end());
    const double mb = med_b[med_b.size() / 2], mf = med_f[med_f.size() / 2];
    displayStats("gqa_bwd (last run)", sb);
    displayStats("gqa_fwd (last run)", sf);
    const double tf_b = flops_bwd / (mb * 1e9), tf_f = flops_fwd / (mf * 1e9);
    std::printf("\nmedian of %d run medians: bwd %.4f ms = %.1f TFLOP/s (4x-forward convention; %.1f executed-MMA), "
                "%.1f%% of 2250 nominal; fwd %.4f ms = %.1f TFLOP/s\n",
                runs, mb, tf_b, tf_b * 2.5 / 4.0, 100.0 * tf_b / 2250.0, mf, tf_f);
    std::printf("{\"harness\": \"gqa_bench\", \"B\": %d, \"Hq\": %d, \"Hkv\": %d, \"S\": %d, \"D\": %d, \"causal\": %d, "
                "\"bwd_ms_median\": %.5f, \"bwd_tflops\": %.2f, \"fwd_ms_median\": %.5f, \"fwd_tflops\": %.2f, "
                "\"gate_pass\": %s, \"dkdv_bit_identical\": %s, \"dq_max_run_delta\": %.3e, "
                "\"rel_rms\": {\"O\": %.3e, \"dQ\": %.3e, \"dK\": %.3e, \"dV\": %.3e}, \"kernel_launches\": %llu}\n",
                B, Hq, Hkv, S, D, causal, mb, tf_b, mf, tf_f, pass ? "true" : "false",
                dkdv_identical ? "true" : "false", dq_max_delta, rep[0].rel_rms, rep[2].rel_rms, rep[3].rel_rms,
                rep[4].rel_rms, gqa_launch_count());
    return pass ? 0 : 4;
}
