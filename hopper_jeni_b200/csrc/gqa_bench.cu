// C++ host driver for the C ABI, in the shape of the reference's drivers
// (src/attention/GQA_bwd_baseline.cu:608-692, src/attention/GQA_fwd_v62.cu:39-131):
//   load data/gqa_*.bin (raw fp32, bf16-representable) -> H2D -> gqa_fwd / gqa_bwd -> D2H ->
//   reportPrecision + checkResult(2e-2, 2e-2) -> determinism probe -> benchmarkKernel -> displayStats.
// Unlike the reference it returns a non-zero exit code when a gate fails, takes S, D and causal from
// the command line, prints one JSON line per run and can drive several GPUs:
//
//   gqa_bench B Hq Hkv [S=4096] [D=64] [causal=0] [--data DIR] [--synthetic] [--iters N] [--warmup N]
//             [--runs N] [--gpus N] [--deterministic]
//
// With --gpus N the (batch x KV-head) groups are cut into N contiguous ranges, one host thread per
// device runs the unmodified single-GPU entry points on its range (a range is itself a GQA problem with
// B' = groups, Hkv' = 1, Hq' = G), and the shards are checked on the host against the same golden
// files; no device-to-device traffic is needed.  The aggregate rate is total FLOPs / slowest device.
//
// Golden files are produced by oracle/make_ref.py (PyTorch fp32 SDPA autograd on the same seeded
// inputs).  With --synthetic the inputs are generated here and only timing, finiteness and determinism
// are reported.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "gqa.h"
#include "gqa_harness.hpp"

namespace {

struct Options {
    int B = 8, Hq = 12, Hkv = 4, S = 4096, D = 64, causal = 0;
    int iters = 100, warmup = 10, runs = 3, gpus = 1;
    bool synthetic = false;
    bool deterministic = false;  // gqa_bwd_ex with GQA_BWD_DETERMINISTIC (ordered dQ reductions)
    std::string data = "data";
};

struct HostData {  // whole problem, fp32 views (inputs are bf16-representable)
    std::vector<float> q, k, v, d_o, ref_o, ref_lse, ref_dq, ref_dk, ref_dv;
    bool have_ref = false;
};

struct ShardResult {
    int rc = 0;  // 0 ok, 2 CUDA error, 3 library error
    bool pass = true, dkdv_identical = true;
    double dq_max_delta = 0, bwd_ms = 0, fwd_ms = 0;
    PrecisionReport rep[5];
    KernelStats last_bwd, last_fwd;
};

std::mutex g_print;

void fill_normal(std::vector<float>& v, unsigned seed) {
    std::mt19937 gen(seed);
    std::normal_distribution<float> dist(0.f, 1.f);
    for (float& x : v) x = __bfloat162float(__float2bfloat16(dist(gen)));
}

bool upload_bf16(const float* src, size_t n, __nv_bfloat16** dev) {
    std::vector<__nv_bfloat16> tmp(n);
    for (size_t i = 0; i < n; ++i) tmp[i] = __float2bfloat16(src[i]);
    if (cudaMalloc(dev, n * sizeof(__nv_bfloat16)) != cudaSuccess) return false;
    return cudaMemcpy(*dev, tmp.data(), n * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice) == cudaSuccess;
}

bool download_bf16(const __nv_bfloat16* dev, size_t n, std::vector<float>& out) {
    std::vector<__nv_bfloat16> tmp(n);
    if (cudaMemcpy(tmp.data(), dev, n * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost) != cudaSuccess) return false;
    out.resize(n);
    for (size_t i = 0; i < n; ++i) out[i] = __bfloat162float(tmp[i]);
    return true;
}

#define CKR(call)                                                                                        \
    do {                                                                                                 \
        if ((call) != cudaSuccess) {                                                                     \
            std::fprintf(stderr, "[gpu %d] CUDA error at %s:%d: %s\n", dev, __FILE__, __LINE__,          \
                         cudaGetErrorString(cudaGetLastError()));                                        \
            r.rc = 2;                                                                                    \
            return;                                                                                      \
        }                                                                                                \
    } while (0)
#define GQR(call)                                                                                            \
    do {                                                                                                     \
        int s__ = (call);                                                                                    \
        if (s__ != GQA_OK) {                                                                                 \
            std::fprintf(stderr, "[gpu %d] %s -> %s | %s\n", dev, #call, gqa_status_string(s__),             \
                         gqa_last_cuda_error());                                                             \
            r.rc = 3;                                                                                        \
            return;                                                                                          \
        }                                                                                                    \
    } while (0)

// Runs groups [g0, g1) of the problem on device `dev` as the GQA problem (Bs, Hqs, Hkvs).
void run_shard(int dev, const Options& o, const HostData& h, int g0, int g1, int Bs, int Hqs, int Hkvs, ShardResult& r) {
    const int S = o.S, D = o.D, G = o.Hq / o.Hkv;
    const float scale = 1.0f / std::sqrt((float)D);
    CKR(cudaSetDevice(dev));
    const size_t q_off = (size_t)g0 * G * S * D, kv_off = (size_t)g0 * S * D, l_off = (size_t)g0 * G * S;
    const size_t nq = (size_t)(g1 - g0) * G * S * D, nkv = (size_t)(g1 - g0) * S * D, nl = (size_t)(g1 - g0) * G * S;
    __nv_bfloat16 *q = nullptr, *k = nullptr, *v = nullptr, *d_o = nullptr, *out = nullptr, *dq = nullptr, *dk = nullptr,
                  *dv = nullptr;
    float* lse = nullptr;
    void* ws = nullptr;
    if (!upload_bf16(h.q.data() + q_off, nq, &q) || !upload_bf16(h.k.data() + kv_off, nkv, &k) ||
        !upload_bf16(h.v.data() + kv_off, nkv, &v) || !upload_bf16(h.d_o.data() + q_off, nq, &d_o)) {
        r.rc = 2;
        return;
    }
    const size_t ws_bytes = gqa_bwd_workspace_bytes(Bs, Hqs, Hkvs, S, D, o.causal);
    CKR(cudaMalloc(&out, nq * 2));
    CKR(cudaMalloc(&dq, nq * 2));
    CKR(cudaMalloc(&dk, nkv * 2));
    CKR(cudaMalloc(&dv, nkv * 2));
    CKR(cudaMalloc(&lse, nl * 4));
    CKR(cudaMalloc(&ws, ws_bytes));
    auto fwd = [&]() { return gqa_fwd(q, k, v, out, lse, Bs, Hqs, Hkvs, S, D, o.causal, scale, nullptr); };
    auto bwd = [&]() {
        return gqa_bwd_ex(q, k, v, out, d_o, lse, dq, dk, dv, Bs, Hqs, Hkvs, S, D, o.causal, scale, ws, ws_bytes, nullptr,
                          o.deterministic ? GQA_BWD_DETERMINISTIC : 0u);
    };
    GQR(fwd());
    GQR(gqa_check_status(nullptr, nullptr));
    GQR(bwd());
    GQR(gqa_check_status(ws, nullptr));
    CKR(cudaDeviceSynchronize());

    std::vector<float> h_o, h_dq, h_dk, h_dv, h_lse(nl);
    if (!download_bf16(out, nq, h_o) || !download_bf16(dq, nq, h_dq) || !download_bf16(dk, nkv, h_dk) ||
        !download_bf16(dv, nkv, h_dv)) {
        r.rc = 2;
        return;
    }
    CKR(cudaMemcpy(h_lse.data(), lse, nl * 4, cudaMemcpyDeviceToHost));
    {
        std::lock_guard<std::mutex> lock(g_print);
        if (h.have_ref) {
            std::printf("\n=== [gpu %d, groups %d-%d] precision vs fp32 SDPA autograd (gate |d| <= 2e-2 + 2e-2|ref|) ===\n", dev,
                        g0, g1 - 1);
            const float* refs[5] = {h.ref_o.data() + q_off, h.ref_lse.data() + l_off, h.ref_dq.data() + q_off,
                                    h.ref_dk.data() + kv_off, h.ref_dv.data() + kv_off};
            const float* gots[5] = {h_o.data(), h_lse.data(), h_dq.data(), h_dk.data(), h_dv.data()};
            const size_t ns[5] = {nq, nl, nq, nkv, nkv};
            const char* names[5] = {"O  ", "LSE", "dQ ", "dK ", "dV "};
            for (int i = 0; i < 5; ++i) {
                r.rep[i] = reportPrecision(names[i], refs[i], gots[i], ns[i]);
                r.pass &= checkResult(refs[i], gots[i], ns[i], 2e-2f, 2e-2f);
            }
        } else {
            for (const std::vector<float>* t : {&h_o, &h_dq, &h_dk, &h_dv})
                for (float x : *t)
                    if (!std::isfinite(x)) r.pass = false;
            std::printf("[gpu %d] synthetic inputs: outputs %s\n", dev, r.pass ? "finite" : "NOT finite");
        }
    }
    // determinism probe: same inputs, 8 runs (precision/vj1d_determinism_probe.cu:32-48)
    {
        std::vector<float> a, b2, c2;
        for (int rep = 0; rep < 8; ++rep) {
            GQR(bwd());
            CKR(cudaDeviceSynchronize());
            if (!download_bf16(dq, nq, a) || !download_bf16(dk, nkv, b2) || !download_bf16(dv, nkv, c2)) {
                r.rc = 2;
                return;
            }
            if (std::memcmp(b2.data(), h_dk.data(), nkv * 4) || std::memcmp(c2.data(), h_dv.data(), nkv * 4))
                r.dkdv_identical = false;
            for (size_t i = 0; i < nq; ++i) r.dq_max_delta = std::max(r.dq_max_delta, (double)std::fabs(a[i] - h_dq[i]));
        }
    }
    // timing: whole gqa_bwd call (preprocess + main + dQ finalise), L2 flushed before every rep
    const double f = 4.0 * (g1 - g0) * G * (double)S * S * D * (o.causal ? 0.5 : 1.0);
    const size_t bytes_bwd = 4 * nq * 2 + 4 * nkv * 2 + nl * 4, bytes_fwd = 2 * nq * 2 + 2 * nkv * 2 + nl * 4;
    std::vector<float> med_b, med_f;
    for (int run = 0; run < o.runs; ++run) {
        r.last_bwd = benchmarkKernel([&] { bwd(); }, o.iters, o.warmup, (long long)(4.0 * f), bytes_bwd);
        r.last_fwd = benchmarkKernel([&] { fwd(); }, o.iters, o.warmup, (long long)f, bytes_fwd);
        if (!r.last_bwd.valid || !r.last_fwd.valid) {
            r.rc = 2;
            return;
        }
        med_b.push_back(r.last_bwd.median_ms);
        med_f.push_back(r.last_fwd.median_ms);
    }
    GQR(gqa_check_status(ws, nullptr));
    std::sort(med_b.begin(), med_b.end());
    std::sort(med_f.begin(), med_f.end());
    r.bwd_ms = med_b[med_b.size() / 2];
    r.fwd_ms = med_f[med_f.size() / 2];
    for (void* p : {(void*)q, (void*)k, (void*)v, (void*)d_o, (void*)out, (void*)dq, (void*)dk, (void*)dv, (void*)lse, ws})
        cudaFree(p);
}

}  // namespace

int main(int argc, char** argv) {
    Options o;
    int pos[6] = {o.B, o.Hq, o.Hkv, o.S, o.D, o.causal}, npos = 0;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        if (a == "--data" && i + 1 < argc) o.data = argv[++i];
        else if (a == "--synthetic") o.synthetic = true;
        else if (a == "--deterministic") o.deterministic = true;
        else if (a == "--iters" && i + 1 < argc) o.iters = std::atoi(argv[++i]);
        else if (a == "--warmup" && i + 1 < argc) o.warmup = std::atoi(argv[++i]);
        else if (a == "--runs" && i + 1 < argc) o.runs = std::atoi(argv[++i]);
        else if (a == "--gpus" && i + 1 < argc) o.gpus = std::atoi(argv[++i]);
        else if (npos < 6) pos[npos++] = std::atoi(argv[i]);
    }
    o.B = pos[0]; o.Hq = pos[1]; o.Hkv = pos[2]; o.S = pos[3]; o.D = pos[4]; o.causal = pos[5];
    const int B = o.B, Hq = o.Hq, Hkv = o.Hkv, S = o.S, D = o.D;
    if (gqa_bwd_workspace_bytes(B, Hq, Hkv, S, D, o.causal) == 0) {
        std::fprintf(stderr, "unsupported shape\n");
        return 1;
    }
    const int G = Hq / Hkv, n_groups = B * Hkv;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || o.gpus < 1 || o.gpus > n_dev || o.gpus > n_groups) {
        std::fprintf(stderr, "--gpus %d: %d device(s) visible, %d groups\n", o.gpus, n_dev, n_groups);
        return 1;
    }
    const size_t nq = (size_t)B * Hq * S * D, nkv = (size_t)B * Hkv * S * D, nl = (size_t)B * Hq * S;
    std::printf("GQA bench: B=%d Hq=%d Hkv=%d (G=%d) S=%d D=%d causal=%d gpus=%d  lib %s\n", B, Hq, Hkv, G, S, D, o.causal,
                o.gpus, gqa_version());

    HostData h;
    h.q.resize(nq); h.d_o.resize(nq); h.k.resize(nkv); h.v.resize(nkv);
    if (!o.synthetic) {
        auto path = [&](const char* name) { return o.data + "/gqa_" + name + ".bin"; };
        bool ok = loadBin(path("q").c_str(), h.q.data(), nq) && loadBin(path("k").c_str(), h.k.data(), nkv) &&
                  loadBin(path("v").c_str(), h.v.data(), nkv) && loadBin(path("do").c_str(), h.d_o.data(), nq);
        if (!ok) {
            std::fprintf(stderr, "missing inputs under %s: run `python oracle/make_ref.py %d %d %d %d %d %d` or pass --synthetic\n",
                         o.data.c_str(), B, Hq, Hkv, S, D, o.causal);
            return 1;
        }
        h.ref_o.resize(nq); h.ref_lse.resize(nl); h.ref_dq.resize(nq); h.ref_dk.resize(nkv); h.ref_dv.resize(nkv);
        h.have_ref = loadBin(path("o").c_str(), h.ref_o.data(), nq) && loadBin(path("lse").c_str(), h.ref_lse.data(), nl) &&
                     loadBin(path("dq").c_str(), h.ref_dq.data(), nq) && loadBin(path("dk").c_str(), h.ref_dk.data(), nkv) &&
                     loadBin(path("dv").c_str(), h.ref_dv.data(), nkv);
        if (!h.have_ref) return 1;
    } else {
        fill_normal(h.q, 42);
        fill_normal(h.k, 43);
        fill_normal(h.v, 44);
        fill_normal(h.d_o, 45);
    }

    std::vector<ShardResult> res(o.gpus);
    if (o.gpus == 1) {
        run_shard(0, o, h, 0, n_groups, B, Hq, Hkv, res[0]);
    } else {
        std::vector<std::thread> th;
        for (int d = 0; d < o.gpus; ++d) {
            const int base = n_groups / o.gpus, extra = n_groups % o.gpus;
            const int g0 = d * base + std::min(d, extra), g1 = g0 + base + (d < extra ? 1 : 0);
            th.emplace_back([&, d, g0, g1] { run_shard(d, o, h, g0, g1, g1 - g0, G, 1, res[d]); });
        }
        for (auto& t : th) t.join();
    }
    bool pass = true, det = true;
    double bwd_ms = 0, fwd_ms = 0, dq_delta = 0;
    for (const ShardResult& r : res) {
        if (r.rc) return r.rc;
        pass &= r.pass;
        det &= r.dkdv_identical;
        bwd_ms = std::max(bwd_ms, r.bwd_ms);
        fwd_ms = std::max(fwd_ms, r.fwd_ms);
        dq_delta = std::max(dq_delta, r.dq_max_delta);
    }
    std::printf("\ndeterminism over 8 runs: dK/dV %s, dQ max|delta| = %.3e\n", det ? "bit-identical" : "DIFFER", dq_delta);
    displayStats("gqa_bwd (device 0, last run)", res[0].last_bwd);
    displayStats("gqa_fwd (device 0, last run)", res[0].last_fwd);
    const double f = 4.0 * B * Hq * (double)S * S * D * (o.causal ? 0.5 : 1.0);
    const double tf_b = 4.0 * f / (bwd_ms * 1e9), tf_f = f / (fwd_ms * 1e9);
    std::printf("\nmedian of %d run medians (slowest of %d device(s)): bwd %.4f ms = %.1f TFLOP/s (4x-forward convention; "
                "%.1f executed-MMA), %.1f%% of %d x 2250 nominal; fwd %.4f ms = %.1f TFLOP/s\n",
                o.runs, o.gpus, bwd_ms, tf_b, tf_b * 2.5 / 4.0, 100.0 * tf_b / (2250.0 * o.gpus), o.gpus, fwd_ms, tf_f);
    // The precision gate only exists with golden files: with --synthetic nothing was compared, and the line says so
    // (gate_pass null, no rel_rms) instead of reporting a gate that did not run.
    char gate[256];
    if (h.have_ref) {
        PrecisionReport worst[5];  // over the shards: the largest relative RMS per tensor
        for (const ShardResult& r : res)
            for (int i = 0; i < 5; ++i)
                if (r.rep[i].rel_rms >= worst[i].rel_rms) worst[i] = r.rep[i];
        std::snprintf(gate, sizeof gate,
                      "\"gate_pass\": %s, \"rel_rms\": {\"O\": %.3e, \"dQ\": %.3e, \"dK\": %.3e, \"dV\": %.3e}, "
                      "\"max_abs\": {\"O\": %.3e, \"dQ\": %.3e, \"dK\": %.3e, \"dV\": %.3e}",
                      pass ? "true" : "false", worst[0].rel_rms, worst[2].rel_rms, worst[3].rel_rms, worst[4].rel_rms,
                      worst[0].max_abs, worst[2].max_abs, worst[3].max_abs, worst[4].max_abs);
    } else {
        std::snprintf(gate, sizeof gate, "\"gate_pass\": null, \"outputs_finite\": %s", pass ? "true" : "false");
    }
    std::printf("{\"harness\": \"gqa_bench\", \"B\": %d, \"Hq\": %d, \"Hkv\": %d, \"S\": %d, \"D\": %d, \"causal\": %d, "
                "\"gpus\": %d, \"bwd_ms_median\": %.5f, \"bwd_tflops\": %.2f, \"fwd_ms_median\": %.5f, \"fwd_tflops\": %.2f, "
                "%s, \"dkdv_bit_identical\": %s, \"dq_max_run_delta\": %.3e, \"kernel_launches\": %llu}\n",
                B, Hq, Hkv, S, D, o.causal, o.gpus, bwd_ms, tf_b, fwd_ms, tf_f, gate, det ? "true" : "false", dq_delta,
                gqa_launch_count());
    return pass ? 0 : 4;
}
