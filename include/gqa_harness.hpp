// Host-side precision and timing harness, source-compatible with the helpers the
// reference's C++ drivers use: loadBin / saveBin / reportPrecision / checkResult
// (include/utils/kernelUtils.cuh:69-118, :176-191) and benchmarkKernel /
// displayStats / KernelStats (include/utils/kernelBench.cuh:12-117).  A driver
// written against those headers compiles against this one unchanged.
//
// Differences, all additive:
//   * nothing here calls exit(): loaders return false, checks return a verdict;
//   * reportPrecision also returns its numbers (plus the relative RMS error);
//   * benchmarkKernel keeps the reference's avg-based TFLOPS field and adds the
//     median-based figure (the reference prints TFLOPS computed from the average).
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <string>
#include <vector>

#ifndef CUDA_CHECK
// Same name as the reference macro; on failure it reports and returns false/non-zero
// from the enclosing function instead of terminating the process.
#define CUDA_CHECK(call)                                                                      \
    do {                                                                                      \
        const cudaError_t status__ = (call);                                                  \
        if (status__ != cudaSuccess) {                                                        \
            std::fprintf(stderr, "CUDA error at %s:%d: %s (%s)\n", __FILE__, __LINE__,        \
                         cudaGetErrorName(status__), cudaGetErrorString(status__));           \
            return {};                                                                        \
        }                                                                                     \
    } while (0)
#endif

// ---- raw float32 files (numpy .tofile()) ------------------------------------------------------

inline bool loadBin(const char* path, float* buf, size_t n) {
    std::FILE* f = std::fopen(path, "rb");
    if (!f) {
        std::fprintf(stderr, "loadBin: cannot open %s\n", path);
        return false;
    }
    const size_t got = std::fread(buf, sizeof(float), n, f);
    std::fclose(f);
    if (got != n) std::fprintf(stderr, "loadBin: expected %zu floats, got %zu from %s\n", n, got, path);
    return got == n;
}

inline bool saveBin(const char* path, const float* buf, size_t n) {
    std::FILE* f = std::fopen(path, "wb");
    if (!f) {
        std::fprintf(stderr, "saveBin: cannot open %s\n", path);
        return false;
    }
    const size_t put = std::fwrite(buf, sizeof(float), n, f);
    std::fclose(f);
    return put == n;
}

// ---- precision -----------------------------------------------------------------------------

struct PrecisionReport {
    double max_abs = 0, mean_abs = 0, max_rel = 0, rel_rms = 0;
};

// max |ref-got|, mean |ref-got|, max relative error (relative only where |ref| > 1e-5, as the
// reference does) and the relative RMS error ||ref-got||_2 / ||ref||_2.
inline PrecisionReport reportPrecision(const char* label, const float* ref, const float* got, size_t n) {
    PrecisionReport r;
    double sum_abs = 0, sum_sq = 0, ref_sq = 0;
    for (size_t i = 0; i < n; ++i) {
        const double a = ref[i], b = got[i];
        const double d = std::fabs(a - b), mag = std::fabs(a);
        r.max_abs = std::max(r.max_abs, d);
        r.max_rel = std::max(r.max_rel, mag > 1e-5 ? d / mag : d);
        sum_abs += d;
        sum_sq += d * d;
        ref_sq += a * a;
    }
    r.mean_abs = n ? sum_abs / (double)n : 0.0;
    r.rel_rms = ref_sq > 0 ? std::sqrt(sum_sq / ref_sq) : std::sqrt(sum_sq);
    std::printf("%s  max_abs=%.3e  mean_abs=%.3e  max_rel=%.3e  rel_rms=%.3e\n", label, r.max_abs, r.mean_abs,
                r.max_rel, r.rel_rms);
    return r;
}

// Element-wise gate |ref - got| <= atol + rtol * |ref| (defaults as in the reference); prints the
// first offender, returns the verdict.  NaN in `got` fails.
inline bool checkResult(const float* hostRef, const float* gpuRef, size_t n, float atol = 1e-5f, float rtol = 1.3e-6f) {
    for (size_t i = 0; i < n; ++i) {
        const float d = std::fabs(hostRef[i] - gpuRef[i]);
        const float tol = atol + rtol * std::fabs(hostRef[i]);
        if (!(d <= tol)) {
            std::printf("\033[31mValues don't match at index %zu!\nRef: %.8f, GPU: %.8f  diff=%.8f tol=%.8f\033[0m\n", i,
                        hostRef[i], gpuRef[i], d, tol);
            return false;
        }
    }
    std::printf("\033[32mValues match!\033[0m\n");
    return true;
}

// ---- timing --------------------------------------------------------------------------------

struct KernelStats {
    float avg_ms = 0, median_ms = 0, std_dev_ms = 0, min_ms = 0, max_ms = 0;
    double tflops = 0;          // from the average, as the reference computes it
    double bandwidth_gb_s = 0;  // from the average
    double tflops_median = 0;   // from the median
    bool valid = false;
};

// Times `kernel_launch` num_iters times with CUDA events on the legacy default stream after
// num_warmup untimed calls.  Before every timed call a 256 MB buffer is overwritten so the
// working set starts outside L2 (the B200 L2 is 126 MB).
template <typename Func>
KernelStats benchmarkKernel(Func kernel_launch, int num_iters = 100, int num_warmup = 10, long long total_flops = 0,
                            size_t total_bytes = 0) {
    constexpr size_t kFlushBytes = size_t(256) << 20;
    KernelStats st;
    cudaEvent_t start = nullptr, stop = nullptr;
    void* flush = nullptr;
    CUDA_CHECK(cudaEventCreate(&start));
    CUDA_CHECK(cudaEventCreate(&stop));
    CUDA_CHECK(cudaMalloc(&flush, kFlushBytes));
    for (int i = 0; i < num_warmup; ++i) kernel_launch();
    CUDA_CHECK(cudaDeviceSynchronize());

    std::vector<float> ms(num_iters > 0 ? num_iters : 0);
    for (float& t : ms) {
        CUDA_CHECK(cudaMemsetAsync(flush, 0, kFlushBytes, 0));
        CUDA_CHECK(cudaEventRecord(start, 0));
        kernel_launch();
        CUDA_CHECK(cudaEventRecord(stop, 0));
        CUDA_CHECK(cudaEventSynchronize(stop));
        CUDA_CHECK(cudaEventElapsedTime(&t, start, stop));
    }
    CUDA_CHECK(cudaFree(flush));
    CUDA_CHECK(cudaEventDestroy(start));
    CUDA_CHECK(cudaEventDestroy(stop));
    if (ms.empty()) return st;

    std::sort(ms.begin(), ms.end());
    const size_t n = ms.size();
    double sum = 0, sq = 0;
    for (float t : ms) {
        sum += t;
        sq += (double)t * t;
    }
    st.avg_ms = (float)(sum / n);
    st.median_ms = (n % 2) ? ms[n / 2] : 0.5f * (ms[n / 2 - 1] + ms[n / 2]);
    st.std_dev_ms = (float)std::sqrt(std::max(0.0, sq / n - (sum / n) * (sum / n)));
    st.min_ms = ms.front();
    st.max_ms = ms.back();
    if (total_flops > 0) {
        st.tflops = (double)total_flops / (st.avg_ms * 1e9);
        st.tflops_median = (double)total_flops / (st.median_ms * 1e9);
    }
    if (total_bytes > 0) st.bandwidth_gb_s = (double)total_bytes / (st.avg_ms * 1e6);
    st.valid = true;
    return st;
}

inline void displayStats(const std::string& name, const KernelStats& s) {
    std::printf("\n----------------------------------------------------------\n");
    std::printf("Benchmark: %s\n", name.c_str());
    std::printf("----------------------------------------------------------\n");
    std::printf("Average Time:  %10.4f ms\nMedian Time:   %10.4f ms\nStd Dev:       %10.4f ms\n", s.avg_ms, s.median_ms,
                s.std_dev_ms);
    std::printf("Min Time:      %10.4f ms\nMax Time:      %10.4f ms\n", s.min_ms, s.max_ms);
    if (s.tflops > 0) {
        std::printf("Performance:   %10.4f TFLOPS\n", s.tflops);
        std::printf("  (median)     %10.4f TFLOPS\n", s.tflops_median);
    }
    if (s.bandwidth_gb_s > 0) std::printf("Bandwidth:     %10.4f GB/s\n", s.bandwidth_gb_s);
    std::printf("----------------------------------------------------------\n");
}
