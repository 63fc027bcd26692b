// Host-side services shared by every entry point: error text, launch counting,
// tensor-map encoding through the driver entry point (no link-time libcuda
// dependency), status strings.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "gqa_common.cuh"

namespace gqa {

static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches{0};

int note_cuda_error(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof g_err, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    return GQA_ERR_CUDA;
}
int note_driver_error(CUresult r, const char* what) {
    snprintf(g_err, sizeof g_err, "%s: CUresult %d", what, (int)r);
    return GQA_ERR_CUDA;
}
int note_device_timeout(unsigned int word) {
    snprintf(g_err, sizeof g_err, "device status 0x%08x: wait site %u gave up in block %u", word, (word >> 20) & 0x7ffu,
             word & 0xfffffu);
    return GQA_ERR_DEVICE_TIMEOUT;
}
void note_text(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}
void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Encoding a tensor map costs several microseconds of host time and the same few (pointer, shape) pairs
// recur call after call, so the last encodings are kept per host thread.
struct TmapKey {
    const void* base;
    uint64_t rows, cols;
    uint32_t box_rows, kind;
    uint64_t n_outer = 0, outer_stride = 0;  // 3-D maps only
    bool operator==(const TmapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && kind == o.kind &&
               n_outer == o.n_outer && outer_stride == o.outer_stride;
    }
};
struct TmapCache {
    static constexpr int kSlots = 32;
    TmapKey keys[kSlots] = {};
    CUtensorMap maps[kSlots];
    bool used[kSlots] = {};
    int next = 0;
    bool find(const TmapKey& k, CUtensorMap* out) const {
        for (int i = 0; i < kSlots; ++i)
            if (used[i] && keys[i] == k) {
                *out = maps[i];
                return true;
            }
        return false;
    }
    void put(const TmapKey& k, const CUtensorMap& m) {
        keys[next] = k;
        maps[next] = m;
        used[next] = true;
        next = (next + 1) % kSlots;
    }
};
static thread_local TmapCache g_tmaps;

int make_panel_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    const TmapKey key{base, rows, cols, box_rows, 0u};
    if (g_tmaps.find(key, out)) return GQA_OK;
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not available");
        return GQA_ERR_CUDA;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * sizeof(__nv_bfloat16)};
    cuuint32_t box[2] = {64u, box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return note_driver_error(r, "cuTensorMapEncodeTiled");
    g_tmaps.put(key, *out);
    return GQA_OK;
}

namespace {
// kind: 3 = bf16 tile, 4 = fp32 box, 5 = bf16 column panel
int make_tmap3(CUtensorMap* out, const void* base, uint64_t cols, uint64_t S, uint64_t n_outer, uint64_t outer_stride,
               uint32_t box_cols, uint32_t box_rows, uint32_t kind) {
    const TmapKey key{base, S, cols, box_rows, kind, n_outer, outer_stride};
    if (g_tmaps.find(key, out)) return GQA_OK;
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not available");
        return GQA_ERR_CUDA;
    }
    const bool f32 = (kind == 4);
    const uint64_t esz = f32 ? sizeof(float) : sizeof(__nv_bfloat16);
    cuuint64_t dims[3] = {cols, S, n_outer};
    cuuint64_t strides[2] = {cols * esz, outer_stride * esz};
    cuuint32_t box[3] = {box_cols, box_rows, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    kind == 5 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                    kind == 5 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return note_driver_error(r, "cuTensorMapEncodeTiled(3-D)");
    g_tmaps.put(key, *out);
    return GQA_OK;
}
}  // namespace

int make_tile3_tmap(CUtensorMap* out, const void* base, uint64_t cols, uint64_t S, uint64_t n_outer,
                    uint64_t outer_stride, uint32_t box_rows) {
    return make_tmap3(out, base, cols, S, n_outer, outer_stride, 64u, box_rows, 3u);
}
int make_f32box3_tmap(CUtensorMap* out, const void* base, uint64_t cols, uint64_t S, uint64_t n_outer, uint32_t box_rows) {
    return make_tmap3(out, base, cols, S, n_outer, S * cols, 32u, box_rows, 4u);
}
int make_col8_3_tmap(CUtensorMap* out, const void* base, uint64_t S, uint64_t n_outer, uint32_t box_rows) {
    return make_tmap3(out, base, 8, S, n_outer, S * 8, 8u, box_rows, 5u);
}

// Status word of the forward kernels: a fixed device array (no allocation), one per GPU that loads the library.
// Reports are sticky: a kernel writes the word only while it is zero, no launch clears it, and
// gqa_check_status(NULL, ...) clears it after reading, so forwards on different streams cannot erase each
// other's report.  Until it has been read, later forward launches on that device return without computing.
static __device__ __align__(256) unsigned int g_forward_status[64];

int forward_status_word(unsigned int** out) {
    constexpr int kMaxDev = 64;
    static unsigned int* words[kMaxDev] = {};
    static std::mutex mu;
    int dev = 0;
    GQA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) return GQA_ERR_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev]) {
        // in host code the array's name is a handle for the runtime, not an address a kernel can use
        void* p = nullptr;
        GQA_CUDA_TRY(cudaGetSymbolAddress(&p, g_forward_status));
        if (!p) return GQA_ERR_CUDA;
        words[dev] = static_cast<unsigned int*>(p);
    }
    *out = words[dev];
    return GQA_OK;
}

}  // namespace gqa

extern "C" const char* gqa_status_string(int status) {
    switch (status) {
        case GQA_OK: return "ok";
        case GQA_ERR_BAD_ARGUMENT: return "bad argument (null, non-positive or misaligned)";
        case GQA_ERR_UNSUPPORTED: return "unsupported shape (need D a multiple of 8 up to 128 (64 or 128 with GQA_LAYOUT_BSHD), Hq % Hkv == 0, B*Hq*S < 2^31)";
        case GQA_ERR_WORKSPACE: return "workspace missing or too small";
        case GQA_ERR_CUDA: return "CUDA call failed";
        case GQA_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        case GQA_ERR_ARCH: return "device is not compute capability 10.x";
        default: return "unknown status";
    }
}
extern "C" const char* gqa_last_cuda_error(void) { return gqa::g_err; }
extern "C" unsigned long long gqa_launch_count(void) { return gqa::g_launches.load(); }
extern "C" const char* gqa_version(void) { return "0.1"; }
