/*
 * gqa.h -- C ABI of the Blackwell (sm_100a) grouped-query-attention library.
 *
 * Every entry point takes plain device pointers and sizes; nothing here depends
 * on a framework.  Tensor contract (same as the reference launchers):
 *   Q, O, dO, dQ : [B, Hq,  S, D]  bf16, contiguous, row-major
 *   K, V, dK, dV : [B, Hkv, S, D]  bf16, contiguous, row-major
 *   LSE          : [B, Hq, S]      fp32, natural log of sum_j exp(scale * q_i . k_j)
 *   query head hq reads KV head hq / (Hq / Hkv)
 * Supported: D a multiple of 8 up to 128 (the reference's tensor-core kernels fix D = 128, its first two
 * generations take D % 16 == 0, src/attention/GQA_bwd.cu:391-393; here D = 64 and D = 128 are the native sizes and
 * the others run on the next one up, reading the missing columns as zeros), any S >= 1 (the reference needs
 * S % 64 == 0 in the backward,
 * src/attention/GQA_bwd_baseline.cu:549-602, and S % 256 == 0 in the forward,
 * src/attention/GQA_fwd_ref.cu:352; here a partial last tile is masked), Hq a multiple of Hkv,
 * all pointers 16-byte aligned, scale finite and > 0.  Anything else returns an error code; the
 * library never exits the process and never traps the device.
 *
 * All functions return GQA_OK (0) or a negative gqa_status.  Work is enqueued
 * on `stream`; the functions do not synchronise it unless stated.
 */
#ifndef GQA_B200_H_
#define GQA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* gqa_stream_t; /* same handle as cudaStream_t */

typedef enum gqa_status {
    GQA_OK = 0,
    GQA_ERR_BAD_ARGUMENT = -1,   /* null pointer, non-positive size, misaligned pointer, scale not finite or <= 0 */
    GQA_ERR_UNSUPPORTED = -2,    /* shape outside the supported set (D % 8 == 0, D <= 128, Hq % Hkv == 0) */
    GQA_ERR_WORKSPACE = -3,      /* workspace missing or smaller than gqa_bwd_workspace_bytes() */
    GQA_ERR_CUDA = -4,           /* a CUDA runtime/driver call failed (see gqa_last_cuda_error) */
    GQA_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait gave up; outputs are invalid */
    GQA_ERR_ARCH = -6            /* the current device is not compute capability 10.x */
} gqa_status;

/*
 * Forward: O = softmax(scale * Q K^T [+ causal mask]) V and LSE.
 * Replaces launch_gqa_v62(Q,K,V,O,LSE,B,Hq,Hkv,S,scale,stream)
 * (src/attention/GQA_fwd_ref.cu:631-651), with D and causal made runtime arguments.
 * LSE may be NULL when the caller does not need it.
 */
int gqa_fwd(const void* Q, const void* K, const void* V, void* O, float* LSE,
            int B, int Hq, int Hkv, int S, int D, int causal, float scale,
            gqa_stream_t stream);

/*
 * Alias of gqa_fwd under the entry name the reference's Python harness loads from a
 * user-supplied shared object (harness/competitors.py:396-415, entry="launch_gqa").
 */
int launch_gqa(const void* Q, const void* K, const void* V, void* O, float* LSE,
               int B, int Hq, int Hkv, int S, int D, int causal, float scale,
               gqa_stream_t stream);

/*
 * gqa_fwd with option flags.  flags = 0 is gqa_fwd.
 * GQA_LAYOUT_BSHD: Q and O are [B,S,Hq,D] and K and V [B,S,Hkv,D] (sequence-major, the layout the reference's
 * harness hands to the FlashAttention and FlashInfer adapters, harness/competitors.py:116-122) instead of the
 * canonical [B,H,S,D]; the tiles are fetched through tensor maps over the B matrices [S, H*D], so no transposed
 * copy is made.  LSE stays [B,Hq,S].  This layout needs D = 64 or D = 128 (a head's columns are followed by the
 * next head's, so nothing reads as zero padding).  Unknown flag bits are refused with GQA_ERR_BAD_ARGUMENT.
 */
#define GQA_LAYOUT_BSHD 2u
int gqa_fwd_ex(const void* Q, const void* K, const void* V, void* O, float* LSE,
               int B, int Hq, int Hkv, int S, int D, int causal, float scale,
               gqa_stream_t stream, unsigned int flags);

/*
* Bytes of device scratch gqa_bwd needs for this shape (per-row LSE and Delta terms,
 * the fp32 dQ accumulator and a status word).  The reference keeps the same buffers as
 * function-static allocations inside its launcher
 * (src/attention/GQA_bwd_baseline.cu:579-587); here the caller owns them.
 */
size_t gqa_bwd_workspace_bytes(int B, int Hq, int Hkv, int S, int D, int causal);

/*
 * Backward: dQ, dK, dV from Q, K, V, O, dO and LSE.
 * Replaces launch_gqa_backward_vj1d<Br,Bc,D>(Q,K,V,O,dO,LSE,dQ,dK,dV,B,Hq,Hkv,G,S,scale)
 * (src/attention/GQA_bwd_baseline.cu:549-602; the same argument list is used by every
 * launcher in src/attention/GQA_bwd.cu).  G is derived as Hq / Hkv.
 * `workspace` must be 256-byte aligned device memory of at least
 * gqa_bwd_workspace_bytes(...) bytes; calls that share a workspace must not overlap.
 * dK and dV are bit-reproducible from run to run; dQ is summed over the KV tiles by fp32 TMA reduce-add
 * operations at L2 whose order varies from run to run (see GQA_BWD_DETERMINISTIC below).
 */
int gqa_bwd(const void* Q, const void* K, const void* V, const void* O, const void* dO,
            const float* LSE, void* dQ, void* dK, void* dV,
            int B, int Hq, int Hkv, int S, int D, int causal, float scale,
            void* workspace, size_t workspace_bytes, gqa_stream_t stream);

/*
 * gqa_bwd with option flags.  flags = 0 is gqa_bwd.
 * GQA_BWD_DETERMINISTIC: the fp32 reductions into every 32-row slice of the dQ accumulator are applied in
 * KV-tile order (a counter per slice in the workspace hands the turn from one thread block to the next), so dQ
 * is bit-reproducible from run to run as dK and dV always are.  The reference's dQ path is order-dependent
 * (cp.reduce.async.bulk add, src/attention/GQA_bwd_baseline.cu:360-365, run-to-run differences noted in
 * docs/report.md:115-116) and has no such switch; its determinism probe
 * (precision/vj1d_determinism_probe.cu:33) is what this mode is checked with.  Slower than the default
 * (the thread blocks of one (batch, KV head) group reduce one after the other).  Same workspace size.  This mode
 * runs one thread block per KV tile (the default mode runs one persistent block per SM): a thread block waits for
 * the turn of the block that owns the previous KV tile of its group, which has a smaller block index, so the mode
 * relies on the hardware starting thread blocks in index order (it does on every CUDA GPU so far, but CUDA does
 * not promise it); the wait is bounded, so a violation would end in GQA_ERR_DEVICE_TIMEOUT, not in a hang.
 * dK and dV of this mode and of the default mode are each bit-reproducible; without a causal mask they differ from
 * each other in the last bits (the default mode starts every KV tile's loop over the query tiles at another tile).
 * GQA_LAYOUT_BSHD (see gqa_fwd_ex): Q, O, dO, dQ are [B,S,Hq,D] and K, V, dK, dV [B,S,Hkv,D]; LSE stays [B,Hq,S].
 * Unknown flag bits are refused with GQA_ERR_BAD_ARGUMENT.
 * GQA_BWD_SPLIT_HEADS: for calls with too few KV tiles to fill the GPU evenly (fewer than two per SM: a
 * long-context problem sharded down to one KV head per GPU, where the longest causal tile alone outlasts the
 * per-SM average).  The library may then cut every KV tile's work over several thread blocks that each loop over a
 * part of the group's query heads, store fp32 partial dK / dV sums in the workspace and add them in a fixed order
 * (the reference's per-head grid + gqa_dkdv_greduce, src/attention/GQA_bwd_baseline.cu:385-403, :594-599, on fp32
 * partials).  Whether and how far it splits is a function of the shape only (an estimate of the schedule's
 * makespan); dK and dV stay bit-reproducible from run to run, but their last bits depend on the split, so results
 * are no longer bit-identical across different shardings of one problem, which is why this is a flag.  The
 * workspace must come from gqa_bwd_workspace_bytes_ex with the same flags.
 * GQA_BWD_DQ_SEPARATE: compute dQ in a separate query-parallel pass (one thread block per 128-row query tile looping
 * over the key tiles, as the reference's first generations do, src/attention/GQA_bwd.cu:29, :415, :1416) instead
 * of accumulating the main kernel's dQ tiles with fp32 reductions.  S and dP are then computed twice, but dQ needs
 * no accumulator, no finalise pass, and is bit-reproducible by construction.  Measured 1.3-1.7x slower than the
 * default at the benchmark shapes, and slower than GQA_BWD_DETERMINISTIC's ordered reductions at all of them but one
 * (B4 Hq32 Hkv8 S8192 D128 causal: 7.7 against 8.6 ms), so no mode selects it by itself.  Same workspace size.
 */
#define GQA_BWD_DETERMINISTIC 1u
#define GQA_BWD_SPLIT_HEADS 4u
#define GQA_BWD_DQ_SEPARATE 8u
size_t gqa_bwd_workspace_bytes_ex(int B, int Hq, int Hkv, int S, int D, int causal, unsigned int flags);
int gqa_bwd_ex(const void* Q, const void* K, const void* V, const void* O, const void* dO,
               const float* LSE, void* dQ, void* dK, void* dV,
               int B, int Hq, int Hkv, int S, int D, int causal, float scale,
               void* workspace, size_t workspace_bytes, gqa_stream_t stream, unsigned int flags);

/*
 * Backward for callers that cannot allocate device memory.  No counterpart in the
 * reference (its launcher grows function-static cudaMalloc buffers on demand).
 *
 * Some hosts of this library may not call cudaMalloc at the point where they need a
 * backward pass: code running inside a framework's memory-planned region, a plugin that
 * is handed only its input and output buffers, a real-time loop where an allocation
 * could stall or fail.  gqa_bwd asks such a caller for a workspace it cannot provide.
 * This variant takes its scratch (Delta, scaled LSE, the fp32 dQ accumulator, the status
 * word) from one fixed array compiled into the library, gqa_bwd_static_scratch_bytes()
 * = 32 MiB, resident on every GPU that loads the library until the process exits.  The
 * caller still passes all inputs and outputs; results equal gqa_bwd's.
 *
 *  - Shapes whose scratch (gqa_bwd_workspace_bytes) exceeds the array are refused with
 *    GQA_ERR_WORKSPACE and an explanation in gqa_last_cuda_error(); nothing is launched.
 *    32 MiB covers e.g. B*Hq*S <= 114 000 rows at D <= 64 or 61 000 rows at D <= 128.
 *  - It calls no cudaMalloc/cudaFree and no allocating library routine.
 *  - The first call on each device looks up the array's device address (one runtime
 *    query, no allocation).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array, and it keeps what the last call left;
 *    each call re-initialises the parts it reads, so back-to-back calls on one stream
 *    are fine, but two calls that overlap on the GPU (different streams, or threads
 *    without ordering) race on it and produce wrong gradients.
 *  - gqa_check_status() cannot be pointed at the array; use gqa_bwd when the status
 *    word matters.
 */
size_t gqa_bwd_static_scratch_bytes(void);
int gqa_bwd_static_scratch(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                           const float* LSE, void* dQ, void* dK, void* dV,
                           int B, int Hq, int Hkv, int S, int D, int causal, float scale,
                           gqa_stream_t stream);

/*
 * Packed variable-length batches (no counterpart in the reference, whose kernels take one S for the whole batch:
 * src/attention/GQA_bwd_baseline.cu:549-554; listed among the shape generalisations a drop-in should add).
 * n_seqs sequences of different lengths lie back to back, sequence-major: Q, O, dO, dQ are [total_tokens, Hq, D],
 * K, V, dK, dV [total_tokens, Hkv, D], LSE [Hq, total_tokens]; sequence i owns the rows cu_seqlens[i] ..
 * cu_seqlens[i+1]-1 and attends only to itself (causal: inside the sequence).  cu_seqlens is n_seqs + 1 int32 in
 * DEVICE memory, cu_seqlens[0] = 0, non-decreasing, cu_seqlens[n_seqs] = total_tokens; max_seqlen must be at least
 * the longest length (it sizes the launch; a larger value only costs empty thread blocks).  The library reads
 * cu_seqlens on the device only, so it cannot check these rules: a longer sequence than max_seqlen is silently
 * truncated in the forward and loses KV tiles in the backward.  Empty sequences are allowed.  D = 64 or 128.
 * The tiles of a sequence are fetched at its row offset through the same tensor maps as GQA_LAYOUT_BSHD with B = 1;
 * rows beyond the end of a sequence (the next sequence's) are masked in the kernels.
 * gqa_bwd_varlen takes a workspace of gqa_bwd_varlen_workspace_bytes(...) bytes under the rules of gqa_bwd; dK and
 * dV are bit-reproducible, dQ is summed by fp32 reduce-add operations (no ordered mode for packed batches).
 */
int gqa_fwd_varlen(const void* Q, const void* K, const void* V, void* O, float* LSE,
                   const int* cu_seqlens, int n_seqs, int total_tokens, int max_seqlen,
                   int Hq, int Hkv, int D, int causal, float scale, gqa_stream_t stream);
size_t gqa_bwd_varlen_workspace_bytes(int total_tokens, int Hq, int Hkv, int D);
int gqa_bwd_varlen(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                   const float* LSE, void* dQ, void* dK, void* dV,
                   const int* cu_seqlens, int n_seqs, int total_tokens, int max_seqlen,
                   int Hq, int Hkv, int D, int causal, float scale,
                   void* workspace, size_t workspace_bytes, gqa_stream_t stream);

/*
 * gqa_bwd with CUDA events recorded on `stream` around its three stages.  Fills
 * stage_ms[0..2] (host memory) with the device time of the Delta preprocess, the
 * tensor-core main kernel and the dQ finalise, and synchronises the stream.  The
 * reference times only the whole launcher (src/attention/GQA_bwd_baseline.cu:684-687);
 * this entry point exists so that the roofline of the dominant kernel can be
 * measured on the launching stream.
 */
int gqa_bwd_stage_times(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                        const float* LSE, void* dQ, void* dK, void* dV,
                        int B, int Hq, int Hkv, int S, int D, int causal, float scale,
                        void* workspace, size_t workspace_bytes, gqa_stream_t stream,
                        float* stage_ms);

/*
 * Delta preprocess on its own: delta[r] = sum_d dO[r,d] * O[r,d] for `rows` rows.
 * Replaces compute_drowsum_v22 (src/attention/GQA_bwd_baseline.cu:273-298).
 */
int gqa_bwd_delta(const void* O, const void* dO, float* delta, size_t rows, int D,
                  gqa_stream_t stream);

/*
 * Reads the status word a previous gqa_fwd/gqa_bwd left on the device and returns
 * GQA_OK or GQA_ERR_DEVICE_TIMEOUT (which wait gave up, in which thread block: gqa_last_cuda_error()).
 * Synchronises `stream`.  For gqa_bwd pass the same workspace (its first word is the status word, cleared
 * at the start of every gqa_bwd call).  For gqa_fwd pass NULL: the forward reports into a 256-byte
 * device array that is part of the library, one per GPU, no allocation.  That report is sticky, like a
 * CUDA error: no launch clears it, so forwards running on several streams cannot erase each other's
 * report, and while it is set every later gqa_fwd on that GPU returns without computing (its thread
 * blocks exit at once).  Reading it with this function clears it.  In both kernels a thread block that
 * starts after another one has given up exits immediately, and the persistent blocks of the backward stop taking
 * work once the word is set, so a wedged launch drains within one wait limit.
 * The reference has no such path: its waits spin without limit (src/attention/GQA_bwd_baseline.cu:85-93).
 */
int gqa_check_status(const void* workspace, gqa_stream_t stream);

/* Human-readable text for a gqa_status. */
const char* gqa_status_string(int status);

/* Text of the last CUDA error or device-timeout report this library saw on the calling thread ("" if none). */
const char* gqa_last_cuda_error(void);

/* Kernels launched by this library since load (all entry points, all threads). */
unsigned long long gqa_launch_count(void);

/* Library version, "major.minor". */
const char* gqa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GQA_B200_H_ */
