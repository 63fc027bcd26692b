// Shared host-side plumbing for the library's translation units: status codes,
// CUDA error capture, the launch counter and tensor-map construction.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gqa.h"

namespace gqa {

// Records the error text for gqa_last_cuda_error() and returns GQA_ERR_CUDA.
int note_cuda_error(cudaError_t e, const char* what);
int note_driver_error(CUresult r, const char* what);
void count_launch(unsigned n = 1);
// printf-style text for gqa_last_cuda_error() (argument errors that deserve an explanation).
void note_text(const char* fmt, ...);
// Records which bounded wait gave up (decoded from the device status word); returns GQA_ERR_DEVICE_TIMEOUT.
int note_device_timeout(unsigned int word);

#define GQA_CUDA_TRY(expr)                                          \
    do {                                                            \
        cudaError_t e__ = (expr);                                   \
        if (e__ != cudaSuccess) return gqa::note_cuda_error(e__, #expr); \
    } while (0)

// 2-D bf16 tensor map over a row-major [rows, cols] matrix, box = [box_rows, 64 columns],
// 128-byte swizzle: one box is a panel of box_rows rows x 128 bytes (used by the UMMA self test).
int make_panel_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// 3-D tensor maps over `n_outer` row-major [S, cols] matrices that lie outer_stride elements apart
// (coordinates: x = column, y = row inside the matrix, z = matrix).  Rows at y >= S are out of bounds: loads
// read zeros there and stores / reductions skip them, which is what lets S be any length.
//   tile3: bf16, box = [box_rows, 64 columns], 128-byte swizzle (one box = a panel, as make_panel_tmap).
//   f32box3: fp32, box = [box_rows, 32 columns], 128-byte swizzle (TMA reduce-add of fp32 tiles).
//   col8_3: bf16 [S, 8] matrices, box = [box_rows, 8 columns], no swizzle (column panels).
int make_tile3_tmap(CUtensorMap* out, const void* base, uint64_t cols, uint64_t S, uint64_t n_outer,
                    uint64_t outer_stride, uint32_t box_rows);
int make_f32box3_tmap(CUtensorMap* out, const void* base, uint64_t cols, uint64_t S, uint64_t n_outer, uint32_t box_rows);
int make_col8_3_tmap(CUtensorMap* out, const void* base, uint64_t S, uint64_t n_outer, uint32_t box_rows);

// Device word that forward kernels report bounded-wait failures into (per device).
int forward_status_word(unsigned int** out);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace gqa
