// Host-side declarations shared by the launchers.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
PFN_encodeTiled mary_encode_fn();
int mary_num_sms();
int* mary_status_ptr();
// dtype_bytes_x2: twice the element size in bytes (2 = one byte, 4 = bf16, 8 = f32) so that packed FP4 data can
// be described as bytes.
int mary_make_tmap_2d(CUtensorMap* m, const void* base, int dtype_bytes_x2, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols, int swizzle128);

#define MARY_CHECK_LAUNCH()                                  \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return MARY_ERR_CUDA;            \
  } while (0)
