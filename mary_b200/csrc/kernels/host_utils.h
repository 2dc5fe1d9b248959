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

// 1 when the environment says MARY_PDL=1 (off by default: in CUDA-graph replay the measured step time was the same with and
// without it, 81.2 ms against 80.1 ms at 16 sequences).
int mary_pdl_enabled();

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the CURRENT device only, so the "already raised" record is kept
// per device ordinal: `slots` is a zero-initialised array of MARY_MAX_DEVICES entries owned by the call site (one per kernel
// instantiation).  Raises the limit when `bytes` exceeds what this device has been given so far.  Returns a MaryStatus.
#define MARY_MAX_DEVICES 64
struct MarySmemSlots { size_t v[MARY_MAX_DEVICES]; };
int mary_ensure_dyn_smem(const void* func, size_t bytes, MarySmemSlots* slots);

// Launch with programmatic dependent launch allowed: the kernel may be scheduled while its predecessor on the stream is still
// draining, and its threads call pdl_sync() (common.cuh) before they touch anything a predecessor wrote.  Only kernels whose
// first statement is pdl_sync() may be launched this way.  A template kernel name goes in parentheses.
#define MARY_LAUNCH(kernel_, grid_, block_, smem_, stream_, ...)                                                     \
  do {                                                                                                             \
    cudaLaunchConfig_t cfg__ = {};                                                                                 \
    cfg__.gridDim = (grid_);                                                                                       \
    cfg__.blockDim = (block_);                                                                                     \
    cfg__.dynamicSmemBytes = (smem_);                                                                              \
    cfg__.stream = (stream_);                                                                                      \
    cudaLaunchAttribute at__[1];                                                                                   \
    at__[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                               \
    at__[0].val.programmaticStreamSerializationAllowed = 1;                                                        \
    cfg__.attrs = at__;                                                                                            \
    cfg__.numAttrs = mary_pdl_enabled() ? 1 : 0;                                                                   \
    if (cudaLaunchKernelEx(&cfg__, kernel_, __VA_ARGS__) != cudaSuccess) return MARY_ERR_CUDA;                     \
  } while (0)

#define MARY_CHECK_LAUNCH()                                  \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return MARY_ERR_CUDA;            \
  } while (0)
