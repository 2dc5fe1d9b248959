// Host-side support shared by all launchers: the per-device status word, the driver entry point used to
// encode TMA tensor maps, and device queries.
#include <mutex>

#include "common.cuh"
#include "host_utils.h"
#include <stdlib.h>

namespace {
__device__ int g_status_fallback[64];
std::mutex g_mu;
int* g_status[64] = {nullptr};
PFN_encodeTiled g_encode = nullptr;
int g_sms[64] = {0};
}  // namespace

int* mary_status_ptr() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_status[dev]) {
    // never null: when the allocation fails the word falls back to a zero-initialised array of the library's device image
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess || cudaMemset(p, 0, 256) != cudaSuccess) {
      cudaGetLastError();
      void* sym = nullptr;
      if (cudaGetSymbolAddress(&sym, g_status_fallback) != cudaSuccess) return nullptr;
      p = (int*)sym;
    }
    g_status[dev] = p;
  }
  return g_status[dev];
}

PFN_encodeTiled mary_encode_fn() {
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = (PFN_encodeTiled)fn;
  }
  return g_encode;
}

int mary_num_sms() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (!g_sms[dev]) cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return g_sms[dev];
}

// 2-D row-major tensor map: inner dimension `cols` (elements), outer `rows`, row pitch `ld` elements.
// Box = box_cols x box_rows.  Out-of-range parts of a box read as zero.
int mary_make_tmap_2d(CUtensorMap* m, const void* base, int dtype_bytes_x2, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols, int swizzle128) {
  PFN_encodeTiled enc = mary_encode_fn();
  if (!enc) return MARY_ERR_CUDA;
  CUtensorMapDataType dt;
  uint64_t elem_bytes_x2 = dtype_bytes_x2;
  if (dtype_bytes_x2 == 4) dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  else if (dtype_bytes_x2 == 2) dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  else if (dtype_bytes_x2 == 8) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  else return MARY_ERR_BAD_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * elem_bytes_x2 / 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (((uintptr_t)base & 15) || (strides[0] & 15)) return MARY_ERR_BAD_ARG;
  CUresult r = enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MARY_OK : MARY_ERR_CUDA;
}

// Read and clear the status word of the current device (synchronises the device).
MARY_API int mary_last_status() {
  int* p = mary_status_ptr();
  if (!p) return MARY_ERR_CUDA;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return MARY_ERR_CUDA;
  if (v) cudaMemset(p, 0, sizeof(int));
  return v;
}

MARY_API int mary_sm_count() { return mary_num_sms(); }

int mary_ensure_dyn_smem(const void* func, size_t bytes, MarySmemSlots* slots) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MARY_MAX_DEVICES) return MARY_ERR_CUDA;
  std::lock_guard<std::mutex> g(g_mu);
  if (bytes > slots->v[dev]) {
    if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) return MARY_ERR_CUDA;
    slots->v[dev] = bytes;
  }
  return MARY_OK;
}

static int g_pdl = -1;          // -1: not decided yet (the environment decides at the first launch)

int mary_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("MARY_PDL");
    g_pdl = (e && e[0] == '1') ? 1 : 0;
  }
  return g_pdl;
}

// Switch programmatic dependent launch on or off for the launches that follow (a model whose step is a chain of small dense GEMMs
// gains from it, one with the expert pipeline in the chain loses: the caller that knows the model decides).  Graphs captured
// before the call keep what they were captured with.
MARY_API void mary_set_pdl(int on) { g_pdl = on ? 1 : 0; }
