// Batch-1 matrix-vector kernels with in-kernel de-quantisation: f16 / bf16, Q8_0 and Q4_0 weights (GGUF block
// formats: 32 elements per block, one f16 scale; Q4_0 packs element j and j+16 of a block into one byte).
// Reference: src/nn/q4.rs:86-252 (q4_matvec_kernel, f16_matvec_kernel with a fused SwiGLU epilogue) and the q8/f16
// matvecs of the voice models (src/models/personaplex/temporal_metal.rs:133-454).  Grid rows/8, block 8 rows x 32 lanes:
// each warp owns one output row, lanes stride over the blocks of that row, f32 accumulation, warp-shuffle reduction.
// epilogue 0: y = W x;  1: y[r] = silu(W[r] x) * (W[r + rows] x)  (gate rows first, up rows second).
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

__device__ __forceinline__ float dot_q4_block(const uint8_t* blk, const __nv_bfloat16* x) {
  const float d = __half2float(*(const __half*)blk);
  const uint8_t* qs = blk + 2;
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int lo = (qs[j] & 0xF) - 8, hi = (qs[j] >> 4) - 8;
    acc += lo * __bfloat162float(x[j]) + hi * __bfloat162float(x[j + 16]);
  }
  return acc * d;
}
__device__ __forceinline__ float dot_q8_block(const uint8_t* blk, const __nv_bfloat16* x) {
  const float d = __half2float(*(const __half*)blk);
  const int8_t* qs = (const int8_t*)(blk + 2);
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) acc += qs[j] * __bfloat162float(x[j]);
  return acc * d;
}

template <int FMT>   // 0 bf16, 1 q8_0, 2 q4_0
__device__ __forceinline__ float row_dot(const uint8_t* w, int64_t row, int cols, const __nv_bfloat16* x, int lane) {
  float acc = 0.f;
  if (FMT == 0) {
    const __nv_bfloat16* wr = (const __nv_bfloat16*)w + row * cols;
    for (int c = lane * 8; c < cols; c += 256) {
      const uint4 a = *(const uint4*)(wr + c), b = *(const uint4*)(x + c);
      const __nv_bfloat162 *ap = (const __nv_bfloat162*)&a, *bp = (const __nv_bfloat162*)&b;
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(ap[j]), g = __bfloat1622float2(bp[j]); acc += f.x * g.x + f.y * g.y; }
    }
  } else {
    const int bb = FMT == 1 ? 34 : 18;
    const int nb = cols / 32;
    const uint8_t* wr = w + row * (int64_t)nb * bb;
    for (int b = lane; b < nb; b += 32)
      acc += FMT == 1 ? dot_q8_block(wr + (int64_t)b * bb, x + b * 32) : dot_q4_block(wr + (int64_t)b * bb, x + b * 32);
  }
  return warp_sum(acc);
}

template <int FMT>
__global__ void matvec_kernel(const uint8_t* __restrict__ w, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int rows,
                              int cols, int epilogue) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float v = row_dot<FMT>(w, row, cols, x, lane);
  if (epilogue == 1) {
    const float u = row_dot<FMT>(w, (int64_t)row + rows, cols, x, lane);
    v = silu_f(v) * u;
  }
  if (lane == 0) y[row] = __float2bfloat16(v);
}

}  // namespace

MARY_API int mary_matvec(const void* w, int fmt, const void* x, void* y, int rows, int cols, int epilogue, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((fmt == 0 && cols % 8) || (fmt != 0 && cols % 32)) return MARY_ERR_BAD_ARG;
  const int grid = (rows + 7) / 8;
  if (fmt == 0) matvec_kernel<0><<<grid, 256, 0, s>>>((const uint8_t*)w, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, cols, epilogue);
  else if (fmt == 1) matvec_kernel<1><<<grid, 256, 0, s>>>((const uint8_t*)w, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, cols, epilogue);
  else if (fmt == 2) matvec_kernel<2><<<grid, 256, 0, s>>>((const uint8_t*)w, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, cols, epilogue);
  else return MARY_ERR_BAD_ARG;
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
