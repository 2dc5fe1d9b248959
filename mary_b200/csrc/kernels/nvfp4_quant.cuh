// NVFP4 activation quantiser pieces shared by the kernels that quantise in flight (dispatch, GLU epilogue).
// Rules (src/models/inkling/fp4quant.rs:10-54): per 16 elements amax -> sf = min(amax / 6, 448) -> E4M3 round-to-nearest-even;
// codes by the thresholds .25 .75 1.25 1.75 2.5 3.5 5 on |x / sf| with >= (ties away from zero), the sign bit kept for values
// that round to zero, a zero block -> scale byte 0 and codes 0.
#pragma once
#include <cuda_fp8.h>

#include "common.cuh"

namespace mary {

__device__ __forceinline__ uint32_t nvfp4_code(float y) {
  const float m = fabsf(y);
  uint32_t c = (m >= 0.25f) + (m >= 0.75f) + (m >= 1.25f) + (m >= 1.75f) + (m >= 2.5f) + (m >= 3.5f) + (m >= 5.0f);
  return c | (signbit(y) ? 8u : 0u);
}
// Scale byte of a block with absolute maximum `amax`, and its decoded value.
__device__ __forceinline__ uint8_t nvfp4_scale_byte(float amax, float* decoded) {
  const float sfv = fminf(__fdiv_rn(amax, 6.0f), 448.0f);
  const __nv_fp8_storage_t sb = __nv_cvt_float_to_fp8(sfv, __NV_SATFINITE, __NV_E4M3);
  *decoded = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
  return (uint8_t)sb;
}

}  // namespace mary
