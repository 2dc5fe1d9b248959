// Fused AdamW step over a flat f32 parameter buffer (LoRA adapters).
// Math of the reference trainer (src/bin/gemma_train_lora.rs:118-165): m = b1 m + (1-b1) g; v = b2 v + (1-b2) g^2;
// p = p - lr * (mhat / (sqrt(vhat) + eps) + wd * p) with bias-corrected mhat, vhat.
#include "common.cuh"
#include "host_utils.h"

namespace {
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, int64_t n,
                             float lr, float b1, float b2, float eps, float wd, float c1, float c2, float grad_scale) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float gi = g[i] * grad_scale;
  const float mi = b1 * m[i] + (1.f - b1) * gi;
  const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
  m[i] = mi; v[i] = vi;
  const float mhat = mi / c1, vhat = vi / c2;
  const float pi = p[i];
  p[i] = pi - lr * (__fdiv_rn(mhat, sqrtf(vhat) + eps) + wd * pi);
}
}  // namespace

MARY_API int mary_adamw(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2, float eps, float wd,
                        int step, float grad_scale, cudaStream_t s) {
  if (n <= 0) return MARY_OK;
  const float c1 = 1.f - powf(b1, (float)step), c2 = 1.f - powf(b2, (float)step);
  adamw_kernel<<<(int)((n + 255) / 256), 256, 0, s>>>(p, g, m, v, n, lr, b1, b2, eps, wd, c1, c2, grad_scale);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
