// Kernels of the streaming audio codec (SEANet convolutions, transformer bottleneck, residual vector quantiser).
//
// The reference runs its codec convolutions as im2col + sgemm on the CPU and as one SIMT kernel per op on the GPU
// (src/models/personaplex/mimi/encoder.rs:33-120, src/models/personaplex/mimi/decoder.rs:483-1099: conv1d / transconv /
// dw_transconv / layernorm / layerscale_add kernels, grid (time, out / ROWS)).  Here the multiply-accumulate work of every
// convolution goes to the tcgen05 GEMM; these kernels are the data movement around it, on time-major activations [L, C]:
//   im2col_causal   gathers the k taps of every output frame into one GEMM row (bf16), applying the preceding ELU on the
//                   way and reading the k - stride samples of left context from the streaming state (zeros or the first
//                   sample repeated on the first chunk); it also writes the next state;
//   overlap_add     turns the GEMM result of a transposed convolution ([frames, k * C_out]) into samples, adding the tail
//                   carried from the previous chunk and carrying the new one;
//   dw_transconv    depthwise transposed convolution (the k4 s2 upsampler);
//   layernorm, act  LayerNorm with affine (f32 in, bf16 out) and ELU / GELU (f32 in, bf16 out) feeding the next GEMM.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

__device__ __forceinline__ float elu_f(float x) { return x > 0.f ? x : expm1f(x); }
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float act_f(int act, float x) { return act == 1 ? elu_f(x) : (act == 2 ? gelu_erf_f(x) : x); }

// col[t, j * Cin + c] = act(src[t * stride + j - ctx]) with src = [state ; x]; one thread per (t, j, c).
__global__ void im2col_causal_kernel(const float* __restrict__ x, const float* __restrict__ state_in, float* __restrict__ state_out,
                                     __nv_bfloat16* __restrict__ col, int ld, int L, int Cin, int k, int stride, int T_out, int act,
                                     int replicate, int have_state) {
  const int ctx = k - stride;
  const int64_t n = (int64_t)T_out * k * Cin;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cin);
    const int j = (int)((i / Cin) % k);
    const int t = (int)(i / ((int64_t)Cin * k));
    const int s = t * stride + j - ctx;
    float v;
    if (s >= 0) v = x[(int64_t)s * Cin + c];
    else if (have_state) v = state_in[(int64_t)(s + ctx) * Cin + c];
    else v = replicate ? x[c] : 0.f;
    col[(int64_t)t * ld + j * Cin + c] = __float2bfloat16(act_f(act, v));
  }
  // next state: the ctx raw samples that follow the consumed ones (consumed = T_out * stride)
  const int64_t ns = (int64_t)ctx * Cin;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < ns; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cin), r = (int)(i / Cin);
    const int s = T_out * stride + r - ctx;               // index into [state ; x] minus ctx
    float v;
    if (s >= 0) v = x[(int64_t)s * Cin + c];
    else if (have_state) v = state_in[(int64_t)(s + ctx) * Cin + c];
    else v = replicate ? x[c] : 0.f;
    state_out[i] = v;
  }
}

// z[t, j * Cout + co] -> y[t * stride + j, co]; one thread per output sample and channel, k / stride contributions each.
__global__ void overlap_add_kernel(const float* __restrict__ z, const float* __restrict__ tail_in, float* __restrict__ tail_out,
                                   const float* __restrict__ bias, float* __restrict__ y, int T_in, int Cout, int k, int stride, int have_tail) {
  const int tail = k - stride;
  const int S = T_in * stride + tail;
  const int64_t n = (int64_t)S * Cout;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int co = (int)(i % Cout), s = (int)(i / Cout);
    float acc = 0.f;
    for (int j = s % stride; j < k; j += stride) {
      const int t = (s - j) / stride;
      if (s - j >= 0 && t < T_in) acc += z[(int64_t)t * k * Cout + (int64_t)j * Cout + co];
    }
    if (have_tail && s < tail) acc += tail_in[(int64_t)s * Cout + co];
    if (s < T_in * stride) y[i] = acc + (bias ? bias[co] : 0.f);
    else tail_out[(int64_t)(s - T_in * stride) * Cout + co] = acc;
  }
}

// depthwise transposed convolution: y[t * stride + j, c] += x[t, c] * w[c, j]
__global__ void dw_transconv_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ tail_in,
                                    float* __restrict__ tail_out, float* __restrict__ y, int T_in, int C, int k, int stride, int have_tail) {
  const int tail = k - stride;
  const int S = T_in * stride + tail;
  const int64_t n = (int64_t)S * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C), s = (int)(i / C);
    float acc = 0.f;
    for (int j = s % stride; j < k; j += stride) {
      const int t = (s - j) / stride;
      if (s - j >= 0 && t < T_in) acc += x[(int64_t)t * C + c] * w[c * k + j];
    }
    if (have_tail && s < tail) acc += tail_in[(int64_t)s * C + c];
    if (s < T_in * stride) y[i] = acc;
    else tail_out[(int64_t)(s - T_in * stride) * C + c] = acc;
  }
}

__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                 __nv_bfloat16* __restrict__ out, int H, float eps) {
  __shared__ float red[32];
  const float* row = x + (int64_t)blockIdx.x * H;
  float s = 0.f, ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = row[i]; s += v; ss += v * v; }
  auto block_sum = [&](float v) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
    return warp_sum(t);
  };
  const float mean = block_sum(s) / H;
  const float var = fmaxf(block_sum(ss) / H - mean * mean, 0.f);
  const float inv = rsqrtf(var + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(int64_t)blockIdx.x * H + i] = __float2bfloat16((row[i] - mean) * inv * w[i] + b[i]);
}

__global__ void act_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, int64_t n, int act) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(act_f(act, x[i]));
}

inline int grid_for(int64_t n) { return (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256 < 1 ? 1 : (n + 255) / 256); }

}  // namespace

// x [L, Cin] f32 (time-major); col [T_out, ld >= k * Cin] bf16 with T_out = L / stride (columns past k * Cin are left as they
// are: zero them once); state_in (null on the first chunk) and state_out [k - stride, Cin] f32 must be different buffers.
// act: 0 none, 1 ELU, 2 GELU applied to the gathered samples.
MARY_API int mary_im2col_causal(const float* x, const float* state_in, float* state_out, void* col, int ld, int L, int Cin, int k,
                                int stride, int act, int replicate, cudaStream_t s) {
  if (L <= 0 || L % stride || k < stride || (k > stride && !state_out) || ld < k * Cin) return MARY_ERR_BAD_ARG;
  const int T_out = L / stride;
  im2col_causal_kernel<<<grid_for((int64_t)T_out * k * Cin), 256, 0, s>>>(x, state_in, state_out, (__nv_bfloat16*)col, ld, L, Cin, k,
                                                                         stride, T_out, act, replicate, state_in ? 1 : 0);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// z [T_in, k * Cout] f32 (GEMM of the frames with the [k * Cout, Cin] weight); y [T_in * stride, Cout] f32; tails [k - stride, Cout].
MARY_API int mary_overlap_add(const float* z, const float* tail_in, float* tail_out, const float* bias, float* y, int T_in, int Cout, int k,
                              int stride, cudaStream_t s) {
  if (T_in <= 0 || k < stride) return MARY_ERR_BAD_ARG;
  overlap_add_kernel<<<grid_for((int64_t)(T_in * stride + k - stride) * Cout), 256, 0, s>>>(z, tail_in, tail_out, bias, y, T_in, Cout, k,
                                                                                           stride, tail_in ? 1 : 0);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_dw_transconv(const float* x, const float* w, const float* tail_in, float* tail_out, float* y, int T_in, int C, int k,
                               int stride, cudaStream_t s) {
  if (T_in <= 0 || k < stride) return MARY_ERR_BAD_ARG;
  dw_transconv_kernel<<<grid_for((int64_t)(T_in * stride + k - stride) * C), 256, 0, s>>>(x, w, tail_in, tail_out, y, T_in, C, k, stride,
                                                                                         tail_in ? 1 : 0);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_layernorm(const float* x, const float* w, const float* b, void* out, int T, int H, float eps, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  layernorm_kernel<<<T, 256, 0, s>>>(x, w, b, (__nv_bfloat16*)out, H, eps);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_act_bf16(const float* x, void* out, int64_t n, int act, cudaStream_t s) {
  if (n <= 0) return MARY_OK;
  act_bf16_kernel<<<grid_for(n), 256, 0, s>>>(x, (__nv_bfloat16*)out, n, act);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
