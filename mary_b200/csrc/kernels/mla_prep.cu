// Small row kernels around multi-head latent attention (MLA):
//   mla_prep:   from the fused projection row [q_a (q_lora) | c_kv (512) | k_rope (64)]:
//               q_a -> RMSNorm (learned gain) -> qa_out;  c_kv -> RMSNorm (learned gain) and k_rope -> split-half RoPE,
//               both written to the latent cache slot of the row ([c_kv_normed (512) | k_rope (64)]).
//   mla_q_rope: RoPE on the 64-dim rope part of every query head, written behind the absorbed 512 latent dims of
//               q_full[T, H, 576].
// Math of the reference MLA: src/models/k3/mla.rs:49-63,102-111 (eps 1e-6 inside MLA; the reference runs NoPE and an
// expanded cache — `inv_freq == nullptr` gives NoPE here, the latent cache is this build's).
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__global__ void mla_prep_kernel(const __nv_bfloat16* __restrict__ qakv, int64_t ld, int q_lora, const __nv_bfloat16* __restrict__ w_qa,
                                const __nv_bfloat16* __restrict__ w_kv, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                const int64_t* __restrict__ slots, __nv_bfloat16* __restrict__ qa_out, __nv_bfloat16* __restrict__ cache,
                                float eps, int64_t n_slots, int* __restrict__ status) {
  pdl_sync();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const __nv_bfloat16* row = qakv + (int64_t)t * ld;
  // q_a norm
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_lora; i += blockDim.x) { float v = __bfloat162float(row[i]); ss += v * v; }
  const float inv_q = rsqrtf(block_sum_256(ss, red) / q_lora + eps);
  for (int i = threadIdx.x; i < q_lora; i += blockDim.x)
    qa_out[(int64_t)t * q_lora + i] = __float2bfloat16(__bfloat162float(row[i]) * inv_q * __bfloat162float(w_qa[i]));
  // latent norm
  const __nv_bfloat16* ckv = row + q_lora;
  ss = 0.f;
  for (int i = threadIdx.x; i < 512; i += blockDim.x) { float v = __bfloat162float(ckv[i]); ss += v * v; }
  const float inv_k = rsqrtf(block_sum_256(ss, red) / 512 + eps);
  if (n_slots > 0 && (slots[t] < 0 || slots[t] >= n_slots)) {                 // a cache slot outside the cache: record it, skip the write
    if (threadIdx.x == 0) atomicCAS(status, 0, (int)MARY_ERR_BOUNDS);
    return;
  }
  __nv_bfloat16* dst = cache + slots[t] * 576;
  for (int i = threadIdx.x; i < 512; i += blockDim.x)
    dst[i] = __float2bfloat16(__bfloat162float(ckv[i]) * inv_k * __bfloat162float(w_kv[i]));
  // rope on the 64 carried dims (split-half pairs (i, i + 32))
  if (threadIdx.x < 32) {
    const int i = threadIdx.x;
    float a = __bfloat162float(ckv[512 + i]), b = __bfloat162float(ckv[512 + 32 + i]);
    if (inv_freq) {
      float s, c;
      sincosf((float)positions[t] * inv_freq[i], &s, &c);
      const float ra = a * c - b * s, rb = a * s + b * c;
      a = ra; b = rb;
    }
    dst[512 + i] = __float2bfloat16(a);
    dst[512 + 32 + i] = __float2bfloat16(b);
  }
}

// qb [T, H, 192] = [nope 128 | rope 64] per head -> q_full[T, H, 512 + i] for the rope part
__global__ void mla_q_rope_kernel(const __nv_bfloat16* qb, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                  __nv_bfloat16* q_full, int H, int T, int64_t dst_stride, int dst_off) {
  pdl_sync();
  const int64_t gw = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (int64_t)T * H) return;
  const int t = (int)(gw / H), i = threadIdx.x & 31;
  const __nv_bfloat16* src = qb + gw * 192 + 128;
  float a = __bfloat162float(src[i]), b = __bfloat162float(src[32 + i]);
  if (inv_freq) {
    float s, c;
    sincosf((float)positions[t] * inv_freq[i], &s, &c);
    const float ra = a * c - b * s, rb = a * s + b * c;
    a = ra; b = rb;
  }
  __nv_bfloat16* dst = q_full + gw * dst_stride + dst_off;        // may be the source row itself: every lane has read its pair
  dst[i] = __float2bfloat16(a);
  dst[32 + i] = __float2bfloat16(b);
}

// K rows of the expanded prefill: the 64 rotated dims every head shares, copied from the latent row behind each head's 128 own dims.
__global__ void mla_fill_k_rope_kernel(const __nv_bfloat16* __restrict__ lat, int64_t lat_stride, __nv_bfloat16* __restrict__ k, int H,
                                       int64_t n_rows) {
  pdl_sync();
  const int64_t gw = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= n_rows * H) return;
  const int64_t n = gw / H;
  const int i = threadIdx.x & 31;
  const uint32_t v = *(const uint32_t*)(lat + n * lat_stride + 512 + 2 * i);
  *(uint32_t*)(k + gw * 192 + 128 + 2 * i) = v;
}

}  // namespace

MARY_API int mary_mla_prep(const void* qakv, int64_t ld, int q_lora, const void* w_qa, const void* w_kv, const float* inv_freq,
                           const int* positions, const int64_t* slots, void* qa_out, void* cache, float eps, int T, int64_t n_slots,
                           cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  MARY_LAUNCH(mla_prep_kernel, T, 256, 0, s, (const __nv_bfloat16*)qakv, ld, q_lora, (const __nv_bfloat16*)w_qa, (const __nv_bfloat16*)w_kv, inv_freq,
                                    positions, slots, (__nv_bfloat16*)qa_out, (__nv_bfloat16*)cache, eps, n_slots, mary_status_ptr());
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_mla_q_rope(const void* qb, const float* inv_freq, const int* positions, void* q_full, int H, int T, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  const int64_t warps = (int64_t)T * H;
  MARY_LAUNCH(mla_q_rope_kernel, (int)((warps + 7) / 8), 256, 0, s, (const __nv_bfloat16*)qb, inv_freq, positions, (__nv_bfloat16*)q_full, H, T,
              (int64_t)576, 512);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// The same rotation written back over the 64 rope dims of qb [T, H, 192] itself (the expanded prefill attends with 192-wide queries).
MARY_API int mary_mla_q_rope_inplace(void* qb, const float* inv_freq, const int* positions, int H, int T, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  const int64_t warps = (int64_t)T * H;
  MARY_LAUNCH(mla_q_rope_kernel, (int)((warps + 7) / 8), 256, 0, s, (const __nv_bfloat16*)qb, inv_freq, positions, (__nv_bfloat16*)qb, H, T,
              (int64_t)192, 128);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// k [n_rows, H, 192]: dims 128..191 of every head <- dims 512..575 of latent row n (row pitch lat_stride elements).
MARY_API int mary_mla_fill_k_rope(const void* lat, int64_t lat_stride, void* k, int H, int64_t n_rows, cudaStream_t s) {
  if (n_rows <= 0) return MARY_OK;
  if (lat_stride & 1) return MARY_ERR_BAD_ARG;
  const int64_t warps = n_rows * H;
  MARY_LAUNCH(mla_fill_k_rope_kernel, (int)((warps + 7) / 8), 256, 0, s, (const __nv_bfloat16*)lat, lat_stride, (__nv_bfloat16*)k, H, n_rows);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
