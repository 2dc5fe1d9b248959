// Bandwidth-bound row kernels: RMSNorm family, GLU, embedding gather, q/k norm + RoPE + paged-cache append,
// short convolution.  Reference kernels: src/models/inkling/resid.rs:180-389 (add_resid, rms_norm),
// src/models/inkling/fp4gemm.rs:154-189 (gate_up_silu), src/models/inkling/sconv.rs:70-340,
// src/models/qwen3tts/megakernel.rs (qkv_rope_cache).  One CTA per token row, 16-byte vector accesses, f32 math,
// a single rounding to bf16 on the way out.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int NT = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

template <typename T> __device__ __forceinline__ float ld(const T* p, int64_t i);
template <> __device__ __forceinline__ float ld<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// 8-element vector access helpers (H % 8 == 0, rows 16-byte aligned)
template <typename T> __device__ __forceinline__ void load8(const T* p, float* f);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
  const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 v = *(const uint4*)p;
  const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(h[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  uint4 v;
  __nv_bfloat162* h = (__nv_bfloat162*)&v;
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  *(uint4*)p = v;
}

// y = rms(x) * w   (w may be null).  x is bf16 or f32, y bf16.
template <typename TI>
__global__ void rmsnorm_kernel(const TI* __restrict__ x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                               int H, int64_t ldx, int64_t ldy, float eps) {
  pdl_sync();
  extern __shared__ float row[];
  __shared__ float red[32];
  const TI* xr = x + (int64_t)blockIdx.x * ldx;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8];
    load8(xr + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) { row[i + j] = f[j]; ss += f[j] * f[j]; }
  }
  const float inv = rsqrtf(block_sum(ss, red) / H + eps);
  __nv_bfloat16* yr = y + (int64_t)blockIdx.x * ldy;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8], g[8];
    if (w) load8(w + i, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = row[i + j] * inv * (w ? g[j] : 1.f);
    store8(yr + i, f);
  }
}

// residual += x (one rounding to bf16); y = rms(residual) * w
template <typename TI>
__global__ void add_rmsnorm_kernel(const TI* __restrict__ x, __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, int H, float eps) {
  pdl_sync();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int64_t o = (int64_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float a[8], r[8];
    load8(x + o + i, a);
    load8(res + o + i, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __bfloat162float(__float2bfloat16(r[j] + a[j]));
    store8(res + o + i, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) { row[i + j] = r[j]; ss += r[j] * r[j]; }
  }
  const float inv = rsqrtf(block_sum(ss, red) / H + eps);
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8], g[8];
    load8(w + i, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = row[i + j] * inv * g[j];
    store8(y + o + i, f);
  }
}

// Gemma sandwich step: h = (h + rms(a) * w_post) * scalar ; x = rms(h) * w_next (skipped when w_next is null)
template <typename TI>
__global__ void norm_add_norm_kernel(const TI* __restrict__ a, const __nv_bfloat16* __restrict__ w_post, __nv_bfloat16* __restrict__ h,
                                     const __nv_bfloat16* __restrict__ w_next, __nv_bfloat16* __restrict__ xo, int H, float eps, float scalar) {
  pdl_sync();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int64_t o = (int64_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8];
    load8(a + o + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) { row[i + j] = f[j]; ss += f[j] * f[j]; }
  }
  const float inv = rsqrtf(block_sum(ss, red) / H + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float g[8], r[8];
    load8(w_post + i, g);
    load8(h + o + i, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // the normed branch output is rounded to bf16 like the unfused op sequence would
      const float n = __bfloat162float(__float2bfloat16(row[i + j] * inv * g[j]));
      r[j] = __bfloat162float(__float2bfloat16((r[j] + n) * scalar));
      row[i + j] = r[j]; ss2 += r[j] * r[j];
    }
    store8(h + o + i, r);
  }
  if (w_next == nullptr) return;
  const float inv2 = rsqrtf(block_sum(ss2, red) / H + eps);
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8], g[8];
    load8(w_next + i, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = row[i + j] * inv2 * g[j];
    store8(xo + o + i, f);
  }
}

__global__ void glu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int F, int64_t n, int act) {
  pdl_sync();
  int64_t idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (idx >= n) return;
  const int64_t t = idx / F, f = idx % F;
  const uint4 g = *(const uint4*)(gu + t * 2 * F + f);
  const uint4 u = *(const uint4*)(gu + t * 2 * F + F + f);
  const __nv_bfloat162* gp = (const __nv_bfloat162*)&g;
  const __nv_bfloat162* up = (const __nv_bfloat162*)&u;
  uint4 o;
  __nv_bfloat162* op = (__nv_bfloat162*)&o;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 gf = __bfloat1622float2(gp[j]), uf = __bfloat1622float2(up[j]);
    op[j] = __floats2bfloat162_rn(glu_f(act, gf.x, uf.x), glu_f(act, gf.y, uf.y));
  }
  *(uint4*)(out + idx) = o;
}

__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ out,
                             int H, float scale, int vocab, int* __restrict__ status) {
  pdl_sync();
  int id = ids[blockIdx.x];
  if (id < 0 || id >= vocab) {                 // recorded, and the access redirected to row 0: no read outside the table
    if (threadIdx.x == 0) atomicCAS(status, 0, (int)MARY_ERR_BOUNDS);
    id = 0;
  }
  const __nv_bfloat16* src = table + (int64_t)id * H;
  __nv_bfloat16* dst = out + (int64_t)blockIdx.x * H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 v = *(const uint4*)(src + i);
    if (scale != 1.0f) {
      __nv_bfloat162* p = (__nv_bfloat162*)&v;
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(p[j]); p[j] = __floats2bfloat162_rn(f.x * scale, f.y * scale); }
    }
    *(uint4*)(dst + i) = v;
  }
}

// One warp per (token, head) of the fused qkv row: optional RMSNorm over the head (learned gain for q and k,
// none for v), split-half RoPE for q and k, then q goes to qo[T, n_q, D] and k, v into their cache slots.
__global__ void qk_norm_rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, int n_q, int n_kv, int D,
                                           const __nv_bfloat16* __restrict__ q_norm, const __nv_bfloat16* __restrict__ k_norm,
                                           int v_norm, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                           const int64_t* __restrict__ slots, __nv_bfloat16* __restrict__ qo,
                                           __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, float eps, int T,
                                           int64_t n_slots, int* __restrict__ status) {
  pdl_sync();
  const int warps_per_block = blockDim.x >> 5;
  const int heads = n_q + 2 * n_kv;
  const int64_t gw = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (gw >= (int64_t)T * heads) return;
  const int t = (int)(gw / heads), hh = (int)(gw % heads);
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* src = qkv + (int64_t)t * heads * D + (int64_t)hh * D;
  const int half = D >> 1;
  // lane handles pairs (i, i + half) for i = lane, lane + 32, ...
  float x1[8], x2[8];   // D <= 512
  const int np = (half + 31) / 32;
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int i = lane + 32 * m;
    if (m < np && i < half) {
      x1[m] = __bfloat162float(src[i]); x2[m] = __bfloat162float(src[i + half]);
      ss += x1[m] * x1[m] + x2[m] * x2[m];
    }
  }
  const bool is_q = hh < n_q, is_k = !is_q && hh < n_q + n_kv;
  const __nv_bfloat16* gain = is_q ? q_norm : (is_k ? k_norm : nullptr);
  const bool do_norm = is_q ? (q_norm != nullptr) : (is_k ? (k_norm != nullptr) : (v_norm != 0));
  float inv = 1.f;
  if (do_norm) inv = rsqrtf(warp_sum(ss) / D + eps);
  const float pos = (float)positions[t];
  __nv_bfloat16* dst;
  if (!is_q && n_slots > 0 && (slots[t] < 0 || slots[t] >= n_slots)) {       // a cache slot outside the cache: record it, skip the write
    if (lane == 0) atomicCAS(status, 0, (int)MARY_ERR_BOUNDS);
    return;
  }
  if (is_q) dst = qo + ((int64_t)t * n_q + hh) * D;
  else if (is_k) dst = kc + (slots[t] * n_kv + (hh - n_q)) * D;
  else dst = vc + (slots[t] * n_kv + (hh - n_q - n_kv)) * D;
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int i = lane + 32 * m;
    if (m < np && i < half) {
      float a = x1[m] * inv, b = x2[m] * inv;
      if (do_norm) {
        // round the normed value to bf16 first, as the unfused sequence (norm kernel then rope kernel) does
        a = __bfloat162float(__float2bfloat16(a * (gain ? __bfloat162float(gain[i]) : 1.f)));
        b = __bfloat162float(__float2bfloat16(b * (gain ? __bfloat162float(gain[i + half]) : 1.f)));
      }
      if (!is_q && !is_k) { dst[i] = __float2bfloat16(a); dst[i + half] = __float2bfloat16(b); continue; }
      if (inv_freq) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        const float ra = a * c - b * s, rb = a * s + b * c;
        a = ra; b = rb;
      }
      dst[i] = __float2bfloat16(a); dst[i + half] = __float2bfloat16(b);
    }
  }
}

// y = x + depthwise causal conv_k(x) with history of the previous k-1 pre-conv rows; one thread per channel,
// rows of one sequence are walked in order (src/models/inkling/block.rs:48-127).  hist is updated in place.
__global__ void short_conv_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, __nv_bfloat16* __restrict__ hist,
                                  __nv_bfloat16* __restrict__ y, int T, int D, int k) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float win[8];
  float wk[8];
  for (int j = 0; j < k; ++j) wk[j] = w[d * k + j];
  for (int j = 0; j < k - 1; ++j) win[j] = __bfloat162float(hist[(int64_t)j * D + d]);
  for (int t = 0; t < T; ++t) {
    const float cur = __bfloat162float(x[(int64_t)t * D + d]);
    win[k - 1] = cur;
    float acc = cur;
    for (int j = 0; j < k; ++j) acc += win[j] * wk[j];
    y[(int64_t)t * D + d] = __float2bfloat16(acc);
    for (int j = 0; j < k - 1; ++j) win[j] = win[j + 1];
  }
  for (int j = 0; j < k - 1; ++j) hist[(int64_t)j * D + d] = __float2bfloat16(win[j]);
}

}  // namespace

MARY_API int mary_rmsnorm(const void* x, int x_is_f32, const void* w, void* y, int T, int H, int64_t ldx, int64_t ldy, float eps,
                          cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  size_t sm = (size_t)H * 4;
  if (sm > 48 * 1024 || (H & 7) || (ldx & 7) || (ldy & 7)) return MARY_ERR_BAD_ARG;
  if (x_is_f32) MARY_LAUNCH((rmsnorm_kernel<float>), T, NT, sm, s, (const float*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, ldx, ldy, eps);
  else MARY_LAUNCH((rmsnorm_kernel<__nv_bfloat16>), T, NT, sm, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, ldx, ldy, eps);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_add_rmsnorm(const void* x, int x_is_f32, void* res, const void* w, void* y, int T, int H, float eps, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  size_t sm = (size_t)H * 4;
  if (sm > 48 * 1024 || (H & 7)) return MARY_ERR_BAD_ARG;
  if (x_is_f32) MARY_LAUNCH((add_rmsnorm_kernel<float>), T, NT, sm, s, (const float*)x, (__nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, eps);
  else MARY_LAUNCH((add_rmsnorm_kernel<__nv_bfloat16>), T, NT, sm, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, eps);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_norm_add_norm(const void* a, int a_is_f32, const void* w_post, void* h, const void* w_next, void* xo, int T, int H,
                                float eps, float scalar, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  size_t sm = (size_t)H * 4;
  if (sm > 48 * 1024 || (H & 7)) return MARY_ERR_BAD_ARG;
  if (a_is_f32) MARY_LAUNCH((norm_add_norm_kernel<float>), T, NT, sm, s, (const float*)a, (const __nv_bfloat16*)w_post, (__nv_bfloat16*)h, (const __nv_bfloat16*)w_next, (__nv_bfloat16*)xo, H, eps, scalar);
  else MARY_LAUNCH((norm_add_norm_kernel<__nv_bfloat16>), T, NT, sm, s, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w_post, (__nv_bfloat16*)h, (const __nv_bfloat16*)w_next, (__nv_bfloat16*)xo, H, eps, scalar);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_glu(const void* gu, void* out, int T, int F, int act, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  if (F % 8) return MARY_ERR_BAD_ARG;
  int64_t n = (int64_t)T * F;
  int blocks = (int)((n / 8 + NT - 1) / NT);
  MARY_LAUNCH(glu_kernel, blocks, NT, 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, F, n, act);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_embed(const int* ids, const void* table, void* out, int T, int H, float scale, int vocab, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  if (H % 8) return MARY_ERR_BAD_ARG;
  MARY_LAUNCH(embed_kernel, T, 128, 0, s, ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, H, scale, vocab, mary_status_ptr());
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_qk_norm_rope_append(const void* qkv, int n_q, int n_kv, int D, const void* q_norm, const void* k_norm, int v_norm,
                                      const float* inv_freq, const int* positions, const int64_t* slots, void* qo, void* kc, void* vc,
                                      float eps, int T, int64_t n_slots, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  if (D > 512 || (D & 1)) return MARY_ERR_BAD_ARG;
  const int64_t warps = (int64_t)T * (n_q + 2 * n_kv);
  const int wpb = 8;
  MARY_LAUNCH(qk_norm_rope_append_kernel, (int)((warps + wpb - 1) / wpb), wpb * 32, 0, s, 
      (const __nv_bfloat16*)qkv, n_q, n_kv, D, (const __nv_bfloat16*)q_norm, (const __nv_bfloat16*)k_norm, v_norm, inv_freq, positions,
      slots, (__nv_bfloat16*)qo, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, eps, T, n_slots, mary_status_ptr());
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_short_conv(const void* x, const float* w, void* hist, void* y, int T, int D, int k, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  if (k > 8 || k < 1) return MARY_ERR_BAD_ARG;
  short_conv_kernel<<<(D + 127) / 128, 128, 0, s>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)hist, (__nv_bfloat16*)y, T, D, k);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// ---------------------------------------------------------------------------------------------------------------------------
// Bandwidth probes (the reference's `stream_read`, src/bin/inkling_membw.rs:50): a read-only sweep and a copy over a buffer far
// larger than L2, 16 bytes per thread per step, grid = 8 CTAs per SM.  `sink` receives a value that depends on every word read.
namespace {
__global__ void stream_read_kernel(const uint4* __restrict__ src, int64_t n16, unsigned* __restrict__ sink) {
  unsigned acc = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = __ldcs(src + i);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0x9e3779b9u) atomicAdd(sink, 1u);            // practically never true: keeps the loads alive without a write per thread
}
__global__ void stream_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t n16) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) __stcs(dst + i, __ldcs(src + i));
}
}  // namespace

MARY_API int mary_stream_read(const void* src, int64_t bytes, void* sink, cudaStream_t s) {
  if (((uintptr_t)src & 15) || bytes < 16) return MARY_ERR_BAD_ARG;
  stream_read_kernel<<<mary_num_sms() * 8, 256, 0, s>>>((const uint4*)src, bytes / 16, (unsigned*)sink);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_stream_copy(const void* src, void* dst, int64_t bytes, cudaStream_t s) {
  if (((uintptr_t)src & 15) || ((uintptr_t)dst & 15) || bytes < 16) return MARY_ERR_BAD_ARG;
  stream_copy_kernel<<<mary_num_sms() * 8, 256, 0, s>>>((const uint4*)src, (uint4*)dst, bytes / 16);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
