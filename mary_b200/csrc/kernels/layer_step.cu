// One-token decode step of a dense pre-norm decoder layer (Mistral / Qwen3 / the Qwen3-TTS talker and code predictor) in FIVE
// launches instead of nine: the stages the reference folds for its talker (src/models/qwen3tts/megakernel.rs:1-722), written for
// one sequence and one new token.  Every stage is a weight-streaming matrix-vector product spread over all SMs, with the
// element-wise work of its neighbours folded in:
//
//   1. step_rms_matvec      x = rms(h) * gain (recomputed by every CTA: a few KB), qkv = W_qkv x
//   2. step_attention       per query head: RMS norm of the q head and of its k head (gains), split-half rotation at the token's
//                           position, append of k / v to the paged cache (one CTA per kv group writes), attention over the
//                           cache pages plus the new token, all in one CTA
//   3. step_matvec_residual h' = h + W_o o
//   4. step_rms_glu         x = rms(h') * gain, m = silu(W_gate x) * (W_up x)
//   5. step_matvec_residual h'' = h' + W_down m
//
// bf16 weights and activations, f32 arithmetic.  A launch of these kernels costs about 3 us in a CUDA graph against 8 us and
// more for a tensor-core GEMM launch with one token (barrier, TMEM and pipeline set-up for a single MMA column), which is what
// a one-token step is bound by; the matrix-vector products read each weight row once with 16-byte loads, four rows in flight
// per warp.
#include "common.cuh"
#include "host_utils.h"

namespace {
using namespace mary;

constexpr int LS_THREADS = 256;
constexpr int LS_MAX_H = 8192;          // widest input vector held in shared memory as f32

__device__ __forceinline__ void ld8f(const __nv_bfloat16* p, float* f) {
  const uint4 v = __ldg((const uint4*)p);
  const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 a = __bfloat1622float2(h[j]); f[2 * j] = a.x; f[2 * j + 1] = a.y; }
}

__device__ __forceinline__ float block_sum_ls(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = (int)threadIdx.x < nw ? red[threadIdx.x] : 0.f;
  if (w == 0) { t = warp_sum(t); if (threadIdx.x == 0) red[0] = t; }
  __syncthreads();
  return red[0];
}

// xs[0 .. K) = the input vector as f32: rms(h) * gain rounded to bf16 (gain != null) or h itself
__device__ __forceinline__ void stage_input(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ gain, float eps, int K,
                                            float* xs, float* red) {
  float ss = 0.f;
  for (int c = threadIdx.x; c < K; c += blockDim.x) {
    const float v = __bfloat162float(h[c]);
    xs[c] = v;
    ss = fmaf(v, v, ss);
  }
  if (gain) {
    const float rstd = rsqrtf(block_sum_ls(ss, red) / (float)K + eps);
    for (int c = threadIdx.x; c < K; c += blockDim.x)
      xs[c] = __bfloat162float(__float2bfloat16(xs[c] * rstd * __bfloat162float(gain[c])));
  }
  __syncthreads();
}

// dot products of up to four weight rows with xs, the lanes of a warp striding over K in 16-byte chunks; four chunks per row are
// requested before the first is used (16 loads of 16 bytes in flight per lane: a one-token product is a pure weight stream and
// its speed is the number of bytes in flight)
// `rot` staggers where in K a warp starts (it walks all of K, wrapping): rows are a power-of-two number of bytes apart, and warps
// that all read the same columns of different rows at the same time would queue on a few memory channels
__device__ __forceinline__ void warp_dot4(const __nv_bfloat16* __restrict__ w, int64_t ldw, const int* rows, int n_rows, const float* xs, int K,
                                          float* out, int rot) {
  const int lane = threadIdx.x & 31;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  constexpr int U = 4;
  const int span = 256 * U, iters = (K + span - 1) / span;
  for (int it = 0; it < iters; ++it) {
    const int c = ((it + rot) % iters) * span + lane * 8;
    uint4 wv[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < 4; ++r)
        if (r < n_rows && c + u * 256 < K) wv[u][r] = __ldg((const uint4*)(w + (int64_t)rows[r] * ldw + c + u * 256));
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int cc = c + u * 256;
      if (cc < K) {
        const float4 x0 = *(const float4*)(xs + cc), x1 = *(const float4*)(xs + cc + 4);
#pragma unroll
        for (int r = 0; r < 4; ++r)
          if (r < n_rows) {
            const __nv_bfloat162* h = (const __nv_bfloat162*)&wv[u][r];
            const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), d = __bfloat1622float2(h[2]), e = __bfloat1622float2(h[3]);
            acc[r] = fmaf(a.x, x0.x, acc[r]); acc[r] = fmaf(a.y, x0.y, acc[r]);
            acc[r] = fmaf(b.x, x0.z, acc[r]); acc[r] = fmaf(b.y, x0.w, acc[r]);
            acc[r] = fmaf(d.x, x1.x, acc[r]); acc[r] = fmaf(d.y, x1.y, acc[r]);
            acc[r] = fmaf(e.x, x1.z, acc[r]); acc[r] = fmaf(e.y, x1.w, acc[r]);
          }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) out[r] = warp_sum(acc[r]);
}

// mode 0: y[n] = W[n] x                     (x = rms(h) * gain when gain != null)
// mode 1: y[n] = res[n] + W[n] x            (residual add)
// mode 2: y[n] = silu(W[n] x) * (W[n + N] x)
__global__ void __launch_bounds__(LS_THREADS) step_matvec_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ gain,
                                                                 float eps, const __nv_bfloat16* __restrict__ w, int64_t ldw, int N, int K,
                                                                 const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ y, int mode,
                                                                 int rpw) {
  pdl_sync();
  extern __shared__ float xs[];
  __shared__ float red[32];
  stage_input(h, gain, eps, K, xs, red);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = LS_THREADS / 32;
  const int gw = blockIdx.x * nw + warp, tw = gridDim.x * nw;
  if (mode == 2) {
    const int pw = rpw >= 2 ? 2 : 1;               // output rows per warp and pass (each is a gate row and an up row)
    for (int n0 = gw * pw; n0 < N; n0 += tw * pw) {
      const int rows[4] = {n0, n0 + N, n0 + 1, n0 + 1 + N};
      const int cnt = (pw == 2 && n0 + 1 < N) ? 4 : 2;
      float d[4];
      warp_dot4(w, ldw, rows, cnt, xs, K, d, gw);
      if (lane == 0) {
        y[n0] = __float2bfloat16(silu_f(d[0]) * d[1]);           // on the f32 sums, as the GEMM's GLU epilogue does
        if (cnt == 4) y[n0 + 1] = __float2bfloat16(silu_f(d[2]) * d[3]);
      }
    }
  } else {
    for (int n0 = gw * rpw; n0 < N; n0 += tw * rpw) {
      const int rows[4] = {n0, n0 + 1, n0 + 2, n0 + 3};
      const int cnt = min(rpw, N - n0);
      float d[4];
      warp_dot4(w, ldw, rows, cnt, xs, K, d, gw);
      if (lane < cnt) {
        float v = lane == 0 ? d[0] : (lane == 1 ? d[1] : (lane == 2 ? d[2] : d[3]));
        if (mode == 1) v = __bfloat162float(res[n0 + lane]) + __bfloat162float(__float2bfloat16(v));
        y[n0 + lane] = __float2bfloat16(v);
      }
    }
  }
}

// One CTA per query head (D = 128, 256 threads = 8 warps).  qkv: the raw fused projection of the token [(n_q + 2 n_kv) * 128].
__global__ void __launch_bounds__(LS_THREADS) step_attention_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_gain,
                                                                    const __nv_bfloat16* __restrict__ k_gain, const float* __restrict__ inv_freq,
                                                                    const int* __restrict__ positions, const int64_t* __restrict__ slot_mapping,
                                                                    const int* __restrict__ page_table, const int* __restrict__ kv_len,
                                                                    __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                                                                    int n_q, int n_kv, int page_size, float eps, float scale,
                                                                    __nv_bfloat16* __restrict__ out, int64_t n_slots, int* __restrict__ status) {
  pdl_sync();
  constexpr int D = 128;
  __shared__ float qs[D], ks[D], vs[D];
  __shared__ float red[32];
  __shared__ float w_m[8], w_l[8], w_o[8][D];
  const int head = blockIdx.x, kvh = head / (n_q / n_kv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = positions[0];
  const int len = kv_len[0];                       // keys visible to the token, the token itself included
  // ---- norm + rotation of the q head and of its k head (threads 0..127: q, 128..255: k), v copied
  {
    const bool is_k = tid >= D;
    const int d = tid & (D - 1);
    const __nv_bfloat16* src = qkv + (is_k ? (n_q + kvh) * D : head * D);
    const float v = __bfloat162float(src[d]);
    // sum of squares per half of the CTA
    float ss = warp_sum(v * v);
    __syncthreads();
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    const float tot = is_k ? red[4] + red[5] + red[6] + red[7] : red[0] + red[1] + red[2] + red[3];
    const __nv_bfloat16* gain = is_k ? k_gain : q_gain;
    float n = v;
    if (gain) n = __bfloat162float(__float2bfloat16(v * rsqrtf(tot / (float)D + eps) * __bfloat162float(gain[d])));
    (is_k ? ks : qs)[d] = n;
    if (tid < D) vs[tid] = __bfloat162float(qkv[(n_q + n_kv + kvh) * D + tid]);
    __syncthreads();
    float r = n;
    if (inv_freq) {
      const int j = d & (D / 2 - 1);
      float sn, cs;
      sincosf((float)pos * inv_freq[j], &sn, &cs);
      const float* a = is_k ? ks : qs;
      r = d < D / 2 ? a[d] * cs - a[d + D / 2] * sn : a[d - D / 2] * sn + a[d] * cs;
      r = __bfloat162float(__float2bfloat16(r));
    }
    __syncthreads();
    (is_k ? ks : qs)[d] = r;
    __syncthreads();
  }
  // ---- append (the first query head of every kv group writes)
  if (head % (n_q / n_kv) == 0 && tid < D) {
    const int64_t slot = slot_mapping[0];
    if (slot >= 0 && slot < n_slots) {
      kcache[(slot * n_kv + kvh) * D + tid] = __float2bfloat16(ks[tid]);
      vcache[(slot * n_kv + kvh) * D + tid] = __float2bfloat16(vs[tid]);
    } else if (tid == 0) atomicCAS(status, 0, MARY_ERR_BOUNDS);
  }
  // ---- attention over positions 0 .. len - 2 from the cache, position len - 1 from shared memory
  float m = -INFINITY, l = 0.f;
  float o[4] = {0.f, 0.f, 0.f, 0.f};               // lane owns dims lane * 4 .. lane * 4 + 3
  float qreg[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) qreg[j] = qs[lane * 4 + j] * scale;
  const int n_old = len - 1;
  for (int k0 = warp * 32; k0 < n_old; k0 += 8 * 32) {
    // every lane scores one key
    const int key = k0 + lane;
    float s = -INFINITY;
    const __nv_bfloat16* kp = nullptr;
    if (key < n_old) {
      const int page = page_table[key / page_size];
      const int64_t slot = (int64_t)page * page_size + key % page_size;
      if (slot >= 0 && slot < n_slots) {
        kp = kcache + (slot * n_kv + kvh) * D;
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < D; c += 8) {
          float kv8[8];
          ld8f(kp + c, kv8);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc = fmaf(kv8[j], qs[c + j], acc);
        }
        s = acc * scale;
      }
    }
    const float mn = fmaxf(m, warp_max(s));
    const float corr = m == -INFINITY ? 0.f : __expf(m - mn);
    const float p = s == -INFINITY ? 0.f : __expf(s - mn);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] *= corr;
    m = mn;
    // weighted values: the warp walks its 32 keys, every lane adds its four dims
    const int cnt = min(32, n_old - k0);
    for (int i = 0; i < cnt; ++i) {
      const float pi = __shfl_sync(0xffffffffu, p, i);
      const int ki = k0 + i;
      const int page = page_table[ki / page_size];
      const int64_t slot = (int64_t)page * page_size + ki % page_size;
      if (slot < 0 || slot >= n_slots) continue;
      const uint2 raw = __ldg((const uint2*)(vcache + (slot * n_kv + kvh) * D + lane * 4));
      const __nv_bfloat162* hv = (const __nv_bfloat162*)&raw;
      const float2 a = __bfloat1622float2(hv[0]), b = __bfloat1622float2(hv[1]);
      o[0] = fmaf(pi, a.x, o[0]); o[1] = fmaf(pi, a.y, o[1]); o[2] = fmaf(pi, b.x, o[2]); o[3] = fmaf(pi, b.y, o[3]);
    }
  }
  // the new token itself (warp 0 takes it)
  if (warp == 0) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc = fmaf(qreg[j], ks[lane * 4 + j], acc);
    const float s = warp_sum(acc);
    const float mn = fmaxf(m, s);
    const float corr = m == -INFINITY ? 0.f : __expf(m - mn);
    const float p = __expf(s - mn);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = o[j] * corr + p * vs[lane * 4 + j];
    m = mn;
  }
  // ---- merge the eight warps
  if (lane == 0) { w_m[warp] = m; w_l[warp] = l; }
#pragma unroll
  for (int j = 0; j < 4; ++j) w_o[warp][lane * 4 + j] = o[j];
  __syncthreads();
  if (tid < D) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) mm = fmaxf(mm, w_m[w]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float c = w_m[w] == -INFINITY ? 0.f : __expf(w_m[w] - mm);
      ll += w_l[w] * c;
      acc += w_o[w][tid] * c;
    }
    out[head * D + tid] = __float2bfloat16(acc / ll);
  }
}
}  // namespace

// y[N] = f(W[N (or 2N), K] x) with the stage's folded neighbours (mode: 0 plain, 1 + residual, 2 SwiGLU over [gate; up] rows);
// gain != null: x = rms(h) * gain, else x = h.
MARY_API int mary_step_matvec(const void* h, const void* gain, float eps, const void* w, int64_t ldw, int N, int K, const void* res, void* y,
                              int mode, cudaStream_t s) {
  if (N <= 0 || K <= 0 || (K & 7) || (ldw & 7) || K > LS_MAX_H || mode < 0 || mode > 2 || (mode == 1 && !res)) return MARY_ERR_BAD_ARG;
  // rows per warp and pass: as many as still give every SM a CTA (a narrow output with one row per warp fills the machine,
  // a wide one keeps four rows of loads in flight per warp)
  const int sms = mary_num_sms(), nw = LS_THREADS / 32;
  int rpw = mode == 2 ? 2 : 4;
  while (rpw > 1 && (N + nw * rpw - 1) / (nw * rpw) < sms) rpw >>= 1;
  int grid = (N + nw * rpw - 1) / (nw * rpw);
  const int cap = 4 * sms;
  if (grid > cap) grid = cap;
  MARY_LAUNCH(step_matvec_kernel, grid, LS_THREADS, (size_t)K * sizeof(float), s, (const __nv_bfloat16*)h, (const __nv_bfloat16*)gain, eps,
              (const __nv_bfloat16*)w, ldw, N, K, (const __nv_bfloat16*)res, (__nv_bfloat16*)y, mode, rpw);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// One token of one sequence: head norms, rotation, cache append and attention (head dim 128).
MARY_API int mary_step_attention(const void* qkv, const void* q_gain, const void* k_gain, const float* inv_freq, const int* positions,
                                 const int64_t* slot_mapping, const int* page_table, const int* kv_len, void* kcache, void* vcache, int n_q,
                                 int n_kv, int head_dim, int page_size, int64_t n_slots, float eps, float scale, void* out, cudaStream_t s) {
  if (head_dim != 128 || n_q < 1 || n_kv < 1 || n_q % n_kv || page_size < 1) return MARY_ERR_BAD_ARG;
  MARY_LAUNCH(step_attention_kernel, n_q, LS_THREADS, 0, s, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)q_gain, (const __nv_bfloat16*)k_gain,
              inv_freq, positions, slot_mapping, page_table, kv_len, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, n_q, n_kv, page_size, eps,
              scale, (__nv_bfloat16*)out, n_slots, mary_status_ptr());
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
