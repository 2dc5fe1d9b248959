// MoE plumbing around the grouped expert GEMM: routing plan (counting sort by expert, padded to the token-tile
// width), gather + NVFP4 activation quantisation, and the weighted un-permute.
//
// Reference pieces: host `RowPlan` (src/models/inkling/moegroup.rs:978-1083), `gather_grouped`
// (moegroup.rs:146-240), `quantize_nvfp4_kernel` (src/models/inkling/fp4quant.rs:122-244; rules :10-54 —
// per 16 elements amax -> min(amax/6, 448) -> E4M3 round-to-nearest-even -> codes by the thresholds
// .25 .75 1.25 1.75 2.5 3.5 5 with ties away from zero, signed zero kept, zero block -> scale byte 0),
// `scatter_weighted` (moegroup.rs:841-939: out[t] = sum_j y[row_j] * w[row_j] in ascending order with fma).
// Here the plan is built on the device, so no readback separates the router from the expert GEMMs
// (the reference blocks on a router readback once per MoE layer, src/bin/inkling_forward.rs:4442-4478).
#include <cuda_fp8.h>

#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

struct Tile { int expert, row0, rows, sf_tile; };

// One CTA.  idx[n_entries] = expert of every (token, slot) entry (negative = entry not routed here).
// Outputs: row_of[n_entries] padded row of each entry (-1 if skipped), src_of[max_rows] token of each padded row
// (-1 for padding), tiles/n_tiles for the grouped GEMM, counts[E], meta = {n_tiles, padded rows}.
__global__ void moe_plan_kernel(const int* __restrict__ idx, int n_entries, int k, int E, int NT, int max_rows, int* __restrict__ row_of,
                                int* __restrict__ src_of, Tile* __restrict__ tiles, int* __restrict__ meta, int* __restrict__ counts_out) {
  pdl_sync();
  extern __shared__ int sh[];
  int* cnt = sh;            // [E]
  int* off = sh + E;        // [E + 1]
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  for (int r = threadIdx.x; r < max_rows; r += blockDim.x) src_of[r] = -1;
  __syncthreads();
  // Slots inside an expert come from a shared-memory counter.  Their order within a chunk of blockDim entries
  // depends on scheduling, which does not matter: every row of the grouped GEMM is independent and the un-permute
  // sums a token's k results in fixed slot order.
  for (int base = 0; base < n_entries; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int e = (i < n_entries) ? idx[i] : -1;
    int slot = -1;
    if (e >= 0 && e < E) slot = atomicAdd(&cnt[e], 1);      // (a warp-aggregated form with match.any measured slower: 108 against 70 us)
    if (i < n_entries) row_of[i] = slot;       // provisional: slot inside the expert
    __syncthreads();
  }
  // exclusive prefix sum of the padded counts as a block scan (warp shuffles + one pass over the warp totals)
  {
    __shared__ int warp_tot[33];
    __shared__ int carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int base = 0; base < E; base += blockDim.x) {
      const int e = base + threadIdx.x;
      const int padded = e < E ? (cnt[e] + NT - 1) / NT * NT : 0;
      int incl = padded;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
      if (lane == 31) warp_tot[wid] = incl;
      __syncthreads();
      if (wid == 0) {
        const int wt = lane < nw ? warp_tot[lane] : 0;
        int wi = wt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, wi, o); if (lane >= o) wi += v; }
        __syncwarp();
        warp_tot[lane] = wi - wt;                      // exclusive offset of warp `lane`
        if (lane == 31) warp_tot[32] = wi;             // total of this pass
      }
      __syncthreads();
      if (e < E) off[e] = carry_s + warp_tot[wid] + incl - padded;
      __syncthreads();
      if (threadIdx.x == 0) carry_s += warp_tot[32];
      __syncthreads();
    }
    if (threadIdx.x == 0) { off[E] = carry_s; meta[0] = carry_s / NT; meta[1] = carry_s; }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (counts_out) counts_out[e] = cnt[e];
    const int c = cnt[e];
    for (int i = 0; i * NT < c; ++i) {
      Tile t{e, off[e] + i * NT, min(NT, c - i * NT), off[e] / NT + i};
      tiles[off[e] / NT + i] = t;
    }
  }
  for (int i = threadIdx.x; i < n_entries; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < E) {
      const int row = off[e] + row_of[i];
      row_of[i] = row;
      src_of[row] = i / k;
    } else row_of[i] = -1;
  }
}

__device__ __forceinline__ uint32_t e2m1_code(float y) {
  const float m = fabsf(y);
  uint32_t c = (m >= 0.25f) + (m >= 0.75f) + (m >= 1.25f) + (m >= 1.75f) + (m >= 2.5f) + (m >= 3.5f) + (m >= 5.0f);
  return c | (signbit(y) ? 8u : 0u);
}

// One CTA per destination row.  src_of[row] < 0 -> padding row, skipped.  identity != 0 -> the source row is `row`
// itself (re-quantising an intermediate that is already in padded-row order; src_of only marks validity, may be null).
// Scales go to the 512-byte block layout of the row's NT-row tile; optionally also row-major (tests, dense users).
// With row_of (entry -> padded row, k entries per token) the grid runs over the ENTRIES instead of the padded rows: a decode
// batch has a few hundred entries but thousands of padded rows, most of them padding.
// 16 consecutive values -> 8 code bytes and the scale byte of their block
__device__ __forceinline__ uint2 nvfp4_block16(const __nv_bfloat16* __restrict__ src, uint8_t* sb_out) {
  const uint4 v0 = *(const uint4*)src, v1 = *(const uint4*)(src + 8);
  float f[16];
  const __nv_bfloat162* p0 = (const __nv_bfloat162*)&v0;
  const __nv_bfloat162* p1 = (const __nv_bfloat162*)&v1;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 a = __bfloat1622float2(p0[j]), c = __bfloat1622float2(p1[j]);
    f[2 * j] = a.x; f[2 * j + 1] = a.y; f[8 + 2 * j] = c.x; f[8 + 2 * j + 1] = c.y;
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
  const float sfv = fminf(__fdiv_rn(amax, 6.0f), 448.0f);
  const __nv_fp8_storage_t sb = __nv_cvt_float_to_fp8(sfv, __NV_SATFINITE, __NV_E4M3);
  const float s = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
  uint32_t lo = 0, hi = 0;
  if (s > 0.f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { lo |= e2m1_code(__fdiv_rn(f[j], s)) << (4 * j); hi |= e2m1_code(__fdiv_rn(f[8 + j], s)) << (4 * j); }
  }
  *sb_out = (uint8_t)sb;
  return make_uint2(lo, hi);
}

__global__ void quant_nvfp4_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const int* __restrict__ src_of, int identity,
                                        int Kd, int NT, uint8_t* __restrict__ xq, uint8_t* __restrict__ sf_tiles,
                                        uint8_t* __restrict__ sf_rowmajor, const int* __restrict__ n_rows,
                                        const int* __restrict__ row_of, int k) {
  pdl_sync();
  int row = blockIdx.x;
  int src = row;
  if (row_of) {
    row = row_of[blockIdx.x];
    if (row < 0) return;
    src = identity ? row : (int)blockIdx.x / k;
  } else {
    if (n_rows && row >= *n_rows) return;
    if (src_of) { const int s = src_of[row]; if (s < 0) return; if (!identity) src = s; }
  }
  const __nv_bfloat16* xr = x + (int64_t)src * ldx;
  const int tile = row / NT, r = row % NT;
  const int64_t sf_base = (int64_t)tile * (Kd / 64) * 512 + (r % 32) * 16 + (r / 32) * 4;
  for (int b = threadIdx.x; b < Kd / 16; b += blockDim.x) {
    uint8_t sb;
    const uint2 code = nvfp4_block16(xr + b * 16, &sb);
    *(uint2*)(xq + (int64_t)row * (Kd / 2) + b * 8) = code;
    if (sf_tiles) sf_tiles[sf_base + (int64_t)(b / 4) * 512 + (b % 4)] = sb;
    if (sf_rowmajor) sf_rowmajor[(int64_t)row * (Kd / 16) + b] = sb;
  }
}

// Token-driven form for batches with many tokens: one CTA per TOKEN quantises the row once and writes the bytes to the padded
// row of each of its k routed entries (the entry-driven form above repeats the arithmetic k times, which dominates once the
// batch has thousands of tokens).  K_ENT: entries per token held in registers (k <= K_ENT).
template <int K_ENT>
__global__ void quant_nvfp4_tokens_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const int* __restrict__ row_of, int k, int Kd,
                                          int NT, uint8_t* __restrict__ xq, uint8_t* __restrict__ sf_tiles) {
  pdl_sync();
  const int t = blockIdx.x;
  int rows[K_ENT];
  int64_t sfb[K_ENT];
#pragma unroll
  for (int j = 0; j < K_ENT; ++j) {
    rows[j] = j < k ? row_of[t * k + j] : -1;
    const int tile = rows[j] / NT, r = rows[j] % NT;
    sfb[j] = (int64_t)tile * (Kd / 64) * 512 + (r % 32) * 16 + (r / 32) * 4;
  }
  const __nv_bfloat16* xr = x + (int64_t)t * ldx;
  for (int b = threadIdx.x; b < Kd / 16; b += blockDim.x) {
    uint8_t sb;
    const uint2 code = nvfp4_block16(xr + b * 16, &sb);
#pragma unroll
    for (int j = 0; j < K_ENT; ++j)
      if (rows[j] >= 0) {
        *(uint2*)(xq + (int64_t)rows[j] * (Kd / 2) + b * 8) = code;
        sf_tiles[sfb[j] + (int64_t)(b / 4) * 512 + (b % 4)] = sb;
      }
  }
}

// out[t, :] = sum_j w[t, j] * y[row_of[t*k + j], :]  (+ add[t, :]) in ascending j with fma; grid (token, column slab): a
// decode batch has few tokens, so the hidden dimension is spread over gridDim.y CTAs to fill the machine.
__global__ void moe_unpermute_kernel(const __nv_bfloat16* __restrict__ y, int64_t ldy, const int* __restrict__ row_of,
                                     const float* __restrict__ w, int k, int H, const __nv_bfloat16* __restrict__ add,
                                     __nv_bfloat16* __restrict__ out) {
  pdl_sync();
  const int t = blockIdx.x;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < H; c += gridDim.y * blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (add) {
      const uint4 a = *(const uint4*)(add + (int64_t)t * H + c);
      const __nv_bfloat162* ap = (const __nv_bfloat162*)&a;
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(ap[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
    }
    for (int j = 0; j < k; ++j) {
      const int row = row_of[t * k + j];
      if (row < 0) continue;
      const float wj = w[t * k + j];
      const uint4 v = *(const uint4*)(y + (int64_t)row * ldy + c);
      const __nv_bfloat162* vp = (const __nv_bfloat162*)&v;
#pragma unroll
      for (int q = 0; q < 4; ++q) { float2 f = __bfloat1622float2(vp[q]); acc[2 * q] = fmaf(f.x, wj, acc[2 * q]); acc[2 * q + 1] = fmaf(f.y, wj, acc[2 * q + 1]); }
    }
    uint4 o;
    __nv_bfloat162* op = (__nv_bfloat162*)&o;
#pragma unroll
    for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *(uint4*)(out + (int64_t)t * H + c) = o;
  }
}

}  // namespace

MARY_API int mary_moe_plan(const int* idx, int n_entries, int k, int E, int NT, int max_rows, int* row_of, int* src_of, void* tiles,
                           int* meta, int* counts, cudaStream_t s) {
  if (E > 4096 || NT <= 0) return MARY_ERR_BAD_ARG;
  MARY_LAUNCH(moe_plan_kernel, 1, 1024, (2 * E + 1) * sizeof(int), s, idx, n_entries, k, E, NT, max_rows, row_of, src_of, (Tile*)tiles, meta, counts);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// Upper bound of padded rows for n_entries routed entries over E experts with tile width NT.
MARY_API int mary_moe_max_rows(int n_entries, int E, int NT) {
  const int worst = n_entries + (n_entries < E ? n_entries : E) * (NT - 1);
  return (worst + NT - 1) / NT * NT;
}

MARY_API int mary_quant_nvfp4_rows(const void* x, int64_t ldx, const int* src_of, int identity, int rows, int K, int NT, void* xq,
                                   void* sf_tiles, void* sf_rowmajor, const int* n_rows, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if ((K % 64) || (ldx % 8)) return MARY_ERR_BAD_ARG;
  int threads = K / 16 < 256 ? ((K / 16 + 31) / 32 * 32) : 256;
  MARY_LAUNCH(quant_nvfp4_rows_kernel, rows, threads, 0, s, (const __nv_bfloat16*)x, ldx, src_of, identity, K, NT, (uint8_t*)xq, (uint8_t*)sf_tiles,
                                                   (uint8_t*)sf_rowmajor, n_rows, nullptr, 1);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// The same quantiser driven by the routed entries: entry i (token i / k) goes to padded row row_of[i] (negative: not routed here).
// identity != 0 re-quantises x's own row row_of[i] (an intermediate already in padded-row order).
MARY_API int mary_quant_nvfp4_entries(const void* x, int64_t ldx, const int* row_of, int n_entries, int k, int identity, int K, int NT,
                                      void* xq, void* sf_tiles, cudaStream_t s) {
  if (n_entries <= 0) return MARY_OK;
  if ((K % 64) || (ldx % 8) || k < 1) return MARY_ERR_BAD_ARG;
  int threads = K / 16 < 256 ? ((K / 16 + 31) / 32 * 32) : 256;
  if (!identity && k > 1 && k <= 16 && n_entries >= 2048 && n_entries % k == 0) {
    if (k <= 8) {
      MARY_LAUNCH(quant_nvfp4_tokens_kernel<8>, n_entries / k, threads, 0, s, (const __nv_bfloat16*)x, ldx, row_of, k, K, NT, (uint8_t*)xq,
                                                                  (uint8_t*)sf_tiles);
    } else {
      MARY_LAUNCH(quant_nvfp4_tokens_kernel<16>, n_entries / k, threads, 0, s, (const __nv_bfloat16*)x, ldx, row_of, k, K, NT, (uint8_t*)xq,
                                                                   (uint8_t*)sf_tiles);
    }
    MARY_CHECK_LAUNCH();
    return MARY_OK;
  }
  MARY_LAUNCH(quant_nvfp4_rows_kernel, n_entries, threads, 0, s, (const __nv_bfloat16*)x, ldx, nullptr, identity, K, NT, (uint8_t*)xq,
                                                        (uint8_t*)sf_tiles, nullptr, nullptr, row_of, k);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_moe_unpermute(const void* y, int64_t ldy, const int* row_of, const float* w, int T, int k, int H, const void* add,
                                void* out, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  if (H % 8) return MARY_ERR_BAD_ARG;
  const int slabs = (H / 8 + 127) / 128;       // 128 threads x 8 columns per CTA
  MARY_LAUNCH(moe_unpermute_kernel, dim3(T, slabs), 128, 0, s, (const __nv_bfloat16*)y, ldy, row_of, w, k, H, (const __nv_bfloat16*)add,
                                                     (__nv_bfloat16*)out);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
