// Fused expert pipeline, the two kernels that run on a token's HOME rank (see ep_ctx.cuh for the whole protocol):
//
//   ep_route_dispatch   router top-k + slot reservation (remote atomics on the owners' arrival counters) + NVFP4 quantisation
//                       of the token row (once, whatever the number of experts it visits) + peer stores of codes, scale
//                       bytes and return words into the owners' slabs + "dispatched" flags from the last CTA;
//   ep_combine          bounded wait for the owners' "returned" flags + weighted sum of the k returned rows in slot order
//                       (+ an optional addend) + optional residual add and RMSNorm for the next block.
//
// Between them run the two grouped NVFP4 GEMMs of gemm_nvfp4.cu in counter mode.  Replaces, per MoE layer: router top-k,
// counts, barrier, plan, dispatch, barrier, quantise, return pointers, barrier, un-permute and add + norm (11 launches with
// three cross-GPU barrier kernels) by these two.  The quantiser follows the reference's rules bit for bit
// (src/models/inkling/fp4quant.rs:10-54: per 16 elements amax -> min(amax / 6, 448) -> E4M3 RNE -> codes by thresholds with
// ties away from zero, signed zero kept, zero block -> scale byte 0); the weighted sum is the reference's `scatter_weighted`
// order (src/models/inkling/moegroup.rs:841-939).
#include <cuda_fp8.h>

#include "common.cuh"
#include "ep_ctx.cuh"
#include "host_utils.h"
#include "nvfp4_quant.cuh"
#include "router_block.cuh"

using namespace mary;

namespace {

struct RouteParams {
  const float* logits; int64_t ld;       // [T, E] f32
  const float* bias;                     // [E] or null
  const __nv_bfloat16* x; int64_t ldx;   // [T, H]
  int T, E, k, mode, n_group, topk_group, renorm, has_shared, H;
  float scale;
  int* idx_out;                          // [T, K1] global expert id of every entry (E = the shared expert)
  float* w_out;                          // [T, K1]
  int* row_out;                          // [T, K1] slab row on the owner, -1 = entry not served (dropped in local_only mode)
  int* flag;                             // set when a router logit is not finite
  int* status;
};

__global__ void __launch_bounds__(256)
ep_route_dispatch_kernel(const RouteParams p, const EpCtx c) {
  pdl_sync();
  __shared__ RouterSmem S;
  __shared__ int s_row[33], s_dst[33];
  extern __shared__ __align__(16) uint8_t dyn[];
  uint2* s_codes = (uint2*)dyn;                         // [H / 16] 8 bytes each
  uint8_t* s_sf = dyn + (size_t)p.H / 2;                // [H / 16]
  const int t = blockIdx.x, tid = threadIdx.x;
  const int K1 = p.k + (p.has_shared ? 1 : 0);
  if (t < p.T) {
    // quantise the row once (its loads are in flight while the router runs; the codes wait in shared memory)
    const __nv_bfloat16* xr = p.x + (int64_t)t * p.ldx;
    for (int b = tid; b < p.H / 16; b += blockDim.x) {
      const uint4 v0 = *(const uint4*)(xr + b * 16), v1 = *(const uint4*)(xr + b * 16 + 8);
      float f[16];
      const __nv_bfloat162* p0 = (const __nv_bfloat162*)&v0;
      const __nv_bfloat162* p1 = (const __nv_bfloat162*)&v1;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 a = __bfloat1622float2(p0[j]), q = __bfloat1622float2(p1[j]);
        f[2 * j] = a.x; f[2 * j + 1] = a.y; f[8 + 2 * j] = q.x; f[8 + 2 * j + 1] = q.y;
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
        for (int j = 0; j < 8; ++j) { lo |= nvfp4_code(__fdiv_rn(f[j], s)) << (4 * j); hi |= nvfp4_code(__fdiv_rn(f[8 + j], s)) << (4 * j); }
      }
      s_codes[b] = make_uint2(lo, hi);
      s_sf[b] = (uint8_t)sb;
    }
    router_block(p.logits + (int64_t)t * p.ld, p.bias, p.E, p.k, p.mode, p.n_group, p.topk_group, p.scale, p.renorm, S, p.flag);
    if (tid < K1) {
      const bool shared = tid >= p.k;
      const int e = shared ? p.E : S.out_i[tid];
      int d, le;
      bool valid = shared || (e >= 0 && e < p.E);
      if (shared) { d = c.rank; le = c.e_local; if (c.local_only && c.world > 1) valid = (t % c.world) == c.rank; }
      else { d = e / c.e_local; le = e - d * c.e_local; if (c.local_only && d != c.rank) valid = false; }
      int row = -1;
      if (valid) {
        const int slot = atomicAdd_system((int*)c.cnt[d] + le, 1);
        if (slot < c.cap_e) row = le * c.cap_e + slot;
        else atomicCAS(p.status, 0, MARY_ERR_BOUNDS);      // the slab region of this expert is full: the entry is dropped
      }
      s_row[tid] = row; s_dst[tid] = valid ? d : c.rank;
      p.idx_out[(int64_t)t * K1 + tid] = e;
      p.w_out[(int64_t)t * K1 + tid] = shared ? 1.0f : S.out_w[tid];
      p.row_out[(int64_t)t * K1 + tid] = row;
    }
    __syncthreads();
    // stores: per destination H / 32 16-byte vectors of codes and H / 64 4-byte groups of scales (four consecutive 16-element
    // blocks are adjacent bytes of the tensor-core scale tile)
    const int n16 = p.H / 32, nsf = p.H / 64, per = n16 + nsf;
    for (int i = tid; i < K1 * per; i += blockDim.x) {
      const int j = i / per, r = i - j * per;
      const int row = s_row[j];
      if (row < 0) continue;
      const int d = s_dst[j];
      if (r < n16) {
        ((uint4*)((uint8_t*)c.xq[d] + (int64_t)row * (p.H / 2)))[r] = ((const uint4*)s_codes)[r];
      } else {
        const int g = r - n16, tile = row / c.NT, rr = row % c.NT;
        uint8_t* sfd = (uint8_t*)c.sf[d] + (int64_t)tile * nsf * 512 + (rr % 32) * 16 + (rr / 32) * 4 + (int64_t)g * 512;
        *(uint32_t*)sfd = ((const uint32_t*)s_sf)[g];
      }
    }
    if (tid < K1 && s_row[tid] >= 0) ((int*)c.meta[s_dst[tid]])[s_row[tid]] = c.rank * c.entry_stride + t * K1 + tid;
  }
  // completion: the CTA that finishes last publishes this rank's "dispatched" flag on every owner
  if (c.local_only) __threadfence(); else __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const int prev = atomicAdd(&c.done[0], 1);
    if (prev == (int)gridDim.x - 1) {
      c.done[0] = 0;
      const uint32_t target = *c.epoch + 1;
      __threadfence_system();
      if (c.local_only) ep_st_release_sys((uint32_t*)c.flags[c.rank] + c.rank, target);
      else for (int d = 0; d < c.world; ++d) ep_st_release_sys((uint32_t*)c.flags[(c.rank + d) % c.world] + c.rank, target);
    }
  }
}

struct CombineParams {
  const float* w;                  // [T, K1]
  const int* rows;                 // [T, K1] (-1: slot skipped)
  const __nv_bfloat16* add;        // [T, H] or null: added to the weighted sum before rounding
  __nv_bfloat16* out;              // [T, H] the weighted sum (mode without residual), or null
  __nv_bfloat16* res;              // [T, H] residual, updated in place (res += sum, one rounding), or null
  const __nv_bfloat16* w_norm;     // gain of the norm applied to the new residual, or null
  __nv_bfloat16* y;                // [T, H] normed output
  int T, K1, H;
  float eps;
  int* status;
};

__global__ void __launch_bounds__(1024)
ep_combine_kernel(const CombineParams p, const EpCtx c) {
  pdl_sync();
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  __shared__ int ok_s;
  const int t = blockIdx.x, tid = threadIdx.x;
  const uint32_t target = *c.epoch + 1;
  if (tid == 0) ok_s = 1;
  __syncthreads();
  if (!c.local_only && c.world > 1 && tid < c.world) {
    if (!ep_wait_flag((const uint32_t*)c.flags[c.rank] + EP_MAX_RANKS + tid, target, c.wait_ns, p.status)) ok_s = 0;
  }
  __syncthreads();
  if (t < p.T && ok_s) {
    const __nv_bfloat16* comb = (const __nv_bfloat16*)c.comb[c.rank];
    float ss = 0.f;
    for (int i = tid * 8; i < p.H; i += blockDim.x * 8) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      if (p.add) {
        const uint4 a = *(const uint4*)(p.add + (int64_t)t * p.H + i);
        const __nv_bfloat162* ap = (const __nv_bfloat162*)&a;
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(ap[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
      }
      for (int j = 0; j < p.K1; ++j) {
        if (p.rows[t * p.K1 + j] < 0) continue;
        const float wj = p.w[t * p.K1 + j];
        // the rows were written by other GPUs' kernels, possibly during this launch's lifetime: L2 loads, never the
        // read-only (non-coherent) path
        const uint4 v = __ldcg((const uint4*)(comb + ((int64_t)t * p.K1 + j) * p.H + i));
        const __nv_bfloat162* vp = (const __nv_bfloat162*)&v;
#pragma unroll
        for (int q = 0; q < 4; ++q) { float2 f = __bfloat1622float2(vp[q]); acc[2 * q] = fmaf(f.x, wj, acc[2 * q]); acc[2 * q + 1] = fmaf(f.y, wj, acc[2 * q + 1]); }
      }
      uint4 o;
      __nv_bfloat162* op = (__nv_bfloat162*)&o;
#pragma unroll
      for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      if (p.out) *(uint4*)(p.out + (int64_t)t * p.H + i) = o;
      if (p.res) {
        uint4 hv = *(const uint4*)(p.res + (int64_t)t * p.H + i);
        __nv_bfloat162* hp = (__nv_bfloat162*)&hv;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(op[j]), h = __bfloat1622float2(hp[j]);
          hp[j] = __floats2bfloat162_rn(h.x + f.x, h.y + f.y);
          const float2 r = __bfloat1622float2(hp[j]);
          rowbuf[i + 2 * j] = r.x; rowbuf[i + 2 * j + 1] = r.y;
          ss += r.x * r.x + r.y * r.y;
        }
        *(uint4*)(p.res + (int64_t)t * p.H + i) = hv;
      }
    }
    if (p.res && p.w_norm) {
      ss = warp_sum(ss);
      const int wi = tid >> 5, l = tid & 31;
      if (l == 0) red[wi] = ss;
      __syncthreads();
      float tot = (l < (int)(blockDim.x >> 5)) ? red[l] : 0.f;
      tot = warp_sum(tot);
      const float inv = rsqrtf(tot / p.H + p.eps);
      for (int i = tid * 8; i < p.H; i += blockDim.x * 8) {
        const uint4 gv = *(const uint4*)(p.w_norm + i);
        const __nv_bfloat162* gp = (const __nv_bfloat162*)&gv;
        uint4 o;
        __nv_bfloat162* op = (__nv_bfloat162*)&o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = __bfloat1622float2(gp[j]);
          op[j] = __floats2bfloat162_rn(rowbuf[i + 2 * j] * inv * g.x, rowbuf[i + 2 * j + 1] * inv * g.y);
        }
        *(uint4*)(p.y + (int64_t)t * p.H + i) = o;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    const int prev = atomicAdd(&c.done[2], 1);
    if (prev == (int)gridDim.x - 1) {            // every CTA has read the epoch: the layer call is over, advance it
      c.done[2] = 0;
      __threadfence();
      *c.epoch = target;
    }
  }
}

}  // namespace

// ctx: an EpCtx by value (the Python side fills the same layout with ctypes).
MARY_API int mary_ep_route_dispatch(const float* logits, int64_t ld, const float* bias, const void* x, int64_t ldx, int T, int E, int k,
                                    int mode, int n_group, int topk_group, float scale, int renorm, int has_shared, int H, int* idx_out,
                                    float* w_out, int* row_out, int* flag, const EpCtx* ctx, cudaStream_t s) {
  const int K1 = k + (has_shared ? 1 : 0);
  if (E > 512 || k < 1 || K1 > 32 || k * 8 > 256 || n_group > 32 || (n_group > 1 && E % n_group) || (H % 64) || (ldx % 8) || T < 0 ||
      ctx->world < 1 || ctx->world > EP_MAX_RANKS || (ctx->cap_e % ctx->NT) || (int64_t)T * K1 > ctx->entry_stride ||
      ctx->n_slots > EP_MAX_TILES)
    return MARY_ERR_BAD_ARG;
  RouteParams p;
  p.logits = logits; p.ld = ld; p.bias = bias; p.x = (const __nv_bfloat16*)x; p.ldx = ldx; p.T = T; p.E = E; p.k = k; p.mode = mode;
  p.n_group = n_group; p.topk_group = topk_group; p.renorm = renorm; p.has_shared = has_shared; p.H = H; p.scale = scale;
  p.idx_out = idx_out; p.w_out = w_out; p.row_out = row_out; p.flag = flag; p.status = mary_status_ptr();
  const size_t sm = (size_t)H / 2 + (size_t)H / 16;
  if (sm > 40 * 1024) return MARY_ERR_BAD_ARG;
  MARY_LAUNCH(ep_route_dispatch_kernel, T > 0 ? T : 1, 256, sm, s, p, *ctx);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// out (weighted sum, may be null when res is given) ; res != null: res += sum (one rounding) and, with w_norm, y = rms(res) * w_norm.
MARY_API int mary_ep_combine(const float* w, const int* rows, const void* add, void* out, void* res, const void* w_norm, void* y, int T,
                             int K1, int H, float eps, const EpCtx* ctx, cudaStream_t s) {
  if ((H % 8) || (size_t)H * 4 > 48 * 1024 || T < 0 || (!out && !res) || (w_norm && (!res || !y))) return MARY_ERR_BAD_ARG;
  CombineParams p;
  p.w = w; p.rows = rows; p.add = (const __nv_bfloat16*)add; p.out = (__nv_bfloat16*)out; p.res = (__nv_bfloat16*)res;
  p.w_norm = (const __nv_bfloat16*)w_norm; p.y = (__nv_bfloat16*)y; p.T = T; p.K1 = K1; p.H = H; p.eps = eps; p.status = mary_status_ptr();
  int threads = (H / 8 + 31) / 32 * 32;              // one 16-byte column vector per thread when the row fits: all loads in flight at once
  threads = threads > 1024 ? 1024 : (threads < 64 ? 64 : threads);
  MARY_LAUNCH(ep_combine_kernel, T > 0 ? T : 1, threads, (size_t)H * 4, s, p, *ctx);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_ep_ctx_bytes() { return (int)sizeof(EpCtx); }
