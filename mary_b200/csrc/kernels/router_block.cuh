// One CTA (256 threads) routes one token: softmax or sigmoid(+bias) scores, optional group-limited pre-selection, the k best
// experts with ties going to the lower index, renormalised weights.  Shared by the stand-alone router kernel (select.cu) and
// the fused route + dispatch kernel of the expert pipeline (ep_fused.cu).
// Rules: sigmoid+bias selection with unbiased weights (src/models/k3/router.rs:9-15, src/models/inkling/routetopk.rs:112-260),
// softmax top-k with renormalisation (src/models/gemma/gemma4/layers.rs:269-325); the group-limited branch, which the
// reference refuses (src/models/k3/router.rs:136-143), keeps the `topk_group` groups whose two best biased scores sum highest.
//
// Decode batches hold tens to hundreds of tokens, and a single warp walking ~400 experts through group scoring and k arg-max
// rounds is a serial chain of thousands of dependent instructions (tens of microseconds).  Here every thread owns at most two
// experts; the groups are scored by different warps at once; every warp extracts the k best of its own 1/8 of the experts and
// warp 0 merges the 8 k candidates.
#pragma once
#include "common.cuh"

namespace mary {

struct MaxIdx { float v; int i; };
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {      // larger value, then smaller index
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ MaxIdx warp_best(MaxIdx a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = better(a, b);
  }
  return a;
}

struct RouterSmem {
  float sc[512], sel[512], g[32], red[8], cv[256];
  int ci[256];
  uint32_t keep;
  int out_i[32];       // the chosen experts, best first
  float out_w[32];     // their weights (renormalised, scaled)
};

// Every thread of the 256-thread CTA calls this; E <= 512, k <= 32, k * 8 <= 256.  On return (after the trailing barrier)
// S.out_i[0 .. k) / S.out_w[0 .. k) hold the result.  A non-finite logit sets *flag.
__device__ __forceinline__ void router_block(const float* __restrict__ row, const float* __restrict__ bias, int E, int k, int mode,
                                             int n_group, int topk_group, float scale, int renorm, RouterSmem& S, int* __restrict__ flag) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float v0 = -INFINITY, v1 = -INFINITY;
  bool bad = false;
  if (tid < E) { v0 = row[tid]; bad |= !isfinite(v0); }
  if (tid + 256 < E) { v1 = row[tid + 256]; bad |= !isfinite(v1); }
  if (bad && flag) atomicExch(flag, 1);
  if (mode == 0) {
    float mx = warp_max(fmaxf(v0, v1));
    if (lane == 0) S.red[warp] = mx;
    __syncthreads();
    mx = S.red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, S.red[w]);
    __syncthreads();
    const float e0 = tid < E ? __expf(v0 - mx) : 0.f, e1 = tid + 256 < E ? __expf(v1 - mx) : 0.f;
    float sum = warp_sum(e0 + e1);
    if (lane == 0) S.red[warp] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += S.red[w];
    if (tid < E) { S.sc[tid] = e0 / sum; S.sel[tid] = e0 / sum; }
    if (tid + 256 < E) { S.sc[tid + 256] = e1 / sum; S.sel[tid + 256] = e1 / sum; }
  } else {
    if (tid < E) { const float sg = 1.0f / (1.0f + __expf(-v0)); S.sc[tid] = sg; S.sel[tid] = sg + (bias ? bias[tid] : 0.f); }
    if (tid + 256 < E) { const float sg = 1.0f / (1.0f + __expf(-v1)); S.sc[tid + 256] = sg; S.sel[tid + 256] = sg + (bias ? bias[tid + 256] : 0.f); }
  }
  __syncthreads();
  if (mode == 1 && n_group > 1) {
    const int gsz = E / n_group;
    for (int g = warp; g < n_group; g += 8) {               // group score = sum of the two best biased scores in the group
      MaxIdx b1{-INFINITY, 0x7fffffff};
      for (int m = lane; m < gsz; m += 32) b1 = better(b1, MaxIdx{S.sel[g * gsz + m], g * gsz + m});
      b1 = warp_best(b1);
      MaxIdx b2{-INFINITY, 0x7fffffff};
      for (int m = lane; m < gsz; m += 32) { const int e = g * gsz + m; if (e != b1.i) b2 = better(b2, MaxIdx{S.sel[e], e}); }
      b2 = warp_best(b2);
      if (lane == 0) S.g[g] = b1.v + b2.v;
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t keep = 0;
      const float mine = lane < n_group ? S.g[lane] : -INFINITY;
      for (int r = 0; r < topk_group; ++r) {
        MaxIdx b = warp_best(MaxIdx{(lane < n_group && !((keep >> lane) & 1u)) ? mine : -INFINITY, lane});
        keep |= 1u << b.i;
      }
      if (lane == 0) S.keep = keep;
    }
    __syncthreads();
    const uint32_t keep = S.keep;
    if (tid < E && !((keep >> (tid / gsz)) & 1u)) S.sel[tid] = -INFINITY;
    if (tid + 256 < E && !((keep >> ((tid + 256) / gsz)) & 1u)) S.sel[tid + 256] = -INFINITY;
    __syncthreads();
  }
  // every warp: the k best of its own slice of the experts
  {
    const int chunk = (E + 7) / 8;                            // <= 64: two experts per lane
    const int base = warp * chunk;
    const int ea = base + lane, eb = base + lane + 32;
    float a = (lane < chunk && ea < E) ? S.sel[ea] : -INFINITY;
    float b = (lane + 32 < chunk && eb < E) ? S.sel[eb] : -INFINITY;
    for (int r = 0; r < k; ++r) {
      MaxIdx best = warp_best(better(MaxIdx{a, ea}, MaxIdx{b, eb}));
      if (best.i == ea) a = -INFINITY;
      if (best.i == eb) b = -INFINITY;
      if (lane == 0) { S.cv[warp * k + r] = best.v; S.ci[warp * k + r] = best.i; }
    }
  }
  __syncthreads();
  if (warp == 0) {
    // merge 8 k candidates (each warp's list is in descending order, which the merge does not need)
    const int n = 8 * k;
    float cv[8];
    int ci[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { const int c = lane + 32 * j; cv[j] = c < n ? S.cv[c] : -INFINITY; ci[j] = c < n ? S.ci[c] : 0x7fffffff; }
    float wsum = 0.f, mine_w = 0.f;
    int mine_i = 0;
    for (int r = 0; r < k; ++r) {
      MaxIdx best{-INFINITY, 0x7fffffff};
#pragma unroll
      for (int j = 0; j < 8; ++j) best = better(best, MaxIdx{cv[j], ci[j]});
      best = warp_best(best);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (ci[j] == best.i) cv[j] = -INFINITY;
      const float wv = (best.i >= 0 && best.i < E) ? S.sc[best.i] : 0.f;
      wsum += wv;
      if (lane == r) { mine_w = wv; mine_i = best.i; }
    }
    if (lane < k) {
      float wv = mine_w;
      if (renorm) wv = wv / (wsum + (mode == 1 ? 1e-20f : 0.f));
      S.out_i[lane] = mine_i;
      S.out_w[lane] = wv * scale;
    }
  }
  __syncthreads();
}

}  // namespace mary
