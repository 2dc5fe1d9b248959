// Selection kernels: vocabulary arg-max / sampler and the MoE routers.
//
// Reference behaviour: host arg-max over a full logits readback, first maximum wins
// (src/models/gemma/gemma4/lm.rs:22-32); device Gumbel-max over top-k in the TTS predictor
// (src/models/qwen3tts/predictor_gpu.rs, gumbel_argmax_kernel); sigmoid+bias top-k router with one thread doing
// k arg-max passes (src/models/inkling/routetopk.rs:112-260); softmax top-k router on the host
// (src/models/gemma/gemma4/layers.rs:269-325); group-limited selection is refused by the reference
// (src/models/k3/router.rs:136-143) and implemented here.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

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

// Philox-4x32-10 counter RNG (one call -> 4 uniforms).
__device__ __forceinline__ uint4 philox(uint2 key, uint4 ctr) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x, hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0; key.y += W1;
  }
  return ctr;
}

// One CTA per row.  mode 0: arg-max of the logits.  mode 1: Gumbel-max sampling at `temperature` restricted to
// logits >= (row max - margin) — an exact sample from the tempered softmax truncated at that margin.
// Soft-capping is monotonic, so it is applied to the reported maximum only.
__global__ void argmax_kernel(const float* __restrict__ logits, int64_t ld, int V, float softcap, int mode, float temperature,
                              float margin, uint64_t seed, uint64_t step, int64_t* __restrict__ out_idx, float* __restrict__ out_val) {
  pdl_sync();
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (int64_t)blockIdx.x * ld;
  MaxIdx best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) best = better(best, MaxIdx{row[i], i});
  best = warp_best(best);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best.v; si[w] = best.i; }
  __syncthreads();
  MaxIdx b = (l < (blockDim.x >> 5)) ? MaxIdx{sv[l], si[l]} : MaxIdx{-INFINITY, 0x7fffffff};
  b = warp_best(b);
  __syncthreads();
  if (mode == 1 && temperature > 0.f) {
    const float rmax = b.v;
    MaxIdx g{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float x = row[i];
      if (softcap > 0.f) x = softcap * tanhf(x / softcap);
      const float cm = softcap > 0.f ? softcap * tanhf(rmax / softcap) : rmax;
      if (x < cm - margin) continue;
      uint4 r = philox(make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)), make_uint4((uint32_t)i, blockIdx.x, (uint32_t)step, (uint32_t)(step >> 32)));
      const float u = ((float)r.x + 0.5f) * (1.0f / 4294967296.0f);
      g = better(g, MaxIdx{x / temperature - __logf(-__logf(u)), i});
    }
    g = warp_best(g);
    if (l == 0) { sv[w] = g.v; si[w] = g.i; }
    __syncthreads();
    b = (l < (blockDim.x >> 5)) ? MaxIdx{sv[l], si[l]} : MaxIdx{-INFINITY, 0x7fffffff};
    b = warp_best(b);
    b.v = row[b.i];
  }
  if (threadIdx.x == 0) {
    out_idx[blockIdx.x] = b.i;
    if (out_val) out_val[blockIdx.x] = softcap > 0.f ? softcap * tanhf(b.v / softcap) : b.v;
  }
}

// One warp per token.  mode 0: softmax over all experts, top-k, optional renormalisation.
// mode 1: scores = sigmoid(logit); selection on scores + bias, optionally limited to the `topk_group` best of
// `n_group` groups (group score = sum of its two best biased scores); weights = unbiased scores of the chosen,
// renormalised by (sum + 1e-20), times `scale`.  Ties resolve to the lower index.  A non-finite logit sets *flag.
constexpr int MAXE_PER_LANE = 16;   // up to 512 experts
__global__ void router_topk_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ bias, int T, int E, int k,
                                   int mode, int n_group, int topk_group, float scale, int renorm, int* __restrict__ out_idx,
                                   float* __restrict__ out_w, int* __restrict__ counts, int* __restrict__ flag) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  const float* row = logits + (int64_t)t * ld;
  float sc[MAXE_PER_LANE], sel[MAXE_PER_LANE];
  const int per = (E + 31) / 32;
  float mx = -INFINITY;
  bool bad = false;
#pragma unroll
  for (int j = 0; j < MAXE_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    sc[j] = -INFINITY;
    if (j < per && e < E) { sc[j] = row[e]; bad |= !isfinite(sc[j]); mx = fmaxf(mx, sc[j]); }
  }
  if (__any_sync(0xffffffffu, bad) && lane == 0 && flag) atomicExch(flag, 1);
  if (mode == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAXE_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (j < per && e < E) { sc[j] = __expf(sc[j] - mx); sum += sc[j]; } else sc[j] = -INFINITY;
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int j = 0; j < MAXE_PER_LANE; ++j) { if (sc[j] != -INFINITY) sc[j] /= sum; sel[j] = sc[j]; }
  } else {
#pragma unroll
    for (int j = 0; j < MAXE_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (j < per && e < E) { sc[j] = 1.0f / (1.0f + __expf(-sc[j])); sel[j] = sc[j] + (bias ? bias[e] : 0.f); }
      else { sc[j] = 0.f; sel[j] = -INFINITY; }
    }
    if (n_group > 1) {
      const int gsz = E / n_group;
      // group score = sum of the two best biased scores in the group; keep the best topk_group groups
      uint32_t keep = 0;
      float gscore_mine = -INFINITY;      // lane g (< n_group) ends up holding the score of group g
      for (int g = 0; g < n_group; ++g) {
        MaxIdx b1{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int j = 0; j < MAXE_PER_LANE; ++j) { const int e = lane + 32 * j; if (j < per && e < E && e / gsz == g) b1 = better(b1, MaxIdx{sel[j], e}); }
        b1 = warp_best(b1);
        MaxIdx b2{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int j = 0; j < MAXE_PER_LANE; ++j) { const int e = lane + 32 * j; if (j < per && e < E && e / gsz == g && e != b1.i) b2 = better(b2, MaxIdx{sel[j], e}); }
        b2 = warp_best(b2);
        if (lane == g) gscore_mine = b1.v + b2.v;
      }
      for (int r = 0; r < topk_group; ++r) {
        MaxIdx b = warp_best(MaxIdx{(lane < n_group && !((keep >> lane) & 1u)) ? gscore_mine : -INFINITY, lane});
        keep |= 1u << b.i;
      }
#pragma unroll
      for (int j = 0; j < MAXE_PER_LANE; ++j) { const int e = lane + 32 * j; if (j < per && e < E && !((keep >> (e / gsz)) & 1u)) sel[j] = -INFINITY; }
    }
  }
  float wsum = 0.f, mine_w = 0.f;
  int mine_i = 0;
  for (int r = 0; r < k; ++r) {
    MaxIdx b{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int j = 0; j < MAXE_PER_LANE; ++j) { const int e = lane + 32 * j; if (j < per && e < E) b = better(b, MaxIdx{sel[j], e}); }
    b = warp_best(b);
    // the owning lane reads the unbiased score and retires the expert
    float wv = 0.f;
#pragma unroll
    for (int j = 0; j < MAXE_PER_LANE; ++j) { if (lane + 32 * j == b.i) { wv = sc[j]; sel[j] = -INFINITY; } }
    wv = __shfl_sync(0xffffffffu, wv, b.i & 31);
    wsum += wv;
    if (lane == r) { mine_w = wv; mine_i = b.i; }
  }
  if (lane < k) {
    float wv = mine_w;
    if (renorm) wv = wv / (wsum + (mode == 1 ? 1e-20f : 0.f));
    out_idx[(int64_t)t * k + lane] = mine_i;
    out_w[(int64_t)t * k + lane] = wv * scale;
    if (counts) atomicAdd(&counts[mine_i], 1);
  }
}


// The same router with one CTA (8 warps) per token: decode batches hold tens to hundreds of tokens, and a single warp
// walking ~400 experts through group scoring and k arg-max rounds is a serial chain of thousands of dependent instructions
// (tens of microseconds).  Here every thread owns at most two experts; the groups are scored by different warps at once; every
// warp extracts the k best of its own 1/8 of the experts and warp 0 merges the 8 k candidates.  Same results, same tie rule.
__global__ void __launch_bounds__(256)
router_topk_block_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ bias, int T, int E, int k, int mode,
                         int n_group, int topk_group, float scale, int renorm, int* __restrict__ out_idx, float* __restrict__ out_w,
                         int* __restrict__ counts, int* __restrict__ flag) {
  pdl_sync();
  __shared__ float s_sc[512], s_sel[512], s_g[32], s_red[8];
  __shared__ float s_cv[256];
  __shared__ int s_ci[256];
  __shared__ uint32_t s_keep;
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* row = logits + (int64_t)t * ld;
  float v0 = -INFINITY, v1 = -INFINITY;
  bool bad = false;
  if (tid < E) { v0 = row[tid]; bad |= !isfinite(v0); }
  if (tid + 256 < E) { v1 = row[tid + 256]; bad |= !isfinite(v1); }
  if (bad && flag) atomicExch(flag, 1);
  if (mode == 0) {
    float mx = warp_max(fmaxf(v0, v1));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, s_red[w]);
    __syncthreads();
    const float e0 = tid < E ? __expf(v0 - mx) : 0.f, e1 = tid + 256 < E ? __expf(v1 - mx) : 0.f;
    float sum = warp_sum(e0 + e1);
    if (lane == 0) s_red[warp] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += s_red[w];
    if (tid < E) { s_sc[tid] = e0 / sum; s_sel[tid] = e0 / sum; }
    if (tid + 256 < E) { s_sc[tid + 256] = e1 / sum; s_sel[tid + 256] = e1 / sum; }
  } else {
    if (tid < E) { const float sg = 1.0f / (1.0f + __expf(-v0)); s_sc[tid] = sg; s_sel[tid] = sg + (bias ? bias[tid] : 0.f); }
    if (tid + 256 < E) { const float sg = 1.0f / (1.0f + __expf(-v1)); s_sc[tid + 256] = sg; s_sel[tid + 256] = sg + (bias ? bias[tid + 256] : 0.f); }
  }
  __syncthreads();
  if (mode == 1 && n_group > 1) {
    const int gsz = E / n_group;
    for (int g = warp; g < n_group; g += 8) {               // group score = sum of the two best biased scores in the group
      MaxIdx b1{-INFINITY, 0x7fffffff};
      for (int m = lane; m < gsz; m += 32) b1 = better(b1, MaxIdx{s_sel[g * gsz + m], g * gsz + m});
      b1 = warp_best(b1);
      MaxIdx b2{-INFINITY, 0x7fffffff};
      for (int m = lane; m < gsz; m += 32) { const int e = g * gsz + m; if (e != b1.i) b2 = better(b2, MaxIdx{s_sel[e], e}); }
      b2 = warp_best(b2);
      if (lane == 0) s_g[g] = b1.v + b2.v;
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t keep = 0;
      const float mine = lane < n_group ? s_g[lane] : -INFINITY;
      for (int r = 0; r < topk_group; ++r) {
        MaxIdx b = warp_best(MaxIdx{(lane < n_group && !((keep >> lane) & 1u)) ? mine : -INFINITY, lane});
        keep |= 1u << b.i;
      }
      if (lane == 0) s_keep = keep;
    }
    __syncthreads();
    const uint32_t keep = s_keep;
    if (tid < E && !((keep >> (tid / gsz)) & 1u)) s_sel[tid] = -INFINITY;
    if (tid + 256 < E && !((keep >> ((tid + 256) / gsz)) & 1u)) s_sel[tid + 256] = -INFINITY;
    __syncthreads();
  }
  // every warp: the k best of its own slice of the experts
  {
    const int chunk = (E + 7) / 8;                            // <= 64: two experts per lane
    const int base = warp * chunk;
    const int ea = base + lane, eb = base + lane + 32;
    float a = (lane < chunk && ea < E) ? s_sel[ea] : -INFINITY;
    float b = (lane + 32 < chunk && eb < E) ? s_sel[eb] : -INFINITY;
    for (int r = 0; r < k; ++r) {
      MaxIdx best = warp_best(better(MaxIdx{a, ea}, MaxIdx{b, eb}));
      if (best.i == ea) a = -INFINITY;
      if (best.i == eb) b = -INFINITY;
      if (lane == 0) { s_cv[warp * k + r] = best.v; s_ci[warp * k + r] = best.i; }
    }
  }
  __syncthreads();
  if (warp == 0) {
    // merge 8 k candidates (each warp's list is in descending order, which the merge does not need)
    const int n = 8 * k;
    float cv[8];
    int ci[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { const int c = lane + 32 * j; cv[j] = c < n ? s_cv[c] : -INFINITY; ci[j] = c < n ? s_ci[c] : 0x7fffffff; }
    float wsum = 0.f, mine_w = 0.f;
    int mine_i = 0;
    for (int r = 0; r < k; ++r) {
      MaxIdx best{-INFINITY, 0x7fffffff};
#pragma unroll
      for (int j = 0; j < 8; ++j) best = better(best, MaxIdx{cv[j], ci[j]});
      best = warp_best(best);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (ci[j] == best.i) cv[j] = -INFINITY;
      const float wv = (best.i >= 0 && best.i < E) ? s_sc[best.i] : 0.f;
      wsum += wv;
      if (lane == r) { mine_w = wv; mine_i = best.i; }
    }
    if (lane < k) {
      float wv = mine_w;
      if (renorm) wv = wv / (wsum + (mode == 1 ? 1e-20f : 0.f));
      out_idx[(int64_t)t * k + lane] = mine_i;
      out_w[(int64_t)t * k + lane] = wv * scale;
      if (counts) atomicAdd(&counts[mine_i], 1);
    }
  }
}

}  // namespace

MARY_API int mary_argmax(const float* logits, int64_t ld, int rows, int V, float softcap, int mode, float temperature, float margin,
                         uint64_t seed, uint64_t step, int64_t* out_idx, float* out_val, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  MARY_LAUNCH(argmax_kernel, rows, 1024, 0, s, logits, ld, V, softcap, mode, temperature, margin, seed, step, out_idx, out_val);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_router_topk(const float* logits, int64_t ld, const float* bias, int T, int E, int k, int mode, int n_group,
                              int topk_group, float scale, int renorm, int* out_idx, float* out_w, int* counts, int* flag,
                              cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  if (E > 32 * MAXE_PER_LANE || k > 32 || n_group > 32 || (n_group > 1 && E % n_group)) return MARY_ERR_BAD_ARG;
  if (T <= 16384 && k * 8 <= 256) {
    // one CTA per token: short dependent chains (decode and ordinary prefill chunks)
    MARY_LAUNCH(router_topk_block_kernel, T, 256, 0, s, logits, ld, bias, T, E, k, mode, n_group, topk_group, scale, renorm, out_idx, out_w,
                                               counts, flag);
    MARY_CHECK_LAUNCH();
    return MARY_OK;
  }
  const int wpb = 4;
  router_topk_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, s>>>(logits, ld, bias, T, E, k, mode, n_group, topk_group, scale, renorm,
                                                            out_idx, out_w, counts, flag);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
