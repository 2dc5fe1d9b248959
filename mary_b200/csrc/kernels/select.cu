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
#include "router_block.cuh"

using namespace mary;

namespace {

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


// The same router with one CTA (8 warps) per token (router_block.cuh): same results, same tie rule.
__global__ void __launch_bounds__(256)
router_topk_block_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ bias, int T, int E, int k, int mode,
                         int n_group, int topk_group, float scale, int renorm, int* __restrict__ out_idx, float* __restrict__ out_w,
                         int* __restrict__ counts, int* __restrict__ flag) {
  pdl_sync();
  __shared__ RouterSmem S;
  const int t = blockIdx.x;
  router_block(logits + (int64_t)t * ld, bias, E, k, mode, n_group, topk_group, scale, renorm, S, flag);
  if ((int)threadIdx.x < k) {
    out_idx[(int64_t)t * k + threadIdx.x] = S.out_i[threadIdx.x];
    out_w[(int64_t)t * k + threadIdx.x] = S.out_w[threadIdx.x];
    if (counts) atomicAdd(&counts[S.out_i[threadIdx.x]], 1);
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
