// Temperature / top-k / top-p (nucleus) sampling of one token per logit row, entirely on the device.
//
// Reference behaviour (src/models/personaplex/sampling.rs:81-140, on the host over a read-back row): non-finite logits count as
// -inf; candidates in descending order, equal logits in index order; keep the k highest (0 = all); softmax of logit / T over the
// survivors; keep the smallest prefix whose mass reaches top_p (>= 1 = all, at least one); multinomial draw.  The speech models
// sample 17 rows per frame, so a read-back and a host sort per row bound the frame rate.
//
// One CTA per row, no sort.  The k-th largest logit is found by a 4-pass radix select over a monotonic 32-bit key of the float,
// the nucleus boundary by the same select over probability MASS instead of counts.  Masses are 2^40 fixed point in 64-bit
// integers: integer addition is associative, so the histogram atomics give the same thresholds (and the same token for a given
// seed) on every run.  Ties at a threshold keep the lowest indices, as a stable sort would.  The draw walks the row in index
// order over the kept set (any fixed order gives the right distribution) with two block scans per tile of 4 * NT logits.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int NT = 512;
constexpr int NW = NT / 32;
constexpr int PER = 4;                       // consecutive logits per thread in the draw walk
constexpr double FIX = 1099511627776.0;      // 2^40

__device__ __forceinline__ float sane(float x) {   // NaN and +-inf -> -inf (by the exponent bits: fast-math leaves those alone)
  return (__float_as_uint(x) & 0x7f800000u) == 0x7f800000u ? -INFINITY : x;
}
__device__ __forceinline__ uint32_t fkey(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }
__device__ __forceinline__ float ldf(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ unsigned long long mass_of(float x, float m, float inv_t) {
  if (x == -INFINITY) return 0ull;
  return (unsigned long long)((double)exp2f((x - m) * inv_t * 1.4426950408889634f) * FIX);
}

__device__ __forceinline__ uint64_t splitmix(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// One histogram update per DISTINCT bin of the warp: logits crowd into a few exponent bins, and 32 same-address atomics per warp
// and element would serialise the pass.
__device__ __forceinline__ void warp_hist_add(bool active, int bin, uint32_t cnt, unsigned long long mass, uint32_t* h_cnt,
                                              unsigned long long* h_mass) {
  uint32_t todo = __ballot_sync(0xffffffffu, active);
  const int lane = threadIdx.x & 31;
  while (todo) {
    const int leader = __ffs(todo) - 1;
    const int b = __shfl_sync(0xffffffffu, bin, leader);
    const bool mine = active && bin == b;
    uint32_t c = mine ? cnt : 0u;
    unsigned long long ms = mine ? mass : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      c += __shfl_xor_sync(0xffffffffu, c, o);
      ms += __shfl_xor_sync(0xffffffffu, ms, o);
    }
    if (lane == leader) {
      if (c) atomicAdd(&h_cnt[b], c);
      if (ms) atomicAdd(&h_mass[b], ms);
    }
    todo &= ~__ballot_sync(0xffffffffu, mine);
  }
}

template <typename V>
__device__ __forceinline__ V block_excl_scan(V v, V* total, V* sm /* NW + 1 */) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  V inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const V t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) sm[w] = inc;
  __syncthreads();
  if (w == 0) {
    V x = lane < NW ? sm[lane] : V(0);
    V xi = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const V t = __shfl_up_sync(0xffffffffu, xi, o);
      if (lane >= o) xi += t;
    }
    if (lane < NW) sm[lane] = xi - x;
    if (lane == NW - 1) sm[NW] = xi;
  }
  __syncthreads();
  const V res = inc - v + sm[w];
  *total = sm[NW];
  __syncthreads();
  return res;
}

template <typename T>
__global__ void __launch_bounds__(NT) sample_kernel(const T* __restrict__ logits, int64_t ld, int V, float inv_t, int top_k, float top_p,
                                                    uint64_t seed, uint64_t step, int* __restrict__ out_idx, float* __restrict__ out_prob) {
  pdl_sync();
  __shared__ uint32_t h_cnt[256];
  __shared__ unsigned long long h_mass[256];
  __shared__ float red_v[NW];
  __shared__ int red_i[NW];
  __shared__ unsigned long long scan64[NW + 1];
  __shared__ uint32_t scan32[NW + 1];
  __shared__ unsigned long long s_acc;
  __shared__ uint32_t s_bin, s_rem;
  __shared__ int s_found;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const T* row = logits + (int64_t)blockIdx.x * ld;

  // ---- row maximum (first index wins)
  float mv = -INFINITY;
  int mi = 0x7fffffff;
  for (int i = tid; i < V; i += NT) {
    const float x = sane(ldf(row, i));
    if (x > mv || (x == mv && i < mi)) { mv = x; mi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, mv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
    if (ov > mv || (ov == mv && oi < mi)) { mv = ov; mi = oi; }
  }
  if (lane == 0) { red_v[w] = mv; red_i[w] = mi; }
  if (tid == 0) s_found = 0;
  __syncthreads();
  mv = red_v[0]; mi = red_i[0];
  for (int k = 1; k < NW; ++k)
    if (red_v[k] > mv || (red_v[k] == mv && red_i[k] < mi)) { mv = red_v[k]; mi = red_i[k]; }
  if (mv == -INFINITY) {                       // nothing finite in the row: nothing to sample from
    if (tid == 0) { out_idx[blockIdx.x] = mi == 0x7fffffff ? 0 : mi; if (out_prob) out_prob[blockIdx.x] = 0.f; }
    return;
  }
  const float m = mv;

  // ---- top-k: the k-th largest key, and how many of its equals are kept
  uint32_t thr = 0u, ties_keep = 0xffffffffu;
  if (top_k > 0 && top_k < V) {
    uint32_t prefix = 0u, mask = 0u, remaining = (uint32_t)top_k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) { h_cnt[tid] = 0u; h_mass[tid] = 0ull; }
      __syncthreads();
      for (int i0 = 0; i0 < V; i0 += NT) {
        const int i = i0 + tid;
        const uint32_t k = i < V ? fkey(sane(ldf(row, i))) : 0u;
        warp_hist_add(i < V && (k & mask) == prefix, (k >> shift) & 255, 1u, 0ull, h_cnt, h_mass);
      }
      __syncthreads();
      if (tid == 0) {
        uint32_t acc = 0u;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + h_cnt[b] >= remaining) break;
          acc += h_cnt[b];
        }
        s_bin = (uint32_t)b; s_rem = remaining - acc;
      }
      __syncthreads();
      prefix |= s_bin << shift; mask |= 0xffu << shift; remaining = s_rem;
      __syncthreads();
    }
    thr = prefix; ties_keep = remaining;
  }

  // ---- mass above the threshold and the number of equals at it
  if (tid == 0) { s_acc = 0ull; s_rem = 0u; }
  __syncthreads();
  {
    unsigned long long ms = 0ull;
    uint32_t ce = 0u;
    for (int i = tid; i < V; i += NT) {
      const float x = sane(ldf(row, i));
      const uint32_t k = fkey(x);
      if (k > thr) ms += mass_of(x, m, inv_t);
      else if (k == thr) ++ce;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { ms += __shfl_xor_sync(0xffffffffu, ms, o); ce += __shfl_xor_sync(0xffffffffu, ce, o); }
    if (lane == 0) { if (ms) atomicAdd(&s_acc, ms); if (ce) atomicAdd(&s_rem, ce); }
  }
  __syncthreads();
  unsigned long long mass_gt = s_acc;
  uint32_t n_eq = min(ties_keep, s_rem);                     // equals at the threshold that survive
  unsigned long long e_thr = mass_of(key_float(thr), m, inv_t);
  unsigned long long S = mass_gt + (unsigned long long)n_eq * e_thr;
  __syncthreads();

  // ---- top-p: the key at which the descending cumulative mass reaches p * S
  if (top_p < 1.f) {
    unsigned long long P = (unsigned long long)((double)top_p * (double)S);
    if (P < 1ull) P = 1ull;
    uint32_t prefix = 0u, mask = 0u;
    unsigned long long above = 0ull;
    uint32_t cnt_at = 0u;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) { h_cnt[tid] = 0u; h_mass[tid] = 0ull; }
      __syncthreads();
      for (int i0 = 0; i0 < V; i0 += NT) {
        const int i = i0 + tid;
        const float x = i < V ? sane(ldf(row, i)) : -INFINITY;
        const uint32_t k = fkey(x);
        warp_hist_add(i < V && k > thr && (k & mask) == prefix, (k >> shift) & 255, 1u, mass_of(x, m, inv_t), h_cnt, h_mass);
      }
      if (tid == 0 && n_eq && (thr & mask) == prefix) {      // the surviving equals of the top-k threshold, added once
        atomicAdd(&h_cnt[(thr >> shift) & 255], n_eq);
        atomicAdd(&h_mass[(thr >> shift) & 255], (unsigned long long)n_eq * e_thr);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long acc = above;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + h_mass[b] >= P) break;
          acc += h_mass[b];
        }
        s_bin = (uint32_t)b; s_acc = acc; s_rem = h_cnt[b];
      }
      __syncthreads();
      prefix |= s_bin << shift; mask |= 0xffu << shift; above = s_acc; cnt_at = s_rem;
      __syncthreads();
    }
    const unsigned long long e_t = mass_of(key_float(prefix), m, inv_t);
    unsigned long long need = P > above ? P - above : 1ull;
    unsigned long long keep = e_t ? (need + e_t - 1ull) / e_t : 1ull;
    if (keep < 1ull) keep = 1ull;
    if (keep > cnt_at) keep = cnt_at;
    if (keep < 1ull) keep = 1ull;
    thr = prefix; ties_keep = (uint32_t)keep; e_thr = e_t; mass_gt = above;
    S = above + keep * e_t;
  }
  if (S == 0ull) {                                            // every kept mass underflowed: the maximum is the only candidate
    if (tid == 0) { out_idx[blockIdx.x] = mi; if (out_prob) out_prob[blockIdx.x] = 1.f; }
    return;
  }

  // ---- the draw: walk the row in index order over the kept set
  const uint64_t r = splitmix(seed ^ splitmix(step ^ splitmix((uint64_t)blockIdx.x)));
  const double u = (double)(r >> 11) * (1.0 / 9007199254740992.0);
  unsigned long long target = (unsigned long long)(u * (double)S);
  if (target >= S) target = S - 1ull;
  unsigned long long run_mass = 0ull;
  uint32_t run_eq = 0u;
  for (int base = 0; base < V; base += NT * PER) {
    float x[PER];
    uint32_t k[PER];
    uint32_t ce = 0u;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = base + tid * PER + j;
      x[j] = i < V ? sane(ldf(row, i)) : -INFINITY;
      k[j] = i < V ? fkey(x[j]) : 0u;
      if (i < V && k[j] == thr) ++ce;
    }
    uint32_t tot_eq;
    uint32_t rank = run_eq + block_excl_scan<uint32_t>(ce, &tot_eq, scan32);
    unsigned long long mj[PER], mine = 0ull;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = base + tid * PER + j;
      bool kept = i < V && k[j] > thr;
      if (i < V && k[j] == thr) { kept = rank < ties_keep; ++rank; }
      mj[j] = kept ? mass_of(x[j], m, inv_t) : 0ull;
      mine += mj[j];
    }
    unsigned long long tot_mass;
    const unsigned long long before = run_mass + block_excl_scan<unsigned long long>(mine, &tot_mass, scan64);
    if (mine && target >= before && target < before + mine) {
      unsigned long long acc = before;
      int pick = -1;
      unsigned long long pm = 0ull;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        if (pick < 0 && mj[j] && target < acc + mj[j]) { pick = base + tid * PER + j; pm = mj[j]; }
        acc += mj[j];
      }
      out_idx[blockIdx.x] = pick;
      if (out_prob) out_prob[blockIdx.x] = (float)((double)pm / (double)S);
      s_found = 1;
    }
    __syncthreads();
    if (s_found) return;
    run_mass += tot_mass; run_eq += tot_eq;
  }
  if (tid == 0) { out_idx[blockIdx.x] = mi; if (out_prob) out_prob[blockIdx.x] = 0.f; }    // unreachable unless the row changed under us
}

}  // namespace

// logits [rows, V] f32 (is_f32 = 1) or bf16, row pitch ld elements; one token id per row into out_idx; out_prob (optional): the
// probability of the drawn token within the kept set.  temperature > 0.  top_k <= 0 or >= V keeps all; top_p >= 1 keeps all.
// The uniform of row r is a function of (seed, step, r) only.
MARY_API int mary_sample_top_k_top_p(const void* logits, int is_f32, int64_t ld, int rows, int V, float temperature, int top_k, float top_p,
                                     uint64_t seed, uint64_t step, int* out_idx, float* out_prob, cudaStream_t s) {
  if (rows <= 0) return MARY_OK;
  if (V <= 0 || !(temperature > 0.f) || !(top_p > 0.f)) return MARY_ERR_BAD_ARG;
  const float inv_t = 1.f / temperature;
  if (is_f32) {
    MARY_LAUNCH(sample_kernel<float>, rows, NT, 0, s, (const float*)logits, ld, V, inv_t, top_k, top_p, seed, step, out_idx, out_prob);
  } else {
    MARY_LAUNCH(sample_kernel<__nv_bfloat16>, rows, NT, 0, s, (const __nv_bfloat16*)logits, ld, V, inv_t, top_k, top_p, seed, step, out_idx,
                out_prob);
  }
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
