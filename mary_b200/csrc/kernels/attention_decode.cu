// Split-KV paged attention for decode-sized query groups (a few rows per kv head), bandwidth-oriented.
//
// The general SIMT kernel (attention_simt.cu) gives every lane its own key and walks the head dimension with dependent
// loads; with one or two query rows per kv head that leaves far too few bytes in flight to approach HBM bandwidth.  Here a
// warp reads WHOLE cache rows: the 32 lanes of a warp cover the D elements of one key (coalesced 4/8/16-byte loads), four
// keys are fetched together (K and V rows: eight independent loads per lane before any use), the R dot products of a key
// are completed with warp shuffles, and every lane keeps the output slice of its own D/32 dims, so P never has to be
// exchanged.  Grid (q block, kv head, kv split), 4 warps per CTA taking keys round-robin in groups of four; partials
// (m, l, o) of warps and splits are merged exactly like in the general kernel (same scratch layout, same combine).
// Reference kernels: attn_partial / attn_combine of the reference's Moshi temporal decoder
// (src/models/personaplex/temporal_metal.rs:133-454) and its windowed SIMT kernel (src/models/inkling/banded.rs:109-299).
#include "common.cuh"
#include "host_utils.h"
#include <type_traits>

using namespace mary;

namespace {

constexpr int WARPS = 4;
constexpr int MAXR = 16;     // scratch stride, shared with attention_simt.cu
constexpr int KG_BYTES = 4096;   // K + V bytes a warp requests before it uses any of them (4 keys at D = 256, 8 at 128 and below)

struct DecParams {
  const __nv_bfloat16* q; const __nv_bfloat16* kc; const __nv_bfloat16* vc; __nv_bfloat16* out;
  const int* page_table; const int* kv_len; const int* q_start; const int* blk_seq; const int* blk_q0;
  float* part_o; float* part_ml;
  int max_pages, page_size;
  int64_t k_tok, k_page, v_tok, v_page;
  int Hq, Hkv, G, RQ, nsplit, window;
  float scale, softcap;
  // 8-bit cache: kc / vc hold one unsigned code per element and the strides count codes; k_sz / v_sz hold (scale, zero) of every
  // (slot, kv head) as two floats, slot-major; element = code * scale + zero
  const float* k_sz; const float* v_sz;
};

template <int E> struct Vec;                       // E bf16 elements per lane
template <> struct Vec<2> { using T = uint32_t; };
template <> struct Vec<4> { using T = uint2; };
template <> struct Vec<8> { using T = uint4; };

template <int E>
__device__ __forceinline__ void unpack(const typename Vec<E>::T& v, float* f) {
  const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int j = 0; j < E / 2; ++j) { float2 t = __bfloat1622float2(h[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
}

template <int E> struct QVec;                      // E 8-bit codes per lane
template <> struct QVec<2> { using T = uint16_t; };
template <> struct QVec<4> { using T = uint32_t; };
template <> struct QVec<8> { using T = uint2; };

template <int E>
__device__ __forceinline__ void unpack_q8(const typename QVec<E>::T& v, float sc, float zero, float* f) {
  const uint8_t* b = (const uint8_t*)&v;
#pragma unroll
  for (int j = 0; j < E; ++j) f[j] = fmaf((float)b[j], sc, zero);
}

// Sums V values (a power of two, at most 32) over the 32 lanes and leaves ALL V totals in every lane.  Instead of one
// five-step butterfly per value (5 V shuffles) the values are halved between the lanes at every step (a lane keeps the half its
// lane bit selects and adds what its partner sends), which costs V - 1 shuffles, and the V totals are then broadcast (V more).
template <int V>
__device__ __forceinline__ void warp_sum_vec(float* v, int lane) {
#pragma unroll
  for (int o = 16; o >= V; o >>= 1) {
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
  }
#pragma unroll
  for (int o = V / 2; o >= 1; o >>= 1) {
    const int n = 2 * o;                                  // values still held before this step
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < o; ++i) {
      const float send = up ? v[i] : v[i + o];
      const float keep = up ? v[i + o] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
    (void)n;
  }
  const float t = v[0];                                   // the total of value (lane % V)
#pragma unroll
  for (int i = 0; i < V; ++i) v[i] = __shfl_sync(0xffffffffu, t, (lane & ~(V - 1)) | i);
}

template <int D, int RMAX, bool Q8>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_kernel(const DecParams p) {
  pdl_sync();
  constexpr int E = D / 32;
  constexpr int KG = KG_BYTES / (4 * D) > 8 ? 8 : KG_BYTES / (4 * D);
  using V = typename Vec<E>::T;
  using KV = typename std::conditional<Q8, typename QVec<E>::T, V>::type;
  __shared__ float red_o[WARPS][RMAX][D];
  __shared__ float red_ml[WARPS][RMAX][2];
  const int nb = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = p.blk_seq[nb], row0 = p.blk_q0[nb];
  const int q_end = p.q_start[seq + 1];
  const int nq = min(p.RQ, q_end - row0);
  const int R = nq * p.G;
  const int kvlen = p.kv_len[seq];
  const int qlen = q_end - p.q_start[seq];
  const int pos0 = kvlen - qlen + (row0 - p.q_start[seq]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  float qf[RMAX][E];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    if (r < R) {
      const int tq = row0 + r / p.G, h = kvh * p.G + r % p.G;
      const V v = *(const V*)(p.q + ((int64_t)tq * p.Hq + h) * D + lane * E);
      unpack<E>(v, qf[r]);
#pragma unroll
      for (int e = 0; e < E; ++e) qf[r][e] *= p.scale;
    }
  }
  int k_lo = 0, k_hi = pos0 + nq;
  if (p.window > 0) k_lo = max(0, pos0 - p.window + 1);
  const int span = k_hi - k_lo;
  const int per = ((span + p.nsplit - 1) / p.nsplit + KG * WARPS - 1) / (KG * WARPS) * (KG * WARPS);
  const int s_lo = k_lo + split * per, s_hi = min(k_hi, s_lo + per);

  float m[RMAX], l[RMAX], o[RMAX][E];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) o[r][e] = 0.f;
  }
  const int* pt = p.page_table + (int64_t)seq * p.max_pages;

  for (int kb = s_lo + warp * KG; kb < s_hi; kb += WARPS * KG) {
    KV kv[KG], vv[KG];
    float2 ksz[KG], vsz[KG];
#pragma unroll
    for (int j = 0; j < KG; ++j) {
      const int kp = min(kb + j, s_hi - 1);          // clamped: masked below
      const int page = pt[kp / p.page_size];
      const int64_t tok = kp % p.page_size;
      if constexpr (Q8) {
        const uint8_t* kq = (const uint8_t*)p.kc;
        const uint8_t* vq = (const uint8_t*)p.vc;
        kv[j] = *(const KV*)(kq + (int64_t)page * p.k_page + tok * p.k_tok + (int64_t)kvh * D + lane * E);
        vv[j] = *(const KV*)(vq + (int64_t)page * p.v_page + tok * p.v_tok + (int64_t)kvh * D + lane * E);
        const int64_t slot = ((int64_t)page * p.page_size + tok) * p.Hkv + kvh;
        ksz[j] = *(const float2*)(p.k_sz + slot * 2);
        vsz[j] = *(const float2*)(p.v_sz + slot * 2);
      } else {
        kv[j] = *(const KV*)(p.kc + (int64_t)page * p.k_page + tok * p.k_tok + (int64_t)kvh * D + lane * E);
        vv[j] = *(const KV*)(p.vc + (int64_t)page * p.v_page + tok * p.v_tok + (int64_t)kvh * D + lane * E);
      }
    }
    float s[KG][RMAX];
#pragma unroll
    for (int j = 0; j < KG; ++j) {
      float kf[E];
      if constexpr (Q8) unpack_q8<E>(kv[j], ksz[j].x, ksz[j].y, kf);
      else unpack<E>(kv[j], kf);
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        float a = 0.f;
        if (r < R) {
#pragma unroll
          for (int e = 0; e < E; ++e) a += qf[r][e] * kf[e];
        }
        s[j][r] = a;
      }
    }
    // finish the dot products over the 32 lanes: all KG * RMAX totals end up in every lane
    {
      constexpr int NV = KG * RMAX;
      float* flat = &s[0][0];
      if constexpr (NV <= 32) {
        warp_sum_vec<NV>(flat, lane);
      } else {
#pragma unroll
        for (int h = 0; h < NV / 32; ++h) warp_sum_vec<32>(flat + 32 * h, lane);
      }
    }
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      if (r < R) {
        const int qp = pos0 + r / p.G;
        float sv[KG];
        float mx = m[r];
#pragma unroll
        for (int j = 0; j < KG; ++j) {
          const int kp = kb + j;
          float x = s[j][r];
          if (p.softcap > 0.f) x = p.softcap * tanhf(x / p.softcap);
          const bool ok = kp < s_hi && kp <= qp && (p.window <= 0 || qp - kp < p.window);
          sv[j] = ok ? x : -INFINITY;
          mx = fmaxf(mx, sv[j]);
        }
        if (mx != -INFINITY) {
          const float corr = __expf(m[r] - mx);
          m[r] = mx;
          l[r] *= corr;
#pragma unroll
          for (int e = 0; e < E; ++e) o[r][e] *= corr;
#pragma unroll
          for (int j = 0; j < KG; ++j) {
            const float pj = (sv[j] == -INFINITY) ? 0.f : __expf(sv[j] - mx);
            l[r] += pj;
            float vf[E];
            if constexpr (Q8) unpack_q8<E>(vv[j], vsz[j].x, vsz[j].y, vf);
            else unpack<E>(vv[j], vf);
#pragma unroll
            for (int e = 0; e < E; ++e) o[r][e] += pj * vf[e];
          }
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    if (r < R) {
      if (lane == 0) { red_ml[warp][r][0] = m[r]; red_ml[warp][r][1] = l[r]; }
#pragma unroll
      for (int e = 0; e < E; ++e) red_o[warp][r][lane * E + e] = o[r][e];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, red_ml[w][r][0]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = red_ml[w][r][0];
      const float c = (mw == -INFINITY) ? 0.f : __expf(mw - mm);
      ll += red_ml[w][r][1] * c;
      acc += red_o[w][r][d] * c;
    }
    if (p.nsplit == 1) {
      const int tq = row0 + r / p.G, h = kvh * p.G + r % p.G;
      p.out[((int64_t)tq * p.Hq + h) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    } else {
      const int64_t pi = (((int64_t)nb * p.Hkv + kvh) * p.nsplit + split) * MAXR + r;
      p.part_o[pi * D + d] = acc;
      if (d == 0) { p.part_ml[pi * 2] = mm; p.part_ml[pi * 2 + 1] = ll; }
    }
  }
}

__global__ void attn_decode_combine_kernel(const DecParams p, int D) {
  pdl_sync();
  const int nb = blockIdx.x, kvh = blockIdx.y;
  const int seq = p.blk_seq[nb], row0 = p.blk_q0[nb];
  const int nq = min(p.RQ, p.q_start[seq + 1] - row0);
  const int R = nq * p.G;
  for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    const int64_t base = (((int64_t)nb * p.Hkv + kvh) * p.nsplit) * MAXR + r;
    float mm = -INFINITY;
    for (int s = 0; s < p.nsplit; ++s) mm = fmaxf(mm, p.part_ml[(base + (int64_t)s * MAXR) * 2]);
    float ll = 0.f, acc = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const int64_t pi = base + (int64_t)s * MAXR;
      const float ms = p.part_ml[pi * 2];
      const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
      ll += p.part_ml[pi * 2 + 1] * c;
      acc += p.part_o[pi * D + d] * c;
    }
    const int tq = row0 + r / p.G, h = kvh * p.G + r % p.G;
    p.out[((int64_t)tq * p.Hq + h) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  }
}

template <int D, int RMAX>
int launch(const DecParams& p, int NB, cudaStream_t s) {
  if (p.k_sz) {
    MARY_LAUNCH((attn_decode_kernel<D, RMAX, true>), dim3(NB, p.Hkv, p.nsplit), WARPS * 32, 0, s, p);
  } else {
    MARY_LAUNCH((attn_decode_kernel<D, RMAX, false>), dim3(NB, p.Hkv, p.nsplit), WARPS * 32, 0, s, p);
  }
  MARY_CHECK_LAUNCH();
  if (p.nsplit > 1) {
    MARY_LAUNCH(attn_decode_combine_kernel, dim3(NB, p.Hkv), 256, 0, s, p, D);
    MARY_CHECK_LAUNCH();
  }
  return MARY_OK;
}

}  // namespace

// Same contract as mary_paged_attention with DK == DV == D in {64, 128, 256} and RQ * (Hq / Hkv) <= 8 (<= 4 for D = 256).
// Scratch (nsplit > 1): mary_paged_attention_scratch_floats(NB, Hkv, nsplit, D).
static int decode_run(const void* q, const void* kc, const void* vc, const float* k_sz, const float* v_sz, void* out, const int* page_table,
                      const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                      int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok, int64_t v_page,
                      int Hq, int Hkv, int D, int RQ, int nsplit, int window, float scale, float softcap,
                      float* scratch, cudaStream_t s) {
  if (NB <= 0) return MARY_OK;
  DecParams p;
  p.k_sz = k_sz; p.v_sz = v_sz;
  p.q = (const __nv_bfloat16*)q; p.kc = (const __nv_bfloat16*)kc; p.vc = (const __nv_bfloat16*)vc; p.out = (__nv_bfloat16*)out;
  p.page_table = page_table; p.kv_len = kv_len; p.q_start = q_start; p.blk_seq = blk_seq; p.blk_q0 = blk_q0;
  p.max_pages = max_pages; p.page_size = page_size; p.k_tok = k_tok; p.k_page = k_page; p.v_tok = v_tok; p.v_page = v_page;
  p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.RQ = RQ; p.nsplit = nsplit < 1 ? 1 : nsplit; p.window = window; p.scale = scale;
  p.softcap = softcap;
  if (p.G * Hkv != Hq) return MARY_ERR_BAD_ARG;
  if (p.nsplit > 1 && !scratch) return MARY_ERR_BAD_ARG;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (int64_t)NB * Hkv * p.nsplit * MAXR * D : nullptr;
  const int R = RQ * p.G;
  if (D == 256) { if (R <= 2) return launch<256, 2>(p, NB, s); if (R <= 4) return launch<256, 4>(p, NB, s); return MARY_ERR_BAD_ARG; }
  if (D == 128) { if (R <= 4) return launch<128, 4>(p, NB, s); if (R <= 8) return launch<128, 8>(p, NB, s); return MARY_ERR_BAD_ARG; }
  if (D == 64) { if (R <= 4) return launch<64, 4>(p, NB, s); if (R <= 8) return launch<64, 8>(p, NB, s); return MARY_ERR_BAD_ARG; }
  return MARY_ERR_BAD_ARG;
}

MARY_API int mary_paged_attention_decode(const void* q, const void* kc, const void* vc, void* out, const int* page_table,
                                         const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                                         int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok, int64_t v_page,
                                         int Hq, int Hkv, int D, int RQ, int nsplit, int window, float scale, float softcap,
                                         float* scratch, cudaStream_t s) {
  return decode_run(q, kc, vc, nullptr, nullptr, out, page_table, kv_len, q_start, blk_seq, blk_q0, NB, max_pages, page_size, k_tok, k_page,
                    v_tok, v_page, Hq, Hkv, D, RQ, nsplit, window, scale, softcap, scratch, s);
}

// The same over an 8-bit cache: kc / vc are code pages [pages, page, Hkv, D] of unsigned bytes (strides in bytes), k_sz / v_sz the
// (scale, zero) pairs [pages * page, Hkv, 2] f32 written by mary_kv_quant_append.  The cache rows are dequantised in registers
// (one fused multiply-add per element), so the kernel streams half the bytes of the bf16 cache.
MARY_API int mary_paged_attention_decode_q8(const void* q, const void* kc, const void* vc, const float* k_sz, const float* v_sz, void* out,
                                            const int* page_table, const int* kv_len, const int* q_start, const int* blk_seq,
                                            const int* blk_q0, int NB, int max_pages, int page_size, int64_t k_tok, int64_t k_page,
                                            int64_t v_tok, int64_t v_page, int Hq, int Hkv, int D, int RQ, int nsplit, int window,
                                            float scale, float softcap, float* scratch, cudaStream_t s) {
  if (!k_sz || !v_sz) return MARY_ERR_BAD_ARG;
  return decode_run(q, kc, vc, k_sz, v_sz, out, page_table, kv_len, q_start, blk_seq, blk_q0, NB, max_pages, page_size, k_tok, k_page,
                    v_tok, v_page, Hq, Hkv, D, RQ, nsplit, window, scale, softcap, scratch, s);
}

namespace {

// One warp per (row, kv head): range of the D values, codes = round((x - min) / scale) with scale = range / 255 (1 when the row is
// constant), as the reference quantises its cache groups (src/models/gemma/gpu_quant.rs:28-90).
__global__ void kv_quant_append_kernel(const __nv_bfloat16* __restrict__ rows, int64_t row_stride, const int64_t* __restrict__ slots,
                                       uint8_t* __restrict__ codes, float* __restrict__ sz, int T, int Hkv, int D, int64_t n_slots,
                                       int* status) {
  pdl_sync();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * Hkv) return;
  const int t = w / Hkv, h = w % Hkv;
  const int64_t slot = slots[t];
  if (slot < 0 || slot >= n_slots) { if (lane == 0) atomicExch(status, MARY_ERR_BOUNDS); return; }
  const __nv_bfloat16* src = rows + (int64_t)t * row_stride + (int64_t)h * D;
  float lo = INFINITY, hi = -INFINITY;
  for (int d = lane; d < D; d += 32) { const float x = __bfloat162float(src[d]); lo = fminf(lo, x); hi = fmaxf(hi, x); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o)); }
  const float range = hi - lo;
  const float sc = range > 0.f ? range / 255.f : 1.f;
  uint8_t* dst = codes + (slot * Hkv + h) * D;
  for (int d = lane; d < D; d += 32) {
    const float x = __bfloat162float(src[d]);
    dst[d] = (uint8_t)fminf(fmaxf(floorf(__fdividef(x - lo, sc) + 0.5f), 0.f), 255.f);
  }
  if (lane == 0) { sz[(slot * Hkv + h) * 2] = sc; sz[(slot * Hkv + h) * 2 + 1] = lo; }
}

}  // namespace

// rows [T, Hkv, D] bf16 (row pitch row_stride elements) -> codes [n_slots, Hkv, D] u8 and sz [n_slots, Hkv, 2] f32 at slots[t].
MARY_API int mary_kv_quant_append(const void* rows, int64_t row_stride, const int64_t* slots, void* codes, float* sz, int T, int Hkv, int D,
                                  int64_t n_slots, cudaStream_t s) {
  if (T <= 0) return MARY_OK;
  const int warps = T * Hkv, per = 8;
  MARY_LAUNCH(kv_quant_append_kernel, (warps + per - 1) / per, per * 32, 0, s, (const __nv_bfloat16*)rows, row_stride, slots, (uint8_t*)codes,
              sz, T, Hkv, D, n_slots, mary_status_ptr());
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
