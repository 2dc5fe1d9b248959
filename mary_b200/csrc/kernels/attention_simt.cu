// Paged attention over the flattened ragged batch, SIMT version with split-KV (flash-decoding) and a combine pass.
//
// Covers every (head_dim, GQA group, window, softcap) combination and is the path for decode steps of GQA
// models, which stream the KV cache once and are bound by HBM bandwidth.  Reference kernels: the windowed
// SIMT kernel src/models/inkling/banded.rs:109-299 (one CTA per (query, head), <= 1024 scores in shared
// memory) and the split-KV partial/combine pair src/models/personaplex/temporal_metal.rs:133-454.
//
// Work unit = (q block, kv head, kv split).  A q block is up to RQ consecutive query rows of one sequence;
// together with the G = Hq/Hkv query heads that share the kv head it forms R = RQ*G score rows.  In the QK
// phase each lane owns one key (16-byte loads along the head dimension, q broadcast from shared memory); in
// the PV phase each lane owns DV/32 output dimensions and the probabilities are broadcast by shuffles.
// Partial results (m, l, o) of each split go to a scratch buffer and are merged by attn_combine_kernel.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int WARPS = 4;
constexpr int MAXR = 16;

struct AttnParams {
  const __nv_bfloat16* q;      // [T, Hq, DK]
  const __nv_bfloat16* kc;     // pages: token stride k_tok, page stride k_page, head offset h * DK
  const __nv_bfloat16* vc;
  __nv_bfloat16* out;          // [T, Hq, DV]
  const int* page_table;       // [S, max_pages]
  const int* kv_len;           // [S]
  const int* q_start;          // [S+1]
  const int* blk_seq;          // [NB] sequence of a q block
  const int* blk_q0;           // [NB] first row (global row index) of a q block
  float* part_o;               // scratch [NB, Hkv, nsplit, R, DV]
  float* part_ml;              // scratch [NB, Hkv, nsplit, R, 2]
  int max_pages, page_size;
  int64_t k_tok, k_page, v_tok, v_page;
  int Hq, Hkv, G, DK, DV, RQ, nsplit, window;
  float scale, softcap;
  // optional additive relative-position bias (the reference's score epilogue, src/models/inkling/scorebias.rs:97-221):
  // rel[(row * Hq + head) * rel_extent + dist] is added to the scaled score of the key `dist` positions back, dist < rel_extent
  const float* rel;
  int rel_extent;
};

template <int VPL, int RMAX>   // V dims per lane = DV / 32; RMAX = most score rows of a q block
__global__ void __launch_bounds__(WARPS * 32)
paged_attn_kernel(const AttnParams p) {
  extern __shared__ float sm[];
  const int nb = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = p.blk_seq[nb], row0 = p.blk_q0[nb];
  const int q_end = p.q_start[seq + 1];
  const int nq = min(p.RQ, q_end - row0);
  const int R = nq * p.G;
  const int kvlen = p.kv_len[seq];
  const int qlen = q_end - p.q_start[seq];
  const int pos0 = kvlen - qlen + (row0 - p.q_start[seq]);      // absolute position of the block's first row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  float* qs = sm;                                   // [MAXR][DK]
  float* red_o = qs + MAXR * p.DK;                  // [WARPS][MAXR][DV]
  float* red_ml = red_o + WARPS * MAXR * p.DV;      // [WARPS][MAXR][2]

  for (int i = threadIdx.x; i < R * p.DK; i += blockDim.x) {
    const int r = i / p.DK, d = i % p.DK;
    const int tq = row0 + r / p.G, h = kvh * p.G + r % p.G;
    qs[r * p.DK + d] = __bfloat162float(p.q[((int64_t)tq * p.Hq + h) * p.DK + d]) * p.scale;
  }
  __syncthreads();

  // key range needed by this block, then this split's share of it (in units of 32 keys per warp step)
  int k_lo = 0, k_hi = pos0 + nq;                   // exclusive; causal: last row sees keys <= pos0+nq-1
  if (p.window > 0) k_lo = max(0, pos0 - p.window + 1);
  const int span = k_hi - k_lo;
  const int per = ((span + p.nsplit - 1) / p.nsplit + 31) & ~31;
  const int s_lo = k_lo + split * per, s_hi = min(k_hi, s_lo + per);

  float m[RMAX], l[RMAX], o[RMAX][VPL];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) o[r][v] = 0.f;
  }
  const int* pt = p.page_table + (int64_t)seq * p.max_pages;

  for (int kb = s_lo + warp * 32; kb < s_hi; kb += WARPS * 32) {
    const int kp = kb + lane;
    const bool valid = kp < s_hi;
    float s[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) s[r] = 0.f;
    if (valid) {
      const int page = pt[kp / p.page_size];
      const __nv_bfloat16* kr = p.kc + (int64_t)page * p.k_page + (int64_t)(kp % p.page_size) * p.k_tok + (int64_t)kvh * p.DK;
      for (int d = 0; d < p.DK; d += 8) {
        const uint4 kk = *(const uint4*)(kr + d);
        const __nv_bfloat162* k2 = (const __nv_bfloat162*)&kk;
        float kf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(k2[j]); kf[2 * j] = f.x; kf[2 * j + 1] = f.y; }
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
          if (r < R) {
            const float* qr = qs + r * p.DK + d;
#pragma unroll
            for (int j = 0; j < 8; ++j) s[r] += qr[j] * kf[j];
          }
        }
      }
    }
    // mask + online softmax, row by row
    float pr[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      pr[r] = 0.f;
      if (r < R) {
        const int qp = pos0 + r / p.G;
        float sv = s[r];
        if (p.rel) {
          const int dist = qp - kp;
          if (valid && dist >= 0 && dist < p.rel_extent)
            sv += p.rel[((int64_t)(row0 + r / p.G) * p.Hq + kvh * p.G + r % p.G) * p.rel_extent + dist];
        }
        if (p.softcap > 0.f) sv = p.softcap * tanhf(sv / p.softcap);
        const bool ok = valid && kp <= qp && (p.window <= 0 || qp - kp < p.window);
        sv = ok ? sv : -INFINITY;
        const float mx = fmaxf(m[r], warp_max(sv));
        if (mx == -INFINITY) continue;              // nothing visible yet for this row
        const float corr = __expf(m[r] - mx);
        const float e = ok ? __expf(sv - mx) : 0.f;
        l[r] = l[r] * corr + warp_sum(e);
        m[r] = mx;
        pr[r] = e;
#pragma unroll
        for (int v = 0; v < VPL; ++v) o[r][v] *= corr;
      }
    }
    // PV: every lane walks the 32 keys of this step and accumulates its own output dims
    const int nk = min(32, s_hi - kb);
    for (int j = 0; j < nk; ++j) {
      const int kj = kb + j;
      const int page = pt[kj / p.page_size];
      const __nv_bfloat16* vr = p.vc + (int64_t)page * p.v_page + (int64_t)(kj % p.page_size) * p.v_tok + (int64_t)kvh * p.DV;
      float vf[VPL];
#pragma unroll
      for (int v = 0; v < VPL; ++v) vf[v] = __bfloat162float(vr[lane + 32 * v]);
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < R) {
          const float pj = __shfl_sync(0xffffffffu, pr[r], j);
#pragma unroll
          for (int v = 0; v < VPL; ++v) o[r][v] += pj * vf[v];
        }
      }
    }
  }

  // merge the warps of the CTA
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    if (r < R) {
      if (lane == 0) { red_ml[(warp * MAXR + r) * 2] = m[r]; red_ml[(warp * MAXR + r) * 2 + 1] = l[r]; }
#pragma unroll
      for (int v = 0; v < VPL; ++v) red_o[((int64_t)warp * MAXR + r) * p.DV + lane + 32 * v] = o[r][v];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R * p.DV; i += blockDim.x) {
    const int r = i / p.DV, d = i % p.DV;
    float mm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, red_ml[(w * MAXR + r) * 2]);
    float ll = 0.f, acc = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      const float mw = red_ml[(w * MAXR + r) * 2];
      const float c = (mw == -INFINITY) ? 0.f : __expf(mw - mm);
      ll += red_ml[(w * MAXR + r) * 2 + 1] * c;
      acc += red_o[((int64_t)w * MAXR + r) * p.DV + d] * c;
    }
    if (p.nsplit == 1) {
      const int tq = row0 + r / p.G, h = kvh * p.G + r % p.G;
      p.out[((int64_t)tq * p.Hq + h) * p.DV + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    } else {
      const int64_t pi = (((int64_t)nb * p.Hkv + kvh) * p.nsplit + split) * MAXR + r;
      p.part_o[pi * p.DV + d] = acc;
      if (d == 0) { p.part_ml[pi * 2] = mm; p.part_ml[pi * 2 + 1] = ll; }
    }
  }
}

__global__ void attn_combine_kernel(const AttnParams p) {
  const int nb = blockIdx.x, kvh = blockIdx.y;
  const int seq = p.blk_seq[nb], row0 = p.blk_q0[nb];
  const int nq = min(p.RQ, p.q_start[seq + 1] - row0);
  const int R = nq * p.G;
  for (int i = threadIdx.x; i < R * p.DV; i += blockDim.x) {
    const int r = i / p.DV, d = i % p.DV;
    const int64_t base = (((int64_t)nb * p.Hkv + kvh) * p.nsplit) * MAXR + r;
    float mm = -INFINITY;
    for (int s = 0; s < p.nsplit; ++s) mm = fmaxf(mm, p.part_ml[(base + (int64_t)s * MAXR) * 2]);
    float ll = 0.f, acc = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const int64_t pi = base + (int64_t)s * MAXR;
      const float ms = p.part_ml[pi * 2];
      const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
      ll += p.part_ml[pi * 2 + 1] * c;
      acc += p.part_o[pi * p.DV + d] * c;
    }
    const int tq = row0 + r / p.G, h = kvh * p.G + r % p.G;
    p.out[((int64_t)tq * p.Hq + h) * p.DV + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  }
}

template <int VPL, int RMAX>
int launch(const AttnParams& p, int NB, cudaStream_t s) {
  if (p.RQ * p.G > RMAX) return MARY_ERR_BAD_ARG;
  size_t sm = ((size_t)MAXR * p.DK + (size_t)WARPS * MAXR * p.DV + WARPS * MAXR * 2) * sizeof(float);
  // the limit is a per-device property of the kernel: raised the first time this device sees a shape that needs more
  static MarySmemSlots smem_set = {};
  if (int rc = mary_ensure_dyn_smem((const void*)paged_attn_kernel<VPL, RMAX>, sm, &smem_set)) return rc;
  dim3 grid(NB, p.Hkv, p.nsplit);
  paged_attn_kernel<VPL, RMAX><<<grid, WARPS * 32, sm, s>>>(p);
  MARY_CHECK_LAUNCH();
  if (p.nsplit > 1) {
    attn_combine_kernel<<<dim3(NB, p.Hkv), 256, 0, s>>>(p);
    MARY_CHECK_LAUNCH();
  }
  return MARY_OK;
}

}  // namespace

// Scratch needed for `nsplit` > 1, in floats: NB * Hkv * nsplit * 16 * (DV + 2).
MARY_API int64_t mary_paged_attention_scratch_floats(int NB, int Hkv, int nsplit, int DV) {
  return nsplit > 1 ? (int64_t)NB * Hkv * nsplit * MAXR * (DV + 2) : 0;
}

MARY_API int mary_paged_attention_max_rows(int DV) { return DV <= 128 ? 16 : (DV <= 256 ? 8 : 4); }

// q [T, Hq, DK] bf16, caches addressed by (page, token-in-page, kv head) with element strides, out [T, Hq, DV].
// blk_seq / blk_q0 describe NB q blocks of at most RQ rows each; RQ * (Hq/Hkv) must not exceed
// mary_paged_attention_max_rows(DV) (the register budget of the DV specialisation).
static int paged_attention_impl(const void* q, const void* kc, const void* vc, void* out, const int* page_table,
                                const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                                int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok, int64_t v_page,
                                int Hq, int Hkv, int DK, int DV, int RQ, int nsplit, int window, float scale, float softcap,
                                float* scratch, const float* rel, int rel_extent, cudaStream_t s);

MARY_API int mary_paged_attention(const void* q, const void* kc, const void* vc, void* out, const int* page_table,
                                  const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                                  int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok, int64_t v_page,
                                  int Hq, int Hkv, int DK, int DV, int RQ, int nsplit, int window, float scale, float softcap,
                                  float* scratch, cudaStream_t s) {
  return paged_attention_impl(q, kc, vc, out, page_table, kv_len, q_start, blk_seq, blk_q0, NB, max_pages, page_size, k_tok, k_page, v_tok,
                              v_page, Hq, Hkv, DK, DV, RQ, nsplit, window, scale, softcap, scratch, nullptr, 0, s);
}

// The same with an additive relative-position bias rel[T, Hq, rel_extent] (f32).
MARY_API int mary_paged_attention_rel(const void* q, const void* kc, const void* vc, void* out, const int* page_table,
                                      const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                                      int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok, int64_t v_page,
                                      int Hq, int Hkv, int DK, int DV, int RQ, int nsplit, int window, float scale, float softcap,
                                      float* scratch, const float* rel, int rel_extent, cudaStream_t s) {
  if (rel && rel_extent <= 0) return MARY_ERR_BAD_ARG;
  return paged_attention_impl(q, kc, vc, out, page_table, kv_len, q_start, blk_seq, blk_q0, NB, max_pages, page_size, k_tok, k_page, v_tok,
                              v_page, Hq, Hkv, DK, DV, RQ, nsplit, window, scale, softcap, scratch, rel, rel_extent, s);
}

static int paged_attention_impl(const void* q, const void* kc, const void* vc, void* out, const int* page_table,
                                const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                                int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok, int64_t v_page,
                                int Hq, int Hkv, int DK, int DV, int RQ, int nsplit, int window, float scale, float softcap,
                                float* scratch, const float* rel, int rel_extent, cudaStream_t s) {
  if (NB <= 0) return MARY_OK;
  AttnParams p;
  p.rel = rel; p.rel_extent = rel_extent;
  p.q = (const __nv_bfloat16*)q; p.kc = (const __nv_bfloat16*)kc; p.vc = (const __nv_bfloat16*)vc; p.out = (__nv_bfloat16*)out;
  p.page_table = page_table; p.kv_len = kv_len; p.q_start = q_start; p.blk_seq = blk_seq; p.blk_q0 = blk_q0;
  p.max_pages = max_pages; p.page_size = page_size; p.k_tok = k_tok; p.k_page = k_page; p.v_tok = v_tok; p.v_page = v_page;
  p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.DK = DK; p.DV = DV; p.RQ = RQ; p.nsplit = nsplit < 1 ? 1 : nsplit;
  p.window = window; p.scale = scale; p.softcap = softcap;
  if (p.G * Hkv != Hq || RQ * p.G > MAXR || (DK & 7) || (DV & 31)) return MARY_ERR_BAD_ARG;
  if (p.nsplit > 1 && !scratch) return MARY_ERR_BAD_ARG;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (int64_t)NB * Hkv * p.nsplit * MAXR * DV : nullptr;
  switch (DV / 32) {
    case 1: return launch<1, 16>(p, NB, s);
    case 2: return launch<2, 16>(p, NB, s);
    case 4: return launch<4, 16>(p, NB, s);
    case 8: return launch<8, 8>(p, NB, s);
    case 16: return launch<16, 4>(p, NB, s);
    default: return MARY_ERR_BAD_ARG;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant (see no_alloc.h for who needs it and what it costs).
#include "no_alloc.h"

namespace {

// Partial results of the split-KV pass for callers that cannot hand us a buffer.  It is part of the library's device
// image: each GPU that loads the library carries these 16 MiB until the process ends.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MARY_NOALLOC_SCRATCH_BYTES];

// Device address of the array per device ordinal, looked up on the first call made with that device current.  The
// array's NAME is only a host-side handle here; handing it to a kernel would pass a host address.
float* g_noalloc_ptr[64] = {nullptr};

int noalloc_setup(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MARY_ERR_CUDA;
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return MARY_ERR_CUDA;
    g_noalloc_ptr[dev] = (float*)p;
  }
  *out = g_noalloc_ptr[dev];
  return MARY_OK;
}

}  // namespace

MARY_API int64_t mary_noalloc_scratch_bytes(void) { return (int64_t)MARY_NOALLOC_SCRATCH_BYTES; }

MARY_API const char* mary_status_string(int code) {
  switch (code) {
    case MARY_OK: return "ok";
    case MARY_ERR_TIMEOUT_TMA: return "a TMA pipeline wait timed out";
    case MARY_ERR_TIMEOUT_MMA: return "an accumulator wait timed out";
    case MARY_ERR_TIMEOUT_PEER: return "a wait on another GPU's flag timed out";
    case MARY_ERR_BAD_ARG: return "bad argument";
    case MARY_ERR_CUDA: return "CUDA runtime error";
    case MARY_ERR_BOUNDS: return "bounds check failed";
    case MARY_ERR_SCRATCH_TOO_LARGE:
      return "the split-KV partial results exceed the library's built-in 16 MiB scratch array: use fewer splits or fewer "
             "query blocks per call, or call mary_paged_attention with a buffer of your own";
    default: return "unknown status";
  }
}

// Same contract as mary_paged_attention, minus the scratch argument.  The first call on a device performs the one-time
// set-up described in no_alloc.h and should be made outside stream capture.
MARY_API int mary_paged_attention_noalloc(const void* q, const void* kc, const void* vc, void* out, const int* page_table,
                                          const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                                          int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok,
                                          int64_t v_page, int Hq, int Hkv, int DK, int DV, int RQ, int nsplit, int window,
                                          float scale, float softcap, cudaStream_t stream) {
  if (nsplit < 1) nsplit = 1;
  const int64_t need = mary_paged_attention_scratch_floats(NB, Hkv, nsplit, DV) * (int64_t)sizeof(float);
  if (need > (int64_t)MARY_NOALLOC_SCRATCH_BYTES) return MARY_ERR_SCRATCH_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = noalloc_setup(&scratch);
  if (rc != MARY_OK) return rc;
  return mary_paged_attention(q, kc, vc, out, page_table, kv_len, q_start, blk_seq, blk_q0, NB, max_pages, page_size, k_tok, k_page,
                              v_tok, v_page, Hq, Hkv, DK, DV, RQ, nsplit, window, scale, softcap, scratch, stream);
}
