// Decode attention for grouped-query models on tcgen05 tensor cores, over the paged K / V caches.
//
// The SIMT decode kernels (attention_decode.cu, attention_simt.cu) spend their instruction issue on the dot products: with G query
// heads per kv head and a few speculative rows they need ~100 warp instructions per key and stall far below HBM bandwidth.
// Here the (query token, head of the group) rows of one sequence and ONE kv head are the M = 64 rows of a tensor-core tile
// (unused rows are padding: the tensor pipe has an order of magnitude more throughput than the cache stream needs), so a CTA
// only moves cache pages and does the softmax.  Reference twins: the split-KV partial / combine kernels of the reference's
// speech decoder (src/models/personaplex/temporal_metal.rs:133-454) and its banded SIMT kernel (src/models/inkling/banded.rs).
//
// One CTA = (block of query tokens of one sequence, kv head, kv split).  32 keys (one 32-token page or two 16-token pages) are one
// pipeline stage:
//   warp 0   TMA: Q once — a 3-D box [64 dims, G heads, RQ tokens] per 64-dim chunk lands as dense rows r = token * G + head in the
//            128-byte-swizzled K-major layout; per stage ONE 5-D operation for the K page and one for the V page (the tensor map
//            orders a cache [pages, page, Hkv, D] as dims-in-chunk, tokens, chunks, kv heads, pages, so the box
//            [64, PAGE, D / 64, 1, 1] lands chunk-major: [chunk][token][64 dims]);
//   warp 1   MMA (M = 64): S[64 x 32] = Q K^T (D / 16 instructions per page, three S buffers in TMEM, issued one stage ahead), then
//            O[64 x D] += P V with V^T read from the V page as an MN-major operand and P (bf16) from shared memory;
//   warps 2-5 softmax: row r of an M = 64 accumulator lives in TMEM lane (r % 16) + 32 * (r / 16), so each warp owns 16 rows in
//            its lanes 0-15: scale, optional soft-cap, causal / sliding-window mask, running max with lazy rescale of O, P to
//            shared memory; at the end O / l to global, or f32 partials when the key range is split.
// Every wait is bounded and reports through the status word.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int TR = 64;                        // rows per CTA (MMA M)
constexpr int CHUNK = 64;                     // dims per 128-byte row
constexpr int NSBUF = 3, NPBUF = 2;
constexpr int NTHREADS = 192;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr int AHEAD = 1;                          // blocks by which Q K^T leads P V
constexpr float LOG2E = 1.4426950408889634f;

template <int D, int PAGE>
struct GCfg {
  static constexpr int NCH = D / CHUNK;
  static constexpr int Q_CHUNK_BYTES = TR * 128;                  // 8 KB
  static constexpr int Q_BYTES = NCH * Q_CHUNK_BYTES;
  static constexpr int PAGE_CHUNK_BYTES = PAGE * 128;             // one 64-dim chunk of one page
  static constexpr int PAGE_BYTES = NCH * PAGE_CHUNK_BYTES;       // K (or V) page
  static constexpr int PPB = 32 / PAGE;                           // pages per pipeline stage: a stage always holds KB = 32 keys
  static constexpr int KB = PAGE * PPB;
  static constexpr int STAGE_BYTES = 2 * PAGE_BYTES * PPB;        // [page of the stage][K page | V page]
  static constexpr int STAGES = D == 256 ? 5 : 5;
  static constexpr int P_BYTES = TR * KB * 2;
  static constexpr int SMEM = Q_BYTES + STAGES * STAGE_BYTES + NPBUF * P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = D <= 128 ? 256 : 512;          // S: 3 x PAGE columns at 0..95, O: D columns at 128..
  static_assert(D % CHUNK == 0 && D <= 256 && (PAGE == 16 || PAGE == 32), "head dim 64..256 in chunks of 64, pages of 16 or 32 tokens");
  static_assert(NSBUF * KB <= 128 && SMEM <= 232448, "budget");
};

struct GqaParams {
  const int* page_table; const int* kv_len; const int* q_start; const int* blk_seq; const int* blk_q0;
  __nv_bfloat16* out;      // [T, Hq, D]
  float* part_o;           // [NB, Hkv, nsplit, 64, D] when nsplit > 1
  float* part_ml;          // [NB, Hkv, nsplit, 64, 2]
  int max_pages, Hq, Hkv, G, RQ, nsplit, window;
  float scale, softcap;
  int* status;
};

__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int w, int v) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v)
      : "memory");
}
// K-major, no swizzle: 8-row core matrices of 128 bytes; LBO = distance between the two 16-byte K chunks of one MMA, SBO =
// distance between 8-row groups.
__device__ __forceinline__ uint64_t desc_kmajor_noswz(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
// MN-major, 128-byte swizzle: 64 contiguous N elements per row, 8 K rows per 1024-byte atom; LBO = distance between 64-element
// groups along N, SBO = distance between 8-row groups along K.
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

template <int D, int PAGE>
__global__ void __launch_bounds__(NTHREADS, 1)
gqa_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const GqaParams p) {
  pdl_sync();
  using C = GCfg<D, PAGE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + C::Q_BYTES;
  uint8_t* sP = sKV + C::STAGES * C::STAGE_BYTES;
  uint64_t* bars = (uint64_t*)(sP + NPBUF * C::P_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = q_full + 1;           // [STAGES]
  uint64_t* k_empty = k_full + C::STAGES;  // [STAGES]
  uint64_t* s_full = k_empty + C::STAGES;  // [NSBUF]
  uint64_t* s_empty = s_full + NSBUF;      // [NSBUF]
  uint64_t* p_full = s_empty + NSBUF;      // [NPBUF]
  uint64_t* pv_done = p_full + NPBUF;      // [NPBUF]
  uint32_t* tmem_slot = (uint32_t*)(pv_done + NPBUF);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = p.blk_seq[nb], tok0 = p.blk_q0[nb];                 // first query token (global row) of this block
  const int q_end = p.q_start[seq + 1];
  const int nq = min(p.RQ, q_end - tok0);
  const int nrows = nq * p.G;
  const int kvlen = p.kv_len[seq];
  const int qlen = q_end - p.q_start[seq];
  const int pos0 = kvlen - qlen + (tok0 - p.q_start[seq]);           // position of the block's first query token
  const int k_hi = pos0 + nq;                                         // keys [k_lo, k_hi) are visible to some row
  const int k_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  constexpr int KB = GCfg<D, PAGE>::KB, PPB = GCfg<D, PAGE>::PPB;
  const int blk_first = k_lo / KB;
  const int nblk_total = (k_hi + KB - 1) / KB - blk_first;
  const int n_pages = (k_hi + PAGE - 1) / PAGE;                       // pages of this sequence that hold visible keys
  const int per = (nblk_total + p.nsplit - 1) / p.nsplit;
  const int b_lo = blk_first + split * per, b_hi = min(blk_first + nblk_total, b_lo + per);
  const int nblk = max(0, b_hi - b_lo);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int b = 0; b < NSBUF; ++b) { mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4); }
    for (int b = 0; b < NPBUF; ++b) { mbar_init(&p_full[b], 4); mbar_init(&pv_done[b], 1); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  {
    // rows past the Q box are never written by the copy: give them zeros, so that their (unused) scores stay finite numbers
    const int box_rows = p.G * p.RQ;
    for (int i = threadIdx.x; i < C::NCH * (TR - box_rows) * 8; i += NTHREADS) {
      const int c = i / ((TR - box_rows) * 8), rem = i % ((TR - box_rows) * 8);
      *(uint4*)(sQ + c * C::Q_CHUNK_BYTES + (box_rows + rem / 8) * 128 + (rem % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;            // NSBUF x PAGE columns
  const uint32_t tmem_O = tmem_base + 128;      // D columns

  if (warp == 0) {
    if (nblk > 0 && lane == 0) {
      // the box holds G * RQ rows; rows of tokens past the block's end belong to other sequences (or are zero fill) and stay unused
      mbar_expect_tx(q_full, (uint32_t)(C::NCH * p.G * p.RQ * 128));
      for (int c = 0; c < C::NCH; ++c) tma_load_3d(sQ + c * C::Q_CHUNK_BYTES, &tm_q, q_full, c * CHUNK, kvh * p.G, tok0);
      const int* pt = p.page_table + (int64_t)seq * p.max_pages;
      int stage = 0; uint32_t phase = 0;
      for (int b = b_lo; b < b_hi; ++b) {
        if (!mbar_wait(&k_empty[stage], phase ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
        mbar_expect_tx(&k_full[stage], C::STAGE_BYTES);
        uint8_t* st = sKV + stage * C::STAGE_BYTES;
#pragma unroll
        for (int pp = 0; pp < PPB; ++pp) {
          const int pi = b * PPB + pp;
          const int page = pt[pi < n_pages ? pi : b * PPB];       // a page past the visible keys repeats the block's first page (masked)
          tma_load_5d(st + pp * 2 * C::PAGE_BYTES, &tm_k, &k_full[stage], 0, 0, 0, kvh, page);
          tma_load_5d(st + pp * 2 * C::PAGE_BYTES + C::PAGE_BYTES, &tm_v, &k_full[stage], 0, 0, 0, kvh, page);
        }
        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nblk > 0) {
      const uint32_t idesc_s = idesc_bf16(TR, PAGE);            // one page of keys per instruction
      const uint32_t idesc_o = idesc_bf16(TR, D) | (1u << 16);           // B operand MN-major
      if (!mbar_wait(q_full, 0, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&](int i) -> bool {        // i = block index relative to b_lo
        const int stage = i % C::STAGES, sb = i % NSBUF;
        if (!mbar_wait(&s_empty[sb], ((i / NSBUF) & 1) ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait(&k_full[stage], (i / C::STAGES) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) return false;
        tc_fence_after();
        const uint32_t kb_addr = smem_u32(sKV + stage * C::STAGE_BYTES);
#pragma unroll
        for (int pp = 0; pp < PPB; ++pp) {
#pragma unroll
          for (int c = 0; c < C::NCH; ++c) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              umma_f16(tmem_S + sb * KB + pp * PAGE, umma_desc_sw128(q_addr + c * C::Q_CHUNK_BYTES + k * 32),
                       umma_desc_sw128(kb_addr + pp * 2 * C::PAGE_BYTES + c * C::PAGE_CHUNK_BYTES + k * 32), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
            }
          }
        }
        umma_commit(&s_full[sb]);
        return true;
      };
      // Q K^T runs AHEAD blocks in front of P V.  A stage is held from its load until the P V of its block, so every block of
      // lead takes one stage away from the loads in flight; one block of lead keeps the softmax warps supplied (they need S of
      // block i + 1 only when they are done with block i) and leaves the rest of the ring to hide the load latency.
#pragma unroll
      for (int a = 0; a < AHEAD; ++a)
        if (a < nblk && !issue_qk(a)) goto done;
      for (int i = 0; i < nblk; ++i) {
        if (i + AHEAD < nblk && !issue_qk(i + AHEAD)) goto done;
        const int pb = i & 1;
        if (!mbar_wait(&p_full[pb], (i >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
        tc_fence_after();
        const int stage = i % C::STAGES;
        const uint32_t st_addr = smem_u32(sKV + stage * C::STAGE_BYTES);
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
          // A = P[:, 16 keys] (K-major, no swizzle: 16-byte key chunks TR*16 bytes apart, 8-row groups 128 bytes apart),
          // B = V^T of those keys from their V page (MN-major, 128B swizzle: 64-dim groups one chunk apart, 8-key groups 1 KB apart)
          const int pp = kk * 16 / PAGE, in_page = kk * 16 % PAGE;
          umma_f16(tmem_O, desc_kmajor_noswz(p_addr + pb * C::P_BYTES + kk * 2 * (TR * 16), TR * 16, 128),
                   desc_mnmajor_sw128(st_addr + pp * 2 * C::PAGE_BYTES + C::PAGE_BYTES + in_page * 128, C::PAGE_CHUNK_BYTES, 1024), idesc_o,
                   (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&k_empty[stage]);       // the stage may be overwritten once PV has read it
        umma_commit(&pv_done[pb]);
      }
    }
  } else if (nblk > 0) {
    // ------------------------------------------------------------------ softmax warps: 16 query rows per warp
    const int q4 = warp & 3;
    const int r = q4 * 16 + (lane & 15);            // accumulator row held by this lane (lanes 16-31 hold nothing)
    const bool row_ok = lane < 16 && r < nrows;
    const int qpos = pos0 + r / p.G;
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
    const float sc2 = p.scale * LOG2E;
    float m_ref = -INFINITY, l = 0.f;
    for (int i = 0; i < nblk; ++i) {
      const int sb = i % NSBUF, pb = i & 1;
      if (!mbar_wait(&s_full[sb], (i / NSBUF) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
      tc_fence_after();
      uint32_t sr[KB];
      tmem_ld_32x32b_x32(tmem_S + lane_off + sb * KB, sr);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      const int key0 = (b_lo + i) * KB;
      // A block that every row sees entirely (all but the last of a decode step and the window's edge) takes the short path: no
      // per-element mask, the maximum on the raw scores, one fused multiply-add and one exponential per element.  A row's scores
      // are processed by ONE lane in sequence, so the instruction count of this loop is the kernel's cycle time.
      const bool full_blk = p.softcap <= 0.f && key0 + KB - 1 <= pos0 && (p.window <= 0 || pos0 + nq - 1 - key0 < p.window);
      const float* sf = (const float*)sr;
      float sv[KB];
      float mx;
      if (full_blk) {
        mx = sf[0];
#pragma unroll
        for (int j = 1; j < KB; ++j) mx = fmaxf(mx, sf[j]);
        mx *= sc2;
      } else {
        mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < KB; ++j) {
          const int kp = key0 + j;
          const bool ok = row_ok && kp <= qpos && (p.window <= 0 || qpos - kp < p.window);
          float x = sf[j];
          if (p.softcap > 0.f) x = p.softcap * tanhf(x * p.scale / p.softcap) * LOG2E;
          else x *= sc2;
          sv[j] = ok ? x : -INFINITY;
          mx = fmaxf(mx, sv[j]);
        }
      }
      // lazy rescale: move the reference only when the new maximum exceeds it by more than the threshold (lanes 16-31 hold no
      // score rows and never vote)
      const bool need = lane < 16 && mx > m_ref + RESCALE_THRESHOLD;
      const bool first = (m_ref == -INFINITY);
      float corr = 1.f;
      if (need) { corr = first ? 0.f : exp2f(m_ref - mx); m_ref = mx; }
      uint32_t pw[KB / 2];
      float psum = 0.f;
      if (full_blk) {
        const float nm = -m_ref;
#pragma unroll
        for (int j = 0; j < KB / 2; ++j) {
          const float a = exp2f(fmaf(sf[2 * j], sc2, nm));
          const float b = exp2f(fmaf(sf[2 * j + 1], sc2, nm));
          __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
          pw[j] = *(uint32_t*)&h;
          psum += a + b;
        }
      } else {
#pragma unroll
        for (int j = 0; j < KB / 2; ++j) {
          const float a = (m_ref == -INFINITY) ? 0.f : exp2f(sv[2 * j] - m_ref);
          const float b = (m_ref == -INFINITY) ? 0.f : exp2f(sv[2 * j + 1] - m_ref);
          __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
          pw[j] = *(uint32_t*)&h;
          float2 back = __bfloat1622float2(h);
          psum += back.x + back.y;
        }
      }
      l = l * corr + psum;
      if (__any_sync(0xffffffffu, need && !first) && i > 0) {
        // O may only be touched once the previous P V has completed
        if (!mbar_wait(&pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_O + lane_off + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
#pragma unroll
          for (int j = 0; j < 32; j += 8) tmem_st_32x32b_x8(tmem_O + lane_off + c0 + j, o + j);
        }
        tmem_st_wait();
      }
      if (i >= NPBUF) {
        // this P buffer was last read by the P V of block i - 2
        if (!mbar_wait(&pv_done[pb], ((i - NPBUF) >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
      }
      // P (bf16) -> shared memory: chunk c holds keys 8c..8c+7 of every row, 16 bytes per row
      if (lane < 16) {
#pragma unroll
        for (int c = 0; c < KB / 8; ++c)
          *(uint4*)(sP + pb * C::P_BYTES + c * (TR * 16) + r * 16) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
      }
      fence_proxy_async();       // make the generic-proxy writes of P visible to the tensor core
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[pb]);
    }
    // ------------------------------------------------------------------ write out
    if (!mbar_wait(&pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
    tc_fence_after();
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    const int tq = tok0 + r / p.G, head = kvh * p.G + r % p.G;
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t o[32];
      tmem_ld_32x32b_x32(tmem_O + lane_off + c0, o);
      tmem_ld_wait();
      if (row_ok) {
        if (p.nsplit == 1) {
          __nv_bfloat16* dst = p.out + ((int64_t)tq * p.Hq + head) * D + c0;
          uint4 w[4];
          uint32_t* wp = (uint32_t*)w;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * inv_l, __uint_as_float(o[2 * j + 1]) * inv_l);
            wp[j] = *(uint32_t*)&h;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) ((uint4*)dst)[j] = w[j];
        } else {
          float* dst = p.part_o + ((((int64_t)nb * p.Hkv + kvh) * p.nsplit + split) * TR + r) * D + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) *(float4*)(dst + j) = make_float4(__uint_as_float(o[j]), __uint_as_float(o[j + 1]), __uint_as_float(o[j + 2]), __uint_as_float(o[j + 3]));
        }
      }
    }
    if (row_ok && p.nsplit > 1) {
      float* ml = p.part_ml + ((((int64_t)nb * p.Hkv + kvh) * p.nsplit + split) * TR + r) * 2;
      ml[0] = m_ref; ml[1] = l;
    }
  } else if (warp >= 2 && p.nsplit > 1) {
    // an empty split still has to publish neutral partials
    const int r = (warp & 3) * 16 + (lane & 15);
    if (lane < 16 && r < nrows) {
      float* ml = p.part_ml + ((((int64_t)nb * p.Hkv + kvh) * p.nsplit + split) * TR + r) * 2;
      ml[0] = -INFINITY; ml[1] = 0.f;
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// Merge split partials: exponents are in the log2 domain.
__global__ void gqa_tc_combine_kernel(const GqaParams p, int D) {
  pdl_sync();
  const int nb = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int seq = p.blk_seq[nb], tok0 = p.blk_q0[nb];
  const int nq = min(p.RQ, p.q_start[seq + 1] - tok0);
  if (r >= nq * p.G) return;
  const int64_t base = (((int64_t)nb * p.Hkv + kvh) * p.nsplit) * TR + r;
  float mm = -INFINITY;
  for (int s = 0; s < p.nsplit; ++s) mm = fmaxf(mm, p.part_ml[(base + (int64_t)s * TR) * 2]);
  float ll = 0.f;
  for (int s = 0; s < p.nsplit; ++s) {
    const float* ml = p.part_ml + (base + (int64_t)s * TR) * 2;
    if (ml[0] != -INFINITY) ll += ml[1] * exp2f(ml[0] - mm);
  }
  const int tq = tok0 + r / p.G, head = kvh * p.G + r % p.G;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const int64_t pi = base + (int64_t)s * TR;
      const float ms = p.part_ml[pi * 2];
      if (ms != -INFINITY) acc += p.part_o[pi * D + d] * exp2f(ms - mm);
    }
    p.out[((int64_t)tq * p.Hq + head) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  }
}

typedef CUresult (*PFN_encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int D, int PAGE>
int launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const GqaParams& p, int NB, cudaStream_t s) {
  using C = GCfg<D, PAGE>;
  static MarySmemSlots smem_set = {};
  if (int rc = mary_ensure_dyn_smem((const void*)gqa_decode_tc_kernel<D, PAGE>, C::SMEM, &smem_set)) return rc;
  MARY_LAUNCH((gqa_decode_tc_kernel<D, PAGE>), dim3(NB, p.Hkv, p.nsplit), NTHREADS, C::SMEM, s, tq, tk, tv, p);
  MARY_CHECK_LAUNCH();
  if (p.nsplit > 1) {
    MARY_LAUNCH(gqa_tc_combine_kernel, dim3(NB, p.Hkv, p.RQ * p.G), 128, 0, s, p, D);
    MARY_CHECK_LAUNCH();
  }
  return MARY_OK;
}

}  // namespace

MARY_API int64_t mary_gqa_tc_scratch_floats(int NB, int Hkv, int nsplit, int D) {
  return nsplit > 1 ? (int64_t)NB * Hkv * nsplit * TR * (D + 2) : 0;
}
MARY_API int mary_gqa_tc_supported(int D, int page_size, int G, int RQ) {
  return ((D == 128 || D == 256) && (page_size == 16 || page_size == 32) && G >= 1 && RQ >= 1 && G * RQ <= TR && G <= 256 && RQ <= 256) ? 1 : 0;
}

// q [T, Hq, D] bf16; K / V caches [pages, page_size, Hkv, D] bf16, contiguous; out [T, Hq, D] bf16.  blk_seq / blk_q0: NB blocks of at
// most RQ query tokens of one sequence (q0 is a global token row).  G = Hq / Hkv heads share a kv head; G * RQ <= 64.
MARY_API int mary_gqa_decode_tc(const void* q, const void* kc, const void* vc, void* out, const int* page_table, const int* kv_len,
                                const int* q_start, const int* blk_seq, const int* blk_q0, int NB, int T, int num_pages, int max_pages,
                                int page_size, int Hq, int Hkv, int D, int RQ, int nsplit, int window, float scale, float softcap,
                                float* scratch, cudaStream_t s) {
  if (NB <= 0) return MARY_OK;
  if (Hkv < 1 || Hq % Hkv) return MARY_ERR_BAD_ARG;
  const int G = Hq / Hkv;
  if (!mary_gqa_tc_supported(D, page_size, G, RQ)) return MARY_ERR_BAD_ARG;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 1 && !scratch) return MARY_ERR_BAD_ARG;
  PFN_encode enc = (PFN_encode)mary_encode_fn();
  if (!enc) return MARY_ERR_CUDA;
  CUtensorMap tq, tk, tv;
  {
    // q as [tokens][heads][D]: the box takes one 64-dim chunk of the G heads of a kv head for RQ consecutive tokens
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)Hq, (cuuint64_t)T};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)Hq * D * 2};
    cuuint32_t box[3] = {CHUNK, (cuuint32_t)G, (cuuint32_t)RQ};
    cuuint32_t estr[3] = {1, 1, 1};
    if (((uintptr_t)q & 15) || enc(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return MARY_ERR_CUDA;
  }
  for (int which = 0; which < 2; ++which) {
    // cache as [pages][kv heads][chunks][tokens][64 dims]: the box is one page of one kv head, chunk-major
    const void* base = which ? vc : kc;
    cuuint64_t dims[5] = {CHUNK, (cuuint64_t)page_size, (cuuint64_t)(D / CHUNK), (cuuint64_t)Hkv, (cuuint64_t)num_pages};
    cuuint64_t strides[4] = {(cuuint64_t)Hkv * D * 2, CHUNK * 2, (cuuint64_t)D * 2, (cuuint64_t)page_size * Hkv * D * 2};
    cuuint32_t box[5] = {CHUNK, (cuuint32_t)page_size, (cuuint32_t)(D / CHUNK), 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    if (((uintptr_t)base & 15) || enc(which ? &tv : &tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return MARY_ERR_CUDA;
  }
  GqaParams p;
  p.page_table = page_table; p.kv_len = kv_len; p.q_start = q_start; p.blk_seq = blk_seq; p.blk_q0 = blk_q0;
  p.out = (__nv_bfloat16*)out; p.part_o = scratch;
  p.part_ml = scratch ? scratch + (int64_t)NB * Hkv * nsplit * TR * D : nullptr;
  p.max_pages = max_pages; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.RQ = RQ; p.nsplit = nsplit; p.window = window;
  p.scale = scale; p.softcap = softcap; p.status = mary_status_ptr();
  if (D == 128) return page_size == 16 ? launch<128, 16>(tq, tk, tv, p, NB, s) : launch<128, 32>(tq, tk, tv, p, NB, s);
  return page_size == 16 ? launch<256, 16>(tq, tk, tv, p, NB, s) : launch<256, 32>(tq, tk, tv, p, NB, s);
}
