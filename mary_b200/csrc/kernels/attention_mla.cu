// Multi-head latent attention over a paged latent cache, on tcgen05 tensor cores.
//
// Every query head attends in latent space (W_UK and W_UV absorbed into the query and the output): keys are the
// cached rows [c_kv (512) | k_rope (64)], values are their first 512 dims, so all heads of a token — and all
// speculative tokens of a sequence — share ONE stream of 1152-byte cache rows.  The reference keeps an expanded
// K/V cache and plain matmuls (src/models/k3/mla.rs:281-293); the latent cache and this kernel are new.
//
// One CTA = (tile of 64 query rows of one sequence, kv split).  A query row is a
// (token, head) pair; rows of one sequence are contiguous in q[T * Hq, 576].  The head dimension (576) makes shared
// memory the binding resource: 64 query rows (72 KB) leave room for FOUR 32-key stages of the cache (4 x 36 KB), deep
// enough that the tensor pipe always has a queued Q K^T while the softmax of an earlier block runs.
//   warp 0   TMA: the Q tile once (9 chunks of [64 x 64]); a 32-key stage is laid out [9 chunks][32 keys][64 dims] with the
//            128-byte swizzle.  With 32-token pages that is ONE 4-D TMA operation per stage (the tensor map orders the cache
//            as dims-in-chunk, tokens, chunks, pages, so the box [64, 32, 9, 1] lands chunk-major): 36 KB per operation.
//            With 16-token pages it takes 18 operations of 2 KB (one per page and chunk, issued by different lanes), and
//            the TMA unit's per-operation cost, not HBM, then bounds the stream;
//   warp 1   MMA (M = 64): S[64 x 32] = Q K^T (9 chunks x 4 MMAs of 64x32x16; three S buffers in TMEM, issued two
//            blocks ahead), then O[64 x 256] += P V with V^T taken from the SAME shared-memory stage as an MN-major
//            B operand (P double buffered in shared memory).  An M = 64 accumulator occupies only lanes 0-15 of each
//            32-lane TMEM group, so the two 256-wide halves of O share the same 256 columns: dims 0-255 in lanes 0-15,
//            dims 256-511 in lanes 16-31;
//   warps 2-5 softmax: TMEM holds row r of an M = 64 accumulator in lane (r % 16) + 32 * (r / 16), so each warp owns 16
//            rows in its lanes 0-15: tcgen05.ld of S, causal mask, running max with lazy rescale of O (only when the
//            max grows by more than 2^8), P written to shared memory as bf16 in the un-swizzled K-major core-matrix
//            layout, final O / l to global (or f32 partials when the kv range is split).
// All waits are bounded.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int DK = 576, DV = 512, DVH = 256;
constexpr int PAGE = 16, KB = 32;                 // keys per stage
constexpr int TR = 64;                            // query rows per CTA (MMA M)
constexpr int CHUNK = 64;                         // dims per 128-byte row
constexpr int NCHUNK = DK / CHUNK;                // 9
constexpr int Q_CHUNK_BYTES = TR * 128;           // 8 KB
constexpr int Q_BYTES = NCHUNK * Q_CHUNK_BYTES;   // 72 KB
constexpr int K_CHUNK_BYTES = KB * 128;           // 4 KB: 32 keys of one 64-dim chunk
constexpr int STAGE_BYTES = NCHUNK * K_CHUNK_BYTES;   // 36 KB
constexpr int STAGES = 4;
constexpr int NSBUF = 3;                          // S accumulators in TMEM
constexpr int NPBUF = 2;                          // P tiles in shared memory
constexpr int P_BYTES = TR * KB * 2;              // 4 KB
constexpr int SMEM = Q_BYTES + STAGES * STAGE_BYTES + NPBUF * P_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;                    // S 3 x 32 at columns 0..95, O 256 at columns 128..383
constexpr int NTHREADS = 192;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr int AHEAD = 1;                          // blocks by which Q K^T leads P V

struct MlaParams {
  const int* page_table; const int* kv_len; const int* q_start; const int* blk_seq; const int* blk_row0;
  __nv_bfloat16* out;      // [T * Hq, 512]
  float* part_o;           // [NB, nsplit, 64, 512] when nsplit > 1
  float* part_ml;          // [NB, nsplit, 64, 2]
  int max_pages, Hq, nsplit, page;
  float scale_log2;        // softmax scale * log2(e)
  int* status;
};

// K-major, no swizzle: 8-row core matrices of 128 bytes; LBO = distance between the two 16-byte K chunks of one
// MMA, SBO = distance between 8-row groups.
__device__ __forceinline__ uint64_t desc_kmajor_noswz(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
// MN-major, 128-byte swizzle: 64 contiguous M/N elements per row, 8 K rows per 1024-byte atom; LBO = distance
// between 64-element groups along M/N, SBO = distance between 8-row groups along K.
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

__global__ void __launch_bounds__(NTHREADS, 1)
mla_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv, const MlaParams p) {
  pdl_sync();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Q_BYTES;
  uint8_t* sP = sK + STAGES * STAGE_BYTES;
  uint64_t* bars = (uint64_t*)(sP + NPBUF * P_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = q_full + 1;           // [STAGES]
  uint64_t* k_empty = k_full + STAGES;     // [STAGES]
  uint64_t* s_full = k_empty + STAGES;     // [NSBUF]
  uint64_t* s_empty = s_full + NSBUF;      // [NSBUF]
  uint64_t* p_full = s_empty + NSBUF;      // [NPBUF]
  uint64_t* pv_done = p_full + NPBUF;      // [NPBUF]
  uint32_t* tmem_slot = (uint32_t*)(pv_done + NPBUF);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = blockIdx.x, split = blockIdx.y;
  const int seq = p.blk_seq[nb], row0 = p.blk_row0[nb];          // row0: global row index (token * Hq + head)
  const int seq_row0 = p.q_start[seq] * p.Hq, seq_row1 = p.q_start[seq + 1] * p.Hq;
  const int nrows = min(TR, seq_row1 - row0);
  const int kvlen = p.kv_len[seq];
  const int qlen = p.q_start[seq + 1] - p.q_start[seq];
  const int pos_first = kvlen - qlen;                             // position of the sequence's first query token
  const int tok_hi = (row0 - seq_row0 + nrows - 1) / p.Hq;
  const int k_hi = pos_first + tok_hi + 1;                        // keys [0, k_hi) are visible to some row of the tile
  const int nblk_total = (k_hi + KB - 1) / KB;
  const int per = (nblk_total + p.nsplit - 1) / p.nsplit;
  const int b_lo = split * per, b_hi = min(nblk_total, b_lo + per);
  const int nblk = max(0, b_hi - b_lo);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int b = 0; b < NSBUF; ++b) { mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4); }
    for (int b = 0; b < NPBUF; ++b) { mbar_init(&p_full[b], 4); mbar_init(&pv_done[b], 1); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_kv);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;            // NSBUF x 32 columns
  const uint32_t tmem_O = tmem_base + 128;      // 256 columns

  if (warp == 0) {
    if (nblk > 0) {
      // every lane of the producer warp issues its own TMA operations; lane 0 owns the barrier bookkeeping
      if (lane == 0) {
        mbar_expect_tx(q_full, Q_BYTES);
        for (int c = 0; c < NCHUNK; ++c) tma_load_2d(sQ + c * Q_CHUNK_BYTES, &tm_q, q_full, c * CHUNK, row0);
      }
      const int* pt = p.page_table + (int64_t)seq * p.max_pages;
      int stage = 0; uint32_t phase = 0;
      for (int b = b_lo; b < b_hi; ++b) {
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(&k_empty[stage], phase ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA) ? 1 : 0;
          if (ok) mbar_expect_tx(&k_full[stage], STAGE_BYTES);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) goto done;
        if (p.page == KB) {
          // one operation brings the whole stage: box [64 dims, 32 tokens, 9 chunks] of one page
          if (lane == 0) {
            const int key0 = b * KB;
            const int page = (key0 < kvlen) ? pt[key0 / KB] : pt[0];
            tma_load_4d(sK + stage * STAGE_BYTES, &tm_kv, &k_full[stage], 0, 0, 0, page);
          }
        } else if (lane < (KB / PAGE) * NCHUNK) {
          // 2 pages x 9 chunks = 18 operations of [16 tokens x 64 dims] (2 KB each)
          const int pg = lane / NCHUNK, c = lane % NCHUNK;
          const int key0 = b * KB + pg * PAGE;
          // pages past the sequence end read the first page (their scores are masked)
          const int page = (key0 < kvlen) ? pt[key0 / PAGE] : pt[0];
          tma_load_3d(sK + stage * STAGE_BYTES + c * K_CHUNK_BYTES + pg * (PAGE * 128), &tm_kv, &k_full[stage], c * CHUNK, 0, page);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nblk > 0) {
      const uint32_t idesc_s = idesc_bf16(TR, KB);
      const uint32_t idesc_o = idesc_bf16(TR, DVH) | (1u << 16);           // B operand MN-major
      if (!mbar_wait(q_full, 0, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&](int i) -> bool {        // i = block index relative to b_lo
        const int stage = i % STAGES, sb = i % NSBUF;
        if (!mbar_wait(&s_empty[sb], ((i / NSBUF) & 1) ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait(&k_full[stage], (i / STAGES) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) return false;
        tc_fence_after();
        const uint32_t kb_addr = smem_u32(sK + stage * STAGE_BYTES);
        for (int c = 0; c < NCHUNK; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_f16(tmem_S + sb * KB, umma_desc_sw128(q_addr + c * Q_CHUNK_BYTES + k * 32),
                     umma_desc_sw128(kb_addr + c * K_CHUNK_BYTES + k * 32), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
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
        const int stage = i % STAGES;
        const uint32_t kb_addr = smem_u32(sK + stage * STAGE_BYTES);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int kk = 0; kk < KB / 16; ++kk) {
            // A = P[:, 16 keys] (K-major, no swizzle: 16-byte key chunks TR*16 bytes apart, 8-row groups 128 bytes apart),
            // B = V^T of those keys from the stage (MN-major, 128B swizzle: 64-dim groups one chunk apart, 8-key groups
            // 1 KB apart); the second half of the value dims accumulates in lanes 16-31 of the same columns
            umma_f16(tmem_O + ((uint32_t)(half * 16) << 16), desc_kmajor_noswz(p_addr + pb * P_BYTES + kk * 2 * (TR * 16), TR * 16, 128),
                     desc_mnmajor_sw128(kb_addr + half * 4 * K_CHUNK_BYTES + kk * 16 * 128, K_CHUNK_BYTES, 1024), idesc_o,
                     (i > 0 || kk > 0) ? 1u : 0u);
          }
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
    const int qpos = pos_first + (row0 - seq_row0 + r) / p.Hq;
    const int qpos_min = pos_first + (row0 - seq_row0) / p.Hq;      // the tile's first row sees the fewest keys
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
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
      // A block that every row of the tile sees entirely (all but the last one or two of a decode step) takes the short path:
      // no per-element mask, the maximum on the raw scores, one fused multiply-add and one exponential per element.  A row's
      // 32 scores are processed by ONE lane in sequence, so the instruction count of this loop is the kernel's cycle time.
      const bool full_blk = key0 + KB - 1 <= qpos_min;
      const float* sf = (const float*)sr;
      float sv[KB];
      float mx;
      if (full_blk) {
        mx = sf[0];
#pragma unroll
        for (int j = 1; j < KB; ++j) mx = fmaxf(mx, sf[j]);
        mx *= p.scale_log2;
      } else {
        mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < KB; ++j) {
          const bool ok = row_ok && (key0 + j) <= qpos;
          sv[j] = ok ? sf[j] * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, sv[j]);
        }
      }
      // lazy rescale: move the reference only when the new maximum exceeds it by more than the threshold (lanes 16-31 hold no
      // score rows and never vote)
      const bool need = lane < 16 && mx > m_ref + RESCALE_THRESHOLD;
      const bool first = (m_ref == -INFINITY);
      float corr = 1.f;
      if (need) { corr = first ? 0.f : exp2f(m_ref - mx); m_ref = mx; }
      // probabilities in registers first: the waits below then overlap this arithmetic of the other warps
      uint32_t pw[KB / 2];
      float psum = 0.f;
      if (full_blk) {
        const float nm = -m_ref;
#pragma unroll
        for (int j = 0; j < KB / 2; ++j) {
          const float a = exp2f(fmaf(sf[2 * j], p.scale_log2, nm));
          const float b = exp2f(fmaf(sf[2 * j + 1], p.scale_log2, nm));
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
      // lanes 16-31 hold the upper value half of row (lane - 16): they rescale with that row's factor
      const float corr_o = __shfl_sync(0xffffffffu, corr, lane & 15);
      if (__any_sync(0xffffffffu, need && !first) && i > 0) {
        // O may only be touched once the previous P V has completed
        if (!mbar_wait(&pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < DVH; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_O + lane_off + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr_o);
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
          *(uint4*)(sP + pb * P_BYTES + c * (TR * 16) + r * 16) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
      }
      fence_proxy_async();       // make the generic-proxy writes of P visible to the tensor core
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[pb]);
    }
    // ------------------------------------------------------------------ write out
    if (!mbar_wait(&pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
    tc_fence_after();
    const float l_row = __shfl_sync(0xffffffffu, l, lane & 15);
    const float inv_l = l_row > 0.f ? 1.f / l_row : 0.f;
    const int half = lane >> 4;                        // lanes 16-31: value dims 256-511 of row (lane - 16)
    const bool out_ok = r < nrows;
#pragma unroll 1
    for (int c0 = 0; c0 < DVH; c0 += 32) {
      uint32_t o[32];
      tmem_ld_32x32b_x32(tmem_O + lane_off + c0, o);
      tmem_ld_wait();
      if (out_ok) {
        if (p.nsplit == 1) {
          __nv_bfloat16* dst = p.out + (int64_t)(row0 + r) * DV + half * DVH + c0;
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
          float* dst = p.part_o + (((int64_t)nb * p.nsplit + split) * TR + r) * DV + half * DVH + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) *(float4*)(dst + j) = make_float4(__uint_as_float(o[j]), __uint_as_float(o[j + 1]), __uint_as_float(o[j + 2]), __uint_as_float(o[j + 3]));
        }
      }
    }
    if (row_ok && p.nsplit > 1) {
      float* ml = p.part_ml + (((int64_t)nb * p.nsplit + split) * TR + r) * 2;
      ml[0] = m_ref; ml[1] = l;
    }
  } else if (warp >= 2 && p.nsplit > 1) {
    // an empty split still has to publish neutral partials
    const int r = (warp & 3) * 16 + (lane & 15);
    if (lane < 16 && r < nrows) {
      float* ml = p.part_ml + (((int64_t)nb * p.nsplit + split) * TR + r) * 2;
      ml[0] = -INFINITY; ml[1] = 0.f;
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// Merge split partials: exponents are in the log2 domain.
__global__ void mla_combine_kernel(const MlaParams p, int NB) {
  pdl_sync();
  const int nb = blockIdx.x, r = blockIdx.y;
  const int seq = p.blk_seq[nb], row0 = p.blk_row0[nb];
  const int nrows = min(TR, p.q_start[seq + 1] * p.Hq - row0);
  if (r >= nrows) return;
  float mm = -INFINITY;
  for (int s = 0; s < p.nsplit; ++s) mm = fmaxf(mm, p.part_ml[(((int64_t)nb * p.nsplit + s) * TR + r) * 2]);
  float ll = 0.f;
  for (int s = 0; s < p.nsplit; ++s) {
    const float* ml = p.part_ml + (((int64_t)nb * p.nsplit + s) * TR + r) * 2;
    if (ml[0] != -INFINITY) ll += ml[1] * exp2f(ml[0] - mm);
  }
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const int64_t pi = ((int64_t)nb * p.nsplit + s) * TR + r;
      const float ms = p.part_ml[pi * 2];
      if (ms != -INFINITY) acc += p.part_o[pi * DV + d] * exp2f(ms - mm);
    }
    p.out[(int64_t)(row0 + r) * DV + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  }
}

typedef CUresult (*PFN_encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

MARY_API int64_t mary_mla_scratch_floats(int NB, int nsplit) { return nsplit > 1 ? (int64_t)NB * nsplit * TR * (DV + 2) : 0; }
MARY_API int mary_mla_tile_rows() { return TR; }

// q [T * Hq, 576] bf16 (rows = token-major, head-minor); cache [pages, page_size (16 or 32), 576] bf16 with element strides
// tok_stride / page_stride; out [T * Hq, 512] bf16.  blk_seq / blk_row0: NB tiles of query rows (row0 is a global
// row index; a tile never crosses a sequence).  Tiles hold at most mary_mla_tile_rows() rows.
MARY_API int mary_mla_attention(const void* q, const void* cache, void* out, const int* page_table, const int* kv_len, const int* q_start,
                                const int* blk_seq, const int* blk_row0, int NB, int total_rows, int num_pages, int max_pages,
                                int64_t tok_stride, int64_t page_stride, int Hq, int nsplit, float scale, float* scratch,
                                int page_size, cudaStream_t s) {
  if (NB <= 0) return MARY_OK;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 1 && !scratch) return MARY_ERR_BAD_ARG;
  if ((tok_stride * 2) % 16 || (page_stride * 2) % 16 || (page_size != PAGE && page_size != KB)) return MARY_ERR_BAD_ARG;
  PFN_encode enc = (PFN_encode)mary_encode_fn();
  if (!enc) return MARY_ERR_CUDA;
  CUtensorMap tq, tkv;
  int rc = mary_make_tmap_2d(&tq, q, 4, (uint64_t)total_rows, DK, DK, TR, CHUNK, 1);
  if (rc) return rc;
  if (page_size == KB) {
    // dims: 64 elements of a chunk, 32 tokens of a page, 9 chunks of a token row, pages; box = one whole page, chunk-major
    cuuint64_t dims[4] = {CHUNK, KB, NCHUNK, (cuuint64_t)num_pages};
    cuuint64_t strides[3] = {(cuuint64_t)tok_stride * 2, CHUNK * 2, (cuuint64_t)page_stride * 2};
    cuuint32_t box[4] = {CHUNK, KB, NCHUNK, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return MARY_ERR_CUDA;
  } else {
    // dims: 576 elements of a token row, 16 tokens of a page, pages; box = [64 dims x 16 tokens] of one page
    cuuint64_t dims[3] = {DK, PAGE, (cuuint64_t)num_pages};
    cuuint64_t strides[2] = {(cuuint64_t)tok_stride * 2, (cuuint64_t)page_stride * 2};
    cuuint32_t box[3] = {CHUNK, PAGE, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&tkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return MARY_ERR_CUDA;
  }
  static MarySmemSlots smem_set = {};
  if (int rc = mary_ensure_dyn_smem((const void*)mla_attn_kernel, SMEM, &smem_set)) return rc;
  MlaParams p;
  p.page_table = page_table; p.kv_len = kv_len; p.q_start = q_start; p.blk_seq = blk_seq; p.blk_row0 = blk_row0;
  p.out = (__nv_bfloat16*)out; p.part_o = scratch; p.part_ml = scratch ? scratch + (int64_t)NB * nsplit * TR * DV : nullptr;
  p.max_pages = max_pages; p.Hq = Hq; p.nsplit = nsplit; p.page = page_size; p.scale_log2 = scale * 1.4426950408889634f; p.status = mary_status_ptr();
  MARY_LAUNCH(mla_attn_kernel, dim3(NB, nsplit), NTHREADS, SMEM, s, tq, tkv, p);
  MARY_CHECK_LAUNCH();
  if (nsplit > 1) {
    MARY_LAUNCH(mla_combine_kernel, dim3(NB, TR), 128, 0, s, p, NB);
    MARY_CHECK_LAUNCH();
  }
  return MARY_OK;
}
