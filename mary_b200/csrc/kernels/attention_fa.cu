// Causal (optionally sliding-window) attention for prefill over the paged KV cache, on tcgen05 tensor cores.
//
// The reference computes prefill attention with a SIMT kernel that gives one CTA to each (query, head) pair
// (src/models/inkling/banded.rs:109-299) or with materialised score blocks and library matmuls
// (src/models/inkling/burn.rs:550-797).  Here one CTA owns 128 query tokens of one head (MMA M = 128) and streams the
// keys and values of its KV head through shared memory 64 keys at a time, page by page:
//   warp 0    TMA for Q (once) and the K ring, a stage laid out [chunks][64 keys][64 dims] with the 128-byte swizzle.  With
//             64-token pages a stage is ONE 4-D operation (the tensor map orders the cache as dims-in-chunk, tokens,
//             chunks, pages, so the box [64, 64, chunks, 1] lands chunk-major); with 16-token pages it takes one
//             [16 tokens x 64 dims] operation per page and chunk, and the TMA unit's per-operation cost bounds the kernel;
//   warp 6    TMA for the V ring (same layout) — a ring of its own, so a K stage is refilled as soon as Q K^T has read
//             it and does not wait for the P V of that block;
//   warp 1    MMA: S[128 x 64] = Q K^T into one of two TMEM buffers (issued two blocks ahead), O[128 x DV] += P V with
//             V^T read from the V stage as an MN-major B operand and P from shared memory;
//   warps 2-5 softmax: thread r owns row r (TMEM lane r): tcgen05.ld of S, scale, causal / window mask, running maximum
//             with lazy rescale of O (only when the maximum grows by more than 2^8), P written to shared memory as bf16
//             in the un-swizzled K-major core-matrix layout, finally O / l to global memory.
// Blocks of keys that no row of the tile can see (beyond the causal diagonal, before the window) are never loaded.
// All waits are bounded; a wait that runs out sets the status word, frees TMEM and returns.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int PAGE = 16, KB = 64, TR = 128, CHUNK = 64;
constexpr int NSBUF = 2, NPBUF = 2;
constexpr int P_BYTES = TR * KB * 2;              // 16 KB
constexpr int NTHREADS = 224;
constexpr float RESCALE_THRESHOLD = 8.0f;

template <int DK, int DV>
struct FaCfg {
  static constexpr int NCK = DK / CHUNK, NCV = DV / CHUNK;
  static constexpr int Q_CHUNK_BYTES = TR * 128;
  static constexpr int Q_BYTES = NCK * Q_CHUNK_BYTES;
  static constexpr int K_CHUNK_BYTES = KB * 128, V_CHUNK_BYTES = KB * 128;
  static constexpr int K_STAGE = NCK * K_CHUNK_BYTES, V_STAGE = NCV * V_CHUNK_BYTES;
  static constexpr int STAGES = (DK + DV > 384) ? 2 : 3;
  static constexpr int SMEM = Q_BYTES + STAGES * (K_STAGE + V_STAGE) + NPBUF * P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = DV <= 128 ? 256 : 512;     // S: 2 x 64 columns at 0..127, O: DV columns at 128..
  static_assert(DK % CHUNK == 0 && DV % CHUNK == 0 && DV <= 256 && DK <= 256, "head dims: multiples of 64 up to 256");
  static_assert(SMEM <= 232448, "shared memory budget");
};

struct FaParams {
  const int* page_table; const int* kv_len; const int* q_start; const int* blk_seq; const int* blk_tok0;
  __nv_bfloat16* out;      // [T, Hq, DV]
  int max_pages, Hq, Hkv, window, page;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ uint64_t fa_desc_kmajor_noswz(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint64_t fa_desc_mnmajor_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS, 1)
fa_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const FaParams p) {
  using C = FaCfg<DK, DV>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;
  uint8_t* sV = sK + STAGES * C::K_STAGE;
  uint8_t* sP = sV + STAGES * C::V_STAGE;
  uint64_t* bars = (uint64_t*)(sP + NPBUF * P_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = q_full + 1;           // [STAGES]
  uint64_t* k_empty = k_full + STAGES;
  uint64_t* v_full = k_empty + STAGES;
  uint64_t* v_empty = v_full + STAGES;
  uint64_t* s_full = v_empty + STAGES;     // [NSBUF]
  uint64_t* s_empty = s_full + NSBUF;
  uint64_t* p_full = s_empty + NSBUF;      // [NPBUF]
  uint64_t* pv_done = p_full + NPBUF;
  uint32_t* tmem_slot = (uint32_t*)(pv_done + NPBUF);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (p.Hq / p.Hkv);
  const int seq = p.blk_seq[nb], tok0 = p.blk_tok0[nb];          // tok0: index into the flattened token axis
  const int seq_tok0 = p.q_start[seq], seq_tok1 = p.q_start[seq + 1];
  const int nrows = min(TR, seq_tok1 - tok0);
  const int kvlen = p.kv_len[seq];
  const int pos_first = kvlen - (seq_tok1 - seq_tok0) + (tok0 - seq_tok0);   // position of the tile's first query token
  const int k_hi = pos_first + nrows;                                         // keys [0, k_hi) are visible to some row
  const int k_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int b_lo = k_lo / KB, b_hi = (k_hi + KB - 1) / KB;
  const int nblk = max(0, b_hi - b_lo);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int b = 0; b < NSBUF; ++b) { mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4); }
    for (int b = 0; b < NPBUF; ++b) { mbar_init(&p_full[b], 4); mbar_init(&pv_done[b], 1); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;            // NSBUF x 64 columns
  const uint32_t tmem_O = tmem_base + 128;      // DV columns

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------------ producers: warp 0 = Q + K ring, warp 6 = V ring
    if (nblk > 0) {
      const bool isK = warp == 0;
      if (isK && lane == 0) {
        mbar_expect_tx(q_full, C::Q_BYTES);
        for (int c = 0; c < C::NCK; ++c) tma_load_2d(sQ + c * C::Q_CHUNK_BYTES, &tm_q, q_full, head * DK + c * CHUNK, tok0);
      }
      const int* pt = p.page_table + (int64_t)seq * p.max_pages;
      uint64_t* full = isK ? k_full : v_full;
      uint64_t* empty = isK ? k_empty : v_empty;
      uint8_t* ring = isK ? sK : sV;
      const int stage_bytes = isK ? C::K_STAGE : C::V_STAGE;
      const int nchunk = isK ? C::NCK : C::NCV;
      const int hd = isK ? DK : DV;
      const CUtensorMap* tm = isK ? &tm_k : &tm_v;
      int stage = 0; uint32_t phase = 0;
      for (int b = b_lo; b < b_hi; ++b) {
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA) ? 1 : 0;
          if (ok) mbar_expect_tx(&full[stage], stage_bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) goto done;
        if (p.page == KB) {
          if (lane == 0) {
            const int key0 = b * KB;
            const int page = (key0 < kvlen) ? pt[key0 / KB] : pt[0];
            tma_load_4d(ring + stage * stage_bytes, tm, &full[stage], 0, 0, kvh * nchunk, page);
          }
        } else
        // (KB / PAGE) pages x nchunk chunks operations of [16 tokens x 64 dims] (2 KB each), spread over the lanes
        for (int op = lane; op < (KB / PAGE) * nchunk; op += 32) {
          const int pg = op / nchunk, c = op % nchunk;
          const int key0 = b * KB + pg * PAGE;
          const int page = (key0 < kvlen) ? pt[key0 / PAGE] : pt[0];     // pages past the end: any valid page (masked)
          tma_load_3d(ring + stage * stage_bytes + c * (KB * 128) + pg * (PAGE * 128), tm, &full[stage], kvh * hd + c * CHUNK, 0, page);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nblk > 0) {
      const uint32_t idesc_s = idesc_bf16(TR, KB);
      const uint32_t idesc_o = idesc_bf16(TR, DV) | (1u << 16);           // B operand MN-major
      if (!mbar_wait(q_full, 0, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&](int i) -> bool {        // i = block index relative to b_lo
        const int stage = i % STAGES, sb = i % NSBUF;
        if (!mbar_wait(&s_empty[sb], ((i / NSBUF) & 1) ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait(&k_full[stage], (i / STAGES) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) return false;
        tc_fence_after();
        const uint32_t kb_addr = smem_u32(sK + stage * C::K_STAGE);
#pragma unroll
        for (int c = 0; c < C::NCK; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_f16(tmem_S + sb * KB, umma_desc_sw128(q_addr + c * C::Q_CHUNK_BYTES + k * 32),
                     umma_desc_sw128(kb_addr + c * C::K_CHUNK_BYTES + k * 32), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&k_empty[stage]);       // the K stage may be refilled once Q K^T has read it
        umma_commit(&s_full[sb]);
        return true;
      };
      if (!issue_qk(0)) goto done;
      if (nblk > 1 && !issue_qk(1)) goto done;
      for (int i = 0; i < nblk; ++i) {
        const int pb = i & 1, stage = i % STAGES;
        if (!mbar_wait(&v_full[stage], (i / STAGES) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
        if (!mbar_wait(&p_full[pb], (i >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
        tc_fence_after();
        const uint32_t vb_addr = smem_u32(sV + stage * C::V_STAGE);
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
          // A = P[:, 16 keys] (K-major, no swizzle: the two 16-byte key chunks of one MMA TR*16 bytes apart, 8-row groups
          // 128 bytes apart); B = V^T of those keys (MN-major, 128B swizzle: 64-dim groups one chunk apart, 8-key groups 1 KB apart)
          umma_f16(tmem_O, fa_desc_kmajor_noswz(p_addr + pb * P_BYTES + kk * 2 * (TR * 16), TR * 16, 128),
                   fa_desc_mnmajor_sw128(vb_addr + kk * 16 * 128, C::V_CHUNK_BYTES, 1024), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[stage]);
        umma_commit(&pv_done[pb]);
        if (i + 2 < nblk && !issue_qk(i + 2)) goto done;
      }
    }
  } else if (nblk > 0) {
    // ------------------------------------------------------------------ softmax warps: thread = query row
    const int q4 = warp & 3;                         // the TMEM lane group this warp may access
    const int r = q4 * 32 + lane;
    const bool row_ok = r < nrows;
    const int qpos = pos_first + r;
    const int lo_key = p.window > 0 ? qpos - p.window + 1 : 0;
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    for (int i = 0; i < nblk; ++i) {
      const int sb = i % NSBUF, pb = i & 1;
      if (!mbar_wait(&s_full[sb], (i / NSBUF) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
      tc_fence_after();
      uint32_t sr[KB];
      tmem_ld_32x32b_x32(tmem_S + lane_off + sb * KB, sr);
      tmem_ld_32x32b_x32(tmem_S + lane_off + sb * KB + 32, sr + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      const int key0 = (b_lo + i) * KB;
      // A block that every row of the tile sees entirely (all blocks left of the diagonal band and inside the window) takes the
      // short path: no per-element mask, the maximum on the raw scores, one fused multiply-add and one exponential per element.
      // A thread owns one query row and walks its 64 scores in sequence, so this loop's instruction count bounds the block rate.
      const bool full_blk = key0 + KB - 1 <= pos_first && (p.window <= 0 || key0 >= pos_first + TR - p.window);
      const float* sf = (const float*)sr;
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
          const int kj = key0 + j;
          const bool ok = row_ok && kj <= qpos && kj >= lo_key;
          const float v = ok ? __uint_as_float(sr[j]) * p.scale_log2 : -INFINITY;
          sr[j] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      }
      const bool need = mx > m_ref + RESCALE_THRESHOLD;
      const bool first = (m_ref == -INFINITY);
      float corr = 1.f;
      if (need) { corr = first ? 0.f : exp2f(m_ref - mx); m_ref = mx; }
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
          const float a = (m_ref == -INFINITY) ? 0.f : exp2f(__uint_as_float(sr[2 * j]) - m_ref);
          const float b = (m_ref == -INFINITY) ? 0.f : exp2f(__uint_as_float(sr[2 * j + 1]) - m_ref);
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
        for (int c0 = 0; c0 < DV; c0 += 32) {
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
#pragma unroll
      for (int c = 0; c < KB / 8; ++c)
        *(uint4*)(sP + pb * P_BYTES + c * (TR * 16) + r * 16) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
      fence_proxy_async();       // make the generic-proxy writes of P visible to the tensor core
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[pb]);
    }
    // ------------------------------------------------------------------ write out
    if (!mbar_wait(&pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
    tc_fence_after();
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
    for (int c0 = 0; c0 < DV; c0 += 32) {
      uint32_t o[32];
      tmem_ld_32x32b_x32(tmem_O + lane_off + c0, o);
      tmem_ld_wait();
      if (row_ok) {
        __nv_bfloat16* dst = p.out + ((int64_t)(tok0 + r) * p.Hq + head) * DV + c0;
        uint4 w[4];
        uint32_t* wp = (uint32_t*)w;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * inv_l, __uint_as_float(o[2 * j + 1]) * inv_l);
          wp[j] = *(uint32_t*)&h;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) ((uint4*)dst)[j] = w[j];
      }
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

int make_cache_map(CUtensorMap* m, const void* cache, int heads, int hd, int num_pages, int64_t tok_stride, int64_t page_stride, int page) {
  PFN_encodeTiled enc = mary_encode_fn();
  if (!enc) return MARY_ERR_CUDA;
  CUresult r;
  if (page == KB) {
    // dims: 64 elements of a chunk, 64 tokens of a page, chunks of a token row (all KV heads), pages; box = all chunks of one head
    cuuint64_t dims[4] = {CHUNK, KB, (cuuint64_t)(heads * hd / CHUNK), (cuuint64_t)num_pages};
    cuuint64_t strides[3] = {(cuuint64_t)tok_stride * 2, CHUNK * 2, (cuuint64_t)page_stride * 2};
    cuuint32_t box[4] = {CHUNK, KB, (cuuint32_t)(hd / CHUNK), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    // dims: elements of one token row (all KV heads), 16 tokens of a page, pages; box = [64 dims x 16 tokens] of one page
    cuuint64_t dims[3] = {(cuuint64_t)(heads * hd), PAGE, (cuuint64_t)num_pages};
    cuuint64_t strides[2] = {(cuuint64_t)tok_stride * 2, (cuuint64_t)page_stride * 2};
    cuuint32_t box[3] = {CHUNK, PAGE, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? MARY_OK : MARY_ERR_CUDA;
}

template <int DK, int DV>
int launch_fa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, int NB, cudaStream_t s) {
  static MarySmemSlots smem_set = {};
  if (int rc = mary_ensure_dyn_smem((const void*)fa_prefill_kernel<DK, DV>, FaCfg<DK, DV>::SMEM, &smem_set)) return rc;
  fa_prefill_kernel<DK, DV><<<dim3(NB, p.Hq), NTHREADS, FaCfg<DK, DV>::SMEM, s>>>(tq, tk, tv, p);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

}  // namespace

MARY_API int mary_attention_prefill_tile_rows() { return TR; }

// 1 when the tensor-core prefill kernel exists for these head dims.
MARY_API int mary_attention_prefill_supported(int DK, int DV) {
  return (DK == 64 && DV == 64) || (DK == 128 && DV == 128) || (DK == 192 && DV == 128) || (DK == 256 && DV == 256);
}

// q [T, Hq, DK] bf16 contiguous; kcache [pages, page_size (16 or 64), Hkv, DK] and vcache [.., Hkv, DV] bf16 with element strides per token
// and per page (heads contiguous inside a token row); out [T, Hq, DV] bf16.  blk_seq / blk_tok0: NB tiles of at most 128 query
// tokens that never cross a sequence.  Causal with the last query token of a sequence at position kv_len - 1; window > 0 keeps
// keys (pos - window, pos].  Returns MARY_ERR_BAD_ARG for head dims without an instantiation.
MARY_API int mary_attention_prefill(const void* q, const void* kcache, const void* vcache, void* out, const int* page_table,
                                    const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_tok0, int NB, int T, int Hq,
                                    int Hkv, int DK, int DV, int num_pages, int max_pages, int64_t k_tok_stride, int64_t k_page_stride,
                                    int64_t v_tok_stride, int64_t v_page_stride, int window, float scale, int page_size,
                                    cudaStream_t s) {
  if (NB <= 0) return MARY_OK;
  if (!mary_attention_prefill_supported(DK, DV) || Hkv < 1 || Hq % Hkv || (page_size != PAGE && page_size != KB)) return MARY_ERR_BAD_ARG;
  if ((k_tok_stride * 2) % 16 || (k_page_stride * 2) % 16 || (v_tok_stride * 2) % 16 || (v_page_stride * 2) % 16) return MARY_ERR_BAD_ARG;
  CUtensorMap tq, tk, tv;
  int rc = mary_make_tmap_2d(&tq, q, 4, (uint64_t)T, (uint64_t)Hq * DK, (uint64_t)Hq * DK, TR, CHUNK, 1);
  if (rc) return rc;
  if ((rc = make_cache_map(&tk, kcache, Hkv, DK, num_pages, k_tok_stride, k_page_stride, page_size))) return rc;
  if ((rc = make_cache_map(&tv, vcache, Hkv, DV, num_pages, v_tok_stride, v_page_stride, page_size))) return rc;
  FaParams p;
  p.page_table = page_table; p.kv_len = kv_len; p.q_start = q_start; p.blk_seq = blk_seq; p.blk_tok0 = blk_tok0;
  p.out = (__nv_bfloat16*)out; p.max_pages = max_pages; p.Hq = Hq; p.Hkv = Hkv; p.window = window; p.page = page_size;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = mary_status_ptr();
  if (DK == 64) return launch_fa<64, 64>(tq, tk, tv, p, NB, s);
  if (DK == 128) return launch_fa<128, 128>(tq, tk, tv, p, NB, s);
  if (DK == 192) return launch_fa<192, 128>(tq, tk, tv, p, NB, s);
  return launch_fa<256, 256>(tq, tk, tv, p, NB, s);
}
