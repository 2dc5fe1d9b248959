// Grouped NVFP4 x NVFP4 GEMM for MoE experts on tcgen05 block-scaled tensor cores.
//
//   y[row, n] = scale2[e] * sum_k  Wq_e[n, k] * sfW_e[n, k/16]  *  Xq[row, k] * sfX[row, k/16]
//
// Both operands are E2M1 codes with one UE4M3 scale per 16 elements (`kind::mxf4nvf4.block_scale.scale_vec::4X`,
// K = 64 per instruction); accumulation is f32 in TMEM; scale2 (the per-expert f32 scale) is applied in the epilogue;
// activations carry no second-level scale.  Replaces the reference's `fp4_linear_grouped`
// (src/models/inkling/moegroup.rs:263-539: one warp per 16x8 `mma.sync m16n8k64` tile, operands straight from
// global memory) and its separate `gate_up_silu` pass (src/models/inkling/fp4gemm.rs:154-189).
//
// Layout of the work:
//   * the WEIGHT rows fill the 128 TMEM lanes (row operand) and an expert's tokens are the MMA N dimension
//     (NT = 32 for decode-sized groups, 128 for prefill), so a decode step streams every weight byte exactly once
//     through TMA while the tensor core idles on the tiny N — the kernel is HBM-bound by construction;
//   * all experts' weights are ONE tensor [E * rows, K/2] bytes addressed through one tensor map (the reference's
//     "offsets into one bound mapping", moegroup.rs:19-32); the token tiles come from a device-built tile list
//     (expert, first padded row, valid rows), so no host round trip separates routing from the expert GEMM;
//   * scale factors are stored pre-arranged in 512-byte blocks (128 rows x 4 scales, byte (r%32)*16 + (r/32)*4 + j),
//     fetched with a bulk copy per stage and moved to TMEM with tcgen05.cp (32x128b.warpx4) right before the MMAs;
//   * with GLU the CTA loads the gate tile and the matching up tile (rows n0 and F + n0), keeps two accumulators and
//     writes act(gate) * up, so the [rows, 2F] intermediate never exists;
//   * persistent CTAs, TMA producer warp / MMA warp / 4 epilogue warps, ring of stages, bounded waits;
//   * the GLU epilogue can write its result ALREADY QUANTISED for the next GEMM (codes + scale tile): a thread holds one
//     feature of 32 token rows, so the 16-feature amax is a half-warp shuffle reduction and 8 codes pack into a word with
//     three more shuffles — the separate quantiser pass between w13 and w2 disappears;
//   * counter mode (ep_ctx.cuh): instead of a tile list from a planning kernel, every CTA waits (bounded) for the source
//     ranks' "dispatched" flags, reads the per-expert arrival counters and builds the tile list in shared memory; the w2
//     instance sends every output row to the combine buffer of the row's home rank (peer stores from the epilogue), and
//     its last CTA zeroes the counters and publishes the "returned" flags.
#include <string.h>

#include "common.cuh"
#include "ep_ctx.cuh"
#include "host_utils.h"
#include "nvfp4_quant.cuh"

using namespace mary;

namespace {

constexpr int BM = 128;
constexpr int BKB = 128;          // bytes of K per stage row = 256 FP4 elements = one 128-byte swizzle row
constexpr int KSTEP = 256;        // elements of K per stage
constexpr int MMAS = 4;           // 4 x (K = 64) per stage
constexpr int SF_STAGE = 2048;    // 4 blocks of 512 bytes
constexpr int NTHREADS = 192;

struct Tile { int expert, row0, rows, sf_tile; };

struct FP4Params {
  const Tile* tiles;
  const int* n_tiles;             // device scalar
  const uint8_t* sfw;             // [E, rows_total/128, K/64, 512]
  const uint8_t* sfx;             // [tile, K/64, 512]
  const float* scale2;            // [E]
  __nv_bfloat16* out;             // [padded rows, n_out]
  const uint64_t* row_ptrs;       // optional: destination address of every padded row (may point into a peer GPU)
  int64_t ldo;
  int n_out;                      // output features (F with GLU)
  int rows_total;                 // weight rows per expert (2F with GLU)
  int K, k_blocks, w_tiles;
  int act;
  int* status;
  uint8_t* q_out;                 // GLU only, optional: the result as NVFP4 codes [padded rows, n_out / 2] ...
  uint8_t* q_sf;                  // ... and scale tiles [tile, n_out / 64, 512] instead of bf16 `out`
  int ep_mode;                    // 0: tile list from memory; 1: counter mode, wait for dispatch; 2: counter mode, return rows + signal
  const int* meta;                // ep_mode 2: return word of every slab row
};

template <int NT, bool GLU>
struct Cfg {
  static constexpr int A_BYTES = BM * BKB;                                // 16 KB
  static constexpr int NA = GLU ? 2 : 1;
  static constexpr int B_BYTES = NT * BKB;
  static constexpr int STAGE_BYTES = NA * (A_BYTES + SF_STAGE) + B_BYTES + SF_STAGE;
  static constexpr int ACC_COLS = NA * NT;
  static constexpr int SF_COLS = 16 * NA + 16;
  static constexpr int ACC_BUFS = (2 * ACC_COLS + SF_COLS <= 512) ? 2 : 1;
  static constexpr int COLS_RAW = ACC_BUFS * ACC_COLS + SF_COLS;
  static constexpr int TMEM_COLS = COLS_RAW <= 32 ? 32 : COLS_RAW <= 64 ? 64 : COLS_RAW <= 128 ? 128 : COLS_RAW <= 256 ? 256 : 512;
  static constexpr int STAGES_RAW = (219 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
};

template <int NT, bool GLU>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_nvfp4_grouped_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const FP4Params p,
                          const EpCtx ep) {
  pdl_sync();
  using C = Cfg<NT, GLU>;
  __shared__ Tile s_tiles[NT == 32 ? EP_MAX_TILES : 1];
  __shared__ unsigned short s_cnt[NT == 32 ? EP_MAX_TILES : 1];   // arrival counters, clamped to cap_e (<= 65535); 16 bits keep the 9-stage ring
  __shared__ int s_ntiles;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~uintptr_t(1023));
  uint64_t* full = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf = tmem_base + C::ACC_BUFS * C::ACC_COLS;     // [SFA gate 16][SFA up 16][SFB 16]

  const Tile* tiles = p.tiles;
  int n_tiles;
  if (NT == 32 && p.ep_mode) {
    // counter mode: the tile list comes from the arrival counters, once every source rank has dispatched
    if (p.ep_mode == 1 && !ep.local_only && ep.world > 1 && (int)threadIdx.x < ep.world) {
      const uint32_t target = *ep.epoch + 1;
      if (!ep_wait_flag((const uint32_t*)ep.flags[ep.rank] + threadIdx.x, target, ep.wait_ns, p.status)) *abort_flag = 1;
    }
    fence_proxy_async_global();                    // the slabs were written by other GPUs' plain stores; TMA reads them next
    __syncthreads();
    {
      // the flags were acquired above, so the counters can be read with plain L2 loads, all of them at once
      const int* cnt = (const int*)ep.cnt[ep.rank];
      for (int e = threadIdx.x; e < ep.n_slots; e += NTHREADS) { const int v = __ldcg(cnt + e); s_cnt[e] = (unsigned short)(v < ep.cap_e ? (v < 0 ? 0 : v) : ep.cap_e); }
    }
    __syncthreads();
    if (warp == 0) {
      int base = 0;
      for (int e0 = 0; e0 < ep.n_slots; e0 += 32) {
        const int e = e0 + lane;
        int c = e < ep.n_slots ? s_cnt[e] : 0;
        c = c < ep.cap_e ? c : ep.cap_e;
        const int nt = (c + NT - 1) / NT;
        int incl = nt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
        const int off = base + incl - nt;
        for (int i = 0; i < nt; ++i)
          if (off + i < EP_MAX_TILES) s_tiles[off + i] = Tile{e, e * ep.cap_e + i * NT, min(NT, c - i * NT), e * (ep.cap_e / NT) + i};
        base += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) {
        if (base > EP_MAX_TILES) { atomicCAS(p.status, 0, MARY_ERR_BOUNDS); base = EP_MAX_TILES; }
        s_ntiles = base;
      }
    }
    __syncthreads();
    tiles = s_tiles;
    n_tiles = *abort_flag ? 0 : s_ntiles;
  } else {
    n_tiles = *p.n_tiles;
  }
  const int total = n_tiles * p.w_tiles;          // work item = (weight row tile, token tile), token tile fastest ...
  // ... except with 128-token tiles (prefill-sized batches): there the quantised activations of all tiles outgrow L2, while an
  // expert has one or two token tiles, so the weight tile runs fastest: a token tile is read from memory once and serves all
  // weight tiles of its expert from L2, and the few token tiles of one expert meet their weight tiles within one wave of CTAs
  constexpr bool WT_FAST = NT == 128;
  const int sf_per_tile = p.k_blocks * SF_STAGE;  // scale bytes of one 128-row block over the whole K

  // stage layout: [A gate 16K][A up 16K]? [B NT*128][SFA gate 2K][SFA up 2K]? [SFB 2K]
  constexpr int OFF_B = C::NA * C::A_BYTES;
  constexpr int OFF_SFA = OFF_B + C::B_BYTES;
  constexpr int OFF_SFB = OFF_SFA + C::NA * SF_STAGE;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      if (p.ep_mode) fence_proxy_async_global();
      for (int w = blockIdx.x; w < total; w += gridDim.x) {
        const Tile t = tiles[WT_FAST ? w / p.w_tiles : w % n_tiles];
        const int wt = WT_FAST ? w % p.w_tiles : w / n_tiles;
        const int wrow = t.expert * p.rows_total + wt * BM;
        const uint8_t* sfa = p.sfw + ((int64_t)t.expert * (p.rows_total / BM) + wt) * sf_per_tile;
        const uint8_t* sfa_up = sfa + (int64_t)(p.n_out / BM) * sf_per_tile;
        const uint8_t* sfb = p.sfx + (int64_t)t.sf_tile * sf_per_tile;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
          uint8_t* st = smem + stage * C::STAGE_BYTES;
          mbar_expect_tx(&full[stage], C::STAGE_BYTES);
          tma_load_2d(st, &tm_w, &full[stage], kb * BKB, wrow);
          if (GLU) tma_load_2d(st + C::A_BYTES, &tm_w, &full[stage], kb * BKB, wrow + p.n_out);
          tma_load_2d(st + OFF_B, &tm_x, &full[stage], kb * BKB, t.row0);
          bulk_load(st + OFF_SFA, sfa + (int64_t)kb * SF_STAGE, SF_STAGE, &full[stage]);
          if (GLU) bulk_load(st + OFF_SFA + SF_STAGE, sfa_up + (int64_t)kb * SF_STAGE, SF_STAGE, &full[stage]);
          bulk_load(st + OFF_SFB, sfb + (int64_t)kb * SF_STAGE, SF_STAGE, &full[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = idesc_nvfp4(BM, NT);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x, ++it) {
        const int buf = C::ACC_BUFS == 2 ? (it & 1) : 0;
        const uint32_t acc_phase = C::ACC_BUFS == 2 ? ((it >> 1) & 1) : (it & 1);
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * C::ACC_COLS;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + stage * C::STAGE_BYTES);
          // scale factors: shared memory -> TMEM (4 blocks per operand tile)
#pragma unroll
          for (int k = 0; k < MMAS; ++k) {
            tmem_cp_32x128b_warpx4(tmem_sf + 4 * k, umma_desc_sf(st + OFF_SFA + 512 * k));
            if (GLU) tmem_cp_32x128b_warpx4(tmem_sf + 16 + 4 * k, umma_desc_sf(st + OFF_SFA + SF_STAGE + 512 * k));
            tmem_cp_32x128b_warpx4(tmem_sf + 16 * C::NA + 4 * k, umma_desc_sf(st + OFF_SFB + 512 * k));
          }
#pragma unroll
          for (int k = 0; k < MMAS; ++k) {
            const uint64_t db = umma_desc_sw128(st + OFF_B + 32 * k);
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            const uint32_t sfb_t = tmem_sf + 16 * C::NA + 4 * k;
            umma_nvfp4(d0, umma_desc_sw128(st + 32 * k), db, idesc, accum, tmem_sf + 4 * k, sfb_t);
            if (GLU) umma_nvfp4(d0 + NT, umma_desc_sw128(st + C::A_BYTES + 32 * k), db, idesc, accum, tmem_sf + 16 + 4 * k, sfb_t);
          }
          umma_commit(&empty[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++it) {
      const Tile t = tiles[WT_FAST ? w / p.w_tiles : w % n_tiles];
      const int wt = WT_FAST ? w % p.w_tiles : w / n_tiles;
      const int buf = C::ACC_BUFS == 2 ? (it & 1) : 0;
      const uint32_t acc_phase = C::ACC_BUFS == 2 ? ((it >> 1) & 1) : (it & 1);
      if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
      tc_fence_after();
      const float s2 = p.scale2[t.expert];
      const int n = wt * BM + q * 32 + lane;                // output feature of this thread
      const uint32_t taddr = tmem_base + buf * C::ACC_COLS + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < NT; c0 += 32) {
        if (c0 >= t.rows) break;
        uint32_t r[32], r2[32];
        tmem_ld_32x32b_x32(taddr + c0, r);
        if (GLU) tmem_ld_32x32b_x32(taddr + NT + c0, r2);
        tmem_ld_wait();
        if (n < p.n_out) {
          if (GLU && p.q_out) {
            // the result goes out quantised for the next GEMM: this thread holds feature n of rows c0 .. c0 + 31; the 16
            // features of a scale block are 16 neighbouring lanes, the 8 features of a code word 8 neighbouring lanes
            const int sub = lane & 7;
            const int64_t sf_base = (int64_t)t.sf_tile * (p.n_out / 64) * 512 + (int64_t)(n / 64) * 512 + ((n / 16) & 3);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float a = __uint_as_float(r[j]) * s2;
              const float v = __bfloat162float(__float2bfloat16(glu_f(p.act, a, __uint_as_float(r2[j]) * s2)));
              float amax = fabsf(v);
              amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
              amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
              amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
              amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
              float s;
              const uint8_t sb = nvfp4_scale_byte(amax, &s);
              uint32_t pk = (s > 0.f ? nvfp4_code(__fdiv_rn(v, s)) : 0u) << (4 * sub);
              pk |= __shfl_xor_sync(0xffffffffu, pk, 1);
              pk |= __shfl_xor_sync(0xffffffffu, pk, 2);
              pk |= __shfl_xor_sync(0xffffffffu, pk, 4);
              if (c0 + j < t.rows) {
                const int rr = c0 + j;                         // row within the tile
                if (sub == 0) *(uint32_t*)(p.q_out + (int64_t)(t.row0 + rr) * (p.n_out / 2) + n / 2) = pk;
                if ((lane & 15) == 0) p.q_sf[sf_base + (rr % 32) * 16 + (rr / 32) * 4] = sb;
              }
            }
          } else {
            // destination of every row: plain output, a caller-given address list, or (counter mode 2) the combine slot of the
            // row's home rank decoded from its return word; lane j resolves row c0 + j and the warp shares the addresses
            uint64_t my_dst = 0;
            if (c0 + lane < t.rows) {
              const int64_t row = t.row0 + c0 + lane;
              if (p.ep_mode == 2) {
                const int m = __ldcg(p.meta + row);        // written by the source rank's plain peer store: read from L2
                const int src = m / ep.entry_stride;
                if (m >= 0 && src < EP_MAX_RANKS) my_dst = ep.comb[src] + (uint64_t)(m - src * ep.entry_stride) * p.n_out * sizeof(__nv_bfloat16);
              } else if (p.row_ptrs) my_dst = p.row_ptrs[row];
              else my_dst = (uint64_t)(p.out + row * p.ldo);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const uint64_t d64 = __shfl_sync(0xffffffffu, my_dst, j);
              if (c0 + j < t.rows && d64) {
                const float a = __uint_as_float(r[j]) * s2;
                const float v = GLU ? glu_f(p.act, a, __uint_as_float(r2[j]) * s2) : a;
                ((__nv_bfloat16*)d64)[n] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (p.ep_mode == 2) __threadfence_system();            // this thread's peer stores are visible before the CTA is counted done
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
  if (NT == 32 && p.ep_mode == 2 && threadIdx.x == 0) {
    // the CTA that finishes last closes the layer on this owner: counters back to zero for the next layer, then the
    // "returned" flag on every home rank (which is what lets that rank dispatch again)
    const int prev = atomicAdd(&ep.done[1], 1);
    if (prev == (int)gridDim.x - 1) {
      ep.done[1] = 0;
      int* cnt = (int*)ep.cnt[ep.rank];
      for (int e = 0; e < ep.n_slots; ++e) cnt[e] = 0;
      const uint32_t target = *ep.epoch + 1;
      __threadfence_system();
      if (!ep.local_only)
        for (int d = 0; d < ep.world; ++d) ep_st_release_sys((uint32_t*)ep.flags[(ep.rank + d) % ep.world] + EP_MAX_RANKS + ep.rank, target);
    }
  }
}

template <int NT, bool GLU>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const FP4Params& p, const EpCtx& ep, cudaStream_t s) {
  using C = Cfg<NT, GLU>;
  // dynamic ring + the kernel's static shared memory (tile list, counters) must fit the 227 KB a CTA can have
  static_assert(C::SMEM + (NT == 32 ? EP_MAX_TILES * (sizeof(Tile) + 2) + 64 : 64) <= 227 * 1024, "shared memory budget");
  static MarySmemSlots smem_set = {};
  if (int rc = mary_ensure_dyn_smem((const void*)gemm_nvfp4_grouped_kernel<NT, GLU>, C::SMEM, &smem_set)) return rc;
  MARY_LAUNCH((gemm_nvfp4_grouped_kernel<NT, GLU>), mary_num_sms(), NTHREADS, C::SMEM, s, tw, tx, p, ep);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

int run(const void* wq, const void* sfw, const float* scale2, const void* xq, const void* sfx, const void* tiles, const int* n_tiles,
        void* out, int64_t ldo, int E, int n_out, int K, int64_t x_rows, int nt, int glu, const uint64_t* row_ptrs, void* q_out, void* q_sf,
        int ep_mode, const int* meta, const EpCtx* ctx, cudaStream_t s) {
  const int rows_total = glu ? 2 * n_out : n_out;
  if ((K % KSTEP) || (n_out % BM) || (nt != 32 && nt != 128)) return MARY_ERR_BAD_ARG;
  if ((q_out != nullptr) != (q_sf != nullptr) || (q_out && (!glu || (n_out % 64)))) return MARY_ERR_BAD_ARG;
  if (ep_mode && (nt != 32 || !ctx || ctx->NT != 32 || (ctx->cap_e % 32) || ctx->cap_e > 65535 || ctx->n_slots > EP_MAX_TILES || ctx->rank < 0 || ctx->rank >= EP_MAX_RANKS ||
                  (int64_t)ctx->n_slots * ctx->cap_e > x_rows || (ep_mode == 2 && !meta)))
    return MARY_ERR_BAD_ARG;
  FP4Params p;
  p.tiles = (const Tile*)tiles; p.n_tiles = n_tiles; p.sfw = (const uint8_t*)sfw; p.sfx = (const uint8_t*)sfx;
  p.scale2 = scale2; p.out = (__nv_bfloat16*)out; p.row_ptrs = row_ptrs; p.ldo = ldo; p.n_out = n_out; p.rows_total = rows_total; p.K = K;
  p.k_blocks = K / KSTEP; p.w_tiles = n_out / BM; p.act = glu ? glu - 1 : 0; p.status = mary_status_ptr();
  p.q_out = (uint8_t*)q_out; p.q_sf = (uint8_t*)q_sf; p.ep_mode = ep_mode; p.meta = meta;
  EpCtx ep;
  if (ctx) ep = *ctx; else memset(&ep, 0, sizeof(ep));
  CUtensorMap tw, tx;
  int rc = mary_make_tmap_2d(&tw, wq, 2, (uint64_t)E * rows_total, K / 2, K / 2, BM, BKB, 1);
  if (rc) return rc;
  rc = mary_make_tmap_2d(&tx, xq, 2, x_rows, K / 2, K / 2, nt, BKB, 1);
  if (rc) return rc;
  if (glu) return nt == 32 ? launch<32, true>(tw, tx, p, ep, s) : launch<128, true>(tw, tx, p, ep, s);
  return nt == 32 ? launch<32, false>(tw, tx, p, ep, s) : launch<128, false>(tw, tx, p, ep, s);
}

}  // namespace

// wq    [E * rows_total, K/2] bytes (rows_total = n_out, or 2 * n_out with glu: gate rows then up rows)
// sfw   [E, rows_total/128, K/64, 512] pre-arranged weight scales;  scale2 [E]
// xq    [padded rows, K/2] bytes;  sfx [tiles, K/64, 512] activation scales in the same block layout (row r of a
//       tile at byte (r%32)*16 + (r/32)*4 + j)
// tiles [max_tiles] of {expert, row0, rows, sf_tile}, *n_tiles valid; nt = token-tile width (32 or 128)
// out   [padded rows, n_out] bf16
//
// row_ptrs (optional, [padded rows] device addresses): when given, row r of the result is written to row_ptrs[r] instead
// of out + r * ldo.  The addresses may lie in another GPU's memory (peer mapping): this is how the expert-parallel
// combine sends every expert output row straight to the rank that owns the token, from inside the GEMM epilogue.
MARY_API int mary_gemm_nvfp4_grouped_ex(const void* wq, const void* sfw, const float* scale2, const void* xq, const void* sfx,
                                        const void* tiles, const int* n_tiles, void* out, int64_t ldo, int E, int n_out, int K,
                                        int64_t x_rows, int nt, int glu, const uint64_t* row_ptrs, cudaStream_t s) {
  return run(wq, sfw, scale2, xq, sfx, tiles, n_tiles, out, ldo, E, n_out, K, x_rows, nt, glu, row_ptrs, nullptr, nullptr, 0, nullptr,
             nullptr, s);
}

MARY_API int mary_gemm_nvfp4_grouped(const void* wq, const void* sfw, const float* scale2, const void* xq, const void* sfx,
                                     const void* tiles, const int* n_tiles, void* out, int64_t ldo, int E, int n_out, int K,
                                     int64_t x_rows, int nt, int glu, cudaStream_t s) {
  return mary_gemm_nvfp4_grouped_ex(wq, sfw, scale2, xq, sfx, tiles, n_tiles, out, ldo, E, n_out, K, x_rows, nt, glu, nullptr, s);
}

// GLU GEMM whose result leaves the kernel quantised for the next NVFP4 GEMM: q_out [padded rows, n_out / 2] codes and
// q_sf [padded rows / nt, n_out / 64, 512] scale tiles (same rules as the stand-alone quantiser applied to the bf16-rounded
// activation, so the bytes equal those of GEMM -> bf16 -> quantise).  Padding rows are left untouched.
MARY_API int mary_gemm_nvfp4_grouped_glu_q(const void* wq, const void* sfw, const float* scale2, const void* xq, const void* sfx,
                                           const void* tiles, const int* n_tiles, void* q_out, void* q_sf, int E, int n_out, int K,
                                           int64_t x_rows, int nt, int glu, cudaStream_t s) {
  if (!glu || !q_out) return MARY_ERR_BAD_ARG;
  return run(wq, sfw, scale2, xq, sfx, tiles, n_tiles, nullptr, 0, E, n_out, K, x_rows, nt, glu, nullptr, q_out, q_sf, 0, nullptr, nullptr, s);
}

// Counter mode (ep_ctx.cuh).  ep_mode 1: the w13 instance — waits for the dispatch flags, tile list from the arrival counters,
// GLU result quantised into q_out / q_sf.  ep_mode 2: the w2 instance — same tile list, every row stored to the combine slot
// its return word (meta) names, counters zeroed and "returned" flags published by the last CTA.  x_rows: rows of the slab.
MARY_API int mary_gemm_nvfp4_grouped_ep(const void* wq, const void* sfw, const float* scale2, const void* xq, const void* sfx, void* q_out,
                                        void* q_sf, const int* meta, int E, int n_out, int K, int64_t x_rows, int glu, int ep_mode,
                                        const EpCtx* ctx, cudaStream_t s) {
  if ((ep_mode != 1 && ep_mode != 2) || !ctx || (ep_mode == 1 && (!glu || !q_out)) || (ep_mode == 2 && glu)) return MARY_ERR_BAD_ARG;
  return run(wq, sfw, scale2, xq, sfx, nullptr, nullptr, nullptr, 0, E, n_out, K, x_rows, 32, glu, nullptr, q_out, q_sf, ep_mode, meta, ctx, s);
}
