// bf16 GEMM on the 5th-generation tensor cores: out[M, N] = X[M, K] * W[N, K]^T  (both operands K-major).
//
// Replaces the reference's hand `mma.sync m16n8k16` kernel (src/models/inkling/bf16gemm.rs:64-136, 2.9 TFLOP/s)
// and its library lanes (bf16gemm.rs:625-658).  Design:
//   * persistent CTAs (one per SM), 192 threads: warp 0 issues TMA loads, warp 1 owns TMEM and issues
//     tcgen05.mma from one elected thread, warps 2-5 run the epilogue (tcgen05.ld -> registers -> global);
//   * operand tiles are [rows x 64] bf16 = rows of 128 bytes in the 128-byte swizzle, moved by TMA into a
//     ring of shared-memory stages guarded by full/empty mbarriers; out-of-range rows/columns read as zero,
//     so M, N and K need no padding (K % 8 == 0 for the 16-byte pitch);
//   * the accumulator (128 lanes x BN columns, f32) lives in TMEM and is double buffered, so the epilogue of
//     tile i overlaps the main loop of tile i+1;
//   * the "row" operand of the MMA (128 rows per tile) is either the activations (large M) or, for decode-sized
//     M, the WEIGHTS (swap: weight rows fill the 128 lanes, the few tokens become the MMA N), which keeps every
//     shared-memory byte of a stage useful when the kernel is weight-streaming bound;
//   * optional GLU epilogue: W = [gate rows ; up rows]; the CTA loads the matching gate and up tiles, keeps two
//     accumulators and writes act(gate) * up;
//   * optional split-K with an f32 reduction epilogue (red.global.add.f32) into a zeroed buffer, which is also
//     the hook for reducing into peer GPUs' buffers.
#include <cstdlib>
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int BM = 128;      // rows of the row-operand tile (TMEM lanes)
constexpr int BK = 64;       // K per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NTHREADS = 192;

enum { EPI_STORE_BF16 = 0, EPI_RED_F32 = 1, EPI_STORE_F32 = 2, EPI_RS_BF16 = 3, EPI_SK_BF16 = 4, EPI_SK_F32 = 5 };

struct GemmParams {
  int rows_r, rows_c;        // extents of the row operand and the column operand (tiles are clipped to them)
  int K;
  int tiles_r, tiles_c, split_k, k_blocks_per_split, k_blocks;
  int glu_offset;            // rows between the gate tile and the up tile of the weight operand (GLU only)
  int act;
  int epi;
  int swap;                  // 1: row operand = weights, D[i][j] -> out[j * ldo + i]
  int64_t ldo;
  int batch;                 // independent problems (z coordinate of both tensor maps)
  int64_t out_batch_stride;  // elements
  void* out;
  // reduce-scatter epilogue (EPI_RS_BF16): token row t belongs to rank t / rs_rpr; this rank's partial row is stored into
  // the owner's staging buffer rs_bufs[owner][rs_src][t % rs_rpr][:] (peer memory for owner != this rank)
  uint64_t rs_bufs[8];
  int rs_rpr, rs_src;
  const float* bias;         // optional, indexed by output feature
  float alpha;
  int* status;
  // split-K finished inside the kernel (EPI_SK_*): every K-slice adds its partial tile into the tile's f32 accumulator in `ws`
  // (red.global.add, spread over L2) and bumps the tile's counter; the slice that arrives last reads the sum once, stores the
  // finished tile in the output type and writes the zeros back, so accumulator and counter are ready for the next call.
  float* ws;
  int* counters;
  // stream-K (sk_units > 0, batch 1): the tiles_r * tiles_c * k_blocks K-blocks are dealt out in equal contiguous runs of
  // sk_units blocks per CTA, so every CTA streams the same number of weight bytes whatever the tile count; a tile whose
  // blocks fall to several CTAs is finished by whichever of them arrives last.
  int sk_units;
  // grouped (mixture-of-experts) mode: the token operand is ONE matrix of padded rows cut into tiles (column tiles of BN rows with
  // swap, 128-row tiles without), tile t belongs to expert g_tiles[4 t] (the routing plan's tile table; g_meta[0] = number of tiles
  // in use) and multiplies that expert's slice of the 3-D weight operand.  Tiles past g_meta[0] are skipped by every role alike.
  const int* g_tiles;
  const int* g_meta;
  int g_experts;
  // 1: the weight operand is constant (model weights) and the launch allows programmatic dependent launch, so the producer may
  // fetch the first weight tiles while the previous kernel of the stream is still draining; activations wait for it as always
  int w_static;
  // > 0: tiles are walked in bands of `raster` column tiles, row tiles fastest inside a band, so the CTAs that run together cover a
  // compact block of the output: the band's weight tiles stay in L2 while the row operand streams past them once per band.  With
  // column tiles fastest (raster 0) a wide output re-reads every weight tile once per row tile.
  int raster;
  // batched problems may SHARE an operand (batch stride 0): its tensor map then has one batch entry and every problem reads it
  int zr_mul, zc_mul;
};

// One unit of work of a CTA: K-blocks [kb0, kb1) of output tile (tr, tc) of problem bz; `seg` of `nseg` partial results of that
// tile, stored in scratch slot `slot`.
struct WorkItem { int bz, tr, tc, tile, kb0, kb1, seg, nseg, slot; };

// LEAN: compile-time promise of the decode-shaped launches (weights are the row operand, plain bf16 store, no routing plan, no
// band walk, no reduce-scatter): the kernel instantiated with it carries none of the other paths' code, which matters for launches
// of a few microseconds that start with a cold instruction cache.
template <bool LEAN>
struct WorkIter {
  const GemmParams& p;
  int tt, unit, end;
  __device__ WorkIter(const GemmParams& p_) : p(p_) {
    tt = blockIdx.x;
    unit = blockIdx.x * p.sk_units;
    end = min(unit + p.sk_units, p.tiles_r * p.tiles_c * p.k_blocks);
  }
  __device__ bool next(WorkItem& w) {
    if (p.sk_units > 0) {
      if (unit >= end) return false;
      const int kb = p.k_blocks, u = p.sk_units;
      w.tile = unit / kb;
      w.kb0 = unit - w.tile * kb;
      w.kb1 = min(kb, w.kb0 + (end - unit));
      w.bz = 0;
      w.tc = w.tile % p.tiles_c;
      w.tr = w.tile / p.tiles_c;
      const int first = (w.tile * kb) / u, last = ((w.tile + 1) * kb - 1) / u;
      w.seg = (int)blockIdx.x - first;
      w.nseg = last - first + 1;
      w.slot = first + w.tile + w.seg;
      unit += w.kb1 - w.kb0;
      return true;
    }
    const int per_batch = p.tiles_r * p.tiles_c * p.split_k;
    if (!LEAN && p.g_tiles) {
      // token tiles the plan does not use: column tiles with swap, row tiles without
      const int used = p.g_meta[0];
      while (tt < per_batch && (p.swap ? tt % p.tiles_c : tt / (p.tiles_c * p.split_k)) >= used) tt += gridDim.x;
    }
    if (tt >= per_batch * p.batch) return false;
    const int t = tt % per_batch;
    w.bz = tt / per_batch;
    int ks;
    if (!LEAN && p.raster > 0) {              // split_k == 1 here
      const int band = t / (p.raster * p.tiles_r), base = band * p.raster;
      const int gw = min(p.raster, p.tiles_c - base), in = t - band * p.raster * p.tiles_r;
      w.tr = in / gw;
      w.tc = base + in % gw;
      ks = 0;
    } else {
      w.tc = t % p.tiles_c;
      ks = (t / p.tiles_c) % p.split_k;
      w.tr = t / (p.tiles_c * p.split_k);
    }
    w.kb0 = ks * p.k_blocks_per_split;
    w.kb1 = min(w.kb0 + p.k_blocks_per_split, p.k_blocks);
    w.tile = (w.bz * p.tiles_r + w.tr) * p.tiles_c + w.tc;
    w.seg = ks;
    w.nseg = p.split_k;
    w.slot = w.tile * p.split_k + ks;
    tt += gridDim.x;
    return true;
  }
};

__device__ __forceinline__ __nv_bfloat16* rs_row(const GemmParams& p, int token_row) {
  const int owner = token_row / p.rs_rpr, lr = token_row - owner * p.rs_rpr;
  return (__nv_bfloat16*)p.rs_bufs[owner] + ((int64_t)p.rs_src * p.rs_rpr + lr) * p.ldo;
}

// SHORT: few pipeline stages (under 100 KB of shared memory) so that two CTAs fit one SM: with programmatic dependent launch the
// next decode-sized GEMM of the stream then sets up and requests its first weight tiles while this one drains.
template <int BN, bool GLU, bool SHORT = false>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;                       // 16 KB
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int ROW_TILES = 1;
  static constexpr int STAGE_BYTES = A_BYTES * (GLU ? 2 : 1) + B_BYTES;
  static constexpr int ACC_COLS = (GLU ? 2 : 1) * BN;
  static constexpr int TMEM_COLS_RAW = 2 * ACC_COLS;
  static constexpr int TMEM_COLS = TMEM_COLS_RAW <= 32 ? 32 : TMEM_COLS_RAW <= 64 ? 64 : TMEM_COLS_RAW <= 128 ? 128
                                   : TMEM_COLS_RAW <= 256 ? 256 : 512;
  static constexpr int MAX_SMEM = 220 * 1024;
  static constexpr int STAGES_RAW = (MAX_SMEM - 1024) / STAGE_BYTES;
  static constexpr int STAGES_SHORT = (96 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = SHORT ? STAGES_SHORT : (STAGES_RAW > 12 ? 12 : STAGES_RAW);
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(TMEM_COLS_RAW <= 512, "accumulators exceed TMEM");
};

// In GLU mode the WEIGHT operand has two tiles (gate, up).  With swap the weights are the row operand (two
// 128-row tiles, two accumulators of BN columns); without swap they are the column operand and the two
// BN-row tiles are... handled by launching the swapped roles only: GLU without swap is expressed by the host
// as two B tiles, see launch code.  To keep one device code path, GLU always means "two row-operand tiles".
template <int BN, bool GLU, int LEAN_MODE>          // 0: every path; 1: decode-shaped launches only; 2: the same with the short pipeline
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_r, const __grid_constant__ CUtensorMap tm_c, const GemmParams p) {
  constexpr bool LEAN = LEAN_MODE != 0;
  using C = Cfg<BN, GLU, LEAN_MODE == 2>;
  const bool swap = LEAN ? true : p.swap != 0;
  const int* const g_tiles = LEAN ? nullptr : p.g_tiles;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~uintptr_t(1023));
  uint64_t* full = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;     // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* sk_last = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x < C::STAGES) { mbar_init(&full[threadIdx.x], 1); mbar_init(&empty[threadIdx.x], 1); }
  if (threadIdx.x >= 32 && threadIdx.x < 34) { mbar_init(&acc_full[threadIdx.x - 32], 1); mbar_init(&acc_empty[threadIdx.x - 32], 4); }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    tma_prefetch_desc(&tm_r);
    tma_prefetch_desc(&tm_c);
  }
  fence_barrier_init();
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // dependents may start only now that this CTA holds its TMEM columns: a successor that allocated first and then waited for this
  // kernel would leave both waiting on each other
  pdl_launch();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      WorkIter<LEAN> iter(p);
      WorkItem w;
      bool have = false;
      int pre = 0;                               // stages whose barrier is armed and whose weight tile is already in flight
      if (p.w_static) {
        // constant weights: the first tiles of this CTA's first work item are requested before the previous kernel has finished
        have = iter.next(w);
        if (have) {
          pre = min(w.kb1 - w.kb0, C::STAGES);
          for (int i = 0; i < pre; ++i) {
            uint8_t* st = smem + i * C::STAGE_BYTES;
            const int kb = w.kb0 + i;
            mbar_expect_tx(&full[i], C::STAGE_BYTES);
            if (swap) {
              tma_load_3d(st, &tm_r, &full[i], kb * BK, w.tr * BM, w.bz * p.zr_mul);
              if (GLU) tma_load_3d(st + C::A_BYTES, &tm_r, &full[i], kb * BK, p.glu_offset + w.tr * BM, w.bz * p.zr_mul);
            } else {
              tma_load_3d(st + C::A_BYTES * (GLU ? 2 : 1), &tm_c, &full[i], kb * BK, w.tc * BN, w.bz * p.zc_mul);
            }
          }
        }
      }
      pdl_wait();
      if (!p.w_static) have = iter.next(w);
      while (have) {
        const int tr = w.tr, tc = w.tc;
        int zr = w.bz * p.zr_mul, zc = w.bz * p.zc_mul;
        if (g_tiles) {
          const int e = min(max(g_tiles[4 * (swap ? tc : tr)], 0), p.g_experts - 1);
          zr = swap ? e : 0;
          zc = swap ? 0 : e;
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          uint8_t* st = smem + stage * C::STAGE_BYTES;
          if (pre > 0) {
            --pre;                               // add the activation tile to the armed stage
            if (swap) tma_load_3d(st + C::A_BYTES * (GLU ? 2 : 1), &tm_c, &full[stage], kb * BK, tc * BN, zc);
            else tma_load_3d(st, &tm_r, &full[stage], kb * BK, tr * BM, zr);
          } else {
            if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
            mbar_expect_tx(&full[stage], C::STAGE_BYTES);
            tma_load_3d(st, &tm_r, &full[stage], kb * BK, tr * BM, zr);
            if (GLU) tma_load_3d(st + C::A_BYTES, &tm_r, &full[stage], kb * BK, p.glu_offset + tr * BM, zr);
            tma_load_3d(st + C::A_BYTES * (GLU ? 2 : 1), &tm_c, &full[stage], kb * BK, tc * BN, zc);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        have = iter.next(w);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = idesc_bf16(BM, BN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      WorkIter<LEAN> iter(p);
      WorkItem w;
      for (; iter.next(w); ++it) {
        const int kb0 = w.kb0, kb1 = w.kb1;
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * C::ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, MARY_ERR_TIMEOUT_TMA)) goto done;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES * (GLU ? 2 : 1);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t db = umma_desc_sw128(sb + k * UMMA_K * 2);
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            umma_f16(d0, umma_desc_sw128(sa + k * UMMA_K * 2), db, idesc, accum);
            if (GLU) umma_f16(d0 + BN, umma_desc_sw128(sa + C::A_BYTES + k * UMMA_K * 2), db, idesc, accum);
          }
          umma_commit(&empty[stage]);      // frees the stage when these MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&acc_full[buf]);       // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    pdl_wait();                            // before the first store: an earlier kernel may still read what this one overwrites
    const int q = warp & 3;                // TMEM lane quarter this warp may access
    int it = 0;
    WorkIter<LEAN> iter(p);
    WorkItem w;
    for (; iter.next(w); ++it) {
      const int bz = w.bz, tc = w.tc, tr = w.tr;
      const int64_t obase = (int64_t)bz * p.out_batch_stride;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag, p.status, MARY_ERR_TIMEOUT_MMA)) goto done;
      tc_fence_after();
      const int i = tr * BM + q * 32 + lane;              // row-operand index of this thread
      const uint32_t taddr = tmem_base + buf * C::ACC_COLS + ((uint32_t)(q * 32) << 16);
      const bool sk_epi = p.epi == EPI_SK_BF16 || p.epi == EPI_SK_F32;
      const int final_epi = LEAN ? (int)EPI_STORE_BF16 : (p.epi == EPI_SK_BF16 ? EPI_STORE_BF16 : (p.epi == EPI_SK_F32 ? EPI_STORE_F32 : p.epi));
      const bool sk = sk_epi && w.nseg > 1;             // a tile computed by one CTA alone is stored directly
      const int tile = w.tile;
      float* slot = sk ? p.ws + (int64_t)tile * (BM * BN) : nullptr;      // the tile's f32 accumulator (zero between calls)
      // stores 32 finished values of this thread's row (columns tc * BN + c0 ..) in the requested form
      auto emit = [&](int c0, const float* v, int epi) {
        const int j0 = tc * BN + c0;
        if (swap) {
          // i = output feature, j = token: out[j * ldo + i]; a warp writes 32 consecutive features per token
          if (i < p.rows_r) {
            const float b = p.bias ? p.bias[i] : 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j0 + j < p.rows_c) {
                const int64_t o = obase + (int64_t)(j0 + j) * p.ldo + i;
                if (LEAN || epi == EPI_STORE_BF16) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16(v[j] + b);
                else if (epi == EPI_RS_BF16) rs_row(p, j0 + j)[i] = __float2bfloat16(v[j] + b);
                else if (epi == EPI_STORE_F32) ((float*)p.out)[o] = v[j] + b;
                else atomicAdd((float*)p.out + o, v[j]);
              }
            }
          }
        } else {
          // i = token, j = output feature: out[i * ldo + j]; each thread writes 32 consecutive features
          if (i < p.rows_r) {
            const int64_t o = obase + (int64_t)i * p.ldo + j0;
            if (epi == EPI_STORE_BF16 || epi == EPI_RS_BF16) {
              __nv_bfloat16* dst = epi == EPI_RS_BF16 ? rs_row(p, i) + j0 : (__nv_bfloat16*)p.out + o;
              if (j0 + 32 <= p.rows_c && ((uintptr_t)dst & 15) == 0) {
                uint4 w[4];
                uint32_t* wp = (uint32_t*)w;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float b0 = p.bias ? p.bias[j0 + 2 * j] : 0.f, b1 = p.bias ? p.bias[j0 + 2 * j + 1] : 0.f;
                  __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j] + b0, v[2 * j + 1] + b1);
                  wp[j] = *(uint32_t*)&h;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) ((uint4*)dst)[j] = w[j];
              } else {
                for (int j = 0; j < 32; ++j)
                  if (j0 + j < p.rows_c) dst[j] = __float2bfloat16(v[j] + (p.bias ? p.bias[j0 + j] : 0.f));
              }
            } else if (epi == EPI_STORE_F32) {
              for (int j = 0; j < 32; ++j)
                if (j0 + j < p.rows_c) ((float*)p.out)[o + j] = v[j] + (p.bias ? p.bias[j0 + j] : 0.f);
            } else {
              for (int j = 0; j < 32; ++j)
                if (j0 + j < p.rows_c) atomicAdd((float*)p.out + o + j, v[j]);
            }
          }
        }
      };
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32], r2[32];
        tmem_ld_32x32b_x32(taddr + c0, r);
        if (GLU) tmem_ld_32x32b_x32(taddr + BN + c0, r2);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float a = __uint_as_float(r[j]) * p.alpha;
          v[j] = GLU ? glu_f(p.act, a, __uint_as_float(r2[j]) * p.alpha) : a;
        }
        if (sk) {
          // add this K-slice into the tile's f32 accumulator in scratch (column-major, so a warp's 32 rows are contiguous:
          // acc[(c0 + j) * BM + row]); the additions of the slices run in L2 in parallel
#pragma unroll
          for (int j = 0; j < 32; ++j) atomicAdd(slot + (c0 + j) * BM + q * 32 + lane, v[j]);
        } else {
          emit(c0, v, final_epi);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      if (sk) {
        // publish the partials, count this split in; the split that arrives last owns the tile
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) *sk_last = (atomicAdd(p.counters + tile, 1) == w.nseg - 1) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*sk_last) {
          __threadfence();
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            float v[32];
            float* a = slot + c0 * BM + q * 32 + lane;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __ldcg(a + j * BM);
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(a + j * BM, 0.f);          // the accumulator is left zero for the next call
            emit(c0, v, final_epi);
          }
          if (threadIdx.x == 64) p.counters[tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");      // sk_last is rewritten by the next work item
      }
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

template <int BN, bool GLU, int LEAN = 0>
int launch(const CUtensorMap& tr, const CUtensorMap& tc, const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<BN, GLU, LEAN == 2>;
  static MarySmemSlots smem_set = {};
  if (int rc = mary_ensure_dyn_smem((const void*)gemm_bf16_kernel<BN, GLU, LEAN>, C::SMEM, &smem_set)) return rc;
  int total = p.tiles_r * p.tiles_c * p.split_k * p.batch;
  int grid = total < mary_num_sms() ? total : mary_num_sms();
  if (p.sk_units > 0) grid = (p.tiles_r * p.tiles_c * p.k_blocks + p.sk_units - 1) / p.sk_units;
  MARY_LAUNCH((gemm_bf16_kernel<BN, GLU, LEAN>), grid, NTHREADS, C::SMEM, stream, tr, tc, p);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

}  // namespace

// out[M, N] (bf16, or f32 for epi 1/2) = alpha * X[M, K] * W[N, K]^T (+ bias[N]).
//   glu != 0: W holds [gate (N rows) ; up (N rows)] and out = act(gate) * up, act = glu - 1 (0 GeGLU, 1 SwiGLU, 2 SiTU).
//   epi: 0 store bf16, 1 atomically add f32 into `out` (caller zeroes it; required when split_k > 1), 2 store f32.
//   swap: -1 = choose automatically, 0 = activations are the row operand, 1 = weights are the row operand.
// Leading dimensions are in elements; all of ldx, ldw must be multiples of 8 and the bases 16-byte aligned.
static int make_tmap_3d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint64_t batch,
                        uint64_t batch_stride, uint32_t box_rows) {
  PFN_encodeTiled enc = mary_encode_fn();
  if (!enc) return MARY_ERR_CUDA;
  if (batch <= 1) { batch = 1; batch_stride = rows * ld; if (batch_stride & 7) batch_stride = (batch_stride + 7) & ~7ull; }
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld * 2, batch_stride * 2};
  cuuint32_t box[3] = {(cuuint32_t)BK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if (((uintptr_t)base & 15) || (strides[0] & 15) || (strides[1] & 15)) return MARY_ERR_BAD_ARG;
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MARY_OK : MARY_ERR_CUDA;
}

// Batched form: `batch` independent problems; operand b starts at base + b * batch_stride (elements).
static thread_local int g_static_weights = 0;
// decode-shaped launches take the short pipeline (two CTAs per SM): on when the environment says MARY_GEMM_SHORT=1
static int short_pipeline_default() {
  const char* e = getenv("MARY_GEMM_SHORT");
  return (e && e[0] == '1') ? 1 : 0;
}
static int g_short_pipeline = short_pipeline_default();

static int gemm_impl(const void* X, const void* W, void* out, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int batch,
                     int64_t bsx, int64_t bsw, int64_t bso, const float* bias, float alpha, int glu, int epi, int split_k, int swap,
                     const uint64_t* rs_bufs, int rs_world, int rs_src, int rs_rpr, cudaStream_t stream, float* ws = nullptr,
                     int64_t ws_floats = 0, int* counters = nullptr, int n_counters = 0, bool stream_k = false,
                     const int* g_tiles = nullptr, const int* g_meta = nullptr, int g_experts = 0, int g_nt = 0);

// Tells the GEMM launchers called next on THIS thread that their W operand holds constant model weights (1) or may have been
// written by an earlier kernel of the stream (0, the default).  Only read when programmatic dependent launch is enabled.
MARY_API void mary_gemm_hint_static_weights(int on) { g_static_weights = on ? 1 : 0; }
MARY_API void mary_gemm_short_pipeline(int on) { g_short_pipeline = on ? 1 : 0; }

MARY_API int mary_gemm_bf16_batched(const void* X, const void* W, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                                    int64_t ldo, int batch, int64_t bsx, int64_t bsw, int64_t bso, const float* bias, float alpha,
                                    int glu, int epi, int split_k, int swap, cudaStream_t stream) {
  return gemm_impl(X, W, out, M, N, K, ldx, ldw, ldo, batch, bsx, bsw, bso, bias, alpha, glu, epi, split_k, swap, nullptr, 0, 0, 0, stream);
}

// Row-parallel GEMM fused with the reduce-scatter transfer: this rank's partial out[M, N] is not stored locally; row t goes
// straight from the epilogue into the staging buffer of the rank that owns token t (rows_per_rank tokens per rank), slot
// `src_rank`, over NVLink peer stores — tile by tile while the next tile's main loop runs.  rs_bufs[r] = address of rank r's
// staging buffer [world][rows_per_rank][ldo] bf16.  The owner sums the `world` slots in a fixed order (comm.cu).
MARY_API int mary_gemm_bf16_rs(const void* X, const void* W, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo,
                               const uint64_t* rs_bufs, int world, int src_rank, int rows_per_rank, int swap, cudaStream_t stream) {
  if (world < 1 || world > 8 || rows_per_rank * world < M) return MARY_ERR_BAD_ARG;
  return gemm_impl(X, W, nullptr, M, N, K, ldx, ldw, ldo, 1, 0, 0, 0, nullptr, 1.0f, 0, EPI_RS_BF16, 1, swap, rs_bufs, world, src_rank,
                   rows_per_rank, stream);
}

static int gemm_impl(const void* X, const void* W, void* out, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int batch,
                     int64_t bsx, int64_t bsw, int64_t bso, const float* bias, float alpha, int glu, int epi, int split_k, int swap,
                     const uint64_t* rs_bufs, int rs_world, int rs_src, int rs_rpr, cudaStream_t stream, float* ws, int64_t ws_floats,
                     int* counters, int n_counters, bool stream_k, const int* g_tiles, const int* g_meta, int g_experts, int g_nt) {
  if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || batch < 1) return MARY_ERR_BAD_ARG;
  if (split_k < 1) split_k = 1;
  const bool sk_epi = epi == EPI_SK_BF16 || epi == EPI_SK_F32;
  if (split_k > 1 && epi != EPI_RED_F32 && !sk_epi) return MARY_ERR_BAD_ARG;
  if (sk_epi && (glu || !ws || !counters)) return MARY_ERR_BAD_ARG;
  if (glu && epi == EPI_RED_F32) return MARY_ERR_BAD_ARG;
  const bool use_swap = glu ? true : (swap < 0 ? (M <= 256) : swap != 0);
  // GLU without swap would need the weight operand on the column side; for large M the host falls back to
  // a plain GEMM followed by the GLU kernel, so here GLU implies swap.
  GemmParams p;
  p.K = K;
  p.k_blocks = (K + BK - 1) / BK;
  if (split_k > p.k_blocks) split_k = p.k_blocks;
  p.k_blocks_per_split = (p.k_blocks + split_k - 1) / split_k;
  p.split_k = (p.k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
  p.glu_offset = N;
  p.act = glu ? glu - 1 : 0;
  p.epi = epi;
  p.swap = use_swap ? 1 : 0;
  p.ldo = ldo;
  p.batch = batch;
  p.out_batch_stride = bso;
  p.out = out;
  for (int i = 0; i < 8; ++i) p.rs_bufs[i] = (rs_bufs && i < rs_world) ? rs_bufs[i] : 0;
  p.rs_rpr = rs_rpr > 0 ? rs_rpr : 1;
  p.rs_src = rs_src;
  p.bias = bias;
  p.alpha = alpha;
  p.status = mary_status_ptr();
  const void *R = use_swap ? W : X, *Cc = use_swap ? X : W;
  const int64_t ldr = use_swap ? ldw : ldx, ldc = use_swap ? ldx : ldw;
  const int64_t bsr = use_swap ? bsw : bsx, bsc = use_swap ? bsx : bsw;
  p.rows_r = use_swap ? N : M;
  p.rows_c = use_swap ? M : N;
  const int rows_r_total = use_swap ? (glu ? 2 * N : N) : M;
  int bn;
  p.tiles_r = (p.rows_r + BM - 1) / BM;
  if (glu) bn = p.rows_c <= 32 ? 32 : (p.rows_c <= 64 ? 64 : 128);
  else if (use_swap) bn = p.rows_c <= 32 ? 32 : (p.rows_c <= 64 ? 64 : (p.rows_c <= 128 ? 128 : 256));
  else {
    // activations are the row operand: take the widest column tile that still gives every SM a tile
    const int sms = mary_num_sms();
    bn = 256;
    while (bn > 64 && (int64_t)p.tiles_r * ((p.rows_c + bn - 1) / bn) * split_k * batch < sms) bn >>= 1;
    if (bn == 256 && split_k == 1 && !sk_epi && !g_tiles && batch == 1) {
      // wave quantisation: the tiles run in waves of one per SM, and a last wave that is a quarter full costs a whole wave (480
      // tiles of 128 x 256 on 148 SMs are 3.24 waves = 4).  A slightly narrower tile can end closer to a full wave: take the width
      // whose waves x width (the time of the slowest SM) is smallest; the narrower widths pay a little per tile, hence the margin.
      int64_t best = 0;
      for (int cand : {256, 224, 192}) {
        const int64_t tiles = (int64_t)p.tiles_r * ((p.rows_c + cand - 1) / cand);
        const int64_t cost = ((tiles + sms - 1) / sms) * cand * (cand == 256 ? 100 : 103);
        if (best == 0 || cost < best) { best = cost; bn = cand; }
      }
    }
  }
  p.tiles_c = (p.rows_c + bn - 1) / bn;
  p.ws = ws;
  p.counters = counters;
  p.sk_units = 0;
  p.g_tiles = g_tiles;
  p.g_meta = g_meta;
  p.g_experts = g_experts;
  p.w_static = (g_static_weights && mary_pdl_enabled() && !g_tiles && !(glu && !use_swap)) ? 1 : 0;
  p.raster = (!g_tiles && p.split_k == 1 && !sk_epi && p.tiles_c >= 16 && p.tiles_r >= 4) ? 8 : 0;
  if (g_tiles) {
    if (batch != 1 || split_k != 1) return MARY_ERR_BAD_ARG;
    if (use_swap) {
      if ((g_nt != 32 && g_nt != 64 && g_nt != 128) || p.rows_c % g_nt) return MARY_ERR_BAD_ARG;
      bn = g_nt;                                  // one column tile = one tile of the routing plan
      p.tiles_c = p.rows_c / bn;
    } else {
      if (g_nt != BM || p.rows_r % BM) return MARY_ERR_BAD_ARG;       // one 128-row tile = one tile of the routing plan
      bn = p.rows_c >= 256 ? 256 : (p.rows_c > 64 ? 128 : 64);
      p.tiles_c = (p.rows_c + bn - 1) / bn;
    }
  }
  if (sk_epi) {
    const int64_t tiles = (int64_t)p.tiles_r * p.tiles_c * batch;
    const int64_t slots = tiles;                 // one f32 accumulator tile per output tile
    if (stream_k && batch == 1) {
      // equal runs of K-blocks per CTA; at least 4 blocks each so that the partial-tile traffic stays small beside the weights
      const int64_t units = tiles * p.k_blocks;
      int64_t g = mary_num_sms();
      if (g > units / 4) g = units / 4 > 0 ? units / 4 : 1;
      p.sk_units = (int)((units + g - 1) / g);
      // at most 16 slices per tile: bounds the contention on one accumulator tile
      if (p.sk_units < (p.k_blocks + 15) / 16) p.sk_units = (p.k_blocks + 15) / 16;
      p.split_k = 1;
    }
    if (tiles > n_counters || slots * BM * bn > ws_floats) return MARY_ERR_BAD_ARG;     // workspace too small
  }
  CUtensorMap tr, tc;
  const bool r_shared = batch > 1 && bsr == 0 && !g_tiles, c_shared = batch > 1 && bsc == 0 && !g_tiles;
  p.zr_mul = r_shared ? 0 : 1;
  p.zc_mul = c_shared ? 0 : 1;
  int rc = make_tmap_3d(&tr, R, rows_r_total, K, ldr, (g_tiles && use_swap) ? g_experts : (r_shared ? 1 : batch), bsr, BM);
  if (rc) return rc;
  rc = make_tmap_3d(&tc, Cc, p.rows_c, K, ldc, (g_tiles && !use_swap) ? g_experts : (c_shared ? 1 : batch), bsc, bn);
  if (rc) return rc;
  // decode-shaped launches (see WorkIter): the instantiation without the other paths' code
  const bool lean = use_swap && !g_tiles && p.raster == 0 && (epi == EPI_STORE_BF16 || epi == EPI_SK_BF16) && bn <= 128;
  if (lean) {
    if (glu) {
      switch (bn) {
        case 32: return launch<32, true, 1>(tr, tc, p, stream);
        case 64: return launch<64, true, 1>(tr, tc, p, stream);
        default: return launch<128, true, 1>(tr, tc, p, stream);
      }
    }
    if (g_short_pipeline) {
      switch (bn) {
        case 32: return launch<32, false, 2>(tr, tc, p, stream);
        case 64: return launch<64, false, 2>(tr, tc, p, stream);
        default: return launch<128, false, 2>(tr, tc, p, stream);
      }
    }
    switch (bn) {
      case 32: return launch<32, false, 1>(tr, tc, p, stream);
      case 64: return launch<64, false, 1>(tr, tc, p, stream);
      default: return launch<128, false, 1>(tr, tc, p, stream);
    }
  }
  if (glu) {
    switch (bn) {
      case 32: return launch<32, true>(tr, tc, p, stream);
      case 64: return launch<64, true>(tr, tc, p, stream);
      default: return launch<128, true>(tr, tc, p, stream);
    }
  }
  switch (bn) {
    case 32: return launch<32, false>(tr, tc, p, stream);
    case 64: return launch<64, false>(tr, tc, p, stream);
    case 128: return launch<128, false>(tr, tc, p, stream);
    case 192: return launch<192, false>(tr, tc, p, stream);
    case 224: return launch<224, false>(tr, tc, p, stream);
    default: return launch<256, false>(tr, tc, p, stream);
  }
}

MARY_API int mary_gemm_bf16(const void* X, const void* W, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                            int64_t ldo, const float* bias, float alpha, int glu, int epi, int split_k, int swap,
                            cudaStream_t stream) {
  return mary_gemm_bf16_batched(X, W, out, M, N, K, ldx, ldw, ldo, 1, 0, 0, 0, bias, alpha, glu, epi, split_k, swap, stream);
}

// Grouped (mixture-of-experts) GEMM with unquantised expert weights: out[rows_pad, N] = X[rows_pad, K] * W[expert of the row's tile]^T,
// optionally with the GLU epilogue (W[e] = [gate; up], 2 N rows).  X holds the routing plan's padded rows (tiles of `nt` = 32, 64 or
// 128 rows, one expert each); `tiles` / `meta` are the plan's tile table and {tiles in use, padded rows}; W is [E][N or 2 N][K] with
// `bsw` elements between experts.  Tiles the plan does not use are skipped.
// `swap` = 1: weights are the 128-row operand, token tiles of nt = 32 / 64 / 128 columns (decode; GLU allowed).  `swap` = 0: tokens are the
// 128-row operand (nt must be 128), the expert's weights the column operand (prefill-sized batches; no GLU epilogue).
MARY_API int mary_gemm_bf16_grouped(const void* X, const void* W, void* out, int rows_pad, int N, int K, int64_t ldx, int64_t ldw,
                                    int64_t ldo, int E, int64_t bsw, const int* tiles, const int* meta, int nt, int glu, int swap,
                                    cudaStream_t stream) {
  if (!tiles || !meta || E < 1 || (glu && !swap)) return MARY_ERR_BAD_ARG;
  return gemm_impl(X, W, out, rows_pad, N, K, ldx, ldw, ldo, 1, 0, bsw, 0, nullptr, 1.0f, glu, EPI_STORE_BF16, 1, swap ? 1 : 0, nullptr, 0, 0, 0,
                   stream, nullptr, 0, nullptr, 0, false, tiles, meta, E, nt);
}

// Split-K finished inside the kernel, without a zero-fill or a cast pass: out (bf16, or f32 when out_f32) = alpha * X W^T + bias
// with K cut into slices that run as separate CTAs.  `ws` (ws_floats f32, ZERO before the first call; the kernel leaves it zero)
// holds one f32 accumulator tile per output tile and `counters` (n_counters ints, zero likewise) one arrival count per tile; both
// are scratch that calls on one stream may share.  Returns MARY_ERR_BAD_ARG when the scratch is too small for this shape.
MARY_API int mary_gemm_bf16_splitk(const void* X, const void* W, void* out, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo,
                                   const float* bias, float alpha, int out_f32, int split_k, int swap, float* ws, int64_t ws_floats,
                                   int* counters, int n_counters, cudaStream_t stream) {
  // split_k == 0: stream-K (equal runs of K-blocks per CTA)
  return gemm_impl(X, W, out, M, N, K, ldx, ldw, ldo, 1, 0, 0, 0, bias, alpha, 0, out_f32 ? EPI_SK_F32 : EPI_SK_BF16,
                   split_k == 0 ? 1 : split_k, swap, nullptr, 0, 0, 0, stream, ws, ws_floats, counters, n_counters, split_k == 0);
}
