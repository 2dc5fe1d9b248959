// Expert-parallel all-to-all for MoE layers whose tokens live on their home rank (data-parallel attention):
// dispatch = route, NVFP4-quantise and write every (token, expert) row straight into the receive slab of the rank that
// owns the expert; combine = the w2 expert GEMM's epilogue writes every output row straight back into the home rank's
// buffer (see row_ptrs in gemm_nvfp4.cu), where a weighted sum in fixed slot order finishes the layer.
//
// All transfers are plain peer stores issued by these kernels (NVLink through NVSwitch); there is no staging copy and no
// library collective.  Phases are separated by the rank barrier of comm.cu (a one-block kernel), never by waits inside
// these kernels, so on a single GPU the same code can be driven rank after rank for testing.
//
//   1. ep_counts      every rank counts its entries per GLOBAL expert and stores the vector into row `rank` of the count
//                     matrix of EVERY rank                                                        -> barrier
//   2. ep_plan        every rank derives, from the same matrix: the padded row offsets and the tile list of its own experts
//                     (rows of one expert are ordered by source rank), and for every global expert the first row its own
//                     entries occupy on the owner
//   3. ep_dispatch    one CTA per entry: quantise the token row (same rules as quant_nvfp4_rows) and store codes, scales (in
//                     the tensor-core tile layout) and the return address of the row into the owner's slabs -> barrier
//   4. grouped GEMMs  w13 (+GLU) -> re-quantise -> w2 with row_ptrs built by ep_return_ptrs            -> barrier
//   5. un-permute     out[t] = sum_j w[t, j] * comb[t * k + j]  (moe_unpermute with an identity row map)
// Row order: inside one expert's block of the owner's slab the rows of one source rank are handed out by an atomic counter
// (ep_dispatch: send_cnt), so WHICH padded row a token lands in differs from run to run.  The layer's output does not depend
// on it (every row of the grouped GEMMs is independent and the home rank sums a token's k results in fixed slot order); a
// combine that added rows in arrival order, or a row-by-row dump of the slabs, would inherit the nondeterminism.
// The reference has no expert parallelism at all (experts are per-node residents of a layer range,
// src/bin/inkling_forward.rs:2103-2438); this is new.
#include <cuda_fp8.h>

#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int MAX_RANKS = 8;
struct Tile { int expert, row0, rows, sf_tile; };

struct Peers {
  uint64_t p[MAX_RANKS];
};

__global__ void ep_counts_kernel(const int* __restrict__ idx, int n_entries, int E, int rank, Peers count_mats) {
  pdl_sync();
  extern __shared__ int cnt[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_entries; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  for (int r = 0; r < MAX_RANKS; ++r) {
    if (!count_mats.p[r]) continue;
    int* dst = (int*)count_mats.p[r] + (int64_t)rank * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = cnt[e];
  }
}

// cm[world][E] (local copy of the count matrix).  Outputs for this rank: tiles / meta {n_tiles, padded rows} of its own
// experts, send_base[E] = first row of this rank's entries of global expert e on the owner, send_cnt[E] zeroed.
// shared_rows > 0: this rank also runs a shared expert (local expert index e_local, "global" id E) over that many of its own rows;
// they are placed behind the received rows (send_base[E]), never leave the rank, and get their own tiles.
__global__ void ep_plan_kernel(const int* __restrict__ cm, int world, int rank, int E, int e_local, int NT, Tile* __restrict__ tiles,
                               int* __restrict__ meta, int* __restrict__ send_base, int* __restrict__ send_cnt, int* __restrict__ recv_src_off,
                               int shared_rows) {
  pdl_sync();
  extern __shared__ int sh[];
  __shared__ int acc_self;
  int* tot = sh;            // [E] rows of every expert over all sources
  int* off = sh + E;        // [E] padded first row of the expert on its owner
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += cm[s * E + e];
    tot[e] = t;
    send_cnt[e] = 0;
  }
  __syncthreads();
  if (threadIdx.x < world) {                         // one thread per owner rank: padded prefix over its experts
    const int d = threadIdx.x;
    int acc = 0;
    for (int j = 0; j < e_local; ++j) { const int e = d * e_local + j; off[e] = acc; acc += (tot[e] + NT - 1) / NT * NT; }
    if (d == rank) {
      acc_self = acc;
      const int sp = (shared_rows + NT - 1) / NT * NT;
      meta[0] = (acc + sp) / NT;
      meta[1] = acc + sp;
      if (shared_rows > 0) { send_base[E] = acc; send_cnt[E] = 0; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i * NT < shared_rows; i += blockDim.x)
    tiles[acc_self / NT + i] = Tile{e_local, acc_self + i * NT, min(NT, shared_rows - i * NT), acc_self / NT + i};
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < rank; ++s) before += cm[s * E + e];
    send_base[e] = off[e] + before;
  }
  for (int j = threadIdx.x; j < e_local; j += blockDim.x) {
    const int e = rank * e_local + j;
    const int c = tot[e];
    for (int i = 0; i * NT < c; ++i) tiles[off[e] / NT + i] = Tile{j, off[e] + i * NT, min(NT, c - i * NT), off[e] / NT + i};
    if (recv_src_off) recv_src_off[j] = off[e];
  }
}

__device__ __forceinline__ uint32_t e2m1_code(float y) {
  const float m = fabsf(y);
  uint32_t c = (m >= 0.25f) + (m >= 0.75f) + (m >= 1.25f) + (m >= 1.75f) + (m >= 2.5f) + (m >= 3.5f) + (m >= 5.0f);
  return c | (signbit(y) ? 8u : 0u);
}

// One CTA per entry i = t * k + j.
__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const int* __restrict__ idx, int k, int E, int e_local,
                                   int Kd, int NT, int rank, int entry_stride, int cap_rows, const int* __restrict__ send_base,
                                   int* __restrict__ send_cnt, Peers xq_slabs, Peers sf_slabs, Peers meta_slabs, int* __restrict__ status) {
  pdl_sync();
  __shared__ int s_row;
  const int i = blockIdx.x;
  const int e = idx[i];
  if (e < 0 || e > E) return;                    // e == E: the shared expert, served on this rank
  if (threadIdx.x == 0) s_row = send_base[e] + atomicAdd(&send_cnt[e], 1);
  __syncthreads();
  const int row = s_row, d = (e == E) ? rank : e / e_local;
  if (row < 0 || row >= cap_rows) {              // never store outside the owner's slabs: record it and drop the row
    if (threadIdx.x == 0) atomicCAS(status, 0, MARY_ERR_BOUNDS);
    return;
  }
  uint8_t* xq = (uint8_t*)xq_slabs.p[d];
  uint8_t* sf = (uint8_t*)sf_slabs.p[d];
  if (threadIdx.x == 0) ((int*)meta_slabs.p[d])[row] = rank * entry_stride + i;
  const __nv_bfloat16* xr = x + (int64_t)(i / k) * ldx;
  const int tile = row / NT, r = row % NT;
  const int64_t sf_base = (int64_t)tile * (Kd / 64) * 512 + (r % 32) * 16 + (r / 32) * 4;
  for (int b = threadIdx.x; b < Kd / 16; b += blockDim.x) {
    const uint4 v0 = *(const uint4*)(xr + b * 16), v1 = *(const uint4*)(xr + b * 16 + 8);
    float f[16];
    const __nv_bfloat162* p0 = (const __nv_bfloat162*)&v0;
    const __nv_bfloat162* p1 = (const __nv_bfloat162*)&v1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = __bfloat1622float2(p0[j]), c = __bfloat1622float2(p1[j]);
      f[2 * j] = a.x; f[2 * j + 1] = a.y; f[8 + 2 * j] = c.x; f[8 + 2 * j + 1] = c.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
    const float sfv = fminf(__fdiv_rn(amax, 6.0f), 448.0f);
    const __nv_fp8_storage_t sb = __nv_cvt_float_to_fp8(sfv, __NV_SATFINITE, __NV_E4M3);
    const float s = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
    uint32_t lo = 0, hi = 0;
    if (s > 0.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { lo |= e2m1_code(__fdiv_rn(f[j], s)) << (4 * j); hi |= e2m1_code(__fdiv_rn(f[8 + j], s)) << (4 * j); }
    }
    *(uint2*)(xq + (int64_t)row * (Kd / 2) + b * 8) = make_uint2(lo, hi);
    sf[sf_base + (int64_t)(b / 4) * 512 + (b % 4)] = (uint8_t)sb;
  }
}

// row_ptrs[row] = address of slot `entry` in the combine buffer of the row's source rank (0 for padding rows).
__global__ void ep_return_ptrs_kernel(const int* __restrict__ meta_rows, const int* __restrict__ plan_meta, const Tile* __restrict__ tiles,
                                      int NT, int entry_stride, int H, Peers comb, uint64_t* __restrict__ row_ptrs) {
  pdl_sync();
  const int t = blockIdx.x;
  if (t >= plan_meta[0]) return;
  const Tile tl = tiles[t];
  for (int j = threadIdx.x; j < NT; j += blockDim.x) {
    const int row = tl.row0 + j;
    uint64_t ptr = 0;
    if (j < tl.rows) {
      const int m = meta_rows[row];
      const int src = m / entry_stride, entry = m % entry_stride;
      ptr = comb.p[src] + (uint64_t)entry * H * sizeof(__nv_bfloat16);
    }
    row_ptrs[row] = ptr;
  }
}

Peers make_peers(const uint64_t* a, int world) {
  Peers p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < world ? a[i] : 0;
  return p;
}

}  // namespace

MARY_API int mary_ep_counts(const int* idx, int n_entries, int E, int rank, int world, const uint64_t* count_mats, cudaStream_t s) {
  if (E > 8192 || world > MAX_RANKS) return MARY_ERR_BAD_ARG;
  MARY_LAUNCH(ep_counts_kernel, 1, 1024, E * sizeof(int), s, idx, n_entries, E, rank, make_peers(count_mats, world));
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// send_base / send_cnt hold E + 1 entries (the last one for the shared expert's rows when shared_rows > 0).
MARY_API int mary_ep_plan(const int* cm, int world, int rank, int E, int e_local, int NT, void* tiles, int* meta, int* send_base,
                          int* send_cnt, int shared_rows, cudaStream_t s) {
  if (E > 4096 || world > MAX_RANKS || e_local * world != E || shared_rows < 0) return MARY_ERR_BAD_ARG;
  MARY_LAUNCH(ep_plan_kernel, 1, 1024, 2 * E * sizeof(int), s, cm, world, rank, E, e_local, NT, (Tile*)tiles, meta, send_base, send_cnt, nullptr,
                                                      shared_rows);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_ep_dispatch(const void* x, int64_t ldx, const int* idx, int n_entries, int k, int E, int e_local, int K, int NT, int rank,
                              int world, int entry_stride, int cap_rows, const int* send_base, int* send_cnt, const uint64_t* xq_slabs,
                              const uint64_t* sf_slabs, const uint64_t* meta_slabs, cudaStream_t s) {
  if (n_entries <= 0) return MARY_OK;
  if ((K % 64) || (ldx % 8) || world > MAX_RANKS || n_entries > entry_stride) return MARY_ERR_BAD_ARG;
  const int threads = K / 16 < 256 ? ((K / 16 + 31) / 32 * 32) : 256;
  MARY_LAUNCH(ep_dispatch_kernel, n_entries, threads, 0, s, (const __nv_bfloat16*)x, ldx, idx, k, E, e_local, K, NT, rank, entry_stride, cap_rows, send_base,
                                                  send_cnt, make_peers(xq_slabs, world), make_peers(sf_slabs, world),
                                                  make_peers(meta_slabs, world), mary_status_ptr());
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_ep_return_ptrs(const int* meta_rows, const int* plan_meta, const void* tiles, int max_tiles, int NT, int entry_stride,
                                 int H, int world, const uint64_t* comb, uint64_t* row_ptrs, cudaStream_t s) {
  if (max_tiles <= 0) return MARY_OK;
  MARY_LAUNCH(ep_return_ptrs_kernel, max_tiles, 32, 0, s, meta_rows, plan_meta, (const Tile*)tiles, NT, entry_stride, H, make_peers(comb, world), row_ptrs);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}
