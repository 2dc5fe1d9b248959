// Collectives over peer memory (NVLink 5 / NVSwitch) written as ordinary kernels.
//
// The reference has no collective backend: its one multi-device mode is a two-stage layer pipeline over a TCP socket
// (src/bin/inkling_forward.rs:1192-1271) and NCCL appears only in a probe script (scripts/interconnect_probe.sh:57-126).
// Here every rank owns a buffer in a symmetric allocation (same size on every rank, all peers' base addresses known)
// plus a small pad of 32-bit flags.  Kernels read and write the peers' buffers directly (P2P ld/st), or through the
// multicast address of the allocation when the switch supports it: `multimem.ld_reduce` returns the sum over all ranks
// computed inside NVSwitch, `multimem.st` writes to all ranks at once.
//
// all-reduce (two-shot): rank r owns slice r of the vector.  barrier -> each rank reduces its slice (one in-switch
// reduction per 16 bytes, or P2P loads from every peer) and writes the result into the output region of EVERY rank ->
// barrier.  Each block synchronises with the same-numbered block of the other ranks only, and touches only chunks
// assigned to its block number, so all ranks must launch the same grid.
//
// Flags are monotonic epochs (one value per call); every wait is bounded in time and records
// MARY_ERR_TIMEOUT_PEER in the status word instead of hanging, after which the kernel returns.
#include "common.cuh"
#include "host_utils.h"

using namespace mary;

namespace {

constexpr int MAX_RANKS = 8;

struct CommCtx {
  uint8_t* bufs[MAX_RANKS];     // peers' symmetric buffers (this rank's own at [rank])
  uint32_t* sigs[MAX_RANKS];    // peers' flag pads
  uint8_t* mc;                  // multicast address of the buffer, or null
  int rank, world;
  uint64_t wait_ns;
  int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier between block `blockIdx.x` of every rank.  slot layout: sig[(blockIdx.x * 2 + which) * MAX_RANKS + src].
// Returns false when a peer did not arrive in time.
__device__ bool rank_barrier(const CommCtx& c, int which, uint32_t epoch, int blk) {
  __shared__ int ok_s;
  __syncthreads();                 // all of this block's earlier writes are issued
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    const size_t slot = ((size_t)blk * 2 + which) * MAX_RANKS;
    __threadfence_system();
    st_release_sys(c.sigs[peer] + slot + c.rank, epoch);
    const uint32_t* mine = c.sigs[c.rank] + slot + peer;
    uint64_t t0 = 0;                        // the timer is read only after a run of failed polls, never on the fast path
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 255u) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > c.wait_ns) {
          atomicCAS(c.status, 0, MARY_ERR_TIMEOUT_PEER);
          ok_s = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  return ok_s != 0;
}

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// In-place on the symmetric buffer: input region at in_off, output region at out_off (bytes), n bf16 elements (n % 8 == 0).
// `blk` of `nblk` is this block's index within its rank's grid.
// The epoch of the flags lives in device memory (`epoch_slot`, one word per block, advanced by the block itself), so a
// launch recorded in a CUDA graph uses a fresh epoch at every replay.
// f32 != 0: the elements are 32-bit floats (n % 4 == 0), summed in f32 (gradient buckets).
__device__ void allreduce_bf16_body(const CommCtx& c, size_t in_off, size_t out_off, int64_t n, uint32_t* epoch_slot, int use_mc, int blk,
                                    int nblk, int f32 = 0) {
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) epoch_s = *epoch_slot + 1;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  if (!rank_barrier(c, 0, epoch, blk)) return;
  const int64_t nvec = f32 ? n / 4 : n / 8;                    // 16-byte vectors
  const int64_t per = (nvec + c.world - 1) / c.world;
  const int64_t lo = (int64_t)c.rank * per, hi = min(nvec, lo + per);
  for (int64_t v = lo + (int64_t)blk * blockDim.x + threadIdx.x; v < hi; v += (int64_t)nblk * blockDim.x) {
    uint4 r;
    if (use_mc) {
      r = f32 ? multimem_ld_reduce_f32x4(c.mc + in_off + v * 16) : multimem_ld_reduce_bf16x8(c.mc + in_off + v * 16);
      multimem_st_v4(c.mc + out_off + v * 16, r);
    } else if (f32) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < c.world; ++p) {
        uint4 x;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w) : "l"(c.bufs[p] + in_off + v * 16) : "memory");   // rank order: same sum everywhere
        acc.x += __uint_as_float(x.x); acc.y += __uint_as_float(x.y); acc.z += __uint_as_float(x.z); acc.w += __uint_as_float(x.w);
      }
      r = make_uint4(__float_as_uint(acc.x), __float_as_uint(acc.y), __float_as_uint(acc.z), __float_as_uint(acc.w));
      for (int p = 0; p < c.world; ++p) *(uint4*)(c.bufs[(c.rank + p) % c.world] + out_off + v * 16) = r;
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < c.world; ++p) {
        uint4 x;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w) : "l"(c.bufs[(c.rank + p) % c.world] + in_off + v * 16) : "memory");
        const __nv_bfloat162* xp = (const __nv_bfloat162*)&x;
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(xp[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
      }
      __nv_bfloat162* rp = (__nv_bfloat162*)&r;
#pragma unroll
      for (int j = 0; j < 4; ++j) rp[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      for (int p = 0; p < c.world; ++p) *(uint4*)(c.bufs[(c.rank + p) % c.world] + out_off + v * 16) = r;
    }
  }
  rank_barrier(c, 1, epoch, blk);
  if (threadIdx.x == 0) *epoch_slot = epoch;
}

__global__ void __launch_bounds__(512)
allreduce_bf16_kernel(const CommCtx c, size_t in_off, size_t out_off, int64_t n, uint32_t* epochs, int use_mc, int f32) {
  pdl_sync();
  allreduce_bf16_body(c, in_off, out_off, n, epochs + blockIdx.x, use_mc, blockIdx.x, gridDim.x, f32);
}

// One-shot all-reduce for small vectors (decode-sized partial sums): every rank stages its partial vector in a symmetric
// staging area, ONE barrier makes the stages complete, and every rank then sums the whole vector by itself — one in-switch
// reduction per 16 bytes through the multicast address, or peer loads in rank order — into a LOCAL output.  Nothing a peer
// reads is written again before the next barrier: the staging area alternates with the parity of the device-resident epoch,
// and a rank can only pass the barrier of call k + 1 after every peer has finished reading the stage of call k.  Compared with
// the two-shot form this saves the second barrier and the all-gather step; it moves world x the bytes, which only pays for
// small vectors.
// Block b owns vectors [b * ONESHOT_VECS, (b + 1) * ONESHOT_VECS) of the stage WHATEVER the length of the call, and its
// barrier and epoch are those of block b alone.  The slice must not depend on the call: the parity of block b's epoch only
// protects bytes that no other block number ever writes, and calls of different lengths (different grids) advance the blocks'
// epochs differently.
constexpr int64_t ONESHOT_VECS = 2048;     // 32 KB of the vector per block

__device__ void allreduce_oneshot_body(const CommCtx& c, const uint4* __restrict__ partial, uint4* __restrict__ out, size_t stage_off,
                                       size_t stage_bytes, int64_t nvec, uint32_t* epoch_slot, int use_mc, int blk) {
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) epoch_s = *epoch_slot + 1;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const size_t off = stage_off + (size_t)(epoch & 1u) * stage_bytes;
  const int64_t lo = (int64_t)blk * ONESHOT_VECS, hi = min(nvec, lo + ONESHOT_VECS);
  uint4* mine = (uint4*)(c.bufs[c.rank] + off);
  for (int64_t v = lo + threadIdx.x; v < hi; v += blockDim.x) mine[v] = partial[v];
  if (!rank_barrier(c, 0, epoch, blk)) return;
  for (int64_t v = lo + threadIdx.x; v < hi; v += blockDim.x) {
    uint4 r;
    if (use_mc) {
      r = multimem_ld_reduce_bf16x8(c.mc + off + v * 16);
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < c.world; ++p) {                    // rank order: every rank computes the same bits
        uint4 x;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w) : "l"(c.bufs[p] + off + v * 16) : "memory");
        const __nv_bfloat162* xp = (const __nv_bfloat162*)&x;
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(xp[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
      }
      __nv_bfloat162* rp = (__nv_bfloat162*)&r;
#pragma unroll
      for (int j = 0; j < 4; ++j) rp[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    }
    out[v] = r;
  }
  if (threadIdx.x == 0) *epoch_slot = epoch;
}

__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(const CommCtx c, const uint4* __restrict__ partial, uint4* __restrict__ out, size_t stage_off, size_t stage_bytes,
                         int64_t nvec, uint32_t* epochs, int use_mc) {
  pdl_sync();
  allreduce_oneshot_body(c, partial, out, stage_off, stage_bytes, nvec, epochs + blockIdx.x, use_mc, blockIdx.x);
}

// All ranks of the one-shot form inside ONE cooperative launch on one GPU: blocks [r * nblk, (r + 1) * nblk) play rank r;
// `partial` and `out` hold the ranks' vectors back to back (stride `nvec`), `epochs` holds world x 64 words.
__global__ void __launch_bounds__(512)
allreduce_oneshot_emulated_kernel(CommCtx c, const uint4* __restrict__ partial, uint4* __restrict__ out, size_t stage_off,
                                  size_t stage_bytes, int64_t nvec, uint32_t* epochs, int nblk) {
  c.rank = blockIdx.x / nblk;
  const int blk = blockIdx.x % nblk;
  allreduce_oneshot_body(c, partial + (size_t)c.rank * nvec, out + (size_t)c.rank * nvec, stage_off, stage_bytes, nvec,
                         epochs + c.rank * 64 + blk, 0, blk);
}

// Every rank of the group inside ONE cooperative launch on one GPU (block groups play the ranks, plain loads and stores
// play the peer accesses): the way to exercise the flag protocol and the data movement where only one GPU is available,
// because kernels that wait on one another must never be separate launches on the same GPU.
__global__ void __launch_bounds__(512)
allreduce_bf16_emulated_kernel(CommCtx c, size_t in_off, size_t out_off, int64_t n, uint32_t* epochs, int nblk, int f32) {
  c.rank = blockIdx.x / nblk;
  allreduce_bf16_body(c, in_off, out_off, n, epochs + blockIdx.x, 0, blockIdx.x % nblk, nblk, f32);
}

// Owner side of the reduce-scatter: one CTA per local token row.  Sums the `world` staged partial rows in rank order
// (deterministic) into a = sum, then
//   w_post == nullptr:  h' = h + a                               (pre-norm decoders)
//   w_post != nullptr:  h' = (h + rms(a) * w_post) * scalar      (sandwich norms: the sum is normed before it joins the residual)
// keeps h' in the residual slice (sequence-sharded: every rank holds only its own rows), applies x = rms(h') * w and writes x
// to EVERY rank's activation buffer — the all-gather — with one multimem store per 16 bytes, or peer stores.
// w == nullptr: no final norm, h' itself (or a, without a residual) is broadcast.
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int wi = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[wi] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  return warp_sum(t);
}

__global__ void rs_add_rmsnorm_kernel(const CommCtx c, const __nv_bfloat16* __restrict__ staging, __nv_bfloat16* __restrict__ h_slice,
                                      const __nv_bfloat16* __restrict__ w_post, const __nv_bfloat16* __restrict__ w, float scalar,
                                      size_t x_off, int rpr, int H, float eps, int use_mc) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const int r = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < c.world; ++s) {
      const uint4 v = *(const uint4*)(staging + ((int64_t)s * rpr + r) * H + i);
      const __nv_bfloat162* vp = (const __nv_bfloat162*)&v;
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(vp[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
    if (h_slice && !w_post) {
      uint4 hv = *(const uint4*)(h_slice + (int64_t)r * H + i);
      __nv_bfloat162* hp = (__nv_bfloat162*)&hv;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(hp[j]);
        hp[j] = __floats2bfloat162_rn(f.x + acc[2 * j], f.y + acc[2 * j + 1]);
        float2 b = __bfloat1622float2(hp[j]);
        acc[2 * j] = b.x; acc[2 * j + 1] = b.y;
      }
      *(uint4*)(h_slice + (int64_t)r * H + i) = hv;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { row[i + j] = acc[j]; ss += acc[j] * acc[j]; }
  }
  if (w_post) {
    const float inv_a = rsqrtf(block_sum_256(ss, red) / H + eps);
    ss = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {        // every thread revisits the columns it wrote
      const uint4 pv = *(const uint4*)(w_post + i);
      const __nv_bfloat162* pp = (const __nv_bfloat162*)&pv;
      uint4 hv = make_uint4(0, 0, 0, 0);
      if (h_slice) hv = *(const uint4*)(h_slice + (int64_t)r * H + i);
      __nv_bfloat162* hp = (__nv_bfloat162*)&hv;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(pp[j]);
        const float2 n = __bfloat1622float2(__floats2bfloat162_rn(row[i + 2 * j] * inv_a * g.x, row[i + 2 * j + 1] * inv_a * g.y));
        const float2 f = __bfloat1622float2(hp[j]);
        hp[j] = __floats2bfloat162_rn((f.x + n.x) * scalar, (f.y + n.y) * scalar);
        const float2 b = __bfloat1622float2(hp[j]);
        row[i + 2 * j] = b.x; row[i + 2 * j + 1] = b.y;
        ss += b.x * b.x + b.y * b.y;
      }
      if (h_slice) *(uint4*)(h_slice + (int64_t)r * H + i) = hv;
    }
  }
  float inv = 1.f;
  if (w) inv = rsqrtf(block_sum_256(ss, red) / H + eps);
  const int64_t grow = (int64_t)c.rank * rpr + r;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 o;
    __nv_bfloat162* op = (__nv_bfloat162*)&o;
    uint4 wv = make_uint4(0, 0, 0, 0);
    if (w) wv = *(const uint4*)(w + i);
    const __nv_bfloat162* wp = (const __nv_bfloat162*)&wv;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 g = w ? __bfloat1622float2(wp[j]) : make_float2(1.f, 1.f);
      op[j] = __floats2bfloat162_rn(row[i + 2 * j] * inv * g.x, row[i + 2 * j + 1] * inv * g.y);
    }
    const size_t off = x_off + ((size_t)grow * H + i) * sizeof(__nv_bfloat16);
    if (use_mc) multimem_st_v4(c.mc + off, o);
    else for (int p = 0; p < c.world; ++p) *(uint4*)(c.bufs[(c.rank + p) % c.world] + off) = o;
  }
}

// Cross-rank arg-max merge for a vocabulary-parallel LM head.  Every rank holds, per token, the best (value, index) of its
// own vocabulary shard; it stores the pair into slot [rank] of EVERY rank's pair table (8-byte peer stores), one barrier
// makes the tables complete, and every rank picks the overall winner locally (larger value; equal values -> lower global
// index, which is what one arg-max over the whole vocabulary would return).  The tables are double-buffered by epoch
// parity, so a rank that races ahead into the next call never overwrites pairs a slower rank still reads.
// Table layout at bufs[r] + pair_off: [2][world][Tmax] of uint2 {value bits, global index}.
__device__ void argmax_merge_body(const CommCtx& c, size_t pair_off, int Tmax, const float* __restrict__ val,
                                  const int64_t* __restrict__ idx, int T, int vocab_off, uint32_t* epoch_slot, int slot_block,
                                  int64_t* __restrict__ out_idx, float* __restrict__ out_val) {
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) epoch_s = *epoch_slot + 1;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const size_t par = epoch & 1u;
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    const uint2 pr = make_uint2(__float_as_uint(val[t]), (uint32_t)((int)idx[t] + vocab_off));
    for (int p = 0; p < c.world; ++p)
      *(uint2*)(c.bufs[(c.rank + p) % c.world] + pair_off + ((par * c.world + c.rank) * Tmax + t) * 8) = pr;
  }
  if (!rank_barrier(c, 0, epoch, slot_block)) return;
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    float bv = 0.f;
    uint32_t bi = 0xffffffffu;
    for (int p = 0; p < c.world; ++p) {
      uint2 pr;
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];"
                   : "=r"(pr.x), "=r"(pr.y) : "l"(c.bufs[c.rank] + pair_off + ((par * c.world + p) * Tmax + t) * 8) : "memory");
      const float v = __uint_as_float(pr.x);
      if (bi == 0xffffffffu || v > bv || (v == bv && pr.y < bi)) { bv = v; bi = pr.y; }
    }
    out_idx[t] = (int64_t)bi;
    out_val[t] = bv;
  }
  if (threadIdx.x == 0) *epoch_slot = epoch;
}

__global__ void __launch_bounds__(256)
argmax_merge_kernel(const CommCtx c, size_t pair_off, int Tmax, const float* val, const int64_t* idx, int T, int vocab_off,
                    uint32_t* epoch_slot, int slot_block, int64_t* out_idx, float* out_val) {
  pdl_sync();
  argmax_merge_body(c, pair_off, Tmax, val, idx, T, vocab_off, epoch_slot, slot_block, out_idx, out_val);
}

// All ranks in one cooperative launch on one GPU (block r plays rank r); inputs and outputs are [world][T] arrays.
__global__ void __launch_bounds__(256)
argmax_merge_emulated_kernel(CommCtx c, size_t pair_off, int Tmax, const float* val, const int64_t* idx, int T, int vocab_per_rank,
                             uint32_t* epoch_slots, int slot_block, int64_t* out_idx, float* out_val) {
  c.rank = blockIdx.x;
  argmax_merge_body(c, pair_off, Tmax, val + (size_t)c.rank * T, idx + (size_t)c.rank * T, T, c.rank * vocab_per_rank,
                    epoch_slots + c.rank, slot_block, out_idx + (size_t)c.rank * T, out_val + (size_t)c.rank * T);
}

__global__ void rank_barrier_kernel(const CommCtx c, uint32_t* epoch_slot, int slot_block) {
  pdl_sync();
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) epoch_s = *epoch_slot + 1;
  __syncthreads();
  rank_barrier(c, 0, epoch_s, slot_block);
  if (threadIdx.x == 0) *epoch_slot = epoch_s;
}

// A wait that nothing satisfies (used by the failure-detection test): returns after wait_ns with the status set.
__global__ void wait_flag_kernel(const CommCtx c, uint32_t slot, uint32_t want) {
  const uint32_t* mine = c.sigs[c.rank] + slot;
  const uint64_t t0 = globaltimer_ns();
  while ((int32_t)(ld_acquire_sys(mine) - want) < 0) {
    if (globaltimer_ns() - t0 > c.wait_ns) { atomicCAS(c.status, 0, MARY_ERR_TIMEOUT_PEER); return; }
  }
}

}  // namespace

// bufs / sigs: arrays of `world` device addresses (as integers).  grid blocks x 512 threads; every rank must pass the
// same grid, n and offsets, and make the same sequence of calls.  Flag pad: at least grid * 2 * 8 words, zeroed once at
// set-up; `epochs`: `grid` device words of this rank (zeroed at set-up), advanced by the kernel.
MARY_API int mary_allreduce_bf16(const uint64_t* bufs, const uint64_t* sigs, uint64_t mc, int rank, int world, uint64_t in_off,
                                 uint64_t out_off, int64_t n, uint32_t* epochs, int grid, int use_mc, uint64_t wait_ns, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (in_off % 16) || (out_off % 16) || grid < 1) return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = (uint8_t*)mc; c.rank = rank; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  MARY_LAUNCH(allreduce_bf16_kernel, grid, 512, 0, s, c, in_off, out_off, n, epochs, (use_mc && mc) ? 1 : 0, 0);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// The same two-shot all-reduce over 32-bit floats (n % 4 == 0), summed in f32: gradient buckets of the data-parallel trainer.
MARY_API int mary_allreduce_f32(const uint64_t* bufs, const uint64_t* sigs, uint64_t mc, int rank, int world, uint64_t in_off,
                                uint64_t out_off, int64_t n, uint32_t* epochs, int grid, int use_mc, uint64_t wait_ns, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || (n % 4) || (in_off % 16) || (out_off % 16) || grid < 1) return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = (uint8_t*)mc; c.rank = rank; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  MARY_LAUNCH(allreduce_bf16_kernel, grid, 512, 0, s, c, in_off, out_off, n, epochs, (use_mc && mc) ? 1 : 0, 1);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// Barrier between the ranks as a kernel of its own (one block): everything launched before it on every rank's stream has
// completed and is visible when it returns.  `slot_block` selects the flag slots (use one that no all-reduce grid touches).
MARY_API int mary_rank_barrier(const uint64_t* sigs, int rank, int world, uint32_t* epoch_slot, int slot_block, uint64_t wait_ns, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS) return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = nullptr; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = nullptr; c.rank = rank; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  MARY_LAUNCH(rank_barrier_kernel, 1, 32, 0, s, c, epoch_slot, slot_block);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// staging: this rank's [world][rows_per_rank][H] bf16 (filled by the peers' GEMM epilogues); h_slice: this rank's residual rows
// (updated in place; may be null); w_post: gain of a norm applied to the reduced sum before the residual add (null = none);
// scalar multiplies the new residual (sandwich-norm decoders; 1 otherwise); w: gain of the final norm (null = no norm); the result
// row is written at byte offset x_off + row * H * 2 of EVERY rank's symmetric buffer bufs[r] (multicast when mc != 0).
// H % 8 == 0, H * 4 <= 48 KB.
MARY_API int mary_rs_add_rmsnorm(const void* staging, void* h_slice, const void* w_post, const void* w, float scalar, const uint64_t* bufs,
                                 uint64_t mc, int rank, int world, uint64_t x_off, int rows_per_rank, int H, float eps, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || (H & 7) || (size_t)H * 4 > 48 * 1024 || (x_off & 15)) return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = nullptr; }
  c.mc = (uint8_t*)mc; c.rank = rank; c.world = world; c.wait_ns = 0; c.status = mary_status_ptr();
  rs_add_rmsnorm_kernel<<<rows_per_rank, 256, (size_t)H * 4, s>>>(c, (const __nv_bfloat16*)staging, (__nv_bfloat16*)h_slice,
                                                                 (const __nv_bfloat16*)w_post, (const __nv_bfloat16*)w, scalar, x_off,
                                                                 rows_per_rank, H, eps, mc ? 1 : 0);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// Single-GPU emulation of a `world`-rank all-reduce: bufs / sigs are `world` distinct buffers on the current device.
MARY_API int mary_allreduce_emulated(const uint64_t* bufs, const uint64_t* sigs, int world, uint64_t in_off, uint64_t out_off,
                                     int64_t n, uint32_t* epochs, int grid, uint64_t wait_ns, int f32, cudaStream_t s);
MARY_API int mary_allreduce_bf16_emulated(const uint64_t* bufs, const uint64_t* sigs, int world, uint64_t in_off, uint64_t out_off,
                                          int64_t n, uint32_t* epochs, int grid, uint64_t wait_ns, cudaStream_t s) {
  return mary_allreduce_emulated(bufs, sigs, world, in_off, out_off, n, epochs, grid, wait_ns, 0, s);
}
MARY_API int mary_allreduce_emulated(const uint64_t* bufs, const uint64_t* sigs, int world, uint64_t in_off, uint64_t out_off,
                                     int64_t n, uint32_t* epochs, int grid, uint64_t wait_ns, int f32, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || (n % (f32 ? 4 : 8)) || grid < 1 || grid * world > mary_num_sms()) return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = nullptr; c.rank = 0; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  size_t io = in_off, oo = out_off;
  void* args[] = {&c, &io, &oo, &n, &epochs, &grid, &f32};
  if (cudaLaunchCooperativeKernel((void*)allreduce_bf16_emulated_kernel, dim3(grid * world), dim3(512), args, 0, s) != cudaSuccess)
    return MARY_ERR_CUDA;
  return MARY_OK;
}

MARY_API int mary_wait_flag(const uint64_t* sigs, int rank, int world, uint32_t slot, uint32_t want, uint64_t wait_ns, cudaStream_t s) {
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = nullptr; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = nullptr; c.rank = rank; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  wait_flag_kernel<<<1, 1, 0, s>>>(c, slot, want);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// val / idx: this rank's per-token best logit and LOCAL index within its vocabulary shard (which starts at vocab_off).
// The pair tables need 2 * world * Tmax * 8 bytes at byte offset pair_off (16-byte aligned) of every rank's symmetric
// buffer.  Every rank must make the same sequence of calls with the same T.
MARY_API int mary_argmax_merge(const void* val, const void* idx, int T, int Tmax, int vocab_off, const uint64_t* bufs, const uint64_t* sigs,
                               uint64_t pair_off, int rank, int world, uint32_t* epoch_slot, int slot_block, uint64_t wait_ns,
                               void* out_idx, void* out_val, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || T < 0 || T > Tmax || (pair_off & 15)) return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = nullptr; c.rank = rank; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  MARY_LAUNCH(argmax_merge_kernel, 1, 256, 0, s, c, pair_off, Tmax, (const float*)val, (const int64_t*)idx, T, vocab_off, epoch_slot, slot_block,
                                        (int64_t*)out_idx, (float*)out_val);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

MARY_API int mary_argmax_merge_emulated(const void* val, const void* idx, int T, int Tmax, int vocab_per_rank, const uint64_t* bufs,
                                        const uint64_t* sigs, uint64_t pair_off, int world, uint32_t* epoch_slots, int slot_block,
                                        uint64_t wait_ns, void* out_idx, void* out_val, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || T < 0 || T > Tmax || (pair_off & 15)) return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = nullptr; c.rank = 0; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  size_t po = pair_off;
  void* args[] = {&c, &po, &Tmax, &val, &idx, &T, &vocab_per_rank, &epoch_slots, &slot_block, &out_idx, &out_val};
  if (cudaLaunchCooperativeKernel((void*)argmax_merge_emulated_kernel, dim3(world), dim3(256), args, 0, s) != cudaSuccess)
    return MARY_ERR_CUDA;
  return MARY_OK;
}

// One-shot form for small vectors: partial (this rank's n bf16, 16-byte aligned, any device memory) -> out (local, n bf16).
// The symmetric buffers need two staging areas of stage_bytes >= n * 2 each at byte offset stage_off.  Block b reduces the
// fixed slice of 2048 16-byte vectors number b, so grid must be ceil(n / 8 / 2048) (at most 64); the same flag pad and epochs
// array as mary_allreduce_bf16 (both forms, and calls of different lengths, may be mixed as long as all ranks make the same calls).
MARY_API int mary_allreduce_bf16_oneshot(const void* partial, void* out, const uint64_t* bufs, const uint64_t* sigs, uint64_t mc, int rank,
                                         int world, uint64_t stage_off, uint64_t stage_bytes, int64_t n, uint32_t* epochs, int grid,
                                         int use_mc, uint64_t wait_ns, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (stage_off % 16) || (stage_bytes % 16) || (uint64_t)n * 2 > stage_bytes || grid < 1 ||
      grid > 64 || (int64_t)grid * ONESHOT_VECS < n / 8 || ((uintptr_t)partial & 15) || ((uintptr_t)out & 15))
    return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = (uint8_t*)mc; c.rank = rank; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  MARY_LAUNCH(allreduce_oneshot_kernel, grid, 512, 0, s, c, (const uint4*)partial, (uint4*)out, (size_t)stage_off, (size_t)stage_bytes,
              n / 8, epochs, (use_mc && mc) ? 1 : 0);
  MARY_CHECK_LAUNCH();
  return MARY_OK;
}

// Single-GPU emulation of the one-shot form: `world` ranks as block groups of one cooperative launch.  partial / out hold the
// ranks' vectors back to back ([world][n] bf16); epochs: world * 64 words (zeroed at set-up); grid = blocks PER RANK.
MARY_API int mary_allreduce_bf16_oneshot_emulated(const void* partial, void* out, const uint64_t* bufs, const uint64_t* sigs, int world,
                                                  uint64_t stage_off, uint64_t stage_bytes, int64_t n, uint32_t* epochs, int grid,
                                                  uint64_t wait_ns, cudaStream_t s) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (stage_off % 16) || (stage_bytes % 16) || (uint64_t)n * 2 > stage_bytes || grid < 1 ||
      grid > 64 || (int64_t)grid * ONESHOT_VECS < n / 8 || grid * world > mary_num_sms())
    return MARY_ERR_BAD_ARG;
  CommCtx c;
  for (int i = 0; i < world; ++i) { c.bufs[i] = (uint8_t*)bufs[i]; c.sigs[i] = (uint32_t*)sigs[i]; }
  c.mc = nullptr; c.rank = 0; c.world = world; c.wait_ns = wait_ns; c.status = mary_status_ptr();
  size_t so = stage_off, sb = stage_bytes;
  int64_t nvec = n / 8;
  void* args[] = {&c, &partial, &out, &so, &sb, &nvec, &epochs, &grid};
  if (cudaLaunchCooperativeKernel((void*)allreduce_oneshot_emulated_kernel, dim3(grid * world), dim3(512), args, 0, s) != cudaSuccess)
    return MARY_ERR_CUDA;
  return MARY_OK;
}
