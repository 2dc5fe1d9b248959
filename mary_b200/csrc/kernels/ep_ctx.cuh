// Shared state of the fused expert pipeline (ep_fused.cu, gemm_nvfp4.cu): one MoE layer is four launches that hand work to
// one another through counters and flags in peer memory instead of through barrier kernels and a planning pass.
//
//   A  route + dispatch   (home rank, one CTA per token): router top-k, then for every (token, expert) entry one remote
//                         atomic on the OWNER's per-expert arrival counter reserves a row of that expert's fixed slab region;
//                         the token row is NVFP4-quantised once and its codes, scale bytes and return address are stored
//                         into every owner's slabs (peer stores).  The last CTA publishes "rank r has dispatched" to all owners.
//   D  w13 grouped GEMM   (owner): waits (bounded) for the dispatch flags of all sources, reads the arrival counters, builds
//                         its tile list in shared memory, runs the GLU GEMM and writes the intermediate already quantised.
//   E  w2 grouped GEMM    (owner): same tile list; the epilogue stores every output row into the combine buffer of the row's
//                         home rank (address from the row's return word).  The last CTA zeroes the counters and publishes
//                         "owner o has returned" to all home ranks.
//   F  combine            (home rank): waits (bounded) for the return flags, sums the k slots of every token in slot order
//                         with the routing weights, and optionally adds the residual and applies the next RMSNorm.
//
// Slab layout on an owner: local expert j owns rows [j * cap_e, (j + 1) * cap_e) (cap_e a multiple of the tile width and
// >= world * t_cap, the worst case), so no rank needs the others' counts before it writes.  The order of rows inside an
// expert is the arrival order of the atomics and differs from run to run; results do not depend on it (GEMM rows are
// independent, the combine sums in slot order at home).
//
// Flags are monotonic epochs: every kernel of a layer call targets *epoch + 1, and F's last CTA advances the word, so launches
// recorded in a CUDA graph use a fresh epoch at every replay.  Why no flag can be overtaken: a rank dispatches layer L + 1
// only after its own F of layer L, which needs the return flag of EVERY owner, which an owner publishes after its w2 GEMM
// has finished reading the slabs and has zeroed its counters.
// With `local_only` the same four launches serve one rank by itself (tokens replicated or a single GPU): entries of experts
// that live elsewhere are dropped at dispatch, every "peer" is the rank itself, and nothing waits on another GPU.
// The reference plans on the host after a blocking readback per layer (src/bin/inkling_forward.rs:4442-4478, planner
// src/models/inkling/moegroup.rs:978-1083); it has no expert parallelism.
#pragma once
#include "common.cuh"

namespace mary {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_MAX_TILES = 512;       // token tiles one owner can hold in the shared-memory tile list

struct EpCtx {
  uint64_t cnt[EP_MAX_RANKS];     // peers' arrival counters: int[e_local + 1] (the last one: the shared expert, served at home)
  uint64_t xq[EP_MAX_RANKS];      // peers' received codes      uint8 [slab_rows, H / 2]
  uint64_t sf[EP_MAX_RANKS];      // peers' received scales     uint8 [slab_rows / NT, H / 64, 512]
  uint64_t meta[EP_MAX_RANKS];    // peers' return words        int   [slab_rows]  = source rank * entry_stride + entry
  uint64_t comb[EP_MAX_RANKS];    // peers' combine buffers     bf16  [entry_stride, H]
  uint64_t flags[EP_MAX_RANKS];   // peers' flag pads           uint32 [2][EP_MAX_RANKS]: [0][src] dispatched, [1][owner] returned
  uint32_t* epoch;                // this rank's epoch word
  int* done;                      // this rank's CTA counters: [0] kernel A, [1] kernel E, [2] kernel F (zero between launches)
  int rank, world;
  int e_local;                    // routed experts per rank
  int n_slots;                    // e_local (+ 1 with a shared expert)
  int cap_e;                      // slab rows per expert
  int NT;                         // token tile width (32)
  int entry_stride;               // t_cap * k_all
  int local_only;
  unsigned long long wait_ns;
};

__device__ __forceinline__ void ep_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ep_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until flag word `p` reaches `target`.  Returns false (and records MARY_ERR_TIMEOUT_PEER) when it does not.
__device__ __forceinline__ bool ep_wait_flag(const uint32_t* p, uint32_t target, unsigned long long wait_ns, int* status) {
  if ((int32_t)(ep_ld_acquire_sys(p) - target) >= 0) return true;
  uint64_t t0 = 0;                          // the timer is read only after a run of failed polls, never on the fast path
  uint32_t spins = 0;
  while ((int32_t)(ep_ld_acquire_sys(p) - target) < 0) {
    if ((++spins & 255u) == 0) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > wait_ns) {
        atomicCAS(status, 0, MARY_ERR_TIMEOUT_PEER);
        return false;
      }
    }
  }
  return true;
}

}  // namespace mary
