// Entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference; it exists for users of this library who run inside a fixed memory
// budget: a serving process that has handed every free byte of the GPU to its KV cache, a stream-capture or
// real-time section where cudaMalloc is forbidden or would synchronise the device, or a host runtime whose
// allocator is owned by another component.  Such callers cannot provide (or let us create) the partial-result
// buffer that split-KV paged attention needs.
//
// mary_paged_attention_noalloc() is mary_paged_attention() with that buffer taken from a fixed array that lives in
// the library's own device image instead of from the caller:
//
//   * the array is MARY_NOALLOC_SCRATCH_BYTES long; every GPU that loads this library holds that much memory until
//     the process exits, whether or not the entry point is ever called;
//   * a problem whose partial results do not fit (see mary_paged_attention_scratch_floats) is refused with
//     MARY_ERR_SCRATCH_TOO_LARGE and nothing is launched — use fewer splits or fewer query blocks per call;
//   * the first call on each device looks the array's device address up (cudaGetSymbolAddress); make that first call
//     outside any stream capture.  The kernel's shared-memory limit is a per-device attribute that is raised whenever a
//     device meets a head width that needs more than it was given before (the widest so far is remembered per device), so
//     the first call with each new, wider head shape should also come before capture; calls after that only launch;
//   * no cudaMalloc, cudaFree or other allocating routine is called, on any path;
//   * all calls on a device share the one array, which keeps whatever the previous call left in it.  Nothing in it
//     needs to start at zero (every slot that the merge pass reads was written by the same call's first pass), but two
//     calls that overlap on the GPU — different streams, or graphs replayed concurrently — race on it.  Serialise them.
//
// Inputs and outputs are still the caller's, exactly as for mary_paged_attention.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MARY_NOALLOC_SCRATCH_BYTES (16u << 20)
#define MARY_ERR_SCRATCH_TOO_LARGE 7

#ifdef __cplusplus
extern "C" {
#endif

int mary_paged_attention_noalloc(const void* q, const void* kc, const void* vc, void* out, const int* page_table,
                                 const int* kv_len, const int* q_start, const int* blk_seq, const int* blk_q0, int NB,
                                 int max_pages, int page_size, int64_t k_tok, int64_t k_page, int64_t v_tok, int64_t v_page,
                                 int Hq, int Hkv, int DK, int DV, int RQ, int nsplit, int window, float scale, float softcap,
                                 cudaStream_t stream);

// Capacity of the built-in array, in bytes (so callers can size their splits against it).
int64_t mary_noalloc_scratch_bytes(void);

// Text for a status code returned by the entry points of this library.
const char* mary_status_string(int code);

#ifdef __cplusplus
}
#endif
