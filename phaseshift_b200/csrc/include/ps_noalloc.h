// Allocation-free entry point (no counterpart in the reference runtime).
//
// Who needs it: code that drives the attention kernel from a context where device memory cannot be
// requested -- inside a region that is being stream-captured, in a real-time control loop that must not
// take the allocator's locks, in a host process that handed its whole device budget to another
// allocator, or from a foreign runtime (a plug-in, another language binding) that has no handle on this
// library's workspace objects.  Such callers still bring their inputs and outputs; what they cannot
// bring is the scratch area split-KV attention needs for its per-split partial results.
//
// What it does: `ps_paged_attention_noalloc` computes exactly what `ps_paged_attention` computes, but
// its partial accumulators live in a fixed array compiled into the library image (static device
// storage, 256-byte aligned, kNoAllocScratchBytes long).  Every GPU that loads the library carries that
// array until the process exits, whether or not the entry point is ever called.
//
// Rules for callers
//   * Size limit: rows * Hq * max_splits * (D + 2) * 4 bytes must not exceed kNoAllocScratchBytes.
//     Larger problems are refused with PS_NOALLOC_TOO_LARGE and a message retrievable through
//     ps_noalloc_last_error(); nothing is launched.
//   * First call on a device: the entry point resolves the device address of the array once per
//     device (with that device current) and remembers it.  Make this first call outside any stream
//     capture; later calls do no set-up work.
//   * The array is shared by every call and keeps whatever the previous call left in it.  The kernels
//     write each slot before they read it, so nothing needs clearing, but two calls whose kernels can
//     overlap on the GPU (different streams, no dependency) race on the array: serialise them.
//   * The entry point never calls cudaMalloc / cudaFree or any allocating library routine.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PS_NOALLOC_TOO_LARGE (-2)
#define PS_NOALLOC_SETUP_FAILED (-3)

enum { kNoAllocScratchBytes = 4 * 1024 * 1024 };

// Same arguments as ps_paged_attention without the two scratch pointers.  Returns 0, a cudaError_t
// value, or one of the PS_NOALLOC_* codes.
int ps_paged_attention_noalloc(const void* q, const void* k_pool, const void* v_pool, const void* k_scale,
                               const void* v_scale, const void* block_table, int max_blocks, int page_tokens,
                               int num_pages, const void* row_slot, const void* row_pos, int rows, int Hq, int Hkv,
                               int D, float sm_scale, int kv_fp8, int split_tokens, int max_splits, int max_visible,
                               const void* gate, int ld_gate, int gate_head_stride, int gate_offset, void* out,
                               void* status, cudaStream_t stream);

// Human-readable reason for the calling thread's most recent PS_NOALLOC_* result ("" if none).
const char* ps_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
