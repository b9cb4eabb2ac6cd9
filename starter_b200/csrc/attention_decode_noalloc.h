// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (alvinyuwen/starter); it exists for users of
// this library whose code runs where cudaMalloc is off limits: inside a process that has handed all
// device memory to another allocator and forbids further driver allocations, in a latency-critical
// serving loop that must never take the allocator's lock, or in a plugin whose host gives it streams
// and buffers but no allocation rights.  The regular entry point (sb_attention_decode_mma) takes its
// split-key scratch from the caller, who in this library gets it from torch's allocator; this one
// keeps the scratch in a fixed array inside the library instead.
//
// What to know before calling it:
//   * The scratch is ONE static device array of SB_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU
//     on which this library is loaded holds that array until the process exits.
//   * A call with more than 8 parts (n_splits) needs rows * heads * n_splits * (head_dim + 2) floats
//     of it; with up to 8 parts the kernel merges inside a thread-block cluster and uses none.  More
//     than the array holds is refused with SB_NOALLOC_TOO_LARGE;
//     sb_attention_decode_noalloc_message() then says how much was asked for and how much there is.
//     Nothing is launched in that case.
//   * All calls share the array and it keeps the last call's contents.  Nothing in it has to start at
//     zero: each call overwrites every entry it later reads (parts that see no key write a neutral
//     entry).  Two calls that overlap on the GPU (different streams, or graphs replayed together)
//     race on it; calls on one stream are safe.
//   * The first call on each device looks up the array's device address and configures the kernel.
//     Make that first call, with that device current, before any stream capture.
//   * It calls no cudaMalloc, cudaFree or other allocating routine, and it runs on the stream given.
#pragma once

#include <cuda_runtime.h>

#define SB_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define SB_NOALLOC_TOO_LARGE (-5)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as sb_attention_decode_mma (bfloat16; head_dim 16, 32, 64 or 128) without
// the two scratch pointers.  Returns 0, a cudaError_t, -2 for sizes the kernel does not take, or
// SB_NOALLOC_TOO_LARGE.
int sb_attention_decode_noalloc(const void* q, void* out, const void* k_store, const void* v_store,
                                const int* block_table, int table_stride, const int* row_slot,
                                const int* row_kv_len, int rows, int heads, int kv_heads, int head_dim,
                                float scale, int window, int n_splits, cudaStream_t stream);

// Text for the last non-zero result of sb_attention_decode_noalloc on this host thread.
const char* sb_attention_decode_noalloc_message(void);

#ifdef __cplusplus
}
#endif
