// The allocation-free variant of the tensor-core decode attention: see attention_decode_noalloc.h.
// The kernels are those of attention_decode_mma.cu, compiled into this library as well; only where
// the split-key scratch lives differs.
#include "attention_decode_noalloc.h"

#include <stdio.h>

#include "attention_decode_mma.cu"

// In device code this name is the array; in host code it is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) float noalloc_scratch[SB_NOALLOC_SCRATCH_FLOATS];

#define NOALLOC_MAX_DEVICES 64
static float* scratch_on_device[NOALLOC_MAX_DEVICES];
static thread_local char message[256] = "";

extern "C" {

const char* sb_attention_decode_noalloc_message(void) { return message; }

int sb_attention_decode_noalloc(const void* q, void* out, const void* k_store, const void* v_store,
                                const int* block_table, int table_stride, const int* row_slot,
                                const int* row_kv_len, int rows, int heads, int kv_heads, int head_dim,
                                float scale, int window, int n_splits, cudaStream_t stream) {
  message[0] = 0;
  if (rows <= 0) return 0;
  if (heads <= 0 || n_splits < 1 || head_dim <= 0) {
    snprintf(message, sizeof message, "heads, head_dim and n_splits must be positive");
    return -2;
  }
  // up to DM_CLUSTER_MAX parts are merged inside a thread-block cluster and touch no scratch at all;
  // only beyond that are the parts written to the array and merged by a second kernel
  const long long need = n_splits > DM_CLUSTER_MAX ? (long long)rows * heads * n_splits * (head_dim + 2) : 0;
  if (need > SB_NOALLOC_SCRATCH_FLOATS) {
    snprintf(message, sizeof message,
             "rows * heads * n_splits * (head_dim + 2) = %lld floats of scratch are needed, the static "
             "array holds %d; use fewer splits or rows, or the entry point that takes scratch",
             need, SB_NOALLOC_SCRATCH_FLOATS);
    return SB_NOALLOC_TOO_LARGE;
  }
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err == cudaSuccess && (device < 0 || device >= NOALLOC_MAX_DEVICES)) err = cudaErrorInvalidDevice;
  if (err == cudaSuccess && scratch_on_device[device] == nullptr) {
    // once per device, with that device current: the device address of the array
    float* address = nullptr;
    err = cudaGetSymbolAddress((void**)&address, noalloc_scratch);
    if (err == cudaSuccess) scratch_on_device[device] = address;
  }
  if (err != cudaSuccess) {
    snprintf(message, sizeof message, "set-up failed: %s", cudaGetErrorString(err));
    return (int)err;
  }
  float* part_acc = scratch_on_device[device];
  float* part_ml = part_acc + (size_t)rows * heads * n_splits * head_dim;
  const int rc = sb_attention_decode_mma(q, out, k_store, v_store, block_table, table_stride, row_slot,
                                         row_kv_len, rows, heads, kv_heads, head_dim, scale, window,
                                         n_splits, part_acc, part_ml, stream);
  if (rc == -2) snprintf(message, sizeof message, "head_dim %d or the head counts are outside what the kernel takes", head_dim);
  else if (rc != 0) snprintf(message, sizeof message, "launch failed: %s", cudaGetErrorString((cudaError_t)rc));
  return rc;
}

}  // extern "C"
