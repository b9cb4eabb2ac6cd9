// TMA descriptors for the kernels of this library: a [rows, cols] row-major bfloat16 matrix read in
// boxes of [box_rows x 64] with 128-byte swizzle (64 bfloat16 are one swizzle atom).  Rows and columns
// past the matrix read as zero.
//
// Encoding a map costs a microsecond or two on the host, and the same matrices (every weight, and
// activation buffers the allocator hands out again) come back step after step: the last maps are
// kept in a small direct-mapped table per host thread, keyed by everything a map is made of.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef CUresult (*SbEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime (the libraries do not link against the driver).
static inline SbEncodeTiledFn sb_encode_fn() {
  static SbEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (SbEncodeTiledFn)p;
  }
  return fn;
}

struct SbMapKey {
  const void* base;
  long long rows, cols;
  int box_rows;
  bool operator==(const SbMapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct SbMapSlot { SbMapKey key; CUtensorMap map; bool used; };

// 0, or -3 if the driver entry point is missing, -4 if the driver refuses the map (the base must be
// 16-byte aligned and cols a multiple of 8).
static inline int sb_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
  static thread_local SbMapSlot cache[512];
  const SbMapKey key = {base, rows, cols, box_rows};
  const size_t h = (((uintptr_t)base >> 8) * 0x9E3779B97F4A7C15ull + (size_t)box_rows * 31 + (size_t)rows) >> 20;
  SbMapSlot& slot = cache[h & 511];
  if (slot.used && slot.key == key) { *map = slot.map; return 0; }
  SbEncodeTiledFn fn = sb_encode_fn();
  if (!fn) return -3;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return -4;
  slot.key = key; slot.map = *map; slot.used = true;
  return 0;
}
