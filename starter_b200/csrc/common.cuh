// Shared device helpers for the sm_100a kernels of this library.
//
// Conventions that every kernel file follows:
//   * activations are packed [tokens, features] row-major; weights are [out, in] row-major;
//   * T is the working type (float or __nv_bfloat16); sums, norms, softmax and angles are float;
//   * rnd<T>(x) rounds a float to the working type and back, which places the casts where the
//     reference's formulas place them (engine/engine.py:75-109) and is the identity for float;
//   * every extern "C" entry returns 0 or a cudaError_t from the launch, never throws, never
//     allocates, and runs on the stream it is given.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SB_PAGE_TOKENS 64
// Every library built from this header says which page size it was compiled for; the Python side
// compares it with the cache's own constant when it loads the library.
extern "C" __attribute__((weak, visibility("default"))) int sb_page_tokens() { return SB_PAGE_TOKENS; }

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ float rnd(float v) { return to_f<T>(from_f<T>(v)); }
// Two values at once.  For bfloat16 one packed conversion and two integer operations give the same
// bits as two single conversions, which run on the quarter-rate conversion pipe.
template <typename T> __device__ __forceinline__ void rnd2(float& a, float& b) { a = rnd<T>(a); b = rnd<T>(b); }
template <> __device__ __forceinline__ void rnd2<__nv_bfloat16>(float& a, float& b) {
  __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  const uint32_t w = *reinterpret_cast<uint32_t*>(&p);
  a = __uint_as_float(w << 16);
  b = __uint_as_float(w & 0xffff0000u);
}
// Two floats that already are bfloat16 values, packed (low half first) without a conversion.
__device__ __forceinline__ uint32_t pack_exact_bf16(float lo, float hi) {
  return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  float out = scratch[32];
  __syncthreads();
  return out;
}

// Address of element (page, head, offset, 0) in a paged key or value store laid out
// [pages][kv_heads][SB_PAGE_TOKENS][head_dim].
__device__ __forceinline__ size_t page_row(int page, int head, int offset, int kv_heads, int head_dim) {
  return (((size_t)page * kv_heads + head) * SB_PAGE_TOKENS + offset) * (size_t)head_dim;
}

#define SB_LAUNCH_RESULT() ((int)cudaGetLastError())

// ---------------------------------------------------------------------------------- dependent launch
// Kernels of a step run back to back on one stream and each is short, so the gap between one
// kernel's last block and the next kernel's first instruction matters.  Launched with
// launch_dependent(), a kernel may start while its predecessor is still running (as soon as every
// block of the predecessor has called pdl_trigger() or exited), do whatever does not depend on the
// predecessor (set up barriers, allocate tensor memory, prefetch WEIGHTS), and then call pdl_wait(),
// which returns once the predecessor has completed and its writes are visible.
//
// The rule that keeps this safe: every kernel calls pdl_wait() before its first read of anything an
// earlier kernel of the stream may have written and before its first write to global memory (a
// buffer may be recycled memory that an earlier kernel still reads).  Because a kernel cannot
// complete before its own pdl_wait() returns, completion is transitive along the stream.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A load through a `const T* __restrict__` parameter counts as invariant (nothing in the kernel can
// change what it reads), so the compiler is free to move it up, across volatile asm and its memory
// clobber too: across pdl_wait().  Then the kernel reads what its predecessor has not written yet.
// (Seen once: the decode attention's first layer in a captured step read its q/k/v row early.)
// SB_BEHIND_WAIT(p), placed after pdl_wait(), hands the compiler the pointer back as a value it
// has not seen before; every load through it depends on that value and stays behind the wait.
// It goes on every parameter an earlier kernel of the stream may have written and that this
// kernel reads with ordinary loads (copies issued by inline asm keep their place by themselves).
#define SB_BEHIND_WAIT(p) asm volatile("" : "+l"(p) : : "memory")
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The same, as thread-block clusters of `cluster` CTAs (every grid dimension a multiple of it).
template <typename... Params, typename... Args>
static inline int launch_dependent_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, dim3 cluster, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  attribute[1].id = cudaLaunchAttributeClusterDimension;
  attribute[1].val.clusterDim.x = cluster.x;
  attribute[1].val.clusterDim.y = cluster.y;
  attribute[1].val.clusterDim.z = cluster.z;
  config.attrs = attribute;
  config.numAttrs = cluster.x * cluster.y * cluster.z > 1 ? 2 : 1;
  return (int)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

template <typename... Params, typename... Args>
static inline int launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                   cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
