// y[m, n] = sum_k x[m, k] * w[n, k] for a handful of rows m: the decode projections.
//
// The cost is streaming w once (engine/engine.py:431-438), so a warp owns one output column at a
// time and walks its weight row with 16-byte loads, several in flight, while the few activation rows
// come from L1/L2.  Products and sums are float (engine/kernels/fused.py:354); the order of the sum
// for one (m, n) does not depend on how many rows the call has.  With `gated`, w holds [gate; up]
// stacked ([2*n_out, k]) and the kernel writes round(silu(gate)) * up (fused.py:89-112), so the
// [rows, 2*inner] intermediate never reaches memory.
#include "common.cuh"

template <typename T, int VEC> struct Pack;
template <> struct Pack<float, 4> { typedef float4 type; };
template <> struct Pack<float, 1> { typedef float type; };
template <> struct Pack<bf16, 8> { typedef uint4 type; };
template <> struct Pack<bf16, 1> { typedef bf16 type; };

template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float* out) {
  typename Pack<T, VEC>::type raw = *reinterpret_cast<const typename Pack<T, VEC>::type*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < VEC; ++i) out[i] = to_f<T>(e[i]);
}

template <typename T, typename O, int MB, int VEC, bool GATED>
__global__ void linear_small_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                    O* __restrict__ y, int rows, int n_out, int k_dim) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  for (int n = warp; n < n_out; n += n_warps) {
    const T* wr = w + (size_t)n * k_dim;
    const T* wr2 = GATED ? w + (size_t)(n + n_out) * k_dim : nullptr;
    for (int m0 = 0; m0 < rows; m0 += MB) {
      float acc[MB], acc2[MB];
#pragma unroll
      for (int m = 0; m < MB; ++m) acc[m] = acc2[m] = 0.f;
#pragma unroll 2
      for (int k = lane * VEC; k < k_dim; k += 32 * VEC) {
        float wv[VEC], wv2[VEC];
        load_vec<T, VEC>(wr + k, wv);
        if (GATED) load_vec<T, VEC>(wr2 + k, wv2);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          if (m0 + m < rows) {
            float xv[VEC];
            load_vec<T, VEC>(x + (size_t)(m0 + m) * k_dim + k, xv);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
              acc[m] += xv[i] * wv[i];
              if (GATED) acc2[m] += xv[i] * wv2[i];
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        float v = warp_sum(acc[m]);
        float v2 = GATED ? warp_sum(acc2[m]) : 0.f;
        if (lane == 0 && m0 + m < rows) {
          if (GATED) {
            // gate and up are the two projection outputs, each rounded to the working type first
            const float g = rnd<T>(v), u = rnd<T>(v2);
            v = rnd<T>(g / (1.f + expf(-g))) * u;
          }
          y[(size_t)(m0 + m) * n_out + n] = from_f<O>(v);
        }
      }
    }
  }
}

template <typename T, typename O, bool GATED>
static int launch(const void* x, const void* w, void* y, int rows, int n_out, int k_dim,
                  cudaStream_t s) {
  if (rows == 0 || n_out == 0) return 0;
  const int threads = 256;
  int blocks = (n_out + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const int full = sizeof(T) == 2 ? 8 : 4;
  const bool vec_ok = k_dim % full == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0);
  const T* xp = (const T*)x;
  const T* wp = (const T*)w;
  O* yp = (O*)y;
#define GO(MB, VEC) linear_small_kernel<T, O, MB, VEC, GATED><<<blocks, threads, 0, s>>>(xp, wp, yp, rows, n_out, k_dim)
  if (vec_ok) {
    constexpr int V = sizeof(T) == 2 ? 8 : 4;
    if (rows == 1) GO(1, V);
    else if (rows == 2) GO(2, V);
    else if (rows <= 4) GO(4, V);
    else GO(8, V);
  } else {
    if (rows == 1) GO(1, 1);
    else if (rows <= 4) GO(4, 1);
    else GO(8, 1);
  }
#undef GO
  return SB_LAUNCH_RESULT();
}

extern "C" {

// dtype: 0 float, 1 bfloat16 (x and w).  out_float != 0 writes y as float whatever dtype is.
// gated != 0: w is [2 * n_out, k_dim] and y[m, n] = round(silu(x.w[n])) * (x.w[n + n_out]).
int sb_linear_small(int dtype, int out_float, int gated, const void* x, const void* w, void* y,
                    int rows, int n_out, int k_dim, cudaStream_t s) {
  if (dtype == 0) {
    return gated ? launch<float, float, true>(x, w, y, rows, n_out, k_dim, s)
                 : launch<float, float, false>(x, w, y, rows, n_out, k_dim, s);
  }
  if (out_float) {
    if (gated) return -1;
    return launch<bf16, float, false>(x, w, y, rows, n_out, k_dim, s);
  }
  return gated ? launch<bf16, bf16, true>(x, w, y, rows, n_out, k_dim, s)
               : launch<bf16, bf16, false>(x, w, y, rows, n_out, k_dim, s);
}

}  // extern "C"
