// Row-wise kernels: embedding gather, RMSNorm (plain, fused with the residual sum, and on selected
// rows), and the gated activation.  One block per row; the row is walked twice (sum of squares, then
// scale) by the same threads over the same columns, so the second pass reads what the first just
// touched.  Formulas and cast placement: engine/engine.py:75-88 (norm), engine/kernels/fused.py:115-144
// (sum in float, rounded to the working type, stored, then normed), fused.py:89-112 (silu rounded to
// the working type before the product).
#include "common.cuh"

// ------------------------------------------------------------------------------------ embedding

template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                 T* __restrict__ out, int hidden, int vocab, int* status) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(tokens);
  const int row = blockIdx.x;
  int tok = tokens[row];
  const bool bad = tok < 0 || tok >= vocab;
  if (bad) {
    if (threadIdx.x == 0 && status) atomicOr(status, 1);
    tok = 0;
  }
  const T* src = table + (size_t)tok * hidden;
  T* dst = out + (size_t)row * hidden;
  constexpr int N = 16 / sizeof(T);
  if (!bad && hidden % N == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
    // 16 bytes a thread and all of a thread's loads in flight together: the row comes from memory
    // nobody has touched for a step, and this kernel stands alone between two steps
    const uint4* src4 = reinterpret_cast<const uint4*>(src);
    uint4* dst4 = reinterpret_cast<uint4*>(dst);
    const int n = hidden / N;
    uint4 v[4];
    for (int c0 = threadIdx.x; c0 < n; c0 += 4 * blockDim.x) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (c0 + i * blockDim.x < n) v[i] = src4[c0 + i * blockDim.x];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (c0 + i * blockDim.x < n) dst4[c0 + i * blockDim.x] = v[i];
    }
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = bad ? from_f<T>(0.f) : src[c];
}

// ------------------------------------------------------------------------------------ norms

// y[r] = gain * round(x[r] * rsqrt(mean(x[r]^2) + eps)).  With `delta`, x[r] is first replaced by
// round(x[r] + delta[r]) and written back (the residual stream).  With `rows`, output row i comes
// from input row rows[i] and nothing is written back.
template <typename T, typename W, bool ADD, bool WRITE_BACK>
__global__ void rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta,
                               const W* __restrict__ gain, T* __restrict__ y,
                               const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(delta);
  SB_BEHIND_WAIT(rows);
  const int out_row = blockIdx.x;
  const int in_row = rows ? rows[out_row] : out_row;
  T* xr = x + (size_t)in_row * hidden;
  const T* dr = ADD ? delta + (size_t)in_row * hidden : nullptr;
  T* yr = y + (size_t)out_row * hidden;

  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = to_f<T>(xr[c]);
    if (ADD) {
      v = rnd<T>(v + to_f<T>(dr[c]));
      if (WRITE_BACK) xr[c] = from_f<T>(v);
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = to_f<T>(xr[c]);
    if (ADD && !WRITE_BACK) v = rnd<T>(v + to_f<T>(dr[c]));
    yr[c] = from_f<T>(rnd<T>(v * inv) * to_f<W>(gain[c]));
  }
}

// The same with 16-byte accesses (8 bfloat16 or 4 floats per thread and step); a thread keeps the up
// to four vectors it owns in registers between the two passes.  Needs hidden % VEC == 0, 16-byte
// aligned rows and hidden <= 4 * VEC * blockDim.
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T, int N> __device__ __forceinline__ void load_vec16(const T* p, float* out) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = to_f<T>(e[i]);
}
template <typename T, int N> __device__ __forceinline__ void store_vec16(T* p, const float* v) {
  uint4 raw;
  if (sizeof(T) == 2) {                   // packed conversions: half as many on the conversion pipe
    uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&two);
    }
  } else {
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) e[i] = from_f<T>(v[i]);
  }
  *reinterpret_cast<uint4*>(p) = raw;
}
// The same for values that already are values of T (they were rounded): no conversion at all.
template <typename T, int N> __device__ __forceinline__ void store_exact16(T* p, const float* v) {
  uint4 raw;
  if (sizeof(T) == 2) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
    for (int i = 0; i < N / 2; ++i) w[i] = pack_exact_bf16(v[2 * i], v[2 * i + 1]);
  } else {
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) e[i] = from_f<T>(v[i]);
  }
  *reinterpret_cast<uint4*>(p) = raw;
}
// N consecutive gains as floats, in one 16-byte load where type and address allow it.
template <typename W, int N> __device__ __forceinline__ void load_gain(const W* p, float* out) {
  if (N * sizeof(W) == 16 && ((uintptr_t)p & 15) == 0) {
    load_vec16<W, N>(p, out);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = to_f<W>(p[i]);
  }
}

template <typename T, typename W, bool ADD, bool WRITE_BACK, bool EARLY>
__global__ void rmsnorm_vec_kernel(T* __restrict__ x, const T* __restrict__ delta,
                                   const W* __restrict__ gain, T* __restrict__ y,
                                   const int* __restrict__ rows, int hidden, float eps) {
  constexpr int N = Vec16<T>::N;
  __shared__ float scratch[33];
  pdl_trigger();
  // EARLY (few rows, where the launch chain's latency is what counts): the gains are weights, they
  // do not depend on the kernel before this one and are on their way while it finishes.  With many
  // rows the registers they would hold are worth more.
  float gn[EARLY ? 4 : 1][N];
  if (EARLY) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int c = (it * blockDim.x + threadIdx.x) * N;
      if (c < hidden) load_gain<W, N>(gain + c, gn[it]);
    }
  }
  pdl_wait();
  SB_BEHIND_WAIT(delta);
  SB_BEHIND_WAIT(rows);
  const int out_row = blockIdx.x;
  const int in_row = rows ? rows[out_row] : out_row;
  T* xr = x + (size_t)in_row * hidden;
  const T* dr = ADD ? delta + (size_t)in_row * hidden : nullptr;
  T* yr = y + (size_t)out_row * hidden;
  float v[4][N];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * N;
    if (c < hidden) {
      load_vec16<T, N>(xr + c, v[it]);
      if (ADD) {
        float d[N];
        load_vec16<T, N>(dr + c, d);
#pragma unroll
        for (int i = 0; i < N; i += 2) {
          v[it][i] += d[i];
          v[it][i + 1] += d[i + 1];
          rnd2<T>(v[it][i], v[it][i + 1]);
        }
        if (WRITE_BACK) store_exact16<T, N>(xr + c, v[it]);
      }
#pragma unroll
      for (int i = 0; i < N; ++i) ss += v[it][i] * v[it][i];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * N;
    if (c < hidden) {
      float o[N];
      if (!EARLY) load_gain<W, N>(gain + c, gn[0]);
      const float* g = gn[EARLY ? it : 0];
#pragma unroll
      for (int i = 0; i < N; i += 2) {
        float a = v[it][i] * inv, b = v[it][i + 1] * inv;
        rnd2<T>(a, b);
        o[i] = a * g[i];
        o[i + 1] = b * g[i + 1];
      }
      store_vec16<T, N>(yr + c, o);
    }
  }
}

// Many rows: a warp per row.  With a block per row a 2,048-row prompt is 2,048 short-lived blocks
// whose chain (load, block reduction with two barriers, store) is latency, in two waves: 10 us for
// 21 MB.  A warp per row needs no barrier, 64 rows are in flight on an SM and all rows at once.  The
// row is read twice (the second time from L1/L2, where this lane's own writes of the sum are).
template <typename T, typename W, bool ADD>
__global__ void rmsnorm_warp_kernel(T* __restrict__ x, const T* __restrict__ delta,
                                    const W* __restrict__ gain, T* __restrict__ y, int n_rows,
                                    int hidden, float eps) {
  constexpr int N = Vec16<T>::N;
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(delta);
  const int row = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  T* xr = x + (size_t)row * hidden;
  const T* dr = ADD ? delta + (size_t)row * hidden : nullptr;
  T* yr = y + (size_t)row * hidden;
  const int vecs = hidden / N;
  float ss = 0.f;
#pragma unroll 4
  for (int i = lane; i < vecs; i += 32) {
    float v[N];
    load_vec16<T, N>(xr + i * N, v);
    if (ADD) {
      float d[N];
      load_vec16<T, N>(dr + i * N, d);
#pragma unroll
      for (int j = 0; j < N; j += 2) {
        v[j] += d[j];
        v[j + 1] += d[j + 1];
        rnd2<T>(v[j], v[j + 1]);
      }
      store_exact16<T, N>(xr + i * N, v);
    }
#pragma unroll
    for (int j = 0; j < N; ++j) ss += v[j] * v[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll 4
  for (int i = lane; i < vecs; i += 32) {
    float v[N], g[N], o[N];
    load_vec16<T, N>(xr + i * N, v);
    load_gain<W, N>(gain + i * N, g);
#pragma unroll
    for (int j = 0; j < N; j += 2) {
      float a = v[j] * inv, b = v[j + 1] * inv;
      rnd2<T>(a, b);
      o[j] = a * g[j];
      o[j + 1] = b * g[j + 1];
    }
    store_vec16<T, N>(yr + i * N, o);
  }
}

template <typename T, typename W>
static int launch_rmsnorm(void* x, const void* delta, const void* gain, void* y, const int* rows,
                          int n_rows, int hidden, float eps, cudaStream_t s) {
  if (n_rows == 0) return 0;
  int threads = hidden >= 4096 ? 1024 : hidden >= 1024 ? 512 : hidden >= 256 ? 256 : 128;
  T* xp = (T*)x;
  const T* dp = (const T*)delta;
  const W* gp = (const W*)gain;
  T* yp = (T*)y;
  constexpr int N = 16 / sizeof(T);
  const bool aligned = hidden % N == 0 && (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)y) & 15) == 0;
  if (aligned && !rows && n_rows > 256 && x != y) {
    const int threads_w = 256;                       // 8 rows a block
    const int blocks = (n_rows + 7) / 8;
    if (delta)
      return launch_dependent(rmsnorm_warp_kernel<T, W, true>, dim3(blocks), dim3(threads_w), 0, s, xp, dp, gp, yp, n_rows, hidden, eps);
    return launch_dependent(rmsnorm_warp_kernel<T, W, false>, dim3(blocks), dim3(threads_w), 0, s, xp, dp, gp, yp, n_rows, hidden, eps);
  }
  if (aligned && hidden <= 4 * N * 1024) {
    int vt = 32;
    while (vt * N * 2 < hidden && vt < 1024) vt *= 2;   // about two vectors per thread
    while (vt * N * 4 < hidden) vt *= 2;
#define VEC_LAUNCH(A, B, E) launch_dependent(rmsnorm_vec_kernel<T, W, A, B, E>, dim3(n_rows), dim3(vt), 0, s, xp, dp, gp, yp, rows, hidden, eps)
    const bool early = n_rows <= 256;
    if (delta && !rows) return early ? VEC_LAUNCH(true, true, true) : VEC_LAUNCH(true, true, false);
    if (delta) return early ? VEC_LAUNCH(true, false, true) : VEC_LAUNCH(true, false, false);
    return early ? VEC_LAUNCH(false, false, true) : VEC_LAUNCH(false, false, false);
#undef VEC_LAUNCH
  }
  if (delta && !rows)
    return launch_dependent(rmsnorm_kernel<T, W, true, true>, dim3(n_rows), dim3(threads), 0, s, xp, dp, gp, yp, rows, hidden, eps);
  if (delta)
    return launch_dependent(rmsnorm_kernel<T, W, true, false>, dim3(n_rows), dim3(threads), 0, s, xp, dp, gp, yp, rows, hidden, eps);
  return launch_dependent(rmsnorm_kernel<T, W, false, false>, dim3(n_rows), dim3(threads), 0, s, xp, dp, gp, yp, rows, hidden, eps);
}

// ------------------------------------------------------------------------------------ gated activation

// act[r, c] = round(silu(gate)) * up with gate = gu[r, c], up = gu[r, inner + c].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int inner, size_t total) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(gu);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t row = i / inner;
    const int col = (int)(i - row * inner);
    const float g = to_f<T>(gu[row * 2 * inner + col]);
    const float u = to_f<T>(gu[row * 2 * inner + inner + col]);
    const float silu = rnd<T>(g / (1.f + expf(-g)));
    act[i] = from_f<T>(silu * u);
  }
}

// The same with 16-byte accesses: N consecutive columns per thread (inner % N == 0, aligned rows).
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ act, int inner, size_t groups) {
  constexpr int N = 16 / sizeof(T);
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(gu);
  const int per_row = inner / N;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < groups; i += stride) {
    const size_t row = i / per_row;
    const int col = (int)(i - row * per_row) * N;
    float g[N], u[N], o[N];
    load_vec16<T, N>(gu + row * 2 * inner + col, g);
    load_vec16<T, N>(gu + row * 2 * inner + inner + col, u);
#pragma unroll
    for (int j = 0; j < N; j += 2) {
      // the result is rounded to 8 bits of mantissa: the fast exponential and quotient (a few
      // float ulp, as in the product kernel's gated epilogue) do not show; float keeps the exact ones
      float s0 = sizeof(T) == 2 ? __fdividef(g[j], 1.f + __expf(-g[j])) : g[j] / (1.f + expf(-g[j]));
      float s1 = sizeof(T) == 2 ? __fdividef(g[j + 1], 1.f + __expf(-g[j + 1])) : g[j + 1] / (1.f + expf(-g[j + 1]));
      rnd2<T>(s0, s1);
      o[j] = s0 * u[j];
      o[j + 1] = s1 * u[j + 1];
    }
    store_vec16<T, N>(act + row * inner + col, o);
  }
}

extern "C" {

// dtype: 0 float, 1 bfloat16.  gain_dtype likewise.
int sb_embedding(int dtype, const int* tokens, const void* table, void* out, int n_tokens, int hidden,
                 int vocab, int* status, int serial, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (serial) {
    // An ordinary launch: it starts only when everything before it on the stream has completed.  As
    // the first kernel of a step it is the fence behind which later kernels of the step may read,
    // before their own dependent-launch wait, whatever earlier steps wrote.
    if (dtype == 0)
      embedding_kernel<float><<<n_tokens, threads, 0, s>>>(tokens, (const float*)table, (float*)out, hidden, vocab, status);
    else
      embedding_kernel<bf16><<<n_tokens, threads, 0, s>>>(tokens, (const bf16*)table, (bf16*)out, hidden, vocab, status);
    return SB_LAUNCH_RESULT();
  }
  if (dtype == 0)
    return launch_dependent(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const float*)table, (float*)out, hidden, vocab, status);
  return launch_dependent(embedding_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const bf16*)table, (bf16*)out, hidden, vocab, status);
}

// x: [*, hidden] read (and, with delta and without rows, updated in place); y: [n_rows, hidden].
int sb_rmsnorm(int dtype, int gain_dtype, void* x, const void* delta, const void* gain, void* y,
               const int* rows, int n_rows, int hidden, float eps, cudaStream_t s) {
  if (dtype == 0 && gain_dtype == 0) return launch_rmsnorm<float, float>(x, delta, gain, y, rows, n_rows, hidden, eps, s);
  if (dtype == 1 && gain_dtype == 1) return launch_rmsnorm<bf16, bf16>(x, delta, gain, y, rows, n_rows, hidden, eps, s);
  if (dtype == 1 && gain_dtype == 0) return launch_rmsnorm<bf16, float>(x, delta, gain, y, rows, n_rows, hidden, eps, s);
  return -1;
}

int sb_swiglu(int dtype, const void* gu, void* act, int n_rows, int inner, cudaStream_t s) {
  const size_t total = (size_t)n_rows * inner;
  if (total == 0) return 0;
  const int threads = 256;
  const int vec = dtype == 0 ? 4 : 8;
  if (inner % vec == 0 && (((uintptr_t)gu | (uintptr_t)act) & 15) == 0) {
    const size_t groups = total / vec;
    size_t vblocks = (groups + threads - 1) / threads;
    if (vblocks > 148 * 32) vblocks = 148 * 32;
    if (dtype == 0)
      return launch_dependent(swiglu_vec_kernel<float>, dim3((int)vblocks), dim3(threads), 0, s, (const float*)gu, (float*)act, inner, groups);
    return launch_dependent(swiglu_vec_kernel<bf16>, dim3((int)vblocks), dim3(threads), 0, s, (const bf16*)gu, (bf16*)act, inner, groups);
  }
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == 0)
    return launch_dependent(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gu, (float*)act, inner, total);
  return launch_dependent(swiglu_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, s, (const bf16*)gu, (bf16*)act, inner, total);
}

}  // extern "C"
