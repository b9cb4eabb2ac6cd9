// True 32-bit y[m, n] = sum_k x[m, k] * w[n, k] for many rows: FFMA only, no reduced-precision
// matrix mode.  This is the prompt-sized projection of the float32 path (the bfloat16 path uses
// tensor cores instead).  128x128 output tile per block, 8-deep k slices, 8x8 outputs per thread.
// The sum for one (m, n) runs over k in order, whatever the other rows of the call are.
#include "common.cuh"

#define TM 128
#define TN 128
#define TK 8

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                int rows, int n_out, int k_dim) {
  __shared__ float xs[TK][TM + 4];
  __shared__ float ws[TK][TN + 4];
  const int tid = threadIdx.x;
  const int m_base = blockIdx.y * TM, n_base = blockIdx.x * TN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 8 x 8 outputs
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  // each thread loads 4 consecutive k of one row of each operand tile: 128 rows x 8 k = 256 x 4
  const int lr = tid >> 1, lk = (tid & 1) * 4;
  for (int k0 = 0; k0 < k_dim; k0 += TK) {
    float xv[4], wv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int m = m_base + lr, n = n_base + lr;
      xv[i] = (m < rows && k < k_dim) ? x[(size_t)m * k_dim + k] : 0.f;
      wv[i] = (n < n_out && k < k_dim) ? w[(size_t)n * k_dim + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xs[lk + i][lr] = xv[i];
      ws[lk + i][lr] = wv[i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[8], b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = xs[k][ty * 8 + i];
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = ws[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m_base + ty * 8 + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n_base + tx + 16 * j;
      if (n < n_out) y[(size_t)m * n_out + n] = acc[i][j];
    }
  }
}

extern "C" {

int sb_sgemm_nt(const float* x, const float* w, float* y, int rows, int n_out, int k_dim,
                cudaStream_t s) {
  if (rows == 0 || n_out == 0) return 0;
  dim3 grid((n_out + TN - 1) / TN, (rows + TM - 1) / TM);
  sgemm_nt_kernel<<<grid, 256, 0, s>>>(x, w, y, rows, n_out, k_dim);
  return SB_LAUNCH_RESULT();
}

}  // extern "C"
