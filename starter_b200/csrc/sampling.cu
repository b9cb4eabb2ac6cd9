// Token selection from float logits: greedy argmax, or a draw from softmax(logits / temperature).
//
// Greedy keeps the lowest index among equal maxima (engine/engine.py:833 uses argmax).  The draw uses
// the Gumbel-max identity: argmax_i(logit_i / t + g_i) with g_i = -log(-log(u_i)) is distributed as
// softmax(logits / t), so sampling is one more argmax and needs no normalisation pass.  u_i comes from
// a counter-based hash of (row key, vocabulary index); the row key is derived from the sampling seed,
// the request's own number and the position of the token being drawn, so a request draws the same
// tokens whatever else is in its batch.  The host-side statement of the same arithmetic is
// starter_b200/sampling/sampler.py:gumbel_noise.
#include "common.cuh"

__host__ __device__ __forceinline__ uint32_t sb_mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

__global__ void sample_kernel(const float* __restrict__ logits, int vocab, size_t row_stride,
                              const float* __restrict__ temperature,
                              const uint32_t* __restrict__ request_key,
                              const int* position, int* __restrict__ out,
                              int* status, int* feed_token, int* feed_pos, int* feed_len) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const int row = blockIdx.x;
  const float* lr = logits + (size_t)row * row_stride;
  const float t = temperature ? temperature[row] : 0.f;
  const bool greedy = !(t > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / t;
  uint32_t row_key = 0;
  if (!greedy) row_key = sb_mix32((uint32_t)position[row] + sb_mix32(request_key[row]));

  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = lr[i] * inv_t;
    if (!greedy) {
      const uint32_t r = sb_mix32((uint32_t)i ^ row_key);
      const float u = ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f);
      v += -logf(-logf(u));
    }
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int warps = blockDim.x >> 5;
    bv = lane < warps ? best_v[lane] : -INFINITY;
    bi = lane < warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      if (bi < 0 || bi >= vocab) {  // every logit was NaN
        if (status) atomicOr(status, 2);
        bi = 0;
      }
      out[row] = bi;
      // self-feeding decode: the drawn token becomes the row's next input, one position further on
      // (engine/engine.py:835-838).  Every thread read position[row] before the barrier above.
      if (feed_token) {
        feed_token[row] = bi;
        feed_pos[row] += 1;
        feed_len[row] += 1;
      }
    }
  }
}

extern "C" {

// logits: [rows, vocab] float with `row_stride` floats between rows.  temperature may be null (all
// greedy); rows with temperature <= 0 are greedy.  request_key and position are read only for rows
// that draw.  With feed_token (all three feed arrays or none), row r also stores its token in
// feed_token[r] and adds one to feed_pos[r] and feed_len[r]; position may alias feed_len.
int sb_sample(const float* logits, int rows, int vocab, long long row_stride, const float* temperature,
              const uint32_t* request_key, const int* position, int* out, int* status,
              int* feed_token, int* feed_pos, int* feed_len, cudaStream_t s) {
  if (rows == 0) return 0;
  const int threads = vocab >= 8192 ? 1024 : 256;
  sample_kernel<<<rows, threads, 0, s>>>(logits, vocab, (size_t)row_stride, temperature, request_key,
                                         position, out, status, feed_token, feed_pos, feed_len);
  return SB_LAUNCH_RESULT();
}

}  // extern "C"
